// umma_q8.cu -- W8A8 block-quantized mul_mat on tcgen05 (kind::i8), Q8_0R weights.
//
//   C[token][out] = sum_blocks float(sum_{32} q_w * q_a) * (d_w * d_a)   (+ bias[out])
//
// The activations never make a round trip through HBM as int8: fp32 rows are pulled in by TMA
// (128 tokens x one 32-element quant block per stage, 128-byte swizzle), quantized from shared
// memory by two warps (absmax, d = vmax / -128, q = round(x / d), bit-exact with the host quantizer)
// and written as the K-major int8 A operand, which stays resident for all weight column blocks of the
// work item (and is double-buffered across items when it is small enough).  The int8 weights stream in
// by TMA.  Every quant block is ONE tcgen05.mma (K = 32, no accumulation) into one of four 128-column
// TMEM slots; sixteen epilogue warps drain a slot, turn the exact int32 block sums into fp32 and
// accumulate sum * d_w * d_a in registers in block order.
//
// Warp roles (20 warps, so that each thread may hold 96 registers): warp 0 = both TMA streams (one
// thread polls the two rings), warp 1 = MMA issue + TMEM owner, warps 2-3 = quantizers (two token rows
// per thread), warps 4-19 = epilogue (four warps per TMEM lane quarter, 32 columns each).
#include <cuda_fp16.h>

#include <cstdlib>
#include <type_traits>

#include "kernels.h"
#include "tma_host.h"

namespace ppml_b200 {

namespace {

constexpr int kTile = 128 * 128;          // bytes: one int8 A tile (128 rows x 128 K) == one weight stage == one raw fp32 stage
constexpr int kMaxKT = 8;                 // K <= 1024
constexpr int kMaxStages = 6;
// Two warp layouts (template parameter QW = number of quantizer warps):
//   QW = 2: warp 0 TMA, 1 MMA, 2-3 quantizers (two token rows per thread), 4-19 epilogue: 20 warps, 96 registers;
//           for items with several column blocks, where the epilogue is the limiter and must not spill.
//   QW = 4: warps 0-3 quantizers (one row per thread), 4-19 epilogue, 20 TMA, 21 MMA: 22 warps, 80 registers;
//           for items with a single column block, where the quantizer is the limiter.
constexpr int kEpiWarps = 16;             // four per TMEM lane quarter, 32 output columns each
constexpr int kFirstEpiWarp = 4;          // a multiple of 4: warp % 4 is the lane quarter
template <int QW> struct Roles;
template <> struct Roles<2> { static constexpr int kFirstQuantWarp = 2, kTmaWarp = 0, kMmaWarp = 1, kThreads = 32 * 20; };
template <> struct Roles<4> { static constexpr int kFirstQuantWarp = 0, kTmaWarp = 20, kMmaWarp = 21, kThreads = 32 * 22; };

struct Q8Params {
    int Mout, Ntok, K, nblk, KT;
    int m_tiles;               // token tiles
    int n_blocks;              // weight column blocks of 128
    int groups, blocks_per_group;
    int flat;                  // 1: every CTA takes a contiguous range of (token tile, column block) units (see item_at)
    int RS, BS;                // ring depths
    int AR;                    // 16 KB slots of quantized A, used as a ring over (item, K step): KT = resident, 2 KT = resident
                               // and double-buffered across items, 3 = a short ring (items with a single column block)
    int dw_tabs;               // scale tables held in smem: n_blocks (all resident, filled once) or 1 (refilled per column block)
    int staged;                // columns of the per-warp store buffer (32 rows x staged fp32: 8, 16 or 32; the results leave
                               // through TMA stores), 0: plain stores from registers
    int preq;                  // 1: the activations were quantized by a kernel of their own: int8 tiles and scale tables
                               //    come in by TMA, the quantizer warps idle (tmX then maps the int8 matrix)
    const __half* da_t;        // preq: activation scales [token tile][nblk][128]
    const __half* Wd;          // weight scales [Mout][nblk]
    float* C;
    const float* bias;
    int* sumi_out;
    int c_trans;
    int vec_ok;
    int vec32_ok;              // C rows and base 32-byte aligned: the unstaged store writes whole 128-byte lines (256-bit stores)
    int dw_vec;                // K a multiple of 256 and aligned scales: the table refill reads eight scales per 16-byte load
    int* err;
};

struct SmemLayout {
    uint32_t a_off, raw_off, w_off, c_off, dw_off, da_off, st_off, bar_off, total;
};

constexpr int kNumBarriers = 4 * kMaxStages + 4 * kMaxKT + 8 + 4;

__host__ __device__ inline SmemLayout q8_layout(int AR, int nblk, int RS, int BS, int dw_tabs, int staged) {
    SmemLayout L;
    L.a_off = 0;
    L.raw_off = L.a_off + AR * kTile;
    L.w_off = L.raw_off + RS * kTile;
    L.c_off = L.w_off + BS * kTile;                  // 128 bytes of 0x80: one core matrix, both operands of the offset MMA
    L.dw_off = L.c_off + 128;                        // float [dw_tabs][nblk][128]
    L.da_off = L.dw_off + dw_tabs * nblk * 128 * 4;  // half  [2][nblk][128]
    L.st_off = L.da_off + 2 * nblk * 128 * 2;        // store buffers: kEpiWarps x (32 rows x staged columns) fp32
    L.st_off = (L.st_off + 1023u) & ~1023u;          // the swizzle patterns of the store buffers repeat every 256 to 1024 bytes
    L.bar_off = L.st_off + kEpiWarps * 32 * staged * 4;
    L.bar_off = (L.bar_off + 15u) & ~15u;
    L.total = L.bar_off + 8 * kNumBarriers + 16;
    return L;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float r; asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c)); return r;
}
__device__ __forceinline__ float min3(float a, float b, float c) {
    float r; asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c)); return r;
}
__device__ __forceinline__ int f2i_rz(float x) {
    int r; asm("cvt.rzi.s32.f32 %0, %1;" : "=r"(r) : "f"(x)); return r;
}
// (c << 16) | (sat_s8(a) << 8) | sat_s8(b)
__device__ __forceinline__ uint32_t pack_s8(int a, int b, uint32_t c) {
    uint32_t r; asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); return r;
}

// Quantizes the 32 fp32 values of one token row of a raw stage (Q8_1 rule) into the int8 A tile and
// returns the block scale.  Bit-exact with the host quantizer:
//   vmax = the first element of maximum magnitude, d = vmax / -128, q = min(round-half-away(x * (1 / d)), 127).
// round-half-away(y) = trunc(y + copysign(0.5, y)) with the addition rounded toward zero (a nearest
// rounding could carry 0.49999997 + 0.5 up to 1); the conversion saturates at [-128, 127].
__device__ __forceinline__ float quantize_row(const uint8_t* raw, uint8_t* at, int row, int c0) {
    float x[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float4 t = *reinterpret_cast<const float4*>(raw + sw128_off(row, c));
        x[4 * c] = t.x; x[4 * c + 1] = t.y; x[4 * c + 2] = t.z; x[4 * c + 3] = t.w;
    }
    float vpos = fmaxf(x[0], x[1]), vneg = fminf(x[0], x[1]);
#pragma unroll
    for (int i = 2; i < 32; i += 2) { vpos = max3(vpos, x[i], x[i + 1]); vneg = min3(vneg, x[i], x[i + 1]); }
    const float amax = fmaxf(vpos, -vneg);
    float vmax;
    if (vpos == -vneg && amax != 0.0f) {        // +a and -a both present: the first one wins
        vmax = 0.0f;
#pragma unroll
        for (int i = 31; i >= 0; --i) if (fabsf(x[i]) == amax) vmax = x[i];
    } else {
        vmax = (vpos == amax) ? vpos : vneg;
    }
    const float d = (amax == 0.0f) ? 0.0f : vmax * -0.0078125f;
    const float inv = (d == 0.0f) ? 0.0f : 1.0f / d;
    const uint64_t inv2 = pack2(inv, inv);
    uint32_t packed[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        int qi[4];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint64_t y2 = fmul2(pack2(x[4 * w + 2 * e], x[4 * w + 2 * e + 1]), inv2);
            const uint64_t h2 = (y2 & 0x8000000080000000ull) | 0x3F0000003F000000ull;     // copysign(0.5, y)
            float t0, t1;
            unpack2(fadd2_rz(y2, h2), t0, t1);
            qi[2 * e] = f2i_rz(t0);
            qi[2 * e + 1] = f2i_rz(t1);
        }
        packed[w] = pack_s8(qi[1], qi[0], pack_s8(qi[3], qi[2], 0u));
    }
    *reinterpret_cast<uint4*>(at + sw128_off(row, c0)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    *reinterpret_cast<uint4*>(at + sw128_off(row, c0 + 1)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    return d;
}

// Two rows at a time (rows `row` and `row + 32`): the two dependency chains interleave, which roughly doubles the
// instruction-level parallelism of the quantizer warps.
__device__ __forceinline__ void quantize_rows2(const uint8_t* raw, uint8_t* at, int row, int c0, float& d_out0, float& d_out1) {
    float x[2][32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const float4 t = *reinterpret_cast<const float4*>(raw + sw128_off(row + 32 * u, c));
            x[u][4 * c] = t.x; x[u][4 * c + 1] = t.y; x[u][4 * c + 2] = t.z; x[u][4 * c + 3] = t.w;
        }
    }
    float vpos[2], vneg[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) { vpos[u] = fmaxf(x[u][0], x[u][1]); vneg[u] = fminf(x[u][0], x[u][1]); }
#pragma unroll
    for (int i = 2; i < 32; i += 2) {
#pragma unroll
        for (int u = 0; u < 2; ++u) { vpos[u] = max3(vpos[u], x[u][i], x[u][i + 1]); vneg[u] = min3(vneg[u], x[u][i], x[u][i + 1]); }
    }
    uint64_t inv2[2];
    float d[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const float amax = fmaxf(vpos[u], -vneg[u]);
        float vmax;
        if (vpos[u] == -vneg[u] && amax != 0.0f) {        // +a and -a both present: the first one wins
            vmax = 0.0f;
#pragma unroll
            for (int i = 31; i >= 0; --i) if (fabsf(x[u][i]) == amax) vmax = x[u][i];
        } else {
            vmax = (vpos[u] == amax) ? vpos[u] : vneg[u];
        }
        d[u] = (amax == 0.0f) ? 0.0f : vmax * -0.0078125f;
        const float inv = (d[u] == 0.0f) ? 0.0f : 1.0f / d[u];
        inv2[u] = pack2(inv, inv);
    }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        uint32_t packed[2][4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                int qi[4];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int i0 = 16 * hf + 4 * w + 2 * e;
                    const uint64_t y2 = fmul2(pack2(x[u][i0], x[u][i0 + 1]), inv2[u]);
                    const uint64_t h2 = (y2 & 0x8000000080000000ull) | 0x3F0000003F000000ull;     // copysign(0.5, y)
                    float t0, t1;
                    unpack2(fadd2_rz(y2, h2), t0, t1);
                    qi[2 * e] = f2i_rz(t0);
                    qi[2 * e + 1] = f2i_rz(t1);
                }
                packed[u][w] = pack_s8(qi[1], qi[0], pack_s8(qi[3], qi[2], 0u));
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
            *reinterpret_cast<uint4*>(at + sw128_off(row + 32 * u, c0 + hf)) = make_uint4(packed[u][0], packed[u][1], packed[u][2], packed[u][3]);
    }
    d_out0 = d[0]; d_out1 = d[1];
}

// Activation quantizer as a kernel of its own (the two-pass form of the product): X fp32 [Ntok][K] -> int8 [Ntok][K]
// plus the block scales as fp16 [token tile][nblk][128], the layout the product kernel's scale table has in shared
// memory.  Eight threads per quant block, four elements each; same rule, bit for bit, as quantize_row above (the first
// element of maximum magnitude gives d = vmax / -128; q = round-half-away(x * (1 / d)) saturated to [-128, 127]).
// Rows past Ntok (the tail of the last token tile) only get a zero scale.
__global__ void __launch_bounds__(256)
quantize_q8_planar_kernel(const float* __restrict__ X, int8_t* __restrict__ Aq, __half* __restrict__ da_t,
                          int Ntok, int K, int nblk, long long nthreads) {
    pdl_launch_dependents();
    pdl_wait();
    const long long g = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (g >= nthreads) return;                    // nthreads is a multiple of 8: whole 8-thread groups leave together
    const int sub = static_cast<int>(g & 7);
    const long long ib = g >> 3;
    const int row = static_cast<int>(ib / nblk), kb = static_cast<int>(ib - static_cast<long long>(row) * nblk);
    const bool live = row < Ntok;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    const size_t off = static_cast<size_t>(row) * K + kb * 32 + sub * 4;
    if (live) v = *reinterpret_cast<const float4*>(X + off);
    const float x[4] = {v.x, v.y, v.z, v.w};
    float amax = fabsf(x[0]), vmax = x[0];
    int idx = sub * 4;
#pragma unroll
    for (int e = 1; e < 4; ++e) {
        if (fabsf(x[e]) > amax) { amax = fabsf(x[e]); vmax = x[e]; idx = sub * 4 + e; }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
        const float ov = __shfl_xor_sync(0xffffffffu, vmax, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oa > amax || (oa == amax && oi < idx)) { amax = oa; vmax = ov; idx = oi; }
    }
    const float d = (amax == 0.0f) ? 0.0f : vmax * -0.0078125f;
    const float inv = (d == 0.0f) ? 0.0f : 1.0f / d;
    if (live) {
        int qi[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float y = x[e] * inv;
            float t;
            asm("add.rz.f32 %0, %1, %2;" : "=f"(t) : "f"(y), "f"(copysignf(0.5f, y)));
            qi[e] = f2i_rz(t);
        }
        *reinterpret_cast<uint32_t*>(Aq + off) = pack_s8(qi[1], qi[0], pack_s8(qi[3], qi[2], 0u));
    }
    if (sub == 0) da_t[(static_cast<size_t>(row >> 7) * nblk + kb) * 128 + (row & 127)] = __float2half_rn(d);
}

// The same quantizer for K a multiple of 128, built for bandwidth: a CTA takes a tile of 128 token rows x KW elements
// (KW = 128 or 256); a thread handles 32-byte pieces (eight values, four threads per quant block), consecutive threads
// consecutive pieces of a row, so a warp reads 1 KB and writes 256 bytes contiguously, with four pieces per thread in
// flight.  The scales of the tile go through shared memory and leave as KW / 32 contiguous rows of 128.
template <int KW>
__global__ void __launch_bounds__(256)
quantize_q8_planar_tile_kernel(const float* __restrict__ X, int8_t* __restrict__ Aq, __half* __restrict__ da_t,
                               int Ntok, int K, int nblk) {
    constexpr int NB = KW / 32;                   // quant blocks per row of the tile
    constexpr int PIECES = 128 * KW / 8;          // 32-byte pieces in the tile
    constexpr int ITERS = PIECES / 256;
    __shared__ __half sc[NB][128];
    pdl_launch_dependents();
    pdl_wait();
    const int tile_row0 = blockIdx.y * 128, k0 = blockIdx.x * KW;
#pragma unroll 4
    for (int it = 0; it < ITERS; ++it) {
        const int c = it * 256 + threadIdx.x;
        const int r = c / (KW / 8), pc = c % (KW / 8);            // row in the tile, piece in the row
        const int row = tile_row0 + r;
        const bool live = row < Ntok;
        const size_t off = static_cast<size_t>(row) * K + k0 + pc * 8;
        float x[8];
        if (live) {
            const float4 v0 = __ldg(reinterpret_cast<const float4*>(X + off));
            const float4 v1 = __ldg(reinterpret_cast<const float4*>(X + off + 4));
            x[0] = v0.x; x[1] = v0.y; x[2] = v0.z; x[3] = v0.w; x[4] = v1.x; x[5] = v1.y; x[6] = v1.z; x[7] = v1.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = 0.0f;
        }
        const int sub = pc & 3;
        float amax = fabsf(x[0]), vmax = x[0];
        int idx = sub * 8;
#pragma unroll
        for (int e = 1; e < 8; ++e) {
            if (fabsf(x[e]) > amax) { amax = fabsf(x[e]); vmax = x[e]; idx = sub * 8 + e; }
        }
#pragma unroll
        for (int o = 2; o > 0; o >>= 1) {
            const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
            const float ov = __shfl_xor_sync(0xffffffffu, vmax, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (oa > amax || (oa == amax && oi < idx)) { amax = oa; vmax = ov; idx = oi; }
        }
        const float d = (amax == 0.0f) ? 0.0f : vmax * -0.0078125f;
        const float inv = (d == 0.0f) ? 0.0f : 1.0f / d;
        if (live) {
            int qi[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float y = x[e] * inv;
                float t;
                asm("add.rz.f32 %0, %1, %2;" : "=f"(t) : "f"(y), "f"(copysignf(0.5f, y)));
                qi[e] = f2i_rz(t);
            }
            uint2 o2;
            o2.x = pack_s8(qi[1], qi[0], pack_s8(qi[3], qi[2], 0u));
            o2.y = pack_s8(qi[5], qi[4], pack_s8(qi[7], qi[6], 0u));
            *reinterpret_cast<uint2*>(Aq + off) = o2;
        }
        if (sub == 0) sc[pc >> 2][r] = __float2half_rn(live ? d : 0.0f);
    }
    __syncthreads();
    // NB rows of 128 scales: [token tile][kb][128]
    for (int i = threadIdx.x; i < NB * 64; i += 256) {
        const int kb = i >> 6, pr = i & 63;
        const __half2 h2 = *reinterpret_cast<const __half2*>(&sc[kb][2 * pr]);
        *reinterpret_cast<__half2*>(da_t + (static_cast<size_t>(blockIdx.y) * nblk + blockIdx.x * NB + kb) * 128 + 2 * pr) = h2;
    }
}

// Refill of the weight-scale table in shared memory, fp32 [nblk][128] of d_w * 2^49 for one weight column block (used
// when the tables of all column blocks do not fit).  Thread `etid` of the 512 epilogue threads handles column
// etid % 128.  Not inlined: these run once per column block and must not take registers from the block loop.
//   load (16-byte form, nblk a multiple of 8): eight consecutive blocks of the column, kept as raw halves so that
//   nothing waits for the load until the values are needed
static __device__ __noinline__ uint4 q8_dw_load_vec(const __half* Wd, int Mout, int nblk, int nbx, int etid) {
    const int mo = nbx * 128 + (etid & 127), kb0 = (etid >> 7) * 8;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (mo < Mout && kb0 < nblk) raw = __ldg(reinterpret_cast<const uint4*>(Wd + static_cast<size_t>(mo) * nblk + kb0));
    return raw;
}
//   publish: wait until every epilogue warp has finished with the table before (phase parity `free_par` of dw_free),
//   write this thread's values, arrive on dw_full
static __device__ __noinline__ bool q8_dw_publish_vec(uint4 raw, float* dw_s, int nblk, int etid, int lane, uint32_t dw_free,
                                                      uint32_t dw_full, uint32_t free_par, volatile int* cta_abort, int* err) {
    if (!mbar_wait(dw_free, free_par, cta_abort, err, 0x1402)) return false;
    const float kTwo49 = __uint_as_float((127u + 49u) << 23);
    const int col = etid & 127, kb0 = (etid >> 7) * 8;
    const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        if (kb0 + 2 * t < nblk) {
            dw_s[(kb0 + 2 * t) * 128 + col] = __half2float(__ushort_as_half(static_cast<unsigned short>(rw[t] & 0xffffu))) * kTwo49;
            dw_s[(kb0 + 2 * t + 1) * 128 + col] = __half2float(__ushort_as_half(static_cast<unsigned short>(rw[t] >> 16))) * kTwo49;
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(dw_full);
    return true;
}
//   any nblk: every fourth block of the column per thread, loaded and published in one go
static __device__ __noinline__ bool q8_dw_fill_scalar(const __half* Wd, int Mout, int nblk, int nbx, float* dw_s, int etid, int lane,
                                                      uint32_t dw_free, uint32_t dw_full, uint32_t free_par,
                                                      volatile int* cta_abort, int* err) {
    const float kTwo49 = __uint_as_float((127u + 49u) << 23);
    const int mo = nbx * 128 + (etid & 127);
    const __half* src = Wd + static_cast<size_t>(mo) * nblk + (etid >> 7);
    float wv[kMaxKT];
#pragma unroll
    for (int t = 0; t < kMaxKT; ++t)
        wv[t] = (mo < Mout && 4 * t + (etid >> 7) < nblk) ? __half2float(src[4 * t]) * kTwo49 : 0.0f;
    if (!mbar_wait(dw_free, free_par, cta_abort, err, 0x1402)) return false;
#pragma unroll
    for (int t = 0; t < kMaxKT; ++t) {
        const int i = etid + t * (32 * kEpiWarps);
        if (i < nblk * 128) dw_s[i] = wv[t];
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(dw_full);
    return true;
}

// SUMI: also write the raw int32 block sums (tests); QW: quantizer warps; RESIDENT: the weight-scale tables of all column
// blocks are in shared memory (the instance then holds no refill code: even unused, it cost the block loop registers,
// 98 against 81 us at 65536 x 128 x 1024)
// STAGED: the results leave through the per-warp store buffers (the instance then holds none of the other store paths).
template <bool SUMI, int QW, bool RESIDENT, bool STAGED>
__global__ void __launch_bounds__(Roles<QW>::kThreads, 1)
umma_q8_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
               const __grid_constant__ CUtensorMap tmC, const Q8Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    uint8_t* sg = smem_raw;
    pdl_launch_dependents();        // the next kernel of the stream may set itself up while this one runs (see pdl_wait below)
    if ((smem_base & 1023u) != 0u) {
        pdl_wait();             // the swizzled tiles need a 1024-byte aligned base: refuse to run otherwise
        if (threadIdx.x == 0) { p.err[0] = ST_DEVICE_ABORT; p.err[1] = 0x1001; }
        return;
    }
    const SmemLayout L = q8_layout(p.AR, p.nblk, p.RS, p.BS, p.dw_tabs, p.staged);
    const uint32_t bar0 = smem_base + L.bar_off;
    auto raw_full = [&](int s) { return bar0 + 8u * s; };
    auto raw_empty = [&](int s) { return bar0 + 8u * (kMaxStages + s); };
    auto w_full = [&](int s) { return bar0 + 8u * (2 * kMaxStages + s); };
    auto w_empty = [&](int s) { return bar0 + 8u * (3 * kMaxStages + s); };
    auto a_full = [&](int slot) { return bar0 + 8u * (4 * kMaxStages + slot); };                  // slot < 2 * kMaxKT
    auto a_empty = [&](int slot) { return bar0 + 8u * (4 * kMaxStages + 2 * kMaxKT + slot); };
    auto t_full = [&](int s) { return bar0 + 8u * (4 * kMaxStages + 4 * kMaxKT + s); };
    auto t_empty = [&](int s) { return bar0 + 8u * (4 * kMaxStages + 4 * kMaxKT + 4 + s); };
    auto epi_done = [&](int b) { return bar0 + 8u * (4 * kMaxStages + 4 * kMaxKT + 8 + b); };
    const uint32_t dw_full = bar0 + 8u * (4 * kMaxStages + 4 * kMaxKT + 10);
    const uint32_t dw_free = bar0 + 8u * (4 * kMaxStages + 4 * kMaxKT + 11);
    uint8_t* tail = sg + L.bar_off + 8 * kNumBarriers;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
    volatile int* cta_abort = reinterpret_cast<volatile int*>(tail + 8);

    float* dw_s = reinterpret_cast<float*>(sg + L.dw_off);
    __half* da_s = reinterpret_cast<__half*>(sg + L.da_off);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kQuantWarps = QW, kFirstQuantWarp = Roles<QW>::kFirstQuantWarp;
    constexpr int kTmaWarp = Roles<QW>::kTmaWarp, kMmaWarp = Roles<QW>::kMmaWarp, kThreads = Roles<QW>::kThreads;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), kQuantWarps);
            mbar_init(w_full(s), 1); mbar_init(w_empty(s), 1);
        }
        for (int k = 0; k < 2 * kMaxKT; ++k) {
            // four arrivals per quantizer warp and K step (a short last step pads); one by the TMA thread when the
            // activations arrive quantized
            mbar_init(a_full(k), p.preq ? 1 : kQuantWarps * 4);
            mbar_init(a_empty(k), 1);
        }
        for (int s = 0; s < 4; ++s) { mbar_init(t_full(s), 1); mbar_init(t_empty(s), kEpiWarps); }
        mbar_init(epi_done(0), kEpiWarps); mbar_init(epi_done(1), kEpiWarps);
        mbar_init(dw_full, kEpiWarps); mbar_init(dw_free, kEpiWarps);
        *cta_abort = 0;
        fence_barrier_init();
    }
    if (warp == kMmaWarp) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512); tmem_relinquish(); }
    if (warp == kTmaWarp && lane == 0) { prefetch_tmap(&tmX); prefetch_tmap(&tmW); }
    if (threadIdx.x < 32) reinterpret_cast<uint32_t*>(sg + L.c_off)[threadIdx.x] = 0x80808080u;
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // barriers, TMEM and descriptors are set up: from here on global memory is touched, which needs the kernels before this
    // one in the stream to be complete
    pdl_wait();

    const int total_items = p.m_tiles * p.groups;
    // The k-th work item of this CTA: token tile `mt`, weight column blocks [nb0, nb1).  Two schedules:
    //   strided: item = (token tile, column-block group), CTA c takes items c, c + grid, c + 2 grid, ...
    //   flat:    the (token tile, column block) units in row-major order are cut into `grid` contiguous ranges of
    //            equal length (to within one unit) and a range is walked token tile by token tile; a token tile cut
    //            by a range boundary is quantized by both neighbours.  Balances the load when there are several,
    //            but not a multiple of `grid`, token tiles per CTA.
    // Every role walks the same sequence.
    auto item_at = [&](uint32_t k, int& mt, int& nb0, int& nb1) -> bool {
        if (p.flat) {
            const long long nB = p.n_blocks, U = static_cast<long long>(p.m_tiles) * nB;
            const long long u0 = U * blockIdx.x / gridDim.x, u1 = U * (blockIdx.x + 1) / gridDim.x;
            if (u1 <= u0) return false;
            mt = static_cast<int>(u0 / nB) + static_cast<int>(k);
            const long long lo = max(u0, mt * nB), hi = min(u1, (mt + 1) * nB);
            if (lo >= hi) return false;
            nb0 = static_cast<int>(lo - mt * nB); nb1 = static_cast<int>(hi - mt * nB);
            return true;
        }
        const long long item = blockIdx.x + static_cast<long long>(k) * gridDim.x;
        if (item >= total_items) return false;
        mt = static_cast<int>(item / p.groups);
        nb0 = static_cast<int>(item % p.groups) * p.blocks_per_group;
        nb1 = min(nb0 + p.blocks_per_group, p.n_blocks);
        return true;
    };

    if (warp == kTmaWarp) {
        // ---------------- both TMA streams, one thread: activations (128 x 32 fp32 per quant block) and
        // weights (128 rows x 128 int8 per K step).  Each ring is served as soon as its next stage is free.
        if (lane == 0) {
            uint32_t x_it = 0, w_it = 0;                 // item counters of the two streams
            int x_kb = 0, x_s = 0; uint32_t x_ph = 0;
            int x_mt = 0, x_nb0 = 0, x_nb1 = 0;
            bool x_done = !item_at(x_it, x_mt, x_nb0, x_nb1);
            int x_row0 = x_mt * 128;
            int w_ks = 0, w_s = 0; uint32_t w_ph = 0;
            int w_mt = 0, w_nb = 0, w_nb1 = 0;
            bool w_done = !item_at(w_it, w_mt, w_nb, w_nb1);
            long long t0 = 0; uint32_t idle = 0;
            while (!(x_done && w_done)) {
                bool progress = false;
                if (p.preq) {
                    // quantized activations: one int8 tile per K step straight into the A ring (x_kb counts K steps, x_s /
                    // x_ph are the ring position); the first step of an item also brings the item's scale table, once the
                    // epilogue has finished with the table of this parity (two items ago)
                    bool can = !x_done && mbar_test(a_empty(x_s), x_ph ^ 1u);
                    if (can && x_kb == 0 && x_it >= 2) can = mbar_test(epi_done(x_it & 1u), ((x_it >> 1) - 1u) & 1u);
                    if (can) {
                        const uint32_t tab = (x_kb == 0) ? static_cast<uint32_t>(p.nblk) * 256u : 0u;
                        mbar_arrive_expect_tx(a_full(x_s), kTile + tab);
                        tma_load_3d(smem_base + L.a_off + x_s * kTile, &tmX, a_full(x_s), x_kb * 128, x_row0, 0);
                        if (tab != 0u)
                            bulk_load(smem_base + L.da_off + (x_it & 1u) * tab, p.da_t + static_cast<size_t>(x_mt) * p.nblk * 128, tab,
                                      a_full(x_s));
                        if (++x_s == p.AR) { x_s = 0; x_ph ^= 1u; }
                        if (++x_kb == p.KT) {
                            x_kb = 0; x_done = !item_at(++x_it, x_mt, x_nb0, x_nb1);
                            x_row0 = x_mt * 128;
                        }
                        progress = true;
                    }
                } else if (!x_done && mbar_test(raw_empty(x_s), x_ph ^ 1u)) {
                    mbar_arrive_expect_tx(raw_full(x_s), kTile);
                    tma_load_3d(smem_base + L.raw_off + x_s * kTile, &tmX, raw_full(x_s), x_kb * 32, x_row0, 0);
                    if (++x_s == p.RS) { x_s = 0; x_ph ^= 1u; }
                    if (++x_kb == p.nblk) {
                        x_kb = 0; x_done = !item_at(++x_it, x_mt, x_nb0, x_nb1);
                        x_row0 = x_mt * 128;
                    }
                    progress = true;
                }
                if (!w_done && mbar_test(w_empty(w_s), w_ph ^ 1u)) {
                    mbar_arrive_expect_tx(w_full(w_s), kTile);
                    tma_load_3d(smem_base + L.w_off + w_s * kTile, &tmW, w_full(w_s), w_ks * 128, w_nb * 128, 0);
                    if (++w_s == p.BS) { w_s = 0; w_ph ^= 1u; }
                    if (++w_ks == p.KT) {
                        w_ks = 0;
                        if (++w_nb == w_nb1) w_done = !item_at(++w_it, w_mt, w_nb, w_nb1);
                    }
                    progress = true;
                }
                if (progress) { idle = 0; continue; }
                if (idle == 0) t0 = clock64();
                if ((++idle & 63u) == 0u) {
                    if (*cta_abort) break;
                    if (clock64() - t0 > kWaitCycles) {
                        *cta_abort = 1; p.err[0] = ST_DEVICE_ABORT; p.err[1] = 0x1101; __threadfence();
                        break;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issue: one instruction per quant block, each into a fresh TMEM slot ----------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(2, 1, 1, 0, 0, 128, 128);
            const uint64_t da0 = make_smem_desc(smem_base + L.a_off, 16, 1024, kLayoutSW128);
            const uint64_t db0 = make_smem_desc(smem_base + L.w_off, 16, 1024, kLayoutSW128);
            // Offset operands: every element is the unsigned byte 128, in the unswizzled K-major layout.  All core
            // matrices (8 rows x 16 bytes) are equal, so both strides of the descriptor are zero and one 128-byte core
            // matrix stands for the whole 128 x 32 operand.  The second instruction adds 32 * 128 * 128 = 2^19 to every
            // block sum: the sums read back by the epilogue are never negative.
            const uint32_t idesc_off = make_idesc(2, 0, 0, 0, 0, 128, 128);
            const uint64_t dc = make_smem_desc(smem_base + L.c_off, 0, 0, 0);
            uint32_t bcnt = 0, n_it = 0, w_ph = 0; int w_s = 0; bool ok = true;
            uint32_t a_slot0 = 0, a_par0 = 0;           // slot and parity of K step 0 of the current item
            int mt = 0, nb0 = 0, nb1 = 0;
            for (; ok && item_at(n_it, mt, nb0, nb1); ++n_it) {
                for (int nb = nb0; nb < nb1 && ok; ++nb) {
                    uint32_t a_slot = a_slot0, a_par = a_par0;              // A slots form a ring over (item, K step)
                    for (int ks = 0; ks < p.KT; ++ks, a_slot = (a_slot + 1 == static_cast<uint32_t>(p.AR)) ? 0u : a_slot + 1u,
                                                    a_par ^= (a_slot == 0u) ? 1u : 0u) {
                        if (nb == nb0) {
                            if (!mbar_wait(a_full(a_slot), a_par, cta_abort, p.err, 0x1301)) { ok = false; break; }
                        }
                        if (!mbar_wait(w_full(w_s), w_ph, cta_abort, p.err, 0x1302)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t da = da0 + static_cast<uint64_t>(a_slot * (kTile >> 4));
                        const uint64_t db = db0 + static_cast<uint64_t>(w_s * (kTile >> 4));
                        const int nstep = min(4, p.nblk - 4 * ks);
                        if ((p.nblk & 3) == 0) {
                            // K a multiple of 128: every K step is four blocks on slots 0..3, handed over in pairs
                            // (slots 0-1 behind barrier 0, slots 2-3 behind barrier 2): half as many handshakes, and
                            // slots, barriers and descriptors are compile-time offsets
                            const uint32_t par = ((bcnt >> 2) & 1u) ^ 1u;
#pragma unroll
                            for (int g = 0; g < 2; ++g) {
                                if (!mbar_wait(t_empty(2 * g), par, cta_abort, p.err, 0x1303)) { ok = false; break; }
                                tc_fence_after();
#pragma unroll
                                for (int j = 2 * g; j < 2 * g + 2; ++j) {
                                    umma<MmaKind::I8>(tmem_base + j * 128u, da + 2u * j, db + 2u * j, idesc, 0u);
                                    umma<MmaKind::I8>(tmem_base + j * 128u, dc, dc, idesc_off, 1u);
                                }
                                umma_commit(t_full(2 * g));
                            }
                            bcnt += 4;
                        } else
                        for (int j = 0; j < nstep; ++j, ++bcnt) {
                            const uint32_t slot = bcnt & 3u;
                            if (!mbar_wait(t_empty(slot), ((bcnt >> 2) & 1u) ^ 1u, cta_abort, p.err, 0x1303)) { ok = false; break; }
                            tc_fence_after();
                            umma<MmaKind::I8>(tmem_base + slot * 128u, da + 2u * j, db + 2u * j, idesc, 0u);
                            umma<MmaKind::I8>(tmem_base + slot * 128u, dc, dc, idesc_off, 1u);
                            umma_commit(t_full(slot));
                        }
                        if (!ok) break;
                        umma_commit(w_empty(w_s));
                        if (++w_s == p.BS) { w_s = 0; w_ph ^= 1u; }
                        if (nb == nb1 - 1) umma_commit(a_empty(a_slot));
                    }
                }
                for (int ks = 0; ks < p.KT; ++ks) { if (++a_slot0 == static_cast<uint32_t>(p.AR)) { a_slot0 = 0; a_par0 ^= 1u; } }
            }
        }
        __syncwarp();
    } else if (warp >= kFirstQuantWarp && warp < kFirstQuantWarp + kQuantWarps) {
        // ---------------- quantizers: warp 2 owns token rows 0-63 of the tile, warp 3 rows 64-127 ------------
        // (nothing to do when the activations arrive quantized)
        const int row0 = (warp - kFirstQuantWarp) * (128 / kQuantWarps) + lane;
        uint32_t n_it = 0, x_ph = 0; int x_s = 0; bool ok = p.preq == 0;
        uint32_t a_slot = 0, a_par = 0;                 // ring position of the K step being quantized
        int mt = 0, nb0 = 0, nb1 = 0;
        for (; ok && item_at(n_it, mt, nb0, nb1); ++n_it) {
            if (n_it >= 2) {    // the scale table of this parity was last read by the epilogue two items ago
                if (!mbar_wait(epi_done(n_it & 1u), ((n_it >> 1) - 1u) & 1u, cta_abort, p.err, 0x1501)) { ok = false; break; }
            }
            __half* da_w = da_s + (n_it & 1u) * p.nblk * 128;
            for (int kb = 0; kb < p.nblk; ++kb) {
                if ((kb & 3) == 0) {     // the tensor core must have finished with the previous user of this slot
                    if (!mbar_wait(a_empty(a_slot), a_par ^ 1u, cta_abort, p.err, 0x1502)) { ok = false; break; }
                }
                if (!mbar_wait(raw_full(x_s), x_ph, cta_abort, p.err, 0x1503)) { ok = false; break; }
                const uint8_t* raw = sg + L.raw_off + x_s * kTile;
                uint8_t* at = sg + L.a_off + a_slot * kTile;
                const int c0 = (kb & 3) * 2;
                float d0 = 1.0f, d1 = 1.0f;
                if (kQuantWarps == 4) d0 = quantize_row(raw, at, row0, c0);
                else quantize_rows2(raw, at, row0, c0, d0, d1);
                da_w[kb * 128 + row0] = __float2half_rn(d0);
                if (kQuantWarps == 2) da_w[kb * 128 + row0 + 32] = __float2half_rn(d1);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(raw_empty(x_s));
                    mbar_arrive(a_full(a_slot));
                    if (kb == p.nblk - 1) { for (int pad = (kb & 3) + 1; pad < 4; ++pad) mbar_arrive(a_full(a_slot)); }
                }
                if (++x_s == p.RS) { x_s = 0; x_ph ^= 1u; }
                if ((kb & 3) == 3 || kb == p.nblk - 1) { if (++a_slot == static_cast<uint32_t>(p.AR)) { a_slot = 0; a_par ^= 1u; } }
            }
        }
    } else {
        // ---------------- epilogue: per-block rescale, fp32 accumulation in registers ----------------------
        const int q = warp & 3;                            // TMEM lane quarter
        const int cg = (warp - kFirstEpiWarp) >> 2;        // which 32 of the 128 columns
        const int etid = threadIdx.x - kFirstEpiWarp * 32; // 0..511
        const int row = q * 32 + lane;                     // token row inside the tile
        const uint32_t taddr0 = tmem_base + cg * 32 + (static_cast<uint32_t>(q * 32) << 16);
        uint32_t bcnt = 0, n_it = 0, dwcnt = 0; bool ok = true;
        const bool dw_resident = RESIDENT || p.dw_tabs == p.n_blocks;  // (one column block in all: trivially resident)
        const float kTwo100 = __uint_as_float((127u + 100u) << 23), kTwo49 = __uint_as_float((127u + 49u) << 23);
        if (dw_resident) {
            for (int i = etid; i < p.n_blocks * p.nblk * 128; i += 32 * kEpiWarps) {
                const int nbq = i / (p.nblk * 128), r = i - nbq * p.nblk * 128;
                const int kb = r >> 7, col = r & 127;
                const int mo = nbq * 128 + col;
                dw_s[i] = (mo < p.Mout) ? __half2float(p.Wd[static_cast<size_t>(mo) * p.nblk + kb]) * kTwo49 : 0.0f;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(dw_full);
            if (!mbar_wait(dw_full, 0u, cta_abort, p.err, 0x1404)) ok = false;
        }
        int mt = 0, nb0 = 0, nb1 = 0;
        for (; ok && item_at(n_it, mt, nb0, nb1); ++n_it) {
            const int tok = mt * 128 + row;
            const uint32_t da_a0 = smem_base + L.da_off + ((n_it & 1u) * p.nblk * 128 + row) * 2;      // this row's d_a, block 0
            for (int nb = nb0; nb < nb1 && ok; ++nb) {
                // weight scales as fp32 [nblk][128] per column block.  When the tables of all column blocks fit
                // they were staged once before the first item; otherwise this block's table is refilled here:
                // wait until every epilogue warp has finished with the previous one, fill, publish.
                const uint32_t dw_a0 = smem_base + L.dw_off + ((p.dw_tabs > 1 ? nb : 0) * p.nblk * 128 + cg * 32) * 4;
                if (!RESIDENT && !dw_resident) {
                    // The first column block of an item fills the table here; the later ones were filled at the end of the
                    // block before them (loads issued before its result stores, table written between them) when the scales
                    // can be read with 16-byte loads.
                    const uint32_t free_par = (dwcnt & 1u) ^ 1u;
                    if (!p.dw_vec) {
                        if (!q8_dw_fill_scalar(p.Wd, p.Mout, p.nblk, nb, dw_s, etid, lane, dw_free, dw_full, free_par, cta_abort, p.err)) { ok = false; break; }
                    } else if (nb == nb0) {
                        const uint4 raw = q8_dw_load_vec(p.Wd, p.Mout, p.nblk, nb, etid);
                        if (!q8_dw_publish_vec(raw, dw_s, p.nblk, etid, lane, dw_free, dw_full, free_par, cta_abort, p.err)) { ok = false; break; }
                    }
                    if (!mbar_wait(dw_full, dwcnt & 1u, cta_abort, p.err, 0x1403)) { ok = false; break; }
                }
                float acc[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[j] = 0.0f;
                // The block sums arrive as non-negative integers s' = s + 2^19 < 2^23.  Read as a float, such a bit
                // pattern is the denormal s' * 2^-149: no int -> float conversion is needed.  With d_a scaled by 2^100
                // and the table holding d_w * 2^49 (exact scalings of fp16 values),
                //   g   = fma(s' * 2^-149, d_a * 2^100, -2^-30 * d_a) = round(s * d_a) * 2^-49   (2^19 * d_a is exact)
                //   acc = fma(g, d_w * 2^49, acc)                                                = acc + s * d_a * d_w
                // The per-thread scalar d_a goes first so that only the second fma needs a table value.
                auto rescale = [&](const uint32_t (&v)[16], int h, int kb, float da, float dc) {
                    const uint32_t dwp = dw_a0 + (kb * 128 + h * 16) * 4;
                    if (SUMI && tok < p.Ntok) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int mo = nb * 128 + cg * 32 + h * 16 + j;
                            if (mo < p.Mout)
                                p.sumi_out[(static_cast<size_t>(tok) * p.Mout + mo) * p.nblk + kb] = static_cast<int>(v[j]) - (1 << 19);
                        }
                    }
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        const float4 w4 = lds_f4(dwp + j4 * 16);
                        acc[h * 16 + j4 * 4 + 0] = fmaf(fmaf(__uint_as_float(v[j4 * 4 + 0]), da, dc), w4.x, acc[h * 16 + j4 * 4 + 0]);
                        acc[h * 16 + j4 * 4 + 1] = fmaf(fmaf(__uint_as_float(v[j4 * 4 + 1]), da, dc), w4.y, acc[h * 16 + j4 * 4 + 1]);
                        acc[h * 16 + j4 * 4 + 2] = fmaf(fmaf(__uint_as_float(v[j4 * 4 + 2]), da, dc), w4.z, acc[h * 16 + j4 * 4 + 2]);
                        acc[h * 16 + j4 * 4 + 3] = fmaf(fmaf(__uint_as_float(v[j4 * 4 + 3]), da, dc), w4.w, acc[h * 16 + j4 * 4 + 3]);
                    }
                };
                // Two 16-column halves per block, software-pipelined: while one half is rescaled the TMEM load of
                // the next half (of this block or of the next one) is in flight.
                uint32_t va[16], vb[16];
                if (!mbar_wait(t_full(bcnt & 3u), (bcnt >> 2) & 1u, cta_abort, p.err, 0x1401)) { ok = false; break; }
                tc_fence_after();
                tmem_ld16(taddr0 + (bcnt & 3u) * 128u, va);
                uint16_t da_raw = lds_u16(da_a0);                     // d_a of block 0 of this row
                // One block held by `slot`; the next block's first half is loaded from `nslot` in the middle.  `rel_bar`
                // (when not 0) is arrived on once this block is in registers, `acq_bar` (when not 0) is waited for
                // with parity `acq_par` before the next block is touched.
                auto one_block = [&](int kb, uint32_t slot, uint32_t nslot, bool has_next, uint32_t rel_bar, uint32_t acq_bar,
                                     uint32_t acq_par) -> bool {
                    const float da = __half2float(__ushort_as_half(da_raw)) * kTwo100;
                    const float dc = da * __uint_as_float(0x80080000u);      // -2^-130 * (d_a * 2^100)
                    tmem_ld_wait();
                    tmem_ld16(taddr0 + slot * 128u + 16u, vb);
                    // the next block's scale, in flight during the math; only when that block is already known to be
                    // complete (same pair): its scale is written by the quantizer just before its MMA can be issued
                    if (has_next && acq_bar == 0u) da_raw = lds_u16(da_a0 + (kb + 1) * 256);
                    rescale(va, 0, kb, da, dc);
                    tmem_ld_wait();
                    if (rel_bar != 0u) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(rel_bar);         // the slot(s) may take their next blocks already
                    }
                    if (has_next) {
                        if (acq_bar != 0u) {
                            if (!mbar_wait(acq_bar, acq_par, cta_abort, p.err, 0x1401)) return false;
                            tc_fence_after();
                            da_raw = lds_u16(da_a0 + (kb + 1) * 256);
                        }
                        tmem_ld16(taddr0 + nslot * 128u, va);
                    }
                    rescale(vb, 1, kb, da, dc);
                    return true;
                };
                if (!SUMI && (STAGED || (p.nblk & 3) == 0)) {      // (the STAGED instances are only launched with K % 128 == 0)
                    // Fast path (every K that is a multiple of 128): groups of four blocks on slots 0..3, handed over in
                    // pairs.  Slot numbers, TMEM offsets and table offsets are compile-time constants; the two table
                    // pointers advance once per group.  Per block: the two 16-column halves are software-pipelined (the
                    // TMEM load of the next half is in flight during the arithmetic of this one).
                    auto half16 = [&](const uint32_t (&v)[16], auto off, float da, float dc, uint32_t dwp, int h) {
                        constexpr int OFF = decltype(off)::value;
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {
                            float4 w4;
                            if (j4 == 0) w4 = lds_f4_at<OFF>(dwp);
                            else if (j4 == 1) w4 = lds_f4_at<OFF + 16>(dwp);
                            else if (j4 == 2) w4 = lds_f4_at<OFF + 32>(dwp);
                            else w4 = lds_f4_at<OFF + 48>(dwp);
                            acc[h * 16 + j4 * 4 + 0] = fmaf(fmaf(__uint_as_float(v[j4 * 4 + 0]), da, dc), w4.x, acc[h * 16 + j4 * 4 + 0]);
                            acc[h * 16 + j4 * 4 + 1] = fmaf(fmaf(__uint_as_float(v[j4 * 4 + 1]), da, dc), w4.y, acc[h * 16 + j4 * 4 + 1]);
                            acc[h * 16 + j4 * 4 + 2] = fmaf(fmaf(__uint_as_float(v[j4 * 4 + 2]), da, dc), w4.z, acc[h * 16 + j4 * 4 + 2]);
                            acc[h * 16 + j4 * 4 + 3] = fmaf(fmaf(__uint_as_float(v[j4 * 4 + 3]), da, dc), w4.w, acc[h * 16 + j4 * 4 + 3]);
                        }
                    };
                    using std::integral_constant;
                    const uint32_t tf0 = t_full(0), tf2 = t_full(2), te0 = t_empty(0), te2 = t_empty(2);
                    const float kDc = __uint_as_float(0x80080000u);           // -2^-130: times d_a * 2^100 gives -2^-30 * d_a
                    uint32_t par = (bcnt >> 2) & 1u;
                    uint32_t dwp = dw_a0, dap = da_a0;
                    const int ngroups = p.nblk >> 2;
                    for (int g4 = 0; g4 < ngroups; ++g4, dwp += 2048u, dap += 1024u, par ^= 1u) {
                        float da, dc;
                        // ---- block 0 (slot 0); block 1 is in the same pair: its sums and its scale are complete
                        da = __half2float(__ushort_as_half(da_raw)) * kTwo100; dc = da * kDc;
                        tmem_ld_wait();
                        tmem_ld16(taddr0 + 16u, vb);
                        da_raw = lds_u16_at<256>(dap);
                        half16(va, integral_constant<int, 0>{}, da, dc, dwp, 0);
                        tmem_ld_wait();
                        tmem_ld16(taddr0 + 128u, va);
                        half16(vb, integral_constant<int, 64>{}, da, dc, dwp, 1);
                        // ---- block 1 (slot 1): releases slots 0-1, then needs the pair 2-3
                        da = __half2float(__ushort_as_half(da_raw)) * kTwo100; dc = da * kDc;
                        tmem_ld_wait();
                        tmem_ld16(taddr0 + 128u + 16u, vb);
                        half16(va, integral_constant<int, 512>{}, da, dc, dwp, 0);
                        tmem_ld_wait();
                        tc_fence_before();
                        mbar_arrive_lane0(te0, lane);
                        if (!mbar_wait(tf2, par, cta_abort, p.err, 0x1401)) { ok = false; break; }
                        tc_fence_after();
                        da_raw = lds_u16_at<512>(dap);
                        tmem_ld16(taddr0 + 256u, va);
                        half16(vb, integral_constant<int, 512 + 64>{}, da, dc, dwp, 1);
                        // ---- block 2 (slot 2)
                        da = __half2float(__ushort_as_half(da_raw)) * kTwo100; dc = da * kDc;
                        tmem_ld_wait();
                        tmem_ld16(taddr0 + 256u + 16u, vb);
                        da_raw = lds_u16_at<768>(dap);
                        half16(va, integral_constant<int, 1024>{}, da, dc, dwp, 0);
                        tmem_ld_wait();
                        tmem_ld16(taddr0 + 384u, va);
                        half16(vb, integral_constant<int, 1024 + 64>{}, da, dc, dwp, 1);
                        // ---- block 3 (slot 3): releases slots 2-3; the next group starts on the pair 0-1
                        da = __half2float(__ushort_as_half(da_raw)) * kTwo100; dc = da * kDc;
                        tmem_ld_wait();
                        tmem_ld16(taddr0 + 384u + 16u, vb);
                        half16(va, integral_constant<int, 1536>{}, da, dc, dwp, 0);
                        tmem_ld_wait();
                        tc_fence_before();
                        mbar_arrive_lane0(te2, lane);
                        if (g4 + 1 < ngroups) {
                            if (!mbar_wait(tf0, par ^ 1u, cta_abort, p.err, 0x1401)) { ok = false; break; }
                            tc_fence_after();
                            da_raw = lds_u16_at<1024>(dap);
                            tmem_ld16(taddr0, va);
                        }
                        half16(vb, integral_constant<int, 1536 + 64>{}, da, dc, dwp, 1);
                    }
                    bcnt += static_cast<uint32_t>(p.nblk);
                } else if (STAGED) {
                } else if ((p.nblk & 3) == 0) {
                    // the same schedule with run-time slot numbers (the instance that also writes the int32 sums)
                    for (int kb0 = 0; kb0 < p.nblk && ok; kb0 += 4, bcnt += 4) {
                        const uint32_t par = (bcnt >> 2) & 1u;
                        const bool more = kb0 + 4 < p.nblk;
                        if (!one_block(kb0 + 0, 0, 1, true, 0u, 0u, 0u) ||
                            !one_block(kb0 + 1, 1, 2, true, t_empty(0), t_full(2), par) ||
                            !one_block(kb0 + 2, 2, 3, true, 0u, 0u, 0u) ||
                            !one_block(kb0 + 3, 3, 0, more, t_empty(2), t_full(0), par ^ 1u)) { ok = false; break; }
                    }
                } else {
                    for (int kb = 0; kb < p.nblk; ++kb, ++bcnt) {
                        const uint32_t nx = bcnt + 1u;
                        if (!one_block(kb, bcnt & 3u, nx & 3u, kb + 1 < p.nblk, t_empty(bcnt & 3u), t_full(nx & 3u), (nx >> 2) & 1u)) { ok = false; break; }
                    }
                }
                if (!ok) break;
                uint4 raw_next = make_uint4(0u, 0u, 0u, 0u);
                bool refill_next = false;
                if constexpr (!RESIDENT) {
                    refill_next = !dw_resident && p.dw_vec && nb + 1 < nb1;
                    if (!dw_resident) { __syncwarp(); if (lane == 0) mbar_arrive(dw_free); ++dwcnt; }
                    if (refill_next) raw_next = q8_dw_load_vec(p.Wd, p.Mout, p.nblk, nb + 1, etid);       // in flight during the result stores
                }
                const int mo0 = nb * 128 + cg * 32;
                if (p.bias != nullptr) {
                    if (mo0 + 32 <= p.Mout && (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.bias + mo0 + j));
                            acc[j] += b4.x; acc[j + 1] += b4.y; acc[j + 2] += b4.z; acc[j + 3] += b4.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (mo0 + j < p.Mout) acc[j] += p.bias[mo0 + j];
                    }
                }
                if (STAGED || (p.c_trans && p.staged)) {
                    // Asynchronous stores, `staged` columns at a time: thread = row writes its 16-byte chunks into the warp's
                    // buffer (rows of 32, 64 or 128 bytes in the TMA swizzle of that width: address bits 4.. XOR address bits
                    // 7.., which also keeps the banks apart), then one lane hands the 32-row box to the TMA unit, which writes
                    // it out while the warp goes on with the next blocks; rows past Ntok and columns past Mout are clipped by
                    // the tensor map.  The buffer is reused once the store before it has finished reading shared memory.
                    auto store_cols = [&](auto sc_c, auto nbuf_c) {
                        constexpr int SC = decltype(sc_c)::value, NBUF = decltype(nbuf_c)::value, PITCH = SC * 4, NCH = SC / 4;
                        const uint32_t stage0 = smem_base + L.st_off + (warp - kFirstEpiWarp) * (32 * PITCH * NBUF);
                        const uint32_t row_off = lane * PITCH;
#pragma unroll
                        for (int c0 = 0; c0 < 32; c0 += SC) {
                            const uint32_t stage = stage0 + ((c0 / SC) % NBUF) * (32 * PITCH);
                            if (lane == 0) { if (NBUF == 2) bulk_wait_read_but_one(); else bulk_wait_read_all(); }
                            __syncwarp();
#pragma unroll
                            for (int j = 0; j < NCH; ++j) {
                                const uint32_t off = row_off + (j << 4);
                                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(stage + (off ^ (((off >> 7) & (NCH - 1)) << 4))),
                                             "f"(acc[c0 + 4 * j]), "f"(acc[c0 + 4 * j + 1]), "f"(acc[c0 + 4 * j + 2]), "f"(acc[c0 + 4 * j + 3]) : "memory");
                            }
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                tma_store_3d(&tmC, stage, mo0 + c0, mt * 128 + q * 32, 0);
                                bulk_commit_group();
                            }
                            // the next table is written while the TMA unit reads the buffer
                            if constexpr (!RESIDENT) {
                                if (c0 == 0 && refill_next) {
                                    refill_next = false;
                                    if (!q8_dw_publish_vec(raw_next, dw_s, p.nblk, etid, lane, dw_free, dw_full, (dwcnt & 1u) ^ 1u, cta_abort, p.err)) ok = false;
                                }
                            }
                        }
                    };
                    using std::integral_constant;
                    // one buffer of 16 columns per warp.  (The template also takes 8 or 32 columns and two buffers used in
                    // turn; every further instance costs the block loop instruction-cache room: 89 against 86 us at
                    // 65536 x 128 x 1024 with four instances.)
                    store_cols(integral_constant<int, 16>{}, integral_constant<int, 1>{});
                } else if (!STAGED && p.vec32_ok && mo0 + 32 <= p.Mout) {
                    // No room for store buffers (K = 1024: the resident A tile).  A thread holds 32 consecutive floats of
                    // its row; stored as they lie, every store instruction would touch 32 different lines with 16 bytes each
                    // and the load/store unit takes one line per cycle.  Regrouped (two exchange steps over the lane bits 3-4),
                    // lane l holds, for s = 0..3, the 32-byte piece (l >> 3) of row 8 s + (l & 7): a store instruction then
                    // writes eight whole 128-byte lines.
                    rows_to_line_pieces(acc, lane);
                    const int piece = lane >> 3;
#pragma unroll
                    for (int s4 = 0; s4 < 4; ++s4) {
                        // register group s4 now holds floats 8 * piece .. 8 * piece + 7 of row (lane & 7) + 8 * s4
                        const int r = q * 32 + (lane & 7) + 8 * s4;
                        const int t2 = mt * 128 + r;
                        if (t2 < p.Ntok) {
                            float* dst = p.C + static_cast<size_t>(t2) * p.Mout + mo0 + 8 * piece;
                            asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst),
                                         "f"(acc[8 * s4]), "f"(acc[8 * s4 + 1]), "f"(acc[8 * s4 + 2]), "f"(acc[8 * s4 + 3]),
                                         "f"(acc[8 * s4 + 4]), "f"(acc[8 * s4 + 5]), "f"(acc[8 * s4 + 6]), "f"(acc[8 * s4 + 7]) : "memory");
                        }
                    }
                } else if (!STAGED && tok < p.Ntok) {
                    if (p.c_trans) {
                        float* dst = p.C + static_cast<size_t>(tok) * p.Mout + mo0;
                        if (p.vec_ok && mo0 + 32 <= p.Mout) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) if (mo0 + j < p.Mout) dst[j] = acc[j];
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (mo0 + j < p.Mout) p.C[static_cast<size_t>(mo0 + j) * p.Ntok + tok] = acc[j];
                    }
                }
                if constexpr (!RESIDENT) {
                    if (refill_next && !q8_dw_publish_vec(raw_next, dw_s, p.nblk, etid, lane, dw_free, dw_full, (dwcnt & 1u) ^ 1u, cta_abort, p.err)) ok = false;
                }
                if (!ok) break;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_done(n_it & 1u));
        }
        if (lane == 0) bulk_wait_all();              // this warp's result stores are complete before the CTA leaves
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace


// W: Q8_0R weights ([Mout*nblk*32] int8 plane followed by [Mout*nblk] half scales); X fp32 [Ntok][K];
// M = weight rows (out features), N = tokens, as in the reference's launcher.
// Bytes of scratch the two-pass form needs for N tokens of K elements: the int8 matrix, then the scale tables.
size_t umma_q8_scratch_bytes(int N, int K) {
    const size_t aq = (static_cast<size_t>(N) * K + 255) & ~static_cast<size_t>(255);
    return aq + static_cast<size_t>((N + 127) / 128) * (K / 32) * 256;
}

// scratch: null = quantize inside the product kernel (one pass over X, nothing written but C); otherwise a device
// buffer of umma_q8_scratch_bytes(N, K) that receives the quantized activations from a kernel of its own first.
int launch_umma_q8(const void* W, const float* X, float* C, int M, int N, int K, int c_trans, const float* bias,
                   int* sumi_out, cudaStream_t st, void* scratch) {
    if (!W || !X || !C || M <= 0 || N <= 0 || K <= 0) return ST_BAD_ARGS;
    if (K % 32) return ST_BAD_K;
    if (K > 128 * kMaxKT) return ST_UNSUPPORTED_PATH;
    if ((reinterpret_cast<uintptr_t>(W) & 15u) || (reinterpret_cast<uintptr_t>(X) & 15u)) return ST_UNSUPPORTED_PATH;
    int* err = device_error_ptr();
    if (!err) return ST_LAUNCH;

    Q8Params p{};
    p.Mout = M; p.Ntok = N; p.K = K; p.nblk = K / 32; p.KT = (K + 127) / 128;
    p.m_tiles = (N + 127) / 128;
    p.n_blocks = (M + 127) / 128;
    const int sms = num_sms();
    int groups = 1;
    if (p.m_tiles < sms) {
        groups = (sms + p.m_tiles - 1) / p.m_tiles;
        if (groups > p.n_blocks) groups = p.n_blocks;
    }
    p.blocks_per_group = (p.n_blocks + groups - 1) / groups;
    p.groups = (p.n_blocks + p.blocks_per_group - 1) / p.blocks_per_group;
    p.vec_ok = c_trans && ((reinterpret_cast<uintptr_t>(C) & 15u) == 0) && (M % 4 == 0);
    p.vec32_ok = c_trans && ((reinterpret_cast<uintptr_t>(C) & 31u) == 0) && (M % 8 == 0);
    // Shared memory: the quantized A tile and the activation-scale table are fixed; then, in this order of
    // preference, a second A tile (the next item is quantized while this one multiplies), the scale tables
    // of all column blocks (no refill, at most 32 KB), the per-warp store buffers; what is left goes to the
    // two rings, and an option is dropped when fewer than five stages would remain.
    const int budget = 227 * 1024;               // the most dynamic shared memory one CTA can have
    const int total_items = p.m_tiles * p.groups;
    // more token tiles than SMs and enough work per token tile (column blocks x K steps; measured break-even at 8) that
    // quantizing the cut tiles twice pays off: cut the work into equal contiguous ranges instead
    p.flat = (p.groups == 1 && p.n_blocks * p.KT >= 8 && p.m_tiles > sms && p.m_tiles % sms != 0) ? 1 : 0;
    p.preq = scratch != nullptr ? 1 : 0;
    int abuf = ((p.KT <= 2 || p.preq) && total_items > sms) ? 2 : 1;
    const bool ring = p.blocks_per_group == 1 && p.KT >= 3;    // every item has one column block: A is consumed once
    p.AR = ring ? (p.preq ? 4 : 3) : p.KT * abuf;
    p.dw_tabs = (p.n_blocks * p.nblk * 512 <= 32 * 1024) ? p.n_blocks : 1;
    p.staged = p.vec_ok ? 16 : 0;
    auto stages_for = [&]() {
        return (budget - static_cast<int>(q8_layout(p.AR, p.nblk, 0, 0, p.dw_tabs, p.staged).total)) / kTile;
    };
    // what is given up, in this order, while fewer than five ring stages would remain (four for the store buffers):
    // the resident scale tables, the second A tile, the store buffers.  (At K = 1024 the resident A tile leaves no room
    // for them: narrower buffers paid for with a raw stage were measured slower, 370 against 334 us at 65536 x 1024 x 512.)
    if (stages_for() < 5 && p.dw_tabs > 1) p.dw_tabs = 1;
    if (stages_for() < 5 && abuf > 1) { abuf = 1; p.AR = p.KT; }
    // (activations that arrive quantized need no raw stages: two weight stages are enough there)
    if (stages_for() < (p.preq ? 2 : 4)) p.staged = 0;
    int stages = stages_for();
    if (stages < (p.preq ? 2 : 3)) return ST_UNSUPPORTED_PATH;
    if (stages > 2 * kMaxStages) stages = 2 * kMaxStages;
    if (p.preq) {
        // no raw fp32 stages: everything goes to the weight ring
        p.RS = 0; p.BS = stages > kMaxStages ? kMaxStages : stages;
    } else if (p.blocks_per_group == 1) {
        // the weights of an item are one pass over K: two stages suffice, the activation ring carries the HBM stream
        p.BS = 2; p.RS = stages - 2;
    } else {
        p.BS = stages / 2; p.RS = stages - p.BS;
    }
    if (p.RS > kMaxStages) p.RS = kMaxStages;
    if (p.BS > kMaxStages) p.BS = kMaxStages;
    const __half* Wd = reinterpret_cast<const __half*>(static_cast<const int8_t*>(W) + static_cast<size_t>(M) * p.nblk * 32);
    p.Wd = Wd; p.C = C; p.bias = bias; p.sumi_out = sumi_out; p.c_trans = c_trans; p.err = err;
    p.dw_vec = (p.nblk % 8 == 0) && ((reinterpret_cast<uintptr_t>(Wd) & 15u) == 0);

    CUtensorMap tmX, tmW, tmC;
    if (p.preq) {
        if (reinterpret_cast<uintptr_t>(scratch) & 255u) return ST_BAD_ARGS;
        int8_t* aq = static_cast<int8_t*>(scratch);
        __half* da_t = reinterpret_cast<__half*>(aq + ((static_cast<size_t>(N) * K + 255) & ~static_cast<size_t>(255)));
        p.da_t = da_t;
        const long long nthreads = static_cast<long long>(p.m_tiles) * 128 * p.nblk * 8;
        const long long qgrid = nthreads / 256;
        if (qgrid > 0x7fffffffLL) return ST_UNSUPPORTED_PATH;
        const bool x_aligned = (reinterpret_cast<uintptr_t>(X) & 15u) == 0;
        // (the tile kernels want a few CTAs per SM; with few token tiles the one-piece-per-thread kernel spreads wider)
        const bool wide = static_cast<long long>(p.m_tiles) * (K / 128) >= 4LL * sms;
        if (wide && x_aligned && K % 256 == 0 && p.m_tiles <= 65535)
            launch_pdl(quantize_q8_planar_tile_kernel<256>, dim3(K / 256, p.m_tiles), dim3(256), 0, st, X, aq, da_t, N, K, p.nblk);
        else if (wide && x_aligned && K % 128 == 0 && p.m_tiles <= 65535)
            launch_pdl(quantize_q8_planar_tile_kernel<128>, dim3(K / 128, p.m_tiles), dim3(256), 0, st, X, aq, da_t, N, K, p.nblk);
        else
            launch_pdl(quantize_q8_planar_kernel, dim3(static_cast<unsigned>(qgrid)), dim3(256), 0, st, X, aq, da_t, N, K, p.nblk, nthreads);
        if (cudaGetLastError() != cudaSuccess) return ST_QUANT;
        if (!make_tmap_3d(&tmX, TmaType::U8, aq, K, N, 1, static_cast<uint64_t>(K), 0, 128, 128, 1)) return ST_UNSUPPORTED_PATH;
    } else
    if (!make_tmap_3d(&tmX, TmaType::F32, X, K, N, 1, static_cast<uint64_t>(K) * 4, 0, 32, 128, 1)) return ST_UNSUPPORTED_PATH;
    if (!make_tmap_3d(&tmW, TmaType::U8, W, K, M, 1, static_cast<uint64_t>(K), 0, 128, 128, 1)) return ST_UNSUPPORTED_PATH;
    tmC = tmW;                                   // only read by the kernel when the results leave through TMA stores
    // box = staged columns x 32 rows; swizzle of the box width (32, 64 or 128 bytes)
    // (one buffer of 16 columns: its second store of a column block waits about 1 200 cycles for the first one to be read)
    if (p.staged && !make_tmap_3d(&tmC, TmaType::F32, C, M, N, 1, static_cast<uint64_t>(M) * 4, 0, p.staged, 32, 3)) p.staged = 0;

    const int smem = static_cast<int>(q8_layout(p.AR, p.nblk, p.RS, p.BS, p.dw_tabs, p.staged).total);
    static int configured_smem[64] = {0};
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && configured_smem[dev] < smem) {
        const auto attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
        bool ok_attr = true;
        auto set = [&](auto kernel) { if (cudaFuncSetAttribute(kernel, attr, 227 * 1024) != cudaSuccess) ok_attr = false; };
        set(umma_q8_kernel<false, 2, true, true>); set(umma_q8_kernel<false, 2, false, true>);
        set(umma_q8_kernel<false, 4, true, true>); set(umma_q8_kernel<false, 4, false, true>);
        set(umma_q8_kernel<false, 2, false, false>); set(umma_q8_kernel<false, 4, false, false>);
        set(umma_q8_kernel<true, 2, false, false>);
        if (!ok_attr) { cudaGetLastError(); return ST_LAUNCH; }
        configured_smem[dev] = 227 * 1024;
    }
    const int grid = total_items < sms ? total_items : sms;
    const bool resident = p.dw_tabs == p.n_blocks;
    // four quantizer warps where the quantizer sets the pace: items with one column block, and K = 1024 with up to four
    // (the A tile is not double-buffered there, so every item starts by waiting for its first blocks; measured 177 against
    // 194 us at 65536 x 1024 x 256, 317 against 324 at N = 512, but 584 against 547 at N = 1024)
    const bool four = p.blocks_per_group == 1 || (!p.preq && p.KT == kMaxKT && p.blocks_per_group <= 4);
    const bool staged = p.staged != 0 && c_trans && (p.nblk & 3) == 0;
    const int th2 = Roles<2>::kThreads, th4 = Roles<4>::kThreads;
    if (sumi_out != nullptr) launch_pdl(umma_q8_kernel<true, 2, false, false>, dim3(grid), dim3(th2), smem, st, tmX, tmW, tmC, p);
    else if (!staged) {
        if (four) launch_pdl(umma_q8_kernel<false, 4, false, false>, dim3(grid), dim3(th4), smem, st, tmX, tmW, tmC, p);
        else launch_pdl(umma_q8_kernel<false, 2, false, false>, dim3(grid), dim3(th2), smem, st, tmX, tmW, tmC, p);
    } else if (four) {
        if (resident) launch_pdl(umma_q8_kernel<false, 4, true, true>, dim3(grid), dim3(th4), smem, st, tmX, tmW, tmC, p);
        else launch_pdl(umma_q8_kernel<false, 4, false, true>, dim3(grid), dim3(th4), smem, st, tmX, tmW, tmC, p);
    } else {
        if (resident) launch_pdl(umma_q8_kernel<false, 2, true, true>, dim3(grid), dim3(th2), smem, st, tmX, tmW, tmC, p);
        else launch_pdl(umma_q8_kernel<false, 2, false, true>, dim3(grid), dim3(th2), smem, st, tmX, tmW, tmC, p);
    }
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

}  // namespace ppml_b200
