// umma_attn.cu -- fused attention forward on tcgen05 for head dim 32 (the model's 8 x 32 heads).
//
//   O = softmax(scale * Q K^T + bias) V,  denominator (l + eps),  LSE = m + log(l + eps)
//
// Work item = one (batch, head, 128-query tile); keys are walked in tiles of 64.  CTAs are persistent, two per SM (256 TMEM
// columns, about 105 KB of shared memory, 192 threads each), so one CTA's softmax overlaps the other's loads and
// tensor work.  (Key tiles of 32 with three CTAs per SM measured 5-15 % slower.)
// Operands: fp32 Q/K/V on kind::tf32 (rounded by the TMA unit), or bf16 / fp16 Q/K/V on kind::f16 with P in the same
// 16-bit type; scores, softmax, running sums and the output are fp32 in both cases.  The 16-bit tiles have rows of
// 64 bytes, so Q and K use the 64-byte swizzle (K-major) and V the same swizzle in its row-index-contiguous form.
//   warp 0      TMA: Q tile once; per key tile the bias tile (128 rows x kBN keys fp32, when a bias is
//               given; it lands in the P buffer of that tile and is overwritten in place by P), K (kBN keys x 32 floats, K-major, 128-byte swizzle) and V (the same
//               box in the 32-byte-chunk swizzle: V[key][d] has d contiguous, which is the "row index contiguous"
//               form of the B operand of P V, so V needs no transposition); fp32 -> tf32 rounding by the TMA unit
//   warp 1      MMA issue: S = Q K^T (four K = 8 tf32 MMAs, N = kBN) into one of two TMEM S buffers,
//               then O_part = P V (kBN / 8 MMAs of K = 8, N = 32) into one of two TMEM O buffers
//   warps 2-5   softmax, one thread per query row: the scores of the tile from TMEM into registers, scale +
//               bias + mask, running max / sum, P (rounded to tf32) into shared memory as the next MMA's K-major
//               A operand, then o = alpha * o + O_part in fp32 registers, one tile late
// Every wait is bounded; rows past L and keys past Lk are zero-filled by TMA and masked.
#include <math_constants.h>

#include "kernels.h"
#include "tma_host.h"

namespace ppml_b200 {

namespace {

constexpr int kD = 32;                       // head dim handled here
constexpr int kBM = 128, kBN = 64;           // query tile, key tile
constexpr int kSubP = 128 * 128;             // bytes: 128 rows of one 128-byte swizzle atom (32 floats or 64 16-bit values)
constexpr int kTileP = (kBN / 32) * kSubP;   // bias tile: 128 rows x 64 floats as two 32-float atoms; fp32 P has the same
                                             //   shape, 16-bit P is the first atom alone
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 256;          // S buffers at columns 0 and kBN, O_part buffers at 2 kBN and 2 kBN + 32
constexpr int kCtasPerSm = 2;

// ELEM: 0 = fp32 operands (tf32 products), 1 = bf16, 2 = fp16.  Shared-memory map (offsets from the 1024-aligned
// base); two CTAs per SM leave about 113 KB each.
template <int ELEM>
struct Cfg {
    static constexpr bool k16 = ELEM != 0;
    static constexpr int kRow = k16 ? 64 : 128;              // bytes of one Q / K / V row of 32 elements
    static constexpr int kTileQ = kBM * kRow;
    static constexpr int kTileKV = kBN * kRow;
    static constexpr int kOffQ = 0;
    static constexpr int kOffK = kOffQ + kTileQ;             // 2 stages
    static constexpr int kOffV = kOffK + 2 * kTileKV;        // 2 stages
    // 2 buffers of bias-then-P: TMA puts the bias tile of key tile j into buffer j % 2 in the layout of fp32 P, every
    // softmax thread reads its bias values and later writes its P values over them
    static constexpr int kOffP = kOffV + 2 * kTileKV;
    static constexpr int kOffBar = kOffP + 2 * kTileP;
    static constexpr int kSmemBytes = kOffBar + 256;         // the dynamic shared memory is declared 1024-byte aligned: no slack
    static constexpr uint32_t kFmt = ELEM == 0 ? 2u : (ELEM == 1 ? 1u : 0u);      // operand format field of the instruction
    static constexpr MmaKind kKind = k16 ? MmaKind::F16 : MmaKind::TF32;
    static constexpr uint32_t kLayQK = k16 ? kLayoutSW64 : kLayoutSW128;
    static constexpr uint32_t kSboQK = k16 ? 512u : 1024u;   // 8 rows of the swizzle atom
    static constexpr int kStepsS = k16 ? 2 : 4;              // instructions per score product (K = 16 or 8 of the 32)
    static_assert(kOffP % 1024 == 0 && kOffK % 512 == 0 && kOffV % 512 == 0, "tile alignment");
};

// 2^x on the transcendental unit (about 2 ulp); results below the normal range flush to 0, 2^-inf = 0
__device__ __forceinline__ float ex2_approx(float x) {
    float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r; asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c)); return r;
}

// act(gate) * O for the 32 values of a row, the reference's formulas (src/backend/CPUKernels.cpp:1903-1916).  The kind is
// tested once per row, not per element (32 copies of the switch with their expf / tanhf bodies made the gate cost as much
// as the rest of the kernel: 20.8 M against 15.3 M executed instructions, stalls on instruction fetch).  Sigmoid and SiLU,
// what the model uses, take the hardware exp2 and reciprocal approximations (2 ulp, far inside the 1e-3 of the tf32 products).
// one instruction each on the transcendental unit (the IEEE-rounded reciprocal is a sequence of a dozen)
__device__ __forceinline__ float ex2_fast(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float rcp_fast(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ void gate_row(int kind, const float (&g)[32], float (&o)[32]) {
    switch (kind) {
        case 1:
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= rcp_fast(1.0f + ex2_fast(-1.4426950408889634f * g[j]));
            break;
        case 2:
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= g[j] * rcp_fast(1.0f + ex2_fast(-1.4426950408889634f * g[j]));
            break;
        case 3:
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= 0.5f * g[j] * (1.0f + tanhf(0.7978845608028654f * (g[j] + 0.044715f * g[j] * g[j] * g[j])));
            break;
        case 4:
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= tanhf(g[j]);
            break;
        case 5:
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= g[j] > 0.0f ? g[j] : 0.0f;
            break;
        default:
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= g[j];
            break;
    }
}

// two probabilities as one 32-bit word of the operand type, the first in the low half (the lower key index)
template <int ELEM>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    uint32_t w;
    if constexpr (ELEM == 1) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
    return w;
}

struct AttnParams {
    int B, H, L, Lk;
    int causal;
    float scale, eps;
    const float* bias;
    long long bias_batch_stride;
    float* O;
    float* LSE;
    int q_tiles, k_tiles;
    int total_items;             // B * H * q_tiles
    int o_align32;               // O rows are 32-byte aligned: they can be written with 256-bit stores
    long long o_b, o_h, o_l;     // element strides of O over batch, head and query row
    long long g_b, g_h, g_l;     // the same for the gate
    const float* gate;           // optional: O = act(gate) * O
    int act;
    int ft_tiles;                // > 0: a row whose first ft_tiles key tiles hold only -inf scores gives O = 0, LSE = -inf,
                                 //      as the reference's CPU kernel does for its first key tile (src/ops/FlashAttn.cpp:94-121)
    int* err;
};

template <int ELEM>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
umma_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmB, const AttnParams p) {
    using C = Cfg<ELEM>;
    constexpr int kOffQ = C::kOffQ, kOffK = C::kOffK, kOffV = C::kOffV, kOffP = C::kOffP, kOffBar = C::kOffBar;
    constexpr int kTileQ = C::kTileQ, kTileKV = C::kTileKV;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t sb = smem_u32(smem_raw);
    uint8_t* sg = smem_raw;
    if ((sb & 1023u) != 0u) {                    // the swizzled tiles need a 1024-byte aligned base: refuse to run otherwise
        if (threadIdx.x == 0) { p.err[0] = ST_DEVICE_ABORT; p.err[1] = 0x2001; }
        return;
    }
    const uint32_t bar0 = sb + kOffBar;
    const uint32_t q_full = bar0, q_empty = bar0 + 8u * 23;
    auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (3 + s); };
    auto v_full = [&](int s) { return bar0 + 8u * (5 + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (7 + s); };
    auto s_full = [&](int s) { return bar0 + 8u * (9 + s); };
    auto s_empty = [&](int s) { return bar0 + 8u * (11 + s); };
    auto o_full = [&](int s) { return bar0 + 8u * (13 + s); };
    auto o_empty = [&](int s) { return bar0 + 8u * (15 + s); };
    auto p_full = [&](int s) { return bar0 + 8u * (17 + s); };
    auto p_empty = [&](int s) { return bar0 + 8u * (19 + s); };
    auto b_full = [&](int s) { return bar0 + 8u * (21 + s); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sg + kOffBar + 8 * 24);
    volatile int* cta_abort = reinterpret_cast<volatile int*>(sg + kOffBar + 8 * 24 + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Work item = (batch * head, 128-query tile).  The CTA is persistent: it walks items blockIdx.x, + gridDim.x, ...
    // and every ring (K, V, S, P / bias, O) keeps running across item boundaries, so the loads and the first score
    // product of the next item overlap the softmax tail and the output stores of the current one.
    auto item_info = [&](int item, int& bh, int& q0, int& ktl) {
        const int qt = item % p.q_tiles;
        bh = item / p.q_tiles;
        q0 = qt * kBM;
        ktl = p.k_tiles;
        // causal: keys beyond the last query row of the tile are never needed
        if (p.causal) { const int last = min(q0 + kBM, p.L); ktl = min(ktl, (min(last, p.Lk) + kBN - 1) / kBN); }
    };

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1); mbar_init(q_empty, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1);
            mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1);
            mbar_init(s_full(s), 1); mbar_init(s_empty(s), 4);
            mbar_init(o_full(s), 1); mbar_init(o_empty(s), 4);
            mbar_init(p_full(s), 4); mbar_init(p_empty(s), 1);
            mbar_init(b_full(s), 1);
        }
        *cta_abort = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols); tmem_relinquish(); }
    if (warp == 0 && lane == 0) { prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); if (p.bias != nullptr) prefetch_tmap(&tmB); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t tc = 0, ic = 0;                     // key tiles and items issued so far
            bool ok = true;
            for (int item = blockIdx.x; item < p.total_items && ok; item += gridDim.x, ++ic) {
                int bh, q0, k_tiles;
                item_info(item, bh, q0, k_tiles);
                const int b = bh / p.H, hh = bh - b * p.H;
                // the Q tile is free once the score products of the previous item have been computed
                if (!mbar_wait(q_empty, (ic & 1u) ^ 1u, cta_abort, p.err, 0x2100)) break;
                mbar_arrive_expect_tx(q_full, kTileQ);
                tma_load_4d(sb + kOffQ, &tmQ, q_full, 0, q0, hh, b);
                const int brow0 = hh * p.L + q0;                         // first bias row of this tile
                const int bbatch = (p.bias_batch_stride != 0) ? b : 0;
                for (int j = 0; j < k_tiles; ++j, ++tc) {
                    const int s = tc & 1; const uint32_t ph = (tc >> 1) & 1u;
                    if (p.bias != nullptr) {
                        // buffer s is free again once the P V product two tiles back has read it
                        if (!mbar_wait(p_empty(s), ph ^ 1u, cta_abort, p.err, 0x2103)) { ok = false; break; }
                        mbar_arrive_expect_tx(b_full(s), kTileP);
#pragma unroll
                        for (int a = 0; a < kBN / 32; ++a)
                            tma_load_3d(sb + kOffP + s * kTileP + a * kSubP, &tmB, b_full(s), j * kBN + 32 * a, brow0, bbatch);
                    }
                    if (!mbar_wait(k_empty(s), ph ^ 1u, cta_abort, p.err, 0x2101)) { ok = false; break; }
                    mbar_arrive_expect_tx(k_full(s), kTileKV);
                    tma_load_4d(sb + kOffK + s * kTileKV, &tmK, k_full(s), 0, j * kBN, hh, b);
                    if (!mbar_wait(v_empty(s), ph ^ 1u, cta_abort, p.err, 0x2102)) { ok = false; break; }
                    mbar_arrive_expect_tx(v_full(s), kTileKV);
                    tma_load_4d(sb + kOffV + s * kTileKV, &tmV, v_full(s), 0, j * kBN, hh, b);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc(1, C::kFmt, C::kFmt, 0, 0, 128, kBN);
            const uint32_t idesc_o = make_idesc(1, C::kFmt, C::kFmt, 0, 1, 128, kD);     // B = V with d (the row index) contiguous
            uint32_t ts = 0, tp = 0, ic = 0;             // score products / P V products / items issued so far
            bool ok = true;
            // software pipeline: S(j+1) is issued before P(j) V(j), so the softmax of tile j+1 can start
            // while the tensor core finishes tile j
            auto issue_s = [&]() -> bool {
                const int s = ts & 1; const uint32_t ph = (ts >> 1) & 1u;
                if (!mbar_wait(k_full(s), ph, cta_abort, p.err, 0x2202)) return false;
                if (!mbar_wait(s_empty(s), ph ^ 1u, cta_abort, p.err, 0x2203)) return false;
                tc_fence_after();
                const uint64_t dq = make_smem_desc(sb + kOffQ, 16, C::kSboQK, C::kLayQK);
                const uint64_t dk = make_smem_desc(sb + kOffK + s * kTileKV, 16, C::kSboQK, C::kLayQK);
#pragma unroll
                for (int kk = 0; kk < C::kStepsS; ++kk)      // 32 bytes of every row per instruction
                    umma<C::kKind>(tmem_base + s * kBN, dq + 2u * kk, dk + 2u * kk, idesc_s, kk ? 1u : 0u);
                umma_commit(k_empty(s));
                umma_commit(s_full(s));
                ++ts;
                return true;
            };
            for (int item = blockIdx.x; item < p.total_items && ok; item += gridDim.x, ++ic) {
                int bh, q0, k_tiles;
                item_info(item, bh, q0, k_tiles);
                if (!mbar_wait(q_full, ic & 1u, cta_abort, p.err, 0x2201)) { ok = false; break; }
                if (!issue_s()) { ok = false; break; }
                if (k_tiles == 1) umma_commit(q_empty);          // every score product of this item has been issued
                for (int j = 0; j < k_tiles && ok; ++j, ++tp) {
                    if (j + 1 < k_tiles) {
                        if (!issue_s()) { ok = false; break; }
                        if (j + 2 == k_tiles) umma_commit(q_empty);
                    }
                    const int s = tp & 1; const uint32_t ph = (tp >> 1) & 1u;
                    if (!mbar_wait(p_full(s), ph, cta_abort, p.err, 0x2204)) { ok = false; break; }
                    if (!mbar_wait(v_full(s), ph, cta_abort, p.err, 0x2205)) { ok = false; break; }
                    if (!mbar_wait(o_empty(s), ph ^ 1u, cta_abort, p.err, 0x2206)) { ok = false; break; }
                    tc_fence_after();
                    if constexpr (C::k16) {
                        // V tile: 64 key rows of 64 bytes in the 64-byte swizzle; a group of 8 keys is 512 bytes (stride
                        // offset), one instruction consumes 16 keys = 1024 bytes.  P: one atom of 64 keys.
                        const uint64_t dv = make_smem_desc(sb + kOffV + s * kTileKV, 4096, 512, kLayoutSW64);
                        const uint64_t dp = make_smem_desc(sb + kOffP + s * kTileP, 16, 1024, kLayoutSW128);
#pragma unroll
                        for (int kk = 0; kk < kBN / 16; ++kk)
                            umma<MmaKind::F16>(tmem_base + 2 * kBN + s * kD, dp + 2u * kk, dv + 64u * kk, idesc_o, kk ? 1u : 0u);
                    } else {
                        // V tile: 64 key rows of 128 bytes in the 32-byte-chunk swizzle; a group of 4 keys is 512 bytes
                        // (stride offset), one instruction consumes 8 keys = 1024 bytes.  P: two 32-key swizzle atoms.
                        const uint64_t dv = make_smem_desc(sb + kOffV + s * kTileKV, 4096, 512, kLayoutSW128Base32);
#pragma unroll
                        for (int a = 0; a < kBN / 32; ++a) {
                            const uint64_t dp = make_smem_desc(sb + kOffP + s * kTileP + a * kSubP, 16, 1024, kLayoutSW128);
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk)
                                umma<MmaKind::TF32>(tmem_base + 2 * kBN + s * kD, dp + 2u * kk, dv + 64u * (a * 4 + kk), idesc_o, (a | kk) ? 1u : 0u);
                        }
                    }
                    umma_commit(p_empty(s));
                    umma_commit(v_empty(s));
                    umma_commit(o_full(s));
                }
            }
        }
        __syncwarp();
    } else {
#include "umma_attn_softmax.inc"
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

}  // namespace

namespace {

template <int ELEM>
int launch_attn_elem(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmB,
                     const AttnParams& p, unsigned grid, cudaStream_t st) {
    static bool configured[64] = {false};
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(umma_attn_kernel<ELEM>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<ELEM>::kSmemBytes) != cudaSuccess) {
            cudaGetLastError();
            return ST_LAUNCH;
        }
        configured[dev] = true;
    }
    umma_attn_kernel<ELEM><<<grid, kThreads, Cfg<ELEM>::kSmemBytes, st>>>(tmQ, tmK, tmV, tmB, p);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

}  // namespace

// elem: 0 = fp32 Q/K/V, 1 = bf16, 2 = fp16 (bias, O and LSE are fp32 in every case)
int launch_umma_attn(const void* Q, const void* K, const void* V, int elem, const float* bias, float* O, float* LSE,
                     int B, int H, int L, int Lk, int d, int causal, float scale, float eps,
                     long long bias_batch_stride, int ft, const AttnLayout& lay, cudaStream_t st) {
    if (d != kD) return ST_UNSUPPORTED_PATH;
    if (ft < 0 || ft % kBN) return ST_UNSUPPORTED_PATH;       // the first-tile rule is checked per key tile of this kernel
    if (elem < 0 || elem > 2) return ST_BAD_ARGS;
    if ((reinterpret_cast<uintptr_t>(Q) & 15u) || (reinterpret_cast<uintptr_t>(K) & 15u) ||
        (reinterpret_cast<uintptr_t>(V) & 15u) || (reinterpret_cast<uintptr_t>(O) & 15u)) return ST_UNSUPPORTED_PATH;
    if (bias && ((reinterpret_cast<uintptr_t>(bias) & 15u) || (Lk % 4) || (bias_batch_stride % 4))) return ST_UNSUPPORTED_PATH;
    int* err = device_error_ptr();
    if (!err) return ST_LAUNCH;
    const long long BH = static_cast<long long>(B) * H;
    AttnParams p{};
    p.B = B; p.H = H; p.L = L; p.Lk = Lk; p.causal = causal; p.scale = scale; p.eps = eps;
    p.bias = bias; p.bias_batch_stride = bias_batch_stride; p.O = O; p.LSE = LSE;
    p.q_tiles = (L + kBM - 1) / kBM; p.k_tiles = (Lk + kBN - 1) / kBN; p.err = err;
    const long long items = BH * p.q_tiles;
    if (items <= 0 || items > 0x7fffffffLL || Lk <= 0) return ST_BAD_ARGS;
    p.total_items = static_cast<int>(items);
    p.o_b = lay.o_b; p.o_h = lay.o_h; p.o_l = lay.o_l; p.gate = lay.gate; p.act = lay.act;
    p.g_b = lay.g_b; p.g_h = lay.g_h; p.g_l = lay.g_l;
    if ((lay.o_b | lay.o_h | lay.o_l) & 3) return ST_UNSUPPORTED_PATH;          // 16-byte rows at least
    if (lay.gate && ((lay.g_b | lay.g_h | lay.g_l) & 3)) return ST_UNSUPPORTED_PATH;
    if (lay.gate && (reinterpret_cast<uintptr_t>(lay.gate) & 15u)) return ST_UNSUPPORTED_PATH;
    p.o_align32 = ((reinterpret_cast<uintptr_t>(O) & 31u) == 0 && ((lay.o_b | lay.o_h | lay.o_l) & 7) == 0 &&
                   (!lay.gate || (reinterpret_cast<uintptr_t>(lay.gate) & 31u) == 0)) ? 1 : 0;
    p.ft_tiles = ft / kBN;
    const long long resident = static_cast<long long>(kCtasPerSm) * num_sms();     // persistent CTAs
    const unsigned grid = static_cast<unsigned>(items < resident ? items : resident);
    CUtensorMap tmQ, tmK, tmV, tmB;
    // fp32 rows are 128 bytes (128-byte swizzle; V in its 32-byte-chunk form), 16-bit rows 64 bytes (64-byte swizzle)
    const TmaType ty = elem == 0 ? TmaType::TF32 : (elem == 1 ? TmaType::BF16 : TmaType::F16);
    const uint64_t es = elem == 0 ? 4 : 2;
    const int sw_qk = elem == 0 ? 1 : 3, sw_v = elem == 0 ? 2 : 3;
    // dims (d, sequence row, head, batch), each with the stride the layout gives it
    if (!make_tmap_4d(&tmQ, ty, Q, kD, L, H, B, lay.q_l * es, lay.q_h * es, lay.q_b * es, kD, kBM, sw_qk)) return ST_UNSUPPORTED_PATH;
    if (!make_tmap_4d(&tmK, ty, K, kD, Lk, H, B, lay.k_l * es, lay.k_h * es, lay.k_b * es, kD, kBN, sw_qk)) return ST_UNSUPPORTED_PATH;
    if (!make_tmap_4d(&tmV, ty, V, kD, Lk, H, B, lay.v_l * es, lay.v_h * es, lay.v_b * es, kD, kBN, sw_v)) return ST_UNSUPPORTED_PATH;
    // bias rows are (head, query) pairs, [B or 1][H * L][Lk]; fp32 as it is (no tf32 rounding)
    tmB = tmQ;
    if (bias) {
        const bool per_batch = bias_batch_stride != 0;
        if (!make_tmap_3d(&tmB, TmaType::F32, bias, Lk, static_cast<uint64_t>(H) * L, per_batch ? B : 1, static_cast<uint64_t>(Lk) * 4,
                          per_batch ? static_cast<uint64_t>(bias_batch_stride) * 4 : 0, 32, kBM, 1)) return ST_UNSUPPORTED_PATH;
    }
    if (elem == 0) return launch_attn_elem<0>(tmQ, tmK, tmV, tmB, p, grid, st);
    if (elem == 1) return launch_attn_elem<1>(tmQ, tmK, tmV, tmB, p, grid, st);
    return launch_attn_elem<2>(tmQ, tmK, tmV, tmB, p, grid, st);
}

}  // namespace ppml_b200
