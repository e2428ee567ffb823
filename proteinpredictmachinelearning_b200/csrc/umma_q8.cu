// umma_q8.cu -- W8A8 block-quantized mul_mat on tcgen05 (kind::i8), Q8_0R weights.
//
//   C[token][out] = sum_blocks float(sum_{32} q_w * q_a) * (d_w * d_a)   (+ bias[out])
//
// The activations never make a round trip through HBM as int8: fp32 rows are pulled in by TMA
// (128 tokens x one 32-element quant block per stage, 128-byte swizzle), quantized from shared
// memory by four warps (one thread per token row: absmax, d = vmax / -128, q = round(x / d)) and
// written as the K-major int8 A operand, which stays resident for all weight column blocks of the
// work item.  The int8 weights stream in by TMA.  Every quant block is ONE tcgen05.mma (K = 32)
// into its own 128-column TMEM slot (four slots rotate); eight epilogue warps drain a slot, convert
// the exact int32 block sums to fp32, scale by d_w * d_a and accumulate in registers in block order.
//
// Warp roles: warps 0-2 = activation TMA (0), weight TMA (1), MMA issue + TMEM owner (2);
// warps 3-18 = epilogue (four warps per TMEM lane quarter, 32 columns each); warps 19.. = quantizers
// (groups of four warps, one thread per token row, groups take quant blocks round-robin).
#include <cuda_fp16.h>

#include "kernels.h"
#include "tma_host.h"

namespace ppml_b200 {

namespace {

// Optional wait profiling (build with -DPPML_Q8_TRACE): CTA 0 adds the cycles each role spends in each
// wait site to a global table; off in normal builds.
#ifdef PPML_Q8_TRACE
__device__ long long g_q8_trace[64];
#define Q8_WAIT(slot, ...)                                                     \
    [&]() {                                                                    \
        const long long t0__ = clock64();                                      \
        const bool r__ = mbar_wait(__VA_ARGS__);                               \
        if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) {                      \
            atomicAdd(reinterpret_cast<unsigned long long*>(&g_q8_trace[slot]), (unsigned long long)(clock64() - t0__)); \
            atomicAdd(reinterpret_cast<unsigned long long*>(&g_q8_trace[32 + slot]), 1ull); }                         \
        return r__;                                                            \
    }()
#define Q8_WAIT_RELAXED(slot, ...) Q8_WAIT(slot, __VA_ARGS__)
#define Q8_WAIT_WARP(slot, ...) Q8_WAIT(slot, __VA_ARGS__)
#define Q8_T0() const long long tq0__ = clock64()
#define Q8_T1(slot) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) {                       \
        atomicAdd(reinterpret_cast<unsigned long long*>(&g_q8_trace[slot]), (unsigned long long)(clock64() - tq0__)); \
        atomicAdd(reinterpret_cast<unsigned long long*>(&g_q8_trace[32 + slot]), 1ull); } } while (0)
#else
#define Q8_WAIT(slot, ...) mbar_wait(__VA_ARGS__)
#define Q8_WAIT_RELAXED(slot, ...) mbar_wait_relaxed(__VA_ARGS__)
#define Q8_WAIT_WARP(slot, ...) mbar_wait(__VA_ARGS__)
#define Q8_T0() do {} while (0)
#define Q8_T1(slot) do {} while (0)
#endif

constexpr int kTile = 128 * 128;          // bytes: one int8 A tile (128 rows x 128 K) == one weight stage == one raw fp32 stage
constexpr int kMaxKT = 8;                 // K <= 1024
constexpr int kMaxStages = 6;
constexpr int kQuantGroups = 1;          // groups of four quantizer warps, taking quant blocks round-robin
constexpr int kEpiWarps = 16;             // four per TMEM lane quarter, 32 output columns each
constexpr int kMiscWarps = 3;             // activation TMA, weight TMA, MMA issue
constexpr int kThreads = 32 * (kMiscWarps + kEpiWarps + 4 * kQuantGroups);

struct Q8Params {
    int Mout, Ntok, K, nblk, KT;
    int m_tiles;               // token tiles
    int n_blocks;              // weight column blocks of 128
    int groups, blocks_per_group;
    int RS, BS;                // ring depths
    int dw_tabs;               // scale tables held in smem: n_blocks (all resident, filled once) or 1 (refilled per column block)
    int staged;                // 1: results leave through per-warp transposition buffers (row-contiguous stores)
    const __half* Wd;          // weight scales [Mout][nblk]
    float* C;
    const float* bias;
    int* sumi_out;
    int c_trans;
    int vec_ok;
    int* err;
};

struct SmemLayout {
    uint32_t a_off, raw_off, w_off, dw_off, da_off, st_off, bar_off, total;
};

constexpr int kStorePitch = 144;                    // bytes per staged row: 32 floats + 16 bytes of padding
constexpr int kStoreBytes = 32 * kStorePitch;       // one epilogue warp's 32 x 32 transposition buffer

__host__ __device__ inline SmemLayout q8_layout(int KT, int nblk, int RS, int BS, int dw_tabs, int staged) {
    SmemLayout L;
    L.a_off = 0;
    L.raw_off = L.a_off + KT * kTile;
    L.w_off = L.raw_off + RS * kTile;
    L.dw_off = L.w_off + BS * kTile;                 // float [dw_tabs][nblk][128]
    L.da_off = L.dw_off + dw_tabs * nblk * 128 * 4;  // half  [2][nblk][128]
    L.st_off = L.da_off + 2 * nblk * 128 * 2;        // staged stores: 16 x kStoreBytes
    L.bar_off = L.st_off + (staged ? 16 * kStoreBytes : 0);
    L.bar_off = (L.bar_off + 15u) & ~15u;
    L.total = L.bar_off + 8 * (4 * kMaxStages + 2 * kMaxKT + 8 + 4) + 16;
    return L;
}

__global__ void __launch_bounds__(kThreads, 1)
umma_q8_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const Q8Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* sg = smem_raw + (smem_base - smem_u32(smem_raw));
    const SmemLayout L = q8_layout(p.KT, p.nblk, p.RS, p.BS, p.dw_tabs, p.staged);
    const uint32_t bar0 = smem_base + L.bar_off;
    auto raw_full = [&](int s) { return bar0 + 8u * s; };
    auto raw_empty = [&](int s) { return bar0 + 8u * (kMaxStages + s); };
    auto w_full = [&](int s) { return bar0 + 8u * (2 * kMaxStages + s); };
    auto w_empty = [&](int s) { return bar0 + 8u * (3 * kMaxStages + s); };
    auto a_full = [&](int k) { return bar0 + 8u * (4 * kMaxStages + k); };
    auto a_empty = [&](int k) { return bar0 + 8u * (4 * kMaxStages + kMaxKT + k); };
    auto t_full = [&](int s) { return bar0 + 8u * (4 * kMaxStages + 2 * kMaxKT + s); };
    auto t_empty = [&](int s) { return bar0 + 8u * (4 * kMaxStages + 2 * kMaxKT + 4 + s); };
    auto epi_done = [&](int b) { return bar0 + 8u * (4 * kMaxStages + 2 * kMaxKT + 8 + b); };
    const uint32_t dw_full = bar0 + 8u * (4 * kMaxStages + 2 * kMaxKT + 10);
    const uint32_t dw_free = bar0 + 8u * (4 * kMaxStages + 2 * kMaxKT + 11);
    uint8_t* tail = sg + L.bar_off + 8 * (4 * kMaxStages + 2 * kMaxKT + 12);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
    volatile int* cta_abort = reinterpret_cast<volatile int*>(tail + 8);

    float* dw_s = reinterpret_cast<float*>(sg + L.dw_off);
    __half* da_s = reinterpret_cast<__half*>(sg + L.da_off);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), 4);
            mbar_init(w_full(s), 1); mbar_init(w_empty(s), 1);
        }
        for (int k = 0; k < kMaxKT; ++k) {
            int nb = p.nblk - 4 * k; nb = nb < 0 ? 0 : (nb > 4 ? 4 : nb);
            mbar_init(a_full(k), nb > 0 ? 4 * nb : 1);
            mbar_init(a_empty(k), 1);
        }
        for (int s = 0; s < 4; ++s) { mbar_init(t_full(s), 1); mbar_init(t_empty(s), kEpiWarps); }
        mbar_init(epi_done(0), kEpiWarps); mbar_init(epi_done(1), kEpiWarps);
        mbar_init(dw_full, kEpiWarps); mbar_init(dw_free, kEpiWarps);
        *cta_abort = 0;
        fence_barrier_init();
    }
    if (warp == 2) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512); tmem_relinquish(); }
    if (warp == 0 && lane == 0) prefetch_tmap(&tmX);
    if (warp == 1 && lane == 0) prefetch_tmap(&tmW);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_items = p.m_tiles * p.groups;
#ifdef PPML_Q8_TRACE
    if (blockIdx.x == 0 && threadIdx.x == 0) g_q8_trace[30] = clock64();
#endif

    if (warp == 0) {
        // ---------------- activation TMA: one 128 x 32 fp32 box per quant block -----------------
        if (lane == 0) {
            uint32_t cnt = 0; bool ok = true;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
                const int mt = item / p.groups;
                for (int kb = 0; kb < p.nblk; ++kb, ++cnt) {
                    const int s = cnt % p.RS; const uint32_t ph = (cnt / p.RS) & 1u;
                    if (!Q8_WAIT_RELAXED(0, raw_empty(s), ph ^ 1u, cta_abort, p.err, 0x1101)) { ok = false; break; }
                    mbar_arrive_expect_tx(raw_full(s), kTile);
                    tma_load_3d(smem_base + L.raw_off + s * kTile, &tmX, raw_full(s), kb * 32, mt * 128, 0);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- weight TMA: 128 rows x 128 int8 per stage ------------------------------
        if (lane == 0) {
            uint32_t cnt = 0; bool ok = true;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
                const int g = item % p.groups;
                const int nb0 = g * p.blocks_per_group;
                const int nb1 = min(nb0 + p.blocks_per_group, p.n_blocks);
                for (int nb = nb0; nb < nb1 && ok; ++nb) {
                    for (int ks = 0; ks < p.KT; ++ks, ++cnt) {
                        const int s = cnt % p.BS; const uint32_t ph = (cnt / p.BS) & 1u;
                        if (!Q8_WAIT_RELAXED(1, w_empty(s), ph ^ 1u, cta_abort, p.err, 0x1201)) { ok = false; break; }
                        mbar_arrive_expect_tx(w_full(s), kTile);
                        tma_load_3d(smem_base + L.w_off + s * kTile, &tmW, w_full(s), ks * 128, nb * 128, 0);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ---------------- MMA issue: one instruction per quant block -----------------------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(2, 1, 1, 0, 0, 128, 128);
            uint32_t wcnt = 0, bcnt = 0, n_it = 0; bool ok = true;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++n_it) {
                const int g = item % p.groups;
                const int nb0 = g * p.blocks_per_group;
                const int nb1 = min(nb0 + p.blocks_per_group, p.n_blocks);
                for (int nb = nb0; nb < nb1 && ok; ++nb) {
                    for (int ks = 0; ks < p.KT && ok; ++ks, ++wcnt) {
                        if (nb == nb0) {
                            if (!Q8_WAIT(2, a_full(ks), n_it & 1u, cta_abort, p.err, 0x1301)) { ok = false; break; }
                        }
                        const int s = wcnt % p.BS; const uint32_t ph = (wcnt / p.BS) & 1u;
                        if (!Q8_WAIT(3, w_full(s), ph, cta_abort, p.err, 0x1302)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t da = make_smem_desc(smem_base + L.a_off + ks * kTile, 16, 1024, kLayoutSW128);
                        const uint64_t db = make_smem_desc(smem_base + L.w_off + s * kTile, 16, 1024, kLayoutSW128);
                        const int nblk_step = min(4, p.nblk - 4 * ks);
                        for (int j = 0; j < nblk_step; ++j, ++bcnt) {
                            const int slot = bcnt & 3; const uint32_t tph = (bcnt >> 2) & 1u;
                            // the epilogue re-arms a slot with the integer whose bit pattern is the float
                            // 1.5 * 2^23; accumulating the block sum onto it yields that float plus the sum
                            if (!Q8_WAIT(4, t_empty(slot), tph, cta_abort, p.err, 0x1303)) { ok = false; break; }
                            tc_fence_after();
                            umma<MmaKind::I8>(tmem_base + slot * 128, da + 2u * j, db + 2u * j, idesc, 1u);
                            umma_commit(t_full(slot));
                        }
                        if (!ok) break;
                        umma_commit(w_empty(s));
                        if (nb == nb1 - 1) umma_commit(a_empty(ks));
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp < kMiscWarps + kEpiWarps) {
        // ---------------- epilogue: per-block rescale, fp32 accumulation in registers -------------
        const int q = warp & 3;                       // TMEM lane quarter
        const int cg = (warp - kMiscWarps) >> 2;      // which 32 of the 128 columns
        const int etid = threadIdx.x - kMiscWarps * 32;   // 0..511
        const int row = q * 32 + lane;                // token row inside the tile
        uint32_t bcnt = 0, n_it = 0, dwcnt = 0; bool ok = true;
        const bool dw_resident = p.dw_tabs == p.n_blocks;    // (one column block in all: trivially resident)
        constexpr uint32_t kMagicBits = 0x4B400000u;   // 1.5 * 2^23 as a float; as an integer it is the slot bias
#pragma unroll
        for (int sl = 0; sl < 4; ++sl) {
            tmem_st32_fill(tmem_base + sl * 128 + cg * 32 + (static_cast<uint32_t>(q * 32) << 16), kMagicBits);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) { for (int sl = 0; sl < 4; ++sl) mbar_arrive(t_empty(sl)); }
        if (dw_resident) {
            for (int i = etid; i < p.n_blocks * p.nblk * 128; i += 32 * kEpiWarps) {
                const int nbq = i / (p.nblk * 128), r = i - nbq * p.nblk * 128;
                const int kb = r >> 7, col = r & 127;
                const int mo = nbq * 128 + col;
                dw_s[i] = (mo < p.Mout) ? __half2float(p.Wd[static_cast<size_t>(mo) * p.nblk + kb]) : 0.0f;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(dw_full);
            if (!Q8_WAIT_WARP(7, dw_full, 0u, cta_abort, p.err, 0x1404)) ok = false;
        }
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++n_it) {
            const int mt = item / p.groups, g = item % p.groups;
            const int nb0 = g * p.blocks_per_group;
            const int nb1 = min(nb0 + p.blocks_per_group, p.n_blocks);
            const int tok = mt * 128 + row;
            const __half* da_row = da_s + (n_it & 1) * p.nblk * 128 + row;
            for (int nb = nb0; nb < nb1 && ok; ++nb) {
                // weight scales as fp32 [nblk][128] per column block.  When the tables of all column blocks fit
                // they were staged once before the first item; otherwise this block's table is refilled here:
                // wait until every epilogue warp has finished with the previous one, fill, publish.
                const float* dw_tab = dw_s + (p.dw_tabs > 1 ? nb : 0) * p.nblk * 128;
                if (!dw_resident) {
                    if (!Q8_WAIT_WARP(6, dw_free, (dwcnt & 1u) ^ 1u, cta_abort, p.err, 0x1402)) { ok = false; break; }
                    for (int i = etid; i < p.nblk * 128; i += 32 * kEpiWarps) {
                        const int kb = i >> 7, col = i & 127;
                        const int mo = nb * 128 + col;
                        dw_s[i] = (mo < p.Mout) ? __half2float(p.Wd[static_cast<size_t>(mo) * p.nblk + kb]) : 0.0f;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(dw_full);
                    if (!Q8_WAIT_WARP(7, dw_full, dwcnt & 1u, cta_abort, p.err, 0x1403)) { ok = false; break; }
                }
                // 32 fp32 accumulators as 16 packed pairs
                uint64_t acc2[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) acc2[j] = 0ull;
                const uint64_t neg_magic2 = pack2(-12582912.0f, -12582912.0f);
                for (int kb = 0; kb < p.nblk; ++kb, ++bcnt) {
                    const int slot = bcnt & 3; const uint32_t tph = (bcnt >> 2) & 1u;
                    if (!Q8_WAIT_WARP(5, t_full(slot), tph, cta_abort, p.err, 0x1401)) { ok = false; break; }
                    tc_fence_after();
                    const float da = __half2float(da_row[kb * 128]);
                    const uint32_t taddr = tmem_base + slot * 128 + cg * 32 + (static_cast<uint32_t>(q * 32) << 16);
                    // two halves of 16 columns keep the live registers under the cap of this 23-warp CTA
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t v[16];
                        { Q8_T0();
                        tmem_ld16(taddr + h * 16, v);
                        tmem_ld_wait();
                        if (h == 1) {
                            tmem_st32_fill(taddr, kMagicBits);         // re-arm the slot for its next block
                            tmem_st_wait();
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(t_empty(slot));
                        }
                        Q8_T1(11); }
                        Q8_T0();
#ifndef PPML_Q8_SCALAR_MATH
                        const uint64_t da2 = pack2(da, da);
                        const ulonglong2* dwp = reinterpret_cast<const ulonglong2*>(dw_tab + kb * 128 + cg * 32 + h * 16);
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {
                            // int32 -> fp32 without the conversion unit: |sum| < 2^22 and the slot was biased by the
                            // bit pattern of 1.5 * 2^23, so the word read back IS the float 1.5 * 2^23 + sum
#ifdef PPML_Q8_EXP_NOLDS
                            const ulonglong2 w4 = make_ulonglong2(neg_magic2, da2);
#else
                            const ulonglong2 w4 = dwp[j4];
#endif
                            const uint64_t f01 = fadd2(pack2(__uint_as_float(v[j4 * 4 + 0]), __uint_as_float(v[j4 * 4 + 1])), neg_magic2);
                            const uint64_t f23 = fadd2(pack2(__uint_as_float(v[j4 * 4 + 2]), __uint_as_float(v[j4 * 4 + 3])), neg_magic2);
                            acc2[h * 8 + j4 * 2 + 0] = ffma2(f01, fmul2(w4.x, da2), acc2[h * 8 + j4 * 2 + 0]);
                            acc2[h * 8 + j4 * 2 + 1] = ffma2(f23, fmul2(w4.y, da2), acc2[h * 8 + j4 * 2 + 1]);
                        }
#else
                        const float4* dwp = reinterpret_cast<const float4*>(dw_tab + kb * 128 + cg * 32 + h * 16);
                        float* accf = reinterpret_cast<float*>(acc2);
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {
                            const float4 w4 = dwp[j4];
                            accf[h * 16 + j4 * 4 + 0] = fmaf(__uint_as_float(v[j4 * 4 + 0]) - 12582912.0f, w4.x * da, accf[h * 16 + j4 * 4 + 0]);
                            accf[h * 16 + j4 * 4 + 1] = fmaf(__uint_as_float(v[j4 * 4 + 1]) - 12582912.0f, w4.y * da, accf[h * 16 + j4 * 4 + 1]);
                            accf[h * 16 + j4 * 4 + 2] = fmaf(__uint_as_float(v[j4 * 4 + 2]) - 12582912.0f, w4.z * da, accf[h * 16 + j4 * 4 + 2]);
                            accf[h * 16 + j4 * 4 + 3] = fmaf(__uint_as_float(v[j4 * 4 + 3]) - 12582912.0f, w4.w * da, accf[h * 16 + j4 * 4 + 3]);
                        }
#endif
                        Q8_T1(12);
                        if (p.sumi_out != nullptr && tok < p.Ntok) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int mo = nb * 128 + cg * 32 + h * 16 + j;
                                if (mo < p.Mout)
                                    p.sumi_out[(static_cast<size_t>(tok) * p.Mout + mo) * p.nblk + kb] = static_cast<int>(v[j] - kMagicBits);
                            }
                        }
                    }
                }
                float acc[32];
#pragma unroll
                for (int j = 0; j < 16; ++j) unpack2(acc2[j], acc[2 * j], acc[2 * j + 1]);
                if (!ok) break;
                if (!dw_resident) { __syncwarp(); if (lane == 0) mbar_arrive(dw_free); ++dwcnt; }
                Q8_T0();
                if (p.c_trans && p.staged) {
                    // row-contiguous stores: thread = row writes its 32 values into the warp's padded buffer,
                    // then eight lanes cover one 128-byte row segment, four rows per store instruction
                    const int mo0 = nb * 128 + cg * 32;
                    uint8_t* stage = sg + L.st_off + (warp - kMiscWarps) * kStoreBytes;
                    if (p.bias != nullptr) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (mo0 + j < p.Mout) acc[j] += p.bias[mo0 + j];
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4*>(stage + lane * kStorePitch + j * 16) =
                            make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
                    __syncwarp();
                    const int cc = lane & 7;
                    const int col = mo0 + cc * 4;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = (lane >> 3) + 4 * i;
                        const int trow = mt * 128 + q * 32 + rr;
                        const float4 val = *reinterpret_cast<const float4*>(stage + rr * kStorePitch + cc * 16);
                        if (trow < p.Ntok && col < p.Mout)      // staged mode requires Mout % 4 == 0
                            *reinterpret_cast<float4*>(p.C + static_cast<size_t>(trow) * p.Mout + col) = val;
                    }
                    __syncwarp();
                } else if (tok < p.Ntok) {
                    const int mo0 = nb * 128 + cg * 32;
                    if (p.bias != nullptr) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (mo0 + j < p.Mout) acc[j] += p.bias[mo0 + j];
                    }
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
                Q8_T1(13);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_done(n_it & 1));
        }
    } else {
        // ---------------- quantizers: one thread per token row, two groups on alternate blocks ----------
        const int qg = (warp - kMiscWarps - kEpiWarps) >> 2;   // quantizer group
        const int row = ((warp - kMiscWarps - kEpiWarps) & 3) * 32 + lane;
        uint32_t base_cnt = 0, n_it = 0; bool ok = true;
        const uint64_t half2c = pack2(0.5f, 0.5f), big2 = pack2(8388608.0f, 8388608.0f);
        const uint64_t nbig2 = pack2(-8388608.0f, -8388608.0f), magic2 = pack2(12582912.0f, 12582912.0f);
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++n_it, base_cnt += p.nblk) {
            if (n_it >= 2) {
                if (!Q8_WAIT_WARP(8, epi_done(n_it & 1), ((n_it >> 1) - 1) & 1u, cta_abort, p.err, 0x1501)) { ok = false; break; }
            }
            __half* da_w = da_s + (n_it & 1) * p.nblk * 128 + row;
            for (int kb = qg; kb < p.nblk; kb += kQuantGroups) {
                const uint32_t cnt = base_cnt + kb;
                const int ks = kb >> 2;
                if ((kb & 3) < kQuantGroups) {       // this group's first block of the K step
                    if (!Q8_WAIT_WARP(9, a_empty(ks), (n_it & 1u) ^ 1u, cta_abort, p.err, 0x1502)) { ok = false; break; }
                }
                const int s = cnt % p.RS; const uint32_t ph = (cnt / p.RS) & 1u;
                if (!Q8_WAIT_WARP(10, raw_full(s), ph, cta_abort, p.err, 0x1503)) { ok = false; break; }
                const uint8_t* raw = sg + L.raw_off + s * kTile;
                float x[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float4 t = *reinterpret_cast<const float4*>(raw + sw128_off(row, c));
                    x[4 * c] = t.x; x[4 * c + 1] = t.y; x[4 * c + 2] = t.z; x[4 * c + 3] = t.w;
                }
                // signed value of the first element that attains the maximum magnitude
                float vpos = x[0], vneg = x[0];
#pragma unroll
                for (int i = 1; i < 32; ++i) { vpos = fmaxf(vpos, x[i]); vneg = fminf(vneg, x[i]); }
                const float amax = fmaxf(vpos, -vneg);
                float vmax;
                if (vpos == -vneg && amax != 0.0f) {        // +a and -a both present: the first one wins
                    vmax = 0.0f;
#pragma unroll
                    for (int i = 31; i >= 0; --i) if (fabsf(x[i]) == amax) vmax = x[i];
                } else {
                    vmax = (vpos == amax) ? vpos : vneg;
                }
                const float d = (amax == 0.0f) ? 0.0f : vmax / -128.0f;
                const float inv = (d == 0.0f) ? 0.0f : 1.0f / d;
                const uint64_t inv2 = pack2(inv, inv);
                // q = min(round-half-away(x * inv), 127), computed without the conversion unit:
                //   m = floor(|y| + 0.5): both additions round toward zero, which never crosses an integer,
                //       and adding 2^23 leaves the integer part; m carries y's sign again, is capped at 127,
                //   and m + 1.5 * 2^23 has the two's-complement byte of q in its low mantissa byte.
                uint32_t packed[8];
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    uint32_t u[4];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const uint64_t y2 = fmul2(pack2(x[4 * w + 2 * e], x[4 * w + 2 * e + 1]), inv2);
                        const uint64_t a2 = y2 & 0x7FFFFFFF7FFFFFFFull;
                        const uint64_t m2 = fadd2(fadd2_rz(fadd2_rz(a2, half2c), big2), nbig2);
                        float z0, z1;
                        unpack2(m2 | (y2 & 0x8000000080000000ull), z0, z1);
                        const uint64_t u2 = fadd2(pack2(fminf(z0, 127.0f), fminf(z1, 127.0f)), magic2);
                        u[2 * e] = static_cast<uint32_t>(u2);
                        u[2 * e + 1] = static_cast<uint32_t>(u2 >> 32);
                    }
                    packed[w] = __byte_perm(__byte_perm(u[0], u[1], 0x0040), __byte_perm(u[2], u[3], 0x0040), 0x5410);
                }
                uint8_t* at = sg + L.a_off + ks * kTile;
                const int c0 = (kb & 3) * 2;
                *reinterpret_cast<uint4*>(at + sw128_off(row, c0)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                *reinterpret_cast<uint4*>(at + sw128_off(row, c0 + 1)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                da_w[kb * 128] = __float2half_rn(d);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) { mbar_arrive(raw_empty(s)); mbar_arrive(a_full(ks)); }
            }
        }
    }

#ifdef PPML_Q8_TRACE
    if (blockIdx.x == 0 && threadIdx.x == 0) g_q8_trace[31] = clock64();
#endif
    tc_fence_before();
    __syncthreads();
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace

#ifdef PPML_Q8_TRACE
extern "C" int ppml_b200_q8_trace_read(long long* out64, int reset) {
    cudaDeviceSynchronize();
    if (cudaMemcpyFromSymbol(out64, g_q8_trace, sizeof(long long) * 64) != cudaSuccess) return 1;
    if (reset) { long long z[64] = {0}; cudaMemcpyToSymbol(g_q8_trace, z, sizeof(z)); }
    return 0;
}
#endif

// W: Q8_0R weights ([Mout*nblk*32] int8 plane followed by [Mout*nblk] half scales); X fp32 [Ntok][K];
// M = weight rows (out features), N = tokens, as in the reference's launcher.
int launch_umma_q8(const void* W, const float* X, float* C, int M, int N, int K, int c_trans, const float* bias,
                   int* sumi_out, cudaStream_t st) {
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
    // Shared memory: the resident A tile and the activation-scale table are fixed; then, in this order of
    // preference, the scale tables of all column blocks (no refill, at most 32 KB), the per-warp store
    // buffers, and at least four ring stages; what is left goes to the rings.
    const int budget = 226 * 1024;
    p.dw_tabs = (p.n_blocks * p.nblk * 512 <= 32 * 1024) ? p.n_blocks : 1;
    p.staged = p.vec_ok ? 1 : 0;
    auto stages_for = [&](int tabs, int staged) {
        return (budget - (static_cast<int>(q8_layout(p.KT, p.nblk, 0, 0, tabs, staged).total) + 1024)) / kTile;
    };
    if (stages_for(p.dw_tabs, p.staged) < 4 && p.dw_tabs > 1) p.dw_tabs = 1;
    if (stages_for(p.dw_tabs, p.staged) < 4) p.staged = 0;
    int stages = stages_for(p.dw_tabs, p.staged);
    if (stages < 3) return ST_UNSUPPORTED_PATH;
    if (stages > 2 * kMaxStages) stages = 2 * kMaxStages;
    p.RS = stages / 2; p.BS = stages - p.RS;
    if (p.RS > kMaxStages) p.RS = kMaxStages;
    if (p.BS > kMaxStages) p.BS = kMaxStages;
    const __half* Wd = reinterpret_cast<const __half*>(static_cast<const int8_t*>(W) + static_cast<size_t>(M) * p.nblk * 32);
    p.Wd = Wd; p.C = C; p.bias = bias; p.sumi_out = sumi_out; p.c_trans = c_trans; p.err = err;

    CUtensorMap tmX, tmW;
    if (!make_tmap_3d(&tmX, TmaType::F32, X, K, N, 1, static_cast<uint64_t>(K) * 4, 0, 32, 128, true)) return ST_UNSUPPORTED_PATH;
    if (!make_tmap_3d(&tmW, TmaType::U8, W, K, M, 1, static_cast<uint64_t>(K), 0, 128, 128, true)) return ST_UNSUPPORTED_PATH;

    const int smem = static_cast<int>(q8_layout(p.KT, p.nblk, p.RS, p.BS, p.dw_tabs, p.staged).total) + 1024;
    static int configured_smem[64] = {0};
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && configured_smem[dev] < smem) {
        if (cudaFuncSetAttribute(umma_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
            cudaGetLastError();
            return ST_LAUNCH;
        }
        configured_smem[dev] = 227 * 1024;
    }
    const int total_items = p.m_tiles * p.groups;
    const int grid = total_items < sms ? total_items : sms;
    umma_q8_kernel<<<grid, kThreads, smem, st>>>(tmX, tmW, p);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

}  // namespace ppml_b200
