// umma_attn.cu -- fused attention forward on tcgen05 for head dim 32 (the model's 8 x 32 heads).
//
//   O = softmax(scale * Q K^T + bias) V,  denominator (l + eps),  LSE = m + log(l + eps)
//
// Work item = one (batch, head, 128-query tile); keys are walked in tiles of 64.  CTAs are persistent, two per SM (256 TMEM
// columns, about 105 KB of shared memory, 192 threads each), so one CTA's softmax overlaps the other's loads and
// tensor work.  (Key tiles of 32 with three CTAs per SM, -DPPML_ATTN_BN=32, measured 5-15 % slower.)
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
#ifndef PPML_ATTN_BN
#define PPML_ATTN_BN 64
#endif
constexpr int kBM = 128, kBN = PPML_ATTN_BN;  // query tile, key tile (32: three CTAs per SM, 64: two)
constexpr int kTileQ = 128 * 128;            // bytes: 128 rows x 32 floats
constexpr int kTileKV = kBN * 128;           // bytes: kBN keys x 32 floats
constexpr int kTileP = (kBN / 32) * kTileQ;  // P: 128 rows x 64 floats as two 32-float swizzle atoms
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = (kBN == 32) ? 128 : 256;   // S buffers at columns 0 and kBN, O_part buffers at 2 kBN and 2 kBN + 32
constexpr int kCtasPerSm = (kBN == 32) ? 3 : 2;

// 2^x on the transcendental unit (about 2 ulp); results below the normal range flush to 0, 2^-inf = 0
__device__ __forceinline__ float ex2_approx(float x) {
    float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r; asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c)); return r;
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
    int o_align32;               // O is 32-byte aligned: rows can be written with 256-bit stores
    int* err;
};

// smem map (offsets from the 1024-aligned base); two CTAs per SM leave about 113 KB each
constexpr int kOffQ = 0;
constexpr int kOffK = kOffQ + kTileQ;               // 2 stages
constexpr int kOffV = kOffK + 2 * kTileKV;          // 2 stages
constexpr int kOffP = kOffV + 2 * kTileKV;          // 2 buffers of bias-then-P: TMA puts the bias tile of key tile j into
                                                    //   buffer j % 2 in the layout of P, every softmax thread reads its bias
                                                    //   values and later writes its P values over them
constexpr int kOffBar = kOffP + 2 * kTileP;
constexpr int kSmemBytes = kOffBar + 256;             // the dynamic shared memory is declared 1024-byte aligned: no slack

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
umma_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmB, const AttnParams p) {
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
                tma_load_3d(sb + kOffQ, &tmQ, q_full, 0, q0, bh);
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
                            tma_load_3d(sb + kOffP + s * kTileP + a * kTileQ, &tmB, b_full(s), j * kBN + 32 * a, brow0, bbatch);
                    }
                    if (!mbar_wait(k_empty(s), ph ^ 1u, cta_abort, p.err, 0x2101)) { ok = false; break; }
                    mbar_arrive_expect_tx(k_full(s), kTileKV);
                    tma_load_3d(sb + kOffK + s * kTileKV, &tmK, k_full(s), 0, j * kBN, bh);
                    if (!mbar_wait(v_empty(s), ph ^ 1u, cta_abort, p.err, 0x2102)) { ok = false; break; }
                    mbar_arrive_expect_tx(v_full(s), kTileKV);
                    tma_load_3d(sb + kOffV + s * kTileKV, &tmV, v_full(s), 0, j * kBN, bh);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc(1, 2, 2, 0, 0, 128, kBN);
            const uint32_t idesc_o = make_idesc(1, 2, 2, 0, 1, 128, kD);     // B = V with d (the row index) contiguous
            uint32_t ts = 0, tp = 0, ic = 0;             // score products / P V products / items issued so far
            bool ok = true;
            // software pipeline: S(j+1) is issued before P(j) V(j), so the softmax of tile j+1 can start
            // while the tensor core finishes tile j
            auto issue_s = [&]() -> bool {
                const int s = ts & 1; const uint32_t ph = (ts >> 1) & 1u;
                if (!mbar_wait(k_full(s), ph, cta_abort, p.err, 0x2202)) return false;
                if (!mbar_wait(s_empty(s), ph ^ 1u, cta_abort, p.err, 0x2203)) return false;
                tc_fence_after();
                const uint64_t dq = make_smem_desc(sb + kOffQ, 16, 1024, kLayoutSW128);
                const uint64_t dk = make_smem_desc(sb + kOffK + s * kTileKV, 16, 1024, kLayoutSW128);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) umma<MmaKind::TF32>(tmem_base + s * kBN, dq + 2u * kk, dk + 2u * kk, idesc_s, kk ? 1u : 0u);
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
                    // V tile: 64 key rows of 128 bytes in the 32-byte-chunk swizzle; a group of 4 keys is 512 bytes
                    // (stride offset), one instruction consumes 8 keys = 1024 bytes.  P: two 32-key swizzle atoms.
                    const uint64_t dv = make_smem_desc(sb + kOffV + s * kTileKV, 4096, 512, kLayoutSW128Base32);
#pragma unroll
                    for (int a = 0; a < kBN / 32; ++a) {
                        const uint64_t dp = make_smem_desc(sb + kOffP + s * kTileP + a * kTileQ, 16, 1024, kLayoutSW128);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma<MmaKind::TF32>(tmem_base + 2 * kBN + s * kD, dp + 2u * kk, dv + 64u * (a * 4 + kk), idesc_o, (a | kk) ? 1u : 0u);
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

int launch_umma_attn(const float* Q, const float* K, const float* V, const float* bias, float* O, float* LSE,
                     int B, int H, int L, int Lk, int d, int causal, float scale, float eps,
                     long long bias_batch_stride, cudaStream_t st) {
    if (d != kD) return ST_UNSUPPORTED_PATH;
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
    p.o_align32 = (reinterpret_cast<uintptr_t>(O) & 31u) == 0 ? 1 : 0;
    const long long resident = static_cast<long long>(kCtasPerSm) * num_sms();     // persistent CTAs
    const long long grid = items < resident ? items : resident;
    CUtensorMap tmQ, tmK, tmV, tmB;
    if (!make_tmap_3d(&tmQ, TmaType::TF32, Q, kD, L, BH, kD * 4, static_cast<uint64_t>(L) * kD * 4, kD, kBM, 1)) return ST_UNSUPPORTED_PATH;
    if (!make_tmap_3d(&tmK, TmaType::TF32, K, kD, Lk, BH, kD * 4, static_cast<uint64_t>(Lk) * kD * 4, kD, kBN, 1)) return ST_UNSUPPORTED_PATH;
    if (!make_tmap_3d(&tmV, TmaType::TF32, V, kD, Lk, BH, kD * 4, static_cast<uint64_t>(Lk) * kD * 4, kD, kBN, 2)) return ST_UNSUPPORTED_PATH;
    // bias rows are (head, query) pairs, [B or 1][H * L][Lk]; fp32 as it is (no tf32 rounding)
    tmB = tmQ;
    if (bias) {
        const bool per_batch = bias_batch_stride != 0;
        if (!make_tmap_3d(&tmB, TmaType::F32, bias, Lk, static_cast<uint64_t>(H) * L, per_batch ? B : 1, static_cast<uint64_t>(Lk) * 4,
                          per_batch ? static_cast<uint64_t>(bias_batch_stride) * 4 : 0, 32, kBM, 1)) return ST_UNSUPPORTED_PATH;
    }
    static bool configured[64] = {false};
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(umma_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
            cudaGetLastError();
            return ST_LAUNCH;
        }
        configured[dev] = true;
    }
    umma_attn_kernel<<<static_cast<unsigned>(grid), kThreads, kSmemBytes, st>>>(tmQ, tmK, tmV, tmB, p);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

}  // namespace ppml_b200
