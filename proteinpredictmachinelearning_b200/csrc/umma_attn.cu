// umma_attn.cu -- fused attention forward on tcgen05 for head dim 32 (the model's 8 x 32 heads).
//
//   O = softmax(scale * Q K^T + bias) V,  denominator (l + eps),  LSE = m + log(l + eps)
//
// One CTA = one (batch, head, 128-query tile); keys are walked in tiles of 128.
//   warp 0      TMA: Q tile once, K tiles (128 keys x 32 floats, 128-byte swizzle, tf32 delivered by TMA)
//   warp 1      MMA issue: S = Q K^T (four K = 8 tf32 MMAs, N = 128) into one of two TMEM S buffers,
//               then O_part = P V (sixteen K = 8 MMAs, N = 32) into one of two TMEM O buffers
//   warps 2-5   softmax, one thread per query row: S from TMEM, scale + bias + mask, running max / sum,
//               P (rounded to tf32) into shared memory as the next MMA's K-major A operand, then
//               o = alpha * o + O_part in fp32 registers
//   warps 6-9   stage V^T: V[key][d] is read row-contiguously and written as the K-major B operand
//               (32 rows of d, keys along K)
// Every wait is bounded; rows past L and keys past Lk are zero-filled by TMA and masked.
#include <math_constants.h>

#include "kernels.h"
#include "tma_host.h"

namespace ppml_b200 {

namespace {

constexpr int kD = 32;                       // head dim handled here
constexpr int kBM = 128, kBN = 128;          // query tile, key tile
constexpr int kTileQK = 128 * 128;           // bytes: 128 rows x 32 floats
constexpr int kTileP = 4 * kTileQK;          // P: 128 rows x 128 floats as four 32-float swizzle atoms
constexpr int kThreads = 320;

struct AttnParams {
    int B, H, L, Lk;
    int causal;
    float scale, eps;
    const float* V;
    const float* bias;
    long long bias_batch_stride;
    float* O;
    float* LSE;
    int q_tiles, k_tiles;
    int* err;
};

// smem map (offsets from the 1024-aligned base)
constexpr int kOffQ = 0;
constexpr int kOffK = kOffQ + kTileQK;              // 2 stages
constexpr int kOffV = kOffK + 2 * kTileQK;          // 2 stages of V^T (32 x 128 floats = 16 KB)
constexpr int kOffP = kOffV + 2 * kTileQK;          // 1 buffer
constexpr int kOffStage = kOffP + kTileP;           // 4 warps x (32 rows x 144 B) output transposition
constexpr int kOffBar = kOffStage + 4 * 32 * 144;
constexpr int kSmemBytes = kOffBar + 256 + 1024;

__global__ void __launch_bounds__(kThreads, 1)
umma_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sb = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* sg = smem_raw + (sb - smem_u32(smem_raw));
    const uint32_t bar0 = sb + kOffBar;
    const uint32_t q_full = bar0;
    auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (3 + s); };
    auto v_full = [&](int s) { return bar0 + 8u * (5 + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (7 + s); };
    auto s_full = [&](int s) { return bar0 + 8u * (9 + s); };
    auto s_empty = [&](int s) { return bar0 + 8u * (11 + s); };
    auto o_full = [&](int s) { return bar0 + 8u * (13 + s); };
    auto o_empty = [&](int s) { return bar0 + 8u * (15 + s); };
    const uint32_t p_full = bar0 + 8u * 17, p_empty = bar0 + 8u * 18;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sg + kOffBar + 8 * 19);
    volatile int* cta_abort = reinterpret_cast<volatile int*>(sg + kOffBar + 8 * 19 + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = blockIdx.x % p.q_tiles;
    const int bh = blockIdx.x / p.q_tiles;
    const int b = bh / p.H, hh = bh - b * p.H;
    const int q0 = qt * kBM;
    // causal: keys beyond the last query row of the tile are never needed
    int k_tiles = p.k_tiles;
    if (p.causal) { const int last = min(q0 + kBM, p.L); k_tiles = min(k_tiles, (min(last, p.Lk) + kBN - 1) / kBN); }

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1);
            mbar_init(v_full(s), 4); mbar_init(v_empty(s), 1);
            mbar_init(s_full(s), 1); mbar_init(s_empty(s), 4);
            mbar_init(o_full(s), 1); mbar_init(o_empty(s), 4);
        }
        mbar_init(p_full, 4); mbar_init(p_empty, 1);
        *cta_abort = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512); tmem_relinquish(); }
    if (warp == 0 && lane == 0) { prefetch_tmap(&tmQ); prefetch_tmap(&tmK); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // TMEM columns: S buffers at 0 and 128, O_part buffers at 256 and 288

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, kTileQK);
            tma_load_3d(sb + kOffQ, &tmQ, q_full, 0, q0, bh);
            for (int j = 0; j < k_tiles; ++j) {
                const int s = j & 1; const uint32_t ph = (j >> 1) & 1u;
                if (!mbar_wait(k_empty(s), ph ^ 1u, cta_abort, p.err, 0x2101)) break;
                mbar_arrive_expect_tx(k_full(s), kTileQK);
                tma_load_3d(sb + kOffK + s * kTileQK, &tmK, k_full(s), 0, j * kBN, bh);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc(1, 2, 2, 0, 0, 128, kBN);
            const uint32_t idesc_o = make_idesc(1, 2, 2, 0, 0, 128, kD);
            bool ok = mbar_wait(q_full, 0, cta_abort, p.err, 0x2201);
            // software pipeline: S(j+1) is issued before P(j) V(j), so the softmax of tile j+1 can start
            // while the tensor core finishes tile j
            auto issue_s = [&](int j) -> bool {
                const int s = j & 1; const uint32_t ph = (j >> 1) & 1u;
                if (!mbar_wait(k_full(s), ph, cta_abort, p.err, 0x2202)) return false;
                if (!mbar_wait(s_empty(s), ph ^ 1u, cta_abort, p.err, 0x2203)) return false;
                tc_fence_after();
                const uint64_t dq = make_smem_desc(sb + kOffQ, 16, 1024, kLayoutSW128);
                const uint64_t dk = make_smem_desc(sb + kOffK + s * kTileQK, 16, 1024, kLayoutSW128);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) umma<MmaKind::TF32>(tmem_base + s * 128, dq + 2u * kk, dk + 2u * kk, idesc_s, kk ? 1u : 0u);
                umma_commit(k_empty(s));
                umma_commit(s_full(s));
                return true;
            };
            if (ok && k_tiles > 0) ok = issue_s(0);
            for (int j = 0; j < k_tiles && ok; ++j) {
                if (j + 1 < k_tiles) { if (!issue_s(j + 1)) { ok = false; break; } }
                const int s = j & 1; const uint32_t ph = (j >> 1) & 1u;
                if (!mbar_wait(p_full, j & 1u, cta_abort, p.err, 0x2204)) { ok = false; break; }
                if (!mbar_wait(v_full(s), ph, cta_abort, p.err, 0x2205)) { ok = false; break; }
                if (!mbar_wait(o_empty(s), ph ^ 1u, cta_abort, p.err, 0x2206)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int a = 0; a < 4; ++a) {            // four 32-key swizzle atoms of P and of V^T
                    const uint64_t dp = make_smem_desc(sb + kOffP + a * kTileQK, 16, 1024, kLayoutSW128);
                    const uint64_t dv = make_smem_desc(sb + kOffV + s * kTileQK + a * 4096, 16, 1024, kLayoutSW128);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma<MmaKind::TF32>(tmem_base + 256 + s * kD, dp + 2u * kk, dv + 2u * kk, idesc_o, (a | kk) ? 1u : 0u);
                }
                umma_commit(p_empty);
                umma_commit(v_empty(s));
                umma_commit(o_full(s));
            }
        }
        __syncwarp();
    } else if (warp < 6) {
#include "umma_attn_softmax.inc"
    } else {
        // ---------------- V^T staging: lane = d, each warp takes every fourth key ------------------------
        const int vw = warp - 6;
        const float* Vb = p.V + static_cast<size_t>(bh) * p.Lk * kD;
        bool ok = true;
        for (int j = 0; j < k_tiles && ok; ++j) {
            const int s = j & 1; const uint32_t ph = (j >> 1) & 1u;
            if (!mbar_wait(v_empty(s), ph ^ 1u, cta_abort, p.err, 0x2401)) { ok = false; break; }
            uint8_t* vt = sg + kOffV + s * kTileQK;
#pragma unroll 4
            for (int kk = vw; kk < kBN; kk += 4) {
                const int key = j * kBN + kk;
                const float v = (key < p.Lk) ? tf32_round(Vb[static_cast<size_t>(key) * kD + lane]) : 0.0f;
                // row = d (lane), column = key inside the tile: atom kk / 32, 16-byte chunk (kk % 32) / 4
                *reinterpret_cast<float*>(vt + (kk >> 5) * 4096 + sw128_off(lane, (kk & 31) >> 2) + (kk & 3) * 4) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(v_full(s));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
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
    p.V = V; p.bias = bias; p.bias_batch_stride = bias_batch_stride; p.O = O; p.LSE = LSE;
    p.q_tiles = (L + kBM - 1) / kBM; p.k_tiles = (Lk + kBN - 1) / kBN; p.err = err;
    const long long grid = BH * p.q_tiles;
    if (grid <= 0 || grid > 0x7fffffffLL) return ST_BAD_ARGS;
    CUtensorMap tmQ, tmK;
    if (!make_tmap_3d(&tmQ, TmaType::TF32, Q, kD, L, BH, kD * 4, static_cast<uint64_t>(L) * kD * 4, kD, kBM, true)) return ST_UNSUPPORTED_PATH;
    if (!make_tmap_3d(&tmK, TmaType::TF32, K, kD, Lk, BH, kD * 4, static_cast<uint64_t>(Lk) * kD * 4, kD, kBN, true)) return ST_UNSUPPORTED_PATH;
    static bool configured[64] = {false};
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(umma_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
            cudaGetLastError();
            return ST_LAUNCH;
        }
        configured[dev] = true;
    }
    umma_attn_kernel<<<static_cast<unsigned>(grid), kThreads, kSmemBytes, st>>>(tmQ, tmK, p);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

}  // namespace ppml_b200
