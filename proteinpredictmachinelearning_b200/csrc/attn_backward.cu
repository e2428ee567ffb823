// Flash-attention backward (the reference's flash_attn_backward_cuda, src/cuda/FlashAttnKernel.cu:1524, same math as
// flash_attn_backward_cpu, src/ops/FlashAttn.cpp:144-216), exact fp32 on CUDA cores, without atomics:
//
//   P_ij = exp(S_ij - LSE_i),  D_i = sum_d dO_id O_id,  dP_ij = sum_d dO_id V_jd,  dS_ij = P_ij (dP_ij - D_i)
//   dQ_id = scale sum_j dS_ij K_jd     dK_jd = scale sum_i dS_ij Q_id     dV_jd = sum_i P_ij dO_id     dbias_ij = dS_ij
//
// Two kernels, each recomputing the scores of its tiles (nothing but the outputs is written, every output element is
// written exactly once, so no zero-fill pass and no atomic adds: the results do not depend on the launch order):
//   attn_bwd_dq_kernel   one CTA = 32 query rows of one (batch, head); walks the key tiles of 32; writes dQ and dbias
//   attn_bwd_dkv_kernel  one CTA = 32 key rows of one (batch, head); walks the query tiles of 32; writes dK and dV
// In both, a warp owns 8 rows of the CTA's 32.  Per tile of 32 partner rows it works in two phases:
//   1. lane = partner row: dot products over d against the warp's rows (own rows broadcast from shared memory, partner
//      rows read from padded tiles), exp, dS; dS (and P) go to a small shared buffer, dbias to global memory (coalesced);
//   2. lane = channel d: accumulates its channel of the 8 rows over the 32 partners (dS broadcast, partner tile read
//      along d), one register per row and channel -- no cross-lane reduction.
// Layouts as the forward: Q, K, V, O, dO, dQ, dK, dV [B, h, L, d]; bias [B, h, L, L] with a batch stride (0: shared);
// dbias [B, h, L, L]; LSE [B, h, L].  d <= 64.
#include <cuda_runtime.h>
#include <math_constants.h>

#include "common.cuh"
#include "kernels.h"

namespace ppml_b200 {

namespace {

constexpr int kRows = 32;        // rows of a CTA (query rows / key rows) = partner rows of a tile
constexpr int kWarps = 4;
constexpr int kRpw = kRows / kWarps;   // rows per warp

struct BwdParams {
    int B, H, L, d, causal;
    float scale;
    const float *Q, *K, *V, *bias, *O, *dO, *LSE;
    long long bias_batch_stride;
    float *dQ, *dK, *dV, *dbias;
};

// rows [r0, r0 + 32) of a [L][d] matrix into a padded shared tile [32][DP + 1] (rows past L and channels past d: 0)
template <int DP>
__device__ __forceinline__ void load_tile(float* dst, const float* src, int r0, int L, int d) {
    for (int idx = threadIdx.x; idx < kRows * DP; idx += kWarps * 32) {
        const int r = idx / DP, c = idx - r * DP;
        dst[r * (DP + 1) + c] = (r0 + r < L && c < d) ? src[static_cast<size_t>(r0 + r) * d + c] : 0.0f;
    }
}

// ---- dQ and dbias -------------------------------------------------------------------------------------------------------
template <int DP>
__global__ void __launch_bounds__(kWarps * 32) attn_bwd_dq_kernel(const BwdParams p) {
    extern __shared__ float sm[];
    float* Ks = sm;                                   // [32][DP + 1]
    float* Vs = Ks + kRows * (DP + 1);                // [32][DP + 1]
    float* Qs = Vs + kRows * (DP + 1);                // [32][DP]   this CTA's query rows
    float* dOs = Qs + kRows * DP;                     // [32][DP]
    float* dS = dOs + kRows * DP;                     // [kWarps][32 partners][kRpw]
    float* Dr = dS + kWarps * 32 * kRpw;              // [32]  D_i
    float* Ls = Dr + kRows;                           // [32]  LSE_i

    const int bh = blockIdx.y, i0 = blockIdx.x * kRows;
    const int b = bh / p.H, hh = bh - b * p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t base = static_cast<size_t>(bh) * p.L * p.d;
    const float* bias = p.bias ? p.bias + static_cast<size_t>(b) * p.bias_batch_stride + static_cast<size_t>(hh) * p.L * p.L : nullptr;
    float* dbias = p.dbias ? p.dbias + static_cast<size_t>(bh) * p.L * p.L : nullptr;

    // this CTA's rows: Q, dO (unpadded rows: they are read as broadcasts), D_i, LSE_i
    for (int idx = threadIdx.x; idx < kRows * DP; idx += kWarps * 32) {
        const int r = idx / DP, c = idx - r * DP;
        const bool in = i0 + r < p.L && c < p.d;
        Qs[idx] = in ? p.Q[base + static_cast<size_t>(i0 + r) * p.d + c] : 0.0f;
        dOs[idx] = in ? p.dO[base + static_cast<size_t>(i0 + r) * p.d + c] : 0.0f;
    }
    if (threadIdx.x < kRows) {
        const int i = i0 + threadIdx.x;
        float D = 0.0f, lse = -CUDART_INF_F;
        if (i < p.L) {
            lse = p.LSE[static_cast<size_t>(bh) * p.L + i];
            for (int c = 0; c < p.d; ++c) D += p.dO[base + static_cast<size_t>(i) * p.d + c] * p.O[base + static_cast<size_t>(i) * p.d + c];
        }
        Dr[threadIdx.x] = D; Ls[threadIdx.x] = lse;
    }
    __syncthreads();

    constexpr int NACC = (DP + 31) / 32;              // channels per lane in phase 2
    float acc[kRpw][NACC];
#pragma unroll
    for (int r = 0; r < kRpw; ++r)
#pragma unroll
        for (int a = 0; a < NACC; ++a) acc[r][a] = 0.0f;

    const int jend = p.causal ? min(p.L, i0 + kRows) : p.L;      // keys past the last row's diagonal are masked for all
    float* dSw = dS + warp * 32 * kRpw;
    for (int j0 = 0; j0 < jend; j0 += kRows) {
        __syncthreads();                               // the tiles of the previous step are no longer read
        load_tile<DP>(Ks, p.K + base, j0, p.L, p.d);
        load_tile<DP>(Vs, p.V + base, j0, p.L, p.d);
        __syncthreads();
        // phase 1: lane = key j0 + lane, against the warp's 8 query rows
        const int j = j0 + lane;
        const float* kr = Ks + lane * (DP + 1);
        const float* vr = Vs + lane * (DP + 1);
#pragma unroll
        for (int r = 0; r < kRpw; ++r) {
            const int rl = warp * kRpw + r, i = i0 + rl;
            const float* q = Qs + rl * DP;
            const float* go = dOs + rl * DP;
            float s = 0.0f, dp = 0.0f;
#pragma unroll 8
            for (int c = 0; c < DP; ++c) { s = fmaf(q[c], kr[c], s); dp = fmaf(go[c], vr[c], dp); }
            const float lse = Ls[rl];
            float ds = 0.0f;
            const bool live = i < p.L && j < p.L && (!p.causal || j <= i) && lse > -CUDART_INF_F;
            if (live) {
                s *= p.scale;
                if (bias) s += bias[static_cast<size_t>(i) * p.L + j];
                ds = expf(s - lse) * (dp - Dr[rl]);
            }
            dSw[lane * kRpw + r] = ds;
            if (dbias && i < p.L && j < p.L) dbias[static_cast<size_t>(i) * p.L + j] = ds;
        }
        __syncwarp();
        // phase 2: lane = channel; dQ[i][c] += dS[i][j] K[j][c] over the 32 keys of the tile
#pragma unroll 4
        for (int jj = 0; jj < kRows; ++jj) {
            float dsr[kRpw];
#pragma unroll
            for (int r = 0; r < kRpw; ++r) dsr[r] = dSw[jj * kRpw + r];
#pragma unroll
            for (int a = 0; a < NACC; ++a) {
                const int c = lane + 32 * a;
                const float kv = (c < DP) ? Ks[jj * (DP + 1) + c] : 0.0f;
#pragma unroll
                for (int r = 0; r < kRpw; ++r) acc[r][a] = fmaf(dsr[r], kv, acc[r][a]);
            }
        }
        __syncwarp();
    }
    // keys past jend of a causal CTA: dbias stays 0 there
    if (dbias && p.causal) {
        for (int r = 0; r < kRpw; ++r) {
            const int i = i0 + warp * kRpw + r;
            if (i < p.L) for (int j = jend + lane; j < p.L; j += 32) dbias[static_cast<size_t>(i) * p.L + j] = 0.0f;
        }
    }
    if (p.dQ) {
#pragma unroll
        for (int r = 0; r < kRpw; ++r) {
            const int i = i0 + warp * kRpw + r;
#pragma unroll
            for (int a = 0; a < NACC; ++a) {
                const int c = lane + 32 * a;
                if (i < p.L && c < p.d) p.dQ[base + static_cast<size_t>(i) * p.d + c] = p.scale * acc[r][a];
            }
        }
    }
}

// ---- dK and dV ----------------------------------------------------------------------------------------------------------
template <int DP>
__global__ void __launch_bounds__(kWarps * 32) attn_bwd_dkv_kernel(const BwdParams p) {
    extern __shared__ float sm[];
    float* Qs = sm;                                   // [32][DP + 1]  query tile (partner rows)
    float* dOs = Qs + kRows * (DP + 1);               // [32][DP + 1]
    float* Ks = dOs + kRows * (DP + 1);               // [32][DP]   this CTA's key rows
    float* Vs = Ks + kRows * DP;                      // [32][DP]
    float* dS = Vs + kRows * DP;                      // [kWarps][32 partners][kRpw]
    float* Ps = dS + kWarps * 32 * kRpw;              // [kWarps][32 partners][kRpw]
    float* Dr = Ps + kWarps * 32 * kRpw;              // [32]  D_i of the query tile
    float* Ls = Dr + kRows;                           // [32]  LSE_i of the query tile

    const int bh = blockIdx.y, j0 = blockIdx.x * kRows;
    const int b = bh / p.H, hh = bh - b * p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t base = static_cast<size_t>(bh) * p.L * p.d;
    const float* bias = p.bias ? p.bias + static_cast<size_t>(b) * p.bias_batch_stride + static_cast<size_t>(hh) * p.L * p.L : nullptr;

    for (int idx = threadIdx.x; idx < kRows * DP; idx += kWarps * 32) {
        const int r = idx / DP, c = idx - r * DP;
        const bool in = j0 + r < p.L && c < p.d;
        Ks[idx] = in ? p.K[base + static_cast<size_t>(j0 + r) * p.d + c] : 0.0f;
        Vs[idx] = in ? p.V[base + static_cast<size_t>(j0 + r) * p.d + c] : 0.0f;
    }

    constexpr int NACC = (DP + 31) / 32;
    float ak[kRpw][NACC], av[kRpw][NACC];
#pragma unroll
    for (int r = 0; r < kRpw; ++r)
#pragma unroll
        for (int a = 0; a < NACC; ++a) { ak[r][a] = 0.0f; av[r][a] = 0.0f; }

    const int ibeg = p.causal ? (j0 / kRows) * kRows : 0;        // query rows before the first key of the tile see none of it
    float* dSw = dS + warp * 32 * kRpw;
    float* Pw = Ps + warp * 32 * kRpw;
    for (int i0 = ibeg; i0 < p.L; i0 += kRows) {
        __syncthreads();
        load_tile<DP>(Qs, p.Q + base, i0, p.L, p.d);
        load_tile<DP>(dOs, p.dO + base, i0, p.L, p.d);
        if (threadIdx.x < kRows) {
            const int i = i0 + threadIdx.x;
            float D = 0.0f, lse = -CUDART_INF_F;
            if (i < p.L) {
                lse = p.LSE[static_cast<size_t>(bh) * p.L + i];
                for (int c = 0; c < p.d; ++c) D += p.dO[base + static_cast<size_t>(i) * p.d + c] * p.O[base + static_cast<size_t>(i) * p.d + c];
            }
            Dr[threadIdx.x] = D; Ls[threadIdx.x] = lse;
        }
        __syncthreads();
        // phase 1: lane = query i0 + lane, against the warp's 8 key rows
        const int i = i0 + lane;
        const float* qr = Qs + lane * (DP + 1);
        const float* gr = dOs + lane * (DP + 1);
        const float lse = Ls[lane], Di = Dr[lane];
#pragma unroll
        for (int r = 0; r < kRpw; ++r) {
            const int rl = warp * kRpw + r, j = j0 + rl;
            const float* k = Ks + rl * DP;
            const float* v = Vs + rl * DP;
            float s = 0.0f, dp = 0.0f;
#pragma unroll 8
            for (int c = 0; c < DP; ++c) { s = fmaf(qr[c], k[c], s); dp = fmaf(gr[c], v[c], dp); }
            float pr = 0.0f, ds = 0.0f;
            const bool live = i < p.L && j < p.L && (!p.causal || j <= i) && lse > -CUDART_INF_F;
            if (live) {
                s *= p.scale;
                if (bias) s += bias[static_cast<size_t>(i) * p.L + j];
                pr = expf(s - lse);
                ds = pr * (dp - Di);
            }
            dSw[lane * kRpw + r] = ds;
            Pw[lane * kRpw + r] = pr;
        }
        __syncwarp();
        // phase 2: lane = channel; dK[j][c] += dS[i][j] Q[i][c], dV[j][c] += P[i][j] dO[i][c] over the 32 queries
#pragma unroll 4
        for (int ii = 0; ii < kRows; ++ii) {
            float dsr[kRpw], prr[kRpw];
#pragma unroll
            for (int r = 0; r < kRpw; ++r) { dsr[r] = dSw[ii * kRpw + r]; prr[r] = Pw[ii * kRpw + r]; }
#pragma unroll
            for (int a = 0; a < NACC; ++a) {
                const int c = lane + 32 * a;
                const float qv = (c < DP) ? Qs[ii * (DP + 1) + c] : 0.0f;
                const float gv = (c < DP) ? dOs[ii * (DP + 1) + c] : 0.0f;
#pragma unroll
                for (int r = 0; r < kRpw; ++r) { ak[r][a] = fmaf(dsr[r], qv, ak[r][a]); av[r][a] = fmaf(prr[r], gv, av[r][a]); }
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int r = 0; r < kRpw; ++r) {
        const int j = j0 + warp * kRpw + r;
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
            const int c = lane + 32 * a;
            if (j < p.L && c < p.d) {
                if (p.dK) p.dK[base + static_cast<size_t>(j) * p.d + c] = p.scale * ak[r][a];
                if (p.dV) p.dV[base + static_cast<size_t>(j) * p.d + c] = av[r][a];
            }
        }
    }
}

template <int DP>
int launch_dp(const BwdParams& p, cudaStream_t st) {
    const dim3 grid((p.L + kRows - 1) / kRows, p.B * p.H);
    if (p.dQ || p.dbias) {
        const size_t smem = sizeof(float) * (2 * kRows * (DP + 1) + 2 * kRows * DP + kWarps * 32 * kRpw + 2 * kRows);
        attn_bwd_dq_kernel<DP><<<grid, kWarps * 32, smem, st>>>(p);
        if (cudaGetLastError() != cudaSuccess) return ST_LAUNCH;
    }
    if (p.dK || p.dV) {
        const size_t smem = sizeof(float) * (2 * kRows * (DP + 1) + 2 * kRows * DP + 2 * kWarps * 32 * kRpw + 2 * kRows);
        attn_bwd_dkv_kernel<DP><<<grid, kWarps * 32, smem, st>>>(p);
        if (cudaGetLastError() != cudaSuccess) return ST_LAUNCH;
    }
    return ST_OK;
}

}  // namespace

int launch_attn_backward(int B, int H, int L, int d, int causal, float scale, const float* Q, const float* K, const float* V,
                         const float* bias, long long bias_batch_stride, const float* O, const float* dO, const float* LSE,
                         float* dQ, float* dK, float* dV, float* dbias, cudaStream_t st) {
    if (d > 64 || static_cast<long long>(B) * H > 65535) return ST_UNSUPPORTED_PATH;
    BwdParams p;
    p.B = B; p.H = H; p.L = L; p.d = d; p.causal = causal; p.scale = scale;
    p.Q = Q; p.K = K; p.V = V; p.bias = bias; p.O = O; p.dO = dO; p.LSE = LSE; p.bias_batch_stride = bias_batch_stride;
    p.dQ = dQ; p.dK = dK; p.dV = dV; p.dbias = dbias;
    if (d <= 8) return launch_dp<8>(p, st);
    if (d <= 16) return launch_dp<16>(p, st);
    if (d <= 32) return launch_dp<32>(p, st);
    return launch_dp<64>(p, st);
}

}  // namespace ppml_b200
