// simt_kernels.cu -- CUDA-core kernels: exact-fp32 contraction for every shape the tensor-core
// paths do not take (unaligned K, inner batch > 1, tiny extents), the block quantizers, casts, the
// dp4a Q8 product and the general attention kernel.  They keep the reference's summation order
// (k ascending per output element) so fp32 results agree with its CPU kernels to rounding.
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <type_traits>

namespace ppml_b200 {

__device__ int g_device_error[4] = {0, 0, 0, 0};

int* device_error_ptr() {
    static int* cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (cached[dev] == nullptr) {
        int* p = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_device_error) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        cached[dev] = p;
    }
    return cached[dev];
}

// =============================================================================================
// Generic strided batched contraction:  D[p][m][n] = epi( sum_k A[pa][m][k] * B[pb][n][k] )
// 64 x 64 output tile, 16-deep K slices, 256 threads, 4 x 4 outputs per thread.
// =============================================================================================
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, bool A_KFAST, bool B_KFAST>
__global__ void __launch_bounds__(256)
simt_contract_kernel(const T* __restrict__ A, const T* __restrict__ B, float* __restrict__ C, SimtContract p) {
    __shared__ float As[16][64 + 4];
    __shared__ float Bs[16][64 + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const long long m0 = static_cast<long long>(blockIdx.y) * 64, n0 = static_cast<long long>(blockIdx.x) * 64;

    for (long long plane = blockIdx.z; plane < p.planes; plane += gridDim.z) {
        const long long i3 = plane / p.ne2, i2 = plane - i3 * p.ne2;
        const T* Ap = A + (i2 / p.a_div2) * p.a_s2 + (i3 / p.a_div3) * p.a_s3;
        const T* Bp = B + i2 * p.b_s2 + i3 * p.b_s3;
        float* Cp = C + i2 * p.c_s2 + i3 * p.c_s3;

        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const long long n = n0 + tx * 4 + j;
                acc[i][j] = (p.bias_seed && p.bias != nullptr && n < p.N) ? p.bias[n] : 0.0f;
            }

        for (long long k0 = 0; k0 < p.K; k0 += 16) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = tid + i * 256;
                int mm, kk;
                if (A_KFAST) { kk = idx & 15; mm = idx >> 4; } else { mm = idx & 63; kk = idx >> 6; }
                const long long m = m0 + mm, k = k0 + kk;
                As[kk][mm] = (m < p.M && k < p.K) ? to_f32<T>(Ap[m * p.a_sm + k * p.a_sk]) : 0.0f;
                int nn, kb;
                if (B_KFAST) { kb = idx & 15; nn = idx >> 4; } else { nn = idx & 63; kb = idx >> 6; }
                const long long n = n0 + nn, k2 = k0 + kb;
                Bs[kb][nn] = (n < p.N && k2 < p.K) ? to_f32<T>(Bp[n * p.b_sn + k2 * p.b_sk]) : 0.0f;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < 16; ++kk) {
                float a[4], b[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            }
            __syncthreads();
        }

#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long m = m0 + ty * 4 + i;
            if (m >= p.M) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const long long n = n0 + tx * 4 + j;
                if (n >= p.N) continue;
                float v = acc[i][j] * p.alpha;
                if (p.ln_stats != nullptr) {           // LayerNorm folded into the Linear (bias_seed is 0 here)
                    const float2 st2 = *reinterpret_cast<const float2*>(p.ln_stats + 2 * m);
                    v = fmaf(-st2.x, p.ln_u[n], v) * st2.y;
                }
                if (!p.bias_seed && p.bias != nullptr) v += p.bias[n];
                if (p.clamp) {
                    if (!(v == v)) v = 0.0f; else v = fminf(fmaxf(v, -1e4f), 1e4f);
                }
                if (p.opm_L > 0) {
                    const long long d1 = m / p.opm_L, ii = m - d1 * p.opm_L;
                    const long long d2 = n / p.opm_L, jj = n - d2 * p.opm_L;
                    Cp[(((d1 * p.opm_D + d2) * p.opm_L + ii) * p.opm_L + jj) * p.opm_B] = v;
                } else {
                    if (p.gate != nullptr) v = act_scalar(p.act, v) * p.gate[m * p.c_sm + n * p.c_sn];
                    else if (p.act != 0) v = act_scalar(p.act, v);
                    Cp[m * p.c_sm + n * p.c_sn] = v;
                }
            }
        }
    }
}

template <typename T>
static int launch_contract_t(const T* A, const T* B, float* C, const SimtContract& p, cudaStream_t st) {
    if (p.M <= 0 || p.N <= 0 || p.planes <= 0) return ST_BAD_ARGS;
    dim3 grid(static_cast<unsigned>((p.N + 63) / 64), static_cast<unsigned>((p.M + 63) / 64),
              static_cast<unsigned>(p.planes < 32768 ? p.planes : 32768));
    if (grid.y > 65535u) return ST_BAD_ARGS;
    const bool ak = (p.a_sk == 1), bk = (p.b_sk == 1);
    if (ak && bk) simt_contract_kernel<T, true, true><<<grid, 256, 0, st>>>(A, B, C, p);
    else if (ak) simt_contract_kernel<T, true, false><<<grid, 256, 0, st>>>(A, B, C, p);
    else if (bk) simt_contract_kernel<T, false, true><<<grid, 256, 0, st>>>(A, B, C, p);
    else simt_contract_kernel<T, false, false><<<grid, 256, 0, st>>>(A, B, C, p);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

int launch_simt_contract(const void* A, const void* B, float* C, const SimtContract& p, int elem, cudaStream_t st) {
    if (elem == 0) return launch_contract_t<float>(static_cast<const float*>(A), static_cast<const float*>(B), C, p, st);
    if (elem == 1) return launch_contract_t<__half>(static_cast<const __half*>(A), static_cast<const __half*>(B), C, p, st);
    return launch_contract_t<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B), C, p, st);
}

// =============================================================================================
// LayerNorm folded into the Linear that follows it: per-row statistics of the activations and the weight-side terms.
// The statistics follow the reference's OP_NORM (src/backend/CPUKernels.cpp:1498-1511): mean, then the mean of the
// squared differences, then 1 / sqrt(var + eps); one warp per row.
// =============================================================================================
__global__ void __launch_bounds__(256)
row_stats_kernel(const float* __restrict__ x, float* __restrict__ mean_rstd, long long M, int K, float eps) {
    const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= M) return;
    const float* xr = x + row * K;
    float s = 0.0f;
    for (int k = lane; k < K; k += 32) s += xr[k];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    const float mean = s / static_cast<float>(K);
    float v = 0.0f;
    for (int k = lane; k < K; k += 32) { const float d = xr[k] - mean; v = fmaf(d, d, v); }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == 0) {
        mean_rstd[2 * row] = mean;
        mean_rstd[2 * row + 1] = 1.0f / sqrtf(v / static_cast<float>(K) + eps);
    }
}

int launch_row_stats(const float* x, float* mean_rstd, long long M, int K, float eps, cudaStream_t st) {
    if (!x || !mean_rstd || M <= 0 || K <= 0) return ST_BAD_ARGS;
    const long long grid = (M + 7) / 8;
    if (grid > 0x7fffffffLL) return ST_BAD_ARGS;
    row_stats_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(x, mean_rstd, M, K, eps);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

// One warp per output feature n: Wg[n][k] = W[n][k] * gamma[k], u[n] = sum_k Wg[n][k], v[n] = sum_k W[n][k] * beta[k] + bias[n]
__global__ void __launch_bounds__(256)
ln_fold_kernel(const float* __restrict__ W, const float* __restrict__ gamma, const float* __restrict__ beta,
               const float* __restrict__ bias, float* __restrict__ Wg, float* __restrict__ u, float* __restrict__ v, int N, int K) {
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (n >= N) return;
    float su = 0.0f, sv = 0.0f;
    for (int k = lane; k < K; k += 32) {
        const float w = W[static_cast<long long>(n) * K + k];
        const float wg = w * gamma[k];
        Wg[static_cast<long long>(n) * K + k] = wg;
        su += wg;
        sv = fmaf(w, beta[k], sv);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) { su += __shfl_xor_sync(0xffffffffu, su, off); sv += __shfl_xor_sync(0xffffffffu, sv, off); }
    if (lane == 0) { u[n] = su; v[n] = sv + (bias ? bias[n] : 0.0f); }
}

int launch_ln_fold(const float* W, const float* gamma, const float* beta, const float* bias, float* Wg, float* u, float* v, int N, int K,
                   cudaStream_t st) {
    if (!W || !gamma || !beta || !Wg || !u || !v || N <= 0 || K <= 0) return ST_BAD_ARGS;
    ln_fold_kernel<<<(N + 7) / 8, 256, 0, st>>>(W, gamma, beta, bias, Wg, u, v, N, K);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

// =============================================================================================
// Casts
// =============================================================================================
__device__ __forceinline__ void cast_store(__half* y, float x) { *y = __float2half_rn(x); }
__device__ __forceinline__ void cast_store(__nv_bfloat16* y, float x) { *y = __float2bfloat16_rn(x); }

template <typename T>
__global__ void cast_kernel(const float* __restrict__ x, T* __restrict__ y, long long n) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        cast_store(y + i, x[i]);
}

int launch_cast(const float* x, void* y, long long n, int to_bf16, cudaStream_t st) {
    if (!x || !y || n <= 0) return ST_BAD_ARGS;
    const int grid = static_cast<int>(((n + 255) / 256) < 148 * 16 ? ((n + 255) / 256) : 148 * 16);
    if (to_bf16) cast_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(x, static_cast<__nv_bfloat16*>(y), n);
    else cast_kernel<__half><<<grid, 256, 0, st>>>(x, static_cast<__half*>(y), n);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

// =============================================================================================
// Block quantizers (one warp per 32-element block, lane = element)
// =============================================================================================
// Activation quantizer, Q8_1: d = vmax / -128 where vmax is the signed value of the FIRST element
// holding the maximum magnitude; q = clamp(round(x * (1/d)), -128, 127); ds = (d, d * sum q) as half.
__global__ void quantize_q8_1_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, long long nblocks) {
    const long long ib = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (ib >= nblocks) return;
    const int lane = threadIdx.x & 31;
    const float v = x[ib * 32 + lane];
    float amax = fabsf(v), vmax = v;
    int idx = lane;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, off);
        const float ov = __shfl_xor_sync(0xffffffffu, vmax, off);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
        if (oa > amax || (oa == amax && oi < idx)) { amax = oa; vmax = ov; idx = oi; }
    }
    const float d = (amax == 0.0f) ? 0.0f : vmax / -128.0f;
    const float inv = (d == 0.0f) ? 0.0f : 1.0f / d;
    float q = roundf(v * inv);
    q = q > 127.0f ? 127.0f : (q < -128.0f ? -128.0f : q);
    const int qi = static_cast<int>(q);
    uint8_t* blk = y + ib * 36;
    reinterpret_cast<int8_t*>(blk)[4 + lane] = static_cast<int8_t>(qi);
    int qsum = qi;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, off);
    if (lane == 0) {
        const __half hd = __float2half_rn(d);
        const __half hs = __float2half_rn(d * static_cast<float>(qsum));
        reinterpret_cast<__half*>(blk)[0] = hd;
        reinterpret_cast<__half*>(blk)[1] = hs;
    }
}

int launch_quantize_q8_1(const float* x, void* y, long long ne, cudaStream_t st) {
    if (!x || !y || ne <= 0 || (ne % 32) != 0) return ST_BAD_ARGS;
    const long long nblocks = ne / 32;
    const long long grid = (nblocks + 7) / 8;
    if (grid > 0x7fffffffLL) return ST_BAD_ARGS;
    quantize_q8_1_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(x, static_cast<uint8_t*>(y), nblocks);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

// Weight quantizer, Q8_0 straight into the planar Q8_0R layout: d = amax / 127 (stored as half),
// q = clamp(round(x * (1/d)), -127, 127); qs plane [nblocks*32], then d plane [nblocks].
__global__ void quantize_q8_0r_kernel(const float* __restrict__ x, int8_t* __restrict__ qs, __half* __restrict__ dpl,
                                      long long nblocks) {
    const long long ib = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (ib >= nblocks) return;
    const int lane = threadIdx.x & 31;
    const float v = x[ib * 32 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float d = amax / 127.0f;
    const float inv = (amax == 0.0f) ? 0.0f : 1.0f / d;
    float q = roundf(v * inv);
    q = q > 127.0f ? 127.0f : (q < -127.0f ? -127.0f : q);
    qs[ib * 32 + lane] = static_cast<int8_t>(q);
    if (lane == 0) dpl[ib] = __float2half_rn(d);
}

int launch_quantize_q8_0r(const float* w, void* out, long long ne, cudaStream_t st) {
    if (!w || !out || ne <= 0 || (ne % 32) != 0) return ST_BAD_ARGS;
    const long long nblocks = ne / 32;
    const long long grid = (nblocks + 7) / 8;
    if (grid > 0x7fffffffLL) return ST_BAD_ARGS;
    int8_t* qs = static_cast<int8_t*>(out);
    __half* dpl = reinterpret_cast<__half*>(qs + nblocks * 32);
    quantize_q8_0r_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(w, qs, dpl, nblocks);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

__global__ void dequantize_q8_kernel(const uint8_t* __restrict__ x, float* __restrict__ y, long long ne, int bsize, int qoff) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= ne) return;
    const long long ib = i >> 5;
    const int iq = static_cast<int>(i & 31);
    const uint8_t* blk = x + ib * bsize;
    const float d = __half2float(*reinterpret_cast<const __half*>(blk));
    y[i] = d * static_cast<float>(reinterpret_cast<const int8_t*>(blk)[qoff + iq]);
}

int launch_dequantize_q8(const void* x, float* y, long long ne, int kind, cudaStream_t st) {
    if (!x || !y || ne <= 0) return ST_BAD_ARGS;
    const long long grid = (ne + 255) / 256;
    if (grid > 0x7fffffffLL) return ST_BAD_ARGS;
    dequantize_q8_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(static_cast<const uint8_t*>(x), y, ne,
                                                                      kind == 0 ? 34 : 36, kind == 0 ? 2 : 4);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

// =============================================================================================
// Q8_0 blocks as they lie on disk (34 bytes: half d, 32 int8; 2-byte aligned) -> planar Q8_0R ([nb * 32] int8, then
// [nb] half scales).  One thread per 4 quants; the thread of a block's first word also moves the scale.
// =============================================================================================
__global__ void __launch_bounds__(256)
repack_q8_0_kernel(const uint8_t* __restrict__ blocks, uint32_t* __restrict__ qs, uint16_t* __restrict__ d, long long nwords) {
    const long long w = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (w >= nwords) return;
    const long long b = w >> 3;
    const int j = static_cast<int>(w & 7);
    const uint8_t* src = blocks + b * 34;
    const uint16_t lo = *reinterpret_cast<const uint16_t*>(src + 2 + 4 * j);
    const uint16_t hi = *reinterpret_cast<const uint16_t*>(src + 4 + 4 * j);
    qs[w] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    if (j == 0) d[b] = *reinterpret_cast<const uint16_t*>(src);
}

int launch_repack_q8_0(const void* blocks34, long long nblocks, void* q8_0r, cudaStream_t st) {
    if (!blocks34 || !q8_0r || nblocks <= 0) return ST_BAD_ARGS;
    if ((reinterpret_cast<uintptr_t>(blocks34) & 1u) || (reinterpret_cast<uintptr_t>(q8_0r) & 3u)) return ST_BAD_ARGS;
    const long long nwords = nblocks * 8;
    const long long grid = (nwords + 255) / 256;
    if (grid > 0x7fffffffLL) return ST_BAD_ARGS;
    uint8_t* out = static_cast<uint8_t*>(q8_0r);
    repack_q8_0_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(static_cast<const uint8_t*>(blocks34), reinterpret_cast<uint32_t*>(out),
                                                                    reinterpret_cast<uint16_t*>(out + nblocks * 32), nwords);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

// =============================================================================================
// Q8 product on CUDA cores (dp4a): one thread per output (m = weight row, n = token).
// acts: Q8_1 blocks [N][nblk] (36 bytes each).  Per block: sumi (int32, exact), then
// acc += float(sumi) * (d_w * d_a), blocks in ascending order.
// =============================================================================================
__device__ __forceinline__ int load_i32_unaligned2(const uint8_t* p) {   // 2-byte aligned source
    const uint16_t lo = *reinterpret_cast<const uint16_t*>(p);
    const uint16_t hi = *reinterpret_cast<const uint16_t*>(p + 2);
    return static_cast<int>(static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16));
}

__global__ void __launch_bounds__(128)
q8_dp4a_kernel(const uint8_t* __restrict__ W, const uint8_t* __restrict__ acts, float* __restrict__ C,
               int M, int N, int nblk, int wtype, int c_trans, const float* __restrict__ bias,
               int* __restrict__ sumi_out) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    const size_t nb_all = static_cast<size_t>(M) * nblk;
    for (int n = blockIdx.y; n < N; n += gridDim.y) {
    const uint8_t* arow = acts + static_cast<size_t>(n) * nblk * 36;
    float acc = 0.0f;
    for (int ib = 0; ib < nblk; ++ib) {
        const size_t blk = static_cast<size_t>(m) * nblk + ib;
        int wq[8];
        float dw;
        if (wtype == 2) {
            const int* q = reinterpret_cast<const int*>(W + blk * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j) wq[j] = q[j];
            dw = __half2float(*reinterpret_cast<const __half*>(W + nb_all * 32 + blk * 2));
        } else if (wtype == 0) {
            const uint8_t* b = W + blk * 34;
#pragma unroll
            for (int j = 0; j < 8; ++j) wq[j] = load_i32_unaligned2(b + 2 + 4 * j);
            dw = __half2float(*reinterpret_cast<const __half*>(b));
        } else {
            const uint8_t* b = W + blk * 36;
            const int* q = reinterpret_cast<const int*>(b + 4);
#pragma unroll
            for (int j = 0; j < 8; ++j) wq[j] = q[j];
            dw = __half2float(*reinterpret_cast<const __half*>(b));
        }
        const uint8_t* ab = arow + static_cast<size_t>(ib) * 36;
        const int* va = reinterpret_cast<const int*>(ab + 4);
        int sumi = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) sumi = __dp4a(wq[j], va[j], sumi);
        if (sumi_out) sumi_out[(static_cast<size_t>(n) * M + m) * nblk + ib] = sumi;
        const float da = __half2float(*reinterpret_cast<const __half*>(ab));
        acc += static_cast<float>(sumi) * (dw * da);
    }
    if (bias) acc += bias[m];
    if (c_trans) C[static_cast<size_t>(n) * M + m] = acc;
    else C[static_cast<size_t>(m) * N + n] = acc;
    }
}

int launch_q8_dp4a(const void* W, const void* acts, float* C, int M, int N, int nblk, int wtype, int c_trans,
                   const float* bias, int* sumi_out, cudaStream_t st) {
    dim3 grid((M + 127) / 128, N < 65535 ? N : 65535);
    q8_dp4a_kernel<<<grid, 128, 0, st>>>(static_cast<const uint8_t*>(W), static_cast<const uint8_t*>(acts), C, M, N,
                                         nblk, wtype, c_trans, bias, sumi_out);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

// =============================================================================================
// Q8 product with very few output columns (the model's pair-bias and outer-product-mean projections: 128 -> 8,
// 256 -> 16, 64 -> 16), planar Q8_0R weights, C[token][M].  The tensor-core kernel is bound by its activation quantizer on
// such shapes; here the whole product is one pass over the activations on CUDA cores.  A lane takes one quant block
// (32 values, 128 contiguous bytes) of one token row, consecutive lanes consecutive blocks: the warp reads its 4 KB with
// eight fully coalesced 16-byte loads per lane into a padded shared-memory buffer and each lane reads its block back
// (a lane loading its own 128 bytes directly makes every load instruction touch 32 lines, which bounds the kernel by
// the L1 tag rate) -- quantizes it in registers by the Q8_1 rule (bit-exact with the host quantizer, see quantize_q8_1_kernel),
// takes its int32 dot products with the MP (padded M) weight rows from shared memory by dp4a, scales them, and the
// K / 32 lanes of a token row add their parts with shuffles.
// =============================================================================================
__device__ __forceinline__ uint32_t sk_pack_s8(int a, int b, uint32_t c) {       // (c << 16) | (sat_s8(a) << 8) | sat_s8(b)
    uint32_t r; asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); return r;
}
__device__ __forceinline__ int sk_round_half_away(float y) {                     // trunc(y + copysign(0.5, y)), the sum rounded toward zero
    float t; asm("add.rz.f32 %0, %1, %2;" : "=f"(t) : "f"(y), "f"(copysignf(0.5f, y)));
    int r; asm("cvt.rzi.s32.f32 %0, %1;" : "=r"(r) : "f"(t)); return r;
}

constexpr int kSkinnyWarps = 4, kSkinnyPitch = 36;     // floats per staged block: 16-byte reads of 8 lanes hit 8 bank groups

template <int MP>
__global__ void __launch_bounds__(32 * kSkinnyWarps)
q8_skinny_kernel(const uint8_t* __restrict__ W, const float* __restrict__ X, float* __restrict__ C, int M, long long units,
                 int nblk, int lg_nblk, const float* __restrict__ bias, int* __restrict__ sumi_out) {
    extern __shared__ __align__(16) int sk_smem[];
    int* ws = sk_smem;                                              // [MP][nblk][12] weight words: 8 used, a pitch of 48 bytes keeps the
                                                                    // 16-byte reads of lanes on different blocks off each other's banks
    float* dws = reinterpret_cast<float*>(ws + MP * nblk * 12);     // [MP][nblk] weight scales
    float* xs = dws + MP * nblk + (threadIdx.x >> 5) * (32 * kSkinnyPitch);     // this warp's 32 staged blocks
    const size_t nb_all = static_cast<size_t>(M) * nblk;
    const int lane = threadIdx.x & 31;
    const long long step = static_cast<long long>(gridDim.x) * (blockDim.x >> 5) * 32;
    long long u0 = (static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 32;
    // the warp's 32 blocks of a step are 256 16-byte words: word g (block g / 8, word g % 8 of it) by lane g % 32.  The first
    // step's words are requested before the weights are staged, every later step's while the one before is worked on
    float4 v[8];
    auto request = [&](long long base) {
        const float4* src = reinterpret_cast<const float4*>(X + base * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int g = j * 32 + lane;
            v[j] = (base + (g >> 3) < units) ? __ldg(src + g) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    if (u0 < units) request(u0);
    for (int e = threadIdx.x; e < MP * nblk * 8; e += blockDim.x) {          // planar: [M][nblk][32] int8, row m block ib at (m nblk + ib) 32
        const int blk = e >> 3;
        ws[blk * 12 + (e & 7)] = blk < M * nblk ? reinterpret_cast<const int*>(W)[e] : 0;
    }
    for (int e = threadIdx.x; e < MP * nblk; e += blockDim.x)
        dws[e] = e < M * nblk ? __half2float(*reinterpret_cast<const __half*>(W + nb_all * 32 + static_cast<size_t>(e) * 2)) : 0.0f;
    __syncthreads();
    for (; u0 < units; u0 += step) {
        const long long u = u0 + lane;
        const bool live = u < units;
        const long long row = u >> lg_nblk;
        const int ib = static_cast<int>(u & (nblk - 1));
        float x[32];
        {
            __syncwarp();                                                           // the previous step's reads are done
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int g = j * 32 + lane;
                *reinterpret_cast<float4*>(xs + (g >> 3) * kSkinnyPitch + (g & 7) * 4) = v[j];
            }
            __syncwarp();
            if (u0 + step < units) request(u0 + step);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 w = *reinterpret_cast<const float4*>(xs + lane * kSkinnyPitch + j * 4);
                x[4 * j] = w.x; x[4 * j + 1] = w.y; x[4 * j + 2] = w.z; x[4 * j + 3] = w.w;
            }
        }
        float amax = fabsf(x[0]), vmax = x[0];                      // the first element of maximum magnitude
#pragma unroll
        for (int j = 1; j < 32; ++j)
            if (fabsf(x[j]) > amax) { amax = fabsf(x[j]); vmax = x[j]; }
        const float d = (amax == 0.0f) ? 0.0f : vmax * -0.0078125f;
        const float inv = (d == 0.0f) ? 0.0f : 1.0f / d;
        uint32_t aq[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int q0 = sk_round_half_away(x[4 * j] * inv), q1 = sk_round_half_away(x[4 * j + 1] * inv);
            const int q2 = sk_round_half_away(x[4 * j + 2] * inv), q3 = sk_round_half_away(x[4 * j + 3] * inv);
            aq[j] = sk_pack_s8(q1, q0, sk_pack_s8(q3, q2, 0u));
        }
        const float da = __half2float(__float2half_rn(d));
        float part[MP];
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            const int4 w0 = *reinterpret_cast<const int4*>(ws + (m * nblk + ib) * 12);
            const int4 w1 = *reinterpret_cast<const int4*>(ws + (m * nblk + ib) * 12 + 4);
            int sumi = __dp4a(w0.x, static_cast<int>(aq[0]), 0);
            sumi = __dp4a(w0.y, static_cast<int>(aq[1]), sumi); sumi = __dp4a(w0.z, static_cast<int>(aq[2]), sumi);
            sumi = __dp4a(w0.w, static_cast<int>(aq[3]), sumi); sumi = __dp4a(w1.x, static_cast<int>(aq[4]), sumi);
            sumi = __dp4a(w1.y, static_cast<int>(aq[5]), sumi); sumi = __dp4a(w1.z, static_cast<int>(aq[6]), sumi);
            sumi = __dp4a(w1.w, static_cast<int>(aq[7]), sumi);
            if (sumi_out != nullptr && live && m < M) sumi_out[(static_cast<size_t>(row) * M + m) * nblk + ib] = sumi;
            part[m] = static_cast<float>(sumi) * (dws[m * nblk + ib] * da);
        }
        for (int off = nblk >> 1; off > 0; off >>= 1) {             // the lanes of a token row are neighbours (nblk is a power of two)
#pragma unroll
            for (int m = 0; m < MP; ++m) part[m] += __shfl_xor_sync(0xffffffffu, part[m], off);
        }
        if (live && ib == 0) {
            float* c = C + static_cast<size_t>(row) * M;
#pragma unroll
            for (int m = 0; m < MP; ++m)
                if (m < M) c[m] = part[m] + (bias != nullptr ? bias[m] : 0.0f);
        }
    }
}

// ST_UNSUPPORTED_PATH unless: planar weights (the caller checks), c_trans, M <= 16, K / 32 a power of two up to 32,
// activations 16-byte aligned
int launch_q8_skinny(const void* W, const float* X, float* C, int M, int N, int K, int c_trans, const float* bias,
                     int* sumi_out, cudaStream_t st) {
    const int nblk = K / 32;
    if (!c_trans || M > 16 || nblk < 1 || nblk > 32 || (nblk & (nblk - 1)) != 0 || (reinterpret_cast<uintptr_t>(X) & 15) != 0 ||
        (reinterpret_cast<uintptr_t>(W) & 3) != 0)
        return ST_UNSUPPORTED_PATH;
    int lg = 0;
    while ((1 << lg) < nblk) ++lg;
    const long long units = static_cast<long long>(N) * nblk;
    long long grid = (units + 32 * kSkinnyWarps - 1) / (32 * kSkinnyWarps);
    const long long cap = 8LL * num_sms();
    if (grid > cap) grid = cap;
    const int mp = M <= 8 ? 8 : 16;
    const size_t smem = static_cast<size_t>(mp) * nblk * (48 + 4) + kSkinnyWarps * 32 * kSkinnyPitch * sizeof(float);   // <= 44.4 KB
    if (mp == 8)
        q8_skinny_kernel<8><<<static_cast<unsigned>(grid), 32 * kSkinnyWarps, smem, st>>>(static_cast<const uint8_t*>(W), X, C, M, units, nblk, lg, bias, sumi_out);
    else
        q8_skinny_kernel<16><<<static_cast<unsigned>(grid), 32 * kSkinnyWarps, smem, st>>>(static_cast<const uint8_t*>(W), X, C, M, units, nblk, lg, bias, sumi_out);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

// =============================================================================================
// General attention forward (any L, Lk, head dim <= 128): a warp per query row at a time, lanes over keys.
// O = softmax(scale * Q K^T + bias) V with denominator (l + eps); LSE = m + log(l + eps);
// a row with no unmasked key gives O = 0, LSE = -inf.
// `ft` > 0 reproduces a property of the reference's CPU kernel (src/ops/FlashAttn.cpp:82-121), which walks the keys in
// tiles of Bc: when every score of the first tile (the first min(ft, visible keys) keys) is -inf, exp(-inf - -inf) turns
// its running sum into NaN, the final test `l > 0` fails and the row comes out as O = 0, LSE = -inf even if later keys are
// finite.  All attention kernels here take the same parameter; 0 gives the ordinary softmax over the visible keys.
// =============================================================================================
__device__ __forceinline__ float attn_ld(const float* p) { return *p; }
__device__ __forceinline__ float attn_ld(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ float attn_ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// CTA = 4 warps x kRowsPerWarp query rows of one (batch, head).  The keys are walked in tiles of 32 that the CTA stages
// in shared memory once for all its rows (K rows padded to d + 1 floats: lane = key reads its row without bank
// conflicts; V unpadded: lane = channel).  Per row and tile: lane j holds the score of key j0 + j, the maximum and the
// sum go through shuffles, then the 32 probabilities are broadcast one by one against the V tile.
// DT: the head dim when it is 32 or 64 (loops unrolled, the query row in registers), 0 = any head dim up to 128.
constexpr int kRowsPerWarp = 4;

template <typename T, int DT>
__global__ void __launch_bounds__(128)
attn_rowwarp_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                    const float* __restrict__ bias, float* __restrict__ O, float* __restrict__ LSE,
                    int H, int L, int Lk, int d, int causal, float scale, float eps, long long bias_batch_stride, int ft,
                    const AttnLayout lay) {
    extern __shared__ float sm[];
    float* ks = sm;                                  // [32][d + 1]
    float* vs = ks + 32 * (d + 1);                   // [32][d]
    float* qs = vs + 32 * d;                         // [4 * kRowsPerWarp][d]
    float* ps = qs + 4 * kRowsPerWarp * d;           // [4 * kRowsPerWarp][32] probabilities of the current tile (DT > 0)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * (4 * kRowsPerWarp);
    const int hh = blockIdx.y, b = blockIdx.z;
    const size_t bh = static_cast<size_t>(b) * H + hh;
    const T* Qb = Q + b * lay.q_b + hh * lay.q_h;
    const T* Kb = K + b * lay.k_b + hh * lay.k_h;
    const T* Vb = V + b * lay.v_b + hh * lay.v_h;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int i = row0 + warp * kRowsPerWarp + r;
        for (int dd = lane; dd < d; dd += 32)
            qs[(warp * kRowsPerWarp + r) * d + dd] = i < L ? attn_ld(Qb + static_cast<size_t>(i) * lay.q_l + dd) : 0.0f;
    }
    const int last_row = min(row0 + 4 * kRowsPerWarp - 1, L - 1);
    const int jend = causal ? min(last_row + 1, Lk) : Lk;     // keys needed by any row of this CTA
    float m[kRowsPerWarp], l[kRowsPerWarp], mfirst[kRowsPerWarp], acc[kRowsPerWarp][4];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        m[r] = -CUDART_INF_F; l[r] = 0.0f; mfirst[r] = -CUDART_INF_F;
#pragma unroll
        for (int t = 0; t < 4; ++t) acc[r][t] = 0.0f;
    }
    for (int j0 = 0; j0 < jend; j0 += 32) {
        __syncthreads();                             // every warp is done with the previous tile (and, first, qs is written)
        for (int key = warp; key < 32; key += 4) {
            const bool ok = j0 + key < Lk;
            const T* kp = Kb + static_cast<size_t>(ok ? j0 + key : 0) * lay.k_l;
            const T* vp = Vb + static_cast<size_t>(ok ? j0 + key : 0) * lay.v_l;
            for (int dd = lane; dd < d; dd += 32) {
                ks[key * (d + 1) + dd] = ok ? attn_ld(kp + dd) : 0.0f;
                vs[key * d + dd] = ok ? attn_ld(vp + dd) : 0.0f;
            }
        }
        __syncthreads();
        if constexpr (DT > 0) {
            // the warp's rows together: one read of a K or V element serves all of them, and the probabilities go to the
            // P V loop through shared memory (16-byte broadcast reads) instead of one shuffle per key and row
            const int j = j0 + lane;
            float dot[kRowsPerWarp];
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) dot[r] = 0.0f;
            const float* k = ks + lane * (DT + 1);
#pragma unroll
            for (int d4 = 0; d4 < DT / 4; ++d4) {
                const float k0 = k[4 * d4], k1 = k[4 * d4 + 1], k2 = k[4 * d4 + 2], k3 = k[4 * d4 + 3];
#pragma unroll
                for (int r = 0; r < kRowsPerWarp; ++r) {
                    const float4 q4 = *reinterpret_cast<const float4*>(qs + (warp * kRowsPerWarp + r) * DT + 4 * d4);
                    dot[r] = fmaf(q4.x, k0, dot[r]); dot[r] = fmaf(q4.y, k1, dot[r]);
                    dot[r] = fmaf(q4.z, k2, dot[r]); dot[r] = fmaf(q4.w, k3, dot[r]);
                }
            }
            float* pw = ps + warp * kRowsPerWarp * 32;
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                const int i = row0 + warp * kRowsPerWarp + r;
                const int jmax = i < L ? (causal ? min(i + 1, Lk) : Lk) : 0;
                float s = -CUDART_INF_F;
                if (j < jmax) {
                    s = dot[r] * scale;
                    if (bias) s += bias[static_cast<size_t>(b) * bias_batch_stride + (static_cast<size_t>(hh) * L + i) * static_cast<size_t>(Lk) + j];
                }
                if (j < ft) mfirst[r] = fmaxf(mfirst[r], s);
                float mt = s;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, off));
                const float m_new = fmaxf(m[r], mt);
                const float alpha = (m[r] == -CUDART_INF_F) ? 0.0f : expf(m[r] - m_new);
                const float pj = (j < jmax && m_new != -CUDART_INF_F) ? expf(s - m_new) : 0.0f;
                float lt = pj;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) lt += __shfl_xor_sync(0xffffffffu, lt, off);
                l[r] = alpha * l[r] + lt;
                m[r] = m_new;
#pragma unroll
                for (int t = 0; t < DT / 32; ++t) acc[r][t] *= alpha;
                pw[r * 32 + lane] = pj;
            }
            __syncwarp();
#pragma unroll 2
            for (int j4 = 0; j4 < 8; ++j4) {
                float v[4][DT / 32];
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int t = 0; t < DT / 32; ++t) v[u][t] = vs[(j4 * 4 + u) * DT + lane + 32 * t];
#pragma unroll
                for (int r = 0; r < kRowsPerWarp; ++r) {
                    const float4 p4 = *reinterpret_cast<const float4*>(pw + r * 32 + j4 * 4);
#pragma unroll
                    for (int t = 0; t < DT / 32; ++t) {
                        acc[r][t] = fmaf(p4.x, v[0][t], acc[r][t]); acc[r][t] = fmaf(p4.y, v[1][t], acc[r][t]);
                        acc[r][t] = fmaf(p4.z, v[2][t], acc[r][t]); acc[r][t] = fmaf(p4.w, v[3][t], acc[r][t]);
                    }
                }
            }
            __syncwarp();                            // the probabilities are read before the next tile overwrites them
            continue;
        }
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int i = row0 + warp * kRowsPerWarp + r;
            const int jmax = i < L ? (causal ? min(i + 1, Lk) : Lk) : 0;
            if (j0 >= jmax) continue;                // the same for every lane of the warp
            const float* myq = qs + (warp * kRowsPerWarp + r) * d;
            const int j = j0 + lane;
            float s = -CUDART_INF_F;
            if (j < jmax) {
                const float* k = ks + lane * (d + 1);
                float dot = 0.0f;
                if constexpr (DT > 0) {
#pragma unroll
                    for (int d4 = 0; d4 < DT / 4; ++d4) {
                        const float4 q4 = *reinterpret_cast<const float4*>(myq + 4 * d4);      // the same address in every lane
                        dot = fmaf(q4.x, k[4 * d4], dot); dot = fmaf(q4.y, k[4 * d4 + 1], dot);
                        dot = fmaf(q4.z, k[4 * d4 + 2], dot); dot = fmaf(q4.w, k[4 * d4 + 3], dot);
                    }
                } else {
                    for (int dd = 0; dd < d; ++dd) dot = fmaf(myq[dd], k[dd], dot);
                }
                s = dot * scale;
                if (bias) s += bias[static_cast<size_t>(b) * bias_batch_stride + (static_cast<size_t>(hh) * L + i) * static_cast<size_t>(Lk) + j];
            }
            if (j < ft) mfirst[r] = fmaxf(mfirst[r], s);
            float mt = s;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, off));
            const float m_new = fmaxf(m[r], mt);
            const float alpha = (m[r] == -CUDART_INF_F) ? 0.0f : expf(m[r] - m_new);
            const float pj = (j < jmax && m_new != -CUDART_INF_F) ? expf(s - m_new) : 0.0f;
            float lt = pj;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) lt += __shfl_xor_sync(0xffffffffu, lt, off);
            l[r] = alpha * l[r] + lt;
            m[r] = m_new;
#pragma unroll
            for (int t = 0; t < 4; ++t) acc[r][t] *= alpha;
            const int nj = (jmax - j0 < 32) ? (jmax - j0) : 32;
            if constexpr (DT > 0) {
                if (nj == 32) {
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) {
                        const float p = __shfl_sync(0xffffffffu, pj, jj);
#pragma unroll
                        for (int t = 0; t < DT / 32; ++t) acc[r][t] = fmaf(p, vs[jj * DT + lane + 32 * t], acc[r][t]);
                    }
                } else {
                    for (int jj = 0; jj < nj; ++jj) {
                        const float p = __shfl_sync(0xffffffffu, pj, jj);
#pragma unroll
                        for (int t = 0; t < DT / 32; ++t) acc[r][t] = fmaf(p, vs[jj * DT + lane + 32 * t], acc[r][t]);
                    }
                }
            } else {
                for (int jj = 0; jj < nj; ++jj) {
                    const float p = __shfl_sync(0xffffffffu, pj, jj);
                    const float* v = vs + jj * d;
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const int dd = lane + 32 * t;
                        if (dd < d) acc[r][t] = fmaf(p, v[dd], acc[r][t]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int i = row0 + warp * kRowsPerWarp + r;
        float mf = mfirst[r];
        if (ft > 0) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mf = fmaxf(mf, __shfl_xor_sync(0xffffffffu, mf, off));
        }
        if (i >= L) continue;
        float lr = l[r];
        if (ft > 0 && mf == -CUDART_INF_F) lr = 0.0f;    // the reference's first key tile is fully masked: O = 0, LSE = -inf
        const long long ooff = b * lay.o_b + hh * lay.o_h + static_cast<long long>(i) * lay.o_l;
        const long long goff = b * lay.g_b + hh * lay.g_h + static_cast<long long>(i) * lay.g_l;
        float* o = O + ooff;
        if (lr > 0.0f) {
            const float inv = 1.0f / (lr + eps);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int dd = lane + 32 * t;
                if (dd < d) o[dd] = lay.gate ? act_scalar(lay.act, lay.gate[goff + dd]) * (acc[r][t] * inv) : acc[r][t] * inv;
            }
            if (LSE && lane == 0) LSE[bh * L + i] = m[r] + logf(lr + eps);
        } else {
#pragma unroll
            for (int t = 0; t < 4; ++t) { const int dd = lane + 32 * t; if (dd < d) o[dd] = 0.0f; }
            if (LSE && lane == 0) LSE[bh * L + i] = -CUDART_INF_F;
        }
    }
}

// =============================================================================================
// Small head dims (4, 8, 16: the extra-MSA blocks use 8): one thread per R query rows, R * NT rows per CTA.  Keys are
// walked in tiles of 16; the K and V tiles are staged in shared memory as fp32 and every thread reads the same key,
// so the reads are broadcasts -- and they are what the load/store pipe spends its time on, which is why a thread owns
// R rows: one 16-byte read of K or V serves R rows.  The arithmetic is packed fp32 pairs (one issue slot for two
// FMAs): the score is summed over channel pairs (even and odd channels apart, one add at the end, the bias as the
// start value), the P V product over key pairs (V is staged with the two keys of a pair interleaved, the
// accumulators of even and odd keys are added at the end).  Running maximum / sum / accumulators are per-thread
// scalars: no shuffles and no cross-lane reductions.  Same arithmetic contract as the kernel above; exp is
// 2^((s - m) log2 e) on the transcendental unit.
// =============================================================================================
// 2^x on the transcendental unit (about 2 ulp); results below the normal range flush to 0, 2^-inf = 0
__device__ __forceinline__ float ex2_fast(float x) {
    float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y;
}

template <typename T, int D, int R, int NT>
__global__ void __launch_bounds__(NT)
attn_rowthread_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                      const float* __restrict__ bias, float* __restrict__ O, float* __restrict__ LSE,
                      int H, int L, int Lk, int causal, float scale, float eps, long long bias_batch_stride, int ft,
                      int bias_vec, const AttnLayout lay) {
    constexpr int kTile = 16;
    constexpr int kRows = R * NT;
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr int kPer = (kTile * D + NT - 1) / NT;             // K (and V) elements each thread moves per tile
    constexpr int kPitch = kTile + 4;                           // 80-byte bias rows: 16-byte reads of 8 lanes hit 8 bank groups
    constexpr int D2 = D / 2, D4 = D / 4;
    // two stages of everything: the next tile's K / V travel through registers and its bias through cp.async while
    // the current tile is consumed
    __shared__ __align__(16) float ks_all[2][kTile * D];        // [key][channel]
    __shared__ __align__(16) float vs_all[2][kTile * D];        // [key pair][channel][key of the pair]
    __shared__ __align__(16) float bs_all[2][kRows * kPitch];   // [row of the CTA][key]
    const int hh = blockIdx.y, b = blockIdx.z;
    const size_t bh = static_cast<size_t>(b) * H + hh;
    const T* Kb = K + b * lay.k_b + hh * lay.k_h;
    const T* Vb = V + b * lay.v_b + hh * lay.v_h;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kRows;
    // row k of this thread: row0 + k * NT + threadIdx.x (a warp's rows of one k are consecutive)
    int jmax[R];
    uint64_t q2[R][D2];
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const int i = row0 + k * NT + threadIdx.x;
        const bool ok = i < L;
        jmax[k] = ok ? (causal ? min(i + 1, Lk) : Lk) : 0;
        const T* qp = Q + b * lay.q_b + hh * lay.q_h + static_cast<long long>(ok ? i : 0) * lay.q_l;
#pragma unroll
        for (int c = 0; c < D2; ++c)
            q2[k][c] = ok ? pack2(attn_ld(qp + 2 * c) * scale, attn_ld(qp + 2 * c + 1) * scale) : 0ull;
    }
    const float* Bh = bias ? bias + static_cast<size_t>(b) * bias_batch_stride + static_cast<size_t>(hh) * L * static_cast<size_t>(Lk)
                           : nullptr;
    // keys needed by any row of this CTA
    const int last_row = min(row0 + kRows - 1, L - 1);
    const int jend = causal ? min(last_row + 1, Lk) : Lk;
    float m[R], mfirst[R];
    uint64_t l2[R], acc2[R][D];                      // sums over even and odd keys apart
#pragma unroll
    for (int k = 0; k < R; ++k) {
        m[k] = -CUDART_INF_F; mfirst[k] = -CUDART_INF_F; l2[k] = 0ull;
#pragma unroll
        for (int dd = 0; dd < D; ++dd) acc2[k][dd] = 0ull;
    }
    float kreg[kPer], vreg[kPer];
    auto fetch_kv = [&](int j0) {
#pragma unroll
        for (int c = 0; c < kPer; ++c) {
            const int e = threadIdx.x + c * NT;
            const bool ok = e < kTile * D && j0 + e / D < Lk;
            kreg[c] = ok ? attn_ld(Kb + static_cast<long long>(j0 + e / D) * lay.k_l + e % D) : 0.0f;
            vreg[c] = ok ? attn_ld(Vb + static_cast<long long>(j0 + e / D) * lay.v_l + e % D) : 0.0f;
        }
    };
    // bias: every warp brings the 32 x 16 tiles of its own rows through shared memory (coalesced on the global side)
    // and each thread then reads its rows back with 16-byte loads
    auto fetch_bias = [&](int j0, int buf) {
        if (Bh) {
#pragma unroll
            for (int k = 0; k < R; ++k) {
                const int rl0 = k * NT + warp * 32;                      // first row (within the CTA) of this 32-row tile
                if (bias_vec) {
                    // 16 bytes per lane: four lanes per row, eight rows per instruction
#pragma unroll
                    for (int it = 0; it < 4; ++it) {
                        const int rl = rl0 + it * 8 + (lane >> 2), c = (lane & 3) * 4;
                        const bool ok = row0 + rl < L && j0 + c < Lk;    // Lk is a multiple of 4 here
                        const float* src = ok ? Bh + static_cast<size_t>(row0 + rl) * Lk + j0 + c : Bh;
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(static_cast<uint32_t>(
                                         __cvta_generic_to_shared(&bs_all[buf][rl * kPitch + c]))), "l"(src), "r"(ok ? 16 : 0) : "memory");
                    }
                } else {
#pragma unroll
                    for (int it = 0; it < 16; ++it) {
                        const int rl = rl0 + it * 2 + (lane >> 4), c = lane & 15;
                        const bool ok = row0 + rl < L && j0 + c < Lk;
                        const float* src = ok ? Bh + static_cast<size_t>(row0 + rl) * Lk + j0 + c : Bh;
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(static_cast<uint32_t>(
                                         __cvta_generic_to_shared(&bs_all[buf][rl * kPitch + c]))), "l"(src), "r"(ok ? 4 : 0) : "memory");
                    }
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch_kv(0);
    fetch_bias(0, 0);
    const uint64_t log2e2 = pack2(kLog2e, kLog2e);
    for (int j0 = 0, tile = 0; j0 < jend; j0 += kTile, ++tile) {
        const int buf = tile & 1;
        float* ks = ks_all[buf];
        float* vs = vs_all[buf];
        const float* bs = bs_all[buf];
        // this stage was last read two tiles ago, and every thread has passed the barrier of the tile in between
#pragma unroll
        for (int c = 0; c < kPer; ++c) {
            const int e = threadIdx.x + c * NT;
            if (e < kTile * D) {
                const int key = e / D, dd = e % D;
                ks[e] = kreg[c];
                vs[((key >> 1) * D + dd) * 2 + (key & 1)] = vreg[c];
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (j0 + kTile < jend) { fetch_kv(j0 + kTile); fetch_bias(j0 + kTile, buf ^ 1); }
        // scores: x[k][t] starts as the bias and becomes q . k_t + bias
        float x[R][kTile];
#pragma unroll
        for (int k = 0; k < R; ++k) {
            if (Bh) {
#pragma unroll
                for (int t4 = 0; t4 < kTile / 4; ++t4) {
                    const float4 b4 = *reinterpret_cast<const float4*>(bs + (k * NT + threadIdx.x) * kPitch + t4 * 4);
                    x[k][t4 * 4] = b4.x; x[k][t4 * 4 + 1] = b4.y; x[k][t4 * 4 + 2] = b4.z; x[k][t4 * 4 + 3] = b4.w;
                }
            } else {
#pragma unroll
                for (int t = 0; t < kTile; ++t) x[k][t] = 0.0f;
            }
        }
#pragma unroll
        for (int t = 0; t < kTile; ++t) {
            uint64_t kk[D2];
#pragma unroll
            for (int c4 = 0; c4 < D4; ++c4) {
                const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(ks + t * D + c4 * 4);
                kk[2 * c4] = v.x; kk[2 * c4 + 1] = v.y;
            }
#pragma unroll
            for (int k = 0; k < R; ++k) {
                uint64_t s = pack2(x[k][t], 0.0f);
#pragma unroll
                for (int c = 0; c < D2; ++c) s = ffma2(q2[k][c], kk[c], s);
                float se, so; unpack2(s, se, so);
                x[k][t] = se + so;
            }
        }
        // per row: mask, maximum, rescale factor, probabilities (in place of the scores)
        uint64_t alpha2[R];
#pragma unroll
        for (int k = 0; k < R; ++k) {
            if (j0 + kTile > jmax[k]) {
#pragma unroll
                for (int t = 0; t < kTile; ++t) if (j0 + t >= jmax[k]) x[k][t] = -CUDART_INF_F;
            }
            float mt = -CUDART_INF_F;
#pragma unroll
            for (int t = 0; t < kTile; ++t) mt = fmaxf(mt, x[k][t]);
            if (j0 < ft) {
                if (j0 + kTile <= ft) mfirst[k] = fmaxf(mfirst[k], mt);
                else {
#pragma unroll
                    for (int t = 0; t < kTile; ++t) if (j0 + t < ft) mfirst[k] = fmaxf(mfirst[k], x[k][t]);
                }
            }
            const float m_new = fmaxf(m[k], mt);
            // nothing visible so far: alpha = 0 and every probability 2^-inf = 0, the state stays empty
            const float alpha = (m[k] == -CUDART_INF_F) ? 0.0f : ex2_fast((m[k] - m_new) * kLog2e);
            const float ml2 = (m_new == -CUDART_INF_F) ? 0.0f : m_new * kLog2e;
            const uint64_t nml2 = pack2(-ml2, -ml2);
            alpha2[k] = pack2(alpha, alpha);
            uint64_t lt = 0ull;
#pragma unroll
            for (int tp = 0; tp < kTile / 2; ++tp) {
                float e0, e1;
                unpack2(ffma2(pack2(x[k][2 * tp], x[k][2 * tp + 1]), log2e2, nml2), e0, e1);
                x[k][2 * tp] = ex2_fast(e0);
                x[k][2 * tp + 1] = ex2_fast(e1);
                lt = fadd2(lt, pack2(x[k][2 * tp], x[k][2 * tp + 1]));
            }
            l2[k] = ffma2(l2[k], alpha2[k], lt);
            m[k] = m_new;
#pragma unroll
            for (int dd = 0; dd < D; ++dd) acc2[k][dd] = fmul2(acc2[k][dd], alpha2[k]);
        }
        // P V over key pairs
#pragma unroll
        for (int tp = 0; tp < kTile / 2; ++tp) {
            uint64_t vv[D];
#pragma unroll
            for (int c2 = 0; c2 < D2; ++c2) {
                const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(vs + tp * 2 * D + c2 * 4);
                vv[2 * c2] = v.x; vv[2 * c2 + 1] = v.y;
            }
#pragma unroll
            for (int k = 0; k < R; ++k) {
                const uint64_t p2 = pack2(x[k][2 * tp], x[k][2 * tp + 1]);
#pragma unroll
                for (int dd = 0; dd < D; ++dd) acc2[k][dd] = ffma2(p2, vv[dd], acc2[k][dd]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const int i = row0 + k * NT + threadIdx.x;
        if (i >= L) continue;
        float le, lo; unpack2(l2[k], le, lo);
        float l = le + lo;
        if (ft > 0 && mfirst[k] == -CUDART_INF_F) l = 0.0f;  // the reference's first key tile is fully masked: O = 0, LSE = -inf
        const long long ooff = b * lay.o_b + hh * lay.o_h + static_cast<long long>(i) * lay.o_l;
        const long long goff = b * lay.g_b + hh * lay.g_h + static_cast<long long>(i) * lay.g_l;
        float* o = O + ooff;
        float inv = 0.0f, lse = -CUDART_INF_F;
        if (l > 0.0f) { inv = 1.0f / (l + eps); lse = m[k] + logf(l + eps); }
        float r[D];
#pragma unroll
        for (int dd = 0; dd < D; ++dd) {
            float ae, ao; unpack2(acc2[k][dd], ae, ao);
            const float v = (ae + ao) * inv;
            r[dd] = lay.gate ? act_scalar(lay.act, lay.gate[goff + dd]) * v : v;
        }
        if ((reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
            for (int c4 = 0; c4 < D4; ++c4)
                *reinterpret_cast<float4*>(o + c4 * 4) = make_float4(r[c4 * 4], r[c4 * 4 + 1], r[c4 * 4 + 2], r[c4 * 4 + 3]);
        } else {
#pragma unroll
            for (int dd = 0; dd < D; ++dd) o[dd] = r[dd];
        }
        if (LSE) LSE[bh * L + i] = lse;
    }
}

// Small head dims with few query rows (global column attention: one query over all keys): one warp per query row,
// every lane keeps a private running maximum / sum / accumulator over the keys lane, lane + 32, ..., and the 32 partial
// results are merged at the end (rescaled to the common maximum, then summed with shuffles).
template <typename T, int D>
__global__ void __launch_bounds__(128)
attn_keylanes_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                     const float* __restrict__ bias, float* __restrict__ O, float* __restrict__ LSE,
                     int H, int L, int Lk, int causal, float scale, float eps, long long bias_batch_stride, long long rows_total,
                     int ft, const AttnLayout lay) {
    constexpr float kLog2e = 1.4426950408889634f;
    const int lane = threadIdx.x & 31;
    const long long row = blockIdx.x * 4LL + (threadIdx.x >> 5);          // flattened (batch, head, query)
    if (row >= rows_total) return;
    const int i = static_cast<int>(row % L);
    const long long bh = row / L;
    const int hh = static_cast<int>(bh % H);
    const long long b = bh / H;
    float q[D];
#pragma unroll
    for (int dd = 0; dd < D; ++dd) q[dd] = attn_ld(Q + b * lay.q_b + hh * lay.q_h + static_cast<long long>(i) * lay.q_l + dd) * scale;
    const T* Kb = K + b * lay.k_b + hh * lay.k_h;
    const T* Vb = V + b * lay.v_b + hh * lay.v_h;
    const float* Bb = bias ? bias + b * bias_batch_stride + (static_cast<long long>(hh) * L + i) * Lk : nullptr;
    const int jmax = causal ? min(i + 1, Lk) : Lk;
    float m = -CUDART_INF_F, l = 0.0f;
    float mfirst = -CUDART_INF_F;                    // maximum over the first `ft` keys
    float acc[D];
#pragma unroll
    for (int dd = 0; dd < D; ++dd) acc[dd] = 0.0f;
#pragma unroll 4
    for (int j = lane; j < jmax; j += 32) {
        float s = 0.0f;
#pragma unroll
        for (int dd = 0; dd < D; ++dd) s = fmaf(q[dd], attn_ld(Kb + static_cast<long long>(j) * lay.k_l + dd), s);
        if (Bb) s += Bb[j];
        if (j < ft) mfirst = fmaxf(mfirst, s);
        const float m_new = fmaxf(m, s);
        if (m_new == -CUDART_INF_F) continue;                             // masked key, nothing visible before it
        const float alpha = exp2f((m - m_new) * kLog2e);                  // m = -inf gives 0
        const float pj = exp2f((s - m_new) * kLog2e);
        l = fmaf(l, alpha, pj);
#pragma unroll
        for (int dd = 0; dd < D; ++dd) acc[dd] = fmaf(acc[dd], alpha, pj * attn_ld(Vb + static_cast<long long>(j) * lay.v_l + dd));
        m = m_new;
    }
    float mw = m;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, off));
    const float f = (m == -CUDART_INF_F) ? 0.0f : exp2f((m - mw) * kLog2e);
    l *= f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
    if (ft > 0) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mfirst = fmaxf(mfirst, __shfl_xor_sync(0xffffffffu, mfirst, off));
        if (mfirst == -CUDART_INF_F) l = 0.0f;       // the reference's first key tile is fully masked: O = 0, LSE = -inf
    }
    float inv = 0.0f, lse = -CUDART_INF_F;
    if (l > 0.0f) { inv = 1.0f / (l + eps); lse = mw + logf(l + eps); }
#pragma unroll
    for (int dd = 0; dd < D; ++dd) {
        float a = acc[dd] * f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        if (lane == 0) {
            const long long oo = b * lay.o_b + hh * lay.o_h + static_cast<long long>(i) * lay.o_l + dd;
            const long long go = b * lay.g_b + hh * lay.g_h + static_cast<long long>(i) * lay.g_l + dd;
            O[oo] = lay.gate ? act_scalar(lay.act, lay.gate[go]) * (a * inv) : a * inv;
        }
    }
    if (LSE && lane == 0) LSE[row] = lse;
}

template <typename T>
bool launch_attn_keylanes(const T* Q, const T* K, const T* V, const float* bias, float* O, float* LSE, int B, int H, int L,
                          int Lk, int d, int causal, float scale, float eps, long long bias_batch_stride, int ft, const AttnLayout& lay, cudaStream_t st) {
    const long long rows = static_cast<long long>(B) * H * L;
    const long long blocks = (rows + 3) / 4;
    if (blocks > 0x7fffffffLL) return false;
    const unsigned grid = static_cast<unsigned>(blocks);
    if (d == 4) attn_keylanes_kernel<T, 4><<<grid, 128, 0, st>>>(Q, K, V, bias, O, LSE, H, L, Lk, causal, scale, eps, bias_batch_stride, rows, ft, lay);
    else if (d == 8) attn_keylanes_kernel<T, 8><<<grid, 128, 0, st>>>(Q, K, V, bias, O, LSE, H, L, Lk, causal, scale, eps, bias_batch_stride, rows, ft, lay);
    else if (d == 16) attn_keylanes_kernel<T, 16><<<grid, 128, 0, st>>>(Q, K, V, bias, O, LSE, H, L, Lk, causal, scale, eps, bias_batch_stride, rows, ft, lay);
    else return false;
    return true;
}

template <typename T, int D>
void launch_attn_rowthread_d(const T* Q, const T* K, const T* V, const float* bias, float* O, float* LSE, int B, int H, int L,
                             int Lk, int causal, float scale, float eps, long long bias_batch_stride, int ft, int bias_vec,
                             const AttnLayout& lay, cudaStream_t st) {
    // two rows per thread; the CTA shrinks with the number of query rows so that short sequences still fill their CTAs
    if (L > 128) {
        dim3 grid((L + 255) / 256, H, B);
        attn_rowthread_kernel<T, D, 2, 128><<<grid, 128, 0, st>>>(Q, K, V, bias, O, LSE, H, L, Lk, causal, scale, eps, bias_batch_stride, ft, bias_vec, lay);
    } else if (L > 64) {
        dim3 grid((L + 127) / 128, H, B);
        attn_rowthread_kernel<T, D, 2, 64><<<grid, 64, 0, st>>>(Q, K, V, bias, O, LSE, H, L, Lk, causal, scale, eps, bias_batch_stride, ft, bias_vec, lay);
    } else {
        dim3 grid((L + 63) / 64, H, B);
        attn_rowthread_kernel<T, D, 2, 32><<<grid, 32, 0, st>>>(Q, K, V, bias, O, LSE, H, L, Lk, causal, scale, eps, bias_batch_stride, ft, bias_vec, lay);
    }
}

template <typename T>
bool launch_attn_rowthread(const T* Q, const T* K, const T* V, const float* bias, float* O, float* LSE, int B, int H, int L,
                           int Lk, int d, int causal, float scale, float eps, long long bias_batch_stride, int ft, const AttnLayout& lay, cudaStream_t st) {
    // 16-byte bias copies need whole 16-byte pieces in every row
    const int bias_vec = bias != nullptr && (Lk & 3) == 0 && (bias_batch_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(bias) & 15) == 0;
    if (d == 4) launch_attn_rowthread_d<T, 4>(Q, K, V, bias, O, LSE, B, H, L, Lk, causal, scale, eps, bias_batch_stride, ft, bias_vec, lay, st);
    else if (d == 8) launch_attn_rowthread_d<T, 8>(Q, K, V, bias, O, LSE, B, H, L, Lk, causal, scale, eps, bias_batch_stride, ft, bias_vec, lay, st);
    else if (d == 16) launch_attn_rowthread_d<T, 16>(Q, K, V, bias, O, LSE, B, H, L, Lk, causal, scale, eps, bias_batch_stride, ft, bias_vec, lay, st);
    else return false;
    return true;
}

int launch_attn_rowwarp(const void* Q, const void* K, const void* V, int elem, const float* bias, float* O, float* LSE,
                        int B, int H, int L, int Lk, int d, int causal, float scale, float eps,
                        long long bias_batch_stride, int ft, const AttnLayout& lay, cudaStream_t st) {
    if (d > 128 || H > 65535 || B > 65535 || elem < 0 || elem > 2) return ST_BAD_ARGS;
    // small head dims with enough query rows to fill CTAs of one thread per row
    if ((d == 4 || d == 8 || d == 16) && L < 32) {
        bool done;
        if (elem == 0) done = launch_attn_keylanes(static_cast<const float*>(Q), static_cast<const float*>(K), static_cast<const float*>(V),
                                                   bias, O, LSE, B, H, L, Lk, d, causal, scale, eps, bias_batch_stride, ft, lay, st);
        else if (elem == 1) done = launch_attn_keylanes(static_cast<const __nv_bfloat16*>(Q), static_cast<const __nv_bfloat16*>(K),
                                                        static_cast<const __nv_bfloat16*>(V), bias, O, LSE, B, H, L, Lk, d, causal, scale, eps,
                                                        bias_batch_stride, ft, lay, st);
        else done = launch_attn_keylanes(static_cast<const __half*>(Q), static_cast<const __half*>(K), static_cast<const __half*>(V),
                                         bias, O, LSE, B, H, L, Lk, d, causal, scale, eps, bias_batch_stride, ft, lay, st);
        if (done) return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
    }
    if ((d == 4 || d == 8 || d == 16) && L >= 32) {
        bool done;
        if (elem == 0) done = launch_attn_rowthread(static_cast<const float*>(Q), static_cast<const float*>(K), static_cast<const float*>(V),
                                                    bias, O, LSE, B, H, L, Lk, d, causal, scale, eps, bias_batch_stride, ft, lay, st);
        else if (elem == 1) done = launch_attn_rowthread(static_cast<const __nv_bfloat16*>(Q), static_cast<const __nv_bfloat16*>(K),
                                                         static_cast<const __nv_bfloat16*>(V), bias, O, LSE, B, H, L, Lk, d, causal, scale, eps,
                                                         bias_batch_stride, ft, lay, st);
        else done = launch_attn_rowthread(static_cast<const __half*>(Q), static_cast<const __half*>(K), static_cast<const __half*>(V),
                                          bias, O, LSE, B, H, L, Lk, d, causal, scale, eps, bias_batch_stride, ft, lay, st);
        if (done) return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
    }
    dim3 grid((L + 4 * kRowsPerWarp - 1) / (4 * kRowsPerWarp), H, B);
    const size_t smem = (32 * (d + 1) + 32 * d + 4 * kRowsPerWarp * (d + 32)) * sizeof(float);     // at most 43 KB (d = 128)
    auto go = [&](auto tag, auto dt) {
        using T = decltype(tag);
        constexpr int DT = decltype(dt)::value;
        attn_rowwarp_kernel<T, DT><<<grid, 128, smem, st>>>(static_cast<const T*>(Q), static_cast<const T*>(K), static_cast<const T*>(V),
                                                            bias, O, LSE, H, L, Lk, d, causal, scale, eps, bias_batch_stride, ft, lay);
    };
    auto by_dim = [&](auto tag) {
        if (d == 32) go(tag, std::integral_constant<int, 32>{});
        else if (d == 64) go(tag, std::integral_constant<int, 64>{});
        else go(tag, std::integral_constant<int, 0>{});
    };
    if (elem == 0) by_dim(float{});
    else if (elem == 1) by_dim(__nv_bfloat16{});
    else by_dim(__half{});
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

}  // namespace ppml_b200
