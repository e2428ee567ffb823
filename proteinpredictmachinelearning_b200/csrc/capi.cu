// capi.cu -- the extern "C" boundary (include/ppml_b200.h): argument checks, choice between the
// tcgen05 and the CUDA-core kernels, launches.  No entry point here computes on the host.
#include <cuda_fp16.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/ppml_b200.h"
#include "kernels.h"

using namespace ppml_b200;

namespace {

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

inline bool path_ok(int path) { return path >= PPML_B200_PATH_AUTO && path <= PPML_B200_PATH_UMMA; }

// Grow-only device scratch for the dp4a Q8 path (Q8_1 activation blocks), one per device, guarded
// by a mutex as the reference's launcher does (src/cuda/MulMatQ8Kernel.cu:430-449).
struct Scratch { void* ptr = nullptr; size_t bytes = 0; };
Scratch g_scratch[64];
std::mutex g_scratch_mtx;

void* ensure_scratch(size_t bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    Scratch& s = g_scratch[dev];
    if (bytes <= s.bytes) return s.ptr;
    if (s.ptr) { cudaFree(s.ptr); s.ptr = nullptr; s.bytes = 0; }
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    s.ptr = p; s.bytes = bytes;
    return p;
}

// Whether the tensor-core Q8 product quantizes its activations in a kernel of its own (into the shared scratch) instead
// of inside the product kernel.  Measured on the sweep shapes: the one-pass form wins wherever there are more token
// tiles than SMs (33 vs 44 us at 65536 x 128 x 128, 126 vs 197 us at 65536 x 1024 x 128: the extra pass over X costs
// more than the quantizer warps do); with few token tiles and a long K the in-kernel quantizer is a serial chain of
// K / 32 steps on two or four warps, and the two-pass form wins (33 vs 41 us at 408 x 1024 x N, 58 vs 68 us at
// 2601 x 1024 x 1024).  PPML_B200_Q8_TWO_PASS=0 / 1 or ppml_b200_set_q8_two_pass() force the choice (measurements, tests).
int g_q8_two_pass = [] { const char* e = std::getenv("PPML_B200_Q8_TWO_PASS"); return e ? (e[0] == '1' ? 1 : 0) : -1; }();
bool q8_two_pass(int M, int N, int K) {
    const int forced = g_q8_two_pass;
    if (forced >= 0) return forced == 1;
    (void)M;
    return (N + 127) / 128 <= num_sms() && K >= 1024;
}

int mul_mat_any(const void* A, const void* B, float* C, int M, int K, int N, const float* bias, int path,
                int elem, int tf32_mode, cudaStream_t st) {
    if (!A || !B || !C || M <= 0 || K <= 0 || N <= 0 || !path_ok(path)) return ST_BAD_ARGS;
    if (path != PPML_B200_PATH_SIMT) {
        UmmaGemmArgs a{};
        a.A = A; a.B = B; a.C = C; a.M = M; a.N = N; a.K = K; a.batch = 1;
        a.lda = K; a.ldb = K; a.a_batch = 0; a.b_batch = 0; a.ldc = N; a.c_batch = 0;
        a.bias = bias; a.alpha = 1.0f; a.clamp = 0; a.opm_D = 0; a.opm_L = 0; a.elem = elem; a.tf32_mode = tf32_mode;
        const int rc = launch_umma_gemm(a, st);
        if (rc != ST_UNSUPPORTED_PATH || path == PPML_B200_PATH_UMMA) return rc;
    }
    SimtContract p{};
    p.M = M; p.N = N; p.K = K;
    p.a_sm = K; p.a_sk = 1; p.b_sn = K; p.b_sk = 1; p.c_sm = N; p.c_sn = 1;
    p.planes = 1; p.ne2 = 1; p.a_div2 = 1; p.a_div3 = 1;
    p.bias = bias; p.bias_seed = (elem == 0) ? 1 : 0; p.alpha = 1.0f;
    return launch_simt_contract(A, B, C, p, elem, st);
}

}  // namespace

extern "C" {

const char* ppml_b200_version(void) { return "ppml_b200 0.1 (sm_100a)"; }

int ppml_b200_hw_supported(int* out_major, int* out_minor) {
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) {
        cudaGetLastError();
        major = minor = 0;
    }
    if (out_major) *out_major = major;
    if (out_minor) *out_minor = minor;
    return major == 10 ? 1 : 0;
}

int ppml_b200_device_status(int* where) {
    if (where) *where = 0;
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return 100 + static_cast<int>(e);
    int* err = device_error_ptr();
    if (!err) return ST_LAUNCH;
    int h[2] = {0, 0};
    if (cudaMemcpy(h, err, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return ST_LAUNCH;
    if (h[0] != 0) {
        if (where) *where = h[1];
        cudaMemset(err, 0, 4 * sizeof(int));
    }
    return h[0];
}

int ppml_b200_mul_mat_f32(const float* A, const float* B, float* C, int M, int K, int N, const float* bias,
                          int path, int tf32_mode, void* stream) {
    if (tf32_mode < 0 || tf32_mode > 2) return ST_BAD_ARGS;
    return mul_mat_any(A, B, C, M, K, N, bias, path, 0, tf32_mode, as_stream(stream));
}

int ppml_b200_mul_mat_f16(const void* A16, const void* B16, float* C, int M, int K, int N, const float* bias,
                          int path, void* stream) {
    return mul_mat_any(A16, B16, C, M, K, N, bias, path, 1, 0, as_stream(stream));
}

int ppml_b200_mul_mat_bf16(const void* A16, const void* B16, float* C, int M, int K, int N, const float* bias,
                           int path, void* stream) {
    return mul_mat_any(A16, B16, C, M, K, N, bias, path, 2, 0, as_stream(stream));
}

int ppml_b200_cast_f32_to_f16(const float* x, void* y, int64_t n, void* stream) {
    return launch_cast(x, y, n, 0, as_stream(stream));
}
int ppml_b200_cast_f32_to_bf16(const float* x, void* y, int64_t n, void* stream) {
    return launch_cast(x, y, n, 1, as_stream(stream));
}

void ppml_b200_set_q8_two_pass(int mode) { g_q8_two_pass = mode < 0 ? -1 : (mode ? 1 : 0); }
int ppml_b200_q8_kernel_launches(int M, int N, int K) { return q8_two_pass(M, N, K) ? 2 : 1; }

int ppml_b200_mul_mat_q8(const void* W, const float* X, float* C, int M, int N, int K, int wtype, int c_trans,
                         const float* bias, int32_t* sumi_out, int path, int* path_out, void* stream) {
    if (path_out) *path_out = 0;
    if (!W || !X || !C || M <= 0 || N <= 0 || K <= 0 || !path_ok(path)) return ST_BAD_ARGS;
    if ((K % 32) != 0) return ST_BAD_K;
    if (wtype < 0 || wtype > 2) return ST_WTYPE;
    cudaStream_t st = as_stream(stream);
    if (path != PPML_B200_PATH_SIMT) {
        int rc = ST_UNSUPPORTED_PATH;
        if (wtype == 2) {
            // two-pass form (activations quantized by a kernel of their own into the shared scratch) or one-pass form
            void* scratch = nullptr;
            std::unique_lock<std::mutex> lock(g_scratch_mtx, std::defer_lock);
            if (q8_two_pass(M, N, K)) {
                lock.lock();
                scratch = ensure_scratch(umma_q8_scratch_bytes(N, K));
            }
            rc = launch_umma_q8(W, X, C, M, N, K, c_trans, bias, sumi_out, st, scratch);
        }
        if (rc == ST_OK && path_out) *path_out = 1;
        if (rc != ST_UNSUPPORTED_PATH || path == PPML_B200_PATH_UMMA) return rc;
    }
    const int nblk = K / 32;
    std::lock_guard<std::mutex> lock(g_scratch_mtx);
    void* qa = ensure_scratch(static_cast<size_t>(nblk) * static_cast<size_t>(N) * 36);
    if (!qa) return ST_SCRATCH;
    if (launch_quantize_q8_1(X, qa, static_cast<long long>(K) * N, st) != ST_OK) return ST_QUANT;
    return launch_q8_dp4a(W, qa, C, M, N, nblk, wtype, c_trans, bias, sumi_out, st);
}

int ppml_b200_quantize_rows_q8_1(const float* x, void* y, int64_t ne, void* stream) {
    return launch_quantize_q8_1(x, y, ne, as_stream(stream));
}
int ppml_b200_dequantize_q8_0(const void* x, float* y, int64_t ne, void* stream) {
    return launch_dequantize_q8(x, y, ne, 0, as_stream(stream));
}
int ppml_b200_dequantize_q8_1(const void* x, float* y, int64_t ne, void* stream) {
    return launch_dequantize_q8(x, y, ne, 1, as_stream(stream));
}
int ppml_b200_quantize_q8_0r(const float* w_dev, void* q8_0r_dev, int64_t ne, void* stream) {
    return launch_quantize_q8_0r(w_dev, q8_0r_dev, ne, as_stream(stream));
}
int64_t ppml_b200_q8_0r_bytes(int64_t numel) { return numel / 32 * 34; }

namespace {
// elem: 0 = fp32, 1 = bf16, 2 = fp16 Q/K/V
int flash_attn_any(const ppml_b200_flash_cfg* cfg, int Lk, int64_t bias_batch_stride, const void* Q, const void* K,
                   const void* V, int elem, const float* bias, float* O, float* LSE, int path, void* stream) {
    if (!cfg || !Q || !K || !V || !O || !path_ok(path)) return ST_BAD_ARGS;
    if (cfg->B <= 0 || cfg->h <= 0 || cfg->L <= 0 || cfg->d <= 0 || Lk <= 0) return ST_BAD_ARGS;
    const float scale = (cfg->scale > 0.f) ? cfg->scale : 1.0f / std::sqrt(static_cast<float>(cfg->d));
    if (path != PPML_B200_PATH_SIMT) {
        const int rc = launch_umma_attn(Q, K, V, elem, bias, O, LSE, cfg->B, cfg->h, cfg->L, Lk, cfg->d, cfg->causal ? 1 : 0,
                                        scale, cfg->softmax_eps, bias_batch_stride, as_stream(stream));
        if (rc != ST_UNSUPPORTED_PATH || path == PPML_B200_PATH_UMMA) return rc;
    }
    return launch_attn_rowwarp(Q, K, V, elem, bias, O, LSE, cfg->B, cfg->h, cfg->L, Lk, cfg->d, cfg->causal ? 1 : 0, scale,
                               cfg->softmax_eps, bias_batch_stride, as_stream(stream));
}
}  // namespace

int ppml_b200_flash_attn_forward_ex(const ppml_b200_flash_cfg* cfg, int Lk, int64_t bias_batch_stride,
                                    const float* Q, const float* K, const float* V, const float* bias,
                                    float* O, float* LSE, int path, void* stream) {
    return flash_attn_any(cfg, Lk, bias_batch_stride, Q, K, V, 0, bias, O, LSE, path, stream);
}

int ppml_b200_flash_attn_forward_16(const ppml_b200_flash_cfg* cfg, int Lk, int64_t bias_batch_stride,
                                    const void* Q16, const void* K16, const void* V16, const float* bias,
                                    float* O, float* LSE, int is_bf16, int path, void* stream) {
    return flash_attn_any(cfg, Lk, bias_batch_stride, Q16, K16, V16, is_bf16 ? 1 : 2, bias, O, LSE, path, stream);
}

int ppml_b200_flash_attn_forward(const ppml_b200_flash_cfg* cfg, const float* Q, const float* K, const float* V,
                                 const float* bias, float* O, float* LSE, int path, void* stream) {
    if (!cfg) return ST_BAD_ARGS;
    return ppml_b200_flash_attn_forward_ex(cfg, cfg->L, static_cast<int64_t>(cfg->h) * cfg->L * cfg->L, Q, K, V, bias,
                                           O, LSE, path, stream);
}

int ppml_b200_out_prod(const float* src0, const float* src1, float* dst,
                       int64_t ne00, int64_t ne01, int64_t ne02, int64_t ne03,
                       int64_t ne10, int64_t ne11, int64_t ne12, int64_t ne13,
                       int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3, int path, void* stream) {
    if (!src0 || !src1 || !dst || !path_ok(path)) return ST_BAD_ARGS;
    if (ne00 <= 0 || ne01 <= 0 || ne02 <= 0 || ne03 <= 0 || ne10 <= 0 || ne12 <= 0 || ne13 <= 0) return ST_BAD_ARGS;
    if (ne11 != ne01 || ne0 != ne00 || ne1 != ne10 || ne2 < ne02 || ne3 < ne03 || ne2 != ne12 || ne3 != ne13) return ST_BAD_ARGS;
    if (ne2 % ne02 || ne3 % ne03) return ST_BAD_ARGS;
    if (path != PPML_B200_PATH_SIMT) {
        int rc = ST_UNSUPPORTED_PATH;
        // dst[plane][i1][i0] = sum_k src1[plane][k][i1] * src0[plane][k][i0]: both operands have the row index
        // contiguous; planes without broadcast only
        if (ne02 == ne2 && ne03 == ne3 && ne2 * ne3 <= 0x7fffffff && ne00 <= 0x7fffffff && ne10 <= 0x7fffffff && ne01 <= 0x7fffffff) {
            UmmaGemmArgs a{};
            a.A = src1; a.B = src0; a.C = dst;
            a.M = static_cast<int>(ne10); a.N = static_cast<int>(ne00); a.K = static_cast<int>(ne01);
            a.batch = static_cast<int>(ne2 * ne3);
            a.lda = ne10; a.ldb = ne00; a.a_batch = ne10 * ne11; a.b_batch = ne00 * ne01;
            a.ldc = ne0; a.c_batch = ne0 * ne1; a.alpha = 1.0f; a.elem = 0; a.tf32_mode = PPML_B200_TF32_TMA; a.mn_major = 1;
            rc = launch_umma_gemm(a, as_stream(stream));
        }
        if (rc != ST_UNSUPPORTED_PATH || path == PPML_B200_PATH_UMMA) return rc;
    }
    SimtContract p{};
    p.M = ne00; p.N = ne10; p.K = ne01;
    p.a_sm = 1; p.a_sk = ne00; p.b_sn = 1; p.b_sk = ne10;
    p.c_sm = 1; p.c_sn = ne0;
    p.planes = ne2 * ne3; p.ne2 = ne2;
    p.a_s2 = ne00 * ne01; p.a_s3 = ne00 * ne01 * ne02; p.a_div2 = ne2 / ne02; p.a_div3 = ne3 / ne03;
    p.b_s2 = ne10 * ne11; p.b_s3 = ne10 * ne11 * ne12;
    p.c_s2 = ne0 * ne1; p.c_s3 = ne0 * ne1 * ne2;
    p.alpha = 1.0f;
    return launch_simt_contract(src0, src1, dst, p, 0, as_stream(stream));
}

static int tri_mul_any(const void* left, const void* right, float* dst, int64_t D, int64_t I, int64_t J,
                       int64_t K, int64_t B, float inv_L, int outgoing, int path, int elem, cudaStream_t st) {
    if (!left || !right || !dst || D <= 0 || I <= 0 || J <= 0 || K <= 0 || B <= 0 || !path_ok(path)) return ST_BAD_ARGS;
    if (path != PPML_B200_PATH_SIMT) {
        int rc = ST_UNSUPPORTED_PATH;
        if (B == 1 && D <= 0x7fffffff && I <= 0x7fffffff && J <= 0x7fffffff && K <= 0x7fffffff) {
            UmmaGemmArgs a{};
            a.A = left; a.B = right; a.C = dst;
            a.M = static_cast<int>(I); a.N = static_cast<int>(J); a.K = static_cast<int>(K); a.batch = static_cast<int>(D);
            if (outgoing) { a.lda = K; a.ldb = K; }                    // left[d][i][k], right[d][j][k]
            else { a.lda = I; a.ldb = J; a.mn_major = 1; }             // left[d][k][i], right[d][k][j]
            a.a_batch = I * K; a.b_batch = J * K; a.ldc = J; a.c_batch = I * J;
            a.bias = nullptr; a.alpha = inv_L; a.clamp = 1; a.elem = elem; a.tf32_mode = PPML_B200_TF32_TMA;
            rc = launch_umma_gemm(a, st);
        }
        if (rc != ST_UNSUPPORTED_PATH || path == PPML_B200_PATH_UMMA) return rc;
    }
    SimtContract p{};
    p.M = I; p.N = J; p.K = K;
    if (outgoing) { p.a_sm = K * B; p.a_sk = B; p.b_sn = K * B; p.b_sk = B; }
    else { p.a_sm = B; p.a_sk = I * B; p.b_sn = B; p.b_sk = J * B; }
    p.c_sm = J * B; p.c_sn = B;
    p.planes = D * B; p.ne2 = B;
    p.a_s2 = 1; p.a_s3 = I * K * B; p.a_div2 = 1; p.a_div3 = 1;
    p.b_s2 = 1; p.b_s3 = J * K * B; p.c_s2 = 1; p.c_s3 = I * J * B;
    p.alpha = inv_L; p.clamp = 1;
    return launch_simt_contract(left, right, dst, p, elem, st);
}

int ppml_b200_tri_mul(const float* left, const float* right, float* dst, int64_t D, int64_t I, int64_t J,
                      int64_t K, int64_t B, float inv_L, int outgoing, int path, void* stream) {
    return tri_mul_any(left, right, dst, D, I, J, K, B, inv_L, outgoing, path, 0, as_stream(stream));
}

int ppml_b200_tri_mul_16(const void* left16, const void* right16, float* dst, int64_t D, int64_t I, int64_t J,
                         int64_t K, int64_t B, float inv_L, int outgoing, int is_bf16, int path, void* stream) {
    return tri_mul_any(left16, right16, dst, D, I, J, K, B, inv_L, outgoing, path, is_bf16 ? 2 : 1, as_stream(stream));
}

// D1 slabs of `left` against all D slabs of `right` (D1 == D for the whole op; D1 < D for one rank's d1 range)
static int outer_prod_mean_any(const void* left, const void* right, float* dst, int64_t D1, int64_t D, int64_t L,
                               int64_t N, int64_t B, float inv_N, int path, int elem, cudaStream_t st) {
    if (!left || !right || !dst || D1 <= 0 || D <= 0 || L <= 0 || N <= 0 || B <= 0 || !path_ok(path)) return ST_BAD_ARGS;
    if (path != PPML_B200_PATH_SIMT) {
        int rc = ST_UNSUPPORTED_PATH;
        if (B == 1 && D * L <= 0x7fffffff && D1 * L <= 0x7fffffff && N <= 0x7fffffff) {
            UmmaGemmArgs a{};
            a.A = left; a.B = right; a.C = dst;
            a.M = static_cast<int>(D1 * L); a.N = static_cast<int>(D * L); a.K = static_cast<int>(N); a.batch = 1;
            a.lda = N; a.ldb = N; a.ldc = D * L; a.alpha = inv_N;
            a.opm_D = static_cast<int>(D); a.opm_L = static_cast<int>(L); a.elem = elem; a.tf32_mode = PPML_B200_TF32_TMA;
            rc = launch_umma_gemm(a, st);
        }
        if (rc != ST_UNSUPPORTED_PATH || path == PPML_B200_PATH_UMMA) return rc;
    }
    SimtContract p{};
    p.M = D1 * L; p.N = D * L; p.K = N;
    p.a_sm = N * B; p.a_sk = B; p.b_sn = N * B; p.b_sk = B;
    p.planes = B; p.ne2 = B;
    p.a_s2 = 1; p.a_div2 = 1; p.a_div3 = 1; p.b_s2 = 1; p.c_s2 = 1;
    p.alpha = inv_N;
    p.opm_D = D; p.opm_L = L; p.opm_B = B;
    return launch_simt_contract(left, right, dst, p, elem, st);
}

int ppml_b200_outer_prod_mean(const float* left, const float* right, float* dst, int64_t D, int64_t L,
                              int64_t N, int64_t B, float inv_N, int path, void* stream) {
    return outer_prod_mean_any(left, right, dst, D, D, L, N, B, inv_N, path, 0, as_stream(stream));
}

int ppml_b200_outer_prod_mean_16(const void* left16, const void* right16, float* dst, int64_t D, int64_t L,
                                 int64_t N, int64_t B, float inv_N, int is_bf16, int path, void* stream) {
    return outer_prod_mean_any(left16, right16, dst, D, D, L, N, B, inv_N, path, is_bf16 ? 2 : 1, as_stream(stream));
}

int ppml_b200_outer_prod_mean_slabs(const float* left, const float* right, float* dst, int64_t D_left, int64_t D,
                                    int64_t L, int64_t N, int64_t B, float inv_N, int path, void* stream) {
    return outer_prod_mean_any(left, right, dst, D_left, D, L, N, B, inv_N, path, 0, as_stream(stream));
}

// ---------------------------------------------------------------------------------------------
// per-shape statistics (PPML_MULMAT_STATS=1)
// ---------------------------------------------------------------------------------------------
namespace {
struct StatRec { int M, K, N; cudaEvent_t e0, e1; std::string path; bool closed; };
std::vector<StatRec> g_stat_open;
std::mutex g_stat_mtx;
bool stats_enabled() {
    static const bool on = [] { const char* e = std::getenv("PPML_MULMAT_STATS"); return e && e[0] == '1'; }();
    return on;
}
}  // namespace

void ppml_b200_mulmat_stats_begin(int M, int K, int N) {
    if (!stats_enabled()) return;
    std::lock_guard<std::mutex> lock(g_stat_mtx);
    StatRec r{M, K, N, nullptr, nullptr, "", false};
    if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) { cudaGetLastError(); return; }
    cudaEventRecord(r.e0, 0);
    g_stat_open.push_back(r);
}

void ppml_b200_mulmat_stats_end(const char* path) {
    if (!stats_enabled()) return;
    std::lock_guard<std::mutex> lock(g_stat_mtx);
    for (auto it = g_stat_open.rbegin(); it != g_stat_open.rend(); ++it) {
        if (!it->closed) { cudaEventRecord(it->e1, 0); it->path = path ? path : "?"; it->closed = true; break; }
    }
}

int ppml_b200_mulmat_stats_dump(char* buf, int cap) {
    if (!buf || cap <= 0) return 0;
    buf[0] = 0;
    if (!stats_enabled()) return 0;
    std::lock_guard<std::mutex> lock(g_stat_mtx);
    cudaDeviceSynchronize();
    std::map<std::tuple<std::string, int, int, int>, std::pair<long long, double>> agg;
    for (auto& r : g_stat_open) {
        if (!r.closed) continue;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.e0, r.e1) != cudaSuccess) { cudaGetLastError(); ms = 0.f; }
        auto& a = agg[std::make_tuple(r.path, r.M, r.K, r.N)];
        a.first += 1; a.second += ms;
        cudaEventDestroy(r.e0); cudaEventDestroy(r.e1);
    }
    g_stat_open.clear();
    int off = 0;
    for (auto& kv : agg) {
        const int n = std::snprintf(buf + off, static_cast<size_t>(cap - off), "%s M=%d K=%d N=%d calls=%lld ms=%.4f\n",
                                    std::get<0>(kv.first).c_str(), std::get<1>(kv.first), std::get<2>(kv.first),
                                    std::get<3>(kv.first), kv.second.first, kv.second.second);
        if (n < 0 || n >= cap - off) break;
        off += n;
    }
    return off;
}

}  // extern "C"
