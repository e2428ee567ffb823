// ppml_forwarders.cpp -- the host launchers of the reference's hot path under their original C++
// names and signatures (namespace ppml), each forwarding to the C ABI of this library.  The
// reference declares these as `extern` free functions inside namespace ppml
// (src/backend/CUDAKernels.cpp:97-345) and CUDABackend::dispatch_node calls them; linking the
// reference's backend against libppml_b200.so instead of its own src/cuda objects for these symbols
// is the whole integration.  All launches go to the legacy default stream, as the reference's do.
//
// Arithmetic of the fp32 entries.  In the reference mul_mat_cuda, out_prod_cuda, tri_mul_cuda and
// outer_prod_mean_cuda and flash_attn_forward_cuda are exact-fp32 CUDA-core kernels; tf32 tensor cores are opt-in through PPML_MUL_MAT_TC, and
// only for nodes without a bias (src/backend/CUDAKernels.cpp:822-842).  The forwarders keep that default: with
// nothing set they run this library's CUDA-core kernels (fp32 accumulation in the reference's order).  The tensor
// cores are switched on by the reference's own variable or by this library's:
//   PPML_MUL_MAT_TC=<not 0>   tf32 tensor cores for every fp32 entry (attention included: tf32 products, fp32
//                             softmax), bias included (the epilogue adds it in fp32)
//   PPML_B200_MATH=fp32|tf32|bf16   same choice spelled out; bf16 = bf16 products behind the fp32 tensors
//                             (ppml_b200_mul_mat_f32_as_bf16; the batched ops stay tf32); overrides PPML_MUL_MAT_TC
// mul_mat_mma_tf32_smem is tf32 by contract and ignores the switch.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/ppml_b200.h"

namespace ppml {

// Layout twins of the reference's types (only what the signatures need).
struct block_q8_0;                          // include/ppml/QuantBlocks.h:33
struct block_q8_1;                          // include/ppml/QuantBlocks.h:38
struct FlashAttnConfig {                    // include/ppml/FlashAttn.h:26-36
    int B = 1;
    int h = 1;
    int L = 0;
    int d = 0;
    bool causal = true;
    float scale = 0.f;
    float softmax_eps = 1e-9f;
    int Br = 64;
    int Bc = 64;
};

namespace {
enum { kMathFp32 = 0, kMathTf32 = 1, kMathBf16 = 2 };
// Read on every call (two getenv look-ups beside a kernel launch), so that one process can switch.
int math_mode() {
    if (const char* m = std::getenv("PPML_B200_MATH")) {
        if (!std::strcmp(m, "bf16")) return kMathBf16;
        if (!std::strcmp(m, "tf32")) return kMathTf32;
        if (!std::strcmp(m, "fp32")) return kMathFp32;
        static bool warned = false;
        if (!warned) std::fprintf(stderr, "[ppml_b200] PPML_B200_MATH=%s not understood (fp32, tf32, bf16): using fp32\n", m);
        warned = true;
        return kMathFp32;
    }
    const char* e = std::getenv("PPML_MUL_MAT_TC");        // parsed as the reference parses it
    return (e && e[0] && e[0] != '0') ? kMathTf32 : kMathFp32;
}
// kernel family of the batched fp32 entries under the current switch
int batched_path() { return math_mode() == kMathFp32 ? PPML_B200_PATH_SIMT : PPML_B200_PATH_AUTO; }
}  // namespace

// src/backend/CUDAKernels.cpp:158 -- no status in the signature: a failure is reported on stderr,
// like the reference's wrappers report theirs.
void mul_mat_cuda(float* A, float* B, float* C, int M, int K, int N, const float* bias) {
    int rc;
    switch (math_mode()) {
        case kMathBf16: rc = ppml_b200_mul_mat_f32_as_bf16(A, B, C, M, K, N, bias, PPML_B200_PATH_AUTO, nullptr); break;
        case kMathTf32: rc = ppml_b200_mul_mat_f32(A, B, C, M, K, N, bias, PPML_B200_PATH_AUTO, PPML_B200_TF32_TMA, nullptr); break;
        default: rc = ppml_b200_mul_mat_f32(A, B, C, M, K, N, bias, PPML_B200_PATH_SIMT, PPML_B200_TF32_TMA, nullptr); break;
    }
    if (rc != 0) std::fprintf(stderr, "[ppml_b200] mul_mat_cuda failed rc=%d (M=%d K=%d N=%d)\n", rc, M, K, N);
}

// src/backend/CUDAKernels.cpp:187 -- 0 = launched, 1 = unsupported (caller falls back to mul_mat_cuda)
int mul_mat_mma_tf32_smem(const void* A, const void* B, float* C, int M, int K, int N) {
    const int rc = ppml_b200_mul_mat_f32(static_cast<const float*>(A), static_cast<const float*>(B), C, M, K, N, nullptr,
                                         PPML_B200_PATH_UMMA, PPML_B200_TF32_TMA, nullptr);
    return rc == 0 ? 0 : 1;
}

// src/backend/CUDAKernels.cpp:199, :195, :182
int mul_mat_mma_f16_smem(const void* A, const void* B, float* C, int M, int K, int N) {
    return ppml_b200_mul_mat_f16(A, B, C, M, K, N, nullptr, PPML_B200_PATH_UMMA, nullptr) == 0 ? 0 : 1;
}
int mul_mat_mma_f16(const void* A, const void* B, float* C, int M, int K, int N) {
    return ppml_b200_mul_mat_f16(A, B, C, M, K, N, nullptr, PPML_B200_PATH_AUTO, nullptr) == 0 ? 0 : 1;
}
void mul_mat_cuda_f16(const void* A, const void* B, float* C, int M, int K, int N) {
    const int rc = ppml_b200_mul_mat_f16(A, B, C, M, K, N, nullptr, PPML_B200_PATH_SIMT, nullptr);
    if (rc != 0) std::fprintf(stderr, "[ppml_b200] mul_mat_cuda_f16 failed rc=%d\n", rc);
}

// src/backend/CUDAKernels.cpp:169
int mul_mat_q8_cuda(const void* W, const float* X, float* C, int M, int N, int K, int wtype, int c_trans,
                    int* path_out) {
    return ppml_b200_mul_mat_q8(W, X, C, M, N, K, wtype, c_trans, nullptr, nullptr, PPML_B200_PATH_AUTO, path_out, nullptr);
}
// Q8 with the bias epilogue the reference lacks (its wrapper skips biased quantized nodes,
// src/backend/CUDAKernels.cpp:741-744); for a caller that relaxes that gate.
int mul_mat_q8_cuda_bias(const void* W, const float* X, float* C, int M, int N, int K, int wtype, int c_trans,
                         const float* bias, int* path_out) {
    return ppml_b200_mul_mat_q8(W, X, C, M, N, K, wtype, c_trans, bias, nullptr, PPML_B200_PATH_AUTO, path_out, nullptr);
}

// src/backend/CUDAKernels.cpp:164-166
int quantize_rows_q8_1_cuda(const float* x, block_q8_1* y, int64_t ne, cudaStream_t stream) {
    return ppml_b200_quantize_rows_q8_1(x, y, ne, stream) == 0 ? 0 : 1;
}
int dequantize_q8_0_cuda(const block_q8_0* x, float* y, int64_t ne, cudaStream_t stream) {
    return ppml_b200_dequantize_q8_0(x, y, ne, stream) == 0 ? 0 : 1;
}
int dequantize_q8_1_cuda(const block_q8_1* x, float* y, int64_t ne, cudaStream_t stream) {
    return ppml_b200_dequantize_q8_1(x, y, ne, stream) == 0 ? 0 : 1;
}

// src/backend/CUDAKernels.cpp:174 -- 0 = launched, 1 = unsupported
int flash_attn_forward_cuda(const FlashAttnConfig& cfg, const float* Q, const float* K, const float* V,
                            const float* bias, float* O, float* LSE) {
    ppml_b200_flash_cfg c;
    c.B = cfg.B; c.h = cfg.h; c.L = cfg.L; c.d = cfg.d; c.causal = cfg.causal ? 1 : 0;
    c.scale = cfg.scale; c.softmax_eps = cfg.softmax_eps; c.Br = cfg.Br; c.Bc = cfg.Bc;
    return ppml_b200_flash_attn_forward(&c, Q, K, V, bias, O, LSE, batched_path(), nullptr) == 0 ? 0 : 1;
}

// src/backend/CUDAKernels.cpp:176 -- 0 = done, 1 = unsupported (the caller then falls back to the CPU routine)
int flash_attn_backward_cuda(const FlashAttnConfig& cfg, const float* Q, const float* K, const float* V,
                             const float* bias, const float* O, const float* dO, const float* LSE,
                             float* dQ, float* dK, float* dV, float* dbias) {
    ppml_b200_flash_cfg c;
    c.B = cfg.B; c.h = cfg.h; c.L = cfg.L; c.d = cfg.d; c.causal = cfg.causal ? 1 : 0;
    c.scale = cfg.scale; c.softmax_eps = cfg.softmax_eps; c.Br = cfg.Br; c.Bc = cfg.Bc;
    return ppml_b200_flash_attn_backward(&c, static_cast<int64_t>(cfg.h) * cfg.L * cfg.L, Q, K, V, bias, O, dO, LSE,
                                         dQ, dK, dV, dbias, nullptr) == 0 ? 0 : 1;
}

// src/backend/CUDAKernels.cpp:201
void out_prod_cuda(const float* src0, const float* src1, float* dst,
                   int64_t ne00, int64_t ne01, int64_t ne02, int64_t ne03,
                   int64_t ne10, int64_t ne11, int64_t ne12, int64_t ne13,
                   int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3) {
    const int rc = ppml_b200_out_prod(src0, src1, dst, ne00, ne01, ne02, ne03, ne10, ne11, ne12, ne13, ne0, ne1, ne2, ne3,
                                      batched_path(), nullptr);
    if (rc != 0) std::fprintf(stderr, "[ppml_b200] out_prod_cuda failed rc=%d\n", rc);
}

// src/backend/CUDAKernels.cpp:316
void tri_mul_cuda(const float* left, const float* right, float* dst, int64_t D, int64_t I, int64_t J, int64_t K,
                  int64_t B, float inv_L, int outgoing) {
    const int rc = ppml_b200_tri_mul(left, right, dst, D, I, J, K, B, inv_L, outgoing, batched_path(), nullptr);
    if (rc != 0) std::fprintf(stderr, "[ppml_b200] tri_mul_cuda failed rc=%d\n", rc);
}

// src/backend/CUDAKernels.cpp:325
void outer_prod_mean_cuda(const float* left, const float* right, float* dst, int64_t D, int64_t L, int64_t N,
                          int64_t B, float inv_N) {
    const int rc = ppml_b200_outer_prod_mean(left, right, dst, D, L, N, B, inv_N, batched_path(), nullptr);
    if (rc != 0) std::fprintf(stderr, "[ppml_b200] outer_prod_mean_cuda failed rc=%d\n", rc);
}

// src/backend/CUDAKernels.cpp:190-191, :147
void mulmat_stats_cuda_begin(int M, int K, int N) { ppml_b200_mulmat_stats_begin(M, K, N); }
void mulmat_stats_cuda_end(const char* path) { ppml_b200_mulmat_stats_end(path); }
bool cutlass_hw_supported(int* out_major, int* out_minor) { return ppml_b200_hw_supported(out_major, out_minor) != 0; }

}  // namespace ppml
