// forwarder_harness.cpp -- calls the drop-in library exactly the way the reference's dispatcher does.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit includes the reference's own headers
// (include/ppml/FlashAttn.h for FlashAttnConfig, include/ppml/QuantBlocks.h for the block types) and
// declares the hot-path launchers word for word as src/backend/CUDAKernels.cpp:147-201 and :316-325
// declare them (`extern` free functions in namespace ppml, default argument included).  It defines
// none of them: the linker resolves every one against libppml_b200.so, which is the whole claim of
// the drop-in -- same mangled names, same parameter types, same struct layout.  Each fh_* function
// below is a plain C entry that a test calls through ctypes with device pointers; it holds no
// arithmetic of its own.
//
// Built by oracle/Makefile (`make drop_in`) where the reference tree is present; the result,
// oracle/_ref/libforwarder_harness.so, looks for libppml_b200.so relative to itself.
#include <cuda_runtime.h>

#include <cstdint>

#include "ppml/FlashAttn.h"
#include "ppml/QuantBlocks.h"

namespace ppml {
// ---- as declared in src/backend/CUDAKernels.cpp ------------------------------------------------------------------
extern bool cutlass_hw_supported(int* out_major, int* out_minor);                                              // :147
extern void mul_mat_cuda(float* A, float* B, float* C, int M, int K, int N, const float* bias = nullptr);      // :158
extern int quantize_rows_q8_1_cuda(const float* x, block_q8_1* y, int64_t ne, cudaStream_t stream);            // :164
extern int dequantize_q8_0_cuda(const block_q8_0* x, float* y, int64_t ne, cudaStream_t stream);               // :165
extern int dequantize_q8_1_cuda(const block_q8_1* x, float* y, int64_t ne, cudaStream_t stream);               // :166
extern int mul_mat_q8_cuda(const void* W, const float* X, float* C, int M, int N, int K, int wtype, int c_trans,
                           int* path_out);                                                                     // :169
extern int flash_attn_forward_cuda(const FlashAttnConfig& cfg, const float* Q, const float* K, const float* V,
                                   const float* bias, float* O, float* LSE);                                   // :174
extern int flash_attn_backward_cuda(const FlashAttnConfig& cfg, const float* Q, const float* K, const float* V,
                                    const float* bias, const float* O, const float* dO, const float* LSE,
                                    float* dQ, float* dK, float* dV, float* dbias);                              // :176
extern void mul_mat_cuda_f16(const void* A, const void* B, float* C, int M, int K, int N);                     // :182
extern int mul_mat_mma_tf32_smem(const void* A, const void* B, float* C, int M, int K, int N);                 // :187
extern void mulmat_stats_cuda_begin(int M, int K, int N);                                                      // :190
extern void mulmat_stats_cuda_end(const char* path);                                                           // :191
extern int mul_mat_mma_f16(const void* A, const void* B, float* C, int M, int K, int N);                       // :195
extern int mul_mat_mma_f16_smem(const void* A, const void* B, float* C, int M, int K, int N);                  // :199
extern void out_prod_cuda(const float* src0, const float* src1, float* dst,
                          int64_t ne00, int64_t ne01, int64_t ne02, int64_t ne03,
                          int64_t ne10, int64_t ne11, int64_t ne12, int64_t ne13,
                          int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3);                                 // :201
extern void tri_mul_cuda(const float* left, const float* right, float* dst, int64_t D, int64_t I, int64_t J,
                         int64_t K, int64_t B, float inv_L, int outgoing);                                     // :316
extern void outer_prod_mean_cuda(const float* left, const float* right, float* dst, int64_t D, int64_t L,
                                 int64_t N, int64_t B, float inv_N);                                           // :325
// ---- the extension for callers that relax the "bias + quantized operand" gate (src/backend/CUDAKernels.cpp:741-744)
extern int mul_mat_q8_cuda_bias(const void* W, const float* X, float* C, int M, int N, int K, int wtype, int c_trans,
                                const float* bias, int* path_out);
}  // namespace ppml

using namespace ppml;

extern "C" {

int fh_hw_supported(int* major, int* minor) { return cutlass_hw_supported(major, minor) ? 1 : 0; }

void fh_mul_mat_cuda(float* A, float* B, float* C, int M, int K, int N, const float* bias) {
    if (bias) mul_mat_cuda(A, B, C, M, K, N, bias);
    else mul_mat_cuda(A, B, C, M, K, N);                  // the default argument, as the wrapper's bias-less call site
}
int fh_mul_mat_mma_tf32_smem(const void* A, const void* B, float* C, int M, int K, int N) {
    return mul_mat_mma_tf32_smem(A, B, C, M, K, N);
}
// which: 0 = mul_mat_mma_f16_smem, 1 = mul_mat_mma_f16, 2 = mul_mat_cuda_f16
int fh_mul_mat_f16(int which, const void* A, const void* B, float* C, int M, int K, int N) {
    if (which == 0) return mul_mat_mma_f16_smem(A, B, C, M, K, N);
    if (which == 1) return mul_mat_mma_f16(A, B, C, M, K, N);
    mul_mat_cuda_f16(A, B, C, M, K, N);
    return 0;
}
int fh_mul_mat_q8_cuda(const void* W, const float* X, float* C, int M, int N, int K, int wtype, int c_trans,
                       const float* bias, int* path_out) {
    mulmat_stats_cuda_begin(M, K, N);
    const int rc = bias ? mul_mat_q8_cuda_bias(W, X, C, M, N, K, wtype, c_trans, bias, path_out)
                        : mul_mat_q8_cuda(W, X, C, M, N, K, wtype, c_trans, path_out);
    mulmat_stats_cuda_end(rc == 0 ? "q8" : "q8-failed");
    return rc;
}
int fh_quantize_rows_q8_1(const float* x, void* y, int64_t ne) {
    return quantize_rows_q8_1_cuda(x, static_cast<block_q8_1*>(y), ne, nullptr);
}
int fh_dequantize_q8(int kind, const void* x, float* y, int64_t ne) {
    return kind == 0 ? dequantize_q8_0_cuda(static_cast<const block_q8_0*>(x), y, ne, nullptr)
                     : dequantize_q8_1_cuda(static_cast<const block_q8_1*>(x), y, ne, nullptr);
}
// The config is built here from the reference's own struct definition and passed by const reference.
int fh_flash_attn_forward(int B, int h, int L, int d, int causal, float scale, float eps, const float* Q,
                          const float* K, const float* V, const float* bias, float* O, float* LSE) {
    FlashAttnConfig cfg;
    cfg.B = B; cfg.h = h; cfg.L = L; cfg.d = d; cfg.causal = causal != 0; cfg.scale = scale; cfg.softmax_eps = eps;
    return flash_attn_forward_cuda(cfg, Q, K, V, bias, O, LSE);
}
int fh_flash_attn_backward(int B, int h, int L, int d, int causal, float scale, const float* Q, const float* K, const float* V,
                           const float* bias, const float* O, const float* dO, const float* LSE,
                           float* dQ, float* dK, float* dV, float* dbias) {
    FlashAttnConfig cfg;
    cfg.B = B; cfg.h = h; cfg.L = L; cfg.d = d; cfg.causal = causal != 0; cfg.scale = scale;
    return flash_attn_backward_cuda(cfg, Q, K, V, bias, O, dO, LSE, dQ, dK, dV, dbias);
}
int fh_sizeof_flash_cfg(void) { return static_cast<int>(sizeof(FlashAttnConfig)); }
void fh_out_prod(const float* s0, const float* s1, float* dst, const int64_t* ne0x, const int64_t* ne1x, const int64_t* nex) {
    out_prod_cuda(s0, s1, dst, ne0x[0], ne0x[1], ne0x[2], ne0x[3], ne1x[0], ne1x[1], ne1x[2], ne1x[3],
                  nex[0], nex[1], nex[2], nex[3]);
}
void fh_tri_mul(const float* left, const float* right, float* dst, int64_t D, int64_t I, int64_t J, int64_t K,
                int64_t B, float inv_L, int outgoing) {
    tri_mul_cuda(left, right, dst, D, I, J, K, B, inv_L, outgoing);
}
void fh_outer_prod_mean(const float* left, const float* right, float* dst, int64_t D, int64_t L, int64_t N, int64_t B,
                        float inv_N) {
    outer_prod_mean_cuda(left, right, dst, D, L, N, B, inv_N);
}

}  // extern "C"
