// kernels.h -- internal launcher interface between the C-ABI layer (capi.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace ppml_b200 {

// Strided batched contraction on CUDA cores (simt_kernels.cu).
//   D[plane][m][n] = epi( sum_k A[..][m*a_sm + k*a_sk] * B[..][n*b_sn + k*b_sk] )
// plane = i3*ne2 + i2; A's plane is (i2 / a_div2, i3 / a_div3) (broadcast as the reference's CPU
// out_prod does, src/backend/CPUKernels.cpp:836-858).
struct SimtContract {
    long long M, N, K;
    long long a_sm, a_sk, b_sn, b_sk;
    long long c_sm, c_sn;
    long long planes, ne2;
    long long a_s2, a_s3, a_div2, a_div3;
    long long b_s2, b_s3, c_s2, c_s3;
    const float* bias;
    int bias_seed;              // 1: accumulator starts at bias[n] (fp32 mul_mat); 0: added at the end
    float alpha;
    int clamp;                  // NaN -> 0, clamp to +-1e4
    long long opm_D, opm_L, opm_B;   // opm_L > 0: blocked outer-product-mean store
    // fused neighbours of a Linear (see GemmParams in umma_gemm.cuh); plain mul_mat only
    const float* ln_stats; const float* ln_u; const float* gate; int act;
};
int launch_simt_contract(const void* A, const void* B, float* C, const SimtContract& p, int elem /*0 f32,1 f16,2 bf16*/,
                         cudaStream_t st);

// per row of x [M][K]: (mean, 1 / sqrt(var + eps)) with the reference's two-pass variance (src/backend/CPUKernels.cpp:1498-1511)
int launch_row_stats(const float* x, float* mean_rstd, long long M, int K, float eps, cudaStream_t st);
// Wg[n][k] = W[n][k] * gamma[k], u[n] = sum_k Wg[n][k], v[n] = sum_k W[n][k] * beta[k] + bias[n]
int launch_ln_fold(const float* W, const float* gamma, const float* beta, const float* bias, float* Wg, float* u, float* v, int N, int K,
                   cudaStream_t st);
int launch_cast(const float* x, void* y, long long n, int to_bf16, cudaStream_t st);
int launch_quantize_q8_1(const float* x, void* y, long long ne, cudaStream_t st);
int launch_quantize_q8_0r(const float* w, void* out, long long ne, cudaStream_t st);
int launch_repack_q8_0(const void* blocks34, long long nblocks, void* q8_0r, cudaStream_t st);
int launch_dequantize_q8(const void* x, float* y, long long ne, int kind, cudaStream_t st);
// Q8 product with at most 16 output columns in one pass on CUDA cores (planar weights, C[token][M]); ST_UNSUPPORTED_PATH otherwise
int launch_q8_skinny(const void* W, const float* X, float* C, int M, int N, int K, int c_trans, const float* bias,
                     int* sumi_out, cudaStream_t st);
int launch_q8_dp4a(const void* W, const void* acts, float* C, int M, int N, int nblk, int wtype, int c_trans,
                   const float* bias, int* sumi_out, cudaStream_t st);
// elem: 0 = fp32 Q/K/V, 1 = bf16, 2 = fp16; bias, O and LSE are fp32
// Where the attention operands live.  Element (b, h, i, dd) of Q is at Q[b * q_b + h * q_h + i * q_l + dd] (K, V, O alike;
// the head dim is always contiguous).  flash(): the fused op's own layout [B][h][L][d] (include/ppml/FlashAttn.h:24-32);
// tokens(): the layout of the Linear that produced the operand, [B][L][ld] with head h in columns [h * d, (h + 1) * d) --
// what the reference only reaches through its permute copies (src/core/ComputeGraphHelper.cpp:455-483).
// gate (optional, strides g_*): O = act(gate) * O, the OP_ACT_MUL node behind every attention of the model
// (src/modules/Attention.cpp:390).
struct AttnLayout {
    long long q_b, q_h, q_l, k_b, k_h, k_l, v_b, v_h, v_l, o_b, o_h, o_l, g_b, g_h, g_l;
    const float* gate; int act;
    static AttnLayout flash(int H, int L, int Lk, int d) {
        AttnLayout a{};
        a.q_l = a.k_l = a.v_l = a.o_l = d;
        a.q_h = a.o_h = static_cast<long long>(L) * d; a.k_h = a.v_h = static_cast<long long>(Lk) * d;
        a.q_b = a.o_b = a.q_h * H; a.k_b = a.v_b = a.k_h * H;
        a.g_b = a.o_b; a.g_h = a.o_h; a.g_l = a.o_l;
        a.gate = nullptr; a.act = 0;
        return a;
    }
};
// ft: keys of the reference's first softmax tile (its Bc); a row whose first ft scores are all -inf gives O = 0, LSE = -inf
// as the reference's CPU kernel does; 0 switches that off
// Flash-attention backward, exact fp32 on CUDA cores (attn_backward.cu): Q, K, V, O, dO, dQ, dK, dV [B, h, L, d];
// bias [.., h, L, L] with a batch stride (0: shared); dbias [B, h, L, L]; LSE [B, h, L]; null outputs are skipped.
int launch_attn_backward(int B, int H, int L, int d, int causal, float scale, const float* Q, const float* K, const float* V,
                         const float* bias, long long bias_batch_stride, const float* O, const float* dO, const float* LSE,
                         float* dQ, float* dK, float* dV, float* dbias, cudaStream_t st);
// head dim 8, fp32 operands with 16-byte aligned K / V rows, at least 16 query rows: warp-level tensor-core kernel (tf32
// products); ST_UNSUPPORTED_PATH otherwise
int launch_attn_d8_mma(const float* Q, const float* K, const float* V, const float* bias, float* O, float* LSE, int B, int H,
                       int L, int Lk, int d, int causal, float scale, float eps, long long bias_batch_stride, int ft,
                       const AttnLayout& lay, cudaStream_t st);
int launch_attn_rowwarp(const void* Q, const void* K, const void* V, int elem, const float* bias, float* O, float* LSE,
                        int B, int H, int L, int Lk, int d, int causal, float scale, float eps,
                        long long bias_batch_stride, int ft, const AttnLayout& lay, cudaStream_t st);

// tcgen05 paths (umma_gemm.cu / umma_q8.cu / umma_attn.cu).  Each returns ST_UNSUPPORTED_PATH when the
// shape or the alignment rules it out, so that the caller can take the CUDA-core kernel.
struct UmmaGemmArgs {
    const void* A; const void* B; float* C;
    int M, N, K, batch;
    long long lda, ldb;                // row strides (elements)
    long long a_batch, b_batch;        // batch strides (elements)
    long long ldc, c_batch;
    const float* bias; float alpha; int clamp;
    int opm_D, opm_L;                  // opm_L > 0: blocked outer-product-mean store
    int elem;                          // 0 fp32 (tf32 math), 1 fp16, 2 bf16
    int tf32_mode;                     // fp32 only: 0 round in smem (rna), 1 TMA tf32 type, 2 truncate
    int mn_major;                      // 1: A[b][k][m], B[b][k][n] (row index contiguous; lda / ldb = k pitch), fp32 only
    const float* ln_stats; const float* ln_u; const float* gate; int act;      // fused LayerNorm algebra / activation gate
};
int launch_umma_gemm(const UmmaGemmArgs& a, cudaStream_t st);

int launch_umma_q8(const void* W, const float* X, float* C, int M, int N, int K, int c_trans, const float* bias,
                   int* sumi_out, cudaStream_t st, void* scratch = nullptr);
size_t umma_q8_scratch_bytes(int N, int K);

int launch_umma_attn(const void* Q, const void* K, const void* V, int elem, const float* bias, float* O, float* LSE,
                     int B, int H, int L, int Lk, int d, int causal, float scale, float eps,
                     long long bias_batch_stride, int ft, const AttnLayout& lay, cudaStream_t st);

int num_sms();

}  // namespace ppml_b200
