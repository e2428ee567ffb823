/*
 * ppml_b200.h -- C ABI of libppml_b200.so: the dense-contraction path of the PPML graph executor,
 * written for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes, launches asynchronously on the given
 * stream (stream = NULL: the legacy default stream, which is what the reference's CUDABackend
 * uses) and returns a status code: 0 = launched; 1 = bad arguments / unsupported; 2 = K not a
 * multiple of 32 (Q8); 3 = scratch allocation failed; 4 = quantize launch failed; 5 = unknown
 * weight type; 6 = kernel launch failed; 7 = the requested kernel family cannot take this shape;
 * 9 = the problem exceeds a fixed capacity (only ppml_b200_mul_mat_q8_noalloc).
 * Buffers stay owned by the caller; nothing is retained after the call returns.
 *
 * Each declaration names the reference interface it stands in for (path inside the reference
 * project : line).  The C++ symbols with the reference's own names and signatures (namespace
 * ppml), which its src/backend/CUDAKernels.cpp binds at link time, are thin forwarders to these
 * (csrc/ppml_forwarders.cpp).
 *
 * Matrix conventions follow the reference: A is [M][K] row-major, B is [N][K] row-major (already
 * "transposed"), C is [M][N] row-major, C[m][n] = bias[n] + sum_k A[m][k] * B[n][k].
 */
#ifndef PPML_B200_H
#define PPML_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* kernel family selectors ("path" arguments) */
#define PPML_B200_PATH_AUTO 0   /* tensor cores when the shape allows, else CUDA cores */
#define PPML_B200_PATH_SIMT 1   /* CUDA cores only (exact fp32 accumulation order)      */
#define PPML_B200_PATH_UMMA 2   /* tcgen05 only; status 7 when the shape is not eligible */

/* how fp32 operands become tf32 on the tensor-core path */
#define PPML_B200_TF32_ROUND 0      /* round to nearest in shared memory (cvt.rna), as the reference's tf32 kernel */
#define PPML_B200_TF32_TMA 1        /* let the TMA unit deliver tf32 */
#define PPML_B200_TF32_TRUNCATE 2   /* feed fp32 words unchanged; the tensor core drops the low mantissa bits */

const char* ppml_b200_version(void);

/* Replaces cutlass_hw_supported (src/backend/CUDAKernels.cpp:147): 1 when the current device is
 * compute capability 10.x; major/minor may be NULL. */
int ppml_b200_hw_supported(int* out_major, int* out_minor);

/* Synchronizes the device and returns 0, or the code a kernel left in the device error word when one
 * of its bounded waits ran out (8); `where` (may be NULL) receives the site id.  Clears the word. */
int ppml_b200_device_status(int* where);

/* ---- OP_MUL_MAT, fp32 operands ------------------------------------------------------------
 * Replaces mul_mat_cuda (src/backend/CUDAKernels.cpp:158; src/cuda/CUDAKernels.cu:1174) and
 * mul_mat_mma_tf32_smem (src/backend/CUDAKernels.cpp:187; src/cuda/CUDAKernels.cu:1675).
 * path AUTO/UMMA compute in tf32 with fp32 accumulation, SIMT in fp32. */
int ppml_b200_mul_mat_f32(const float* A, const float* B, float* C, int M, int K, int N, const float* bias,
                          int path, int tf32_mode, void* stream);

/* A Linear fused with its elementwise neighbours (no counterpart as one call in the reference, which runs them as
 * separate graph nodes):
 *   LayerNorm in front (LayerNorm::forward, src/model/Embedding.cpp:268-289 = OP_NORM, src/backend/CPUKernels.cpp:1488-1512,
 *   then * gamma + beta): pass ln_mean_rstd [M][2] from ppml_b200_row_stats on the raw activations A, ln_u [N], the
 *   weights Wg and the vector v (as `bias`) from ppml_b200_layernorm_fold; the result is LayerNorm(A) W^T + b without
 *   the normalised activations ever being written:  out = rstd_m * (A Wg^T - mean_m * u) + v.
 *   Activation gate behind (OP_ACT_MUL, src/backend/CPUKernels.cpp:1947-1967; act_mul(gate_logits, x, kind) in
 *   src/modules/Attention.cpp:390): with `gate` [M][N] the result is act(out) * gate; with gate == NULL and act != 0
 *   it is act(out).  act: 0 none, 1 sigmoid, 2 silu, 3 gelu (tanh form), 4 tanh, 5 relu, the reference's formulas.
 * Both are optional and combine.  The product runs on the raw rows of A: when |mean| is much larger than the standard
 * deviation of a row the tf32 path loses accuracy by that ratio; path = PPML_B200_PATH_SIMT is exact fp32. */
int ppml_b200_mul_mat_f32_fused(const float* A, const float* B, float* C, int M, int K, int N, const float* bias,
                                const float* ln_mean_rstd, const float* ln_u, const float* gate, int act,
                                int path, int tf32_mode, void* stream);
/* (mean, 1 / sqrt(var + eps)) of every row of x [M][K], variance as in OP_NORM (mean of squared differences). */
int ppml_b200_row_stats(const float* x, float* mean_rstd, int64_t M, int K, float eps, void* stream);
/* Weight-side terms, once per layer: Wg[n][k] = W[n][k] * gamma[k], u[n] = sum_k Wg[n][k], v[n] = sum_k W[n][k] * beta[k] + bias[n]
 * (bias may be NULL). */
int ppml_b200_layernorm_fold(const float* W, const float* gamma, const float* beta, const float* bias, float* Wg, float* u, float* v,
                             int N, int K, void* stream);

/* ---- OP_MUL_MAT, 16-bit operands, fp32 output ------------------------------------------------
 * fp16: replaces mul_mat_mma_f16_smem / mul_mat_mma_f16 / mul_mat_cuda_f16
 * (src/backend/CUDAKernels.cpp:199, :195, :182).  bf16 has no counterpart in the reference (its type
 * enum has no bf16 storage); same contract with bfloat16 operands.  bias may be NULL. */
int ppml_b200_mul_mat_f16(const void* A16, const void* B16, float* C, int M, int K, int N, const float* bias,
                          int path, void* stream);
int ppml_b200_mul_mat_bf16(const void* A16, const void* B16, float* C, int M, int K, int N, const float* bias,
                           int path, void* stream);

/* bf16 products behind fp32 tensors (no counterpart in the reference, whose type enum has no bf16,
 * include/ppml/Tensor.h:35-64): A (activations) and B (weights) are fp32 in device memory; A is cast to bf16 into
 * library-owned scratch on the stream, B into a cached bf16 copy keyed by (device, B, N, K) that is made on the first
 * call and reused afterwards -- call ppml_b200_bf16_shadow_invalidate(B) (NULL: every cached copy) after the weights
 * change.  Creating a cached copy or growing the scratch allocates, which is refused (status 3) during stream
 * capture: make the first call with each weight before capturing.  Tolerance against the fp32 product: 1e-2. */
int ppml_b200_mul_mat_f32_as_bf16(const float* A, const float* B, float* C, int M, int K, int N, const float* bias,
                                  int path, void* stream);
void ppml_b200_bf16_shadow_invalidate(const void* B);

/* fp32 -> fp16 / bf16 (round to nearest even); no counterpart in the reference (it has no cast op). */
int ppml_b200_cast_f32_to_f16(const float* x, void* y, int64_t n, void* stream);
int ppml_b200_cast_f32_to_bf16(const float* x, void* y, int64_t n, void* stream);

/* ---- Q8 block-quantized OP_MUL_MAT ----------------------------------------------------------
 * Replaces mul_mat_q8_cuda (src/backend/CUDAKernels.cpp:169; src/cuda/MulMatQ8Kernel.cu:476-547).
 * W: quantized weights, M rows (out features) of K; wtype 0 = Q8_0 (34-byte blocks), 1 = Q8_1
 * (36-byte blocks), 2 = Q8_0R ([M*K/32*32] int8 plane then [M*K/32] half scales).  X: fp32
 * activations [N][K], quantized on the fly per 32-block.  c_trans 0: C[m*N+n]; 1: C[n*M+m].
 * path_out (may be NULL): 1 = tensor cores, 0 = dp4a on CUDA cores.  PPML_B200_PATH_AUTO runs the tensor-core kernel,
 * except for planar weights with M <= 16 (the model's pair-bias and outer-product-mean projections), where that kernel
 * is bound by its activation quantizer and a one-pass CUDA-core kernel is faster (same quantization, int32 block sums
 * bit for bit the same); PPML_B200_PATH_SIMT is the two-kernel dp4a form of the reference's fallback.
 * Extensions over the reference: bias[M] (may be NULL) is added after the last block;
 * sumi_out (may be NULL) receives the exact int32 block sums as [N][M][K/32]. */
int ppml_b200_mul_mat_q8(const void* W, const float* X, float* C, int M, int N, int K, int wtype, int c_trans,
                         const float* bias, int32_t* sumi_out, int path, int* path_out, void* stream);
/* The tensor-core form either quantizes the activations inside the product kernel (one pass over X) or in a kernel
 * of its own into a library-owned scratch buffer, as the reference's launcher does (src/cuda/MulMatQ8Kernel.cu:483-487);
 * results are identical bit for bit.  mode < 0: chosen per shape (default), 0: always one pass, 1: always two. */
void ppml_b200_set_q8_two_pass(int mode);
/* Kernels one tensor-core call of this shape launches under the current mode (1 or 2); for launch accounting. */
int ppml_b200_q8_kernel_launches(int M, int N, int K);

/* Q8 mul_mat that never allocates device memory.  It has no counterpart in the reference (whose launcher
 * grows a cudaMalloc'ed scratch, src/cuda/MulMatQ8Kernel.cu:430-449).  For callers that cannot allocate
 * at call time -- inside an executor whose arena was planned up front, under a fixed memory budget, or
 * when another allocator owns all free device memory.  Same arguments and result as
 * ppml_b200_mul_mat_q8 on its CUDA-core path (dp4a), bias included; the quantized activations go through
 * a fixed 4 MiB array inside the library image (held by every GPU that loads the library), so
 * N * (K / 32) * 36 bytes must fit: otherwise status 9 and a message on stderr.  All calls share that
 * array: issue them on one stream, overlapping calls race.  The first call on a device looks up the
 * array's address and should be made before any stream capture on that device; the CUDA runtime may
 * load the library's device code and back the array during that first call (free memory can drop once,
 * then never again), so make it before the memory is capped or given away. */
#define PPML_B200_NOALLOC_SCRATCH_BYTES (4u << 20)
int ppml_b200_mul_mat_q8_noalloc(const void* W, const float* X, float* C, int M, int N, int K, int wtype,
                                 int c_trans, const float* bias, void* stream);

/* Replace quantize_rows_q8_1_cuda / dequantize_q8_0_cuda / dequantize_q8_1_cuda
 * (src/backend/CUDAKernels.cpp:164-166; src/cuda/QuantKernels.cu:86-109).  ne = element count. */
int ppml_b200_quantize_rows_q8_1(const float* x, void* y, int64_t ne, void* stream);
int ppml_b200_dequantize_q8_0(const void* x, float* y, int64_t ne, void* stream);
int ppml_b200_dequantize_q8_1(const void* x, float* y, int64_t ne, void* stream);

/* Weight preparation.  Host versions replace quantize_q8_0_host + repack_q8_0_host
 * (include/ppml/QuantBlocks.h:62-79, :128-135) as used by PPMLModel::quantize_big_weight_matrices
 * (src/model/PPML.cpp:4504-4524); the device version does both steps in one kernel. */
int ppml_b200_quantize_q8_0_host(const float* src, void* blocks34, int64_t n);
int ppml_b200_repack_q8_0_host(const void* blocks34, int64_t nblocks, void* q8_0r);
int ppml_b200_quantize_q8_0r(const float* w_dev, void* q8_0r_dev, int64_t ne, void* stream);
int64_t ppml_b200_q8_0r_bytes(int64_t numel);
/* repack_q8_0_host on the device: 34-byte Q8_0 blocks (device, 2-byte aligned) -> planar Q8_0R (device, 4-byte aligned). */
int ppml_b200_repack_q8_0(const void* blocks34_dev, int64_t nblocks, void* q8_0r_dev, void* stream);

/* ---- Q8_0 weights on disk --------------------------------------------------------------------
 * No counterpart in the reference, which refuses to save quantized tensors (src/model/GGUF.cpp:204-213) and
 * re-quantizes on the host at every start (src/model/PPML.cpp:4504-4524).  The container is the reference's
 * GGUF dialect (magic 0x46554747, version 3, "layout_hash" metadata, absolute tensor offsets, 32-byte alignment);
 * tensors are fp32 (type 0) or ggml Q8_0 (type 8: 34-byte blocks of half d + 32 int8), quantized with the host
 * rule of include/ppml/QuantBlocks.h:62-79.  Shapes are rows x cols with cols innermost; Q8_0 needs cols % 32 == 0.
 * write: 0 ok, 1 bad arguments, 2 cols not a multiple of 32, 3 cannot open, 4 write error.
 * load: puts tensor `index` into device memory -- a Q8_0 tensor as planar Q8_0R (ppml_b200_q8_file_nbytes bytes), an
 * fp32 tensor as it is; with scratch_dev (same size, device) the blocks are split by a kernel, without it on the host.
 * The call returns after the copy has finished.  0 ok, 1 bad arguments, 3 pinned allocation, 4 read error, 6 copy. */
int ppml_b200_q8_file_write(const char* path, int n_tensors, const char* const* names, const float* const* weights_host,
                            const int64_t* rows, const int64_t* cols, const int* as_q8);
void* ppml_b200_q8_file_open(const char* path);              /* NULL when the file is missing or malformed */
void ppml_b200_q8_file_close(void* handle);
int ppml_b200_q8_file_count(void* handle);
int ppml_b200_q8_file_find(void* handle, const char* name);  /* index or -1 */
int ppml_b200_q8_file_info(void* handle, int index, char* name, int name_cap, int64_t* rows, int64_t* cols, int* is_q8);
int64_t ppml_b200_q8_file_nbytes(void* handle, int index);
int ppml_b200_q8_file_layout_hash(void* handle, char* hex17); /* 0: the stored hash matches names and shapes, 2: it does not */
int ppml_b200_q8_file_load(void* handle, int index, void* dst_dev, void* scratch_dev, void* stream);

/* ---- OP_FLASH_ATTN_EXT forward ---------------------------------------------------------------
 * Replaces flash_attn_forward_cuda (src/backend/CUDAKernels.cpp:174; include/ppml/FlashAttn.h:60;
 * src/cuda/FlashAttnKernel.cu:206-251).  Q/K/V/O [B][h][L][d] (d innermost), bias [B][h][L][L] or
 * NULL, LSE [B][h][L] or NULL.  O = softmax(scale*Q K^T + bias) V with denominator (l + eps).
 * scale <= 0 means 1/sqrt(d).
 * path: PPML_B200_PATH_SIMT runs the exact fp32 kernels for every head dim.  PPML_B200_PATH_AUTO takes a tensor-core
 * kernel where there is one -- head dim 32 (tcgen05) and head dim 8 with at least 16 query rows (warp-level mma), both
 * with tf32 products and fp32 softmax, 1e-3 on O and 2e-3 on LSE -- when the operands are 16-byte aligned (head dim 32
 * with a bias: bias rows a multiple of 16 bytes), and the exact kernels otherwise.  PPML_B200_PATH_UMMA returns
 * status 1 instead of falling back. */
typedef struct ppml_b200_flash_cfg {
    int B, h, L, d;
    int causal;
    float scale;
    float softmax_eps;
    int Br, Bc;               /* the kernels pick their own tiles.  Bc (0 = 64, as in the reference) still decides one
                                 thing: a query row whose first Bc scores are all -inf comes out as O = 0, LSE = -inf
                                 even when later keys are visible, because the reference's CPU kernel turns such a row
                                 into NaN and then into zeros (src/ops/FlashAttn.cpp:94-121).  Bc < 0 switches this
                                 off: the ordinary softmax over the visible keys (no counterpart in the reference).
                                 The tensor-core kernel takes Bc that are multiples of 64. */
} ppml_b200_flash_cfg;

int ppml_b200_flash_attn_forward(const ppml_b200_flash_cfg* cfg, const float* Q, const float* K, const float* V,
                                 const float* bias, float* O, float* LSE, int path, void* stream);

/* Flash-attention backward: replaces flash_attn_backward_cuda (src/backend/CUDAKernels.cpp:176, :920;
 * include/ppml/FlashAttn.h:85-88; device code src/cuda/FlashAttnKernel.cu:538-1670), same math as
 * flash_attn_backward_cpu (src/ops/FlashAttn.cpp:144-216):
 *   P = exp(S - LSE), D_i = sum_d dO O, dS = P (dO V^T - D), dQ = scale dS K, dK = scale dS^T Q, dV = P^T dO, dbias = dS.
 * Q, K, V, O, dO and the gradients [B, h, L, d]; LSE [B, h, L] as the forward wrote it (a row with LSE = -inf gets zero
 * gradients); bias [B, h, L, L], or one [h, L, L] for every batch with bias_batch_stride = 0 (the reference passes
 * h * L * L); dbias always [B, h, L, L] (masked positions 0).  Any of dQ / dK / dV / dbias may be NULL and is then not
 * computed.  Differences from the reference's launcher: no zero-fill pass and no atomic adds (every output element is
 * written once, results do not depend on scheduling), head dims up to 64 (the reference stops at 32).  Exact fp32 on CUDA
 * cores.  Returns 0, or 7 when the shape is not supported (d > 64). */
int ppml_b200_flash_attn_backward(const ppml_b200_flash_cfg* cfg, int64_t bias_batch_stride, const float* Q, const float* K,
                                  const float* V, const float* bias, const float* O, const float* dO, const float* LSE,
                                  float* dQ, float* dK, float* dV, float* dbias, void* stream);

/* Extended form (no counterpart in the reference, whose config has a single L): Lk keys per query row
 * (K/V [B][h][Lk][d], bias rows of Lk), and bias_batch_stride in elements between batches
 * (h*L*Lk for a full bias tensor, 0 to share one [h][L][Lk] bias across the batch). */
int ppml_b200_flash_attn_forward_ex(const ppml_b200_flash_cfg* cfg, int Lk, int64_t bias_batch_stride,
                                    const float* Q, const float* K, const float* V, const float* bias,
                                    float* O, float* LSE, int path, void* stream);

/* The extended form with 16-bit Q/K/V (fp16, or bfloat16 when is_bf16 != 0): products on the 16-bit tensor-core
 * path, softmax in fp32, bias / O / LSE fp32.  No counterpart in the reference (its tensor type enum has no
 * 16-bit attention, include/ppml/Tensor.h:35-64); same layouts and semantics as above. */
int ppml_b200_flash_attn_forward_16(const ppml_b200_flash_cfg* cfg, int Lk, int64_t bias_batch_stride,
                                    const void* Q16, const void* K16, const void* V16, const float* bias,
                                    float* O, float* LSE, int is_bf16, int path, void* stream);

/* The fused op on token-major operands, with the output gate folded in (no counterpart in the reference as one call: there
 * every attention is wrapped in permute copies -- head split {2,0,1,3} in src/modules/Attention.cpp:363-370, flash layout
 * {1,0,2,3} three times in and once out in src/core/ComputeGraphHelper.cpp:455-483, head merge {1,2,0,3} in
 * src/modules/Attention.cpp:385 -- and followed by act_mul(gate, merged, sigmoid), :390).  Q, K, V are the outputs of the
 * projection Linears as they lie: [B][L][ld_q] and [B][Lk][ld_kv] fp32 with head h in columns [h*d, (h+1)*d) (ld >= h*d,
 * so Q, K, V may also be column ranges of one wider fused projection).  O is written token-major too, [B][L][ld_o], which
 * is what the output Linear reads; with `gate` ([B][L][ld_gate], the gate Linear's output) the result is
 * act(gate) * softmax(..) V (act as in ppml_b200_mul_mat_f32_fused; the model uses sigmoid).  bias, LSE, Lk and
 * bias_batch_stride as in ppml_b200_flash_attn_forward_ex. */
int ppml_b200_flash_attn_forward_tokens(const ppml_b200_flash_cfg* cfg, int Lk, int64_t bias_batch_stride,
                                        const float* Q, const float* K, const float* V, int64_t ld_q, int64_t ld_kv,
                                        const float* bias, const float* gate, int64_t ld_gate, int act, float* O, int64_t ld_o,
                                        float* LSE, int path, void* stream);

/* ---- OP_OUT_PROD -------------------------------------------------------------------------------
 * Replaces out_prod_cuda (src/backend/CUDAKernels.cpp:201; src/cuda/OutProdKernel.cu:211-260):
 * dst[i0,i1,i2,i3] = sum_k s0[i0,k,i2/(ne2/ne02),i3/(ne3/ne03)] * s1[i1,k,i2,i3]; dims in the graph's
 * order (index 0 innermost).  dst is fully overwritten. */
int ppml_b200_out_prod(const float* src0, const float* src1, float* dst,
                       int64_t ne00, int64_t ne01, int64_t ne02, int64_t ne03,
                       int64_t ne10, int64_t ne11, int64_t ne12, int64_t ne13,
                       int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3, int path, void* stream);

/* ---- OP_TRI_MUL ---------------------------------------------------------------------------------
 * Replaces tri_mul_cuda (src/backend/CUDAKernels.cpp:316; src/cuda/PairKernels.cu:47-77, :514-523).
 * Flat layout with D outermost and B innermost: outgoing left[d][i][k][b], right[d][j][k][b];
 * incoming left[d][k][i][b], right[d][k][j][b]; dst[d][i][j][b] = clamp(inv_L * sum_k ..., +-1e4),
 * NaN -> 0. */
int ppml_b200_tri_mul(const float* left, const float* right, float* dst, int64_t D, int64_t I, int64_t J,
                      int64_t K, int64_t B, float inv_L, int outgoing, int path, void* stream);
/* Same contraction with 16-bit operands (fp16, or bfloat16 when is_bf16 != 0), fp32 accumulation and output.
 * No counterpart in the reference (its pair track is fp32); same layouts and semantics as above. */
int ppml_b200_tri_mul_16(const void* left16, const void* right16, float* dst, int64_t D, int64_t I, int64_t J,
                         int64_t K, int64_t B, float inv_L, int outgoing, int is_bf16, int path, void* stream);

/* ---- OP_OUTER_PROD_MEAN ---------------------------------------------------------------------------
 * Replaces outer_prod_mean_cuda (src/backend/CUDAKernels.cpp:325; src/cuda/PairKernels.cu:177-199,
 * :553-561): left/right flat [D][L][N][B]; dst[(d1*D+d2)][i][j][b] = inv_N * sum_n left[d1][i][n][b] *
 * right[d2][j][n][b]. */
int ppml_b200_outer_prod_mean(const float* left, const float* right, float* dst, int64_t D, int64_t L,
                              int64_t N, int64_t B, float inv_N, int path, void* stream);
/* 16-bit operands (fp16 / bfloat16), fp32 accumulation and output; no counterpart in the reference. */
int ppml_b200_outer_prod_mean_16(const void* left16, const void* right16, float* dst, int64_t D, int64_t L,
                                 int64_t N, int64_t B, float inv_N, int is_bf16, int path, void* stream);
/* One rank's share of the op when `left` is split into contiguous d1 slabs across GPUs: D_left slabs of `left`
 * ([D_left][L][N][B]) against all D slabs of `right`; dst [D_left * D][L][L][B] is that rank's contiguous part of
 * the full result (src/backend/CPUKernels.cpp:1022-1028: output block (d1, d2) reads slab d1 of left and slab d2
 * of right only). */
int ppml_b200_outer_prod_mean_slabs(const float* left, const float* right, float* dst, int64_t D_left, int64_t D,
                                    int64_t L, int64_t N, int64_t B, float inv_N, int path, void* stream);

/* ---- exchanges of the sharded block over peer memory --------------------------------------------------
 * No counterpart in the reference (it has no multi-GPU path).  One process per GPU; buffers that peers write into and
 * the flag block are plain device allocations shared through CUDA IPC at set-up:
 *   p = ppml_b200_peer_alloc(bytes) (zero-filled), ppml_b200_peer_export(p, handle[64]) -> send the 64 bytes to the other
 *   ranks by any means -> q = ppml_b200_peer_open(handle) maps a peer's allocation (ppml_b200_peer_close / _free at the end).
 * dst_ptrs / out_ptrs / flag_ptrs are host arrays of `world` device pointers, entry r = rank r's buffer as mapped in THIS
 * process (entry `rank` = the local allocation).  Flag blocks hold ppml_b200_peer_flag_bytes() bytes.  `site` (0..15)
 * names the exchange inside the block: every site has its own flags and epoch, and all ranks must run the same sequence of
 * sites.  Each call is one kernel on `stream`: arrive round, plain stores into the peers' buffers, landed round; when it
 * has run, this rank's own buffer is complete and every later kernel on the stream may read it (locally).  A launch can
 * be recorded in a CUDA graph.  Waits are bounded: a rank whose peers do not show up within about 1.5 s leaves status 8 in
 * the device error word (ppml_b200_device_status) and returns.  world <= 8.
 *   all_gather: `bytes_per_rank` (multiple of 16) from src to offset rank * bytes_per_rank of every rank's buffer.
 *   transpose:  x [n_loc][L][C] fp32, this rank's n range of an [n][l][C] activation -> out [L / world][world * n_loc][C] on
 *               the rank that owns l: the reference's (n, l) permute copies (src/modules/Attention.cpp:489, :744). */
int ppml_b200_peer_flag_bytes(void);
void* ppml_b200_peer_alloc(int64_t bytes);
void ppml_b200_peer_free(void* p);
int ppml_b200_peer_export(void* p, void* handle64);
void* ppml_b200_peer_open(const void* handle64);
void ppml_b200_peer_close(void* p);
int ppml_b200_peer_all_gather(const void* src, void* const* dst_ptrs, int64_t bytes_per_rank, int rank, int world,
                              void* const* flag_ptrs, int site, void* stream);
int ppml_b200_peer_transpose(const float* x, void* const* out_ptrs, int n_loc, int L, int C, int rank, int world,
                             void* const* flag_ptrs, int site, void* stream);

/* ---- per-shape statistics ----------------------------------------------------------------------------
 * Replace mulmat_stats_cuda_begin / mulmat_stats_cuda_end (src/backend/CUDAKernels.cpp:190-191;
 * src/cuda/CUDAKernels.cu:1693-1732): event pair around one launch, totals per (path, M, K, N).
 * Active only when the environment has PPML_MULMAT_STATS=1.  ppml_b200_mulmat_stats_dump writes
 * the table (one line per shape) into buf, clears it and returns the number of bytes written; what is
 * left at process exit is printed to stderr, as the reference prints its table
 * (include/ppml/MulMatStats.h:137-145).  At most 4096 event pairs are kept open at a time. */
void ppml_b200_mulmat_stats_begin(int M, int K, int N);
void ppml_b200_mulmat_stats_end(const char* path);
int ppml_b200_mulmat_stats_dump(char* buf, int cap);

#ifdef __cplusplus
}
#endif
#endif /* PPML_B200_H */
