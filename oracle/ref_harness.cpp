// ref_harness.cpp -- C-ABI shim around the UNMODIFIED reference CPU implementation.
//
// TEST INFRASTRUCTURE ONLY (same rule as ppml_oracle.c): used to validate the
// restatement, to generate golden fixtures and as the timed CPU baseline.
//
// This file holds no arithmetic of its own.  Each entry builds the one-node graph
// the reference's graph constructors produce (src/core/ComputeGraphHelper.cpp:
// mul_mat :262, out_prod :318, triangle_mul :390, outer_product_mean :1748),
// binds the caller's host buffers to the leaves and runs the reference's own
// CPUBackend::graph_compute (src/backend/CPUBackend.cpp:177), i.e. the kernels in
// src/backend/CPUKernels.cpp.  Attention calls the reference's public functions
// from src/ops/FlashAttn.cpp directly; the quantizers are the inline host
// functions of include/ppml/QuantBlocks.h.
//
// It is compiled by oracle/Makefile together with the reference's sources where
// they lie; the result goes to oracle/_ref/libppml_ref.so.
#include <cstdint>
#include <cstring>
#include <memory>
#include <vector>

#include "ppml/Backend.h"
#include "ppml/ComputeGraph.h"
#include "ppml/Context.h"
#include "ppml/FlashAttn.h"
#include "ppml/GGUF.h"
#include "ppml/QuantBlocks.h"

using namespace ppml;

// The reference's CUDA dispatcher lives in a translation unit that needs every
// .cu launcher; this CPU-only build never dispatches to it.
namespace ppml {
Status CUDABackend::dispatch_node(TensorF32*, ComputeParams*) { return Status::NOT_SUPPORTED; }
}

namespace {

struct ArenaScope {               // frees the graph nodes built inside one call
    void* mark;
    ArenaScope() : mark(context().mark_objects()) {}
    ~ArenaScope() { context().reset_objects_to(mark); }
};

TensorF32* leaf(const std::vector<int64_t>& dims, const void* host, tensor_type type = TENSOR_TYPE_F32) {
    int64_t ne[4] = {1, 1, 1, 1};
    for (size_t i = 0; i < dims.size() && i < 4; ++i) ne[i] = dims[i];
    TensorF32* t = context().new_tensor<float>(static_cast<int>(dims.size()), ne);
    t->type = type;
    t->bind_data(const_cast<void*>(host));
    return t;
}

CPUBackend& backend(int n_threads) {
    static std::unique_ptr<CPUBackend> be;
    static int cur = -1;
    if (!be || cur != n_threads) { be.reset(); be = std::make_unique<CPUBackend>(n_threads); cur = n_threads; }
    return *be;
}

int run(TensorF32* out, float* dst, int n_threads) {
    ComputeGraph* g = ComputeGraph::new_graph(&context());
    g->build_forward_expand(out);
    if (backend(n_threads).graph_compute(g) != Status::SUCCESS) return 1;
    std::memcpy(dst, out->data(), static_cast<size_t>(out->numel()) * sizeof(float));
    return 0;
}

}  // namespace

extern "C" {

// OP_MUL_MAT, fp32 (f16 = 0) or 16-bit half operands (f16 = 1); bias may be null.
int ref_mul_mat(const void* a, const void* b, const float* bias, float* c,
                int M, int K, int N, int f16, int n_threads) {
    ArenaScope scope;
    const tensor_type ty = f16 ? TENSOR_TYPE_F16 : TENSOR_TYPE_F32;
    TensorF32* la = leaf({K, M}, a, ty);
    TensorF32* lb = leaf({K, N}, b, ty);
    TensorF32* lbias = bias ? leaf({N}, bias) : nullptr;
    return run(mul_mat(la, lb, lbias), c, n_threads);
}

int ref_out_prod(const float* s0, const float* s1, float* dst,
                 int64_t ne00, int64_t ne01, int64_t ne02, int64_t ne03,
                 int64_t ne10, int64_t ne11, int64_t ne12, int64_t ne13, int n_threads) {
    ArenaScope scope;
    TensorF32* a = leaf({ne00, ne01, ne02, ne03}, s0);
    TensorF32* b = leaf({ne10, ne11, ne12, ne13}, s1);
    return run(out_prod(a, b), dst, n_threads);
}

// left/right dims as the graph passes them: outgoing [D,I,K,B]/[D,J,K,B], incoming [D,K,I,B]/[D,K,J,B].
int ref_tri_mul(const float* left, const float* right, float* dst,
                int64_t D, int64_t I, int64_t J, int64_t K, int64_t B, float L, int outgoing,
                int n_threads) {
    ArenaScope scope;
    TensorF32* l = outgoing ? leaf({D, I, K, B}, left) : leaf({D, K, I, B}, left);
    TensorF32* r = outgoing ? leaf({D, J, K, B}, right) : leaf({D, K, J, B}, right);
    return run(triangle_mul(l, r, L, outgoing != 0), dst, n_threads);
}

int ref_outer_prod_mean(const float* left, const float* right, float* dst,
                        int64_t D, int64_t L, int64_t N, int64_t B, int n_threads) {
    ArenaScope scope;
    TensorF32* l = leaf({D, L, N, B}, left);
    TensorF32* r = leaf({D, L, N, B}, right);
    return run(outer_product_mean(l, r, static_cast<int>(N)), dst, n_threads);
}

int ref_flash_attn_forward(int B, int h, int L, int d, int causal, float scale, float eps, int Bc,
                           const float* Q, const float* K, const float* V, const float* bias,
                           float* O, float* LSE, int naive) {
    FlashAttnConfig cfg;
    cfg.B = B; cfg.h = h; cfg.L = L; cfg.d = d; cfg.causal = causal != 0;
    cfg.scale = scale; cfg.softmax_eps = eps; cfg.Bc = Bc;
    const bool ok = naive ? flash_attn_forward_ref_cpu(cfg, Q, K, V, bias, O, LSE)
                          : flash_attn_forward_cpu(cfg, Q, K, V, bias, O, LSE);
    return ok ? 0 : 1;
}

// flash_attn_backward_cpu (src/ops/FlashAttn.cpp:144-216): bias and dbias [B,h,L,L]; null outputs are skipped.
int ref_flash_attn_backward(int B, int h, int L, int d, int causal, float scale, float eps,
                            const float* Q, const float* K, const float* V, const float* bias,
                            const float* O, const float* dO, const float* LSE,
                            float* dQ, float* dK, float* dV, float* dbias) {
    FlashAttnConfig cfg;
    cfg.B = B; cfg.h = h; cfg.L = L; cfg.d = d; cfg.causal = causal != 0;
    cfg.scale = scale; cfg.softmax_eps = eps;
    return flash_attn_backward_cpu(cfg, Q, K, V, bias, O, dO, LSE, dQ, dK, dV, dbias) ? 0 : 1;
}

// The unfused attention graph of SelfAttention::forward_graph (src/modules/Attention.cpp:267-283),
// Q [Lq,D,H,B], K/V [Lk,D,H,B] (sequence innermost), bias [Lk,Lq,H,B] or null, out [Lq,D,H,B].
int ref_attention_legacy(const float* Q, const float* K, const float* V, const float* bias, float* O,
                         int64_t Lq, int64_t Lk, int64_t D, int64_t H, int64_t B, float scale_val,
                         int n_threads) {
    ArenaScope scope;
    TensorF32* q = leaf({Lq, D, H, B}, Q);
    TensorF32* k = leaf({Lk, D, H, B}, K);
    TensorF32* v = leaf({Lk, D, H, B}, V);
    TensorF32* scaled = scale(out_prod(k, q), scale_val);
    if (bias) scaled = add_impl(scaled, leaf({Lk, Lq, H, B}, bias), false);
    TensorF32* attn = softmax(scaled);
    TensorF32* out = out_prod(permute(attn, {1, 0, 2, 3}), permute(v, {1, 0, 2, 3}));
    return run(out, O, n_threads);
}

int ref_quantize_q8_0(const float* src, void* dst, int64_t n) {
    return quantize_q8_0_host(src, static_cast<block_q8_0*>(dst), n) ? 0 : 1;
}
int ref_quantize_q8_1(const float* src, void* dst, int64_t n) {
    return quantize_q8_1_host(src, static_cast<block_q8_1*>(dst), n) ? 0 : 1;
}
void ref_repack_q8_0(const void* src, int64_t nblocks, void* dst) {
    repack_q8_0_host(static_cast<const block_q8_0*>(src), nblocks, dst);
}
void ref_dequantize_q8_0(const void* src, float* dst, int64_t n) {
    dequantize_q8_0_host(static_cast<const block_q8_0*>(src), dst, n);
}
void ref_dequantize_q8_1(const void* src, float* dst, int64_t n) {
    dequantize_q8_1_host(static_cast<const block_q8_1*>(src), dst, n);
}

// The reference's own checkpoint reader (src/model/GGUF.cpp:314-470) on a file of fp32 tensors: builds parameter tensors
// of the given shapes (rows x cols, cols innermost), calls load_gguf with the names (so the stored layout hash is
// checked against names and shapes) and copies the loaded values out.  0 ok, 1 the reader threw.
int ref_gguf_load(const char* path, int n, const char* const* names, const int64_t* rows, const int64_t* cols, float* const* out) {
    ArenaScope scope;
    try {
        std::vector<TensorF32*> params;
        std::vector<std::string> tnames;
        std::vector<std::vector<float>> store(static_cast<size_t>(n));
        for (int i = 0; i < n; ++i) {
            store[i].assign(static_cast<size_t>(rows[i] * cols[i]), 0.0f);
            params.push_back(leaf({cols[i], rows[i]}, store[i].data()));
            tnames.push_back(names[i]);
        }
        load_gguf(path, params, tnames);
        for (int i = 0; i < n; ++i) std::memcpy(out[i], store[i].data(), store[i].size() * sizeof(float));
        return 0;
    } catch (const std::exception&) {
        return 1;
    }
}

}  // extern "C"
