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

// Library-owned device scratch, one set per device, guarded by a mutex as the reference's launcher guards its own
// (src/cuda/MulMatQ8Kernel.cu:430-449).  Three independent buffers, so that a launch recorded in a CUDA graph never
// sees its buffer move:
//   kScratchDp4a   Q8_1 activation blocks of the dp4a path                      (grows)
//   kScratchTwoPass int8 activations + scale tables of the two-pass tensor-core form: that form is only chosen for
//                  at most num_sms token tiles and K <= 1024, so the buffer is allocated once at its maximum size
//                  (about 20 MB) and its address never changes
//   kScratchCast   bf16 copy of fp32 activations (ppml_b200_mul_mat_f32_as_bf16) (grows)
// A buffer that has to grow is replaced, never freed: the old one stays allocated until the process exits, because a
// captured graph may still hold its address (sizes at least double, so the retired ones add up to less than the live
// one).  Growing is refused (null) while the stream is being captured: allocation is not a stream operation.
enum { kScratchDp4a = 0, kScratchTwoPass = 1, kScratchCast = 2, kScratchKinds = 3 };
struct Scratch { void* ptr = nullptr; size_t bytes = 0; };
Scratch g_scratch[64][kScratchKinds];
std::vector<void*>* g_retired = nullptr;     // leaked on purpose
std::mutex g_scratch_mtx;

bool stream_is_capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) { cudaGetLastError(); return false; }
    return cs != cudaStreamCaptureStatusNone;
}

// Caller holds g_scratch_mtx.
void* ensure_scratch(int kind, size_t bytes, cudaStream_t st) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    Scratch& s = g_scratch[dev][kind];
    if (bytes <= s.bytes) return s.ptr;
    if (stream_is_capturing(st)) return nullptr;
    size_t want = bytes;
    if (kind != kScratchTwoPass && want < 2 * s.bytes) want = 2 * s.bytes;
    void* p = nullptr;
    if (cudaMalloc(&p, want) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (s.ptr) {
        if (!g_retired) g_retired = new std::vector<void*>();
        g_retired->push_back(s.ptr);
    }
    s.ptr = p; s.bytes = want;
    return p;
}

// Whether the tensor-core Q8 product quantizes its activations in a kernel of its own (into the shared scratch) instead
// of inside the product kernel.  Measured on the sweep shapes: the one-pass form wins wherever there are more token
// tiles than SMs (33 vs 44 us at 65536 x 128 x 128, 126 vs 197 us at 65536 x 1024 x 128: the extra pass over X costs
// more than the quantizer warps do); with few token tiles and a long K the in-kernel quantizer is a serial chain of
// K / 32 steps on two or four warps, and the two-pass form wins (33 vs 41 us at 408 x 1024 x N, 58 vs 68 us at
// 2601 x 1024 x 1024).  M = weight rows, N = tokens.  PPML_B200_Q8_TWO_PASS=0 / 1 or ppml_b200_set_q8_two_pass() force the choice (measurements, tests).
int g_q8_two_pass = [] { const char* e = std::getenv("PPML_B200_Q8_TWO_PASS"); return e ? (e[0] == '1' ? 1 : 0) : -1; }();
bool q8_two_pass(int M, int N, int K) {
    const int forced = g_q8_two_pass;
    if (forced >= 0) return forced == 1;
    // K >= 1024: the quantized A tile fills the shared memory, and the one-pass form has no room for its result store
    // buffers.  With two or more weight column blocks the two-pass form, which needs no raw activation stages and keeps
    // the buffers, is faster although it reads the activations twice (442 vs 495 us at 65536 x 1024 x 1024, 258 vs 291 at
    // 512 weight rows, 165 vs 168 at 256; 126 vs 110 at 128).
    if (K < 1024) return false;
    return (N + 127) / 128 <= num_sms() || M >= 256;
}

struct FusedEpi { const float* ln_stats = nullptr; const float* ln_u = nullptr; const float* gate = nullptr; int act = 0; };

int mul_mat_any(const void* A, const void* B, float* C, int M, int K, int N, const float* bias, int path,
                int elem, int tf32_mode, cudaStream_t st, const FusedEpi& fe = FusedEpi()) {
    if (!A || !B || !C || M <= 0 || K <= 0 || N <= 0 || !path_ok(path)) return ST_BAD_ARGS;
    if (path != PPML_B200_PATH_SIMT) {
        UmmaGemmArgs a{};
        a.A = A; a.B = B; a.C = C; a.M = M; a.N = N; a.K = K; a.batch = 1;
        a.lda = K; a.ldb = K; a.a_batch = 0; a.b_batch = 0; a.ldc = N; a.c_batch = 0;
        a.bias = bias; a.alpha = 1.0f; a.clamp = 0; a.opm_D = 0; a.opm_L = 0; a.elem = elem; a.tf32_mode = tf32_mode;
        a.ln_stats = fe.ln_stats; a.ln_u = fe.ln_u; a.gate = fe.gate; a.act = fe.act;
        const int rc = launch_umma_gemm(a, st);
        if (rc != ST_UNSUPPORTED_PATH || path == PPML_B200_PATH_UMMA) return rc;
    }
    SimtContract p{};
    p.M = M; p.N = N; p.K = K;
    p.a_sm = K; p.a_sk = 1; p.b_sn = K; p.b_sk = 1; p.c_sm = N; p.c_sn = 1;
    p.planes = 1; p.ne2 = 1; p.a_div2 = 1; p.a_div3 = 1;
    p.bias = bias; p.bias_seed = (elem == 0 && fe.ln_stats == nullptr) ? 1 : 0; p.alpha = 1.0f;
    p.ln_stats = fe.ln_stats; p.ln_u = fe.ln_u; p.gate = fe.gate; p.act = fe.act;
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

int ppml_b200_mul_mat_f32_fused(const float* A, const float* B, float* C, int M, int K, int N, const float* bias,
                                const float* ln_mean_rstd, const float* ln_u, const float* gate, int act,
                                int path, int tf32_mode, void* stream) {
    if (tf32_mode < 0 || tf32_mode > 2 || act < 0 || act > 5) return ST_BAD_ARGS;
    if ((ln_mean_rstd == nullptr) != (ln_u == nullptr)) return ST_BAD_ARGS;
    if (ln_mean_rstd && (reinterpret_cast<uintptr_t>(ln_mean_rstd) & 7u)) return ST_BAD_ARGS;
    if (gate && (reinterpret_cast<uintptr_t>(gate) & 15u) && (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15u) == 0)) return ST_BAD_ARGS;
    FusedEpi fe;
    fe.ln_stats = ln_mean_rstd; fe.ln_u = ln_u; fe.gate = gate; fe.act = act;
    return mul_mat_any(A, B, C, M, K, N, bias, path, 0, tf32_mode, as_stream(stream), fe);
}
int ppml_b200_row_stats(const float* x, float* mean_rstd, int64_t M, int K, float eps, void* stream) {
    return launch_row_stats(x, mean_rstd, M, K, eps, as_stream(stream));
}
int ppml_b200_layernorm_fold(const float* W, const float* gamma, const float* beta, const float* bias, float* Wg, float* u, float* v,
                             int N, int K, void* stream) {
    return launch_ln_fold(W, gamma, beta, bias, Wg, u, v, N, K, as_stream(stream));
}

int ppml_b200_mul_mat_f16(const void* A16, const void* B16, float* C, int M, int K, int N, const float* bias,
                          int path, void* stream) {
    return mul_mat_any(A16, B16, C, M, K, N, bias, path, 1, 0, as_stream(stream));
}

int ppml_b200_mul_mat_bf16(const void* A16, const void* B16, float* C, int M, int K, int N, const float* bias,
                           int path, void* stream) {
    return mul_mat_any(A16, B16, C, M, K, N, bias, path, 2, 0, as_stream(stream));
}

// fp32 tensors, bf16 products: the activations are cast into library scratch on the stream, the weights into a
// cached bf16 copy keyed by (device, pointer, N, K) that is made on first use and lives until it is invalidated.
namespace {
std::map<std::tuple<int, const void*, int, int>, void*>* g_shadow = nullptr;     // leaked on purpose
}
int ppml_b200_mul_mat_f32_as_bf16(const float* A, const float* B, float* C, int M, int K, int N, const float* bias,
                                  int path, void* stream) {
    if (!A || !B || !C || M <= 0 || K <= 0 || N <= 0 || !path_ok(path)) return ST_BAD_ARGS;
    cudaStream_t st = as_stream(stream);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return ST_LAUNCH; }
    std::lock_guard<std::mutex> lock(g_scratch_mtx);
    if (!g_shadow) g_shadow = new std::map<std::tuple<int, const void*, int, int>, void*>();
    const auto key = std::make_tuple(dev, static_cast<const void*>(B), N, K);
    void* b16 = nullptr;
    auto it = g_shadow->find(key);
    if (it != g_shadow->end()) {
        b16 = it->second;
    } else {
        if (stream_is_capturing(st)) return ST_SCRATCH;
        if (cudaMalloc(&b16, static_cast<size_t>(N) * K * 2) != cudaSuccess) { cudaGetLastError(); return ST_SCRATCH; }
        if (launch_cast(B, b16, static_cast<long long>(N) * K, 1, st) != ST_OK) { cudaFree(b16); return ST_LAUNCH; }
        (*g_shadow)[key] = b16;
    }
    void* a16 = ensure_scratch(kScratchCast, static_cast<size_t>(M) * K * 2, st);
    if (!a16) return ST_SCRATCH;
    const int rc = launch_cast(A, a16, static_cast<long long>(M) * K, 1, st);
    if (rc != ST_OK) return rc;
    return mul_mat_any(a16, b16, C, M, K, N, bias, path, 2, 0, st);
}
void ppml_b200_bf16_shadow_invalidate(const void* B) {
    std::lock_guard<std::mutex> lock(g_scratch_mtx);
    if (!g_shadow) return;
    cudaDeviceSynchronize();
    for (auto it = g_shadow->begin(); it != g_shadow->end();) {
        if (B == nullptr || std::get<1>(it->first) == B) { cudaFree(it->second); it = g_shadow->erase(it); }
        else ++it;
    }
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
        if (wtype == 2 && path == PPML_B200_PATH_AUTO && M <= 16) {
            // very few output columns: the tensor-core kernel would be bound by its activation quantizer (measured at
            // 65536 tokens: 128 -> 8 11 against 21 us, 256 -> 16 32 against 32, 64 -> 16 at 262144 tokens 29 against 56; at the
            // 8192 tokens of an eight-way shard 4 against 8 and 6 against 12).  The choice must not depend on the token
            // count: a shard of the tokens and the whole have to take the same kernel to give the same bits.
            const int rs = launch_q8_skinny(W, X, C, M, N, K, c_trans, bias, sumi_out, st);
            if (rs != ST_UNSUPPORTED_PATH) return rs;
        }
        if (wtype == 2) {
            // two-pass form (activations quantized by a kernel of their own into the shared scratch) or one-pass form
            void* scratch = nullptr;
            std::unique_lock<std::mutex> lock(g_scratch_mtx, std::defer_lock);
            if (q8_two_pass(M, N, K)) {
                lock.lock();
                // the largest problem this form is chosen for (forced mode aside): one token tile per SM, K = 1024
                size_t need = umma_q8_scratch_bytes(N, K);
                const size_t fixed = umma_q8_scratch_bytes(num_sms() * 128, 1024);
                if (need < fixed) need = fixed;
                scratch = ensure_scratch(kScratchTwoPass, need, st);
                if (!scratch) return ST_SCRATCH;
            }
            rc = launch_umma_q8(W, X, C, M, N, K, c_trans, bias, sumi_out, st, scratch);
        }
        if (rc == ST_OK && path_out) *path_out = 1;
        if (rc != ST_UNSUPPORTED_PATH || path == PPML_B200_PATH_UMMA) return rc;
    }
    const int nblk = K / 32;
    std::lock_guard<std::mutex> lock(g_scratch_mtx);
    void* qa = ensure_scratch(kScratchDp4a, static_cast<size_t>(nblk) * static_cast<size_t>(N) * 36, st);
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
int ppml_b200_repack_q8_0(const void* blocks34_dev, int64_t nblocks, void* q8_0r_dev, void* stream) {
    return launch_repack_q8_0(blocks34_dev, nblocks, q8_0r_dev, as_stream(stream));
}

namespace {
// elem: 0 = fp32, 1 = bf16, 2 = fp16 Q/K/V
int flash_attn_any(const ppml_b200_flash_cfg* cfg, int Lk, int64_t bias_batch_stride, const void* Q, const void* K,
                   const void* V, int elem, const float* bias, float* O, float* LSE, int path, void* stream,
                   const AttnLayout* layout = nullptr) {
    if (!cfg || !Q || !K || !V || !O || !path_ok(path)) return ST_BAD_ARGS;
    if (cfg->B <= 0 || cfg->h <= 0 || cfg->L <= 0 || cfg->d <= 0 || Lk <= 0) return ST_BAD_ARGS;
    const AttnLayout lay = layout ? *layout : AttnLayout::flash(cfg->h, cfg->L, Lk, cfg->d);
    const float scale = (cfg->scale > 0.f) ? cfg->scale : 1.0f / std::sqrt(static_cast<float>(cfg->d));
    // Bc is the key tile of the reference's CPU kernel (<= 0 there means 64, src/ops/FlashAttn.cpp:58); it only matters
    // for rows whose first Bc scores are all -inf, which that kernel turns into O = 0, LSE = -inf.  Bc < 0 here switches
    // that rule off (ordinary softmax over the visible keys).
    const int ft = cfg->Bc < 0 ? 0 : (cfg->Bc == 0 ? 64 : cfg->Bc);
    if (path != PPML_B200_PATH_SIMT) {
        const int rc = launch_umma_attn(Q, K, V, elem, bias, O, LSE, cfg->B, cfg->h, cfg->L, Lk, cfg->d, cfg->causal ? 1 : 0,
                                        scale, cfg->softmax_eps, bias_batch_stride, ft, lay, as_stream(stream));
        if (rc != ST_UNSUPPORTED_PATH) return rc;
        if (elem == 0) {
            const int rc8 = launch_attn_d8_mma(static_cast<const float*>(Q), static_cast<const float*>(K), static_cast<const float*>(V),
                                               bias, O, LSE, cfg->B, cfg->h, cfg->L, Lk, cfg->d, cfg->causal ? 1 : 0, scale,
                                               cfg->softmax_eps, bias_batch_stride, ft, lay, as_stream(stream));
            if (rc8 != ST_UNSUPPORTED_PATH) return rc8;
        }
        if (path == PPML_B200_PATH_UMMA) return rc;
    }
    return launch_attn_rowwarp(Q, K, V, elem, bias, O, LSE, cfg->B, cfg->h, cfg->L, Lk, cfg->d, cfg->causal ? 1 : 0, scale,
                               cfg->softmax_eps, bias_batch_stride, ft, lay, as_stream(stream));
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

int ppml_b200_flash_attn_forward_tokens(const ppml_b200_flash_cfg* cfg, int Lk, int64_t bias_batch_stride,
                                        const float* Q, const float* K, const float* V, int64_t ld_q, int64_t ld_kv,
                                        const float* bias, const float* gate, int64_t ld_gate, int act, float* O, int64_t ld_o,
                                        float* LSE, int path, void* stream) {
    if (!cfg || cfg->h <= 0 || cfg->d <= 0 || cfg->L <= 0 || Lk <= 0) return ST_BAD_ARGS;
    const int64_t hd = static_cast<int64_t>(cfg->h) * cfg->d;
    if (ld_q < hd || ld_kv < hd || ld_o < hd || (gate && ld_gate < hd) || act < 0 || act > 5) return ST_BAD_ARGS;
    AttnLayout lay{};
    lay.q_l = ld_q; lay.q_h = cfg->d; lay.q_b = ld_q * cfg->L;
    lay.k_l = lay.v_l = ld_kv; lay.k_h = lay.v_h = cfg->d; lay.k_b = lay.v_b = ld_kv * Lk;
    lay.o_l = ld_o; lay.o_h = cfg->d; lay.o_b = ld_o * cfg->L;
    lay.g_l = ld_gate; lay.g_h = cfg->d; lay.g_b = ld_gate * cfg->L;
    lay.gate = gate; lay.act = gate ? act : 0;
    return flash_attn_any(cfg, Lk, bias_batch_stride, Q, K, V, 0, bias, O, LSE, path, stream, &lay);
}

int ppml_b200_flash_attn_backward(const ppml_b200_flash_cfg* cfg, int64_t bias_batch_stride, const float* Q, const float* K,
                                  const float* V, const float* bias, const float* O, const float* dO, const float* LSE,
                                  float* dQ, float* dK, float* dV, float* dbias, void* stream) {
    if (!cfg || !Q || !K || !V || !O || !dO || !LSE) return ST_BAD_ARGS;
    if (cfg->B <= 0 || cfg->h <= 0 || cfg->L <= 0 || cfg->d <= 0) return ST_BAD_ARGS;
    if (!dQ && !dK && !dV && !dbias) return ST_BAD_ARGS;
    const float scale = (cfg->scale > 0.f) ? cfg->scale : 1.0f / std::sqrt(static_cast<float>(cfg->d));
    return launch_attn_backward(cfg->B, cfg->h, cfg->L, cfg->d, cfg->causal ? 1 : 0, scale, Q, K, V, bias, bias_batch_stride,
                                O, dO, LSE, dQ, dK, dV, dbias, as_stream(stream));
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
struct StatAgg { long long calls = 0; double ms = 0.0; };
std::vector<StatRec>* g_stat_open = nullptr;                                       // leaked on purpose: used at exit
std::map<std::tuple<std::string, int, int, int>, StatAgg>* g_stat_agg = nullptr;
std::mutex g_stat_mtx;
constexpr size_t kStatOpenCap = 4096;      // event pairs kept before they are folded into the table
bool stats_enabled() {
    static const bool on = [] { const char* e = std::getenv("PPML_MULMAT_STATS"); return e && e[0] == '1'; }();
    return on;
}
// Folds every closed record into the table (waits for its end event) and destroys its events.  Caller holds the mutex.
void stats_fold() {
    if (!g_stat_open) return;
    if (!g_stat_agg) g_stat_agg = new std::map<std::tuple<std::string, int, int, int>, StatAgg>();
    std::vector<StatRec> keep;
    for (auto& r : *g_stat_open) {
        if (!r.closed) { keep.push_back(r); continue; }
        float ms = 0.f;
        if (cudaEventSynchronize(r.e1) != cudaSuccess || cudaEventElapsedTime(&ms, r.e0, r.e1) != cudaSuccess) {
            cudaGetLastError(); ms = 0.f;
        }
        StatAgg& a = (*g_stat_agg)[std::make_tuple(r.path, r.M, r.K, r.N)];
        a.calls += 1; a.ms += ms;
        cudaEventDestroy(r.e0); cudaEventDestroy(r.e1);
    }
    g_stat_open->swap(keep);
}
int stats_format(char* buf, int cap) {
    int off = 0;
    if (!g_stat_agg) return 0;
    for (auto& kv : *g_stat_agg) {
        const int n = std::snprintf(buf + off, static_cast<size_t>(cap - off), "%s M=%d K=%d N=%d calls=%lld ms=%.4f\n",
                                    std::get<0>(kv.first).c_str(), std::get<1>(kv.first), std::get<2>(kv.first),
                                    std::get<3>(kv.first), kv.second.calls, kv.second.ms);
        if (n < 0 || n >= cap - off) break;
        off += n;
    }
    return off;
}
// At process exit the table goes to stderr, the way the reference prints its own at exit
// (include/ppml/MulMatStats.h:137-145).  The reference's table lives in its own binary and cannot be fed from here.
void stats_at_exit() {
    std::lock_guard<std::mutex> lock(g_stat_mtx);
    stats_fold();
    static char buf[1 << 16];
    if (stats_format(buf, sizeof(buf)) > 0) std::fprintf(stderr, "[ppml_b200 MULMAT-STATS] per shape (CUDA events)\n%s", buf);
}
}  // namespace

void ppml_b200_mulmat_stats_begin(int M, int K, int N) {
    if (!stats_enabled()) return;
    std::lock_guard<std::mutex> lock(g_stat_mtx);
    if (!g_stat_open) { g_stat_open = new std::vector<StatRec>(); std::atexit(stats_at_exit); }
    if (g_stat_open->size() >= kStatOpenCap) stats_fold();
    StatRec r{M, K, N, nullptr, nullptr, "", false};
    if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) { cudaGetLastError(); return; }
    cudaEventRecord(r.e0, 0);
    g_stat_open->push_back(r);
}

void ppml_b200_mulmat_stats_end(const char* path) {
    if (!stats_enabled()) return;
    std::lock_guard<std::mutex> lock(g_stat_mtx);
    if (!g_stat_open) return;
    for (auto it = g_stat_open->rbegin(); it != g_stat_open->rend(); ++it) {
        if (!it->closed) { cudaEventRecord(it->e1, 0); it->path = path ? path : "?"; it->closed = true; break; }
    }
}

// Writes the table accumulated so far into buf and clears it.
int ppml_b200_mulmat_stats_dump(char* buf, int cap) {
    if (!buf || cap <= 0) return 0;
    buf[0] = 0;
    if (!stats_enabled()) return 0;
    std::lock_guard<std::mutex> lock(g_stat_mtx);
    stats_fold();
    const int off = stats_format(buf, cap);
    if (g_stat_agg) g_stat_agg->clear();
    return off;
}

}  // extern "C"
