"""Host-side mirror of the reference's per-op launcher interface for the dense-contraction path
(the free functions CUDABackend::dispatch_node calls, src/backend/CUDAKernels.cpp:97-345), over the
C ABI of libppml_b200.so.  Same names, argument meaning and error behaviour; tensors are torch CUDA
tensors used only as device memory.  A non-zero status raises RuntimeError."""
import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import PATH_AUTO, PATH_SIMT, PATH_UMMA, TF32_ROUND, TF32_TMA, FlashCfg


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    s = torch.cuda.current_stream().cuda_stream
    return C.c_void_p(s) if s else None


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed with status {rc}")


def _f32c(t):
    assert t.is_cuda and t.dtype == torch.float32
    return t.contiguous()


def device_status():
    """Synchronizes; returns (code, where): (0, 0) unless a kernel gave up a bounded wait."""
    where = C.c_int(0)
    rc = _lib.load().ppml_b200_device_status(C.byref(where))
    return rc, where.value


def mul_mat_cuda(A, B, bias=None, path=PATH_AUTO, tf32_mode=TF32_TMA, out=None):
    """C[M,N] = A[M,K] @ B[N,K]^T (+ bias[N]); replaces mul_mat_cuda / mul_mat_mma_tf32_smem.  The default
    tf32_mode is the one the C++ forwarders under the reference's names use (the TMA unit delivers tf32)."""
    A, B = _f32c(A), _f32c(B)
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K
    Cout = out if out is not None else torch.empty((M, N), device=A.device, dtype=torch.float32)
    rc = _lib.load().ppml_b200_mul_mat_f32(_p(A), _p(B), _p(Cout), M, K, N, _p(bias), path, tf32_mode, _stream())
    _check(rc, "mul_mat_f32")
    return Cout


ACT = {"none": 0, "sigmoid": 1, "silu": 2, "gelu": 3, "tanh": 4, "relu": 5}


def layernorm_fold(W, gamma, beta, bias=None):
    """Weight-side terms of LayerNorm -> Linear, once per layer: (Wg, u, v)."""
    W = _f32c(W)
    N, K = W.shape
    Wg, u, v = torch.empty_like(W), torch.empty(N, device=W.device), torch.empty(N, device=W.device)
    _check(_lib.load().ppml_b200_layernorm_fold(_p(W), _p(gamma), _p(beta), _p(bias), _p(Wg), _p(u), _p(v), N, K, _stream()), "layernorm_fold")
    return Wg, u, v


def row_stats(x, eps=1e-5):
    x = _f32c(x)
    M, K = x.shape
    out = torch.empty((M, 2), device=x.device, dtype=torch.float32)
    _check(_lib.load().ppml_b200_row_stats(_p(x), _p(out), M, K, float(eps), _stream()), "row_stats")
    return out


def mul_mat_fused(A, B, bias=None, ln_stats=None, ln_u=None, gate=None, act="none", path=PATH_AUTO, tf32_mode=TF32_TMA, out=None):
    """A Linear with LayerNorm folded in front (ln_stats from row_stats(A), B / bias / ln_u from layernorm_fold) and / or an
    activation gate behind (act(out) * gate)."""
    A, B = _f32c(A), _f32c(B)
    M, K = A.shape
    N = B.shape[0]
    Cout = out if out is not None else torch.empty((M, N), device=A.device, dtype=torch.float32)
    rc = _lib.load().ppml_b200_mul_mat_f32_fused(_p(A), _p(B), _p(Cout), M, K, N, _p(bias), _p(ln_stats), _p(ln_u), _p(gate), ACT[act],
                                                 path, tf32_mode, _stream())
    _check(rc, "mul_mat_f32_fused")
    return Cout


def mul_mat_16(A16, B16, bias=None, path=PATH_AUTO, out=None):
    """16-bit operands (torch.float16 or torch.bfloat16), fp32 output; replaces the mul_mat_*f16* launchers."""
    assert A16.dtype == B16.dtype and A16.dtype in (torch.float16, torch.bfloat16)
    A16, B16 = A16.contiguous(), B16.contiguous()
    M, K = A16.shape
    N = B16.shape[0]
    Cout = out if out is not None else torch.empty((M, N), device=A16.device, dtype=torch.float32)
    fn = _lib.load().ppml_b200_mul_mat_f16 if A16.dtype == torch.float16 else _lib.load().ppml_b200_mul_mat_bf16
    _check(fn(_p(A16), _p(B16), _p(Cout), M, K, N, _p(bias), path, _stream()), "mul_mat_16")
    return Cout


def mul_mat_f32_as_bf16(A, B, bias=None, path=PATH_AUTO, out=None):
    """fp32 tensors, bf16 products (activations cast into library scratch, weights into a cached bf16 copy)."""
    A, B = _f32c(A), _f32c(B)
    M, K = A.shape
    N = B.shape[0]
    Cout = out if out is not None else torch.empty((M, N), device=A.device, dtype=torch.float32)
    rc = _lib.load().ppml_b200_mul_mat_f32_as_bf16(_p(A), _p(B), _p(Cout), M, K, N, _p(bias), path, _stream())
    _check(rc, "mul_mat_f32_as_bf16")
    return Cout


def bf16_shadow_invalidate(B=None):
    _lib.load().ppml_b200_bf16_shadow_invalidate(_p(B))


def cast(x, dtype):
    x = _f32c(x)
    y = torch.empty(x.shape, device=x.device, dtype=dtype)
    fn = _lib.load().ppml_b200_cast_f32_to_f16 if dtype == torch.float16 else _lib.load().ppml_b200_cast_f32_to_bf16
    _check(fn(_p(x), _p(y), x.numel(), _stream()), "cast")
    return y


def quantize_q8_0r(W):
    """fp32 weights [M,K] (device) -> planar Q8_0R bytes (device uint8), K % 32 == 0."""
    W = _f32c(W)
    out = torch.empty(W.numel() // 32 * 34, device=W.device, dtype=torch.uint8)
    _check(_lib.load().ppml_b200_quantize_q8_0r(_p(W), _p(out), W.numel(), _stream()), "quantize_q8_0r")
    return out


def quantize_q8_0_host(w):
    """numpy fp32 -> 34-byte Q8_0 blocks (host)."""
    w = np.ascontiguousarray(w, np.float32)
    out = np.empty(w.size // 32 * 34, np.uint8)
    _check(_lib.load().ppml_b200_quantize_q8_0_host(w.ctypes.data, out.ctypes.data, w.size), "quantize_q8_0_host")
    return out


def repack_q8_0_host(blocks):
    nb = blocks.size // 34
    out = np.empty(nb * 34, np.uint8)
    _check(_lib.load().ppml_b200_repack_q8_0_host(blocks.ctypes.data, nb, out.ctypes.data), "repack_q8_0_host")
    return out


def quantize_rows_q8_1_cuda(x):
    x = _f32c(x)
    out = torch.empty(x.numel() // 32 * 36, device=x.device, dtype=torch.uint8)
    _check(_lib.load().ppml_b200_quantize_rows_q8_1(_p(x), _p(out), x.numel(), _stream()), "quantize_rows_q8_1")
    return out


def dequantize_q8_cuda(blocks, kind):
    bs = 34 if kind == 0 else 36
    ne = blocks.numel() // bs * 32
    y = torch.empty(ne, device=blocks.device, dtype=torch.float32)
    fn = _lib.load().ppml_b200_dequantize_q8_0 if kind == 0 else _lib.load().ppml_b200_dequantize_q8_1
    _check(fn(_p(blocks), _p(y), ne, _stream()), "dequantize")
    return y


def mul_mat_q8_cuda(W, X, M, wtype=2, c_trans=1, bias=None, path=PATH_AUTO, want_sumi=False, out=None):
    """W: quantized weight bytes (device uint8), M rows of K; X fp32 [N,K].  Returns C ([N,M] if c_trans
    else [M,N]), the path taken (1 tensor cores / 0 dp4a) and, if asked, the int32 block sums [N,M,K/32]."""
    X = _f32c(X)
    N, K = X.shape
    Cout = out if out is not None else torch.empty((N, M) if c_trans else (M, N), device=X.device, dtype=torch.float32)
    sumi = torch.empty((N, M, K // 32), device=X.device, dtype=torch.int32) if want_sumi else None
    taken = C.c_int(0)
    rc = _lib.load().ppml_b200_mul_mat_q8(_p(W), _p(X), _p(Cout), M, N, K, wtype, c_trans, _p(bias), _p(sumi), path,
                                          C.byref(taken), _stream())
    _check(rc, "mul_mat_q8")
    return (Cout, taken.value, sumi) if want_sumi else (Cout, taken.value)


def mul_mat_q8_noalloc(W, X, M, wtype=2, c_trans=1, bias=None, out=None):
    """Same product as mul_mat_q8_cuda(path=PATH_SIMT), for callers that must not allocate device memory:
    the quantized activations use a fixed 4 MiB array inside the library.  Raises (status 9) when
    N * (K / 32) * 36 bytes do not fit.  `out` lets the caller pass its own result buffer."""
    X = _f32c(X)
    N, K = X.shape
    Cout = out if out is not None else torch.empty((N, M) if c_trans else (M, N), device=X.device, dtype=torch.float32)
    rc = _lib.load().ppml_b200_mul_mat_q8_noalloc(_p(W), _p(X), _p(Cout), M, N, K, wtype, c_trans, _p(bias), _stream())
    _check(rc, "mul_mat_q8_noalloc")
    return Cout


def flash_attn_forward_cuda(Q, K, V, bias=None, scale=0.0, causal=False, eps=1e-9, bias_bcast=False, path=PATH_AUTO, out=None,
                            Bc=64):
    """Q [B,h,L,d], K/V [B,h,Lk,d], bias [B,h,L,Lk] (or [h,L,Lk] shared over B with bias_bcast).
    Returns (O, LSE).  Lk != L and bias_bcast go through the extended entry.  `out` is an optional contiguous
    fp32 destination of Q's shape (any 16-byte-aligned address).  Bc: the reference's key tile (a row whose first
    Bc scores are all -inf gives zeros, as in the reference); Bc < 0 switches that rule off."""
    half = Q.dtype in (torch.float16, torch.bfloat16)         # 16-bit Q/K/V: fp32 softmax, bias, output
    if half:
        assert K.dtype == Q.dtype and V.dtype == Q.dtype
        Q, K, V = Q.contiguous(), K.contiguous(), V.contiguous()
    else:
        Q, K, V = _f32c(Q), _f32c(K), _f32c(V)
    B, h, L, d = Q.shape
    Lk = K.shape[2]
    O = torch.empty(Q.shape, device=Q.device, dtype=torch.float32) if out is None else out
    assert O.is_contiguous() and O.dtype == torch.float32 and O.shape == Q.shape
    LSE = torch.empty((B, h, L), device=Q.device, dtype=torch.float32)
    cfg = FlashCfg(B, h, L, d, int(causal), float(scale), float(eps), 64, int(Bc))
    lib = _lib.load()
    if bias is not None:
        bias = _f32c(bias)
    stride = 0 if (bias is None or bias_bcast) else h * L * Lk
    if half:
        rc = lib.ppml_b200_flash_attn_forward_16(C.byref(cfg), Lk, stride, _p(Q), _p(K), _p(V), _p(bias), _p(O), _p(LSE),
                                                 int(Q.dtype == torch.bfloat16), path, _stream())
    elif Lk == L and not bias_bcast:
        rc = lib.ppml_b200_flash_attn_forward(C.byref(cfg), _p(Q), _p(K), _p(V), _p(bias), _p(O), _p(LSE), path, _stream())
    else:
        rc = lib.ppml_b200_flash_attn_forward_ex(C.byref(cfg), Lk, stride, _p(Q), _p(K), _p(V), _p(bias), _p(O), _p(LSE),
                                                 path, _stream())
    _check(rc, "flash_attn_forward")
    return O, LSE


def flash_attn_tokens(Q, K, V, heads, bias=None, gate=None, act="sigmoid", scale=0.0, causal=False, eps=1e-9, bias_bcast=False,
                      path=PATH_AUTO, out=None, Bc=64):
    """Attention on token-major operands: Q [B, L, >= heads*d] (a column range of a wider tensor is fine: the row stride is
    taken from the tensor), K / V [B, Lk, ...]; O [B, L, heads*d] token-major; gate (optional, O's shape): act(gate) * O.
    Returns (O, LSE [B, heads, L])."""
    B, L, _ = Q.shape
    Lk = K.shape[1]
    assert Q.stride(2) == 1 and K.stride(2) == 1 and V.stride(2) == 1 and K.stride(1) == V.stride(1)
    d = (out.shape[2] if out is not None else (gate.shape[2] if gate is not None else Q.shape[2])) // heads
    hd = heads * d
    O = torch.empty((B, L, hd), device=Q.device, dtype=torch.float32) if out is None else out
    assert Q.stride(0) == Q.stride(1) * L and K.stride(0) == K.stride(1) * Lk and V.stride(0) == V.stride(1) * Lk
    assert O.stride(2) == 1 and O.stride(0) == O.stride(1) * L
    ld_g = 0
    if gate is not None:
        assert gate.stride(2) == 1 and gate.stride(0) == gate.stride(1) * L
        ld_g = gate.stride(1)
    LSE = torch.empty((B, heads, L), device=Q.device, dtype=torch.float32)
    cfg = FlashCfg(B, heads, L, d, int(causal), float(scale), float(eps), 64, int(Bc))
    if bias is not None:
        bias = _f32c(bias)
    stride = 0 if (bias is None or bias_bcast) else heads * L * Lk
    rc = _lib.load().ppml_b200_flash_attn_forward_tokens(C.byref(cfg), Lk, stride, _p(Q), _p(K), _p(V), Q.stride(1), K.stride(1), _p(bias),
                                                        _p(gate), ld_g, ACT[act], _p(O), O.stride(1), _p(LSE), path, _stream())
    _check(rc, "flash_attn_forward_tokens")
    return O, LSE


def flash_attn_backward_cuda(Q, K, V, O, dO, LSE, bias=None, scale=0.0, causal=False, bias_bcast=False,
                             want=("dQ", "dK", "dV", "dbias"), out=None):
    """Gradients of the fused attention: Q, K, V, O, dO [B, h, L, d], LSE [B, h, L], bias [B, h, L, L] (or [h, L, L] with
    bias_bcast).  Returns a dict with the requested ones of dQ, dK, dV [B, h, L, d] and dbias [B, h, L, L] (`out`: a dict
    of tensors to write into instead of new ones)."""
    Q, K, V, O, dO, LSE = (_f32c(t) for t in (Q, K, V, O, dO, LSE))
    B, h, L, d = Q.shape
    if bias is not None:
        bias = _f32c(bias)
    if out is None:
        out = {}
        for name in want:
            shape = (B, h, L, L) if name == "dbias" else (B, h, L, d)
            out[name] = torch.full(shape, float("nan"), device=Q.device, dtype=torch.float32)
    cfg = FlashCfg(B, h, L, d, int(causal), float(scale), 1e-9, 64, 64)
    stride = 0 if (bias is None or bias_bcast) else h * L * L
    rc = _lib.load().ppml_b200_flash_attn_backward(C.byref(cfg), stride, _p(Q), _p(K), _p(V), _p(bias), _p(O), _p(dO), _p(LSE),
                                                   _p(out.get("dQ")), _p(out.get("dK")), _p(out.get("dV")), _p(out.get("dbias")),
                                                   _stream())
    _check(rc, "flash_attn_backward")
    return out


def out_prod_cuda(s0, s1, path=PATH_AUTO):
    """s0 [ne03,ne02,K,ne00], s1 [ne13,ne12,K,ne10] (torch order = reversed graph dims) -> [ne3,ne2,ne10,ne00]."""
    s0, s1 = _f32c(s0), _f32c(s1)
    ne03, ne02, ne01, ne00 = s0.shape
    ne13, ne12, ne11, ne10 = s1.shape
    ne2, ne3 = max(ne02, ne12), max(ne03, ne13)
    dst = torch.empty((ne3, ne2, ne10, ne00), device=s0.device, dtype=torch.float32)
    rc = _lib.load().ppml_b200_out_prod(_p(s0), _p(s1), _p(dst), ne00, ne01, ne02, ne03, ne10, ne11, ne12, ne13,
                                        ne00, ne10, ne2, ne3, path, _stream())
    _check(rc, "out_prod")
    return dst


def tri_mul_cuda(left, right, L, outgoing, path=PATH_AUTO):
    """Flat layout, D outermost, B innermost: outgoing left [D,I,K,B], right [D,J,K,B]; incoming left
    [D,K,I,B], right [D,K,J,B] -> dst [D,I,J,B]."""
    half = left.dtype in (torch.float16, torch.bfloat16)      # 16-bit operands: fp32 accumulation and output
    if half:
        assert right.dtype == left.dtype
        left, right = left.contiguous(), right.contiguous()
    else:
        left, right = _f32c(left), _f32c(right)
    if outgoing:
        D, I, K, B = left.shape
        J = right.shape[1]
    else:
        D, K, I, B = left.shape
        J = right.shape[2]
    dst = torch.empty((D, I, J, B), device=left.device, dtype=torch.float32)
    if half:
        rc = _lib.load().ppml_b200_tri_mul_16(_p(left), _p(right), _p(dst), D, I, J, K, B, 1.0 / float(L), int(bool(outgoing)),
                                              int(left.dtype == torch.bfloat16), path, _stream())
    else:
        rc = _lib.load().ppml_b200_tri_mul(_p(left), _p(right), _p(dst), D, I, J, K, B, 1.0 / float(L), int(bool(outgoing)),
                                           path, _stream())
    _check(rc, "tri_mul")
    return dst


def outer_prod_mean_cuda(left, right, path=PATH_AUTO):
    """left/right flat [D,L,N,B] -> [D*D, L, L, B], mean over N."""
    half = left.dtype in (torch.float16, torch.bfloat16)      # 16-bit operands: fp32 accumulation and output
    if half:
        assert right.dtype == left.dtype
        left, right = left.contiguous(), right.contiguous()
    else:
        left, right = _f32c(left), _f32c(right)
    D, L, N, B = left.shape
    dst = torch.empty((D * D, L, L, B), device=left.device, dtype=torch.float32)
    if half:
        rc = _lib.load().ppml_b200_outer_prod_mean_16(_p(left), _p(right), _p(dst), D, L, N, B, 1.0 / float(N),
                                                      int(left.dtype == torch.bfloat16), path, _stream())
    else:
        rc = _lib.load().ppml_b200_outer_prod_mean(_p(left), _p(right), _p(dst), D, L, N, B, 1.0 / float(N), path, _stream())
    _check(rc, "outer_prod_mean")
    return dst


def outer_prod_mean_slabs_cuda(left_slabs, right, path=PATH_AUTO, out=None):
    """One rank's share of the outer-product-mean: left_slabs [D_left,L,N,B] (a contiguous d1 range), right
    [D,L,N,B] (all of it) -> [D_left*D, L, L, B], the rank's contiguous part of the full result."""
    left_slabs, right = _f32c(left_slabs), _f32c(right)
    D1, L, N, B = left_slabs.shape
    D = right.shape[0]
    assert right.shape[1:] == left_slabs.shape[1:]
    dst = torch.empty((D1 * D, L, L, B), device=right.device, dtype=torch.float32) if out is None else out
    rc = _lib.load().ppml_b200_outer_prod_mean_slabs(_p(left_slabs), _p(right), _p(dst), D1, D, L, N, B, 1.0 / float(N),
                                                     path, _stream())
    _check(rc, "outer_prod_mean_slabs")
    return dst
