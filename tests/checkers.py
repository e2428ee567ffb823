"""ctypes bindings of the two CPU checkers used by the tests, the smoke check and the CPU-baseline
leg of the benchmark: the C restatement (oracle/ppml_oracle.c) and, where it was built, the
reference's own CPU sources behind oracle/ref_harness.cpp (oracle/_ref/libppml_ref.so).

Test infrastructure: the product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_ORACLE_SO = os.path.join(_ROOT, "oracle", "libppml_oracle.so")
_REF_SO = os.path.join(_ROOT, "oracle", "_ref", "libppml_ref.so")

_f32p = C.POINTER(C.c_float)
_i64 = C.c_int64


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def build_oracle():
    subprocess.check_call(["make", "-s", "-C", os.path.join(_ROOT, "oracle"), "oracle"])


def load_oracle():
    if not os.path.exists(_ORACLE_SO):
        build_oracle()
    return C.CDLL(_ORACLE_SO)


def have_ref():
    return os.path.exists(_REF_SO)


def load_ref():
    return C.CDLL(_REF_SO)


class Oracle:
    """numpy front end of oracle/ppml_oracle.c."""

    def __init__(self):
        self.lib = load_oracle()
        L = self.lib
        L.oracle_f32_to_f16.restype = C.c_uint16
        L.oracle_f32_to_f16.argtypes = [C.c_float]
        L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f32_to_bf16.restype = C.c_uint16
        L.oracle_f32_to_bf16.argtypes = [C.c_float]
        L.oracle_mul_mat_q8.restype = C.c_int
        L.oracle_flash_attn_forward.restype = C.c_int
        L.oracle_flash_attn_backward.restype = C.c_int

    def mul_mat_f32(self, a, b, bias=None):
        a, b, bias = _f32(a), _f32(b), _f32(bias)
        M, K = a.shape
        N = b.shape[0]
        c = np.empty((M, N), np.float32)
        self.lib.oracle_mul_mat_f32(_ptr(a), _ptr(b), _ptr(bias), _ptr(c), M, K, N)
        return c

    def mul_mat_16(self, a16, b16, bias=None, kind="f16"):
        a16 = np.ascontiguousarray(a16, np.uint16)
        b16 = np.ascontiguousarray(b16, np.uint16)
        bias = _f32(bias)
        M, K = a16.shape
        N = b16.shape[0]
        c = np.empty((M, N), np.float32)
        fn = self.lib.oracle_mul_mat_f16 if kind == "f16" else self.lib.oracle_mul_mat_bf16
        fn(_ptr(a16), _ptr(b16), _ptr(bias), _ptr(c), M, K, N)
        return c

    def out_prod(self, s0, s1):
        """s0 [ne03,ne02,K,ne00], s1 [ne13,ne12,K,ne10] (numpy order = reversed ggml dims)."""
        s0, s1 = _f32(s0), _f32(s1)
        ne03, ne02, ne01, ne00 = s0.shape
        ne13, ne12, ne11, ne10 = s1.shape
        ne2, ne3 = max(ne02, ne12), max(ne03, ne13)
        dst = np.empty((ne3, ne2, ne10, ne00), np.float32)
        self.lib.oracle_out_prod(_ptr(s0), _ptr(s1), _ptr(dst),
                                 _i64(ne00), _i64(ne01), _i64(ne02), _i64(ne03),
                                 _i64(ne10), _i64(ne11), _i64(ne12), _i64(ne13),
                                 _i64(ne00), _i64(ne10), _i64(ne2), _i64(ne3))
        return dst

    def tri_mul(self, left, right, L, outgoing, B=1):
        """flat layout: outgoing left [D,I,K,B] right [D,J,K,B]; incoming left [D,K,I,B] right [D,K,J,B]
        (numpy order, D outermost)."""
        left, right = _f32(left), _f32(right)
        if outgoing:
            D, I, K = left.shape[:3]
            J = right.shape[1]
        else:
            D, K, I = left.shape[:3]
            J = right.shape[2]
        dst = np.empty((D, I, J, B), np.float32)
        self.lib.oracle_tri_mul(_ptr(left), _ptr(right), _ptr(dst), _i64(D), _i64(I), _i64(J), _i64(K),
                                _i64(B), C.c_float(L), int(bool(outgoing)))
        return dst

    def outer_prod_mean(self, left, right, B=1):
        """left/right flat [D,L,N,B] (numpy order) -> [D*D, L, L, B]."""
        left, right = _f32(left), _f32(right)
        D, L, N = left.shape[:3]
        dst = np.empty((D * D, L, L, B), np.float32)
        self.lib.oracle_outer_prod_mean(_ptr(left), _ptr(right), _ptr(dst), _i64(D), _i64(L), _i64(N), _i64(B))
        return dst

    def flash_attn(self, Q, K, V, bias=None, scale=0.0, causal=False, eps=1e-9, Bc=64, bias_bcast=False):
        """Q [B,h,L,d], K/V [B,h,Lk,d], bias [B,h,L,Lk] (or [h,L,Lk] with bias_bcast)."""
        Q, K, V, bias = _f32(Q), _f32(K), _f32(V), _f32(bias)
        B, h, L, d = Q.shape
        Lk = K.shape[2]
        O = np.empty_like(Q)
        LSE = np.empty((B, h, L), np.float32)
        stride = 0 if (bias is None or bias_bcast) else h * L * Lk
        ok = self.lib.oracle_flash_attn_forward(B, h, L, Lk, d, int(causal), C.c_float(scale), C.c_float(eps),
                                                Bc, _ptr(Q), _ptr(K), _ptr(V), _ptr(bias), _i64(stride),
                                                _ptr(O), _ptr(LSE))
        assert ok
        return O, LSE

    def flash_attn_backward(self, Q, K, V, O, dO, LSE, bias=None, scale=0.0, causal=False, bias_bcast=False,
                            want=("dQ", "dK", "dV", "dbias")):
        """Q, K, V, O, dO [B,h,L,d], LSE [B,h,L], bias [B,h,L,L] (or [h,L,L] with bias_bcast) -> dict of gradients."""
        Q, K, V, O, dO, LSE, bias = (_f32(t) for t in (Q, K, V, O, dO, LSE, bias))
        B, h, L, d = Q.shape
        out = {n: np.full((B, h, L, L) if n == "dbias" else (B, h, L, d), np.nan, np.float32) for n in want}
        stride = 0 if (bias is None or bias_bcast) else h * L * L
        ok = self.lib.oracle_flash_attn_backward(B, h, L, d, int(causal), C.c_float(scale), _ptr(Q), _ptr(K), _ptr(V), _ptr(bias),
                                                 _i64(stride), _ptr(O), _ptr(dO), _ptr(LSE), _ptr(out.get("dQ")),
                                                 _ptr(out.get("dK")), _ptr(out.get("dV")), _ptr(out.get("dbias")))
        assert ok
        return out

    def attention_legacy(self, Q, K, V, bias, scale, bias_bcast=False):
        Q, K, V, bias = _f32(Q), _f32(K), _f32(V), _f32(bias)
        B, h, Lq, d = Q.shape
        Lk = K.shape[2]
        O = np.empty_like(Q)
        stride = 0 if (bias is None or bias_bcast) else h * Lq * Lk
        self.lib.oracle_attention_legacy(B, h, Lq, Lk, d, C.c_float(scale), _ptr(Q), _ptr(K), _ptr(V),
                                         _ptr(bias), _i64(stride), _ptr(O))
        return O

    def quantize_q8_0(self, x):
        x = _f32(x)
        out = np.empty(x.size // 32 * 34, np.uint8)
        assert self.lib.oracle_quantize_q8_0(_ptr(x), _ptr(out), _i64(x.size))
        return out

    def quantize_q8_1(self, x):
        x = _f32(x)
        out = np.empty(x.size // 32 * 36, np.uint8)
        assert self.lib.oracle_quantize_q8_1(_ptr(x), _ptr(out), _i64(x.size))
        return out

    def repack_q8_0(self, blocks):
        nb = blocks.size // 34
        out = np.empty(nb * 34, np.uint8)
        self.lib.oracle_repack_q8_0(_ptr(blocks), _i64(nb), _ptr(out))
        return out

    def dequantize(self, blocks, kind):
        bs = 34 if kind == 0 else 36
        nb = blocks.size // bs
        out = np.empty(nb * 32, np.float32)
        (self.lib.oracle_dequantize_q8_0 if kind == 0 else self.lib.oracle_dequantize_q8_1)(
            _ptr(blocks), _ptr(out), _i64(nb * 32))
        return out

    def mul_mat_q8(self, W, X, M, wtype=2, c_trans=1, bias=None, want_sumi=False):
        """W: packed weight bytes (M rows of K), X [N,K] fp32 -> C ([N,M] if c_trans else [M,N])."""
        X, bias = _f32(X), _f32(bias)
        N, K = X.shape
        Cout = np.empty((N, M) if c_trans else (M, N), np.float32)
        sumi = np.empty((N, M, K // 32), np.int32) if want_sumi else None
        rc = self.lib.oracle_mul_mat_q8(_ptr(W), _ptr(X), _ptr(Cout), M, N, K, wtype, c_trans, _ptr(bias), _ptr(sumi))
        assert rc == 0, rc
        return (Cout, sumi) if want_sumi else Cout


def layer_norm_f32(x, gamma, beta, eps):
    """LayerNorm::forward of the reference (src/model/Embedding.cpp:268-289): OP_NORM along the feature axis
    (src/backend/CPUKernels.cpp:1498-1512: mean, mean of squared differences, 1 / sqrt(var + eps), all in fp32 and in
    this order), then * gamma + beta."""
    x = np.asarray(x, np.float32)
    D = np.float32(x.shape[1])
    mean = (np.add.reduce(x, axis=1, dtype=np.float32) / D).astype(np.float32)
    diff = (x - mean[:, None]).astype(np.float32)
    var = (np.add.reduce(diff * diff, axis=1, dtype=np.float32) / D).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt(var + np.float32(eps))).astype(np.float32)
    return ((diff * inv[:, None]) * np.asarray(gamma, np.float32) + np.asarray(beta, np.float32)).astype(np.float32)


def act_mul_f32(x, g, kind):
    """OP_ACT_MUL (src/backend/CPUKernels.cpp:1903-1916, :1947-1967): act(x) * g with the reference's formulas in fp32."""
    x = np.asarray(x, np.float32)
    one = np.float32(1.0)
    if kind == "sigmoid":
        a = one / (one + np.exp(-x))
    elif kind == "silu":
        a = x / (one + np.exp(-x))
    elif kind == "gelu":
        a = np.float32(0.5) * x * (one + np.tanh(np.float32(np.sqrt(2.0 / np.pi)) * (x + np.float32(0.044715) * x * x * x)))
    elif kind == "tanh":
        a = np.tanh(x)
    elif kind == "relu":
        a = np.maximum(x, np.float32(0.0))
    else:
        a = x
    return (a.astype(np.float32) * np.asarray(g, np.float32)).astype(np.float32)


class Ref:
    """numpy front end of the reference's own CPU implementation (oracle/_ref/libppml_ref.so)."""

    def __init__(self, n_threads=1):
        self.lib = load_ref()
        self.nt = n_threads

    def mul_mat(self, a, b, bias=None, f16=False):
        if f16:
            a = np.ascontiguousarray(a, np.uint16)
            b = np.ascontiguousarray(b, np.uint16)
        else:
            a, b = _f32(a), _f32(b)
        bias = _f32(bias)
        M, K = a.shape
        N = b.shape[0]
        c = np.empty((M, N), np.float32)
        rc = self.lib.ref_mul_mat(_ptr(a), _ptr(b), _ptr(bias), _ptr(c), M, K, N, int(f16), self.nt)
        assert rc == 0
        return c

    def out_prod(self, s0, s1):
        s0, s1 = _f32(s0), _f32(s1)
        ne03, ne02, ne01, ne00 = s0.shape
        ne13, ne12, ne11, ne10 = s1.shape
        dst = np.empty((max(ne03, ne13), max(ne02, ne12), ne10, ne00), np.float32)
        rc = self.lib.ref_out_prod(_ptr(s0), _ptr(s1), _ptr(dst), _i64(ne00), _i64(ne01), _i64(ne02), _i64(ne03),
                                   _i64(ne10), _i64(ne11), _i64(ne12), _i64(ne13), self.nt)
        assert rc == 0
        return dst

    def tri_mul(self, left, right, L, outgoing, B=1):
        left, right = _f32(left), _f32(right)
        if outgoing:
            D, I, K = left.shape[:3]
            J = right.shape[1]
        else:
            D, K, I = left.shape[:3]
            J = right.shape[2]
        dst = np.empty((D, I, J, B), np.float32)
        # the graph passes dims in ggml order [d0..d3] = (D, I|K, K|I, B): the harness rebuilds them
        rc = self.lib.ref_tri_mul(_ptr(left), _ptr(right), _ptr(dst), _i64(D), _i64(I), _i64(J), _i64(K), _i64(B),
                                  C.c_float(L), int(bool(outgoing)), self.nt)
        assert rc == 0
        return dst

    def outer_prod_mean(self, left, right, B=1):
        left, right = _f32(left), _f32(right)
        D, L, N = left.shape[:3]
        dst = np.empty((D * D, L, L, B), np.float32)
        rc = self.lib.ref_outer_prod_mean(_ptr(left), _ptr(right), _ptr(dst), _i64(D), _i64(L), _i64(N), _i64(B), self.nt)
        assert rc == 0
        return dst

    def flash_attn(self, Q, K, V, bias=None, scale=0.0, causal=False, eps=1e-9, Bc=64, naive=False):
        Q, K, V, bias = _f32(Q), _f32(K), _f32(V), _f32(bias)
        B, h, L, d = Q.shape
        O = np.empty_like(Q)
        LSE = np.empty((B, h, L), np.float32)
        rc = self.lib.ref_flash_attn_forward(B, h, L, d, int(causal), C.c_float(scale), C.c_float(eps), Bc,
                                             _ptr(Q), _ptr(K), _ptr(V), _ptr(bias), _ptr(O), _ptr(LSE), int(naive))
        assert rc == 0
        return O, LSE

    def flash_attn_backward(self, Q, K, V, O, dO, LSE, bias=None, scale=0.0, causal=False):
        Q, K, V, O, dO, LSE, bias = (_f32(t) for t in (Q, K, V, O, dO, LSE, bias))
        B, h, L, d = Q.shape
        out = {n: np.empty((B, h, L, L) if n == "dbias" else (B, h, L, d), np.float32) for n in ("dQ", "dK", "dV", "dbias")}
        rc = self.lib.ref_flash_attn_backward(B, h, L, d, int(causal), C.c_float(scale), C.c_float(1e-9), _ptr(Q), _ptr(K), _ptr(V),
                                              _ptr(bias), _ptr(O), _ptr(dO), _ptr(LSE), _ptr(out["dQ"]), _ptr(out["dK"]),
                                              _ptr(out["dV"]), _ptr(out["dbias"]))
        assert rc == 0
        return out

    def attention_legacy(self, Q, K, V, bias, scale):
        """Q [B,h,Lq,d] etc. in the fused op's layout; transposed here into the unfused graph's
        sequence-innermost layout and back."""
        Q, K, V, bias = _f32(Q), _f32(K), _f32(V), _f32(bias)
        B, h, Lq, d = Q.shape
        Lk = K.shape[2]
        q = np.ascontiguousarray(Q.transpose(0, 1, 3, 2))
        k = np.ascontiguousarray(K.transpose(0, 1, 3, 2))
        v = np.ascontiguousarray(V.transpose(0, 1, 3, 2))
        o = np.empty((B, h, d, Lq), np.float32)
        rc = self.lib.ref_attention_legacy(_ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(o), _i64(Lq), _i64(Lk),
                                           _i64(d), _i64(h), _i64(B), C.c_float(scale), self.nt)
        assert rc == 0
        return np.ascontiguousarray(o.transpose(0, 1, 3, 2))

    def quantize_q8_0(self, x):
        x = _f32(x)
        out = np.empty(x.size // 32 * 34, np.uint8)
        assert self.lib.ref_quantize_q8_0(_ptr(x), _ptr(out), _i64(x.size)) == 0
        return out

    def quantize_q8_1(self, x):
        x = _f32(x)
        out = np.empty(x.size // 32 * 36, np.uint8)
        assert self.lib.ref_quantize_q8_1(_ptr(x), _ptr(out), _i64(x.size)) == 0
        return out

    def repack_q8_0(self, blocks):
        nb = blocks.size // 34
        out = np.empty(nb * 34, np.uint8)
        self.lib.ref_repack_q8_0(_ptr(blocks), _i64(nb), _ptr(out))
        return out

    def dequantize(self, blocks, kind):
        bs = 34 if kind == 0 else 36
        nb = blocks.size // bs
        out = np.empty(nb * 32, np.float32)
        (self.lib.ref_dequantize_q8_0 if kind == 0 else self.lib.ref_dequantize_q8_1)(_ptr(blocks), _ptr(out), _i64(nb * 32))
        return out


def check_block_calls(trace, oracle, heads=8):
    """Every call a traced block made (proteinpredictmachinelearning_b200.block_bench.Block with trace=True) against the
    CPU checker on the very tensors the call saw.  Returns one dict per call: op, tag, shape, us (the call's own CUDA-event
    time), err (normalised max error)."""
    host = lambda t: None if t is None else t.detach().float().cpu().numpy()

    def rel(got, ref):
        return float(np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))

    out = []
    for c in trace:
        op, got = c["op"], host(c["out"])
        if op == "mul_mat":
            x, w = host(c["x"]), host(c["w"])
            ref = oracle.mul_mat_f32(x, w, host(c["bias"]))
            shape = f"M={x.shape[0]} K={x.shape[1]} N={w.shape[0]}"
        elif op == "mul_mat_q8":
            x = host(c["x"])
            wq = c["w"].detach().cpu().numpy()
            n_out = got.shape[1]
            ref = oracle.mul_mat_q8(wq, x, n_out, wtype=2, c_trans=1, bias=host(c["bias"]))
            shape = f"M={x.shape[0]} K={x.shape[1]} N={n_out} (Q8)"
        elif op in ("flash_attn", "flash_attn_tokens"):
            q, k, v, bias = host(c["q"]), host(c["k"]), host(c["v"]), host(c["bias"])
            if op == "flash_attn_tokens":                   # [B, L, h*d] token-major -> [B, h, L, d]
                split = lambda t: np.ascontiguousarray(t.reshape(t.shape[0], t.shape[1], heads, -1).transpose(0, 2, 1, 3))
                q, k, v = split(q), split(k), split(v)
            ref, _ = oracle.flash_attn(q, k, v, bias, scale=c["scale"], bias_bcast=bias is not None)
            if op == "flash_attn_tokens":
                ref = np.ascontiguousarray(ref.transpose(0, 2, 1, 3)).reshape(got.shape)
                if c.get("gate") is not None:
                    ref = act_mul_f32(host(c["gate"]), ref, "sigmoid")
            shape = f"B'={q.shape[0]} h={q.shape[1]} Lq={q.shape[2]} Lk={k.shape[2]} d={q.shape[3]}" + (", bias" if bias is not None else "")
        elif op == "tri_mul":
            left, right = host(c["left"]), host(c["right"])
            ref = oracle.tri_mul(left, right, float(left.shape[1]), c["outgoing"])
            shape = f"D={left.shape[0]} L={left.shape[1]} " + ("outgoing" if c["outgoing"] else "incoming")
        elif op == "outer_prod_mean":
            left, right = host(c["left"]), host(c["right"])
            ref = oracle.outer_prod_mean(left, right)
            shape = f"c={left.shape[0]} L={left.shape[1]} N={left.shape[2]}"
        else:
            raise ValueError(op)
        e0, e1 = c["events"]
        out.append({"op": op, "tag": c["tag"], "shape": shape, "us": e0.elapsed_time(e1) * 1e3, "err": rel(got, ref)})
    return out
