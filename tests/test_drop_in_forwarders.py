"""The C++ forwarders under the reference's own names, called the way the reference's dispatcher calls them.

oracle/forwarder_harness.cpp includes the reference's headers (FlashAttnConfig, the Q8 block types), declares the
launchers word for word as src/backend/CUDAKernels.cpp does and is linked against libppml_b200.so with
--no-undefined, so the mangled names, parameter types and the struct layout are the reference's, not a twin's.  It is
built where the reference tree is present (`make -C oracle drop_in`, done by __graft_entry__.build()) and travels as a
built library.  Every forwarder is called here on device buffers and checked against the CPU checker, in each
arithmetic mode the environment switches select (PPML_MUL_MAT_TC / PPML_B200_MATH)."""
import ctypes as C
import os

import numpy as np
import pytest

import cases

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

HARNESS = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libforwarder_harness.so")
TOL_FP32, TOL_TF32, TOL_16 = 1e-5, 1e-3, 1e-2


@pytest.fixture(scope="module")
def fh():
    if not os.path.exists(HARNESS):
        pytest.skip("oracle/_ref/libforwarder_harness.so not built (needs the reference tree: make -C oracle drop_in)")
    lib = C.CDLL(HARNESS)
    vp, i, i64, f = C.c_void_p, C.c_int, C.c_int64, C.c_float
    lib.fh_mul_mat_cuda.argtypes = [vp, vp, vp, i, i, i, vp]
    lib.fh_mul_mat_cuda.restype = None
    lib.fh_mul_mat_mma_tf32_smem.argtypes = [vp, vp, vp, i, i, i]
    lib.fh_mul_mat_f16.argtypes = [i, vp, vp, vp, i, i, i]
    lib.fh_mul_mat_q8_cuda.argtypes = [vp, vp, vp, i, i, i, i, i, vp, C.POINTER(i)]
    lib.fh_quantize_rows_q8_1.argtypes = [vp, vp, i64]
    lib.fh_dequantize_q8.argtypes = [i, vp, vp, i64]
    lib.fh_flash_attn_forward.argtypes = [i, i, i, i, i, f, f, vp, vp, vp, vp, vp, vp]
    lib.fh_flash_attn_backward.argtypes = [i, i, i, i, i, f] + [vp] * 11
    lib.fh_out_prod.argtypes = [vp, vp, vp, C.POINTER(i64), C.POINTER(i64), C.POINTER(i64)]
    lib.fh_out_prod.restype = None
    lib.fh_tri_mul.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, f, i]
    lib.fh_tri_mul.restype = None
    lib.fh_outer_prod_mean.argtypes = [vp, vp, vp, i64, i64, i64, i64, f]
    lib.fh_outer_prod_mean.restype = None
    lib.fh_hw_supported.argtypes = [C.POINTER(i), C.POINTER(i)]
    return lib


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.detach().cpu().numpy()


def p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


@pytest.fixture
def math_mode(monkeypatch):
    """Sets the arithmetic switch the forwarders read on every call."""
    def set_mode(mode):
        monkeypatch.delenv("PPML_MUL_MAT_TC", raising=False)
        monkeypatch.delenv("PPML_B200_MATH", raising=False)
        if mode == "tc":
            monkeypatch.setenv("PPML_MUL_MAT_TC", "1")          # the reference's own switch
        elif mode is not None:
            monkeypatch.setenv("PPML_B200_MATH", mode)
    return set_mode


def test_hw_probe_and_struct_size(fh):
    major, minor = C.c_int(0), C.c_int(0)
    assert fh.fh_hw_supported(C.byref(major), C.byref(minor)) == 1 and major.value == 10
    assert fh.fh_sizeof_flash_cfg() == 36          # 4 ints, bool + padding, 2 floats, 2 ints


@pytest.mark.parametrize("mode,tol", [(None, TOL_FP32), ("fp32", TOL_FP32), ("tc", TOL_TF32), ("tf32", TOL_TF32), ("bf16", TOL_16)])
@pytest.mark.parametrize("M,K,N", [(408, 256, 256), (255, 33, 32), (2601, 128, 8)])
def test_mul_mat_cuda_forwarder(fh, oracle, math_mode, mode, tol, M, K, N):
    """Default = exact fp32 as in the reference; tensor cores only when the switch asks for them (bias included)."""
    math_mode(mode)
    a, b, bi = cases.mul_mat_case(M, K, N, seed=1)
    A, B, Bi = dev(a), dev(b), dev(bi)
    for bias in (Bi, None):
        Cd = torch.zeros((M, N), device="cuda")
        torch.cuda.synchronize()
        fh.fh_mul_mat_cuda(p(A), p(B), p(Cd), M, K, N, p(bias))
        assert cases.rel_err(host(Cd), oracle.mul_mat_f32(a, b, bi if bias is not None else None)) <= tol
    if mode == "bf16":
        from proteinpredictmachinelearning_b200 import ops
        ops.bf16_shadow_invalidate(None)


def test_tensor_core_launchers(fh, oracle):
    a, b, _ = cases.mul_mat_case(408, 256, 256, seed=1, bias=False)
    A, B = dev(a), dev(b)
    Cd = torch.zeros((408, 256), device="cuda")
    torch.cuda.synchronize()
    assert fh.fh_mul_mat_mma_tf32_smem(p(A), p(B), p(Cd), 408, 256, 256) == 0
    assert cases.rel_err(host(Cd), oracle.mul_mat_f32(a, b)) <= TOL_TF32
    a33, b33, _ = cases.mul_mat_case(255, 33, 32, seed=1, bias=False)          # row pitch not a multiple of 16 bytes
    A33, B33 = dev(a33), dev(b33)
    assert fh.fh_mul_mat_mma_tf32_smem(p(A33), p(B33), p(Cd), 255, 33, 32) == 1      # caller falls back
    a16, b16 = A.half(), B.half()
    ref16 = oracle.mul_mat_16(host(a16.view(torch.int16)).view(np.uint16), host(b16.view(torch.int16)).view(np.uint16), None)
    for which in (0, 1, 2):
        Cd.zero_()
        torch.cuda.synchronize()
        assert fh.fh_mul_mat_f16(which, p(a16), p(b16), p(Cd), 408, 256, 256) == 0
        assert cases.rel_err(host(Cd), ref16) <= TOL_FP32


@pytest.mark.parametrize("with_bias", [False, True])
def test_q8_forwarders(fh, oracle, with_bias, monkeypatch):
    monkeypatch.setenv("PPML_MULMAT_STATS", "0")
    Mout, Ntok, K = 256, 408, 256
    w, x = cases.q8_case(Mout, Ntok, K, seed=2)
    W = oracle.repack_q8_0(oracle.quantize_q8_0(w))
    bias = (np.random.default_rng(3).standard_normal(Mout) * 0.1).astype(np.float32) if with_bias else None
    Cd = torch.zeros((Ntok, Mout), device="cuda")
    path = C.c_int(-1)
    torch.cuda.synchronize()
    Bd = None if bias is None else dev(bias)
    Wd, Xd = dev(W), dev(x)                     # keep every device buffer alive until the results have been read
    assert fh.fh_mul_mat_q8_cuda(p(Wd), p(Xd), p(Cd), Mout, Ntok, K, 2, 1, p(Bd), C.byref(path)) == 0
    assert path.value == 1                                                    # tensor cores
    assert cases.rel_err(host(Cd), oracle.mul_mat_q8(W, x, Mout, bias=bias)) <= TOL_FP32
    # the quantize / dequantize helpers
    q81 = torch.zeros(x.size // 32 * 36, dtype=torch.uint8, device="cuda")
    assert fh.fh_quantize_rows_q8_1(p(Xd), p(q81), x.size) == 0
    assert np.array_equal(host(q81), oracle.quantize_q8_1(x))
    y = torch.zeros(x.size, device="cuda")
    assert fh.fh_dequantize_q8(1, p(q81), p(y), x.size) == 0
    assert np.array_equal(host(y), oracle.dequantize(oracle.quantize_q8_1(x), 1))
    q80 = oracle.quantize_q8_0(w)
    yw = torch.zeros(w.size, device="cuda")
    Q80d = dev(q80)
    assert fh.fh_dequantize_q8(0, p(Q80d), p(yw), w.size) == 0
    assert np.array_equal(host(yw), oracle.dequantize(q80, 0))


@pytest.mark.parametrize("mode,tol,ltol", [(None, TOL_FP32, 1e-5), ("tc", TOL_TF32, 2e-3)])
@pytest.mark.parametrize("causal", [False, True])
def test_flash_attn_forwarder_takes_the_reference_struct(fh, oracle, math_mode, mode, tol, ltol, causal):
    """FlashAttnConfig has a bool between ints and floats: every field after it must land where the library reads it."""
    math_mode(mode)
    B, h, L, d = 3, 2, 132, 32
    Q, K, V, bi = cases.attn_case(B, h, L, d, seed=3)
    O = torch.zeros((B, h, L, d), device="cuda")
    LSE = torch.zeros((B, h, L), device="cuda")
    scale, eps = 0.21, 1e-6                     # not the defaults: both must reach the kernel
    torch.cuda.synchronize()
    Qd, Kd, Vd, Bd = dev(Q), dev(K), dev(V), dev(bi)
    rc = fh.fh_flash_attn_forward(B, h, L, d, int(causal), scale, eps, p(Qd), p(Kd), p(Vd), p(Bd), p(O), p(LSE))
    assert rc == 0
    rO, rL = oracle.flash_attn(Q, K, V, bi, scale=scale, causal=causal, eps=eps)
    assert cases.rel_err(host(O), rO) <= tol
    assert np.abs(host(LSE) - rL).max() <= ltol


def test_flash_attn_backward_forwarder(fh, oracle):
    """flash_attn_backward_cuda as the reference's dispatcher declares it (src/backend/CUDAKernels.cpp:176): full bias
    [B, h, L, L], every gradient, then with dbias and dK left out (null pointers are skipped)."""
    B, h, L, d = 2, 3, 77, 32
    Q, K, V, bi, dO = cases.attn_backward_case(B, h, L, d, seed=12, masked_rows=(4,))
    scale = 0.19
    rO, rL = oracle.flash_attn(Q, K, V, bi, scale=scale)
    ref = oracle.flash_attn_backward(Q, K, V, rO, dO, rL, bi, scale=scale)
    t = [dev(x) for x in (Q, K, V, bi, rO, dO, rL)]
    g = {n: torch.full((B, h, L, L) if n == "dbias" else (B, h, L, d), float("nan"), device="cuda") for n in ("dQ", "dK", "dV", "dbias")}
    torch.cuda.synchronize()
    rc = fh.fh_flash_attn_backward(B, h, L, d, 0, scale, *[p(x) for x in t], p(g["dQ"]), p(g["dK"]), p(g["dV"]), p(g["dbias"]))
    assert rc == 0
    for n in g:
        assert cases.rel_err(host(g[n]), ref[n]) <= TOL_FP32, n
    keep = g["dK"].clone()
    g["dK"].fill_(7.0)
    rc = fh.fh_flash_attn_backward(B, h, L, d, 0, scale, *[p(x) for x in t], p(g["dQ"]), None, p(g["dV"]), None)
    assert rc == 0 and bool((g["dK"] == 7.0).all()) and cases.rel_err(host(g["dV"]), ref["dV"]) <= TOL_FP32
    del keep


@pytest.mark.parametrize("mode,tol", [(None, TOL_FP32), ("tc", TOL_TF32)])
def test_batched_forwarders(fh, oracle, math_mode, mode, tol):
    math_mode(mode)
    # out_prod
    s0, s1 = cases.out_prod_case(64, 48, 40, 3, 2)
    dst = torch.zeros((2, 3, 48, 64), device="cuda")
    ne0 = (C.c_int64 * 4)(64, 40, 3, 2)
    ne1 = (C.c_int64 * 4)(48, 40, 3, 2)
    ne = (C.c_int64 * 4)(64, 48, 3, 2)
    torch.cuda.synchronize()
    S0, S1 = dev(s0), dev(s1)
    fh.fh_out_prod(p(S0), p(S1), p(dst), ne0, ne1, ne)
    assert cases.rel_err(host(dst), oracle.out_prod(s0, s1)) <= tol
    # tri_mul, both directions
    for outgoing in (True, False):
        l, r = cases.tri_case(6, 128, 128, 128, outgoing=outgoing)
        dst = torch.zeros((6, 128, 128, 1), device="cuda")
        torch.cuda.synchronize()
        Ld, Rd = dev(l), dev(r)
        fh.fh_tri_mul(p(Ld), p(Rd), p(dst), 6, 128, 128, 128, 1, 1.0 / 128, int(outgoing))
        assert cases.rel_err(host(dst), oracle.tri_mul(l, r, 128.0, outgoing)) <= tol
    # outer_prod_mean
    l, r = cases.opm_case(8, 64, 128)
    dst = torch.zeros((64, 64, 64, 1), device="cuda")
    torch.cuda.synchronize()
    Ld, Rd = dev(l), dev(r)
    fh.fh_outer_prod_mean(p(Ld), p(Rd), p(dst), 8, 64, 128, 1, 1.0 / 128)
    assert cases.rel_err(host(dst), oracle.outer_prod_mean(l, r)) <= tol


def test_mulmat_stats_table(monkeypatch):
    """PPML_MULMAT_STATS=1 must be set before the library first looks (a fresh process): begin / end pairs land in the
    table that ppml_b200_mulmat_stats_dump returns, and the open list stays bounded."""
    import subprocess
    import sys
    code = (
        "import ctypes as C, torch\n"
        "from proteinpredictmachinelearning_b200 import load, ops\n"
        "lib = load()\n"
        "a = torch.randn(408, 256, device='cuda'); b = torch.randn(256, 256, device='cuda')\n"
        "for _ in range(5000):\n"
        "    lib.ppml_b200_mulmat_stats_begin(408, 256, 256); lib.ppml_b200_mulmat_stats_end(b'tf32')\n"
        "lib.ppml_b200_mulmat_stats_begin(408, 256, 256); ops.mul_mat_cuda(a, b); lib.ppml_b200_mulmat_stats_end(b'tf32')\n"
        "buf = C.create_string_buffer(4096); n = lib.ppml_b200_mulmat_stats_dump(buf, 4096)\n"
        "print(buf.value.decode())\n")
    env = dict(os.environ, PPML_MULMAT_STATS="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert "tf32 M=408 K=256 N=256 calls=5001" in out.stdout
