"""Pins the CPU restatement (oracle/ppml_oracle.c): against the known-answer vectors of the reference's
own unit tests, against fixtures produced by the reference's unmodified CPU sources
(tests/golden/reference_cpu.npz, generator beside it), and -- where that library was built -- against
the reference's CPU sources live."""
import os

import numpy as np
import pytest

import cases
from checkers import Ref, have_ref

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu.npz"))


# ---- known answers restated from the reference's tests --------------------------------------------
def test_mul_mat_known_answer(oracle):
    """tests/test_cuda.cpp:133-167 (MulMat): 17 x 9 x 23, inputs from index arithmetic, tol 1e-3."""
    M, K, N = 17, 9, 23
    A = (np.arange(M * K) % 11).astype(np.float32) * 0.5 - 2.0
    B = (np.arange(N * K) % 13).astype(np.float32) * 0.25 + 0.5
    got = oracle.mul_mat_f32(A.reshape(M, K), B.reshape(N, K))
    ref = A.reshape(M, K).astype(np.float64) @ B.reshape(N, K).astype(np.float64).T
    assert np.abs(got - ref).max() <= 1e-3


def test_out_prod_known_answer(oracle):
    """tests/test_cuda.cpp:207-245 (OutProd): C0=4, C1=5, K=3, flat index-0-innermost layout, tol 1e-4."""
    C0, C1, K = 4, 5, 3
    a = (np.arange(C0 * K) % 7).astype(np.float32) * 0.5
    b = (np.arange(C1 * K) % 9).astype(np.float32) * 0.25 - 1.0
    got = oracle.out_prod(a.reshape(1, 1, K, C0), b.reshape(1, 1, K, C1)).reshape(C1, C0)
    for i0 in range(C0):
        for i1 in range(C1):
            s = sum(float(a[i0 + k * C0]) * float(b[i1 + k * C1]) for k in range(K))
            assert abs(got[i1, i0] - s) <= 1e-4


def test_tf32_case_exact_in_fp32(oracle):
    """tests/test_cuda.cpp:1710-1740 (TF32GemmCorrectness) inputs: multiples of 1/8, exact in tf32."""
    M = K = N = 32
    A = ((np.arange(M * K) % 7).astype(np.float32) * 0.25 - 0.5).reshape(M, K)
    B = ((np.arange(N * K) % 11).astype(np.float32) * 0.125 + 0.1).reshape(N, K)
    got = oracle.mul_mat_f32(A, B)
    ref = A.astype(np.float64) @ B.astype(np.float64).T
    assert np.abs(got - ref).max() <= 0.02 * (np.abs(ref).mean() + 1e-3)


def test_outer_product_mean_value_identity(oracle):
    """tests/test_outer_product_mean.cpp pins the mean-of-outer-products value; same identity on the
    graph op's flat layout: constant inputs a, b give a*b everywhere."""
    l = np.full((3, 4, 5, 1), 2.0, np.float32)
    r = np.full((3, 4, 5, 1), -1.5, np.float32)
    assert np.array_equal(oracle.outer_prod_mean(l, r), np.full((9, 4, 4, 1), -3.0, np.float32))


# ---- fixtures produced by the reference's own CPU code ---------------------------------------------
@pytest.mark.parametrize("M,K,N", [(17, 9, 23), (408, 256, 256), (51, 128, 8), (255, 33, 32), (130, 64, 128)])
def test_mul_mat_golden(oracle, M, K, N):
    a, b, bi = cases.mul_mat_case(M, K, N, seed=1)
    assert np.array_equal(oracle.mul_mat_f32(a, b), GOLD[f"mm_{M}_{K}_{N}"])
    assert np.array_equal(oracle.mul_mat_f32(a, b, bi), GOLD[f"mmb_{M}_{K}_{N}"])


def test_mul_mat_f16_golden(oracle):
    a, b, bi = cases.mul_mat_case(40, 64, 48, seed=11)
    got = oracle.mul_mat_16(a.astype(np.float16).view(np.uint16), b.astype(np.float16).view(np.uint16), bi)
    assert np.array_equal(got, GOLD["mm16_40_64_48"])


def test_attention_first_key_tile_masked_golden(oracle):
    """The reference's CPU kernel gives O = 0, LSE = -inf for a row whose first 64 scores are all -inf, even with
    visible keys behind them (src/ops/FlashAttn.cpp:94-121); the restatement does the same, bit for bit."""
    Q, K, V, bi = cases.attn_masked_first_tile_case(d=8, L=100, Lk=200)
    O, LSE = oracle.flash_attn(Q, K, V, bi, scale=1 / np.sqrt(32.0))
    assert np.array_equal(O, GOLD["fa_masked_O"]) and np.array_equal(LSE, GOLD["fa_masked_LSE"])
    assert np.all(O[:, :, 3] == 0) and np.all(LSE[:, :, 3] == -np.inf) and np.any(O[:, :, 4] != 0)


def _q8_inputs():
    w, x = cases.q8_case(24, 20, 128, seed=2)
    x[3, :32] = 0.0
    x[4, 0], x[4, 1] = 2.5, -2.5
    x[5, 0], x[5, 1] = -1.5, 1.5
    return w, x


def test_quantizers_golden_bit_exact(oracle):
    w, x = _q8_inputs()
    q80 = oracle.quantize_q8_0(w)
    assert np.array_equal(q80, GOLD["q80_w"])
    assert np.array_equal(oracle.repack_q8_0(q80), GOLD["q80r_w"])
    q81 = oracle.quantize_q8_1(x)
    assert np.array_equal(q81, GOLD["q81_x"])
    assert np.array_equal(oracle.dequantize(q80, 0), GOLD["deq80_w"])
    assert np.array_equal(oracle.dequantize(q81, 1), GOLD["deq81_x"])


def test_q8_mul_mat_bounded_by_dequantized_product(oracle):
    """No CPU kernel for Q8 exists in the reference; its restatement must at least equal the fp32 product
    of the reference-dequantized operands up to fp32 summation error, and the int32 block sums must be
    exactly the integer dot products."""
    w, x = _q8_inputs()
    q80 = oracle.quantize_q8_0(w)
    W = oracle.repack_q8_0(q80)
    C, sumi = oracle.mul_mat_q8(W, x, 24, wtype=2, c_trans=1, want_sumi=True)
    wd = GOLD["deq80_w"].reshape(24, 128).astype(np.float64)
    xd = GOLD["deq81_x"].reshape(20, 128).astype(np.float64)
    assert cases.rel_err(C, xd @ wd.T) < 1e-5
    qw = q80.reshape(-1, 34)[:, 2:].view(np.int8).reshape(24, 4, 32).astype(np.int64)
    qx = oracle.quantize_q8_1(x).reshape(-1, 36)[:, 4:].view(np.int8).reshape(20, 4, 32).astype(np.int64)
    assert np.array_equal(sumi, np.einsum("nbk,mbk->nmb", qx, qw).astype(np.int32))
    for wt, blocks in ((0, q80), (2, W)):
        assert np.array_equal(oracle.mul_mat_q8(blocks, x, 24, wtype=wt, c_trans=0), C.T)


def test_attention_golden(oracle):
    Q, K, V, bi = cases.attn_case(2, 3, 70, 32, seed=3)
    O, LSE = oracle.flash_attn(Q, K, V, bi, scale=1 / np.sqrt(32.0))
    assert np.array_equal(O, GOLD["fa_O"]) and np.array_equal(LSE, GOLD["fa_LSE"])
    O, LSE = oracle.flash_attn(Q, K, V, None, causal=True)
    assert np.array_equal(O, GOLD["fa_causal_O"]) and np.array_equal(LSE, GOLD["fa_causal_LSE"])
    legacy = oracle.attention_legacy(Q, K, V, bi, 1 / np.sqrt(32.0))
    assert np.array_equal(legacy, GOLD["fa_legacy_O"])
    # fused vs naive vs unfused agree to fp32 summation error (src/cuda/FlashAttnKernel.cu:274 quotes ~1e-4)
    assert cases.rel_err(GOLD["fa_O"], GOLD["fa_naive_O"]) < 1e-5
    assert cases.rel_err(GOLD["fa_O"], GOLD["fa_legacy_O"]) < 1e-5


def test_attention_backward_golden(oracle):
    """The restated backward against gradients produced by the reference's flash_attn_backward_cpu, bit for bit; rows 5
    and 17 are fully masked (LSE = -inf): all their gradients are zero."""
    Q, K, V, bi, dO = cases.attn_backward_case(2, 3, 45, 32, seed=7, masked_rows=(5, 17))
    O, LSE = oracle.flash_attn(Q, K, V, bi, scale=1 / np.sqrt(32.0))
    assert np.all(LSE[:, :, 5] == -np.inf) and np.all(LSE[:, :, 17] == -np.inf)
    g = oracle.flash_attn_backward(Q, K, V, O, dO, LSE, bi, scale=1 / np.sqrt(32.0))
    for n in ("dQ", "dK", "dV", "dbias"):
        assert np.array_equal(g[n], GOLD["fab_" + n]), n
    assert np.all(g["dQ"][:, :, 5] == 0) and np.all(g["dbias"][:, :, 17] == 0)
    O, LSE = oracle.flash_attn(Q, K, V, None, causal=True)
    g = oracle.flash_attn_backward(Q, K, V, O, dO, LSE, None, causal=True)
    for n in ("dQ", "dK", "dV", "dbias"):
        assert np.array_equal(g[n], GOLD["fab_causal_" + n]), n
    assert np.all(np.triu(g["dbias"][0, 0], 1) == 0)
    # a null output is skipped, the others are unchanged
    g2 = oracle.flash_attn_backward(Q, K, V, O, dO, LSE, None, causal=True, want=("dK",))
    assert list(g2) == ["dK"] and np.array_equal(g2["dK"], g["dK"])


def test_attention_backward_is_the_gradient(oracle):
    """Finite differences of sum(O * dO) in float64 against dQ, dK, dV and dbias (small case, eps of the forward = 0)."""
    Q, K, V, bi, dO = cases.attn_backward_case(1, 2, 9, 4, seed=21)
    sc = 0.5
    def fwd(q, k, v, b):
        s = np.einsum("bhid,bhjd->bhij", q, k) * sc + b
        p = np.exp(s - s.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
        return np.einsum("bhij,bhjd->bhid", p, v)
    q64, k64, v64, b64, g64 = (t.astype(np.float64) for t in (Q, K, V, bi, dO))
    O = fwd(q64, k64, v64, b64)
    s = np.einsum("bhid,bhjd->bhij", q64, k64) * sc + b64
    LSE = np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)
    g = oracle.flash_attn_backward(Q, K, V, O.astype(np.float32), dO, LSE.astype(np.float32), bi, scale=sc)
    for name, arr in (("dQ", q64), ("dK", k64), ("dV", v64), ("dbias", b64)):
        num = np.zeros_like(arr)
        it = np.nditer(arr, flags=["multi_index"])
        for _ in it:
            idx = it.multi_index
            old = arr[idx]
            arr[idx] = old + 1e-5; up = (fwd(q64, k64, v64, b64) * g64).sum()
            arr[idx] = old - 1e-5; dn = (fwd(q64, k64, v64, b64) * g64).sum()
            arr[idx] = old
            num[idx] = (up - dn) / 2e-5
        assert cases.rel_err(g[name], num) < 2e-4, name


def test_attention_lq_ne_lk_matches_unfused_graph(oracle):
    Q, K, V, bi = cases.attn_case(3, 2, 1, 8, Lk=40, seed=33)
    assert np.array_equal(oracle.attention_legacy(Q, K, V, bi, 1 / np.sqrt(32.0)), GOLD["fa_legacy_q1_O"])
    O, _ = oracle.flash_attn(Q, K, V, bi, scale=1 / np.sqrt(32.0))
    assert cases.rel_err(O, GOLD["fa_legacy_q1_O"]) < 1e-5


def test_attention_fully_masked_row(oracle):
    Q, K, V, bi = cases.attn_case(1, 1, 4, 8, seed=7)
    bi[0, 0, 2, :] = -np.inf
    O, LSE = oracle.flash_attn(Q, K, V, bi)
    assert np.all(O[0, 0, 2] == 0) and LSE[0, 0, 2] == -np.inf and np.isfinite(O).all()


def test_pair_ops_golden(oracle):
    l, r = cases.tri_case(6, 20, 24, 28, outgoing=True)
    assert np.array_equal(oracle.tri_mul(l, r, 28.0, True), GOLD["tri_out"])
    l, r = cases.tri_case(6, 20, 24, 28, outgoing=False)
    assert np.array_equal(oracle.tri_mul(l, r, 28.0, False), GOLD["tri_in"])
    l, r = cases.tri_case(3, 5, 6, 7, B=2, outgoing=True, seed=44)
    assert np.array_equal(oracle.tri_mul(l, r, 7.0, True, B=2), GOLD["tri_out_b2"])
    l = np.full((1, 2, 2, 1), 3e3, np.float32)
    got = oracle.tri_mul(l, l, 1.0, True)
    assert np.array_equal(got, GOLD["tri_clamp"]) and np.all(got == 1e4)
    l, r = cases.opm_case(4, 12, 9)
    assert np.array_equal(oracle.outer_prod_mean(l, r), GOLD["opm"])
    s0, s1 = cases.out_prod_case(13, 11, 17, 3, 2)
    assert np.array_equal(oracle.out_prod(s0, s1), GOLD["out_prod"])
    s0, s1 = cases.out_prod_case(13, 11, 17, 4, 2, ne02=2, ne03=1)
    assert np.array_equal(oracle.out_prod(s0, s1), GOLD["out_prod_bcast"])


def test_tri_mul_nan_scrub(oracle):
    l, r = cases.tri_case(1, 2, 2, 3)
    l[0, 0, 1, 0] = np.nan
    got = oracle.tri_mul(l, r, 3.0, True)
    assert np.all(got[0, 0] == 0) and np.isfinite(got).all()


# ---- live comparison with the reference's CPU sources (this container only) ------------------------
@pytest.mark.skipif(not have_ref(), reason="oracle/_ref not built (needs the reference tree)")
def test_oracle_equals_reference_live(oracle):
    os.environ["PPML_CPU_F16C"] = "0"
    ref = Ref(n_threads=3)
    r = np.random.default_rng(99)
    for (M, K, N) in [(1, 1, 1), (5, 7, 3), (64, 32, 16), (33, 100, 65)]:
        a, b, bi = cases.mul_mat_case(M, K, N, seed=M + K + N)
        assert np.array_equal(oracle.mul_mat_f32(a, b, bi), ref.mul_mat(a, b, bi))
    x = (r.standard_normal(32 * 257) * 10.0 ** r.integers(-6, 4, 32 * 257)).astype(np.float32)
    assert np.array_equal(oracle.quantize_q8_0(x), ref.quantize_q8_0(x))
    assert np.array_equal(oracle.quantize_q8_1(x), ref.quantize_q8_1(x))
    Q, K, V, bi = cases.attn_case(1, 2, 130, 16, seed=5)
    for causal in (False, True):
        o1 = oracle.flash_attn(Q, K, V, bi, causal=causal, Bc=32)
        o2 = ref.flash_attn(Q, K, V, bi, causal=causal, Bc=32)
        assert np.array_equal(o1[0], o2[0]) and np.array_equal(o1[1], o2[1])
