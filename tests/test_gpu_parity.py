"""Parity of the CUDA path (through the C ABI) with the CPU checker on identical seeded inputs.

Tolerances (normalised error = max|got-ref| / max|ref|):
  CUDA-core fp32 kernels        1e-5   (same summation order, FMA contraction only)
  tf32 tensor-core kernels      1e-3   (the required bound for fp32 / tf32)
  fp16 / bf16 operand kernels   1e-5 against the checker fed the same 16-bit operands
                                1e-2 against the fp32 product (the required bound for bf16)
  Q8: quantized bytes, scales and int32 block sums bit-exact; fp32 result 1e-5
"""
import os

import numpy as np
import pytest

import cases

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from proteinpredictmachinelearning_b200 import PATH_AUTO, PATH_SIMT, PATH_UMMA, TF32_ROUND, TF32_TMA, TF32_TRUNCATE  # noqa: E402
from proteinpredictmachinelearning_b200 import ops  # noqa: E402

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu.npz"))
TOL_FP32, TOL_TF32, TOL_16 = 1e-5, 1e-3, 1e-2


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.detach().cpu().numpy()


@pytest.fixture(autouse=True)
def _no_device_abort():
    yield
    code, where = ops.device_status()
    assert code == 0, f"a kernel gave up a bounded wait: code {code} at site {where:#x}"


# ------------------------------------------------------------------------------------------------
# OP_MUL_MAT fp32
# ------------------------------------------------------------------------------------------------
MM_SHAPES = [(17, 9, 23), (408, 256, 256), (51, 128, 8), (255, 33, 32), (130, 64, 128), (1, 1, 1), (2601, 128, 256),
             (300, 1024, 256), (129, 36, 260)]


@pytest.mark.parametrize("M,K,N", MM_SHAPES)
@pytest.mark.parametrize("bias", [False, True])
def test_mul_mat_simt(oracle, M, K, N, bias):
    a, b, bi = cases.mul_mat_case(M, K, N, seed=1, bias=bias)
    got = host(ops.mul_mat_cuda(dev(a), dev(b), None if bi is None else dev(bi), path=PATH_SIMT))
    key = f"{'mmb' if bias else 'mm'}_{M}_{K}_{N}"
    ref = GOLD[key] if key in GOLD else oracle.mul_mat_f32(a, b, bi)
    assert cases.rel_err(got, ref) <= TOL_FP32


@pytest.mark.parametrize("M,K,N", [s for s in MM_SHAPES if s[1] % 4 == 0])
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("mode", [TF32_ROUND, TF32_TMA])
def test_mul_mat_tf32_umma(oracle, M, K, N, bias, mode):
    """Both ways of rounding fp32 to tf32 (in shared memory with cvt.rna, or by the TMA unit: the mode the C++
    forwarders and the benchmark use) meet the required 1e-3."""
    a, b, bi = cases.mul_mat_case(M, K, N, seed=1, bias=bias)
    got = host(ops.mul_mat_cuda(dev(a), dev(b), None if bi is None else dev(bi), path=PATH_UMMA, tf32_mode=mode))
    key = f"{'mmb' if bias else 'mm'}_{M}_{K}_{N}"
    ref = GOLD[key] if key in GOLD else oracle.mul_mat_f32(a, b, bi)
    assert cases.rel_err(got, ref) <= TOL_TF32


# the (M, K, N) shapes that carry most OP_MUL_MAT executions of the dev-size forward (L = 51, MSA depth 8), incl. the
# SE3 radial MLPs with K = 33 (row pitch not a multiple of 16 bytes) and the skinny N = 8 / 32 heads
CENSUS_SHAPES = [(2601, 128, 256), (2601, 128, 128), (2601, 256, 128), (408, 256, 256), (2550, 32, 1024), (2601, 64, 128),
                 (2550, 32, 256), (408, 256, 1024), (408, 1024, 256), (2550, 32, 32), (2550, 33, 32), (2601, 128, 8)]


@pytest.mark.parametrize("M,K,N", CENSUS_SHAPES)
@pytest.mark.parametrize("mode", [TF32_ROUND, TF32_TMA])
def test_mul_mat_dev_forward_census(oracle, M, K, N, mode):
    """Tensor-core dispatch (what the executor gets with PPML_MUL_MAT_TC=1): tensor cores where TMA can address the
    operands, CUDA cores otherwise."""
    a, b, bi = cases.mul_mat_case(M, K, N, seed=1, bias=True)
    ref = oracle.mul_mat_f32(a, b, bi)
    assert cases.rel_err(host(ops.mul_mat_cuda(dev(a), dev(b), dev(bi), path=PATH_AUTO, tf32_mode=mode)), ref) <= TOL_TF32
    assert cases.rel_err(host(ops.mul_mat_cuda(dev(a), dev(b), dev(bi), path=PATH_SIMT)), ref) <= TOL_FP32
    a16, b16 = dev(a).bfloat16(), dev(b).bfloat16()
    ref16 = oracle.mul_mat_f32(host(a16.float()), host(b16.float()), bi)
    assert cases.rel_err(host(ops.mul_mat_16(a16, b16, dev(bi), path=PATH_AUTO)), ref16) <= TOL_FP32


def test_mul_mat_umma_rejects_unaligned_k_and_auto_falls_back(oracle):
    a, b, bi = cases.mul_mat_case(255, 33, 32, seed=1)
    with pytest.raises(RuntimeError):
        ops.mul_mat_cuda(dev(a), dev(b), dev(bi), path=PATH_UMMA)
    got = host(ops.mul_mat_cuda(dev(a), dev(b), dev(bi), path=PATH_AUTO))
    assert cases.rel_err(got, GOLD["mmb_255_33_32"]) <= TOL_FP32


def test_mul_mat_tf32_known_answer_exact():
    """Reference TF32GemmCorrectness inputs (tests/test_cuda.cpp:1710-1740) are exact in tf32."""
    M = K = N = 32
    A = ((np.arange(M * K) % 7).astype(np.float32) * 0.25 - 0.5).reshape(M, K)
    B = ((np.arange(N * K) % 8).astype(np.float32) * 0.125 + 0.25).reshape(N, K)
    got = host(ops.mul_mat_cuda(dev(A), dev(B), path=PATH_UMMA))
    ref = A.astype(np.float64) @ B.astype(np.float64).T
    assert np.abs(got - ref).max() <= 1e-4


@pytest.mark.parametrize("mode", [TF32_ROUND, TF32_TMA, TF32_TRUNCATE])
def test_mul_mat_tf32_modes_report_error(oracle, mode):
    """All three ways of feeding fp32 to the tf32 tensor core stay within a loose 4e-3; the default
    (rounding) must meet 1e-3.  The measured errors are printed for the record."""
    a, b, bi = cases.mul_mat_case(2048, 256, 256, seed=8, bias=False)
    a = np.abs(a)
    b = np.abs(b)                      # same-sign products expose a truncation bias
    got = host(ops.mul_mat_cuda(dev(a), dev(b), path=PATH_UMMA, tf32_mode=mode))
    err = cases.rel_err(got, oracle.mul_mat_f32(a, b))
    print(f"tf32 mode {mode}: normalised error {err:.3e}")
    assert err <= (TOL_TF32 if mode == TF32_ROUND else 4e-3)


def _tf32_host(x, mode):
    """fp32 -> tf32 (10 explicit mantissa bits) on the host: 'rna' nearest, ties away from zero (cvt.rna.tf32.f32),
    'rne' nearest, ties to even, 'rz' truncation.  Finite normal inputs."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    if mode == "rna":
        u = u + 0x1000
    elif mode == "rne":
        u = u + 0xFFF + ((u >> 13) & 1)
    return (u & 0xFFFFE000).astype(np.uint32).view(np.float32)


def test_mul_mat_tf32_rounding_of_each_mode():
    """What each tf32 mode does to an fp32 operand, observed exactly: with B = identity every output is one product
    a * 1, so C is the operand as the tensor core saw it.  Rounding in shared memory is cvt.rna (nearest, ties away from
    zero); the TMA unit's conversion rounds to nearest with ties to even, so the two differ on exact ties only (one tf32
    unit in the last place there); feeding fp32 words unchanged truncates."""
    r = np.random.default_rng(8)
    M, K = 512, 256
    a = (r.standard_normal((M, K)) * 10.0 ** r.integers(-3, 4, (M, K))).astype(np.float32)
    ties = (1.0 + (2 * r.integers(0, 512, K) + 1) * 2.0 ** -11).astype(np.float32)       # exactly between two tf32 values
    a[5], a[6] = ties, -ties
    a[7, :4] = [0.0, 1.0, -1.0, 1.0 + 2.0 ** -10]
    eye = np.eye(K, dtype=np.float32)
    got = {m: host(ops.mul_mat_cuda(dev(a), dev(eye), path=PATH_UMMA, tf32_mode=m)) for m in (TF32_ROUND, TF32_TMA, TF32_TRUNCATE)}
    rna, rne, rz = (_tf32_host(a, m) for m in ("rna", "rne", "rz"))
    assert np.array_equal(got[TF32_ROUND], rna)
    assert np.array_equal(got[TF32_TRUNCATE], rz)
    # measured on B200: the TMA unit rounds to nearest, ties to EVEN -- it differs from cvt.rna only on exact ties
    assert np.array_equal(got[TF32_TMA], rne)
    assert not np.array_equal(rne, rna)                               # the tie rows of the input tell the two apart


# ------------------------------------------------------------------------------------------------
# a Linear fused with its neighbours: LayerNorm in front, activation gate behind
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,K,N", [(408, 256, 256), (2601, 128, 128), (300, 1024, 256), (255, 33, 32), (130, 64, 100)])
@pytest.mark.parametrize("path,tol", [(PATH_SIMT, 2e-5), (PATH_AUTO, TOL_TF32)])
def test_linear_with_layernorm_and_gate_fused(oracle, M, K, N, path, tol):
    """LayerNorm(x) W^T + b, then sigmoid(.) * other, as the reference computes them node by node (OP_NORM, mul, add,
    OP_MUL_MAT, OP_ACT_MUL) against one fused launch (plus the per-row statistics and, once per layer, the folded
    weights)."""
    from checkers import act_mul_f32, layer_norm_f32
    r = np.random.default_rng(M + K + N)
    x = (r.standard_normal((M, K)) * 1.5 + 0.5).astype(np.float32)
    w = (r.standard_normal((N, K)) * 0.02).astype(np.float32)
    b = (r.standard_normal(N) * 0.1).astype(np.float32)
    gamma = (1.0 + 0.1 * r.standard_normal(K)).astype(np.float32)
    beta = (0.1 * r.standard_normal(K)).astype(np.float32)
    other = r.standard_normal((M, N)).astype(np.float32)
    eps = 1e-5
    lin = oracle.mul_mat_f32(layer_norm_f32(x, gamma, beta, eps), w, b)
    Wg, u, v = ops.layernorm_fold(dev(w), dev(gamma), dev(beta), dev(b))
    X = dev(x)
    stats = ops.row_stats(X, eps)
    # LayerNorm -> Linear
    got = host(ops.mul_mat_fused(X, Wg, bias=v, ln_stats=stats, ln_u=u, path=path))
    assert cases.rel_err(got, lin) <= tol
    # LayerNorm -> Linear -> sigmoid gate
    got = host(ops.mul_mat_fused(X, Wg, bias=v, ln_stats=stats, ln_u=u, gate=dev(other), act="sigmoid", path=path))
    assert cases.rel_err(got, act_mul_f32(lin, other, "sigmoid")) <= tol
    # Linear -> gate alone, every activation kind
    plain = oracle.mul_mat_f32(x, w, b)
    for kind in ("sigmoid", "silu", "gelu", "tanh", "relu"):
        got = host(ops.mul_mat_fused(X, dev(w), bias=dev(b), gate=dev(other), act=kind, path=path))
        assert cases.rel_err(got, act_mul_f32(plain, other, kind)) <= tol, kind
    got = host(ops.mul_mat_fused(X, dev(w), bias=dev(b), act="relu", path=path))          # activation without a gate
    assert cases.rel_err(got, np.maximum(plain, 0)) <= tol


def test_row_stats_follow_op_norm(oracle):
    r = np.random.default_rng(3)
    x = (r.standard_normal((1000, 256)) * 2 + 3).astype(np.float32)
    st = host(ops.row_stats(dev(x), 1e-5))
    mean = x.mean(axis=1, dtype=np.float64)
    var = ((x - mean[:, None]) ** 2).mean(axis=1)
    assert np.abs(st[:, 0] - mean).max() <= 1e-5 and np.abs(st[:, 1] - 1 / np.sqrt(var + 1e-5)).max() <= 1e-5


# ------------------------------------------------------------------------------------------------
# 16-bit operands
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("path", [PATH_SIMT, PATH_UMMA])
@pytest.mark.parametrize("M,K,N", [(40, 64, 48), (408, 256, 256), (2601, 128, 128), (130, 72, 136)])
def test_mul_mat_16bit(oracle, dtype, path, M, K, N):
    a, b, bi = cases.mul_mat_case(M, K, N, seed=11)
    tdt = torch.float16 if dtype == "f16" else torch.bfloat16
    a16, b16 = ops.cast(dev(a), tdt), ops.cast(dev(b), tdt)
    ref_cast = dev(a).to(tdt)
    assert torch.equal(a16, ref_cast)                                  # the cast kernel rounds to nearest even
    got = host(ops.mul_mat_16(a16, b16, dev(bi), path=path))
    ref16 = oracle.mul_mat_16(host(a16.view(torch.int16)).view(np.uint16), host(b16.view(torch.int16)).view(np.uint16), bi, kind=dtype)
    assert cases.rel_err(got, ref16) <= TOL_FP32
    assert cases.rel_err(got, oracle.mul_mat_f32(a, b, bi)) <= TOL_16
    if dtype == "f16" and (M, K, N) == (40, 64, 48):
        assert cases.rel_err(got, GOLD["mm16_40_64_48"]) <= TOL_FP32


# ------------------------------------------------------------------------------------------------
# Q8
# ------------------------------------------------------------------------------------------------
def _q8_special(x):
    x[3, :32] = 0.0
    x[4, 0], x[4, 1] = 2.5, -2.5
    x[5, 0], x[5, 1] = -1.5, 1.5
    return x


def test_quantizers_bit_exact(oracle):
    w, x = cases.q8_case(24, 20, 128, seed=2)
    x = _q8_special(x)
    assert np.array_equal(host(ops.quantize_rows_q8_1_cuda(dev(x))), GOLD["q81_x"])
    assert np.array_equal(host(ops.quantize_q8_0r(dev(w))), GOLD["q80r_w"])
    assert np.array_equal(host(ops.dequantize_q8_cuda(dev(GOLD["q80_w"]), 0)), GOLD["deq80_w"])
    assert np.array_equal(host(ops.dequantize_q8_cuda(dev(GOLD["q81_x"]), 1)), GOLD["deq81_x"])
    r = np.random.default_rng(7)
    big = (r.standard_normal(32 * 4099) * 10.0 ** r.integers(-5, 3, 32 * 4099)).astype(np.float32)
    assert np.array_equal(host(ops.quantize_rows_q8_1_cuda(dev(big))), oracle.quantize_q8_1(big))
    assert np.array_equal(host(ops.quantize_q8_0r(dev(big))), oracle.repack_q8_0(oracle.quantize_q8_0(big)))


Q8_SHAPES = [(24, 20, 128), (128, 408, 128), (256, 408, 256), (512, 300, 1024), (1024, 130, 256), (136, 257, 96),
             (256, 2601, 128)]


@pytest.mark.parametrize("Mout,Ntok,K", Q8_SHAPES)
@pytest.mark.parametrize("path", [PATH_SIMT, PATH_UMMA])
def test_mul_mat_q8(oracle, Mout, Ntok, K, path):
    w, x = cases.q8_case(Mout, Ntok, K, seed=2)
    if Ntok >= 6:
        x = _q8_special(x)
    W = oracle.repack_q8_0(oracle.quantize_q8_0(w))
    bias = (np.random.default_rng(3).standard_normal(Mout) * 0.1).astype(np.float32)
    ref, ref_sumi = oracle.mul_mat_q8(W, x, Mout, wtype=2, c_trans=1, bias=bias, want_sumi=True)
    got, taken, sumi = ops.mul_mat_q8_cuda(dev(W), dev(x), Mout, wtype=2, c_trans=1, bias=dev(bias), path=path, want_sumi=True)
    assert taken == (1 if path == PATH_UMMA else 0)
    assert np.array_equal(host(sumi), ref_sumi)                      # int32 block dot products: bit-exact
    assert cases.rel_err(host(got), ref) <= TOL_FP32


@pytest.mark.parametrize("Mout,Ntok,K", Q8_SHAPES + [(384, 1000, 1024), (128, 19000, 512)])
def test_mul_mat_q8_one_and_two_pass_forms(oracle, Mout, Ntok, K):
    """Quantizing inside the product kernel or in a kernel of its own gives the same int32 block sums and the same
    fp32 results, bit for bit; both match the checker."""
    from proteinpredictmachinelearning_b200 import _lib
    w, x = cases.q8_case(Mout, Ntok, K, seed=12)
    x = _q8_special(x)
    W = oracle.repack_q8_0(oracle.quantize_q8_0(w))
    bias = (np.random.default_rng(3).standard_normal(Mout) * 0.1).astype(np.float32)
    ref, ref_sumi = oracle.mul_mat_q8(W, x, Mout, wtype=2, c_trans=1, bias=bias, want_sumi=True)
    out = {}
    try:
        for mode in (0, 1):
            _lib.load().ppml_b200_set_q8_two_pass(mode)
            got, taken, sumi = ops.mul_mat_q8_cuda(dev(W), dev(x), Mout, wtype=2, c_trans=1, bias=dev(bias), path=PATH_UMMA,
                                                   want_sumi=True)
            fast, _ = ops.mul_mat_q8_cuda(dev(W), dev(x), Mout, wtype=2, c_trans=1, bias=dev(bias), path=PATH_UMMA)
            assert taken == 1
            out[mode] = (host(got), host(sumi), host(fast))
    finally:
        _lib.load().ppml_b200_set_q8_two_pass(-1)
    assert np.array_equal(out[0][1], ref_sumi) and np.array_equal(out[1][1], ref_sumi)
    assert np.array_equal(out[0][0], out[1][0]) and np.array_equal(out[0][2], out[1][2])
    assert np.array_equal(out[0][0], out[0][2])
    assert cases.rel_err(out[1][0], ref) <= TOL_FP32


@pytest.mark.parametrize("Mout,Ntok,K", [(8, 2601, 128), (16, 408, 256), (16, 1000, 64), (5, 300, 1024), (1, 4099, 32), (13, 70, 512)])
def test_mul_mat_q8_few_output_columns(oracle, Mout, Ntok, K):
    """At most 16 output columns (the model's pair-bias and outer-product-mean projections): PATH_AUTO takes the one-pass
    CUDA-core kernel -- quantization in registers, dp4a against the weights in shared memory.  int32 block sums bit-exact,
    fp32 output 1e-5, and the same results as the tensor-core kernel asked for by name."""
    w, x = cases.q8_case(Mout, Ntok, K, seed=7)
    x = _q8_special(x)
    W = oracle.repack_q8_0(oracle.quantize_q8_0(w))
    bias = (np.random.default_rng(3).standard_normal(Mout) * 0.1).astype(np.float32)
    ref, ref_sumi = oracle.mul_mat_q8(W, x, Mout, wtype=2, c_trans=1, bias=bias, want_sumi=True)
    got, taken, sumi = ops.mul_mat_q8_cuda(dev(W), dev(x), Mout, wtype=2, c_trans=1, bias=dev(bias), path=PATH_AUTO, want_sumi=True)
    assert taken == 0                                                  # CUDA cores (every case here is inside the rule)
    assert np.array_equal(host(sumi), ref_sumi)
    assert cases.rel_err(host(got), ref) <= TOL_FP32
    fast, _ = ops.mul_mat_q8_cuda(dev(W), dev(x), Mout, wtype=2, c_trans=1, path=PATH_AUTO)          # without bias, without sums
    ref_nb = oracle.mul_mat_q8(W, x, Mout, wtype=2, c_trans=1)
    assert cases.rel_err(host(fast), ref_nb) <= TOL_FP32
    tc, taken_tc = ops.mul_mat_q8_cuda(dev(W), dev(x), Mout, wtype=2, c_trans=1, bias=dev(bias), path=PATH_UMMA)
    assert taken_tc == 1 and cases.rel_err(host(tc), host(got)) <= TOL_FP32


@pytest.mark.parametrize("wtype", [0, 1, 2])
@pytest.mark.parametrize("c_trans", [0, 1])
def test_mul_mat_q8_weight_layouts(oracle, wtype, c_trans):
    w, x = cases.q8_case(72, 50, 160, seed=2)
    q80 = oracle.quantize_q8_0(w)
    if wtype == 0:
        W = q80
    elif wtype == 2:
        W = oracle.repack_q8_0(q80)
    else:                                                              # Q8_1-typed weights: same d, extra sum field
        blocks = q80.reshape(-1, 34)
        W = np.zeros((blocks.shape[0], 36), np.uint8)
        W[:, :2] = blocks[:, :2]
        W[:, 4:] = blocks[:, 2:]
        W = W.reshape(-1)
    ref = oracle.mul_mat_q8(W, x, 72, wtype=wtype, c_trans=c_trans)
    got, taken = ops.mul_mat_q8_cuda(dev(W), dev(x), 72, wtype=wtype, c_trans=c_trans)
    assert cases.rel_err(host(got), ref) <= TOL_FP32
    if wtype == 2:
        got2, taken2 = ops.mul_mat_q8_cuda(dev(W), dev(x), 72, wtype=2, c_trans=c_trans, path=PATH_UMMA)
        assert taken2 == 1 and cases.rel_err(host(got2), ref) <= TOL_FP32


def test_mul_mat_q8_full_size_property():
    """M = 65536 tokens (the sweep's largest size): tensor-core and dp4a paths must agree exactly on the
    block sums' consequence -- the fp32 outputs agree to rounding -- and a row permutation of X
    permutes the rows of C."""
    g = torch.Generator(device="cuda").manual_seed(2)
    X = torch.randn((65536, 256), device="cuda", generator=g)
    Wf = torch.randn((256, 256), device="cuda", generator=g) * 0.02
    W = ops.quantize_q8_0r(Wf)
    c_t, taken = ops.mul_mat_q8_cuda(W, X, 256, path=PATH_UMMA)
    c_s, _ = ops.mul_mat_q8_cuda(W, X, 256, path=PATH_SIMT)
    assert taken == 1
    assert float((c_t - c_s).abs().max() / c_s.abs().max()) <= TOL_FP32
    perm = torch.randperm(65536, device="cuda", generator=g)
    c_p, _ = ops.mul_mat_q8_cuda(W, X[perm].contiguous(), 256, path=PATH_UMMA)
    assert torch.equal(c_p, c_t[perm])


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------
def test_attention_golden(oracle):
    Q, K, V, bi = cases.attn_case(2, 3, 70, 32, seed=3)
    O, LSE = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), dev(bi), scale=1 / np.sqrt(32.0), path=PATH_SIMT)
    assert cases.rel_err(host(O), GOLD["fa_O"]) <= TOL_FP32
    assert np.abs(host(LSE) - GOLD["fa_LSE"]).max() <= 1e-5
    O, LSE = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), None, causal=True, path=PATH_SIMT)
    assert cases.rel_err(host(O), GOLD["fa_causal_O"]) <= TOL_FP32
    assert np.abs(host(LSE) - GOLD["fa_causal_LSE"]).max() <= 1e-5
    # tensor-core path (head dim 32, no bias so that Lk = 70 is admissible): tf32 tolerance
    O, LSE = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), None, causal=True, path=PATH_UMMA)
    assert cases.rel_err(host(O), GOLD["fa_causal_O"]) <= TOL_TF32
    assert np.abs(host(LSE) - GOLD["fa_causal_LSE"]).max() <= 2e-3
    # with the bias the key count must be a multiple of 4 for the tensor-core path: AUTO takes the CUDA-core kernel
    with pytest.raises(RuntimeError):
        ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), dev(bi), path=PATH_UMMA)
    O, _ = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), dev(bi), scale=1 / np.sqrt(32.0), path=PATH_AUTO)
    assert cases.rel_err(host(O), GOLD["fa_O"]) <= TOL_FP32


@pytest.mark.parametrize("B,h,L,d,Lk,bias,bcast", [
    (8, 8, 51, 32, None, True, False),      # dev-size MSA row attention
    (51, 8, 8, 32, None, False, False),     # dev-size MSA column attention
    (8, 8, 51, 8, None, True, False),       # extra-MSA block, head dim 8
    (51, 8, 1, 8, 8, False, False),         # global column attention, one query over N keys
    (4, 8, 256, 32, None, True, True),      # full-size rows, one bias shared by the batch
    (2, 4, 100, 64, 77, True, False),
])
def test_attention_shapes(oracle, B, h, L, d, Lk, bias, bcast):
    Q, K, V, bi = cases.attn_case(B, h, L, d, Lk=Lk, seed=3, bias=bias, bias_bcast=bcast)
    scale = 1 / np.sqrt(32.0)
    O, LSE = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), None if bi is None else dev(bi), scale=scale, bias_bcast=bcast,
                                         path=PATH_SIMT)
    rO, rL = oracle.flash_attn(Q, K, V, bi, scale=scale, bias_bcast=bcast)
    assert cases.rel_err(host(O), rO) <= TOL_FP32
    assert np.abs(host(LSE) - rL).max() <= 1e-5
    legacy = oracle.attention_legacy(Q, K, V, bi, scale, bias_bcast=bcast)   # ground truth when Lq != Lk
    assert cases.rel_err(host(O), legacy) <= TOL_FP32


@pytest.mark.parametrize("B,h,L,d,Lk,bias,bcast,causal", [
    (2, 3, 200, 8, None, True, True, False),    # thread-per-row kernel: two row tiles, shared bias
    (2, 2, 70, 16, 45, True, False, False),     # Lq != Lk, ragged key tile
    (2, 2, 150, 4, None, False, False, True),   # causal: row tiles see different key ranges
    (3, 2, 33, 8, 130, True, False, True),      # causal with Lk > L
    (2, 3, 5, 4, 100, True, False, False),      # few query rows: keys over lanes, with bias
    (4, 2, 1, 8, 1024, False, False, False),    # global column attention at full key count
    (2, 2, 20, 16, None, False, False, True),   # few rows, causal (lanes without any visible key)
])
@pytest.mark.parametrize("path", [PATH_SIMT, PATH_AUTO])
def test_attention_small_head_dims(oracle, B, h, L, d, Lk, bias, bcast, causal, path):
    """The exact CUDA-core kernels (PATH_SIMT), and whatever PATH_AUTO picks: for d = 8 with 16 or more query rows that
    is the warp-level tensor-core kernel with tf32 products."""
    tensor = path == PATH_AUTO and d == 8 and L >= 16
    tol_o, tol_l = (TOL_TF32, 2e-3) if tensor else (TOL_FP32, 1e-5)
    Q, K, V, bi = cases.attn_case(B, h, L, d, Lk=Lk, seed=9, bias=bias, bias_bcast=bcast)
    if bi is not None:
        bi[..., 1, :] = -np.inf                  # one fully masked query row per head
        bi[..., 0, ::3] = -np.inf                # and a partly masked one
    scale = 1 / np.sqrt(32.0)
    O, LSE = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), None if bi is None else dev(bi), scale=scale, bias_bcast=bcast,
                                         causal=causal, path=path)
    rO, rL = oracle.flash_attn(Q, K, V, bi, scale=scale, bias_bcast=bcast, causal=causal)
    O, LSE = host(O), host(LSE)
    assert np.isfinite(O).all()
    assert cases.rel_err(O, rO) <= tol_o
    fin = np.isfinite(rL)
    assert np.array_equal(np.isfinite(LSE), fin) and np.abs(LSE[fin] - rL[fin]).max() <= tol_l


@pytest.mark.parametrize("B,h,L,Lk,bias,bcast,causal", [
    (1024 // 64, 8, 256, None, True, True, False),   # extra-MSA rows (fewer batch elements): four batch elements per CTA
    (6, 3, 100, None, True, True, False),       # batch not a multiple of 4, rows not a multiple of 32, ragged key tile
    (5, 2, 130, 70, True, False, False),        # a bias per batch element: 128 rows of one batch element per CTA
    (4, 2, 200, 203, True, True, False),        # key count not a multiple of 4: the bias tile comes in 4-byte pieces
    (3, 2, 90, None, True, True, False),        # fewer than four batch elements
    (4, 2, 150, None, False, False, True),      # causal without bias
    (4, 2, 33, 130, True, True, True),          # causal with Lk > L
    (8, 4, 16, 300, False, False, False),       # a single m tile of rows, five key tiles
])
def test_attention_head_dim_8_tensor_cores(oracle, B, h, L, Lk, bias, bcast, causal):
    """Head dim 8 on the warp-level tensor-core kernel (tf32 products, fp32 softmax) against the oracle, with a fully
    masked and a partly masked query row, and against the exact CUDA-core kernel."""
    Q, K, V, bi = cases.attn_case(B, h, L, 8, Lk=Lk, seed=21, bias=bias, bias_bcast=bcast)
    if bi is not None:
        bi[..., 1, :] = -np.inf
        bi[..., 0, ::3] = -np.inf
    scale = 1 / np.sqrt(8.0)
    args = (dev(Q), dev(K), dev(V), None if bi is None else dev(bi))
    O, LSE = ops.flash_attn_forward_cuda(*args, scale=scale, bias_bcast=bcast, causal=causal, path=PATH_UMMA)
    rO, rL = oracle.flash_attn(Q, K, V, bi, scale=scale, bias_bcast=bcast, causal=causal)
    O, LSE = host(O), host(LSE)
    assert np.isfinite(O).all() and cases.rel_err(O, rO) <= TOL_TF32
    fin = np.isfinite(rL)
    assert np.array_equal(np.isfinite(LSE), fin) and np.abs(LSE[fin] - rL[fin]).max() <= 2e-3
    if bi is not None:
        assert np.all(O[:, :, 1] == 0) and np.all(LSE[:, :, 1] == -np.inf)
    Oe, _ = ops.flash_attn_forward_cuda(*args, scale=scale, bias_bcast=bcast, causal=causal, path=PATH_SIMT)
    assert cases.rel_err(O, host(Oe)) <= TOL_TF32


@pytest.mark.parametrize("B,h,L,Lk,bias,bcast,causal", [
    (4, 8, 256, None, True, True, False),       # full-size rows, one bias shared by the batch
    (3, 2, 256, None, True, False, False),      # full bias tensor
    (2, 4, 51, None, False, False, False),      # dev size without bias (51 keys: zero-filled tail, masked)
    (2, 2, 300, None, True, False, False),      # three key tiles: both S / O buffers are reused
    (2, 3, 100, 76, True, False, False),        # Lq != Lk
    (1, 2, 1, 40, False, False, False),         # one query over 40 keys (global column attention)
    (2, 2, 200, None, False, False, True),      # causal
])
def test_attention_tensor_cores(oracle, B, h, L, Lk, bias, bcast, causal):
    Q, K, V, bi = cases.attn_case(B, h, L, 32, Lk=Lk, seed=3, bias=bias, bias_bcast=bcast)
    scale = 1 / np.sqrt(32.0)
    O, LSE = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), None if bi is None else dev(bi), scale=scale, bias_bcast=bcast,
                                         causal=causal, path=PATH_UMMA)
    rO, rL = oracle.flash_attn(Q, K, V, bi, scale=scale, bias_bcast=bcast, causal=causal)
    assert cases.rel_err(host(O), rO) <= TOL_TF32
    assert np.abs(host(LSE) - rL).max() <= 2e-3
    if not causal:
        assert cases.rel_err(host(O), oracle.attention_legacy(Q, K, V, bi, scale, bias_bcast=bcast)) <= TOL_TF32


def test_attention_tensor_cores_masked_rows():
    Q, K, V, bi = cases.attn_case(1, 1, 8, 32, Lk=8, seed=7)
    bi[0, 0, 2, :] = -np.inf                     # fully masked row
    bi[0, 0, 5, :4] = -np.inf                    # partly masked row
    O, LSE = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), dev(bi), path=PATH_UMMA)
    O, LSE = host(O), host(LSE)
    assert np.all(O[0, 0, 2] == 0) and LSE[0, 0, 2] == -np.inf and np.isfinite(O).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,h,L,d,Lk,bias,bcast,causal", [
    (4, 8, 256, 32, None, True, True, False),      # full-size rows, one bias shared by the batch
    (3, 2, 256, 32, None, True, False, False),     # full bias tensor
    (2, 4, 51, 32, None, False, False, False),     # dev size without bias (zero-filled key tail, masked)
    (2, 2, 300, 32, None, True, False, False),     # three key tiles: every ring wraps
    (2, 3, 100, 32, 76, True, False, False),       # Lq != Lk
    (2, 2, 200, 32, None, False, False, True),     # causal
    (2, 2, 40, 8, None, True, False, False),       # head dim 8: CUDA-core kernel on 16-bit operands
])
def test_attention_16bit(oracle, dtype, B, h, L, d, Lk, bias, bcast, causal):
    """16-bit Q/K/V: against the fp32 checker fed the rounded operands (P is rounded to 16 bits on the tensor-core
    path, hence 1e-2 there) and against the unrounded ones (1e-2)."""
    Q, K, V, bi = cases.attn_case(B, h, L, d, Lk=Lk, seed=5, bias=bias, bias_bcast=bcast)
    scale = 1 / np.sqrt(32.0)
    q16, k16, v16 = dev(Q).to(dtype), dev(K).to(dtype), dev(V).to(dtype)
    r16, l16 = oracle.flash_attn(host(q16.float()), host(k16.float()), host(v16.float()), bi, scale=scale, bias_bcast=bcast,
                                 causal=causal)
    r32, _ = oracle.flash_attn(Q, K, V, bi, scale=scale, bias_bcast=bcast, causal=causal)
    b = None if bi is None else dev(bi)
    for path in (PATH_SIMT, PATH_AUTO) + ((PATH_UMMA,) if d == 32 else ()):
        O, LSE = ops.flash_attn_forward_cuda(q16, k16, v16, b, scale=scale, bias_bcast=bcast, causal=causal, path=path)
        tol = TOL_FP32 if (path == PATH_SIMT or d != 32) else 1e-2
        assert cases.rel_err(host(O), r16) <= tol, (path, cases.rel_err(host(O), r16))
        assert np.abs(host(LSE) - l16).max() <= (1e-5 if tol == TOL_FP32 else 2e-3)
        assert cases.rel_err(host(O), r32) <= 1e-2
    if d != 32:
        with pytest.raises(RuntimeError):
            ops.flash_attn_forward_cuda(q16, k16, v16, b, scale=scale, path=PATH_UMMA)


def test_attention_output_at_16_byte_offset(oracle):
    """The destination only has to be 16-byte aligned: an address that is not a multiple of 32 takes the 128-bit stores."""
    import torch
    Q, K, V, bi = cases.attn_case(2, 2, 100, 32, seed=11)
    buf = torch.zeros(Q.size + 8, device="cuda", dtype=torch.float32)
    out = buf[4:4 + Q.size].view(*Q.shape)
    assert out.data_ptr() % 32 == 16
    O, _ = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), dev(bi), scale=1 / np.sqrt(32.0), path=PATH_UMMA, out=out)
    rO, _ = oracle.flash_attn(Q, K, V, bi, scale=1 / np.sqrt(32.0))
    assert cases.rel_err(host(O), rO) <= TOL_TF32
    assert float(buf[:4].abs().max()) == 0 and float(buf[-4:].abs().max()) == 0


@pytest.mark.parametrize("d,L,Lk,path", [(32, 100, 200, PATH_UMMA), (32, 100, 200, PATH_SIMT), (8, 100, 200, PATH_SIMT),
                                         (8, 100, 200, PATH_UMMA), (8, 5, 200, PATH_AUTO), (64, 40, 136, PATH_AUTO)])
def test_attention_first_key_tile_masked(oracle, d, L, Lk, path):
    """A query row whose first 64 scores (the reference's first key tile) are all -inf: the reference's CPU kernel turns
    it into O = 0, LSE = -inf although later keys are visible (src/ops/FlashAttn.cpp:94-121); every kernel here does the
    same.  A row with 63 masked keys is an ordinary row.  Bc < 0 switches the rule off and gives the softmax over the
    visible keys."""
    Q, K, V, bi = cases.attn_masked_first_tile_case(d=d, L=L, Lk=Lk)
    scale = 1 / np.sqrt(32.0)
    tol_o, tol_l = (TOL_TF32, 2e-3) if path == PATH_UMMA else (TOL_FP32, 1e-5)
    O, LSE = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), dev(bi), scale=scale, path=path)
    rO, rL = oracle.flash_attn(Q, K, V, bi, scale=scale)
    O, LSE = host(O), host(LSE)
    assert np.all(rO[:, :, 3] == 0) and np.all(rL[:, :, 3] == -np.inf)      # what the reference does
    assert np.all(rO[:, :, 2] == 0) and np.any(rO[:, :, 4] != 0)
    assert np.all(O[:, :, 3] == 0) and np.all(LSE[:, :, 3] == -np.inf) and np.all(O[:, :, 2] == 0)
    assert np.isfinite(O).all() and cases.rel_err(O, rO) <= tol_o
    if (d, L, Lk) == (8, 100, 200):
        assert cases.rel_err(O, GOLD["fa_masked_O"]) <= tol_o       # produced by the reference's own CPU code
    fin = np.isfinite(rL)
    assert np.array_equal(np.isfinite(LSE), fin) and np.abs(LSE[fin] - rL[fin]).max() <= tol_l
    # rule off: the defined softmax (checked against torch)
    O2, LSE2 = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), dev(bi), scale=scale, path=path, Bc=-1)
    s = torch.einsum("bhid,bhjd->bhij", dev(Q), dev(K)) * scale + dev(bi)
    ref2 = torch.einsum("bhij,bhjd->bhid", torch.softmax(s, dim=-1), dev(V))
    assert float((O2 - ref2).abs().max() / ref2.abs().max()) <= max(tol_o, 1e-5)
    assert float((LSE2 - torch.logsumexp(s, dim=-1)).abs().max()) <= max(tol_l, 1e-4)


@pytest.mark.parametrize("B,h,L,d,causal,bias,bcast,masked", [
    (2, 3, 45, 32, False, True, False, (5, 17)),     # the golden case: two fully masked rows
    (2, 3, 45, 32, True, False, False, ()),          # causal, no bias (golden)
    (2, 8, 51, 32, False, True, True, ()),           # dev size, one bias for every batch
    (3, 8, 100, 8, False, True, False, (0,)),        # extra-MSA heads
    (2, 2, 70, 64, True, True, False, ()),           # d = 64 (two channels per lane), causal with bias
    (1, 4, 256, 32, False, True, True, ()),          # main-track size of one batch
    (2, 2, 33, 20, False, False, False, ()),         # a head dim that is no power of two, one row past a tile
])
def test_attention_backward(oracle, B, h, L, d, causal, bias, bcast, masked):
    """flash_attn_backward against the restated CPU routine of the reference (src/ops/FlashAttn.cpp:144-216) on the
    forward's own O and LSE; exact fp32 kernels, 1e-5 of the largest gradient entry."""
    Q, K, V, bi, dO = cases.attn_backward_case(B, h, L, d, seed=7, bias=bias, bias_bcast=bcast, masked_rows=masked)
    scale = 1 / np.sqrt(32.0)
    O, LSE = oracle.flash_attn(Q, K, V, bi, scale=scale, causal=causal, bias_bcast=bcast)
    ref = oracle.flash_attn_backward(Q, K, V, O, dO, LSE, bi, scale=scale, causal=causal, bias_bcast=bcast)
    got = ops.flash_attn_backward_cuda(dev(Q), dev(K), dev(V), dev(O), dev(dO), dev(LSE), (dev(bi) if bi is not None else None), scale=scale, causal=causal,
                                       bias_bcast=bcast)
    for n in ("dQ", "dK", "dV", "dbias"):
        g = host(got[n])
        assert np.isfinite(g).all(), n
        assert cases.rel_err(g, ref[n]) <= TOL_FP32, (n, cases.rel_err(g, ref[n]))
    for r in masked:
        assert np.all(host(got["dQ"])[:, :, r] == 0) and np.all(host(got["dbias"])[:, :, r] == 0)
    if causal:
        assert np.all(np.triu(host(got["dbias"])[0, 0], 1) == 0)
    if (B, h, L, d) == (2, 3, 45, 32):
        tag = "fab_causal_" if causal else "fab_"
        for n in ("dQ", "dK", "dV", "dbias"):
            assert cases.rel_err(host(got[n]), GOLD[tag + n]) <= TOL_FP32       # produced by the reference's own CPU code
    # only some gradients wanted: the others are not touched, the wanted ones do not change
    part = ops.flash_attn_backward_cuda(dev(Q), dev(K), dev(V), dev(O), dev(dO), dev(LSE), (dev(bi) if bi is not None else None), scale=scale, causal=causal,
                                        bias_bcast=bcast, want=("dV", "dQ"))
    assert sorted(part) == ["dQ", "dV"]
    assert torch.equal(part["dV"], got["dV"]) and torch.equal(part["dQ"], got["dQ"])


def test_attention_backward_from_the_cuda_forward(oracle):
    """Forward on the tensor cores, backward on its O and LSE: the chain a training step runs (1e-3: the forward is tf32)."""
    Q, K, V, bi, dO = cases.attn_backward_case(2, 8, 128, 32, seed=9, bias_bcast=True)
    scale = 1 / np.sqrt(32.0)
    O, LSE = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), (dev(bi) if bi is not None else None), scale=scale, bias_bcast=True)
    got = ops.flash_attn_backward_cuda(dev(Q), dev(K), dev(V), O, dev(dO), LSE, (dev(bi) if bi is not None else None), scale=scale, bias_bcast=True)
    rO, rL = oracle.flash_attn(Q, K, V, bi, scale=scale, bias_bcast=True)
    ref = oracle.flash_attn_backward(Q, K, V, rO, dO, rL, bi, scale=scale, bias_bcast=True)
    for n in ("dQ", "dK", "dV", "dbias"):
        assert cases.rel_err(host(got[n]), ref[n]) <= 2 * TOL_TF32, n


def test_backward_shapes_of_a_linear(oracle):
    """The two products a Linear's backward sends through the same entries (src/backend/CUDAKernels.cpp:823): the input
    gradient dX = dY W is a mul_mat against the transposed weight, the weight gradient dW = dY^T X is an out_prod whose
    contraction runs over the tokens."""
    M, K, N = 2601, 128, 256                          # tokens, in features, out features (a dev-size pair Linear)
    r = cases.rng(17)
    X = r.standard_normal((M, K)).astype(np.float32)
    W = (r.standard_normal((N, K)) * 0.02).astype(np.float32)
    dY = r.standard_normal((M, N)).astype(np.float32)
    dX = host(ops.mul_mat_cuda(dev(dY), dev(np.ascontiguousarray(W.T)), path=PATH_SIMT))          # [M, N] x [K, N]^T
    assert cases.rel_err(dX, oracle.mul_mat_f32(dY, np.ascontiguousarray(W.T))) <= TOL_FP32
    dXt = host(ops.mul_mat_cuda(dev(dY), dev(np.ascontiguousarray(W.T)), path=PATH_UMMA))
    assert cases.rel_err(dXt, dX) <= TOL_TF32
    # dW[n][k] = sum_m dY[m][n] X[m][k]: out_prod of the planes [tokens][N] and [tokens][K]
    s0 = np.ascontiguousarray(X.reshape(1, 1, M, K)); s1 = np.ascontiguousarray(dY.reshape(1, 1, M, N))
    dW = host(ops.out_prod_cuda(dev(s0), dev(s1)))[0, 0]
    ref = oracle.out_prod(s0, s1)[0, 0]
    assert dW.shape == (N, K) and cases.rel_err(dW, ref) <= TOL_TF32
    assert cases.rel_err(dW, dY.T.astype(np.float64) @ X.astype(np.float64)) <= TOL_TF32


@pytest.mark.parametrize("B,h,L,d,Lk,bias,path,tol,ltol", [
    (3, 8, 256, 32, None, True, PATH_UMMA, TOL_TF32, 2e-3),      # main-track heads on the tensor cores
    (2, 8, 51, 32, None, True, PATH_AUTO, TOL_FP32, 1e-5),       # dev size: 51 keys with a bias -> CUDA cores
    (4, 8, 100, 8, None, True, PATH_SIMT, TOL_FP32, 1e-5),       # extra-MSA heads (d = 8): thread-per-row kernel
    (5, 8, 100, 8, None, True, PATH_AUTO, TOL_TF32, 2e-3),       # extra-MSA heads (d = 8): warp-level tensor-core kernel
    (5, 8, 1, 8, 64, False, PATH_AUTO, TOL_FP32, 1e-5),          # global column attention: one query, keys over lanes
    (2, 4, 70, 64, 44, True, PATH_AUTO, TOL_FP32, 1e-5),         # generic kernel
])
def test_attention_on_token_major_operands_with_gate(oracle, B, h, L, d, Lk, bias, path, tol, ltol):
    """The projections' outputs as they lie ([B][L][h*d], here as column ranges of one fused [B][L][4*h*d] buffer) in,
    the gated, head-merged result out -- against the reference's chain: head-split permutes, fused attention in its own
    layout, head-merge permute, act_mul(gate, merged, sigmoid)."""
    from checkers import act_mul_f32
    r = np.random.default_rng(B + L + d)
    hd = h * d
    Lk_ = L if Lk is None else Lk
    qg = (r.standard_normal((B, L, 2 * hd)) / np.sqrt(32.0)).astype(np.float32)        # [q | gate logits]
    kv = (r.standard_normal((B, Lk_, 2 * hd)) / np.sqrt(32.0)).astype(np.float32)      # [k | v]
    qg[..., hd:] *= 4.0
    bi = r.standard_normal((h, L, Lk_)).astype(np.float32) if bias else None
    scale = 1 / np.sqrt(32.0)
    split = lambda t, n: np.ascontiguousarray(t.reshape(t.shape[0], n, h, d).transpose(0, 2, 1, 3))   # [B][h][n][d]
    rO, rL = oracle.flash_attn(split(qg[..., :hd], L), split(kv[..., :hd], Lk_), split(kv[..., hd:], Lk_), bi, scale=scale,
                               bias_bcast=bias)
    merged = np.ascontiguousarray(rO.transpose(0, 2, 1, 3)).reshape(B, L, hd)
    ref = act_mul_f32(qg[..., hd:], merged, "sigmoid")
    QG, KV = dev(qg), dev(kv)
    O, LSE = ops.flash_attn_tokens(QG[..., :hd], KV[..., :hd], KV[..., hd:], h, bias=None if bi is None else dev(bi),
                                   gate=QG[..., hd:], act="sigmoid", scale=scale, bias_bcast=bias, path=path)
    assert cases.rel_err(host(O), ref) <= tol
    assert np.abs(host(LSE) - rL).max() <= ltol
    O2, _ = ops.flash_attn_tokens(QG[..., :hd], KV[..., :hd], KV[..., hd:], h, bias=None if bi is None else dev(bi),
                                  scale=scale, bias_bcast=bias, path=path)             # without the gate
    assert cases.rel_err(host(O2), merged) <= tol


def test_attention_fully_masked_row():
    Q, K, V, bi = cases.attn_case(1, 1, 4, 8, seed=7)
    bi[0, 0, 2, :] = -np.inf
    O, LSE = ops.flash_attn_forward_cuda(dev(Q), dev(K), dev(V), dev(bi))
    O, LSE = host(O), host(LSE)
    assert np.all(O[0, 0, 2] == 0) and LSE[0, 0, 2] == -np.inf and np.isfinite(O).all()


# ------------------------------------------------------------------------------------------------
# pair-track contractions
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("path,tol", [(PATH_SIMT, TOL_FP32), (PATH_AUTO, TOL_TF32)])
def test_tri_mul_golden(oracle, path, tol):
    l, r = cases.tri_case(6, 20, 24, 28, outgoing=True)
    assert cases.rel_err(host(ops.tri_mul_cuda(dev(l), dev(r), 28.0, True, path=path)), GOLD["tri_out"]) <= tol
    l, r = cases.tri_case(6, 20, 24, 28, outgoing=False)
    assert cases.rel_err(host(ops.tri_mul_cuda(dev(l), dev(r), 28.0, False, path=path)), GOLD["tri_in"]) <= tol
    l, r = cases.tri_case(3, 5, 6, 7, B=2, outgoing=True, seed=44)
    assert cases.rel_err(host(ops.tri_mul_cuda(dev(l), dev(r), 7.0, True, path=path)), GOLD["tri_out_b2"]) <= tol
    l = np.full((1, 2, 2, 1), 3e3, np.float32)
    assert np.array_equal(host(ops.tri_mul_cuda(dev(l), dev(l), 1.0, True, path=path)), GOLD["tri_clamp"])
    l, r = cases.tri_case(1, 2, 2, 3)
    l[0, 0, 1, 0] = np.nan
    got = host(ops.tri_mul_cuda(dev(l), dev(r), 3.0, True, path=path))
    assert np.all(got[0, 0] == 0) and np.isfinite(got).all()


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("L", [51, 128])
def test_tri_mul_model_shapes(oracle, outgoing, L):
    l, r = cases.tri_case(16, L, L, L, outgoing=outgoing)
    ref = oracle.tri_mul(l, r, float(L), outgoing)
    assert cases.rel_err(host(ops.tri_mul_cuda(dev(l), dev(r), float(L), outgoing, path=PATH_SIMT)), ref) <= TOL_FP32
    assert cases.rel_err(host(ops.tri_mul_cuda(dev(l), dev(r), float(L), outgoing, path=PATH_AUTO)), ref) <= TOL_TF32


@pytest.mark.parametrize("outgoing", [True, False])
def test_tri_mul_tensor_core_ragged(oracle, outgoing):
    """I, J, K not multiples of the tile (I, J multiples of 4 for the 16-byte rule): zero fill at every edge."""
    for (D, I, J, K) in [(5, 132, 36, 44), (3, 260, 300, 100)]:
        l, r = cases.tri_case(D, I, J, K, outgoing=outgoing, seed=D)
        ref = oracle.tri_mul(l, r, float(K), outgoing)
        assert cases.rel_err(host(ops.tri_mul_cuda(dev(l), dev(r), float(K), outgoing, path=PATH_UMMA)), ref) <= TOL_TF32


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("outgoing", [True, False])
def test_tri_mul_16bit(oracle, dtype, outgoing):
    """16-bit operands: against the fp32 checker fed the rounded operands (1e-5) and the unrounded ones (1e-2)."""
    for (D, I, J, K) in [(4, 128, 128, 128), (3, 136, 72, 40), (2, 256, 256, 256)]:
        l, r = cases.tri_case(D, I, J, K, outgoing=outgoing, seed=11 + D)
        l16, r16 = dev(l).to(dtype), dev(r).to(dtype)
        ref16 = oracle.tri_mul(host(l16.float()), host(r16.float()), float(K), outgoing)
        ref32 = oracle.tri_mul(l, r, float(K), outgoing)
        for path in (PATH_SIMT, PATH_UMMA, PATH_AUTO):
            got = host(ops.tri_mul_cuda(l16, r16, float(K), outgoing, path=path))
            assert cases.rel_err(got, ref16) <= TOL_FP32, (D, I, J, K, path)
            assert cases.rel_err(got, ref32) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_outer_prod_mean_16bit(oracle, dtype):
    for (D, L, N) in [(4, 40, 64), (8, 51, 8), (16, 64, 256)]:
        l, r = cases.opm_case(D, L, N, seed=5 + D)
        l16, r16 = dev(l).to(dtype), dev(r).to(dtype)
        ref16 = oracle.outer_prod_mean(host(l16.float()), host(r16.float()))
        for path in (PATH_SIMT, PATH_AUTO):
            got = host(ops.outer_prod_mean_cuda(l16, r16, path=path))
            assert cases.rel_err(got, ref16) <= TOL_FP32, (D, L, N, path)
        assert cases.rel_err(got, oracle.outer_prod_mean(l, r)) <= 1e-2


@pytest.mark.parametrize("path,tol", [(PATH_SIMT, TOL_FP32), (PATH_AUTO, TOL_TF32)])
def test_outer_prod_mean_slabs(oracle, path, tol):
    """A d1 range of `left` against all of `right` is the matching contiguous part of the whole result."""
    for (D, L, N, lo, hi) in [(8, 64, 128, 2, 5), (16, 32, 64, 14, 16), (4, 51, 8, 0, 1)]:
        l, r = cases.opm_case(D, L, N, seed=21 + D)
        ref = oracle.outer_prod_mean(l, r)
        got = host(ops.outer_prod_mean_slabs_cuda(dev(l[lo:hi]), dev(r), path=path))
        assert got.shape[0] == (hi - lo) * D
        assert cases.rel_err(got, ref[lo * D:hi * D]) <= tol, (D, L, N, path)


@pytest.mark.parametrize("path,tol", [(PATH_SIMT, TOL_FP32), (PATH_AUTO, TOL_TF32)])
def test_outer_prod_mean(oracle, path, tol):
    l, r = cases.opm_case(4, 12, 9)
    assert cases.rel_err(host(ops.outer_prod_mean_cuda(dev(l), dev(r), path=path)), GOLD["opm"]) <= tol
    l, r = cases.opm_case(8, 51, 8)                                  # dev size: D*L = 408, N = 8
    assert cases.rel_err(host(ops.outer_prod_mean_cuda(dev(l), dev(r), path=path)), oracle.outer_prod_mean(l, r)) <= tol
    l, r = cases.opm_case(4, 40, 64, B=2, seed=9)
    assert cases.rel_err(host(ops.outer_prod_mean_cuda(dev(l), dev(r), path=path)), oracle.outer_prod_mean(l, r, B=2)) <= tol


def test_out_prod(oracle):
    s0, s1 = cases.out_prod_case(13, 11, 17, 3, 2)
    assert cases.rel_err(host(ops.out_prod_cuda(dev(s0), dev(s1))), GOLD["out_prod"]) <= TOL_FP32
    s0, s1 = cases.out_prod_case(13, 11, 17, 4, 2, ne02=2, ne03=1)
    assert cases.rel_err(host(ops.out_prod_cuda(dev(s0), dev(s1))), GOLD["out_prod_bcast"]) <= TOL_FP32
    # the reference's "real shape" case (tests/test_cuda.cpp:262-341): ne0 = ne1 = 51, K = 51, 16 x 64 planes (cut to 16 x 4)
    s0, s1 = cases.out_prod_case(51, 51, 51, 16, 4)
    assert cases.rel_err(host(ops.out_prod_cuda(dev(s0), dev(s1))), oracle.out_prod(s0, s1)) <= TOL_FP32
    # aligned planes go to the tensor cores (both operands with the row index contiguous); K not a multiple of 32
    for (n0, n1, k, p2, p3) in [(64, 48, 40, 3, 2), (256, 132, 256, 2, 1), (20, 36, 7, 1, 1)]:
        s0, s1 = cases.out_prod_case(n0, n1, k, p2, p3)
        ref = oracle.out_prod(s0, s1)
        assert cases.rel_err(host(ops.out_prod_cuda(dev(s0), dev(s1), path=PATH_SIMT)), ref) <= TOL_FP32
        assert cases.rel_err(host(ops.out_prod_cuda(dev(s0), dev(s1), path=PATH_UMMA)), ref) <= TOL_TF32
        assert cases.rel_err(host(ops.out_prod_cuda(dev(s0), dev(s1), path=PATH_AUTO)), ref) <= TOL_TF32
    # known answer of tests/test_cuda.cpp:207-245
    a = (np.arange(12) % 7).astype(np.float32) * 0.5
    b = (np.arange(15) % 9).astype(np.float32) * 0.25 - 1.0
    got = host(ops.out_prod_cuda(dev(a.reshape(1, 1, 3, 4)), dev(b.reshape(1, 1, 3, 5)))).reshape(5, 4)
    for i0 in range(4):
        for i1 in range(5):
            assert abs(got[i1, i0] - sum(float(a[i0 + k * 4]) * float(b[i1 + k * 5]) for k in range(3))) <= 1e-4


def test_attention_full_size_properties():
    """The full-size attention case (MSA depth 256, L = 256, 8 heads x 32, shared pair bias): the tensor-core kernel
    agrees with the CUDA-core kernel, a permutation of the batch permutes the output, and exp(LSE) equals the
    softmax denominator recomputed from one batch's scores."""
    g = torch.Generator(device="cuda").manual_seed(3)
    B, h, L = 256, 8, 256
    Q, K, V = (torch.randn(B, h, L, 32, device="cuda", generator=g) / 32 ** 0.5 for _ in range(3))
    bias = torch.randn(h, L, L, device="cuda", generator=g)
    scale = 1 / 32 ** 0.5
    o_t, l_t = ops.flash_attn_forward_cuda(Q, K, V, bias, scale=scale, bias_bcast=True, path=PATH_UMMA)
    o_s, l_s = ops.flash_attn_forward_cuda(Q, K, V, bias, scale=scale, bias_bcast=True, path=PATH_SIMT)
    assert float((o_t - o_s).abs().max() / o_s.abs().max()) <= TOL_TF32
    assert float((l_t - l_s).abs().max()) <= 2e-3
    perm = torch.randperm(B, device="cuda", generator=g)
    o_p, _ = ops.flash_attn_forward_cuda(Q[perm].contiguous(), K[perm].contiguous(), V[perm].contiguous(), bias, scale=scale,
                                         bias_bcast=True, path=PATH_UMMA)
    assert torch.equal(o_p, o_t[perm])
    s = torch.einsum("hid,hjd->hij", Q[7], K[7]) * scale + bias
    assert float((torch.logsumexp(s, dim=-1) - l_t[7]).abs().max()) <= 2e-3
    o16, _ = ops.flash_attn_forward_cuda(Q.bfloat16(), K.bfloat16(), V.bfloat16(), bias, scale=scale, bias_bcast=True, path=PATH_UMMA)
    assert float((o16 - o_s).abs().max() / o_s.abs().max()) <= TOL_16


def test_pair_track_full_size_properties():
    """The full-size pair-track cases: triangle multiplication over 128 channel slabs at L = 384 and the outer-product-mean
    at c = 32 (8192 x 8192 x 256): tensor cores against CUDA cores, and the slab structure (a slab of the result depends on
    that slab of the operands only)."""
    g = torch.Generator(device="cuda").manual_seed(4)
    D, L = 128, 384
    left, right = torch.randn(D, L, L, 1, device="cuda", generator=g), torch.randn(D, L, L, 1, device="cuda", generator=g)
    for outgoing in (True, False):
        t = ops.tri_mul_cuda(left, right, float(L), outgoing, path=PATH_UMMA)
        s_ = ops.tri_mul_cuda(left, right, float(L), outgoing, path=PATH_SIMT)
        assert float((t - s_).abs().max() / s_.abs().max()) <= TOL_TF32
        part = ops.tri_mul_cuda(left[40:72].contiguous(), right[40:72].contiguous(), float(L), outgoing, path=PATH_UMMA)
        assert torch.equal(part, t[40:72])
    c, Lr, N = 32, 256, 256
    a, b = torch.randn(c, Lr, N, 1, device="cuda", generator=g), torch.randn(c, Lr, N, 1, device="cuda", generator=g)
    full = ops.outer_prod_mean_cuda(a, b, path=PATH_UMMA)
    assert float((full - ops.outer_prod_mean_cuda(a, b, path=PATH_SIMT)).abs().max() / full.abs().max()) <= TOL_TF32
    assert torch.equal(ops.outer_prod_mean_slabs_cuda(a[8:12].contiguous(), b, path=PATH_UMMA), full[8 * c:12 * c])
    d1, d2, i, j = 5, 17, 100, 31                     # one entry against its definition
    ref = float((a[d1, i, :, 0].double() * b[d2, j, :, 0].double()).sum() / N)
    assert abs(float(full[d1 * c + d2, i, j, 0]) - ref) <= 1e-3 * max(1.0, abs(ref))


def test_iter_block_sequence_runs(capsys):
    """The full-size op sequence of one main IterBlock runs on one GPU and reports a time per op class."""
    import json
    from proteinpredictmachinelearning_b200 import block_bench
    block_bench.run(1, 1, 3)
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["value"] > 0 and line["n_gpus"] == 1
    assert {"attention", "linear_q8", "linear_tf32", "tri_mul", "outer_prod_mean"} <= set(line["split_ms_rank0"])
