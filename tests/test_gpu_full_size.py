"""Full-size workloads against the CPU checker on sampled units.

Token rows (mul_mat, Q8), attention batches, triangle-multiplication slabs and outer-product-mean blocks are
independent under the reference's semantics, so the checker only has to compute a sample of them: the CUDA path
runs the whole problem at the benchmark's size, the sampled units are copied back and compared with
oracle/ppml_oracle.c on exactly those units' inputs.  Tolerances as in test_gpu_parity.py; int32 block sums and
everything else integer bit-exact.

Covered: all 36 shapes of the Q8 sweep (seed 2), the three axial-attention cases (seed 3; fp32 and bf16 operands),
triangle multiplication at L = 256 and 384 and the outer-product-mean at c = 32 (seed 4)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from proteinpredictmachinelearning_b200 import PATH_AUTO, PATH_UMMA, TF32_TMA, ops  # noqa: E402

import cases  # noqa: E402

TOL_FP32, TOL_TF32, TOL_16 = 1e-5, 1e-3, 1e-2


def host(t):
    return t.detach().cpu().numpy()


@pytest.fixture(autouse=True)
def _no_device_abort():
    yield
    code, where = ops.device_status()
    assert code == 0, f"a kernel gave up a bounded wait: code {code} at site {where:#x}"


SWEEP = [(M, K, N) for M in (408, 2601, 65536) for K in (128, 256, 1024) for N in (128, 256, 512, 1024)]


def _sample_rows(M, n, seed):
    r = np.random.default_rng(seed)
    rows = np.unique(np.concatenate([[0, M - 1, min(M - 1, 127), min(M - 1, 128)], r.integers(0, M, n)]))
    return rows


@pytest.mark.parametrize("M,K,N", SWEEP)
def test_q8_sweep_shape_against_oracle_on_sampled_rows(oracle, M, K, N):
    """Every shape of the benchmark's sweep: the timed kernel instance (no block-sum output) and the instance that also
    writes the int32 block sums, both at full size, compared with the checker on 256 sampled token rows."""
    g = torch.Generator(device="cuda").manual_seed(2)
    X = torch.randn((M, K), device="cuda", generator=g)
    w = (np.random.default_rng(2).standard_normal((N, K)) * 0.02).astype(np.float32)
    W = oracle.repack_q8_0(oracle.quantize_q8_0(w))
    Wd = torch.from_numpy(W).cuda()
    assert np.array_equal(host(ops.quantize_q8_0r(torch.from_numpy(w).cuda())), W)      # device weight prep == checker's
    rows = _sample_rows(M, 256, seed=M + K + N)
    xs = host(X[torch.from_numpy(rows).cuda()])
    ref, ref_sumi = oracle.mul_mat_q8(W, xs, N, wtype=2, c_trans=1, want_sumi=True)
    got, taken = ops.mul_mat_q8_cuda(Wd, X, N, path=PATH_UMMA)
    assert taken == 1
    assert cases.rel_err(host(got[torch.from_numpy(rows).cuda()]), ref) <= TOL_FP32
    got2, taken2, sumi = ops.mul_mat_q8_cuda(Wd, X, N, path=PATH_UMMA, want_sumi=True)
    idx = torch.from_numpy(rows).cuda()
    assert np.array_equal(host(sumi[idx]), ref_sumi)                                      # int32 block sums: bit-exact
    assert cases.rel_err(host(got2[idx]), ref) <= TOL_FP32
    del sumi


@pytest.mark.parametrize("M,K,N", [(65536, 256, 256), (65536, 1024, 1024), (65536, 128, 1024), (2601, 1024, 512)])
@pytest.mark.parametrize("kind", ["tf32", "bf16", "f32_as_bf16"])
def test_mul_mat_sweep_shape_against_oracle_on_sampled_rows(oracle, M, K, N, kind):
    g = torch.Generator(device="cuda").manual_seed(2)
    A = torch.randn((M, K), device="cuda", generator=g)
    Bw = torch.randn((N, K), device="cuda", generator=g) * 0.02
    bias = torch.randn((N,), device="cuda", generator=g) * 0.1
    rows = _sample_rows(M, 128, seed=M + K + N)
    idx = torch.from_numpy(rows).cuda()
    ref32 = oracle.mul_mat_f32(host(A[idx]), host(Bw), host(bias))
    if kind == "tf32":
        got = ops.mul_mat_cuda(A, Bw, bias, path=PATH_UMMA, tf32_mode=TF32_TMA)
        assert cases.rel_err(host(got[idx]), ref32) <= TOL_TF32
    elif kind == "bf16":
        a16, b16 = A.bfloat16(), Bw.bfloat16()
        got = ops.mul_mat_16(a16, b16, bias, path=PATH_UMMA)
        ref16 = oracle.mul_mat_f32(host(a16[idx].float()), host(b16.float()), host(bias))
        assert cases.rel_err(host(got[idx]), ref16) <= TOL_FP32
        assert cases.rel_err(host(got[idx]), ref32) <= TOL_16
    else:
        got = ops.mul_mat_f32_as_bf16(A, Bw, bias, path=PATH_UMMA)
        ref16 = oracle.mul_mat_f32(host(A[idx].bfloat16().float()), host(Bw.bfloat16().float()), host(bias))
        assert cases.rel_err(host(got[idx]), ref16) <= TOL_FP32
        assert cases.rel_err(host(got[idx]), ref32) <= TOL_16
        again = ops.mul_mat_f32_as_bf16(A, Bw, bias, path=PATH_UMMA)        # second call: the cached weight copy
        assert torch.equal(again, got)
        ops.bf16_shadow_invalidate(Bw)


# (name, batches B', heads, L, bias shared over the batch?)
ATTN_CASES = [("msa_row", 256, 8, 256, True), ("msa_col", 256, 8, 256, None), ("pair_h8", 256, 8, 256, True),
              ("pair_h4", 256, 4, 256, True)]


@pytest.mark.parametrize("name,B,h,L,bias", ATTN_CASES)
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_attention_full_size_against_oracle_on_sampled_batches(oracle, name, B, h, L, bias, dtype):
    g = torch.Generator(device="cuda").manual_seed(3)
    Q, K, V = (torch.randn(B, h, L, 32, device="cuda", generator=g) / 32 ** 0.5 for _ in range(3))
    bi = torch.randn(h, L, L, device="cuda", generator=g) if bias else None
    scale = 1 / 16 ** 0.5 if name.startswith("pair") else 1 / 32 ** 0.5      # the pair track scales by 1/sqrt(16)
    if dtype == "bf16":
        Q, K, V = Q.bfloat16(), K.bfloat16(), V.bfloat16()
    O, LSE = ops.flash_attn_forward_cuda(Q, K, V, bi, scale=scale, bias_bcast=bias is not None, path=PATH_UMMA)
    for b in (0, B // 2 + 1, B - 1)[:2 if dtype == "bf16" else 3]:
        q, k, v = (host(t[b:b + 1].float()) for t in (Q, K, V))
        rO, rL = oracle.flash_attn(q, k, v, None if bi is None else host(bi), scale=scale, bias_bcast=bias is not None)
        tol_o, tol_l = (TOL_TF32, 2e-3) if dtype == "f32" else (TOL_16, 2e-3)
        assert cases.rel_err(host(O[b:b + 1]), rO) <= tol_o, (name, b)
        assert np.abs(host(LSE[b:b + 1]) - rL).max() <= tol_l


@pytest.mark.parametrize("L", [256, 384])
@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_tri_mul_full_size_against_oracle_on_sampled_slabs(oracle, L, outgoing, dtype):
    g = torch.Generator(device="cuda").manual_seed(4)
    D = 128
    left, right = torch.randn(D, L, L, 1, device="cuda", generator=g), torch.randn(D, L, L, 1, device="cuda", generator=g)
    if dtype == "bf16":
        left, right = left.bfloat16(), right.bfloat16()
    got = ops.tri_mul_cuda(left, right, float(L), outgoing, path=PATH_UMMA)
    for d in (0, 77, D - 1)[:2 if L == 384 else 3]:
        ref = oracle.tri_mul(host(left[d:d + 1].float()), host(right[d:d + 1].float()), float(L), outgoing)
        assert cases.rel_err(host(got[d:d + 1]), ref) <= (TOL_TF32 if dtype == "f32" else TOL_FP32), (L, outgoing, d)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_outer_prod_mean_c32_against_oracle_on_sampled_blocks(oracle, dtype):
    """c = 32, L = N = 256: an 8192 x 8192 x 256 product stored as 32 x 32 blocks of L x L; block (d1, d2) is slab d1 of
    `left` against slab d2 of `right`, so the checker computes sampled blocks as one-slab problems."""
    g = torch.Generator(device="cuda").manual_seed(4)
    c, L, N = 32, 256, 256
    left, right = torch.randn(c, L, N, 1, device="cuda", generator=g), torch.randn(c, L, N, 1, device="cuda", generator=g)
    if dtype == "bf16":
        left, right = left.bfloat16(), right.bfloat16()
    full = ops.outer_prod_mean_cuda(left, right, path=PATH_UMMA)
    for (d1, d2) in [(0, 0), (5, 17), (31, 30), (16, 1)]:
        ref = oracle.outer_prod_mean(host(left[d1:d1 + 1].float()), host(right[d2:d2 + 1].float()))
        assert cases.rel_err(host(full[d1 * c + d2:d1 * c + d2 + 1]), ref) <= (TOL_TF32 if dtype == "f32" else TOL_FP32), (d1, d2)
    # the per-rank share (left slabs 8..11 against all of right) is the matching contiguous part of the whole
    if dtype == "f32":
        part = ops.outer_prod_mean_slabs_cuda(left[8:12].contiguous(), right, path=PATH_AUTO)
        assert torch.equal(part, full[8 * c:12 * c])
