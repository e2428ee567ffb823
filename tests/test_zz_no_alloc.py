"""The allocation-free Q8 entry point (ppml_b200_mul_mat_q8_noalloc), through the C ABI.

It exists for callers that cannot allocate device memory when they need the product (an executor with a
pre-planned arena, a fixed memory budget, another allocator owning the free memory); its scratch is a fixed
array inside the library.  Two calls in a row must each match the regular entry point's CUDA-core path --
the same kernels, so the results are compared bit for bit (and within the suite's fp32 tolerance of 1e-5
against the CPU checker) -- which also shows that the second call is not disturbed by what the first one
left in the shared array.  This file is collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

import cases

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_noalloc_matches_regular_entry_twice(oracle):
    from proteinpredictmachinelearning_b200 import PATH_SIMT, ops
    free_before = None
    for call, (Mout, Ntok, K, seed) in enumerate([(256, 408, 256, 21), (136, 257, 96, 22)]):
        w, x = cases.q8_case(Mout, Ntok, K, seed=seed)
        W = oracle.repack_q8_0(oracle.quantize_q8_0(w))
        bias = (np.random.default_rng(seed).standard_normal(Mout) * 0.1).astype(np.float32)
        Wd, Xd, Bd = _dev(W), _dev(x), _dev(bias)
        ref, _ = ops.mul_mat_q8_cuda(Wd, Xd, Mout, bias=Bd, path=PATH_SIMT)
        out = torch.empty_like(ref)
        torch.cuda.synchronize()
        if call == 1:
            free_before = torch.cuda.mem_get_info()[0]
        got = ops.mul_mat_q8_noalloc(Wd, Xd, Mout, bias=Bd, out=out)
        torch.cuda.synchronize()
        if call == 1:
            assert torch.cuda.mem_get_info()[0] == free_before      # no device allocation happened
        assert torch.equal(got, ref)
        assert cases.rel_err(got.cpu().numpy(), oracle.mul_mat_q8(W, x, Mout, bias=bias)) <= 1e-5
    code, where = ops.device_status()
    assert code == 0, (code, hex(where))


def test_noalloc_rejects_problems_beyond_the_fixed_array(lib):
    from proteinpredictmachinelearning_b200._lib import NOALLOC_SCRATCH_BYTES as cap
    p = C.c_void_p(256)
    n_tok = cap // (1024 // 32 * 36) + 1            # one token row too many at K = 1024
    assert lib.ppml_b200_mul_mat_q8_noalloc(p, p, p, 128, n_tok, 1024, 2, 1, None, None) == 9
    assert lib.ppml_b200_mul_mat_q8_noalloc(p, p, p, 128, 16, 48, 2, 1, None, None) == 2     # K % 32
    assert lib.ppml_b200_mul_mat_q8_noalloc(None, p, p, 128, 16, 64, 2, 1, None, None) == 1
