"""The op sequence of the dev-size forward's blocks (51 residues, MSA depth 8, fp32 weights: one extra-MSA block, one main
block), every mul_mat / attention / tri_mul / outer-product-mean call checked against the CPU checker on the tensors the
call saw -- on the exact CUDA-core kernels (what the drop-in forwarders run by default) and on the tensor-core path."""
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("path_name,tol", [("PATH_SIMT", 1e-5), ("PATH_AUTO", 1e-3)])
def test_every_call_of_the_dev_size_blocks(oracle, path_name, tol, fused):
    import torch
    import proteinpredictmachinelearning_b200 as pkg
    from proteinpredictmachinelearning_b200 import block_bench, ops
    from checkers import check_block_calls
    blocks = block_bench.dev_blocks(torch, ops, torch.device("cuda", 0), path=getattr(pkg, path_name), fused=fused)
    n = 0
    for kind, blk in blocks.items():
        calls = check_block_calls(blk.trace, oracle)
        # main: 4 attention calls, 2 tri_mul, 1 outer-product-mean and the Linears around them; extra: the same with global
        # column attention in place of column attention
        assert sum(c["op"].startswith("flash_attn") for c in calls) == 4
        assert sum(c["op"] == "tri_mul" for c in calls) == 2 and sum(c["op"] == "outer_prod_mean" for c in calls) == 1
        assert sum(c["op"] == "mul_mat" for c in calls) >= 26
        for c in calls:
            assert c["err"] <= tol, (kind, c)
        n += len(calls)
    assert n >= 60
