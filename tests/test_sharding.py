"""The N > 1 host logic on CPU: two gloo ranks shard each op as the GPU ranks do (contiguous flat
chunks), compute their part with the CPU checker, and the gathered result must equal the unsharded
one bit for bit."""
import os
import socket

import numpy as np
import pytest

import cases

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    sys.path.insert(0, os.path.dirname(here))
    from checkers import Oracle
    from proteinpredictmachinelearning_b200 import shard
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    o = Oracle()
    ok = {}

    # token-row sharding: mul_mat and Q8 mul_mat
    a, b, bi = cases.mul_mat_case(102, 64, 48, seed=1)
    lo, hi = shard.token_rows(102, world, rank)
    part = torch.from_numpy(o.mul_mat_f32(a[lo:hi], b, bi))
    full = shard.all_gather_rows(part, world).numpy()
    ok["mul_mat"] = np.array_equal(full, o.mul_mat_f32(a, b, bi))

    w, x = cases.q8_case(40, 64, 128, seed=2)
    W = o.repack_q8_0(o.quantize_q8_0(w))
    lo, hi = shard.token_rows(64, world, rank)
    full = shard.all_gather_rows(torch.from_numpy(o.mul_mat_q8(W, x[lo:hi], 40)), world).numpy()
    ok["q8"] = np.array_equal(full, o.mul_mat_q8(W, x, 40))

    # attention: batch sharding with one bias shared by all ranks
    Q, K, V, bias = cases.attn_case(6, 2, 20, 8, seed=3, bias_bcast=True)
    lo, hi = shard.attention_batches(6, world, rank)
    O, _ = o.flash_attn(Q[lo:hi], K[lo:hi], V[lo:hi], bias, bias_bcast=True)
    full = shard.all_gather_rows(torch.from_numpy(O), world).numpy()
    ok["attn"] = np.array_equal(full, o.flash_attn(Q, K, V, bias, bias_bcast=True)[0])

    # triangle multiplication: channel slabs, no exchange
    l, r = cases.tri_case(8, 10, 10, 10, outgoing=False)
    lo, hi = shard.tri_mul_slabs(8, world, rank)
    full = shard.all_gather_rows(torch.from_numpy(o.tri_mul(l[lo:hi], r[lo:hi], 10.0, False)), world).numpy()
    ok["tri"] = np.array_equal(full, o.tri_mul(l, r, 10.0, False))

    # outer-product-mean: rank owns slabs d1 of `left`; `right` is all-gathered from the ranks' shards
    D, L, N = 4, 6, 5
    left, right = cases.opm_case(D, L, N)
    lo, hi = shard.opm_slabs(D, world, rank)
    right_full = shard.all_gather_rows(torch.from_numpy(right[lo:hi].copy()), world).numpy()
    ok["opm_gather"] = np.array_equal(right_full, right)
    ref = o.outer_prod_mean(left, right).reshape(D, D, L, L)
    mine = np.empty((hi - lo, D, L, L), np.float32)
    for d1 in range(lo, hi):                       # block (d1, :) = one (L x N) x (D*L x N)^T product
        blk = o.mul_mat_f32(left[d1, :, :, 0], right_full[:, :, :, 0].reshape(D * L, N)) * np.float32(1.0 / N)
        mine[d1 - lo] = blk.reshape(L, D, L).transpose(1, 0, 2)
    full = shard.all_gather_rows(torch.from_numpy(mine), world).numpy()
    ok["opm"] = np.array_equal(full, ref)

    # the (n, l) transpose that closes MSA column attention and pair row attention: one all-to-all plus local re-layouts
    Nn, Ll, Cc = 6, 8, 3
    x = np.arange(Nn * Ll * Cc, dtype=np.float32).reshape(Nn, Ll, Cc)
    lo, hi = shard.split(Nn, world, rank)
    mine = shard.transpose_exchange(torch.from_numpy(x[lo:hi].copy()), world)
    full = shard.all_gather_rows(mine, world).numpy()
    ok["transpose"] = np.array_equal(full, x.transpose(1, 0, 2))

    # unequal shards (7 rows over 2 ranks: 4 + 3) must be refused on every rank, not entered into a collective
    lo, hi = shard.split(7, world, rank)
    part = torch.zeros((hi - lo, 5))
    try:
        shard.all_gather_rows(part, world)
        ok["unequal_gather_refused"] = False
    except ValueError:
        ok["unequal_gather_refused"] = True
    try:
        shard.transpose_exchange(torch.zeros((hi - lo, 4, 2)), world)
        ok["unequal_transpose_refused"] = False
    except ValueError:
        ok["unequal_transpose_refused"] = True

    if rank == 0:
        q.put(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok.values()), ok


def test_split_properties():
    from proteinpredictmachinelearning_b200 import shard
    for total in (0, 1, 7, 128, 65536):
        for world in (1, 2, 4, 8):
            for align in (1, 16):
                parts = [shard.split(total, world, r, align) for r in range(world)]
                assert parts[0][0] == 0 and parts[-1][1] == total
                for (a0, a1), (b0, b1) in zip(parts, parts[1:]):
                    assert a1 == b0 and a0 <= a1
                assert all(lo % align == 0 or lo == total for lo, _ in parts)
    with pytest.raises(ValueError):
        shard.split(10, 2, 2)


@pytest.mark.gpu
def test_peer_exchange_kernels_on_one_rank():
    """The exchange kernels with a world of one rank (the flag rounds see only the rank itself): the all-gather is a copy,
    the (n, l) transpose a local transpose; repeated launches advance the epoch, also when replayed from a CUDA graph."""
    from proteinpredictmachinelearning_b200 import ops, shard
    peers = shard.PeerBuffers(1, 0)
    try:
        g = torch.Generator(device="cuda").manual_seed(1)
        x = torch.randn((6, 8, 12), device="cuda", generator=g)
        out, out_ptrs = peers.tensor((8, 6, 12))
        gat, gat_ptrs = peers.tensor((6, 8, 12))
        for _ in range(3):
            peers.transpose(x, out_ptrs, 6, 8, 12, site=1)
            peers.all_gather(x, gat_ptrs, site=0)
        torch.cuda.synchronize()
        assert torch.equal(out, x.permute(1, 0, 2).contiguous()) and torch.equal(gat, x)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            peers.transpose(x, out_ptrs, 6, 8, 12, site=1)
        x.mul_(2.0)
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, x.permute(1, 0, 2).contiguous())
        assert ops.device_status() == (0, 0)
        del out, gat
    finally:
        peers.close()
