"""Host-side plumbing of the block benchmark (no GPU): layer shapes of both block kinds at full and dev size, and the
exchanged bytes per rank, against the reference's layer table (src/model/PPML.cpp:2164-2273)."""
import types

import pytest
import torch

from proteinpredictmachinelearning_b200 import block_bench as bb


def _weights(kind, size):
    ops = types.SimpleNamespace(quantize_q8_0r=lambda w: ("q8", tuple(w.shape)))
    return bb.make_inputs_and_weights(torch, ops, torch.device("cpu"), kind, 2, size=size)


@pytest.mark.parametrize("kind,N,D,hd", [("main", 256, 256, 32), ("extra", 1024, 64, 8)])
def test_full_size_layers(kind, N, D, hd):
    inputs, weights = _weights(kind, "full")
    L = 256
    assert inputs["x_msa"].shape == (N * L, D) and inputs["x_pair"].shape == (L * L, 128)
    # attention projections are on the reference's Q8 list, fused and single
    assert weights[("mrqkvg", D, 4 * 8 * hd, True)][0] == ("q8", (4 * 8 * hd, D))
    assert ("mrq", D, 8 * hd, True) in weights and ("mro", 8 * hd, D, True) in weights
    assert ("prqkvg", 128, 1024, True) in weights and ("pcqkvg", 128, 1024, True) in weights
    for tag in ("mrb", "prb", "pcb"):
        assert (tag, 128, 8, True) in weights                       # pair bias 128 -> 8
    assert ("ol", D, 16, True) in weights and ("or", D, 16, True) in weights and ("oo", 256, 128, True) in weights
    assert ("ff1", D, 4 * D, False) in weights and ("ff2", 4 * D, D, False) in weights
    assert ("tgatesout", 128, 384, False) in weights and ("tlin", 128, 128, False) in weights
    if kind == "main":
        assert ("mcqkvg", D, 1024, True) in weights and "x_qmean" not in inputs
    else:
        # global column attention: fp32 projections, one query per chunk of N flat positions, partial sums per rank
        assert ("gcqkvg", 64, 256, False) in weights and ("gco", 64, 64, False) in weights
        assert inputs["x_qmean"].shape == (L, 64) and inputs["x_qsum"].shape == (2 * L, 64)


@pytest.mark.parametrize("kind", ["main", "extra"])
def test_dev_size_layers_are_fp32(kind):
    inputs, weights = _weights(kind, "dev")
    assert inputs["x_msa"].shape[0] == 51 * 8 and inputs["x_pair"].shape[0] == 51 * 51
    assert all(not key[3] for key in weights)                      # config 0 has no quantized weights
    assert all(not isinstance(w, tuple) for (w, _) in weights.values())


def test_exchange_bytes():
    assert bb.exchange_bytes(1) == {} and bb.exchange_bytes(1, "extra") == {}
    main = bb.exchange_bytes(8)
    assert main["all_to_all MSA (n, l) transpose [N*L, 256] / G"] == 256 * 256 * 256 * 4 // 8 * 7 // 8
    assert main["all_gather outer-product-mean right [N*L, 16]"] == 256 * 256 * 16 * 4 * 7 // 8
    extra = bb.exchange_bytes(8, "extra")
    assert extra["all_gather outer-product-mean right [N*L, 16]"] == 1024 * 256 * 16 * 4 * 7 // 8
    assert not any("MSA (n, l) transpose" in k for k in extra)
    assert extra["all_gather partial sums of the global query [L, 64] per rank"] == 256 * 64 * 4 * 7
