"""Hot-path op sequence of one main IterBlock of the reference model at full size, on 1..8 GPUs of one box.

The block's dense contractions and attention calls (src/model/PPML.cpp:2164-2273 for the layer shapes,
src/model/PPML.cpp:908-994 for the op order, src/modules/Attention.cpp:223-284, :361-392, :468-489, :717-744 for the
attention call sites) at L = 256 residues, MSA depth N = 256, d_msa = 256, d_pair = 128, 8 heads x 32:

  MSA row attention   5 Linears 256->256 on N*L tokens, pair bias Linear 128->8 on L*L tokens, attention
                      (batch N, shared bias [8, L, L], scale 1/sqrt(32))
  MSA column attn     5 Linears 256->256, attention without bias (batch = chunks of N flat positions)
  MSA feed-forward    256->1024, 1024->256
  MSA -> pair         left / right 256->16, outer-product-mean (16 slabs), out 256->128 on L*L tokens
  triangle mult.      out and in: 6 Linears 128->128 each, tri_mul over 128 channel slabs of L x L
  pair row / col attn each: 4 Linears 128->256, bias 128->8, out 256->128, attention (batch L, shared bias,
                      scale 1/sqrt(16): the reference takes it from config.head_dim)
  pair feed-forward   128->256, 256->128

Linears that the reference converts to Q8 (attention projections and the MSA->pair projections,
src/model/PPML.cpp:4434-4437) run the Q8 kernel with its bias epilogue, the others the fp32 (tf32 tensor-core) kernel.
LayerNorm, gating, residual adds and the head split views are the reference's elementwise glue and are not part of
this path: they are not run here, so the figure is the sum of the path's kernels and exchanges, not a forward time.

Sharding over G ranks follows the reference's flat-buffer semantics: every activation is cut into G contiguous
flat chunks (token rows; attention batches; tri_mul channel slabs; outer-product-mean d1 slabs).  Exchanges per
block, all through NCCL into local memory before any kernel reads them: all-gather of each pair bias ([L*L, 8],
2 MiB, three times), all-gather of the outer-product-mean's `right` operand (4 MiB), and two all-to-alls of 64 MiB in
total that stand for the (n, l) transposes closing MSA column attention and pair row attention
(src/modules/Attention.cpp:489, :744).  With G = 1 there is no exchange.  Total work is fixed as G grows ("strong").
The exchanges run in stream order between the kernels.  Running them asynchronously behind independent products
(bias gathered during the projections, the Linear before a transpose cut into row chunks whose all-to-alls follow
the next chunk's product) was measured slower on two GPUs (2.43 against 1.78 ms per block): the collectives' CTAs
take SMs that the one-CTA-per-SM persistent kernels count on, and every product then ends with a second wave.

The block is timed twice: launched op by op from the host ("eager_ms", with the per-op split of rank 0 from a pass with
events around every op class), and with the seven compute segments between the exchanges captured as CUDA graphs and
replayed, the collectives still launched from the host ("value": with several ranks the kernels are short and host
launch overhead, about 40 us per call through the Python mirror, would otherwise dominate).  Collectives are never
captured: a captured block with NCCL inside did not finish on two ranks here.
Prints one JSON line; times are CUDA-event times, maximum over ranks.
"""
import argparse
import json
import os

L_RES, N_MSA, D_MSA, D_PAIR, HEADS, HEAD_DIM, OPM_D, TRI_D = 256, 256, 256, 128, 8, 32, 16, 128


def run(gpus, steps, warmup, use_graph=True):
    import torch
    import torch.distributed as dist
    from proteinpredictmachinelearning_b200 import PATH_AUTO, TF32_TMA, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    G = world
    L, N = L_RES, N_MSA
    for total in (N * L, L * L, N, L, OPM_D, TRI_D):
        if total % G:
            raise SystemExit(f"{G} ranks do not divide the block's partitions")
    g = torch.Generator(device=dev).manual_seed(5 + 1000 * rank)
    rnd = lambda *shape: torch.randn(shape, device=dev, generator=g)

    tok_msa, tok_pair = N * L // G, L * L // G          # this rank's token rows
    x_msa, x_pair = rnd(tok_msa, D_MSA), rnd(tok_pair, D_PAIR)
    x_ff, x_pff, x_opm = rnd(tok_msa, 4 * D_MSA), rnd(tok_pair, 2 * D_PAIR), rnd(tok_pair, OPM_D * OPM_D)

    weights = {}

    def linear(x, n_out, q8, tag):
        """One Linear with bias on this rank's token rows."""
        k = x.shape[1]
        key = (tag, k, n_out, q8)
        if key not in weights:
            w = rnd(n_out, k) * 0.02
            weights[key] = (ops.quantize_q8_0r(w) if q8 else w, torch.zeros(n_out, device=dev),
                            torch.empty(x.shape[0], n_out, device=dev))
        w, b, out = weights[key]
        if q8:
            ops.mul_mat_q8_cuda(w, x, n_out, wtype=2, c_trans=1, bias=b, path=PATH_AUTO, out=out)
        else:
            ops.mul_mat_cuda(x, w, bias=b, path=PATH_AUTO, tf32_mode=TF32_TMA, out=out)
        return out

    bufs = {}

    def gather_rows(x, tag):
        """All-gather of the ranks' contiguous row ranges (rank order = row order) into a buffer that keeps its address."""
        if G == 1:
            return x
        if tag not in bufs:
            bufs[tag] = torch.empty((x.shape[0] * G,) + tuple(x.shape[1:]), device=dev, dtype=x.dtype)
        dist.all_gather_into_tensor(bufs[tag], x)
        return bufs[tag]

    def exchange(x, tag):
        """The all-to-all behind a (n, l) transpose of a [rows, channels] activation: every rank keeps 1/G of its rows."""
        if G == 1:
            return x
        if tag not in bufs:
            bufs[tag] = torch.empty_like(x)
        dist.all_to_all_single(bufs[tag], x)
        return bufs[tag]

    timers = {}
    state = {"capturing": False}

    class timed:
        def __init__(self, name):
            self.name = name

        def __enter__(self):
            if state["capturing"]:
                return
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e1 = torch.cuda.Event(enable_timing=True)
            self.e0.record()

        def __exit__(self, *a):
            if state["capturing"]:
                return
            self.e1.record()
            timers.setdefault(self.name, []).append((self.e0, self.e1))

    def attention(qkv_src, batch, bias_all, scale, tag):
        """Projections, fused attention over this rank's batches (with the gathered pair bias, if any), output Linear."""
        d_in = qkv_src.shape[1]
        with timed("linear_q8"):
            q = linear(qkv_src, HEADS * HEAD_DIM, True, tag + "q")
            k = linear(qkv_src, HEADS * HEAD_DIM, True, tag + "k")
            v = linear(qkv_src, HEADS * HEAD_DIM, True, tag + "v")
            linear(qkv_src, HEADS * HEAD_DIM, True, tag + "g")
        bias = None
        if bias_all is not None:
            with timed("exchange"):
                bias = bias_all.t().contiguous().view(HEADS, L, L)              # [8, L, L], shared by every batch
        seq = q.shape[0] // batch
        shape = (batch, HEADS, seq, HEAD_DIM)                                  # flat reinterpretation, as the reference's views
        with timed("attention"):
            o, _ = ops.flash_attn_forward_cuda(q.view(shape), k.view(shape), v.view(shape), bias, scale=scale,
                                               bias_bcast=bias is not None)
        with timed("linear_q8"):
            out = linear(o.view(-1, HEADS * HEAD_DIM), d_in, True, tag + "o")
        return out

    def pair_bias(tag):
        with timed("linear_q8"):
            return linear(x_pair, HEADS, True, tag + "b")                       # [L*L/G, 8]

    # The block as an alternation of compute segments (this library's kernels only: each can be captured as a CUDA
    # graph) and exchanges (collectives, always launched from the host).  `ctx` carries tensors between them; all of
    # them keep their addresses from step to step.
    ctx = {}

    def seg_a():
        ctx["mr_b"] = pair_bias("mr")

    def seg_b():
        attention(x_msa, N // G, ctx["mr_bias"], 1.0 / 32 ** 0.5, "mr")
        ctx["col"] = attention(x_msa, N // G, None, 1.0 / 32 ** 0.5, "mc")

    def seg_c():
        with timed("linear_tf32"):
            linear(x_msa, 4 * D_MSA, False, "ff1")
            linear(x_ff, D_MSA, False, "ff2")
        with timed("linear_q8"):
            ctx["left"] = linear(x_msa, OPM_D, True, "ol")
            ctx["right"] = linear(x_msa, OPM_D, True, "or")

    def seg_d():
        with timed("outer_prod_mean"):
            ops.outer_prod_mean_slabs_cuda(ctx["left"].view(OPM_D // G, L, N, 1), ctx["right_all"].view(OPM_D, L, N, 1))
        with timed("linear_q8"):
            linear(x_opm, D_PAIR, True, "oo")
        for direction in (True, False):
            with timed("linear_tf32"):
                a = linear(x_pair, TRI_D, False, "tl" + str(direction))
                b = linear(x_pair, TRI_D, False, "tr" + str(direction))
                for t in ("tlg", "trg", "tg"):
                    linear(x_pair, TRI_D, False, t + str(direction))
            with timed("tri_mul"):
                tm = ops.tri_mul_cuda(a.view(TRI_D // G, L, L, 1), b.view(TRI_D // G, L, L, 1), float(L), direction)
            with timed("linear_tf32"):
                linear(tm.view(tok_pair, TRI_D), D_PAIR, False, "to" + str(direction))
        ctx["pr_b"] = pair_bias("pr")

    def seg_e():
        ctx["row"] = attention(x_pair, L // G, ctx["pr_bias"], 1.0 / 16 ** 0.5, "pr")

    def seg_f():
        ctx["pc_b"] = pair_bias("pc")

    def seg_g():
        attention(x_pair, L // G, ctx["pc_bias"], 1.0 / 16 ** 0.5, "pc")
        with timed("linear_tf32"):
            linear(x_pair, 2 * D_PAIR, False, "pf1")
            linear(x_pff, D_PAIR, False, "pf2")

    def ex(fn, src, dst):
        def step():
            with timed("exchange"):
                ctx[dst] = fn(ctx[src], dst)
        return step

    segments = [seg_a, seg_b, seg_c, seg_d, seg_e, seg_f, seg_g]
    exchanges = [ex(gather_rows, "mr_b", "mr_bias"),      # pair bias of MSA row attention
                 ex(exchange, "col", "col_t"),            # (n, l) transpose closing column attention
                 ex(gather_rows, "right", "right_all"),   # [N*L, 16] flat = [16][L][N]
                 ex(gather_rows, "pr_b", "pr_bias"),
                 ex(exchange, "row", "row_t"),            # transpose closing pair row attention
                 ex(gather_rows, "pc_b", "pc_bias")]

    def block(graphs=None):
        for i, seg in enumerate(segments):
            if graphs is not None and graphs[i] is not None:
                graphs[i].replay()
            else:
                seg()
            if i < len(exchanges):
                exchanges[i]()

    def barrier():
        if G > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        block()
    code, where = ops.device_status()
    if code != 0:
        raise RuntimeError(f"device abort {code} at {where:#x}")
    # per-op split: one eager pass sequence with events around every op class
    timers.clear()
    barrier()
    for _ in range(steps):
        block()
    barrier()
    split = {k: sum(a.elapsed_time(b) for a, b in v) / steps for k, v in timers.items()}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        block()
    e1.record()
    barrier()
    eager_ms = e0.elapsed_time(e1) / steps
    # the whole block as one CUDA graph (kernels and collectives): with eight ranks the kernels are short enough that
    # launching them one by one from the host is what takes the time
    graph_ms, graph_note = None, ""
    if use_graph:
        graphs = []
        state["capturing"] = True
        for seg in segments:                 # no collective is ever captured; a segment that cannot be captured stays eager
            try:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    seg()
                graphs.append(gr)
            except Exception as exc:
                graphs.append(None)
                graph_note = f"a segment stayed eager: {type(exc).__name__}"
        state["capturing"] = False
        for _ in range(2):
            block(graphs)
        barrier()
        e0.record()
        for _ in range(steps):
            block(graphs)
        e1.record()
        barrier()
        graph_ms = e0.elapsed_time(e1) / steps
        code, where = ops.device_status()
        if code != 0:
            raise RuntimeError(f"device abort {code} at {where:#x}")
    best = graph_ms if graph_ms is not None else eager_ms
    ms = torch.tensor([best, eager_ms], device=dev, dtype=torch.float64)
    if G > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"metric": "main IterBlock hot-path ops, ms per block", "value": float(ms[0].item()), "unit": "ms",
                          "launch": ("cuda graphs for the compute segments, collectives from the host" + (" (" + graph_note + ")" if graph_note else ""))
                                    if graph_ms is not None else "eager",
                          "eager_ms": float(ms[1].item()),
                          "n_gpus": G, "steps": steps, "warmup": max(warmup, 3), "higher_is_better": False,
                          "scaling": "strong", "dtype": "q8 + tf32, fp32 accumulate", "data": "synthetic",
                          "config": {"workload": "one main IterBlock: L=256, MSA depth 256, d_msa 256, d_pair 128, 8x32 heads",
                                     "blocks_per_structure": 32},
                          "ms_per_32_blocks": float(ms[0].item()) * 32,
                          "split_ms_rank0": {k: round(v, 4) for k, v in sorted(split.items())}}), flush=True)
    if G > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true", help="time eager launches only")
    a = ap.parse_args()
    run(a.gpus, a.steps, a.warmup, use_graph=not a.no_graph)


if __name__ == "__main__":
    main()
