"""Hot-path op sequence of one main IterBlock of the reference model at full size, on 1..8 GPUs of one box.

The block's dense contractions and attention calls (src/model/PPML.cpp:2164-2273 for the layer shapes,
src/model/PPML.cpp:908-994 for the op order, src/modules/Attention.cpp:223-284, :361-392, :468-489, :717-744 for the
attention call sites) at L = 256 residues, MSA depth N = 256, d_msa = 256, d_pair = 128, 8 heads x 32:

  MSA row attention   5 Linears 256->256 on N*L tokens, pair bias Linear 128->8 on L*L tokens, attention
                      (batch N, shared bias [8, L, L], scale 1/sqrt(32))
  MSA column attn     5 Linears 256->256, attention without bias (batch = chunks of N flat positions), (n, l) transpose
  MSA feed-forward    256->1024, 1024->256
  MSA -> pair         left / right 256->16, outer-product-mean (16 slabs), out 256->128 on L*L tokens
  triangle mult.      out and in: 6 Linears 128->128 each, tri_mul over 128 channel slabs of L x L
  pair row / col attn each: 4 Linears 128->256, bias 128->8, out 256->128, attention (batch L, shared bias,
                      scale 1/sqrt(16): the reference takes it from config.head_dim); the row variant ends with a transpose
  pair feed-forward   128->256, 256->128

Linears that the reference converts to Q8 (attention projections and the MSA->pair projections,
src/model/PPML.cpp:4434-4437) run the Q8 kernel with its bias epilogue, the others the fp32 (tf32 tensor-core) kernel.
LayerNorm, gating, residual adds and the head split views are the reference's elementwise glue and are not part of
this path: they are not run here, so the figure is the sum of the path's kernels and exchanges, not a forward time.
Every op takes its input from a tensor generated from a seed common to all ranks (the op chains that need no glue
between them -- projections -> attention -> output Linear, left / right -> outer-product-mean -- are connected).

Fused form (default; PPML_B200_BLOCK_FUSED=0 gives the op-by-op form above): projections of one input that feed one
consumer are one Linear over the concatenated weights -- Q, K, V and the gate of an attention call (4 x 256 -> one
N = 1024 product), the three gate projections of a triangle multiplication (N = 384) -- and the attention call reads
Q, K, V as column ranges of that product's output (token-major operands, row stride 1024), applies sigmoid(gate) to its
output in the store and writes it token-major for the output Linear.  44 Linears become 28, and the permute / gate passes
of the reference around attention (src/model/PPML.cpp:1386-1520) have no counterpart at all.

Sharding over G ranks follows the reference's flat-buffer semantics: every activation is cut into G contiguous
flat chunks (token rows; attention batches; tri_mul channel slabs; outer-product-mean d1 slabs).  Exchanges per
block, all through NCCL into local memory before any kernel reads them: all-gather of each pair bias ([L*L, 8],
2 MiB, three times), all-gather of the outer-product-mean's `right` operand (4 MiB), and two (n, l) transposes
(src/modules/Attention.cpp:489, :744: one all-to-all of 64 MiB in total plus local re-layouts each).  With G = 1 the
transposes are local copies and nothing else is exchanged.  Total work is fixed as G grows ("strong").

Parity: the same block code runs a second time on the rank's own GPU with G = 1 (the unsharded block, same inputs and
weights), and every op's sharded result must equal the matching contiguous part of the unsharded result bit for bit
(token rows, batches and slabs are independent and go through the same tiles in the same order).

Extra-MSA block (`kind="extra"`, src/model/PPML.cpp:1526-1590, layer shapes :2243-2273): the same pair track, and an MSA
track on the 1024-row extra MSA with 64 channels and 8 heads x 8: row attention with the pair bias (projections Q8, the
head-dim-8 attention kernel), global column attention (src/modules/Attention.cpp:582-641: fp32 projections 64 -> 64 of
every token, one query per chunk of N flat positions -- the mean over the MSA rows, elementwise glue, here a common
input -- over the chunk's 1024 keys, no (n, l) transpose; the mean's partial sums [L, 64] per rank are gathered where the
reference would all-reduce them), feed-forward 64 -> 256 -> 64, left / right 64 -> 16 and the outer-product-mean over
1024 rows.

Timing: the block is timed launched op by op from the host ("eager_ms", with a per-class split from events around
every op), and with the compute segments between the exchanges captured as CUDA graphs and replayed, the collectives
still launched from the host ("ms_per_block").  Collectives are never captured.  Times are CUDA-event times, maximum
over ranks.
"""
import argparse
import json
import os

L_RES, N_MSA, D_MSA, D_PAIR, HEADS, HEAD_DIM, OPM_D, TRI_D = 256, 256, 256, 128, 8, 32, 16, 128
# MSA track of the two block kinds: rows, channels, head dim
KINDS = {"main": (N_MSA, D_MSA, HEAD_DIM), "extra": (1024, 64, 8)}
# dev size (BASELINE config 0): one chain of 51 residues, MSA depth 8, every Linear fp32
DEV_L, DEV_N = 51, 8


class Block:
    """The op sequence for one rank of a G-way partition (G = 1: the unsharded block).  Inputs and weights are shared
    between instances; every instance owns its outputs."""

    SITES = {"mr_bias": 0, "col_t": 1, "qsum": 1, "right": 2, "pr_bias": 3, "row_t": 4, "pc_bias": 5}

    def __init__(self, torch, dist, ops, inputs, weights, G, rank, dev, peers=None, fused=True, kind="main", size="full",
                 path=None, trace=False):
        self.torch, self.dist, self.ops = torch, dist, ops
        self.fused = fused
        self.inp, self.weights, self.G, self.rank, self.dev = inputs, weights, G, rank, dev
        self.peers = peers if G > 1 else None      # shard.PeerBuffers: exchanges as single kernels over peer memory
        self.peer_ptrs = {}
        self.out = {}            # named results of the last run
        self.bufs = {}           # tensors that keep their address from step to step
        self.timers = {}
        self.capturing = False
        self.ctx = {}
        self.kind = kind
        self.N, self.D, self.hd_msa = KINDS[kind]
        self.L = L_RES
        self.use_q8 = size == "full"             # the dev-size forward is fp32 throughout
        if size == "dev":
            self.L, self.N = DEV_L, DEV_N
        self.path = path                         # None: PATH_AUTO
        self.trace = [] if trace else None       # one entry per mul_mat / attention / pair-track call: what went in, what came out
        L, N = self.L, self.N
        self.tok_msa, self.tok_pair = N * L // G, L * L // G

    # ---- helpers -----------------------------------------------------------------------------------------------
    def rows(self, name):
        """This rank's contiguous token rows of a common input."""
        x = self.inp[name]
        n = x.shape[0] // self.G
        return x[self.rank * n:(self.rank + 1) * n]

    def timed(self, name):
        blk, torch = self, self.torch

        class _T:
            def __enter__(self):
                if blk.capturing:
                    return
                self.e0 = torch.cuda.Event(enable_timing=True)
                self.e1 = torch.cuda.Event(enable_timing=True)
                self.e0.record()

            def __exit__(self, *a):
                if blk.capturing:
                    return
                self.e1.record()
                blk.timers.setdefault(name, []).append((self.e0, self.e1))
        return _T()

    def buf(self, tag, shape, like=None):
        if tag not in self.bufs:
            self.bufs[tag] = self.torch.empty(shape, device=self.dev, dtype=self.torch.float32 if like is None else like.dtype)
        return self.bufs[tag]

    def linear(self, x, n_out, q8, tag):
        """One Linear with bias on this rank's token rows."""
        from proteinpredictmachinelearning_b200 import PATH_AUTO, TF32_TMA
        q8 = q8 and self.use_q8
        path = PATH_AUTO if self.path is None else self.path
        w, b = self.weights[(tag, x.shape[1], n_out, q8)]
        out = self.buf("lin_" + tag, (x.shape[0], n_out))
        ev = self.call_begin()
        if q8:
            self.ops.mul_mat_q8_cuda(w, x, n_out, wtype=2, c_trans=1, bias=b, path=path, out=out)
        else:
            self.ops.mul_mat_cuda(x, w, bias=b, path=path, tf32_mode=TF32_TMA, out=out)
        self.call_end(ev, "mul_mat_q8" if q8 else "mul_mat", tag, x=x, w=w, bias=b, out=out)
        self.out["lin_" + tag] = out
        return out

    def call_begin(self):
        if self.trace is None or self.capturing:
            return None
        e0 = self.torch.cuda.Event(enable_timing=True)
        e0.record()
        return e0

    def call_end(self, e0, op, tag, **tensors):
        if e0 is None:
            return
        e1 = self.torch.cuda.Event(enable_timing=True)
        e1.record()
        self.trace.append(dict(op=op, tag=tag, events=(e0, e1), **tensors))

    def gather_rows(self, x, tag):
        """All-gather of the ranks' contiguous row ranges (rank order = row order)."""
        if self.G == 1:
            return x
        if self.peers is not None:
            key = "ag_" + tag
            if key not in self.bufs:
                self.bufs[key], self.peer_ptrs[key] = self.peers.tensor((x.shape[0] * self.G,) + tuple(x.shape[1:]))
            self.peers.all_gather(x, self.peer_ptrs[key], self.SITES[tag])
            return self.bufs[key]
        full = self.buf("ag_" + tag, (x.shape[0] * self.G,) + tuple(x.shape[1:]))
        self.dist.all_gather_into_tensor(full, x)
        return full

    def transpose_nl(self, x, n_total, tag):
        """The (n, l) transpose of an activation [n * l tokens, C] whose n range is cut over the ranks, as the reference's
        `permute({0,2,1,3})` copies do on one device: returns this rank's rows [l_loc * n_total, C] of the transposed tensor."""
        G, C = self.G, x.shape[1]
        n_loc = n_total // G
        l_tot = x.shape[0] // n_loc
        x3 = x.view(n_loc, l_tot, C)
        if G == 1:
            out = self.buf("tr_" + tag, (l_tot, n_loc, C))
            out.copy_(x3.permute(1, 0, 2))
            return out.view(l_tot * n_loc, C)
        l_loc = l_tot // G
        if self.peers is not None:
            key = "tr_" + tag
            if key not in self.bufs:
                self.bufs[key], self.peer_ptrs[key] = self.peers.tensor((l_loc, G * n_loc, C))
            self.peers.transpose(x, self.peer_ptrs[key], n_loc, l_tot, C, self.SITES[tag])
            return self.bufs[key].view(l_loc * G * n_loc, C)
        send = self.buf("trs_" + tag, (G, n_loc, l_loc, C))
        send.copy_(x3.view(n_loc, G, l_loc, C).permute(1, 0, 2, 3))          # [to rank][n][l][c]
        recv = self.buf("trr_" + tag, (G, n_loc, l_loc, C))
        self.dist.all_to_all_single(recv, send)
        out = self.buf("tr_" + tag, (l_loc, G * n_loc, C))
        out.view(l_loc, G, n_loc, C).copy_(recv.permute(2, 0, 1, 3))         # [l][from rank][n][c]
        return out.view(l_loc * G * n_loc, C)

    def attention(self, src, batch, bias, scale, tag, head_dim=HEAD_DIM):
        """Projections, fused attention over this rank's batches (with the gathered pair bias, if any), output Linear."""
        d_in = src.shape[1]
        hd = HEADS * head_dim
        if self.fused:
            with self.timed("linear_q8"):
                qkvg = self.linear(src, 4 * hd, True, tag + "qkvg")
            seq = qkvg.shape[0] // batch
            t = qkvg.view(batch, seq, 4 * hd)
            o = self.buf("att_" + tag, (batch, seq, hd))
            with self.timed("attention"):
                ev = self.call_begin()
                self.ops.flash_attn_tokens(t[:, :, 0:hd], t[:, :, hd:2 * hd], t[:, :, 2 * hd:3 * hd], HEADS, bias=bias,
                                           gate=t[:, :, 3 * hd:4 * hd], act="sigmoid", scale=scale,
                                           bias_bcast=bias is not None, out=o, **self.path_kw())
                self.call_end(ev, "flash_attn_tokens", tag, q=t[:, :, 0:hd], k=t[:, :, hd:2 * hd], v=t[:, :, 2 * hd:3 * hd],
                              gate=t[:, :, 3 * hd:4 * hd], bias=bias, scale=scale, out=o)
            self.out["att_" + tag] = o
            with self.timed("linear_q8"):
                return self.linear(o.view(-1, hd), d_in, True, tag + "o")
        with self.timed("linear_q8"):
            q = self.linear(src, hd, True, tag + "q")
            k = self.linear(src, hd, True, tag + "k")
            v = self.linear(src, hd, True, tag + "v")
            self.linear(src, hd, True, tag + "g")
        seq = q.shape[0] // batch
        shape = (batch, HEADS, seq, head_dim)                                  # flat reinterpretation, as the reference's views
        o = self.buf("att_" + tag, shape)
        with self.timed("attention"):
            ev = self.call_begin()
            self.ops.flash_attn_forward_cuda(q.view(shape), k.view(shape), v.view(shape), bias, scale=scale,
                                             bias_bcast=bias is not None, out=o, **self.path_kw())
            self.call_end(ev, "flash_attn", tag, q=q.view(shape), k=k.view(shape), v=v.view(shape), bias=bias, scale=scale, out=o)
        self.out["att_" + tag] = o
        with self.timed("linear_q8"):
            return self.linear(o.view(-1, hd), d_in, True, tag + "o")

    def path_kw(self):
        return {} if self.path is None else {"path": self.path}

    def global_column_attention(self, x):
        """Extra-MSA block: projections of every token (fp32 Linears: not on the reference's Q8 list), one query per chunk
        of N flat positions over the chunk's N keys, output Linear.  The query (mean over the MSA rows of the Q
        projection) and the broadcast of the result over the rows times sigmoid(gate) are elementwise glue: common inputs."""
        N, hd = self.N, HEADS * self.hd_msa
        chunks = x.shape[0] // N
        with self.timed("linear_tf32"):
            if self.fused:
                t = self.linear(x, 4 * hd, False, "gcqkvg").view(chunks, N, 4 * hd)
                k, v = t[:, :, hd:2 * hd], t[:, :, 2 * hd:3 * hd]
            else:
                self.linear(x, hd, False, "gcq")
                k, v = self.linear(x, hd, False, "gck").view(chunks, N, hd), self.linear(x, hd, False, "gcv").view(chunks, N, hd)
                self.linear(x, hd, False, "gcg")
        q = self.rows("x_qmean").view(chunks, 1, hd)
        o = self.buf("att_gc", (chunks, 1, hd))
        with self.timed("attention"):
            ev = self.call_begin()
            self.ops.flash_attn_tokens(q, k, v, HEADS, scale=1.0 / self.hd_msa ** 0.5, out=o, **self.path_kw())
            self.call_end(ev, "flash_attn_tokens", "gc", q=q, k=k, v=v, gate=None, bias=None, scale=1.0 / self.hd_msa ** 0.5, out=o)
        self.out["att_gc"] = o
        with self.timed("linear_tf32"):
            return self.linear(self.rows("x_gc"), self.D, False, "gco")

    def pair_bias(self, tag):
        with self.timed("linear_q8"):
            return self.linear(self.rows("x_pair"), HEADS, True, tag + "b")          # [L*L/G, 8]

    def bias_layout(self, gathered, tag):
        """[L*L, 8] token-major -> [8, L, L], shared by every batch (the reference's permute copy)."""
        b = self.buf("bias_" + tag, (HEADS, self.L, self.L))
        b.view(HEADS, self.L * self.L).copy_(gathered.t())
        self.out["bias_" + tag] = b
        return b

    # ---- compute segments (this library's kernels only: each can be captured as a CUDA graph) ---------------------
    def seg_a(self):
        self.ctx["mr_b"] = self.pair_bias("mr")

    def seg_b(self):
        x = self.rows("x_msa")
        self.attention(x, self.N // self.G, self.ctx["mr_bias"], 1.0 / self.hd_msa ** 0.5, "mr", self.hd_msa)
        if self.kind == "main":
            self.ctx["col"] = self.attention(x, self.N // self.G, None, 1.0 / 32 ** 0.5, "mc")
        else:
            self.global_column_attention(x)
            self.ctx["qsum"] = self.rows("x_qsum")

    def seg_c(self):
        x = self.rows("x_msa")
        with self.timed("linear_tf32"):
            self.linear(x, 4 * self.D, False, "ff1")
            self.linear(self.rows("x_ff"), self.D, False, "ff2")
        with self.timed("linear_q8"):
            self.ctx["left"] = self.linear(x, OPM_D, True, "ol")
            self.ctx["right"] = self.linear(x, OPM_D, True, "or")

    def seg_d(self):
        G, L, N = self.G, self.L, self.N
        opm = self.buf("opm", (OPM_D // G * OPM_D, L, L, 1))
        with self.timed("outer_prod_mean"):
            ev = self.call_begin()
            self.ops.outer_prod_mean_slabs_cuda(self.ctx["left"].view(OPM_D // G, L, N, 1), self.ctx["right_all"].view(OPM_D, L, N, 1), out=opm,
                                                **self.path_kw())
            self.call_end(ev, "outer_prod_mean", "opm", left=self.ctx["left"].view(OPM_D // G, L, N, 1),
                          right=self.ctx["right_all"].view(OPM_D, L, N, 1), out=opm)
        self.out["opm"] = opm
        with self.timed("linear_q8"):
            self.linear(self.rows("x_opm"), D_PAIR, True, "oo")
        x = self.rows("x_pair")
        for direction in (True, False):
            d = "out" if direction else "in"
            with self.timed("linear_tf32"):
                a = self.linear(x, TRI_D, False, "tl" + d)
                b = self.linear(x, TRI_D, False, "tr" + d)
                if self.fused:
                    self.linear(x, 3 * TRI_D, False, "tgates" + d)
                else:
                    for t in ("tlg", "trg", "tg"):
                        self.linear(x, TRI_D, False, t + d)
            with self.timed("tri_mul"):
                ev = self.call_begin()
                tm = self.ops.tri_mul_cuda(a.view(TRI_D // G, L, L, 1), b.view(TRI_D // G, L, L, 1), float(L), direction, **self.path_kw())
                self.call_end(ev, "tri_mul", d, left=a.view(TRI_D // G, L, L, 1), right=b.view(TRI_D // G, L, L, 1), outgoing=direction, out=tm)
            self.out["tri_" + d] = tm
            with self.timed("linear_tf32"):
                self.linear(tm.view(self.tok_pair, TRI_D), D_PAIR, False, "to" + d)
        self.ctx["pr_b"] = self.pair_bias("pr")

    def seg_e(self):
        self.ctx["row"] = self.attention(self.rows("x_pair"), self.L // self.G, self.ctx["pr_bias"], 1.0 / 16 ** 0.5, "pr")

    def seg_f(self):
        self.ctx["pc_b"] = self.pair_bias("pc")

    def seg_g(self):
        x = self.rows("x_pair")
        self.attention(x, self.L // self.G, self.ctx["pc_bias"], 1.0 / 16 ** 0.5, "pc")
        with self.timed("linear_tf32"):
            self.linear(x, 2 * D_PAIR, False, "pf1")
            self.linear(self.rows("x_pff"), D_PAIR, False, "pf2")

    # ---- exchanges (collectives, always launched from the host) ---------------------------------------------------
    def ex_bias(self, src, dst):
        def step():
            with self.timed("exchange"):
                self.ctx[dst] = self.bias_layout(self.gather_rows(self.ctx[src], dst), dst)
        return step

    def ex_right(self):
        with self.timed("exchange"):
            self.ctx["right_all"] = self.gather_rows(self.ctx["right"], "right")          # [N*L, 16] flat = [16][L][N]
            self.out["right_all"] = self.ctx["right_all"]

    def ex_qsum(self):
        with self.timed("exchange"):
            self.out["qsum_all"] = self.gather_rows(self.ctx["qsum"], "qsum")               # [G * L, 64] partial sums of the query mean

    def ex_transpose(self, src, n_total, dst):
        def step():
            with self.timed("exchange"):
                self.ctx[dst] = self.transpose_nl(self.ctx[src], n_total, dst)
                self.out[dst] = self.ctx[dst]
        return step

    def plan(self):
        segments = [self.seg_a, self.seg_b, self.seg_c, self.seg_d, self.seg_e, self.seg_f, self.seg_g]
        exchanges = [self.ex_bias("mr_b", "mr_bias"),                # pair bias of MSA row attention
                     self.ex_transpose("col", self.N, "col_t") if self.kind == "main"       # (n, l) transpose closing column attention
                     else self.ex_qsum,                                                  # partial sums of the global query
                     self.ex_right,
                     self.ex_bias("pr_b", "pr_bias"),
                     self.ex_transpose("row", self.L, "row_t"),       # transpose closing pair row attention
                     self.ex_bias("pc_b", "pc_bias")]
        return segments, exchanges

    def run(self, graphs=None):
        segments, exchanges = self.plan()
        for i, seg in enumerate(segments):
            if graphs is not None and graphs[i] is not None:
                graphs[i].replay()
            else:
                seg()
            if i < len(exchanges):
                exchanges[i]()


# per rank and block: bytes received by each collective at G ranks (fp32)
def exchange_bytes(G, kind="main"):
    if G == 1:
        return {}
    frac = (G - 1) / G
    N, D, _ = KINDS[kind]
    out = {"all_gather pair bias [L*L, 8] (x3)": int(L_RES * L_RES * HEADS * 4 * frac),
           "all_gather outer-product-mean right [N*L, 16]": int(N * L_RES * OPM_D * 4 * frac),
           "all_to_all pair (row, col) transpose [L*L, 128] / G": int(L_RES * L_RES * D_PAIR * 4 / G * frac)}
    if kind == "main":
        out["all_to_all MSA (n, l) transpose [N*L, 256] / G"] = int(N * L_RES * D * 4 / G * frac)
    else:
        out["all_gather partial sums of the global query [L, 64] per rank"] = int(L_RES * D * 4 * (G - 1))
    return out


def make_inputs_and_weights(torch, ops, dev, kind="main", G=1, size="full"):
    """Inputs and weights from one seed, identical on every rank.  size = "dev": 51 residues, MSA depth 8, fp32 weights only."""
    g = torch.Generator(device=dev).manual_seed(5 if size == "full" else 1)
    rnd = lambda *shape: torch.randn(shape, device=dev, generator=g)
    N, D_M, hd_m = KINDS[kind]
    L = L_RES
    if size == "dev":
        L, N = DEV_L, DEV_N
    use_q8 = size == "full"
    inputs = {"x_msa": rnd(N * L, D_M), "x_pair": rnd(L * L, D_PAIR), "x_ff": rnd(N * L, 4 * D_M),
              "x_pff": rnd(L * L, 2 * D_PAIR), "x_opm": rnd(L * L, OPM_D * OPM_D)}
    attn = [("mr", D_M, hd_m), ("pr", D_PAIR, HEAD_DIM), ("pc", D_PAIR, HEAD_DIM)] + ([("mc", D_M, hd_m)] if kind == "main" else [])
    spec = []
    for tag, d_in, hd in attn:
        spec += [(tag + t, d_in, HEADS * hd, True) for t in "qkvg"] + [(tag + "o", HEADS * hd, d_in, True)]
    if kind == "extra":
        # global column attention: the query per chunk of N flat positions (their number is L), the gated result per token,
        # and every rank's partial sums of the query mean
        inputs.update({"x_qmean": rnd(L, HEADS * hd_m) / hd_m ** 0.5, "x_gc": rnd(N * L, HEADS * hd_m), "x_qsum": rnd(G * L, D_M)})
        spec += [("gc" + t, D_M, HEADS * hd_m, False) for t in "qkvg"] + [("gco", HEADS * hd_m, D_M, False)]
    spec += [(tag + "b", D_PAIR, HEADS, True) for tag in ("mr", "pr", "pc")]
    spec += [("ff1", D_M, 4 * D_M, False), ("ff2", 4 * D_M, D_M, False), ("ol", D_M, OPM_D, True), ("or", D_M, OPM_D, True),
             ("oo", OPM_D * OPM_D, D_PAIR, True), ("pf1", D_PAIR, 2 * D_PAIR, False), ("pf2", 2 * D_PAIR, D_PAIR, False)]
    for d in ("out", "in"):
        spec += [(t + d, D_PAIR, TRI_D, False) for t in ("tl", "tr", "tlg", "trg", "tg")] + [("to" + d, TRI_D, D_PAIR, False)]
    weights, raw = {}, {}
    for (tag, k, n_out, q8) in spec:
        w = rnd(n_out, k) * 0.02
        b = rnd(n_out) * 0.1
        raw[tag] = (w, b)
        q8 = q8 and use_q8
        weights[(tag, k, n_out, q8)] = (ops.quantize_q8_0r(w) if q8 else w, b)
    # concatenated weights of the fused form
    cat = lambda tags: (torch.cat([raw[t][0] for t in tags], 0).contiguous(), torch.cat([raw[t][1] for t in tags], 0).contiguous())
    for tag, d_in, hd in attn:
        w, b = cat([tag + t for t in "qkvg"])
        weights[(tag + "qkvg", d_in, 4 * HEADS * hd, use_q8)] = (ops.quantize_q8_0r(w) if use_q8 else w, b)
    if kind == "extra":
        weights[("gcqkvg", D_M, 4 * HEADS * hd_m, False)] = cat(["gc" + t for t in "qkvg"])
    for d in ("out", "in"):
        weights[("tgates" + d, D_PAIR, 3 * TRI_D, False)] = cat([t + d for t in ("tlg", "trg", "tg")])
    return inputs, weights


def dev_blocks(torch, ops, dev, path=None, fused=True):
    """The blocks of the dev-size forward (BASELINE config 0: 51 residues, MSA depth 8, fp32 weights; 1 extra + 2 main blocks,
    of which one of each kind is run: the second main block makes the same calls) with every call traced: returns
    {kind: Block}; each Block's `trace` lists its mul_mat / attention / tri_mul / outer-product-mean calls with their
    operands, results and CUDA events, and `graph_us` is the block's time replayed from a CUDA graph.  Checking them against the CPU checker is the caller's business (tests, bench)."""
    blocks = {}
    for kind in ("extra", "main"):
        inputs, weights = make_inputs_and_weights(torch, ops, dev, kind, 1, size="dev")
        warm = Block(torch, None, ops, inputs, weights, 1, 0, dev, fused=fused, kind=kind, size="dev", path=path)
        warm.run()                               # first-use costs (module load, attributes) stay out of the per-call times
        blk = Block(torch, None, ops, inputs, weights, 1, 0, dev, fused=fused, kind=kind, size="dev", path=path, trace=True)
        blk.run()                                # its results come from fresh device allocations: not the run to time
        torch.cuda.synchronize()
        blk.out.clear()
        blk.trace.clear()
        blk.run()
        torch.cuda.synchronize()
        # the same block replayed from a CUDA graph: its time without the host's launch cost
        warm.capturing = True
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            warm.run()
        for _ in range(3):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        blk.graph_us = e0.elapsed_time(e1) * 1e3 / 20
        blocks[kind] = blk
    return blocks


def verify(torch, sharded, full, G, rank):
    """Every named result of the sharded run against the matching contiguous part of the unsharded run, bit for bit."""
    bad, n = [], 0
    for name, got in sharded.out.items():
        ref = full.out[name]
        if name.startswith("bias_") or name in ("right_all", "qsum_all"):
            part = ref                                           # gathered: the whole tensor on every rank
        else:
            flat = ref.reshape(-1)
            per = flat.numel() // G
            part = flat[rank * per:(rank + 1) * per]
        n += 1
        if not torch.equal(got.reshape(-1), part.reshape(-1)):
            bad.append(name)
    return n, bad


def measure(steps=5, warmup=3, use_graph=True, check=True, kind="main"):
    """Runs the block on this process's rank (torch.distributed already initialised when WORLD_SIZE > 1) and returns the
    record (identical on every rank as far as the timing goes; rank 0's split)."""
    import torch
    import torch.distributed as dist
    from proteinpredictmachinelearning_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    G = world
    L, N = L_RES, KINDS[kind][0]
    for total in (N * L, L * L, N, L, OPM_D, TRI_D):
        if total % G:
            return {"unavailable": f"{G} ranks do not divide the block's partitions"}
    inputs, weights = make_inputs_and_weights(torch, ops, dev, kind, G)
    # exchanges: single kernels over peer memory (CUDA IPC) by default, NCCL collectives launched from the host when
    # that cannot be set up or PPML_B200_EXCHANGE=nccl asks for them
    peers, exchange_mode = None, "none (one rank)"
    if G > 1:
        exchange_mode = "nccl collectives launched from the host"
        if os.environ.get("PPML_B200_EXCHANGE", "peer") != "nccl":
            from proteinpredictmachinelearning_b200 import shard
            try:
                peers = shard.PeerBuffers(G, rank)
                good = 1
            except Exception:
                peers, good = None, 0
            flag = torch.tensor([good], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:
                peers = None
            else:
                exchange_mode = "one kernel per exchange: stores into the peers' buffers between two flag rounds"
    fused = os.environ.get("PPML_B200_BLOCK_FUSED", "1") != "0"
    blk = Block(torch, dist, ops, inputs, weights, G, rank, dev, peers=peers, fused=fused, kind=kind)

    def barrier():
        if G > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        blk.run()
    code, where = ops.device_status()
    if code != 0:
        raise RuntimeError(f"device abort {code} at {where:#x}")

    # ---- parity: the unsharded block on this GPU, same inputs and weights ----------------------------------------
    n_checked, bad = 0, []
    if check:
        if G > 1:
            full = Block(torch, dist, ops, inputs, weights, 1, 0, dev, fused=fused, kind=kind)
            full.run()
            torch.cuda.synchronize()
            n_checked, bad = verify(torch, blk, full, G, rank)
            del full
        else:
            # one rank: the sharded and the unsharded block are the same code path; check determinism of a second run
            first = {k: v.clone() for k, v in blk.out.items()}
            blk.run()
            torch.cuda.synchronize()
            n_checked = len(first)
            bad = [k for k, v in first.items() if not torch.equal(v, blk.out[k])]
            del first
        flag = torch.tensor([len(bad)], device=dev)
        if G > 1:
            dist.all_reduce(flag)
        n_bad_all = int(flag.item())
    else:
        n_bad_all = None

    # ---- per-class split and eager time ----------------------------------------------------------------------------
    blk.timers.clear()
    barrier()
    for _ in range(steps):
        blk.run()
    barrier()
    split = {k: sum(a.elapsed_time(b) for a, b in v) / steps for k, v in blk.timers.items()}
    blk.timers.clear()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    blk.capturing = True                     # no per-op events from here on
    barrier()
    e0.record()
    for _ in range(steps):
        blk.run()
    e1.record()
    barrier()
    eager_ms = e0.elapsed_time(e1) / steps
    graph_ms, graph_note = None, ""
    if use_graph:
        whole = None
        if G == 1 or peers is not None:
            # no NCCL call inside: the whole block (compute and exchange kernels) is one graph
            try:
                whole = torch.cuda.CUDAGraph()
                with torch.cuda.graph(whole):
                    blk.run()
            except Exception as exc:
                whole, graph_note = None, f"whole-block capture failed: {type(exc).__name__}"
            if G > 1:                        # all ranks replay, or none does
                flag = torch.tensor([1 if whole is not None else 0], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                if int(flag.item()) == 0:
                    whole = None
        graphs = []
        if whole is None:
            segments, _ = blk.plan()
            for seg in segments:             # no collective is ever captured; a segment that cannot be captured stays eager
                try:
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr):
                        seg()
                    graphs.append(gr)
                except Exception as exc:
                    graphs.append(None)
                    graph_note = f"a segment stayed eager: {type(exc).__name__}"
        step = whole.replay if whole is not None else (lambda: blk.run(graphs))
        for _ in range(2):
            step()
        barrier()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
        graph_ms = e0.elapsed_time(e1) / steps
        if whole is not None:
            graph_note = "the whole block is one graph"
        code, where = ops.device_status()
        if code != 0:
            raise RuntimeError(f"device abort {code} at {where:#x}")
    blk.capturing = False
    best = graph_ms if graph_ms is not None else eager_ms
    ms = torch.tensor([best, eager_ms], device=dev, dtype=torch.float64)
    if G > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_split = sum(split.values()) or 1.0
    if peers is not None:
        torch.cuda.synchronize()
        if G > 1:
            dist.barrier()
        blk.bufs.clear()
        peers.close()
    n_blocks = 32 if kind == "main" else 4               # blocks of this kind in the full-size model
    if kind == "main":
        workload = ("one main IterBlock: L=256, MSA depth 256, d_msa 256, d_pair 128, 8x32 heads; "
                    + ("14 Q8 Linears (Q, K, V and gate of an attention call as one), 14 fp32 Linears (the gates of a triangle "
                       "multiplication as one), 4 attention calls on token-major operands with the gate applied in the store, "
                       if fused else "26 Q8 Linears, 18 fp32 Linears, 4 attention calls, ")
                    + "2 tri_mul, 1 outer-product-mean")
    else:
        workload = ("one extra-MSA FullBlock: L=256, extra MSA depth 1024, d_msa 64 with 8x8 heads (row attention with pair "
                    "bias on the head-dim-8 kernel, global column attention: one query over 1024 keys per chunk), d_pair 128 "
                    "with 8x32 heads; " + ("fused projections, " if fused else "") + "2 tri_mul, 1 outer-product-mean over 1024 rows")
    return {"metric": ("main IterBlock" if kind == "main" else "extra-MSA FullBlock") + " hot-path ops, ms per block",
            "ms_per_block": float(ms[0].item()), "unit": "ms",
            f"ms_per_{n_blocks}_blocks": float(ms[0].item()) * n_blocks, "eager_ms": float(ms[1].item()), "n_gpus": G, "steps": steps,
            "scaling": "strong", "higher_is_better": False, "dtype": "q8 + tf32, fp32 accumulate", "data": "synthetic, seed 5",
            "launch": ("cuda graphs" + (" (" + graph_note + ")" if graph_note else " for the compute segments, collectives from the host"))
                      if graph_ms is not None else "eager",
            "exchange": exchange_mode,
            "workload": workload,
            "fused_projections": fused,
            "split_ms_rank0": {k: round(v, 4) for k, v in sorted(split.items())},
            "exchange_share": round(split.get("exchange", 0.0) / total_split, 4),
            "exchange_bytes_per_rank": exchange_bytes(G, kind),
            "parity": {"ops_checked": n_checked, "mismatching_over_ranks": n_bad_all, "mismatching_here": bad,
                       "against": "the unsharded block on the same GPU, same inputs and weights, bit for bit" if G > 1
                                  else "a second run of the same block (one rank: sharded and unsharded coincide), bit for bit"}}


def run(gpus, steps, warmup, use_graph=True, kind="main"):
    import torch.distributed as dist
    rec = measure(steps, warmup, use_graph, kind=kind)
    if int(os.environ.get("RANK", "0")) == 0:
        rec["value"] = rec.get("ms_per_block")
        print(json.dumps(rec), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true", help="time eager launches only")
    ap.add_argument("--kind", choices=sorted(KINDS), default="main", help="main IterBlock or extra-MSA FullBlock")
    a = ap.parse_args()
    run(a.gpus, a.steps, a.warmup, use_graph=not a.no_graph, kind=a.kind)


if __name__ == "__main__":
    main()
