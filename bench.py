#!/usr/bin/env python
"""Benchmark of the dense-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (the reference's Q8 benchmark configuration): the Q8 block-quantized mul_mat sweep -- weights
W[N,K] ~ N(0, 0.02) quantized to int8 blocks of 32 with an fp16 scale (planar Q8_0R), activations X[M,K] ~ N(0,1)
quantized on the fly; K in {128, 256, 1024}, N in {128, 256, 512, 1024}, M in {408, 2601, 65536}; seed 2.
One pass = the 36 shapes, captured once as a CUDA graph; one step = `passes_per_step` replays of it (so that a
step lasts 0.125 s or more, the timed region 2.6 s or more, and the clock sampler sees it).  `value`, `ms_per_step` and `roofline` all come
from that one timed region (inputs resident in HBM); `e2e` is the same pass through the C ABI with pinned host
buffers, copies inside the timed region.  After the timed region sampled token rows of every shape are compared
with the CPU checker (`checked`).  At N > 1 GPUs every rank runs the sweep on its own token rows (weak scaling, no
data-path collective: token rows are independent).

Beside the headline the line carries
  `kernels`        one record per other kernel of the path (fp32/tf32 and bf16 mul_mat on the sweep's large shapes,
                   the three axial-attention cases in fp32 and bf16, triangle multiplication, outer-product-mean and the
                   Linear behind it), each timed from its own CUDA graph, each with its roofline
                   (min(tensor peak, intensity x HBM bandwidth), peaks from MEASURED_PEAKS.json);
  `dev_forward_calls`  BASELINE config 0's shapes: every mul_mat / attention / pair-track call of the dev-size blocks
                   (51 residues, MSA depth 8, fp32) timed and checked against the CPU checker, on both paths;
  `sharded_block`  the hot-path op sequence of one main IterBlock at full size cut over the N ranks (strong scaling,
                   ms per block, per-class split, exchanged bytes, every op's shard checked against the unsharded op);
  `sharded_extra_block`  the same for one extra-MSA FullBlock (1024 MSA rows of 64 channels, 8 heads x 8, global column
                   attention);
  `cpu_baseline`   the host-core figures: the Q8 arithmetic restated on the CPU (the reference has no CPU Q8 kernel,
                   include/ppml/QuantBlocks.h:56) and, where the reference's own CPU kernels were compiled
                   (oracle/_ref), those kernels on bounded samples.

`--impl reference` times the CPU side alone on the same configuration (rank 0; other ranks exit).
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

KS = (128, 256, 1024)
NS = (128, 256, 512, 1024)
MS = (408, 2601, 65536)
SEED = 2
L2_BYTES = 126e6


def shapes(ms=MS):
    return [(m, k, n) for m in ms for k in KS for n in NS]


def mm_flops(m, k, n):
    return 2.0 * m * k * n


def q8_bytes(m, k, n):
    """Algorithmic HBM bytes of one Q8 mul_mat: planar int8 weights with half scales, fp32 activations in, fp32 result out."""
    return (34.0 / 32.0) * n * k + 4.0 * m * k + 4.0 * m * n


def mm_bytes(m, k, n, e):
    """fp32 (e = 4) or 16-bit (e = 2) operands, fp32 result."""
    return e * (m * k + n * k) + 4.0 * m * n


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


def roofline(flops, nbytes, us, peaks, tensor_scale):
    """Roofline of one launch: the time floor is the slower of (bytes / HBM bandwidth) and (flops / tensor peak);
    tensor_scale = 1 for 16-bit operands, 0.5 for tf32 (half the measured bf16 rate), 2 for int8."""
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9)
    t_tc = flops / (peaks["bf16_tflops"] * tensor_scale * 1e12)
    t = us * 1e-6
    if t_hbm >= t_tc:
        return {"bound": "hbm", "achieved": nbytes / t / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": t_hbm / t, "peak_kind": peaks["kind"]}
    return {"bound": "tensor", "achieved": flops / t / 1e12, "peak": peaks["bf16_tflops"] * tensor_scale, "unit": "TFLOP/s",
            "frac": t_tc / t, "peak_kind": peaks["kind"]}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU side: the restated Q8 arithmetic (port) and the reference's own CPU kernels (oracle/_ref)
# ------------------------------------------------------------------------------------------------
CPU_SAMPLE_ROWS = {408: 408, 2601: 2601, 65536: 2048}       # token rows of each M the CPU side computes


def cpu_q8_pass(oracle, sample, threads):
    """One pass of the CPU port over `sample` = [(W_packed, X, M_out)], token rows split over threads."""
    import numpy as np

    def work(W, X, m_out, out, lo, hi):
        out[lo:hi] = oracle.mul_mat_q8(W, X[lo:hi], m_out, wtype=2, c_trans=1)

    t0 = time.perf_counter()
    for W, X, m_out in sample:
        out = np.empty((X.shape[0], m_out), np.float32)
        n = X.shape[0]
        step = (n + threads - 1) // threads
        ts = [threading.Thread(target=work, args=(W, X, m_out, out, lo, min(lo + step, n))) for lo in range(0, n, step)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
    return time.perf_counter() - t0


def make_cpu_sample(oracle):
    """All 36 shapes of the sweep; the M = 65536 shapes on a sample of 2048 token rows (rows are independent)."""
    import numpy as np
    r = np.random.default_rng(SEED)
    sample, flops = [], 0.0
    for (m, k, n) in shapes():
        rows = CPU_SAMPLE_ROWS[m]
        w = (r.standard_normal((n, k)) * 0.02).astype(np.float32)
        x = r.standard_normal((rows, k)).astype(np.float32)
        sample.append((oracle.repack_q8_0(oracle.quantize_q8_0(w)), x, n))
        flops += mm_flops(rows, k, n)
    return sample, flops


CPU_SAMPLE_NOTE = ("all 36 (M,K,N) shapes per pass, the M=65536 shapes on 2048 sampled token rows (rows are independent); the "
                   "reference has no CPU Q8 kernel, this is its CUDA arithmetic restated in C, threaded over token rows")


def reference_cpu_kernels(budget_s=12.0):
    """The reference's own CPU kernels (compiled from its sources into oracle/_ref/libppml_ref.so) on bounded samples
    of the other workloads, at all cores and at the reference's default of 4 threads.  Empty when the library is absent."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import checkers
    if not checkers.have_ref():
        return []
    import numpy as np
    r = np.random.default_rng(4)
    cores = os.cpu_count() or 1
    out = []

    def timed(name, sample, flops, fn, threads_list):
        for nt in threads_list:
            ref = checkers.Ref(n_threads=nt)
            t0 = time.perf_counter()
            fn(ref)
            dt = time.perf_counter() - t0
            out.append({"op": name, "sample": sample, "threads": nt, "seconds": dt, "gflops": flops / dt / 1e9, "kind": "reference"})

    a = r.standard_normal((2048, 256)).astype(np.float32)
    b = (r.standard_normal((256, 256)) * 0.02).astype(np.float32)
    bi = np.zeros(256, np.float32)
    timed("mul_mat fp32 + bias", "2048 token rows x K=256 x N=256", mm_flops(2048, 256, 256), lambda ref: ref.mul_mat(a, b, bi), (cores, 4))
    a2 = r.standard_normal((512, 1024)).astype(np.float32)
    b2 = (r.standard_normal((1024, 1024)) * 0.02).astype(np.float32)
    timed("mul_mat fp32", "512 token rows x K=1024 x N=1024", mm_flops(512, 1024, 1024), lambda ref: ref.mul_mat(a2, b2, None), (cores, 4))
    Q, K, V = (r.standard_normal((1, 8, 256, 32)).astype(np.float32) / np.float32(32 ** 0.5) for _ in range(3))
    bias = r.standard_normal((1, 8, 256, 256)).astype(np.float32)
    timed("flash_attn_forward (single-threaded by construction)", "1 of 256 batches, 8 heads, L=256, d=32, bias",
          4.0 * 8 * 256 * 256 * 32, lambda ref: ref.flash_attn(Q, K, V, bias, scale=1 / 32 ** 0.5), (1,))
    l = r.standard_normal((4, 256, 256, 1)).astype(np.float32)
    rr = r.standard_normal((4, 256, 256, 1)).astype(np.float32)
    timed("tri_mul outgoing", "4 of 128 channel slabs, L=256", 2.0 * 4 * 256 ** 3, lambda ref: ref.tri_mul(l, rr, 256.0, True), (cores, 4))
    ol = r.standard_normal((4, 128, 256, 1)).astype(np.float32)
    orr = r.standard_normal((4, 128, 256, 1)).astype(np.float32)
    timed("outer_prod_mean", "c=4, L=128, N=256 (full size: c=32, L=256)", 2.0 * (4 * 128) ** 2 * 256,
          lambda ref: ref.outer_prod_mean(ol, orr), (cores, 4))
    return out


def cpu_baseline_record(budget_s=10.0):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from checkers import Oracle
    oracle = Oracle()
    threads = os.cpu_count() or 1
    sample, flops = make_cpu_sample(oracle)
    t = cpu_q8_pass(oracle, sample, threads)
    reps = 1
    while t < budget_s and reps < 50:
        t += cpu_q8_pass(oracle, sample, threads)
        reps += 1
    return {"value": flops * reps / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{CPU_SAMPLE_NOTE}; {reps} pass(es)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from checkers import Oracle
    oracle = Oracle()
    threads = os.cpu_count() or 1
    sample, flops = make_cpu_sample(oracle)
    for _ in range(min(args.warmup, 2)):
        cpu_q8_pass(oracle, sample, threads)
    t = 0.0
    for _ in range(args.steps):
        t += cpu_q8_pass(oracle, sample, threads)
    val = flops * args.steps / t / 1e12
    line = {
        "impl": "reference", "metric": "mul_mat TFLOPS", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 2), "ms_per_step": 1e3 * t / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "q8 (int8 x int8 -> int32, fp32 rescale)", "data": "synthetic",
        "config": {"workload": "configs[1] Q8 block-quantized mul_mat sweep", "K": list(KS), "N": list(NS), "M": list(MS),
                   "sample": CPU_SAMPLE_NOTE},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": CPU_SAMPLE_NOTE},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if not args.no_kernels:
        line["reference_cpu_kernels"] = reference_cpu_kernels()
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU side helpers
# ------------------------------------------------------------------------------------------------
def graph_time_us(torch, issue, launches, reps=20, warm=3):
    """CUDA-event time per launch of `issue()` (which issues `launches` kernels of one kind on the current stream),
    replayed from a captured graph; falls back to direct calls if the capture fails."""
    for _ in range(2):
        issue()
    torch.cuda.synchronize()
    run = issue
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            issue()
        run = g.replay
    except Exception:
        run = issue
    for _ in range(warm):
        run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    return 1e3 * e0.elapsed_time(e1) / (reps * launches)


def rotations(working_set_bytes):
    """Copies of a small workload to cycle through so that consecutive launches do not find their inputs in L2."""
    return int(min(48, max(1, math.ceil(1.5 * L2_BYTES / max(working_set_bytes, 1.0)))))


def dev_forward_calls(torch, dev, oracle):
    """BASELINE config 0's shapes: the blocks of the dev-size forward (51 residues, MSA depth 8, fp32 weights; one extra-MSA and
    one main block are run, the forward has 1 + 2), every mul_mat / attention / tri_mul / outer-product-mean call timed by its
    own CUDA events and checked against the CPU checker on the tensors it saw -- once on the exact CUDA-core kernels (the
    forwarders' default) and once on the tensor-core path."""
    from proteinpredictmachinelearning_b200 import PATH_AUTO, PATH_SIMT, block_bench, ops
    from checkers import check_block_calls
    rec = {"workload": "dev-size blocks: L=51, MSA depth 8, d_msa 256 (extra: 64), d_pair 128, fp32 weights, seed 1; op by op "
                       "(no fused projections), one launch per call, eager", "paths": {}}
    for name, path, tol in (("cuda cores, exact fp32", PATH_SIMT, 1e-5), ("tensor cores where a kernel exists, tf32 products", PATH_AUTO, 1e-3)):
        blocks = block_bench.dev_blocks(torch, ops, dev, path=path, fused=False)
        entry = {"tolerance": tol, "blocks": {}}
        worst, total_us, graph_us, n_calls = 0.0, 0.0, 0.0, 0
        for kind, blk in blocks.items():
            calls = check_block_calls(blk.trace, oracle)
            mult = 2 if kind == "main" else 1
            us = sum(c["us"] for c in calls)
            entry["blocks"][kind] = {"calls": [{**c, "us": round(c["us"], 2), "err": float(f"{c['err']:.3g}")} for c in calls],
                                     "us_per_block": round(us, 1), "us_per_block_from_a_cuda_graph": round(blk.graph_us, 1),
                                     "blocks_in_the_forward": mult}
            worst = max(worst, max(c["err"] for c in calls))
            total_us += mult * us
            graph_us += mult * blk.graph_us
            n_calls += len(calls)
        entry.update({"calls_checked": n_calls, "worst_err": float(f"{worst:.3g}"), "checked": bool(worst <= tol),
                      "us_per_forward_hot_path": round(total_us, 1), "us_per_forward_hot_path_from_cuda_graphs": round(graph_us, 1)})
        rec["paths"][name] = entry
    rec["checked"] = all(e["checked"] for e in rec["paths"].values())
    return rec


def kernel_records(torch, dev, peaks, oracle):
    """One record per other kernel of the path, each timed from its own CUDA graph (launches back to back, small
    workloads rotating over enough copies to exceed L2), each with its roofline and a check of a sampled unit."""
    import numpy as np
    from proteinpredictmachinelearning_b200 import PATH_UMMA, TF32_TMA, ops
    recs = []
    g = torch.Generator(device=dev).manual_seed(3)
    rnd = lambda *s: torch.randn(s, device=dev, generator=g)
    host = lambda t: t.detach().float().cpu().numpy()

    def rel(got, ref):
        return float(np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))

    # ---- mul_mat on the sweep's M = 65536 shapes: fp32 operands (tf32 products) and bf16 operands ----
    for kind, e, scale in (("tf32", 4, 0.5), ("bf16", 2, 1.0)):
        total_us, total_fl, total_by = 0.0, 0.0, 0.0
        for (k, n) in [(k, n) for k in KS for n in NS]:
            m = 65536
            A, Bw, Cc = rnd(m, k), rnd(n, k) * 0.02, torch.empty((m, n), device=dev)
            if kind == "bf16":
                A, Bw = A.bfloat16(), Bw.bfloat16()
                f = lambda: ops.mul_mat_16(A, Bw, path=PATH_UMMA, out=Cc)
            else:
                f = lambda: ops.mul_mat_cuda(A, Bw, path=PATH_UMMA, tf32_mode=TF32_TMA, out=Cc)
            us = graph_time_us(torch, lambda: [f() for _ in range(4)], 4)
            fl, by = mm_flops(m, k, n), mm_bytes(m, k, n, e)
            total_us += us; total_fl += fl; total_by += by
            rows = torch.tensor([0, 12345, m - 1], device=dev)
            ref = oracle.mul_mat_f32(host(A[rows]), host(Bw))
            ok = rel(host(Cc[rows]), ref) <= (1e-3 if kind == "tf32" else 1e-5)
            recs.append({"kernel": "umma_gemm_kernel", "op": f"mul_mat {kind}", "workload": f"M={m} K={k} N={n}", "us": us,
                         "tflops": fl / us / 1e6, "gbs": by / us / 1e3, "roofline": roofline(fl, by, us, peaks, scale), "checked": bool(ok)})
            del A, Bw, Cc
        recs.append({"kernel": "umma_gemm_kernel", "op": f"mul_mat {kind}", "workload": "the 12 M=65536 shapes of the sweep, summed",
                     "us": total_us, "tflops": total_fl / total_us / 1e6, "gbs": total_by / total_us / 1e3})

    # ---- axial attention (configs[2]): MSA rows with shared pair bias, MSA columns without, pair rows (4 and 8 heads) ----
    for name, B, h, L, with_bias, scale in (("MSA row, shared pair bias", 256, 8, 256, True, 32 ** -0.5),
                                            ("MSA column, no bias", 256, 8, 256, False, 32 ** -0.5),
                                            ("pair, 8 heads, shared bias", 256, 8, 256, True, 16 ** -0.5),
                                            ("pair, 4 heads, shared bias", 256, 4, 256, True, 16 ** -0.5)):
        Q, K, V = (rnd(B, h, L, 32) / 32 ** 0.5 for _ in range(3))
        bias = rnd(h, L, L) if with_bias else None
        O = torch.empty((B, h, L, 32), device=dev)
        for kind, e, ts in (("fp32 operands (tf32 products)", 4, 0.5), ("bf16 operands", 2, 1.0)):
            q, k_, v = (Q, K, V) if e == 4 else (Q.bfloat16(), K.bfloat16(), V.bfloat16())
            f = lambda: ops.flash_attn_forward_cuda(q, k_, v, bias, scale=scale, bias_bcast=with_bias, path=PATH_UMMA, out=O)
            us = graph_time_us(torch, lambda: [f() for _ in range(4)], 4)
            fl = 4.0 * B * h * L * L * 32
            by = (3 * e + 4.0) * B * h * L * 32 + (4.0 * h * L * L if with_bias else 0.0) + 4.0 * B * h * L
            b0 = B // 3
            rO, _ = oracle.flash_attn(host(q[b0:b0 + 1]), host(k_[b0:b0 + 1]), host(v[b0:b0 + 1]), None if bias is None else host(bias),
                                      scale=scale, bias_bcast=with_bias)
            ok = rel(host(O[b0:b0 + 1]), rO) <= (1e-3 if e == 4 else 1e-2)
            recs.append({"kernel": "umma_attn_kernel", "op": "flash_attn_forward, " + kind, "workload": f"{name}: B'={B} h={h} L={L} d=32",
                         "us": us, "tflops": fl / us / 1e6, "gbs": by / us / 1e3, "roofline": roofline(fl, by, us, peaks, ts), "checked": bool(ok)})
        del Q, K, V, O

    # ---- the same attention on token-major operands (Q, K, V as column ranges of one fused projection output) with the
    # sigmoid gate applied in the store, and the backward (exact fp32 CUDA-core kernels) on the forward's O and LSE ----
    B, h, L, hd = 256, 8, 256, 256
    t = rnd(B, L, 4 * hd) / 32 ** 0.5
    bias = rnd(h, L, L)
    Ot = torch.empty((B, L, hd), device=dev)
    f = lambda: ops.flash_attn_tokens(t[:, :, 0:hd], t[:, :, hd:2 * hd], t[:, :, 2 * hd:3 * hd], h, bias=bias, gate=t[:, :, 3 * hd:],
                                      act="sigmoid", scale=32 ** -0.5, bias_bcast=True, path=PATH_UMMA, out=Ot)
    us = graph_time_us(torch, lambda: [f() for _ in range(4)], 4)
    fl = 4.0 * B * h * L * L * 32
    by = 5 * 4.0 * B * L * hd + 4.0 * h * L * L                       # Q, K, V, gate read, O written, shared bias
    b0 = B // 3
    heads = lambda x: host(x[b0:b0 + 1]).reshape(1, L, h, 32).transpose(0, 2, 1, 3)
    rO, _ = oracle.flash_attn(heads(t[:, :, 0:hd]), heads(t[:, :, hd:2 * hd]), heads(t[:, :, 2 * hd:3 * hd]), host(bias),
                              scale=32 ** -0.5, bias_bcast=True)
    rO = rO * (1.0 / (1.0 + np.exp(-heads(t[:, :, 3 * hd:]).astype(np.float64))))
    ok = rel(host(Ot[b0:b0 + 1]).reshape(1, L, h, 32).transpose(0, 2, 1, 3), rO) <= 1e-3
    recs.append({"kernel": "umma_attn_kernel", "op": "flash_attn_forward on token-major operands, sigmoid(gate) * O in the store",
                 "workload": f"MSA row, shared pair bias: B'={B} h={h} L={L} d=32, row stride 1024", "us": us, "tflops": fl / us / 1e6,
                 "gbs": by / us / 1e3, "roofline": roofline(fl, by, us, peaks, 0.5), "checked": bool(ok)})
    del t, Ot
    B = 64
    Q, K, V, dO = (rnd(B, h, L, 32) / 32 ** 0.5 for _ in range(4))
    O, LSE = ops.flash_attn_forward_cuda(Q, K, V, bias, scale=32 ** -0.5, bias_bcast=True, path=PATH_UMMA)
    grads = {"dQ": torch.empty_like(Q), "dK": torch.empty_like(Q), "dV": torch.empty_like(Q), "dbias": torch.empty((B, h, L, L), device=dev)}
    def issue_bwd():
        ops.flash_attn_backward_cuda(Q, K, V, O, dO, LSE, bias, scale=32 ** -0.5, bias_bcast=True, out=grads)
    us = graph_time_us(torch, issue_bwd, 1, reps=5)
    fl = 2 * 5 * 2.0 * B * h * L * L * 32                              # five products, each computed by both kernels' tiles
    by = 4.0 * (8 * B * h * L * 32 + h * L * L + B * h * L * L)        # Q, K, V, O, dO read; dQ, dK, dV, dbias written
    b0 = B // 3
    rO, rL = oracle.flash_attn(host(Q[b0:b0 + 1]), host(K[b0:b0 + 1]), host(V[b0:b0 + 1]), host(bias), scale=32 ** -0.5, bias_bcast=True)
    ref = oracle.flash_attn_backward(host(Q[b0:b0 + 1]), host(K[b0:b0 + 1]), host(V[b0:b0 + 1]), rO, host(dO[b0:b0 + 1]), rL, host(bias),
                                     scale=32 ** -0.5, bias_bcast=True)
    ok = all(rel(host(grads[n][b0:b0 + 1]), ref[n]) <= 2e-3 for n in ("dQ", "dK", "dV", "dbias"))      # the forward ran in tf32
    recs.append({"kernel": "attn_bwd_dq_kernel + attn_bwd_dkv_kernel", "op": "flash_attn_backward (dQ, dK, dV, dbias), exact fp32 on CUDA cores",
                 "workload": f"MSA row, shared pair bias: B'={B} h={h} L={L} d=32", "us": us, "tflops": fl / us / 1e6, "gbs": by / us / 1e3,
                 "roofline": {"bound": "fp32 CUDA cores", "achieved": fl / us / 1e6, "peak": None, "unit": "TFLOP/s", "frac": None},
                 "checked": bool(ok)})
    del Q, K, V, dO, O, LSE, grads

    # ---- extra-MSA row attention (head dim 8, shared pair bias): the warp-level tensor-core kernel ----
    B, h, L = 1024, 8, 256
    Q, K, V = (rnd(B, h, L, 8) / 8 ** 0.5 for _ in range(3))
    bias = rnd(h, L, L)
    O = torch.empty((B, h, L, 8), device=dev)
    f = lambda: ops.flash_attn_forward_cuda(Q, K, V, bias, scale=8 ** -0.5, bias_bcast=True, path=PATH_UMMA, out=O)
    us = graph_time_us(torch, lambda: [f() for _ in range(2)], 2)
    fl = 4.0 * B * h * L * L * 8
    by = 16.0 * B * h * L * 8 + 4.0 * h * L * L + 4.0 * B * h * L
    b0 = B // 3
    rO, _ = oracle.flash_attn(host(Q[b0:b0 + 1]), host(K[b0:b0 + 1]), host(V[b0:b0 + 1]), host(bias), scale=8 ** -0.5, bias_bcast=True)
    ok = rel(host(O[b0:b0 + 1]), rO) <= 1e-3
    recs.append({"kernel": "attn_d8_mma_kernel", "op": "flash_attn_forward, fp32 operands (tf32 products, mma.sync)",
                 "workload": f"extra-MSA row, shared pair bias: B'={B} h={h} L={L} d=8", "us": us, "tflops": fl / us / 1e6,
                 "gbs": by / us / 1e3, "roofline": roofline(fl, by, us, peaks, 0.5), "checked": bool(ok)})
    del Q, K, V, O

    # ---- pair-track contractions (configs[3]) ----
    D = 128
    for L in (128, 256, 384):
        for outgoing in (True, False):
            ws = 3 * 4.0 * D * L * L
            R = rotations(ws)
            lefts = [rnd(D, L, L, 1) for _ in range(R)]
            rights = [rnd(D, L, L, 1) for _ in range(R)]
            for kind, e, ts in (("fp32 operands (tf32 products)", 4, 0.5), ("bf16 operands", 2, 1.0)):
                ls, rs = (lefts, rights) if e == 4 else ([t.bfloat16() for t in lefts], [t.bfloat16() for t in rights])
                out = []

                def issue():
                    out.clear()
                    for i in range(max(R, 4)):
                        out.append(ops.tri_mul_cuda(ls[i % R], rs[i % R], float(L), outgoing, path=PATH_UMMA))
                us = graph_time_us(torch, issue, max(R, 4))
                fl, by = 2.0 * D * L ** 3, (2 * e + 4.0) * D * L * L
                ref = oracle.tri_mul(host(ls[0][5:6]), host(rs[0][5:6]), float(L), outgoing)
                ok = rel(host(out[0][5:6]), ref) <= (1e-3 if e == 4 else 1e-5)
                recs.append({"kernel": "umma_gemm_kernel", "op": "tri_mul " + ("outgoing" if outgoing else "incoming") + ", " + kind,
                             "workload": f"D=128 channel slabs, L={L}", "us": us, "tflops": fl / us / 1e6, "gbs": by / us / 1e3,
                             "roofline": roofline(fl, by, us, peaks, ts), "checked": bool(ok)})
            del lefts, rights
    c, L, N = 32, 256, 256
    left, right = rnd(c, L, N, 1), rnd(c, L, N, 1)
    for kind, e, ts in (("fp32 operands (tf32 products)", 4, 0.5), ("bf16 operands", 2, 1.0)):
        l_, r_ = (left, right) if e == 4 else (left.bfloat16(), right.bfloat16())
        out = []

        def issue():
            out.clear()
            for _ in range(2):
                out.append(ops.outer_prod_mean_cuda(l_, r_, path=PATH_UMMA))
        us = graph_time_us(torch, issue, 2, reps=10)
        fl, by = 2.0 * (c * L) ** 2 * N, 2 * e * c * L * N + 4.0 * (c * L) ** 2
        ref = oracle.outer_prod_mean(host(l_[3:4]), host(r_[9:10]))
        ok = rel(host(out[0][3 * c + 9:3 * c + 10]), ref) <= (1e-3 if e == 4 else 1e-5)
        recs.append({"kernel": "umma_gemm_kernel", "op": "outer_prod_mean, " + kind, "workload": f"c={c} L={L} N={N} (8192 x 8192 x 256)",
                     "us": us, "tflops": fl / us / 1e6, "gbs": by / us / 1e3, "roofline": roofline(fl, by, us, peaks, ts), "checked": bool(ok)})
    del left, right
    return recs


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from proteinpredictmachinelearning_b200 import PATH_AUTO, _lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        tt = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    peaks = load_peaks()
    # resident inputs: one X per (M, K), one W per (K, N), one C per (M, N); each rank seeds its own shard
    g = torch.Generator(device=dev).manual_seed(SEED + 1000 * rank)
    sh = shapes()
    if args.only:
        sh = [tuple(int(v) for v in args.only.split(","))]
    X = {(m, k): torch.randn((m, k), device=dev, generator=g) for (m, k) in sorted({(s[0], s[1]) for s in sh})}
    Wf = {(k, n): torch.randn((n, k), device=dev, generator=g) * 0.02 for (k, n) in sorted({(s[1], s[2]) for s in sh})}
    W = {kn: ops.quantize_q8_0r(w) for kn, w in Wf.items()}
    Cout = {s: torch.empty((s[0], s[2]), device=dev) for s in sh}          # one result buffer per shape (1.6 GB in all)
    pass_flops = sum(mm_flops(*s) for s in sh)
    pass_bytes = sum(q8_bytes(*s) for s in sh)

    def launch(m, k, n, Xs, Cs):
        _, taken = ops.mul_mat_q8_cuda(W[(k, n)], Xs[(m, k)], n, wtype=2, c_trans=1, path=PATH_AUTO, out=Cs[(m, k, n)])
        return taken

    taken_by_shape = {}

    def one_pass():
        for (m, k, n) in sh:
            taken_by_shape[(m, k, n)] = launch(m, k, n, X, Cout)

    for _ in range(max(args.warmup, 3)):
        one_pass()
    code, where = ops.device_status()
    if code != 0:
        raise RuntimeError(f"device abort {code} at {where:#x}")

    # ---- the timed region: K steps of `passes` replays of the captured pass -------------------------------------------
    graph, launch_mode = None, "eager, one call per launch"
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                one_pass()
            launch_mode = "one CUDA graph per pass (36 shapes), replayed"
        except Exception as exc:           # capture not possible: eager launches
            graph, launch_mode = None, f"eager (graph capture failed: {type(exc).__name__})"
    if world > 1:                          # every rank must run the same way
        flag = torch.tensor([1 if graph is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            graph = None
    run = graph.replay if graph is not None else one_pass
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        run()
    barrier()
    e0.record()
    for _ in range(5):
        run()
    e1.record()
    barrier()
    pass_ms_est = max_over_ranks(e0.elapsed_time(e1) / 5)
    # a step lasts at least 0.125 s and the timed region at least 2.6 s, so that the 100 ms clock sampler sees 20+ samples
    step_ms = max(125.0, 2600.0 / max(args.steps, 1))
    passes = args.passes if args.passes > 0 else max(1, int(math.ceil(step_ms / max(pass_ms_est, 1e-3))))
    for _ in range(max(args.warmup, 3)):   # W warm-up steps of the timed form
        for _ in range(passes if args.warmup_full else 1):
            run()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    e0.record()
    for _ in range(args.steps):
        for _ in range(passes):
            run()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else None
    code, where = ops.device_status()
    if code != 0:
        raise RuntimeError(f"device abort {code} at {where:#x}")
    n_pass = args.steps * passes
    umma_launches = sum(1 for s in sh if taken_by_shape.get(s) == 1) * n_pass
    kernel_launches = sum((_lib.load().ppml_b200_q8_kernel_launches(s[2], s[0], s[1]) if taken_by_shape.get(s) == 1 else 2)
                          for s in sh) * n_pass

    # ---- check of the timed launches' results: sampled token rows of every shape against the CPU checker --------------
    checked, check_note = None, "skipped (--no-check)"
    if not args.no_check:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from checkers import Oracle
        oracle = Oracle()
        worst, checked = 0.0, True
        r = np.random.default_rng(11 + rank)
        for (m, k, n) in sh:
            rows = np.unique(np.concatenate([[0, m - 1], r.integers(0, m, 30)]))
            idx = torch.from_numpy(rows).to(dev)
            w_host = W[(k, n)].cpu().numpy()
            ref = oracle.mul_mat_q8(w_host, X[(m, k)][idx].cpu().numpy(), n, wtype=2, c_trans=1)
            got = Cout[(m, k, n)][idx].cpu().numpy()       # what the last timed pass wrote
            err = float(np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))
            worst = max(worst, err)
            checked = checked and err <= 1e-5
        check_note = f"32 sampled token rows of each of the {len(sh)} shapes against the CPU checker, worst normalised error {worst:.2e} (bound 1e-5)"
        if world > 1:
            flag = torch.tensor([1 if checked else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            checked = bool(int(flag.item()))

    # ---- per-shape times: every shape from its own graph, small shapes rotating over copies larger than L2 -------------
    per_shape = []
    if rank == 0 and not args.no_per_shape:
        for (m, k, n) in sh:
            R = rotations(4.0 * m * (k + n)) if m < 65536 else 1
            xs = [X[(m, k)]] + [torch.randn((m, k), device=dev, generator=g) for _ in range(R - 1)]
            cs = [Cout[(m, k, n)]] + [torch.empty((m, n), device=dev) for _ in range(R - 1)]
            L = max(R, 4)

            def issue():
                for i in range(L):
                    ops.mul_mat_q8_cuda(W[(k, n)], xs[i % R], n, wtype=2, c_trans=1, path=PATH_AUTO, out=cs[i % R])
            us = graph_time_us(torch, issue, L, reps=10)
            fl, by = mm_flops(m, k, n), q8_bytes(m, k, n)
            per_shape.append({"M": m, "K": k, "N": n, "us": us, "tflops": fl / us / 1e6, "gbs": by / us / 1e3,
                              "hbm_frac": by / us / 1e3 / peaks["hbm_gbs"], "tensor_cores": taken_by_shape.get((m, k, n))})
            del xs, cs

    if args.no_e2e:
        if rank == 0:
            print(json.dumps({"only": args.only, "ms_per_pass": ms / n_pass, "passes_per_step": passes,
                              "tflops": pass_flops * n_pass * world / (ms * 1e-3) / 1e12,
                              "gbs": pass_bytes * n_pass / (ms * 1e-3) / 1e9, "checked": checked,
                              "per_shape_us": {"%dx%dx%d" % (p["M"], p["K"], p["N"]): round(p["us"], 2) for p in per_shape}}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end with host buffers ("e2e") ----------------------------------------------------------------------
    Xh = {key: torch.empty(t.shape, dtype=torch.float32).pin_memory().copy_(t.cpu()) for key, t in X.items()}
    Ch = {key: torch.empty(t.shape, dtype=torch.float32).pin_memory() for key, t in Cout.items()}
    h2d = sum(t.numel() * 4 for t in Xh.values())
    d2h = sum(t.numel() * 4 for t in Ch.values())
    # Three streams: host -> device copies, kernels, device -> host copies.  Inputs and results are double-buffered on
    # the device, so the copies of step i + 1 (in) and of step i (out) overlap; every step still copies all of its
    # inputs in and the result of every one of its 36 products out.
    Xd = [X, {key: torch.empty_like(t) for key, t in X.items()}]
    Cd = [Cout, {key: torch.empty_like(t) for key, t in Cout.items()}]
    comp = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    done_comp, done_out = [None, None], [None, None]

    def e2e_step(i):
        buf = i & 1
        if done_comp[buf] is not None:
            s_in.wait_event(done_comp[buf])        # the kernels of step i - 2 have read these inputs
        ev_in = {}
        with torch.cuda.stream(s_in):
            for key, t in Xh.items():
                Xd[buf][key].copy_(t, non_blocking=True)
                ev_in[key] = torch.cuda.Event()
                ev_in[key].record(s_in)
        if done_out[buf] is not None:
            comp.wait_event(done_out[buf])         # the results of step i - 2 have left these buffers
        ev_c, seen = {}, set()
        for idx, (m, k, n) in enumerate(sh):
            if (m, k) not in seen:
                comp.wait_event(ev_in[(m, k)])
                seen.add((m, k))
            launch(m, k, n, Xd[buf], Cd[buf])
            ev_c[(m, k, n)] = torch.cuda.Event()
            ev_c[(m, k, n)].record(comp)
        done_comp[buf] = torch.cuda.Event()
        done_comp[buf].record(comp)
        with torch.cuda.stream(s_out):
            for key, ev in ev_c.items():
                s_out.wait_event(ev)
                Ch[key].copy_(Cd[buf][key], non_blocking=True)
            done_out[buf] = torch.cuda.Event()
            done_out[buf].record(s_out)

    def e2e_drain():
        for ev in done_out:
            if ev is not None:
                comp.wait_event(ev)

    e2e_steps = max(3, min(args.steps, 10))
    e2e_step(0)
    e2e_drain()
    barrier()
    done_comp, done_out = [None, None], [None, None]
    e0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_drain()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    code, where = ops.device_status()
    if code != 0:
        raise RuntimeError(f"device abort {code} at {where:#x}")
    del Xh, Ch, Xd, Cd

    # ---- the other kernels of the path (rank 0) and the sharded block (all ranks) -----------------------------------
    kernels = dev_calls = None
    if rank == 0 and not args.no_kernels:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from checkers import Oracle
        oracle = Oracle()
        kernels = kernel_records(torch, dev, peaks, oracle)
        dev_calls = dev_forward_calls(torch, dev, oracle)
    barrier()
    block = extra_block = None
    if not args.no_block:
        from proteinpredictmachinelearning_b200 import block_bench
        block = block_bench.measure(steps=max(5, min(args.steps, 20)), warmup=3)
        extra_block = block_bench.measure(steps=max(5, min(args.steps, 20)), warmup=3, kind="extra")
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    achieved = pass_bytes * n_pass / (ms * 1e-3) / 1e9
    value = pass_flops * n_pass * world / (ms * 1e-3) / 1e12
    line = {
        "metric": "mul_mat TFLOPS", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "q8 (int8 x int8 -> int32, fp32 rescale)", "data": "synthetic",
        "config": {"workload": "configs[1] Q8 block-quantized mul_mat sweep, 36 shapes per pass", "K": list(KS),
                   "N": list(NS), "M": list(MS), "seed": SEED, "sharding": f"token rows, {world} shard(s)",
                   "passes_per_step": passes, "ms_per_pass": ms / n_pass,
                   "l2": "working set per pass (~0.9 GB) exceeds L2, no explicit flush", "launch": launch_mode},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "traffic": Q8_SWEEP_DRAM_BYTES_PER_LAUNCH if not args.only else None,
                     "algorithmic_bytes_per_launch": pass_bytes / max(len(sh), 1), "peak_kind": peaks["kind"],
                     "kernel": "umma_q8_kernel: algorithmic bytes of all launches of the timed region / its CUDA-event duration "
                               "(the same region `value` comes from; it also holds the activation quantizer launches of the two-pass shapes)"},
        "e2e": {"value": pass_flops * e2e_steps * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
        "gpu_launches": kernel_launches, "tensor_core_launches": umma_launches, "clocks": clocks,
        "checked": checked, "check": check_note,
        "per_shape": per_shape,
    }
    if kernels is not None:
        line["kernels"] = kernels
        line["checked_kernels"] = all(k.get("checked", True) for k in kernels)
        line["dev_forward_calls"] = dev_calls
    if block is not None:
        line["sharded_block"] = block
        line["sharded_extra_block"] = extra_block
    # CPU baseline on rank 0, N = 1 only
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_record()
        if not args.no_kernels:
            line["cpu_baseline"]["reference_cpu_kernels"] = reference_cpu_kernels()
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one pass of the sweep (36 launches of umma_q8_kernel and the 11
# activation-quantizer launches of its two-pass shapes, as in the timed region) from one ncu capture on a B200, divided
# by 36; the capture command and the per-kernel figures are in profiles/q8_sweep_launches_and_dram.md.
Q8_SWEEP_DRAM_BYTES_PER_LAUNCH = 82.9e6


def single_kernel(args):
    """Profiling runs (--kernel ...): one kernel on one workload, launched directly (no graph) so that ncu sees plain
    launches; prints one JSON line with the CUDA-event time."""
    import torch
    from proteinpredictmachinelearning_b200 import PATH_UMMA, TF32_TMA, ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    if args.kernel in ("attn", "attn_bf16", "attn8"):
        B, h, L = (int(v) for v in args.only.split(",")) if args.only else (64, 8, 256)
        d = 8 if args.kernel == "attn8" else 32                  # attn8: the extra-MSA head dim (warp-level tensor-core kernel)
        Q, K, V = (torch.randn(B, h, L, d, device=dev, generator=g) / d ** 0.5 for _ in range(3))
        bias = torch.randn(h, L, L, device=dev, generator=g)
        if args.kernel == "attn_bf16":
            Q, K, V = Q.bfloat16(), K.bfloat16(), V.bfloat16()
        f = lambda: ops.flash_attn_forward_cuda(Q, K, V, bias, scale=1 / d ** 0.5, bias_bcast=True, path=PATH_UMMA)
        what = {"B": B, "h": h, "L": L, "d": d}
    else:
        m, k, n = (int(v) for v in args.only.split(",")) if args.only else (65536, 256, 256)
        A, Bw = torch.randn(m, k, device=dev, generator=g), torch.randn(n, k, device=dev, generator=g) * 0.02
        Cc = torch.empty((m, n), device=dev)
        if args.kernel == "bf16":
            A, Bw = A.bfloat16(), Bw.bfloat16()
            f = lambda: ops.mul_mat_16(A, Bw, path=PATH_UMMA, out=Cc)
        else:
            f = lambda: ops.mul_mat_cuda(A, Bw, path=PATH_UMMA, tf32_mode=TF32_TMA, out=Cc)
        what = {"M": m, "K": k, "N": n}
    for _ in range(max(args.warmup, 3)):
        f()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        f()
    e1.record()
    torch.cuda.synchronize()
    what.update({"kernel": args.kernel, "us": e0.elapsed_time(e1) / args.steps * 1e3})
    print(json.dumps(what), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--passes", type=int, default=0, help="replays of the sweep per step (0: as many as make a step last 0.125 s or more and the timed region 2.6 s)")
    ap.add_argument("--warmup-full", action="store_true", help="warm-up steps replay `passes` passes too (default: one pass each)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="stop after the device-resident region (profiling runs)")
    ap.add_argument("--no-graph", action="store_true", help="launch the passes one call at a time (ncu launch lists)")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--no-per-shape", action="store_true")
    ap.add_argument("--no-kernels", action="store_true", help="skip the records of the other kernels")
    ap.add_argument("--no-block", action="store_true", help="skip the sharded IterBlock record")
    ap.add_argument("--only", default="", help="M,K,N: run a single shape of the sweep (profiling runs); B,h,L with --kernel attn")
    ap.add_argument("--kernel", default="q8", choices=["q8", "tf32", "bf16", "attn", "attn_bf16", "attn8"],
                    help="profiling runs: one launch kind on one workload, launched directly")
    ap.add_argument("--workload", default="sweep", choices=["sweep", "block", "extra_block"],
                    help="block / extra_block: only the sharded IterBlock / extra-MSA FullBlock record "
                         "(proteinpredictmachinelearning_b200/block_bench.py)")
    args = ap.parse_args()
    if args.workload in ("block", "extra_block"):
        from proteinpredictmachinelearning_b200 import block_bench
        return block_bench.run(args.gpus, args.steps, args.warmup, kind="main" if args.workload == "block" else "extra")
    if args.kernel != "q8":
        return single_kernel(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
