#!/usr/bin/env python
"""Benchmark of the dense-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the reference's Q8 benchmark configuration): the Q8 block-quantized mul_mat sweep -- weights W[N,K] ~
N(0, 0.02) quantized to int8 blocks of 32 with an fp16 scale (planar Q8_0R), activations X[M,K] ~ N(0,1)
quantized on the fly; K in {128, 256, 1024}, N in {128, 256, 512, 1024}, M in {408, 2601, 65536}; seed 2.
One step = one pass over all 36 shapes.  `value` is the whole-job rate with inputs resident in HBM;
`e2e` is the same pass through the C ABI with host buffers (pinned), copies inside the timed region.
At N > 1 GPUs every rank runs the sweep on its own shard of token rows (weak scaling, no data-path
collective: token rows are independent).

`--impl reference` times the reference arithmetic on the host cores: the reference ships no CPU kernel
for Q8 mul_mat (include/ppml/QuantBlocks.h:56), so this arm runs the CPU restatement of its CUDA kernel
(oracle/ppml_oracle.c) on a bounded sample of the same sweep, threaded over token rows.
"""
import argparse
import json
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


def shapes(ms=MS):
    return [(m, k, n) for m in ms for k in KS for n in NS]


def q8_flops(m, k, n):
    return 2.0 * m * k * n


def q8_bytes(m, k, n):
    """Algorithmic HBM bytes of one Q8 mul_mat: planar int8 weights with half scales, fp32
    activations in, fp32 result out."""
    return (34.0 / 32.0) * n * k + 4.0 * m * k + 4.0 * m * n


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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
# reference arm / CPU baseline: the restated reference arithmetic on the host cores
# ------------------------------------------------------------------------------------------------
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


def make_cpu_sample(oracle, ms):
    import numpy as np
    r = np.random.default_rng(SEED)
    sample, flops = [], 0.0
    for (m, k, n) in shapes(ms):
        w = (r.standard_normal((n, k)) * 0.02).astype(np.float32)
        x = r.standard_normal((m, k)).astype(np.float32)
        sample.append((oracle.repack_q8_0(oracle.quantize_q8_0(w)), x, n))
        flops += q8_flops(m, k, n)
    return sample, flops


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from checkers import Oracle
    oracle = Oracle()
    threads = os.cpu_count() or 1
    sample_ms = (408,)          # bounded sample: the 12 (K, N) pairs at M = 408 tokens
    sample, flops = make_cpu_sample(oracle, sample_ms)
    for _ in range(args.warmup):
        cpu_q8_pass(oracle, sample, threads)
    t = 0.0
    for _ in range(args.steps):
        t += cpu_q8_pass(oracle, sample, threads)
    val = flops * args.steps / t / 1e12
    line = {
        "impl": "reference", "metric": "mul_mat TFLOPS", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "q8 (int8 x int8 -> int32, fp32 rescale)", "data": "synthetic",
        "config": {"workload": "configs[1] Q8 block-quantized mul_mat sweep", "K": list(KS), "N": list(NS), "M": list(MS)},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": "the 12 (K,N) pairs of the sweep at M=408 tokens per step (the reference has no CPU "
                                   "Q8 kernel; restated CUDA arithmetic, threaded over token rows)"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from proteinpredictmachinelearning_b200 import PATH_AUTO, ops

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

    # resident inputs: one X per (M, K), one W per (K, N), one C per (M, N); each rank seeds its own shard
    g = torch.Generator(device=dev).manual_seed(SEED + 1000 * rank)
    sh = shapes()
    if args.only:
        sh = [tuple(int(v) for v in args.only.split(","))]
    X = {(m, k): torch.randn((m, k), device=dev, generator=g) for (m, k) in sorted({(s[0], s[1]) for s in sh})}
    Wf = {(k, n): torch.randn((n, k), device=dev, generator=g) * 0.02 for (k, n) in sorted({(s[1], s[2]) for s in sh})}
    W = {kn: ops.quantize_q8_0r(w) for kn, w in Wf.items()}
    Cout = {(m, n): torch.empty((m, n), device=dev) for (m, n) in sorted({(s[0], s[2]) for s in sh})}
    if args.kernel == "bf16":
        X16 = {key: t.bfloat16() for key, t in X.items()}
        W16 = {key: t.bfloat16() for key, t in Wf.items()}
    step_flops = sum(q8_flops(*s) for s in sh)
    step_bytes = sum(q8_bytes(*s) for s in sh)

    def launch(m, k, n, Xs, Cs):
        if args.kernel == "q8":
            _, taken = ops.mul_mat_q8_cuda(W[(k, n)], Xs[(m, k)], n, wtype=2, c_trans=1, path=PATH_AUTO, out=Cs[(m, n)])
        elif args.kernel == "tf32":
            ops.mul_mat_cuda(Xs[(m, k)], Wf[(k, n)], path=PATH_AUTO, tf32_mode=1, out=Cs[(m, n)])
            taken = 1
        else:
            ops.mul_mat_16(X16[(m, k)], W16[(k, n)], path=PATH_AUTO, out=Cs[(m, n)])
            taken = 1
        return taken

    def one_pass(events=None):
        for (m, k, n) in sh:
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
            taken = launch(m, k, n, X, Cout)
            if events is not None:
                e1.record()
                events.append(((m, k, n), taken, e0, e1))

    for _ in range(max(args.warmup, 3)):
        one_pass()
    code, where = ops.device_status()
    if code != 0:
        raise RuntimeError(f"device abort {code} at {where:#x}")

    # ---- timed region 1: device-resident ("value") --------------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    events = []
    barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        one_pass(events)
    t1.record()
    barrier()
    eager_ms = t0.elapsed_time(t1)
    # The same K passes replayed from one captured CUDA graph: with 24 of the 36 launches lasting 10-20 us, launching
    # them one by one from Python leaves the GPU waiting for the host between kernels.  The per-launch events above
    # (roofline, per-shape times) come from the eager passes; `value` from the replay when capture is possible.
    ms, launch_mode, graph = eager_ms, "eager, one call per launch", None
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                one_pass()
        except Exception as exc:           # capture not possible: the eager figure stands
            graph, launch_mode = None, f"eager (graph capture failed: {type(exc).__name__})"
        # every rank takes the same barriers whether or not its capture worked
        run = graph.replay if graph is not None else one_pass
        for _ in range(2):
            run()
        barrier()
        t0.record()
        for _ in range(args.steps):
            run()
        t1.record()
        barrier()
        if graph is not None:
            ms, launch_mode = t0.elapsed_time(t1), "one CUDA graph per pass (36 launches), replayed"
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    kernel_ms = sum(e0.elapsed_time(e1) for (_, _, e0, e1) in events)
    per_shape = {}
    for (s, taken, e0, e1) in events:
        d = per_shape.setdefault(s, [0.0, 0, taken])
        d[0] += e0.elapsed_time(e1)
        d[1] += 1
    umma_launches = sum(1 for (_, taken, _, _) in events if taken == 1)
    # kernels launched in the timed region: the product kernel of every shape, plus the activation quantizer of the
    # shapes that take the two-pass form (the library reports which)
    from proteinpredictmachinelearning_b200 import _lib
    kernel_launches = sum((_lib.load().ppml_b200_q8_kernel_launches(s[2], s[0], s[1]) if (taken == 1 and args.kernel == "q8") else 1)
                          for (s, taken, _, _) in events)

    # ---- timed region 2: end to end with host buffers ("e2e") ----------------------------------------
    if args.no_e2e:
        if rank == 0:
            print(json.dumps({"only": args.only, "ms_per_step": ms / args.steps, "kernel_ms_per_step": kernel_ms / args.steps,
                              "tflops": step_flops * args.steps / (kernel_ms * 1e-3) / 1e12,
                              "gbs": step_bytes * args.steps / (kernel_ms * 1e-3) / 1e9,
                              "per_shape_us": {"%dx%dx%d" % s: 1e3 * v[0] / v[1] for s, v in sorted(per_shape.items())}}),
                  flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    Xh = {key: torch.empty(t.shape, dtype=torch.float32).pin_memory().copy_(t.cpu()) for key, t in X.items()}
    Ch = {key: torch.empty(t.shape, dtype=torch.float32).pin_memory() for key, t in Cout.items()}
    h2d = sum(t.numel() * 4 for t in Xh.values())
    d2h = sum(t.numel() * 4 for t in Ch.values())

    # Three streams: host -> device copies, kernels, device -> host copies.  Inputs and results are double-buffered on
    # the device, so the copies of step i + 1 (in) and of step i (out) overlap; every step still copies all of its
    # inputs in and all of its results out.
    Xd = [X, {key: torch.empty_like(t) for key, t in X.items()}]
    Cd = [Cout, {key: torch.empty_like(t) for key, t in Cout.items()}]
    comp = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    last_writer = {}
    for idx, (m, k, n) in enumerate(sh):
        last_writer[(m, n)] = idx
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
            if last_writer[(m, n)] == idx:
                ev_c[(m, n)] = torch.cuda.Event()
                ev_c[(m, n)].record(comp)
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

    e2e_steps = max(1, min(args.steps, 5))
    e2e_step(0)
    e2e_drain()
    barrier()
    done_comp, done_out = [None, None], [None, None]
    u0 = torch.cuda.Event(enable_timing=True)
    u1 = torch.cuda.Event(enable_timing=True)
    u0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_drain()
    u1.record()
    barrier()
    e2e_ms = u0.elapsed_time(u1)
    if world > 1:
        tt = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item())
    code, where = ops.device_status()
    if code != 0:
        raise RuntimeError(f"device abort {code} at {where:#x}")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = load_peaks()
    achieved = step_bytes * args.steps / (kernel_ms * 1e-3) / 1e9
    value = step_flops * args.steps * world / (ms * 1e-3) / 1e12
    line = {
        "metric": "mul_mat TFLOPS", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "q8 (int8 x int8 -> int32, fp32 rescale)", "data": "synthetic",
        "config": {"workload": "configs[1] Q8 block-quantized mul_mat sweep, 36 shapes per step", "K": list(KS),
                   "N": list(NS), "M": list(MS), "seed": SEED, "sharding": f"token rows, {world} shard(s)",
                   "l2": "working set per step (~0.9 GB) exceeds L2, no explicit flush", "launch": launch_mode,
                   "eager_ms_per_step": eager_ms / args.steps},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": Q8_SWEEP_DRAM_BYTES_PER_LAUNCH if not args.only else None,
                     "algorithmic_bytes_per_launch": step_bytes / max(len(sh), 1), "peak_kind": peak_kind,
                     "kernel": "umma_q8_kernel, all launches of the timed region (sum of algorithmic bytes / sum of durations)"},
        "e2e": {"value": step_flops * e2e_steps * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": kernel_launches, "tensor_core_launches": umma_launches, "clocks": clocks,
        "per_shape": [{"M": s[0], "K": s[1], "N": s[2], "us": 1e3 * v[0] / v[1],
                       "tflops": q8_flops(*s) / (v[0] / v[1] * 1e-3) / 1e12,
                       "gbs": q8_bytes(*s) / (v[0] / v[1] * 1e-3) / 1e9, "tensor_cores": v[2]} for s, v in sorted(per_shape.items())],
    }

    # CPU baseline on rank 0, N = 1 only: the restated reference arithmetic on a bounded sample
    if world == 1 and not args.no_cpu_baseline:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from checkers import Oracle
        oracle = Oracle()
        threads = os.cpu_count() or 1
        sample, flops = make_cpu_sample(oracle, (408,))
        t = cpu_q8_pass(oracle, sample, threads)
        reps = 1
        while t < 10.0 and reps < 50:
            t += cpu_q8_pass(oracle, sample, threads)
            reps += 1
        line["cpu_baseline"] = {"value": flops * reps / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": f"the 12 (K,N) pairs at M=408 tokens, {reps} pass(es), threaded over token rows; "
                                          "the reference has no CPU Q8 kernel, this is the restated CUDA arithmetic"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one pass of the sweep (36 launches of umma_q8_kernel) from one ncu
# capture on a B200, divided by 36; the capture command and the per-launch figures are in
# profiles/q8_sweep_dram_traffic.md.  Below the algorithmic bytes: part of each result is still in L2 at kernel end.
Q8_SWEEP_DRAM_BYTES_PER_LAUNCH = 71.8e6


def attn_profile(args):
    """Profiling run (--kernel attn --no-e2e): MSA row attention of configs[2] cut to `--only B,h,L` (default
    64,8,256), head dim 32, shared pair bias [h, L, L]; prints one JSON line with the CUDA-event time."""
    import torch
    from proteinpredictmachinelearning_b200 import ops, PATH_UMMA
    dev = torch.device("cuda", 0)
    B, h, L = (int(v) for v in args.only.split(",")) if args.only else (64, 8, 256)
    g = torch.Generator(device=dev).manual_seed(3)
    Q, K, V = (torch.randn(B, h, L, 32, device=dev, generator=g) / 32 ** 0.5 for _ in range(3))
    bias = torch.randn(h, L, L, device=dev, generator=g)
    half = args.kernel == "attn_bf16"                       # bf16 Q/K/V (kind::f16 products), fp32 bias / softmax / output
    if half:
        Q, K, V = Q.bfloat16(), K.bfloat16(), V.bfloat16()
    f = lambda: ops.flash_attn_forward_cuda(Q, K, V, bias, scale=1 / 32 ** 0.5, bias_bcast=True, path=PATH_UMMA)
    for _ in range(max(args.warmup, 3)):
        f()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        f()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / args.steps * 1e3
    flops = 4.0 * B * h * L * L * 32
    nbytes = (10.0 if half else 16.0) * B * h * L * 32 + 4.0 * h * L * L + 4.0 * B * h * L
    print(json.dumps({"kernel": "umma_attn_kernel<bf16>" if half else "umma_attn_kernel", "B": B, "h": h, "L": L, "us": us, "tflops": flops / us / 1e6,
                      "gbs": nbytes / us / 1e3}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="stop after the device-resident region (profiling runs)")
    ap.add_argument("--no-graph", action="store_true", help="time the device-resident region with eager launches only")
    ap.add_argument("--only", default="", help="M,K,N: run a single shape of the sweep (profiling runs)")
    ap.add_argument("--kernel", default="q8", choices=["q8", "tf32", "bf16", "attn", "attn_bf16"],
                    help="profiling runs with --no-e2e: time the fp32 (tf32 tensor-core) or bf16 mul_mat on the same shapes")
    ap.add_argument("--workload", default="sweep", choices=["sweep", "block"],
                    help="block: the hot-path op sequence of one main IterBlock at full size, sharded over --gpus ranks "
                         "(proteinpredictmachinelearning_b200/block_bench.py); prints its own JSON line")
    args = ap.parse_args()
    if args.workload == "block":
        from proteinpredictmachinelearning_b200 import block_bench
        return block_bench.run(args.gpus, args.steps, args.warmup)
    if args.kernel in ("attn", "attn_bf16"):
        return attn_profile(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
