"""Throughput of the pairwise-reduction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload``): batched ``minkowski_distances(p=3)`` forward + backward in fp32 on
X, Y [16, 4096, 256] i.i.d. N(0,1) with an upstream gradient [16, 4096, 4096] -- 268.4 M pairs per
step, seeded synthetic data.  One step = one forward + backward over the batch.  With N > 1 ranks
every rank runs its own 16 batches (the path shards by batch with no data-path collective), so the
job is weakly scaled and ``value`` is the sum over ranks divided by the slowest rank's time.

One JSON line is printed by rank 0.  ``value`` is timed with the inputs resident in HBM; ``e2e``
times the same step through the public API from pinned host buffers (inputs copied in, both
gradients copied out, every step).  ``roofline`` describes the dominant kernel (the backward tile
kernel, two launches per step), timed alone with CUDA events on its stream; its bound is the fp32
issue rate, measured live by the library's register-only microbenchmark, and ``roofline_hbm``
restates the same launch against the measured copy bandwidth.  ``cpu_baseline`` times the
reference's own CPU operators (built from its sources into oracle/_ref) on a bounded row block.

``--impl reference`` times that CPU implementation alone, on the same workload definition, each
step a bounded row block.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "Gpairs/s, minkowski_distances(p=3) forward+backward, fp32"
B, N1, N2, D, P = 16, 4096, 4096, 256, 3.0
PAIRS_PER_STEP = B * N1 * N2
# lane-operations of the dominant kernel per pair and feature: subtract, d*|d|, fused multiply-add
BWD_OPS_PER_ELEMENT = 3
# algorithmic HBM bytes of one backward launch: upstream gradient + forward output read once,
# both operands read once, one gradient written
BWD_BYTES_PER_LAUNCH = 4 * (2 * B * N1 * N2 + 3 * B * N1 * D)
# dram__bytes_read.sum + dram__bytes_write.sum of one backward launch: 589.6 MB measured by ncu at
# batch 4 (profiles/lp_kernels_c2_minkowski_p3.md); the traffic is the streamed gradient and forward
# output, so it grows in proportion to the batch
BWD_DRAM_TRAFFIC_BYTES_PER_BATCH = 589.6e6 / 4

REF_SO = ROOT / "oracle" / "_ref" / "torchpairwise_ref.so"


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []
        self.t_begin = self.t_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def mark_begin(self):
        self.t_begin = time.perf_counter()

    def mark_end(self):
        self.t_end = time.perf_counter()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [ln for t, ln in self.lines if self.t_begin is None or (self.t_begin <= t <= (self.t_end or t) + 0.06)]
        if not inside:  # region shorter than one sampling period: take the samples nearest to it
            inside = [ln for _, ln in self.lines[-2:]]
        for ln in inside:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_reference_step(rows: int, threads: int):
    """One forward + backward of the reference's CPU operators on a row block of the workload:
    X[1, rows, 256] against Y[1, 4096, 256].  Returns (seconds, pairs, kind)."""
    import torch
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    X = torch.randn(1, rows, D, generator=g).requires_grad_(True)
    Y = torch.randn(1, N2, D, generator=g).requires_grad_(True)
    G = torch.randn(1, rows, N2, generator=g)
    if REF_SO.exists():
        if not getattr(cpu_reference_step, "_loaded", False):
            torch.ops.load_library(str(REF_SO))
            cpu_reference_step._loaded = True
        fn = lambda: torch.ops.torchpairwise.minkowski_distances(X, Y, P).backward(G)  # noqa: E731
        kind = "reference"
    else:
        from oracle import pairwise_oracle as O
        xn, yn, gn = X.detach().numpy(), Y.detach().numpy(), G.numpy()
        fn = lambda: O.cdist_backward(gn, xn, yn, P, out=O.cdist(xn, yn, P))  # noqa: E731
        kind = "port"
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0, rows * N2, kind


def run_reference(args, rank: int):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows = 512  # the same row block as the cpu_baseline leg of the GPU arm
    cpu_reference_step(rows, threads)  # library load + first-touch, not counted as a warm-up step
    for _ in range(args.warmup):
        cpu_reference_step(rows, threads)
    t0 = time.perf_counter()
    kind = "port"
    for _ in range(args.steps):
        _, pairs, kind = cpu_reference_step(rows, threads)
    dt = time.perf_counter() - t0
    value = args.steps * rows * N2 / dt / 1e9
    sample = f"per step: batch 1 of 16, rows 0:{rows} of 4096 against all 4096 columns, D=256, forward+backward"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "Gpairs/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C2 minkowski p=3 fwd+bwd: X,Y[16,4096,256], G[16,4096,4096] fp32 N(0,1) seed 0",
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": "Gpairs/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "Gpairs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist
    import torchpairwise_b200 as tpw
    from torchpairwise_b200 import _abi

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # per-rank seeded synthetic inputs, generated on the host so that the e2e leg can reuse them
    g = torch.Generator().manual_seed(1000 + rank)
    Xh = torch.randn(B, N1, D, generator=g).pin_memory()
    Yh = torch.randn(B, N2, D, generator=g).pin_memory()
    Gh = torch.randn(B, N1, N2, generator=g).pin_memory()
    X = Xh.to(dev).requires_grad_(True)
    Y = Yh.to(dev).requires_grad_(True)
    G = Gh.to(dev)

    def step():
        X.grad = None
        Y.grad = None
        out = tpw.minkowski_distances(X, Y, P)
        out.backward(G)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # started before the warm-up so that nvidia-smi is already streaming in the timed region
    for _ in range(args.warmup):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark_begin()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    sampler.mark_end()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = world * args.steps * PAIRS_PER_STEP / (ms * 1e-3) / 1e9
    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "not_a_bench_value": value, "batches": B, "ms_per_step": ms / args.steps}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end: host buffers in, gradients out, every step ---------------------------------
    g1h = torch.empty(B, N1, D).pin_memory()
    g2h = torch.empty(B, N2, D).pin_memory()

    from torchpairwise_b200.host_pipeline import forward_backward_from_host

    def e2e_step():
        # public API for host-resident operands: copies of chunk c+1 overlap the kernels of chunk c
        forward_backward_from_host(tpw.minkowski_distances, Xh, Yh, Gh, g1h, g2h, dev, chunk=2, p=P)

    e2e_step()
    barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    e2e = world * args.steps * PAIRS_PER_STEP / (ms_e2e * 1e-3) / 1e9

    # ---- row-sharded dense metric with x2 broadcast over NCCL (strong scaling; reported beside the headline) ----
    sharded = None
    if world > 1:
        from torchpairwise_b200 import sharding
        rows_total, cols, feat = 131072, 16384, 512
        kind, ranges = sharding.plan_shards((rows_total, feat), world)
        lo, hi = ranges[rank]
        gs = torch.Generator().manual_seed(2000 + rank)
        Xs = torch.randn(hi - lo, feat, generator=gs).to(dev)
        Ys = torch.randn(cols, feat, generator=torch.Generator().manual_seed(7)).to(dev) if rank == 0 else torch.empty(cols, feat, device=dev)

        def sharded_step():
            with torch.no_grad():
                return sharding.sharded_pairwise(tpw.sqeuclidean_distances, Xs, Ys, src=0)

        for _ in range(2):
            slab = sharded_step()
        barrier()
        e0.record()
        for _ in range(5):
            slab = sharded_step()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1) / 5], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sharded = {"workload": "C4 sqeuclidean X[131072,512] row-sharded, Y[16384,512] broadcast from rank 0 every step (NCCL)",
                   "ms_per_step": float(t.item()), "Gpairs_s": rows_total * cols / (float(t.item()) * 1e-3) / 1e9,
                   "slab_rows_rank0": hi - lo, "scaling": "strong"}
        del slab, Xs, Ys

    line = None
    if rank == 0:
        # ---- dominant kernel alone: backward w.r.t. x1 (grad + forward output streamed) -----------
        with torch.no_grad():
            out = tpw.minkowski_distances(X, Y, P)
        g1 = torch.empty_like(X)
        stream = torch.cuda.current_stream().cuda_stream

        def bwd_launch():
            _abi.check(_abi.lib.tpw_lp_backward(_abi.F32, _abi.LP_BWD_CDIST, G.data_ptr(), out.data_ptr(),
                                                X.data_ptr(), Y.data_ptr(), None, g1.data_ptr(), None,
                                                B, N1, N2, D, P, stream))

        for _ in range(3):
            bwd_launch()
        torch.cuda.synchronize()
        reps = max(5, args.steps)
        e0.record()
        for _ in range(reps):
            bwd_launch()
        e1.record()
        torch.cuda.synchronize()
        k_ms = e0.elapsed_time(e1) / reps
        ops = PAIRS_PER_STEP * D * BWD_OPS_PER_ELEMENT
        fp32_peak = tpw.measure_issue_peak(0)
        achieved = ops / (k_ms * 1e-3)
        hbm_peak, hbm_src = load_peaks()
        roofline = {"bound": "fp32_issue", "achieved": achieved / 1e12, "peak": fp32_peak / 1e12,
                    "unit": "Tlane-op/s", "frac": achieved / fp32_peak, "traffic": BWD_DRAM_TRAFFIC_BYTES_PER_BATCH * B,
                    "kernel": "lp_backward_kernel (grad_x1 pass, p=3)", "ms_per_launch": k_ms,
                    "peak_source": "live register-only FFMA microbenchmark (tpw_measure_issue_peak)"}
        roofline_hbm = {"bound": "hbm", "achieved": BWD_BYTES_PER_LAUNCH / (k_ms * 1e-3) / 1e9, "peak": hbm_peak,
                        "unit": "GB/s", "frac": BWD_BYTES_PER_LAUNCH / (k_ms * 1e-3) / 1e9 / hbm_peak,
                        "traffic": BWD_DRAM_TRAFFIC_BYTES_PER_BATCH * B, "peak_source": hbm_src}
        # ---- other metrics of the path, a few launches each (not part of the timed K steps) --------
        extra = {}

        def timeit(fn, n=3):
            fn()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n

        def cheb():
            X.grad = None
            Y.grad = None
            tpw.chebyshev_distances(X, Y).backward(G)

        extra["chebyshev_fwd_bwd_C2_Gpairs_s"] = PAIRS_PER_STEP / (timeit(cheb) * 1e-3) / 1e9
        with torch.no_grad():
            extra["minkowski_p3_fwd_C2_Gpairs_s"] = PAIRS_PER_STEP / (timeit(lambda: tpw.minkowski_distances(X, Y, P)) * 1e-3) / 1e9
        del out, g1
        # ---- CPU baseline: the reference's own operators on a bounded row block -------------------
        threads = os.cpu_count() or 1
        rows = 512
        cpu_reference_step(64, threads)
        secs, pairs, kind = cpu_reference_step(rows, threads)
        cpu_baseline = {"value": pairs / secs / 1e9, "unit": "Gpairs/s", "cores": threads, "kind": kind,
                        "sample": f"batch 1 of 16, rows 0:{rows} of 4096 against all 4096 columns, D=256, forward+backward, "
                                  f"{secs:.1f} s"}
        line = {
            "metric": METRIC, "value": value, "unit": "Gpairs/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "C2 minkowski p=3 fwd+bwd: X,Y[16,4096,256], G[16,4096,4096] fp32 N(0,1) per GPU",
                       "pairs_per_step_per_gpu": PAIRS_PER_STEP, "parallelism": f"batch-sharded x{world}, no collective",
                       "l2": "inputs larger than L2 (2.1 GB of gradient + output streamed per step)"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "Gpairs/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": 4 * (B * N1 * D + B * N2 * D + B * N1 * N2),
                    "d2h_bytes_per_step": 4 * (B * N1 * D + B * N2 * D)},
            "gpu_launches": 3 * args.steps,
            "roofline": roofline, "roofline_hbm": roofline_hbm, "cpu_baseline": cpu_baseline, "extra": extra,
            "sharded_dense": sharded,
            "device_status": tpw.device_status(),
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def run_suite(args):
    """Kernel-level throughput of every metric on the five benchmark configurations (1 GPU).

    Times are CUDA-event averages over ``--steps`` launches after ``--warmup`` launches, inputs
    resident in HBM, outputs larger than L2 except where noted.  Roofline fractions use the issue
    rates measured live by the library (fp32 FMA, POPC), the copy bandwidth and the sustained
    bf16 matmul rate of MEASURED_PEAKS.json."""
    import torch
    import torchpairwise_b200 as tpw

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    fp32_peak = tpw.measure_issue_peak(0)
    popc_peak = tpw.measure_issue_peak(2)
    hbm_peak, _ = load_peaks()
    pk = ROOT / "MEASURED_PEAKS.json"
    bf16_peak = float(json.loads(pk.read_text())["bf16_tflops_sustained"]) * 1e12 if pk.exists() else 1.4e15
    only = set(filter(None, args.suite_only.split(",")))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    res = {"peaks": {"fp32_lane_ops_per_s": fp32_peak, "popc_per_s": popc_peak, "hbm_GBps": hbm_peak,
                     "bf16_flops_per_s_sustained": bf16_peak}, "entries": {}}

    def timeit(fn):
        for _ in range(max(1, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps * 1e-3

    def entry(name, pairs, secs, bound, work, peak, out_bytes):
        res["entries"][name] = {"ms": secs * 1e3, "Gpairs_s": pairs / secs / 1e9, "bound": bound,
                                "frac_of_bound": work / secs / peak, "hbm_frac_output_only": out_bytes / secs / 1e9 / hbm_peak}

    g = torch.Generator().manual_seed(0)
    want = lambda n: not only or n in only  # noqa: E731
    # ---- C1: X[1024,128], Y[2048,128] (tiny: launch-latency bound, L2 resident) ---------------------
    X, Y = torch.randn(1024, 128, generator=g).to(dev), torch.randn(2048, 128, generator=g).to(dev)
    n = 1024 * 2048
    for name, fn, ops in (("C1_euclidean", tpw.euclidean_distances, 2), ("C1_manhattan", tpw.manhattan_distances, 2),
                          ("C1_cosine", tpw.cosine_distances, 1)):
        if want(name):
            entry(name, n, timeit(lambda: fn(X, Y)), "fp32_issue (L2 resident, launch bound)", n * 128 * ops, fp32_peak, 4 * n)
    # ---- C2: X,Y[16,4096,256] forward and backward kernels ------------------------------------------
    X = torch.randn(args.batches, 4096, 256, generator=g).to(dev).requires_grad_(True)
    Y = torch.randn(args.batches, 4096, 256, generator=g).to(dev).requires_grad_(True)
    G = torch.randn(args.batches, 4096, 4096, generator=g).to(dev)
    n = args.batches * 4096 * 4096
    for name, p, fo, bo in (("C2_minkowski_p3", 3.0, 3, 6), ("C2_chebyshev", math.inf, 2, 8), ("C2_manhattan", 1.0, 2, 8),
                            ("C2_minkowski_p2.5", 2.5, 5, 12)):
        if want(name + "_fwd"):
            with torch.no_grad():
                entry(name + "_fwd", n, timeit(lambda: tpw.minkowski_distances(X, Y, p)), "fp32_issue", n * 256 * fo, fp32_peak, 4 * n)
        if want(name + "_bwd"):
            out = tpw.minkowski_distances(X, Y, p)

            def bwd():
                X.grad = None
                Y.grad = None
                out.backward(G, retain_graph=True)
            entry(name + "_bwd", n, timeit(bwd), "fp32_issue", n * 256 * bo, fp32_peak, 0)
            del out
    # weighted Minkowski p = 3 at C2 (w [16,256]): forward, and backward including grad_w
    if want("C2_wminkowski_p3_fwd") or want("C2_wminkowski_p3_bwd"):
        W = (torch.rand(args.batches, 256, generator=g) + 0.5).to(dev).requires_grad_(True)
        if want("C2_wminkowski_p3_fwd"):
            with torch.no_grad():
                entry("C2_wminkowski_p3_fwd", n, timeit(lambda: tpw.wminkowski_distances(X, Y, 3.0, W)), "fp32_issue", n * 256 * 3, fp32_peak, 4 * n)
        if want("C2_wminkowski_p3_bwd"):
            out = tpw.wminkowski_distances(X, Y, 3.0, W)

            def bwdw():
                X.grad = None
                Y.grad = None
                W.grad = None
                out.backward(G, retain_graph=True)
            entry("C2_wminkowski_p3_bwd", n, timeit(bwdw), "fp32_issue (coefficient forward + grad_x1, grad_x2, grad_w passes)", n * 256 * (3 + 4 + 4 + 4), fp32_peak, 0)
            del out
        del W
    # canberra at C2: a sum of two-argument terms (one approximate reciprocal per term)
    if want("C2_canberra_fwd"):
        with torch.no_grad():
            entry("C2_canberra_fwd", n, timeit(lambda: tpw.canberra_distances(X, Y)), "fp32_issue (4 lane-ops + 1 MUFU per term)", n * 256 * 4, fp32_peak, 4 * n)
    if want("C2_canberra_bwd"):
        out = tpw.canberra_distances(X, Y)

        def bwdc():
            X.grad = None
            Y.grad = None
            out.backward(G, retain_graph=True)
        entry("C2_canberra_bwd", n, timeit(bwdc), "fp32_issue (two passes)", n * 256 * 2 * 8, fp32_peak, 0)
        del out
    # Jensen-Shannon at C2 shape on non-negative rows: bound by the special-function unit (one reciprocal and two
    # logarithms per term forward, one and one backward; 16 per clock and SM)
    mufu_peak = fp32_peak / 8.0
    if want("C2_jensenshannon_fwd") or want("C2_jensenshannon_bwd"):
        Hx, Hy = X.detach().abs().requires_grad_(True), Y.detach().abs().requires_grad_(True)
        if want("C2_jensenshannon_fwd"):
            with torch.no_grad():
                entry("C2_jensenshannon_fwd", n, timeit(lambda: tpw.jensenshannon_distances(Hx, Hy)), "mufu (3 per term)", n * 256 * 3, mufu_peak, 4 * n)
        if want("C2_jensenshannon_bwd"):
            out = tpw.jensenshannon_distances(Hx, Hy)

            def bwdj():
                Hx.grad = None
                Hy.grad = None
                out.backward(G, retain_graph=True)
            entry("C2_jensenshannon_bwd", n, timeit(bwdj), "mufu (two passes, 2 per term)", n * 256 * 2 * 2, mufu_peak, 0)
            del out
        del Hx, Hy
    # haversine on (latitude, longitude) rows: D = 2, the forward writes 4 bytes per pair, the backward reads 4
    if want("haversine_fwd") or want("haversine_bwd"):
        scale = torch.tensor([math.pi, 2 * math.pi])
        P1 = ((torch.rand(32768, 2, generator=g) - 0.5) * scale).to(dev).requires_grad_(True)
        P2 = ((torch.rand(16384, 2, generator=g) - 0.5) * scale).to(dev).requires_grad_(True)
        nh = 32768 * 16384
        if want("haversine_fwd"):
            with torch.no_grad():
                entry("haversine_fwd", nh, timeit(lambda: tpw.haversine_distances(P1, P2)), "hbm (output write)", 4 * nh, hbm_peak * 1e9, 4 * nh)
        if want("haversine_bwd"):
            out = tpw.haversine_distances(P1, P2)
            GH = torch.randn(32768, 16384, generator=g).to(dev)

            def bwdh():
                P1.grad = None
                P2.grad = None
                out.backward(GH, retain_graph=True)
            entry("haversine_bwd", nh, timeit(bwdh), "hbm (gradient read twice)", 8 * nh, hbm_peak * 1e9, 0)
            del out, GH
        del P1, P2
    # dense-contraction backward at C2: two tf32x3 tensor-core products per call (executed flops = 3 x 4 n D);
    # the tf32 rate is taken as half of the measured sustained bf16 rate
    for name, fn in (("C2_sqeuclidean_bwd", tpw.sqeuclidean_distances), ("C2_euclidean_bwd", tpw.euclidean_distances),
                     ("C2_cosine_bwd", tpw.cosine_distances)):
        if want(name):
            out = fn(X, Y)

            def bwd():
                X.grad = None
                Y.grad = None
                out.backward(G, retain_graph=True)
            entry(name, n, timeit(bwd), "tf32 tensor (executed flops = 3 x algorithmic; split pre-pass included)", 3 * 4 * n * 256, bf16_peak / 2, 0)
            del out
    if want("C2_sqeuclidean_bwd_simt"):
        tpw.set_dot_engine("simt")
        out = tpw.sqeuclidean_distances(X, Y)

        def bwd():
            X.grad = None
            Y.grad = None
            out.backward(G, retain_graph=True)
        entry("C2_sqeuclidean_bwd_simt", n, timeit(bwd), "fp32_issue", n * 256 * 4, fp32_peak, 0)
        del out
        tpw.set_dot_engine("auto")
    if want("C2_manhattan_rowmin"):
        with torch.no_grad():
            entry("C2_manhattan_rowmin", n, timeit(lambda: tpw.pairwise_argmin_min(X, Y, "manhattan")), "fp32_issue (matrix never written)",
                  n * 256 * 2, fp32_peak, 0)
    del X, Y, G
    # ---- C3: bool X[65536,1024], Y[16384,1024] -------------------------------------------------------
    r3 = args.rows or 65536
    Xb, Yb = (torch.rand(r3, 1024, generator=g) < 0.1).to(dev), (torch.rand(16384, 1024, generator=g) < 0.1).to(dev)
    n = r3 * 16384
    for name, fn in (("C3_hamming", tpw.hamming_distances), ("C3_jaccard", tpw.jaccard_distances)):
        if want(name):
            entry(name, n, timeit(lambda: fn(Xb, Yb)), "popc_issue (executed: 0.5 POPC per word pair; bit-pack pre-pass included)", n * 32 * 0.5, popc_peak, 4 * n)
    del Xb, Yb
    # ---- C4: X[131072,512], Y[16384,512] --------------------------------------------------------------
    r4 = args.rows or 131072
    X, Y = torch.randn(r4, 512, generator=g).to(dev), torch.randn(16384, 512, generator=g).to(dev)
    n = r4 * 16384
    for name, fn in (("C4_sqeuclidean", tpw.sqeuclidean_distances), ("C4_cosine", tpw.cosine_distances)):
        if want(name):
            entry(name, n, timeit(lambda: fn(X, Y)), "bf16 tensor (executed flops = 3 x algorithmic)", 3 * 2 * n * 512, bf16_peak, 4 * n)
    if want("C4_sqeuclidean_rowmin"):
        entry("C4_sqeuclidean_rowmin", n, timeit(lambda: tpw.pairwise_argmin_min(X, Y, "sqeuclidean")),
              "bf16 tensor (executed flops = 3 x algorithmic; matrix never written)", 3 * 2 * n * 512, bf16_peak, 0)
    for kk in (8, 16):
        if want(f"C4_sqeuclidean_top{kk}"):
            entry(f"C4_sqeuclidean_top{kk}", n, timeit(lambda: tpw.pairwise_argkmin(X, Y, kk, "sqeuclidean")),
                  "bf16 tensor (executed flops = 3 x algorithmic; matrix never written)", 3 * 2 * n * 512, bf16_peak, 0)
    if want("C4_sqeuclidean_bwd"):
        Xg, Yg = X.clone().requires_grad_(True), Y.clone().requires_grad_(True)
        out = tpw.sqeuclidean_distances(Xg, Yg)
        G4 = torch.empty_like(out).normal_(generator=torch.Generator(device=dev).manual_seed(1))

        def bwd4():
            Xg.grad = None
            Yg.grad = None
            out.backward(G4, retain_graph=True)
        entry("C4_sqeuclidean_bwd", n, timeit(bwd4), "tf32 tensor (executed flops = 3 x algorithmic; split pre-pass included; row-blocked under the 8 GB scratch cap)",
              3 * 4 * n * 512, bf16_peak / 2, 0)
        del Xg, Yg, out, G4
    if want("C4_sqeuclidean_simt"):
        tpw.set_dot_engine("simt")
        entry("C4_sqeuclidean_simt", n, timeit(lambda: tpw.sqeuclidean_distances(X, Y)), "fp32_issue", n * 512 * 2, fp32_peak, 4 * n)
        tpw.set_dot_engine("auto")
    del X, Y
    # ---- output-bound shapes (small D): achieved HBM write bandwidth -------------------------------------------
    ro = args.rows or 65536
    X, Y = torch.randn(ro, 16, generator=g).to(dev), torch.randn(16384, 16, generator=g).to(dev)
    n = ro * 16384
    for name, fn in (("OB_manhattan_D16", tpw.manhattan_distances), ("OB_chebyshev_D16", tpw.chebyshev_distances),
                     ("OB_sqeuclidean_D16", tpw.sqeuclidean_distances)):
        if want(name):
            entry(name, n, timeit(lambda: fn(X, Y)), "hbm (output write)", 4 * n / 1e9, hbm_peak, 4 * n)
    # D = 16 costs 32 lane-operations per 4-byte output: the fp32 pipe (0.92 ms at peak) bounds it before the write
    # does (0.66 ms).  D = 8, 4 and 3 are the shapes the output write really bounds.
    for dd in (8, 4, 3):
        if want(f"OB_manhattan_D{dd}") or want(f"OB_euclidean_D{dd}"):
            Xs, Ys = torch.randn(ro, dd, generator=g).to(dev), torch.randn(16384, dd, generator=g).to(dev)
            if want(f"OB_manhattan_D{dd}"):
                entry(f"OB_manhattan_D{dd}", n, timeit(lambda: tpw.manhattan_distances(Xs, Ys)), "hbm (output write)", 4 * n / 1e9, hbm_peak, 4 * n)
            if want(f"OB_euclidean_D{dd}"):
                entry(f"OB_euclidean_D{dd}", n, timeit(lambda: tpw.euclidean_distances(Xs, Ys)), "hbm (output write)", 4 * n / 1e9, hbm_peak, 4 * n)
            del Xs, Ys
    if want("NN_euclidean_D3"):
        Xs, Ys = torch.randn(ro, 3, generator=g).to(dev), torch.randn(16384, 3, generator=g).to(dev)
        entry("NN_euclidean_D3", n, timeit(lambda: tpw.pairwise_argmin_min(Xs, Ys, "euclidean")),
              "fp32_issue (nearest row of 16384 for every point, matrix never written)", n * 3 * 2, fp32_peak, 0)
        del Xs, Ys
    if want("KNN8_euclidean_D3") or want("KNN16_euclidean_D3"):
        Xs, Ys = torch.randn(ro, 3, generator=g).to(dev), torch.randn(16384, 3, generator=g).to(dev)
        for kk in (8, 16):
            if want(f"KNN{kk}_euclidean_D3"):
                entry(f"KNN{kk}_euclidean_D3", n, timeit(lambda: tpw.pairwise_argkmin(Xs, Ys, kk, "euclidean")),
                      f"fp32_issue ({kk} nearest of 16384 points for every point, matrix never written)", n * 3 * 2, fp32_peak, 0)
        del Xs, Ys
    if want("RM_euclidean_D3"):
        Xs, Ys = torch.randn(ro, 3, generator=g).to(dev), torch.randn(16384, 3, generator=g).to(dev)
        entry("RM_euclidean_D3", n, timeit(lambda: tpw.radius_neighbors_mask(Xs, Ys, 1.0, "euclidean")),
              "fp32_issue (radius test, one byte per pair)", n * 3 * 2, fp32_peak, n)
        del Xs, Ys
    if want("OB_manhattan_D16_rowmin"):
        entry("OB_manhattan_D16_rowmin", n, timeit(lambda: tpw.pairwise_argmin_min(X, Y, "manhattan")),
              "fp32_issue (matrix never written)", n * 16 * 2, fp32_peak, 0)
    Xb, Yb = (torch.rand(ro, 64, generator=g) < 0.3).to(dev), (torch.rand(16384, 64, generator=g) < 0.3).to(dev)
    if want("OB_jaccard_D64"):
        entry("OB_jaccard_D64", n, timeit(lambda: tpw.jaccard_distances(Xb, Yb)), "hbm (output write)", 4 * n / 1e9, hbm_peak, 4 * n)
    X, Y = torch.randn(ro, 64, generator=g).to(dev), torch.randn(16384, 64, generator=g).to(dev)
    if want("OB_cosine_D64_tensor"):
        entry("OB_cosine_D64_tensor", n, timeit(lambda: tpw.cosine_distances(X, Y)), "hbm (output write)", 4 * n / 1e9, hbm_peak, 4 * n)
    del X, Y, Xb, Yb
    # ---- condensed self-distances: X[32768,256], 537 M pairs (i < j), against the full 1.07 G-pair matrix ----
    if want("PD_manhattan_pdist") or want("PD_manhattan_cdist_self"):
        Xp = torch.randn(32768, 256, generator=g).to(dev)
        npairs = 32768 * 32767 // 2
        if want("PD_manhattan_pdist"):
            entry("PD_manhattan_pdist", npairs, timeit(lambda: tpw.pdist(Xp, "manhattan")), "fp32_issue (pairs i < j only)", npairs * 256 * 2, fp32_peak, 4 * npairs)
        if want("PD_manhattan_cdist_self"):
            entry("PD_manhattan_cdist_self", 32768 * 32768, timeit(lambda: tpw.manhattan_distances(Xp)), "fp32_issue", 32768 * 32768 * 256 * 2, fp32_peak, 4 * 32768 * 32768)
        del Xp
    # ---- C5: point clouds [64,1,8192,3] ------------------------------------------------------------------
    P_ = torch.rand(64, 8192, 3, generator=g) * 2 - 1
    Q_ = P_ + 0.05 * torch.randn(64, 8192, 3, generator=g)
    x1, x2 = P_[:, None].to(dev).requires_grad_(True), Q_[:, None].to(dev).requires_grad_(True)
    n = 64 * 8192 * 8192
    if want("C5_hausdorff_fwd"):
        with torch.no_grad():
            entry("C5_hausdorff_fwd", n, timeit(lambda: tpw.directed_hausdorff_distances(x1, x2)), "fp32_issue (point pairs)", n * 9, fp32_peak, 0)
    if want("C5_hausdorff_fwd_bwd"):
        def hd():
            x1.grad = None
            x2.grad = None
            tpw.directed_hausdorff_distances(x1, x2)[0].sum().backward()
        entry("C5_hausdorff_fwd_bwd", n, timeit(hd), "fp32_issue (point pairs)", n * 9, fp32_peak, 0)
    res["device_status"] = tpw.device_status()
    print(json.dumps(res), flush=True)


def main():
    global B, PAIRS_PER_STEP, BWD_BYTES_PER_LAUNCH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batches", type=int, default=B,
                    help="batches per GPU (default 16 = the benchmark workload; smaller only for profiler captures)")
    ap.add_argument("--suite", action="store_true",
                    help="time every metric of the five benchmark configurations on one GPU (kernel time, inputs resident) "
                         "and print one JSON object with throughputs and roofline fractions; not the driver's bench line")
    ap.add_argument("--suite-only", default="", help="comma-separated subset of suite entries (for profiler captures)")
    ap.add_argument("--rows", type=int, default=0, help="suite: cap N1 of the unbatched configurations (profiler captures)")
    ap.add_argument("--profile", action="store_true",
                    help="run only the warm-up and timed steps (for ncu captures); prints a reduced line that is not a bench value")
    args = ap.parse_args()
    if args.batches != B:
        B = args.batches
        PAIRS_PER_STEP = B * N1 * N2
        BWD_BYTES_PER_LAUNCH = 4 * (2 * B * N1 * N2 + 3 * B * N1 * D)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.suite:
        run_suite(args)
    elif args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
