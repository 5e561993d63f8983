"""Throughput of the pairwise-reduction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload``): batched ``minkowski_distances(p=3)`` forward + backward in fp32 on
X, Y [16, 4096, 256] i.i.d. N(0,1) with an upstream gradient [16, 4096, 4096] -- 268.4 M pairs per
step, seeded synthetic data.  One step = one forward + backward over the batch.  With N > 1 ranks
every rank runs its own 16 batches (the path shards by batch with no data-path collective), so the
job is weakly scaled and ``value`` is the sum over ranks divided by the slowest rank's time.

One JSON line is printed by rank 0.  ``value`` is timed with the inputs resident in HBM through
``torch.ops.torchpairwise.minkowski_distances`` -- the reference's own operator name, served for CUDA
tensors by this package's C++ host layer (``drop_in`` puts the Python mirror of the same call beside
it).  ``e2e`` times the same step from pinned host buffers (inputs copied in, both gradients copied
out, every step) and carries the measured host-to-device ceiling of the box at this N.  ``roofline``
describes the dominant kernel (the one-pass backward: a pair's term is formed once and added to both
gradient sums; its finishing kernel that adds the row-block sums of grad_x2 is inside the timed call),
timed alone with CUDA events on its stream: ``frac`` counts the algorithmic lane-operations
(difference, shape term and two accumulations per pair and feature), which is also what the kernel
executes; the bound is the fp32 issue rate measured live by the library's register-only
microbenchmark, and ``roofline_hbm`` restates the same call against the measured copy bandwidth.
``two_launch_ms`` is the older form (one launch per gradient, 6 operations executed) on the same data.  ``cpu_baseline`` times the reference's own CPU operators (built from
its sources into oracle/_ref) on a bounded row block, best of three.

On one GPU the line also carries ``configs`` -- every benchmark configuration (C1 euclidean /
manhattan / cosine, C2 minkowski p=3 / chebyshev, C3 hamming / jaccard, C4 sqeuclidean / cosine, C5
directed Hausdorff) with its time, throughput and fraction of the bounding rate on the algorithmic
and on the executed work -- and ``parity``: the same outputs and gradients compared with the
reference's CPU operators on a row block (max error over tolerance; 0 mismatches for the boolean
metrics).  ``sharded_dense`` is the row-sharded C4 workload with the broadcast of Y inside the step
(at every N, with a same-run one-GPU time), ``sharded_backward`` the row-sharded forward + backward
whose x2 gradient is all-reduced (N > 1).

``--impl reference`` times the CPU implementation alone, on the same workload definition, each
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
# lane-operations of the dominant kernel per pair and feature: subtract, d*|d| and one fused multiply-add into each of
# the two gradient sums -- the algorithmic count for both gradients, and what the one-pass kernel executes
BWD_OPS_PER_ELEMENT = 4
# lane-operations per point pair of the Hausdorff row-minimum loop as executed
HAUSDORFF_EXECUTED_OPS = 7
# algorithmic HBM bytes of the backward: upstream gradient + forward output read once, both operands read once,
# both gradients written
BWD_BYTES_PER_LAUNCH = 4 * (2 * B * N1 * N2 + 2 * B * N1 * D + 2 * B * N2 * D)
# dram__bytes_read.sum + dram__bytes_write.sum of the backward call measured by ncu at batch 4
# (profiles/lp_kernels_c2_minkowski_p3.md): 831.9 MB in the one-pass kernel (gradient and forward output streamed
# once, 256 MB of row-block sums written) + 281.3 MB in the finishing kernel that reads them back; both grow in
# proportion to the batch
BWD_DRAM_TRAFFIC_BYTES_PER_BATCH = (831.9e6 + 281.3e6) / 4

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


RTOL, ATOL = 1e-4, 1e-5  # the fp32 parity contract; boolean metrics and Hausdorff indices are compared bit for bit


def load_reference_ops():
    """``torch.ops.torchpairwise`` served by the reference's own CPU operators (oracle/_ref), or None."""
    import torch
    if not REF_SO.exists():
        return None
    if not getattr(load_reference_ops, "_loaded", False):
        torch.ops.load_library(str(REF_SO))
        load_reference_ops._loaded = True
    return torch.ops.torchpairwise


def err_over_tol(got, ref, scale: float = 1.0) -> float:
    """max |got - ref| / (atol * scale + rtol * |ref|) over all elements; <= 1 meets the contract."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    if got.numel() == 0:
        return 0.0
    return float(((got - ref).abs() / (ATOL * scale + RTOL * ref.abs())).max())


def grad_scale(ref) -> float:
    """Gradients are sums of thousands of terms: their absolute tolerance is taken relative to the largest entry."""
    return 10.0 * max(1.0, float(ref.abs().max()))


def mismatches(got, ref) -> int:
    return int((got.cpu() != ref.cpu()).sum())


def best_of(fn, n: int = 3, warm: int = 1) -> float:
    for _ in range(warm):
        fn()
    best = math.inf
    for _ in range(n):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return best


def c2_inputs(seed: int):
    """X, Y [16,4096,256] and the upstream gradient [16,4096,4096] drawn in that order from one CPU generator."""
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randn(B, N1, D, generator=g), torch.randn(B, N2, D, generator=g), torch.randn(B, N1, N2, generator=g)


def c2_block(X, Y, G, rows: int):
    """Batch 0, rows 0:rows of X against all of Y: the row block the CPU reference is timed and compared on."""
    return X[0:1, :rows].clone(), Y[0:1].clone(), G[0:1, :rows].clone()


def cpu_fwd_bwd(op, x1, x2, g, **kw):
    """One forward + backward of a reference operator on CPU tensors; returns (out, grad_x1, grad_x2)."""
    a, b = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True)
    out = op(a, b, **kw)
    out.backward(g)
    return out.detach(), a.grad, b.grad


def run_reference(args, rank: int):
    """The reference's CPU implementation alone: every step is one forward + backward on the row block."""
    if rank != 0:
        return
    import torch
    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    rows = 512
    Xb, Yb, Gb = c2_block(*c2_inputs_block(0, rows), rows)
    T = load_reference_ops()
    if T is not None:
        kind = "reference"
        step = lambda: cpu_fwd_bwd(T.minkowski_distances, Xb, Yb, Gb, p=P)  # noqa: E731
    else:
        from oracle import pairwise_oracle as O
        kind = "port"
        xn, yn, gn = Xb.numpy(), Yb.numpy(), Gb.numpy()
        step = lambda: O.cdist_backward(gn, xn, yn, P, out=O.cdist(xn, yn, P))  # noqa: E731
    step()  # library load and first touch, not counted as a warm-up step
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
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


def c2_inputs_block(seed: int, rows: int):
    """The same draws as ``c2_inputs`` restricted to what the row block needs (batch 0), without the 1 GB gradient:
    X and Y are drawn in full, of the gradient only batch 0."""
    import torch
    g = torch.Generator().manual_seed(seed)
    X, Y = torch.randn(B, N1, D, generator=g), torch.randn(B, N2, D, generator=g)
    G0 = torch.randn(1, N1, N2, generator=g)  # the first N1*N2 draws of the [16,4096,4096] gradient are its batch 0
    return X, Y, G0


def load_tensor_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16_burst": float(d["bf16_tflops"]) * 1e12, "bf16_sustained": float(d["bf16_tflops_sustained"]) * 1e12,
                "tensor_source": "measured"}
    return {"bf16_burst": 1.59e15, "bf16_sustained": 1.4e15, "tensor_source": "fallback"}


def run_sharded_dense(T, tpw, dev, rank, world, barrier, max_over_ranks, gpu_ms):
    """C4 sqeuclidean with the rows of X cut over the ranks and Y broadcast from rank 0 by NCCL in every step
    (strong scaling).  Reports the step with and without the broadcast, a same-run one-GPU time of the whole
    problem, and the worst error of a sampled row block of every rank's slab against a float64 evaluation."""
    import torch
    from torchpairwise_b200 import sharding
    rows_total, cols, feat = 131072, 16384, 512
    _, ranges = sharding.plan_shards((rows_total, feat), world)
    lo, hi = ranges[rank]
    Xs = torch.randn(hi - lo, feat, generator=torch.Generator().manual_seed(2000 + rank)).to(dev)
    Ys = torch.randn(cols, feat, generator=torch.Generator().manual_seed(7)).to(dev) if rank == 0 else torch.empty(cols, feat, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, reps=5, warm=2):
        for _ in range(warm):
            fn()
        barrier()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / reps)

    slab = [None]

    def sharded_step():
        with torch.no_grad():
            slab[0] = sharding.sharded_pairwise(T.sqeuclidean_distances, Xs, Ys, src=0)

    def kernel_only():
        with torch.no_grad():
            slab[0] = T.sqeuclidean_distances(Xs, Ys)

    def panel_step():
        # Y crosses NVLink in two row chunks; the contraction of the first column panel runs while the second chunk lands
        slab[0] = sharding.sharded_pairwise_panels(T.sqeuclidean_distances, Xs, Ys, src=0, panels=2)

    ms_single = timed(sharded_step)
    ms_kernel = timed(kernel_only)  # Y is local on every rank after the broadcasts above
    ms_step = timed(panel_step) if world > 1 else ms_single
    if world > 1:   # the panels against the one-piece slab, bit for bit
        panels = slab[0]
        sharded_step()
        same = bool(torch.equal(torch.cat(panels, -1), slab[0]))
        del panels
    else:
        same = True
    sharded_step()
    blk = slice(max(0, (hi - lo) - 256), hi - lo)
    xd, yd = Xs[blk].double(), Ys.double()
    ref = (xd * xd).sum(1)[:, None] + (yd * yd).sum(1)[None, :] - 2.0 * (xd @ yd.t())
    err = float(((slab[0][blk].double() - ref).abs() / (ATOL + RTOL * ref.abs())).max())
    del xd, yd, ref
    worst = max_over_ranks(err)
    all_same = bool(max_over_ranks(0.0 if same else 1.0) == 0.0)   # a collective: every rank calls it
    slab[0] = None
    t1 = ms_step
    if world > 1:
        t1 = None
        if rank == 0:
            Xfull = torch.randn(rows_total, feat, device=dev)
            with torch.no_grad():
                t1 = gpu_ms(lambda: T.sqeuclidean_distances(Xfull, Ys), reps=3, warm=1)
            del Xfull
    del Xs, Ys
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    return {"workload": "C4 sqeuclidean X[131072,512] row-sharded (each rank generates its block in place), Y[16384,512] "
                        "broadcast from rank 0 every step (NCCL) in two row chunks, the second under the first column panel's kernel" if world > 1 else
                        "C4 sqeuclidean X[131072,512] x Y[16384,512] on one GPU (nothing to broadcast)",
            "ms_per_step": ms_step, "ms_per_step_one_broadcast": ms_single, "kernel_only_ms": ms_kernel,
            "panels_equal_one_piece_slab": all_same,
            "Gpairs_s": rows_total * cols / (ms_step * 1e-3) / 1e9,
            "one_gpu_ms_same_run": t1, "efficiency_vs_n1": t1 / (world * ms_step),
            "kernel_only_efficiency_vs_n1": t1 / (world * ms_kernel),
            "slab_rows_rank0": hi - lo, "scaling": "strong",
            "parity_worst_err_over_tol": worst,
            "parity_what": "last 256 rows of every rank's slab against a float64 evaluation on the same GPU, all 16384 columns, "
                           "max over ranks of max |err| / (1e-5 + 1e-4 |ref|)"}


def run_sharded_backward(T, dev, rank, world, barrier, max_over_ranks):
    """Forward + backward of minkowski p=3 with the rows of x1 cut over the ranks inside each batch: x2 is broadcast
    from rank 0 and the x2-gradient partials are summed by one all-reduce, the one collective that follows a
    kernel on this path.  Every rank also runs the whole problem alone and compares its slab and gradients."""
    import torch
    from torchpairwise_b200 import sharding
    nb = 2 if world > 2 else 1  # fewer batches than ranks, so the plan cuts rows
    g = torch.Generator().manual_seed(99)
    X1 = torch.randn(nb, 4096, 256, generator=g).to(dev)
    X2 = torch.randn(nb, 4096, 256, generator=g).to(dev)
    Gf = torch.randn(nb, 4096, 4096, generator=g).to(dev)
    kind, ranges = sharding.plan_shards(tuple(X1.shape), world)
    lo, hi = ranges[rank]
    x1l = sharding.local_block(X1, kind, ranges, rank).contiguous().requires_grad_(True)
    x2l = (X2.clone() if rank == 0 else torch.zeros_like(X2)).requires_grad_(True)
    gl = sharding.local_block(Gf, kind, ranges, rank).contiguous()
    out = [None]

    def step():
        x1l.grad = None
        x2l.grad = None
        out[0] = sharding.sharded_pairwise(T.minkowski_distances, x1l, x2l, src=0, p=P)
        out[0].backward(gl)

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(2):
        step()
    barrier()
    e0.record()
    for _ in range(5):
        step()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1) / 5)
    a, b = X1.clone().requires_grad_(True), X2.clone().requires_grad_(True)
    full = T.minkowski_distances(a, b, P)
    full.backward(Gf)
    sl = (slice(None), slice(lo, hi))
    errs = {"out": err_over_tol(out[0], full.detach()[sl]),
            "grad_x1": err_over_tol(x1l.grad, a.grad[sl], grad_scale(a.grad)),
            "grad_x2_after_all_reduce": err_over_tol(x2l.grad, b.grad, grad_scale(b.grad))}
    errs = {k: max_over_ranks(v) for k, v in errs.items()}
    if rank != 0:
        return None
    return {"workload": f"minkowski p=3 forward+backward, X1,X2[{nb},4096,256], plan '{kind}' over {world} ranks: x2 broadcast from "
                        "rank 0, x2-gradient partials all-reduced (NCCL), every step",
            "ms_per_step": ms, "Gpairs_s": nb * 4096 * 4096 / (ms * 1e-3) / 1e9,
            "parity_err_over_tol_vs_one_gpu": errs}


def run_configs(T, R, dev, gpu_ms, peaks, X, Y, G, hosts, args):
    """Every benchmark configuration on one GPU: time, throughput, fraction of the bounding rate on the algorithmic
    and on the executed work, and parity with the reference's CPU operators on the row block (or, for the small
    configurations, the whole problem).  Returns (configs, parity)."""
    import torch
    cfg, par = {}, {}
    fp32, popc, hbm = peaks["fp32"], peaks["popc"], peaks["hbm"]
    g0 = torch.Generator().manual_seed(0)

    def cpu_time(fn, n=1, warm=0):
        return best_of(fn, n=n, warm=warm) if R is not None else None

    def rate(pairs, secs):
        return None if not secs else pairs / secs / 1e9

    # ---- C1: X[1024,128] x Y[2048,128], whole problem on both sides --------------------------------------------
    X1, Y1 = torch.randn(1024, 128, generator=g0), torch.randn(2048, 128, generator=g0)
    G1 = torch.randn(1024, 2048, generator=g0)
    n = 1024 * 2048
    for name, lane_ops in (("euclidean_distances", 2), ("manhattan_distances", 2), ("cosine_distances", 1)):
        op = getattr(T, name)
        a, b, gd = X1.to(dev).requires_grad_(True), Y1.to(dev).requires_grad_(True), G1.to(dev)

        def fb():
            a.grad = None
            b.grad = None
            op(a, b).backward(gd)
        fwd = gpu_ms(lambda: op(a.detach(), b.detach()), reps=20, warm=3)
        both = gpu_ms(fb, reps=20, warm=3)
        e = {"fwd_ms": fwd, "fwd_bwd_ms": both, "Gpairs_s_fwd": n / (fwd * 1e-3) / 1e9, "Gpairs_s_fwd_bwd": n / (both * 1e-3) / 1e9,
             "bound": "launch latency and host overhead (2.1 M pairs, L2 resident)",
             "frac_algorithmic": n * 128 * lane_ops / (fwd * 1e-3) / fp32, "frac_of": "fp32 issue, forward"}
        if R is not None:
            ref = cpu_fwd_bwd(getattr(R, name), X1, Y1, G1)
            e["cpu_Gpairs_s_fwd_bwd"] = rate(n, cpu_time(lambda: cpu_fwd_bwd(getattr(R, name), X1, Y1, G1), n=3, warm=1))
            fb()
            got = op(a.detach(), b.detach())
            exact = getattr(R, name)(X1.double(), Y1.double())   # the same operator in float64: which side an error is on
            par["C1/" + name] = {"fwd": err_over_tol(got, ref[0]),
                                 "grad_x1": err_over_tol(a.grad, ref[1], grad_scale(ref[1])),
                                 "grad_x2": err_over_tol(b.grad, ref[2], grad_scale(ref[2])),
                                 "fwd_gpu_vs_float64": err_over_tol(got, exact), "fwd_cpu_reference_vs_float64": err_over_tol(ref[0], exact)}
        cfg["C1/" + name] = e
    # ---- C2: the resident benchmark tensors; CPU on batch 0, rows 0:512 ---------------------------------------------
    rows = 512
    Xb, Yb, Gb = c2_block(*hosts, rows)
    pairs = B * N1 * N2
    for name, kw, fwd_alg, bwd_alg, fwd_exe, bwd_exe in (("minkowski_distances", {"p": P}, 3, 4, 3, 4),
                                                         ("chebyshev_distances", {}, 2, 2, 2, 4)):
        op = getattr(T, name)

        def fb():
            X.grad = None
            Y.grad = None
            res = op(X, Y, **kw)
            res.backward(G)
            return res
        fwd = gpu_ms(lambda: op(X.detach(), Y.detach(), **kw), reps=5)
        both = gpu_ms(fb, reps=5)
        key = "C2/" + name + ("_p3" if kw else "")
        e = {"fwd_ms": fwd, "fwd_bwd_ms": both, "Gpairs_s_fwd": pairs / (fwd * 1e-3) / 1e9,
             "Gpairs_s_fwd_bwd": pairs / (both * 1e-3) / 1e9, "bound": "fp32_issue",
             "frac_algorithmic": pairs * D * (fwd_alg + bwd_alg) / (both * 1e-3) / fp32,
             "frac_executed": pairs * D * (fwd_exe + bwd_exe) / (both * 1e-3) / fp32,
             "fwd_frac_algorithmic": pairs * D * fwd_alg / (fwd * 1e-3) / fp32,
             "bwd_frac_algorithmic": pairs * D * bwd_alg / ((both - fwd) * 1e-3) / fp32,
             "lane_ops_per_pair_feature": {"algorithmic": [fwd_alg, bwd_alg], "executed": [fwd_exe, bwd_exe]}}
        if R is not None:
            ref = [None]

            def cpu():
                ref[0] = cpu_fwd_bwd(getattr(R, name), Xb, Yb, Gb, **kw)
            e["cpu_Gpairs_s_fwd_bwd"] = rate(rows * N2, cpu_time(cpu))
            e["cpu_sample"] = f"batch 1 of 16, rows 0:{rows}"
            res = fb()  # the full-size step: its output rows and grad_x1 rows of the block are compared as they are
            xb, yb = X[0:1, :rows].detach().clone().requires_grad_(True), Y[0:1].detach().clone().requires_grad_(True)
            op(xb, yb, **kw).backward(G[0:1, :rows])  # grad_x2 needs every row of x1: compared on the block alone
            par[key] = {"fwd": err_over_tol(res[0:1, :rows], ref[0][0]),
                        "grad_x1": err_over_tol(X.grad[0:1, :rows], ref[0][1], grad_scale(ref[0][1])),
                        "grad_x2": err_over_tol(yb.grad, ref[0][2], grad_scale(ref[0][2]))}
            del res, xb, yb
        cfg[key] = e
    X.grad = None
    Y.grad = None
    torch.cuda.empty_cache()
    # ---- C3: bool X[65536,1024] x Y[16384,1024], Bernoulli(0.1); CPU on rows 0:1024 ------------------------------
    rows = 1024
    Xb3, Yb3 = torch.rand(65536, 1024, generator=g0) < 0.1, torch.rand(16384, 1024, generator=g0) < 0.1
    xd, yd = Xb3.to(dev), Yb3.to(dev)
    pairs = 65536 * 16384
    for name in ("hamming_distances", "jaccard_distances"):
        op = getattr(T, name)
        t = gpu_ms(lambda: op(xd, yd), reps=3)
        e = {"fwd_ms": t, "Gpairs_s_fwd": pairs / (t * 1e-3) / 1e9,
             "bound": "hbm: the 4.29 GB output write (the pair counts are an 8-bit integer contraction on the tensor cores, "
                      "operands streamed from L2; on the popcount tile the bound was the POPC issue rate)",
             "frac_algorithmic": 4 * pairs / (t * 1e-3) / hbm, "frac_executed": 4 * pairs / (t * 1e-3) / hbm,
             "tensor_int8_TOPs": 2 * pairs * 1024 / (t * 1e-3) / 1e12,
             "vs_popc_issue_bound": pairs * 32 / (t * 1e-3) / popc,
             "work_per_pair": "algorithmic 4 bytes written; 2 x 1024 integer operations on the tensor cores; "
                              "vs_popc_issue_bound = 32 POPC per pair over the measured POPC rate (> 1: faster than any popcount kernel)"}
        if R is not None:
            ref = [None]

            def cpu():
                ref[0] = getattr(R, name)(Xb3[:rows], Yb3)
            e["cpu_Gpairs_s_fwd"] = rate(rows * 16384, cpu_time(cpu))
            e["cpu_sample"] = f"rows 0:{rows} against all 16384"
            par["C3/" + name] = {"mismatching_elements": mismatches(op(xd, yd)[:rows], ref[0]), "rule": "bit-exact"}
        cfg["C3/" + name] = e
    del xd, yd, Xb3, Yb3
    torch.cuda.empty_cache()
    # ---- C4: X[131072,512] x Y[16384,512]; CPU on rows 0:1024 -------------------------------------------------
    X4, Y4 = torch.randn(131072, 512, generator=g0), torch.randn(16384, 512, generator=g0)
    xd, yd = X4.to(dev), Y4.to(dev)
    pairs = 131072 * 16384
    for name, rows in (("sqeuclidean_distances", 1024), ("cosine_distances", 1024)):
        op = getattr(T, name)
        t = gpu_ms(lambda: op(xd, yd), reps=3)
        e = {"fwd_ms": t, "Gpairs_s_fwd": pairs / (t * 1e-3) / 1e9, "bound": "tensor (bf16, fp32 accumulate), then the 8.59 GB output write",
             "frac_algorithmic": pairs * 512 * 2 / (t * 1e-3) / peaks["bf16_burst"],
             "frac_executed": pairs * 512 * 6 / (t * 1e-3) / peaks["bf16_burst"],
             "frac_executed_of_sustained": pairs * 512 * 6 / (t * 1e-3) / peaks["bf16_sustained"],
             "frac_hbm_output_write": 4 * pairs / (t * 1e-3) / hbm,
             "work_per_pair": "algorithmic 2 D flop; executed 6 D (three bf16 products keep the fp32 tolerance); split pre-pass included",
             "peak_source": peaks["tensor_source"]}
        if R is not None:
            ref = [None]

            def cpu():
                ref[0] = getattr(R, name)(X4[:rows], Y4)
            e["cpu_Gpairs_s_fwd"] = rate(rows * 16384, cpu_time(cpu))
            e["cpu_sample"] = f"rows 0:{rows} against all 16384"
            par["C4/" + name] = {"fwd": err_over_tol(op(xd, yd)[:rows], ref[0])}
        cfg["C4/" + name] = e
    del xd, yd, X4, Y4
    torch.cuda.empty_cache()
    # ---- C5: 64 clouds of 8192 points, whole problem on both sides ------------------------------------------------
    P5 = torch.rand(64, 8192, 3, generator=g0) * 2 - 1
    Q5 = P5 + 0.05 * torch.randn(64, 8192, 3, generator=g0)
    x1h, x2h = P5[:, None].contiguous(), Q5[:, None].contiguous()
    a, b = x1h.to(dev).requires_grad_(True), x2h.to(dev).requires_grad_(True)
    ppairs = 64 * 8192 * 8192
    op = T.directed_hausdorff_distances

    def hd():
        a.grad = None
        b.grad = None
        res = op(a, b)
        res[0].backward(torch.ones_like(res[0]))
        return res
    fwd = gpu_ms(lambda: op(a.detach(), b.detach()), reps=5)
    both = gpu_ms(hd, reps=5)
    e = {"fwd_ms": fwd, "fwd_bwd_ms": both, "Gpointpairs_s_fwd": ppairs / (fwd * 1e-3) / 1e9,
         "Gpointpairs_s_fwd_bwd": ppairs / (both * 1e-3) / 1e9, "bound": "fp32_issue (point pairs; nothing but 64 results written)",
         "frac_algorithmic": ppairs * 7 / (both * 1e-3) / fp32, "frac_executed": ppairs * HAUSDORFF_EXECUTED_OPS / (both * 1e-3) / fp32,
         "fwd_frac_algorithmic": ppairs * 7 / (fwd * 1e-3) / fp32,
         "work_per_point_pair": f"algorithmic 7 lane-ops (3 subtract, multiply, 2 fused multiply-add, minimum); executed {HAUSDORFF_EXECUTED_OPS}"}
    if R is not None:
        ref = [None]

        def cpu():
            u, v = x1h.clone().requires_grad_(True), x2h.clone().requires_grad_(True)
            r = R.directed_hausdorff_distances(u, v)
            r[0].backward(torch.ones_like(r[0]))
            ref[0] = (r[0].detach(), r[1], r[2], u.grad, v.grad)
        e["cpu_Gpointpairs_s_fwd_bwd"] = rate(ppairs, cpu_time(cpu, n=3, warm=1))
        e["cpu_note"] = "the reference's loop leaves a row as soon as it falls below the running maximum, so it visits a fraction of the point pairs"
        res = hd()
        par["C5/directed_hausdorff_distances"] = {
            "fwd": err_over_tol(res[0], ref[0][0]), "values_bit_equal": bool(torch.equal(res[0].detach().cpu(), ref[0][0])),
            "index_mismatches": mismatches(res[1], ref[0][1]) + mismatches(res[2], ref[0][2]),
            "grad_x1": err_over_tol(a.grad, ref[0][3]), "grad_x2": err_over_tol(b.grad, ref[0][4])}
    cfg["C5/directed_hausdorff_distances"] = e
    return cfg, par


def bind_host_threads_near_gpu(local_rank: int):
    """Keep this process (and the pinned buffers it allocates afterwards) on the CPUs that sit next to its GPU,
    when the operating system says which those are and the process is allowed to run there.  Returns a note."""
    try:
        bus = subprocess.run(["nvidia-smi", "-i", str(local_rank), "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.strip().lower()
        node = Path(f"/sys/bus/pci/devices/{bus}/local_cpulist")
        if not node.exists():  # nvidia-smi prints an 8-digit PCI domain, sysfs a 4-digit one
            node = Path(f"/sys/bus/pci/devices/{bus[-12:]}/local_cpulist")
        cpus = set()
        for part in node.read_text().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        near = cpus & allowed
        if near and near != allowed:
            bind_host_threads_near_gpu.allowed = allowed
            os.sched_setaffinity(0, near)
            return f"bound to {len(near)} of {len(allowed)} allowed CPUs local to GPU {local_rank}"
        return f"all {len(allowed)} allowed CPUs are " + ("local" if near else "remote") + f" to GPU {local_rank}"
    except Exception as e:  # no sysfs entry, no permission: timing still valid, just not placed
        return f"not bound ({type(e).__name__})"


def host_threads_everywhere() -> int:
    """Undo ``bind_host_threads_near_gpu`` (the CPU reference legs get every CPU the process may use); returns how many."""
    allowed = getattr(bind_host_threads_near_gpu, "allowed", None)
    if allowed:
        os.sched_setaffinity(0, allowed)
    return len(os.sched_getaffinity(0))


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    affinity = bind_host_threads_near_gpu(local_rank)
    # The reference's CPU library first (when it was built): it defines the schemas and keeps serving CPU tensors;
    # the host layer of this package then registers the CUDA and AutogradCUDA kernels under the same names.
    R = load_reference_ops()
    import torchpairwise_b200 as tpw
    from torchpairwise_b200 import _abi
    tpw.load_torch_ops()
    T = torch.ops.torchpairwise
    if world > 1:
        # a short collective timeout: a rank that falls out of step ends the job in minutes, not in the default ten
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def gpu_ms(fn, reps: int = 3, warm: int = 1) -> float:
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    # per-rank seeded synthetic inputs (rank 0: seed 0), generated on the host so that the e2e leg can reuse them
    Xc, Yc, Gc = c2_inputs(rank)
    Xh, Yh, Gh = Xc.pin_memory(), Yc.pin_memory(), Gc.pin_memory()
    del Xc, Yc, Gc
    X = Xh.to(dev).requires_grad_(True)
    Y = Yh.to(dev).requires_grad_(True)
    G = Gh.to(dev)

    def step():  # the drop-in: the reference's operator name, dispatched to the sm_100a kernels for CUDA tensors
        X.grad = None
        Y.grad = None
        T.minkowski_distances(X, Y, P).backward(G)

    def mirror_step():  # the same kernels through the Python mirror of the operator surface (ctypes on the C ABI)
        X.grad = None
        Y.grad = None
        tpw.minkowski_distances(X, Y, P).backward(G)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # started before the warm-up so that nvidia-smi is already streaming in the timed region
    for _ in range(args.warmup):
        step()
    barrier()
    sampler.mark_begin()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    sampler.mark_end()
    ms = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else None
    value = world * args.steps * PAIRS_PER_STEP / (ms * 1e-3) / 1e9
    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "not_a_bench_value": value, "batches": B, "ms_per_step": ms / args.steps}))
        if world > 1:
            dist.destroy_process_group()
        return
    mirror_ms = gpu_ms(mirror_step, reps=max(3, args.steps // 2))

    # ---- end to end: host buffers in, gradients out, every step ---------------------------------
    g1h = torch.empty(B, N1, D).pin_memory()
    g2h = torch.empty(B, N2, D).pin_memory()
    from torchpairwise_b200.host_pipeline import forward_backward_from_host

    def e2e_step():
        # public API for host-resident operands: copies of chunk c+1 overlap the kernels of chunk c
        forward_backward_from_host(T.minkowski_distances, Xh, Yh, Gh, g1h, g2h, dev, chunk=2, p=P)

    e2e_step()
    barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))
    e2e = world * args.steps * PAIRS_PER_STEP / (ms_e2e * 1e-3) / 1e9
    h2d_bytes = 4 * (B * N1 * D + B * N2 * D + B * N1 * N2)
    # what the host side can deliver at this N: every rank copies the same pinned buffers to its GPU, nothing else runs
    stage = [torch.empty_like(t, device=dev) for t in (Xh, Yh, Gh)]

    def copy_in():
        for d_, h_ in zip(stage, (Xh, Yh, Gh)):
            d_.copy_(h_, non_blocking=True)

    copy_in()
    barrier()
    e0.record()
    for _ in range(3):
        copy_in()
    e1.record()
    barrier()
    ms_copy = max_over_ranks(e0.elapsed_time(e1) / 3)
    del stage
    h2d_ceiling = {"GBps_all_ranks": world * h2d_bytes / (ms_copy * 1e-3) / 1e9, "ms_per_step_floor": ms_copy,
                   "what": f"{world} rank(s) copying the step's {h2d_bytes / 1e9:.2f} GB of pinned inputs concurrently, no compute"}

    # ---- the split the path shards by when it is not batched: X rows over ranks, Y broadcast (C4) -------------
    sharded = run_sharded_dense(T, tpw, dev, rank, world, barrier, max_over_ranks, gpu_ms)
    sharded_bwd = run_sharded_backward(T, dev, rank, world, barrier, max_over_ranks) if world > 1 else None

    line = None
    if rank == 0:
        fp32_peak = tpw.measure_issue_peak(0)
        hbm_peak, hbm_src = load_peaks()
        # ---- dominant kernel alone: backward w.r.t. x1 (grad + forward output streamed) -----------
        with torch.no_grad():
            out = T.minkowski_distances(X, Y, P)
            drop_in_same_bits = bool(torch.equal(out, tpw.minkowski_distances(X, Y, P)))
        g1, g2 = torch.empty_like(X), torch.empty_like(Y)
        stream = torch.cuda.current_stream().cuda_stream
        nbytes = _abi.lib.tpw_lp_backward_scratch_bytes(_abi.F32, _abi.LP_BWD_CDIST, B, N1, N2, D, P)
        scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)

        def bwd_launch():
            _abi.check(_abi.lib.tpw_lp_backward_ws(_abi.F32, _abi.LP_BWD_CDIST, G.data_ptr(), out.data_ptr(),
                                                   X.data_ptr(), Y.data_ptr(), None, g1.data_ptr(), g2.data_ptr(),
                                                   B, N1, N2, D, P, scratch.data_ptr(), nbytes, stream))

        def bwd_two_launches():
            _abi.check(_abi.lib.tpw_lp_backward(_abi.F32, _abi.LP_BWD_CDIST, G.data_ptr(), out.data_ptr(),
                                                X.data_ptr(), Y.data_ptr(), None, g1.data_ptr(), g2.data_ptr(),
                                                B, N1, N2, D, P, stream))

        k_ms = gpu_ms(bwd_launch, reps=max(5, args.steps), warm=3)
        two_ms = gpu_ms(bwd_two_launches, reps=5, warm=2)
        algorithmic = PAIRS_PER_STEP * D * BWD_OPS_PER_ELEMENT
        fwd_ms = gpu_ms(lambda: T.minkowski_distances(X.detach(), Y.detach(), P), reps=5)
        step_ms = ms / args.steps
        roofline = {"bound": "fp32_issue", "achieved": algorithmic / (k_ms * 1e-3) / 1e12, "peak": fp32_peak / 1e12,
                    "unit": "Tlane-op/s", "frac": algorithmic / (k_ms * 1e-3) / fp32_peak,
                    "frac_executed": algorithmic / (k_ms * 1e-3) / fp32_peak,
                    "traffic": BWD_DRAM_TRAFFIC_BYTES_PER_BATCH * B,
                    "kernel": "lp_backward_onepass_kernel (both gradients, p=3) with its finishing lp_backward_onepass_sum_kernel"
                              if nbytes > 0 else "lp_backward_kernel, two launches",
                    "ms_per_launch": k_ms, "two_launch_ms": two_ms,
                    "algorithmic_work": "4 lane-ops per pair and feature for both gradients (subtract, d*|d|, one fused multiply-add "
                                        "into each sum); the one-pass kernel executes exactly these, the two-launch form 6",
                    "step_frac_algorithmic": PAIRS_PER_STEP * D * 7 / (step_ms * 1e-3) / fp32_peak,
                    "backward_frac_algorithmic": PAIRS_PER_STEP * D * 4 / ((step_ms - fwd_ms) * 1e-3) / fp32_peak,
                    "forward_frac_algorithmic": PAIRS_PER_STEP * D * 3 / (fwd_ms * 1e-3) / fp32_peak,
                    "peak_source": "live register-only FFMA microbenchmark (tpw_measure_issue_peak)"}
        roofline_hbm = {"bound": "hbm", "achieved": BWD_BYTES_PER_LAUNCH / (k_ms * 1e-3) / 1e9, "peak": hbm_peak,
                        "unit": "GB/s", "frac": BWD_BYTES_PER_LAUNCH / (k_ms * 1e-3) / 1e9 / hbm_peak,
                        "traffic": BWD_DRAM_TRAFFIC_BYTES_PER_BATCH * B, "peak_source": hbm_src}
        del out, g1, g2, scratch
        # ---- CPU baseline and parity on the row block: the reference's own operators ---------------
        threads = host_threads_everywhere()
        torch.set_num_threads(threads)
        rows = 512
        Xb, Yb, Gb = c2_block(Xh, Yh, Gh, rows)
        configs, parity = {}, {}
        if R is not None:
            secs = best_of(lambda: cpu_fwd_bwd(R.minkowski_distances, Xb, Yb, Gb, p=P), n=3, warm=1)
            kind = "reference"
        else:
            from oracle import pairwise_oracle as O
            xn, yn, gn = Xb.numpy(), Yb.numpy(), Gb.numpy()
            secs = best_of(lambda: O.cdist_backward(gn, xn, yn, P, out=O.cdist(xn, yn, P)), n=1, warm=0)
            kind = "port"
        cpu_baseline = {"value": rows * N2 / secs / 1e9, "unit": "Gpairs/s", "cores": threads, "kind": kind,
                        "sample": f"batch 1 of 16, rows 0:{rows} of 4096 against all 4096 columns, D=256, forward+backward, "
                                  f"best of 3 after one warm-up, {secs:.2f} s"}
        if world == 1 and not args.no_configs:
            peaks = {"fp32": fp32_peak, "popc": tpw.measure_issue_peak(2), "hbm": hbm_peak * 1e9}
            peaks.update(load_tensor_peaks())
            configs, parity = run_configs(T, R, dev, gpu_ms, peaks, X, Y, G, (Xh, Yh, Gh), args)
        line = {
            "metric": METRIC, "value": value, "unit": "Gpairs/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "C2 minkowski p=3 fwd+bwd: X,Y[16,4096,256], G[16,4096,4096] fp32 N(0,1) per GPU",
                       "pairs_per_step_per_gpu": PAIRS_PER_STEP, "parallelism": f"batch-sharded x{world}, no collective",
                       "l2": "inputs larger than L2 (2.1 GB of gradient + output streamed per step)",
                       "api": "torch.ops.torchpairwise.minkowski_distances (the reference's operator name; CUDA tensors are "
                              "served by libtpw_b200_torch.so)",
                       "reference_cpu_library_loaded": R is not None},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "Gpairs/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4 * (B * N1 * D + B * N2 * D),
                    "host_h2d_gbs_ceiling": h2d_ceiling, "host_placement": affinity},
            "gpu_launches": 3 * args.steps,
            "roofline": roofline, "roofline_hbm": roofline_hbm, "cpu_baseline": cpu_baseline,
            "drop_in": {"ms_per_step": ms / args.steps, "python_mirror_ms_per_step": mirror_ms,
                        "same_bits_as_mirror": drop_in_same_bits},
            "configs": configs, "parity": parity,
            "sharded_dense": sharded, "sharded_backward": sharded_bwd,
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
            entry("C5_hausdorff_fwd", n, timeit(lambda: tpw.directed_hausdorff_distances(x1, x2)), "fp32_issue (point pairs)", n * 7, fp32_peak, 0)
    if want("C5_hausdorff_fwd_bwd"):
        def hd():
            x1.grad = None
            x2.grad = None
            tpw.directed_hausdorff_distances(x1, x2)[0].sum().backward()
        entry("C5_hausdorff_fwd_bwd", n, timeit(hd), "fp32_issue (point pairs)", n * 7, fp32_peak, 0)
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
    ap.add_argument("--no-configs", action="store_true",
                    help="skip the per-configuration entries and their CPU parity legs (headline, e2e and roofline only)")
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
