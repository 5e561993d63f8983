"""Generates the golden vectors under tests/golden/ from the reference itself.

Needs ``oracle/_ref/torchpairwise_ref.so`` (``make -C oracle``: the unmodified CPU operators of
inspiros/torchpairwise v0.3.0 compiled from its own sources).  Every vector is the output of
``torch.ops.torchpairwise.*`` on CPU for small seeded inputs; inputs are stored next to outputs,
except for the config-shaped cases whose inputs are regenerated from the seed (their float64
checksum is stored so that a generator drift is detected rather than mis-reported as a parity
failure).

    python tests/golden/make_golden.py            # everything
    python tests/golden/make_golden.py composed   # one file
"""
from __future__ import annotations

import math
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(HERE.parent))
from cases import (BOOL_METRICS, FLOAT_CASES, FLOAT_METRICS, HAUSDORFF_CASES, NARROW_CASES, NARROW_METRICS, config_inputs,  # noqa: E402
                   float_inputs, bool_inputs, hausdorff_inputs, narrow_inputs, BOOL_CASES, call_metric)

torch.ops.load_library(str(ROOT / "oracle" / "_ref" / "torchpairwise_ref.so"))
T = torch.ops.torchpairwise


def npy(t):
    return t.detach().cpu().numpy()


def float_golden():
    out = {}
    for case in FLOAT_CASES:
        x1, x2, w, g = float_inputs(case)
        out[f"{case['name']}/x1"], out[f"{case['name']}/x2"] = npy(x1), npy(x2)
        out[f"{case['name']}/w"], out[f"{case['name']}/g"] = npy(w), npy(g)
        for metric in FLOAT_METRICS:
            if metric.get("needs_square") and not case.get("square", False) and x1.dim() == 3:
                continue  # the reference's batched weighted check only passes when N1 == D
            a = x1.clone().requires_grad_(True)
            b = x2.clone().requires_grad_(True)
            ww = w.clone().requires_grad_(True)
            res = call_metric(T, metric, a, b, ww)
            key = f"{case['name']}/{metric['name']}"
            st = case.get("stride", 1)  # large outputs are stored sub-sampled
            out[key + "/out"] = npy(res[..., ::st, ::st])
            if metric.get("grad", True):
                res.backward(g)
                out[key + "/gx1"], out[key + "/gx2"] = npy(a.grad), npy(b.grad)
                if metric.get("weighted"):
                    out[key + "/gw"] = npy(ww.grad)
    np.savez_compressed(HERE / "float_metrics.npz", **out)
    print("float_metrics.npz", len(out), "arrays")


def bool_golden():
    out = {}
    for case in BOOL_CASES:
        x1, x2 = bool_inputs(case)
        out[f"{case['name']}/x1"], out[f"{case['name']}/x2"] = npy(x1), npy(x2)
        for name in BOOL_METRICS:
            fn = getattr(T, name)
            if name.startswith("pw") and name[2:5] in ("and", "or_", "xor") and x1.dtype != torch.bool:
                continue
            with torch.no_grad():
                import warnings
                with warnings.catch_warnings():
                    warnings.simplefilter("ignore")
                    res = fn(x1, x2)
            out[f"{case['name']}/{name}"] = npy(res)
    np.savez_compressed(HERE / "bool_metrics.npz", **out)
    print("bool_metrics.npz", len(out), "arrays")


def hausdorff_golden():
    out = {}
    for case in HAUSDORFF_CASES:
        x1, x2, g = hausdorff_inputs(case)
        a = x1.clone().requires_grad_(True)
        b = x2.clone().requires_grad_(True)
        res, i1, i2 = T.directed_hausdorff_distances(a, b, shuffle=False)
        res.backward(g)
        n = case["name"]
        out[f"{n}/x1"], out[f"{n}/x2"], out[f"{n}/g"] = npy(x1), npy(x2), npy(g)
        out[f"{n}/out"], out[f"{n}/idx1"], out[f"{n}/idx2"] = npy(res), npy(i1), npy(i2)
        out[f"{n}/gx1"], out[f"{n}/gx2"] = npy(a.grad), npy(b.grad)
    np.savez_compressed(HERE / "hausdorff.npz", **out)
    print("hausdorff.npz", len(out), "arrays")


def config_golden():
    out = {}
    # C1: X[1024,128], Y[2048,128] fp32, rows ::128 of the output
    X, Y = config_inputs("C1")
    out["C1/checksum"] = np.array([X.double().sum().item(), Y.double().sum().item()])
    for name in ("euclidean_distances", "manhattan_distances", "cosine_distances", "chebyshev_distances",
                 "sqeuclidean_distances", "correlation_distances"):
        out[f"C1/{name}"] = npy(getattr(T, name)(X, Y)[::128])
    # C2: batch 0, rows 0:512 against all 4096 columns: minkowski p=3 and chebyshev, forward + backward (sub-sampled)
    X, Y, G = config_inputs("C2")
    out["C2/checksum"] = np.array([X.double().sum().item(), Y.double().sum().item(), G.double().sum().item()])
    for name, fn in (("minkowski3", lambda a, b: T.minkowski_distances(a, b, 3.0)),
                     ("chebyshev", lambda a, b: T.chebyshev_distances(a, b))):
        a = X.clone().requires_grad_(True)
        b = Y.clone().requires_grad_(True)
        res = fn(a, b)
        res.backward(G)
        out[f"C2/{name}/out"] = npy(res[:, ::8, ::16])
        out[f"C2/{name}/gx1"] = npy(a.grad[:, ::8])
        out[f"C2/{name}/gx2"] = npy(b.grad[:, ::16])
    # C3: bool X rows 0:1024 against all 16384 rows of Y (sub-sampled)
    X, Y = config_inputs("C3")
    out["C3/checksum"] = np.array([X.double().sum().item(), Y.double().sum().item()])
    out["C3/hamming_distances"] = npy(T.hamming_distances(X, Y)[::16, ::64])
    out["C3/jaccard_distances"] = npy(T.jaccard_distances(X, Y)[::16, ::64])
    # C4: X rows 0:1024 against all 16384 rows of Y (sub-sampled)
    X, Y = config_inputs("C4")
    out["C4/checksum"] = np.array([X.double().sum().item(), Y.double().sum().item()])
    out["C4/sqeuclidean_distances"] = npy(T.sqeuclidean_distances(X, Y)[::16, ::64])
    out["C4/cosine_distances"] = npy(T.cosine_distances(X, Y)[::16, ::64])
    # C5 whole: x1, x2 [64,1,8192,3]
    X, Y = config_inputs("C5")
    out["C5/checksum"] = np.array([X.double().sum().item(), Y.double().sum().item()])
    a = X.clone().requires_grad_(True)
    b = Y.clone().requires_grad_(True)
    res, i1, i2 = T.directed_hausdorff_distances(a, b, shuffle=False)
    res.backward(torch.ones_like(res))
    out["C5/out"], out["C5/idx1"], out["C5/idx2"] = npy(res), npy(i1), npy(i2)
    rows1 = a.grad.abs().sum(-1).nonzero()
    rows2 = b.grad.abs().sum(-1).nonzero()
    out["C5/gx1_rows"], out["C5/gx1_vals"] = npy(rows1), npy(a.grad[tuple(rows1.t())])
    out["C5/gx2_rows"], out["C5/gx2_vals"] = npy(rows2), npy(b.grad[tuple(rows2.t())])
    np.savez_compressed(HERE / "configs.npz", **out)
    print("configs.npz", len(out), "arrays")


def extras_golden():
    """seuclidean and the neighbour masks (callers of the path), small unbatched inputs."""
    out = {}
    g = torch.Generator().manual_seed(41)
    x1, x2 = torch.randn(14, 6, generator=g), torch.randn(9, 6, generator=g)
    V = torch.rand(6, generator=g) + 0.2
    up1, up2 = torch.randn(14, 14, generator=g), torch.randn(14, 9, generator=g)
    out["x1"], out["x2"], out["V"], out["up1"], out["up2"] = npy(x1), npy(x2), npy(V), npy(up1), npy(up2)
    a = x1.clone().requires_grad_(True)
    r = T.seuclidean_distances(a, None, V)  # V=None trips a dangling IntArrayRef in the reference (OPS/pairwise_metrics.cpp:259)
    r.backward(up1)
    out["seuclidean_self/out"], out["seuclidean_self/gx1"] = npy(r), npy(a.grad)
    a, b = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True)
    r = T.seuclidean_distances(a, b, V)
    r.backward(up2)
    out["seuclidean/out"], out["seuclidean/gx1"], out["seuclidean/gx2"] = npy(r), npy(a.grad), npy(b.grad)
    out["cdist_seuclidean"] = npy(T.cdist(x1, x2, "seuclidean", V=V))
    out["k_neighbors_k3"] = npy(T.k_neighbors_mask(x1, x2, 3))
    out["k_neighbors_self_k2_manhattan"] = npy(T.k_neighbors_mask(x1, None, 2, "manhattan"))
    out["radius_2.5"] = npy(T.radius_neighbors_mask(x1, x2, 2.5))
    out["radius_self_3_minkowski3"] = npy(T.radius_neighbors_mask(x1, None, 3.0, "minkowski", p=3.0))
    np.savez_compressed(HERE / "extras.npz", **out)
    print("extras.npz", len(out), "arrays")


def composed_golden():
    """braycurtis, snr and mahalanobis: reference kernels of their own (OPS/cpu/braycurtis_kernel.cpp,
    snr_kernel.cpp, sqmahalanobis_kernel.cpp) that the B200 build states as compositions of the
    path's kernels.  Unbatched and batched inputs, float32 and float64, forward and gradients."""
    out = {}
    g = torch.Generator().manual_seed(57)
    for tag, s1, s2, dt in (("u32", (14, 6), (9, 6), torch.float32), ("b64", (2, 7, 5), (2, 8, 5), torch.float64)):
        x1, x2 = torch.randn(*s1, generator=g, dtype=dt), torch.randn(*s2, generator=g, dtype=dt)
        d = s1[-1]
        A = torch.randn(*s1[:-2], d, d, generator=g, dtype=dt)
        VI = A @ A.transpose(-1, -2) / d + 0.5 * torch.eye(d, dtype=dt) + 0.1 * torch.randn(*s1[:-2], d, d, generator=g, dtype=dt)
        up = torch.randn(*s1[:-1], s2[-2], generator=g, dtype=dt)
        ups = torch.randn(*s1[:-1], s1[-2], generator=g, dtype=dt)
        out[f"{tag}/x1"], out[f"{tag}/x2"], out[f"{tag}/VI"], out[f"{tag}/up"], out[f"{tag}/ups"] = npy(x1), npy(x2), npy(VI), npy(up), npy(ups)
        for name in ("braycurtis_distances", "snr_distances"):
            a, b = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True)
            r = getattr(T, name)(a, b)
            r.backward(up)
            out[f"{tag}/{name}/out"], out[f"{tag}/{name}/gx1"], out[f"{tag}/{name}/gx2"] = npy(r), npy(a.grad), npy(b.grad)
            a = x1.clone().requires_grad_(True)
            r = getattr(T, name)(a, None)
            out[f"{tag}/{name}/self_out"] = npy(r)
        a, b, v = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True), VI.clone().requires_grad_(True)
        r = T.mahalanobis_distances(a, b, v)
        r.backward(up)
        out[f"{tag}/mahalanobis_distances/out"] = npy(r)
        out[f"{tag}/mahalanobis_distances/gx1"], out[f"{tag}/mahalanobis_distances/gx2"] = npy(a.grad), npy(b.grad)
        out[f"{tag}/mahalanobis_distances/gVI"] = npy(v.grad)
        if len(s1) == 2:
            out[f"{tag}/cdist_braycurtis"] = npy(T.cdist(x1, x2, "braycurtis"))
            out[f"{tag}/cdist_snr"] = npy(T.cdist(x1, x2, "snr"))
            out[f"{tag}/cdist_mahalanobis"] = npy(T.cdist(x1, x2, "mahalanobis", VI=VI))
            big = torch.randn(40, 6, generator=g, dtype=dt)
            out[f"{tag}/big"] = npy(big)
            out[f"{tag}/mahalanobis_default_VI"] = npy(T.mahalanobis_distances(big, None, None))
    np.savez_compressed(HERE / "composed.npz", **out)
    print("composed.npz", len(out), "arrays")


def pair_sums_golden():
    """canberra and the chi-squared kernels: sums of two-argument terms with reference kernels of their
    own (OPS/cpu/canberra_kernel.cpp, additive_chi2_kernel.cpp).  Mixed-sign inputs for canberra,
    non-negative histograms (with exact zeros, so that skipped terms occur) for chi2."""
    out = {}
    g = torch.Generator().manual_seed(63)
    for tag, s1, s2, dt in (("u32", (33, 19), (21, 19), torch.float32), ("b64", (2, 9, 7), (2, 6, 7), torch.float64),
                            ("w32", (140, 70), (131, 70), torch.float32)):
        x1, x2 = torch.randn(*s1, generator=g, dtype=dt), torch.randn(*s2, generator=g, dtype=dt)
        h1, h2 = torch.rand(*s1, generator=g, dtype=dt), torch.rand(*s2, generator=g, dtype=dt)
        h1[..., 0, :3] = 0
        h2[..., 1, :4] = 0
        up = torch.randn(*s1[:-1], s2[-2], generator=g, dtype=dt)
        for k, v in (("x1", x1), ("x2", x2), ("h1", h1), ("h2", h2), ("up", up)):
            out[f"{tag}/{k}"] = npy(v)
        for name, a0, b0, kw in (("canberra_distances", x1, x2, {}), ("additive_chi2_kernel", h1, h2, {}),
                                 ("chi2_kernel", h1, h2, {"gamma": 0.7})):
            a, b = a0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
            r = getattr(T, name)(a, b, **kw)
            r.backward(up)
            out[f"{tag}/{name}/out"], out[f"{tag}/{name}/gx1"], out[f"{tag}/{name}/gx2"] = npy(r), npy(a.grad), npy(b.grad)
            out[f"{tag}/{name}/self_out"] = npy(getattr(T, name)(a0, None, **kw))
        if len(s1) == 2:
            out[f"{tag}/cdist_canberra"] = npy(T.cdist(x1, x2, "canberra"))
    np.savez_compressed(HERE / "pair_sums.npz", **out)
    print("pair_sums.npz", len(out), "arrays")


def jensenshannon_golden():
    """jensenshannon_distances and _sqjensenshannon (OPS/cpu/sqjensenshannon_kernel.cpp): non-negative
    histograms with exact zeros (terms that vanish on one or both sides), with and without a base."""
    out = {}
    g = torch.Generator().manual_seed(64)
    for tag, s1, s2, dt in (("u32", (33, 19), (21, 19), torch.float32), ("b64", (2, 9, 7), (2, 6, 7), torch.float64),
                            ("w32", (140, 70), (131, 70), torch.float32)):
        h1, h2 = torch.rand(*s1, generator=g, dtype=dt), torch.rand(*s2, generator=g, dtype=dt)
        h1[..., 0, :3] = 0
        h2[..., 1, :4] = 0
        h2[..., 2, 2:9] = 0
        up = torch.randn(*s1[:-1], s2[-2], generator=g, dtype=dt)
        for k, v in (("h1", h1), ("h2", h2), ("up", up)):
            out[f"{tag}/{k}"] = npy(v)
        for name, base in (("nat", None), ("base2", 2.0)):
            a, b = h1.clone().requires_grad_(True), h2.clone().requires_grad_(True)
            r = T.jensenshannon_distances(a, b, base)
            r.backward(up)
            out[f"{tag}/{name}/out"], out[f"{tag}/{name}/gx1"], out[f"{tag}/{name}/gx2"] = npy(r), npy(a.grad), npy(b.grad)
            n1, n2 = h1 / h1.sum(-1, keepdim=True), h2 / h2.sum(-1, keepdim=True)
            a, b = n1.clone().requires_grad_(True), n2.clone().requires_grad_(True)
            r = T._sqjensenshannon(a, b, base)
            r.backward(up)
            out[f"{tag}/{name}/sq_out"], out[f"{tag}/{name}/sq_gx1"], out[f"{tag}/{name}/sq_gx2"] = npy(r), npy(a.grad), npy(b.grad)
        out[f"{tag}/self_out"] = npy(T.jensenshannon_distances(h1, None, None))
        if len(s1) == 2:
            out[f"{tag}/cdist_base3"] = npy(T.cdist(h1, h2, "jensenshannon", base=3.0))
    np.savez_compressed(HERE / "jensenshannon.npz", **out)
    print("jensenshannon.npz", len(out), "arrays")


def haversine_golden():
    """haversine_distances (OPS/cpu/haversine_kernel.cpp): latitudes in [-pi/2, pi/2], longitudes in [-pi, pi]."""
    out = {}
    g = torch.Generator().manual_seed(65)
    for tag, s1, s2, dt in (("u32", (37, 2), (23, 2), torch.float32), ("b64", (2, 9, 2), (2, 6, 2), torch.float64),
                            ("w32", (150, 2), (261, 2), torch.float32)):
        scale = torch.tensor([math.pi, 2 * math.pi], dtype=dt)
        x1 = (torch.rand(*s1, generator=g, dtype=dt) - 0.5) * scale
        x2 = (torch.rand(*s2, generator=g, dtype=dt) - 0.5) * scale
        up = torch.randn(*s1[:-1], s2[-2], generator=g, dtype=dt)
        for k, v in (("x1", x1), ("x2", x2), ("up", up)):
            out[f"{tag}/{k}"] = npy(v)
        a, b = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True)
        r = T.haversine_distances(a, b)
        r.backward(up)
        out[f"{tag}/out"], out[f"{tag}/gx1"], out[f"{tag}/gx2"] = npy(r), npy(a.grad), npy(b.grad)
        out[f"{tag}/self_out"] = npy(T.haversine_distances(x1, None))
        if tag == "u32":
            out[f"{tag}/cdist"] = npy(T.cdist(x1, x2, "haversine"))
    np.savez_compressed(HERE / "haversine.npz", **out)
    print("haversine.npz", len(out), "arrays")


def narrow_golden():
    """float16 / bfloat16 inputs: the reference's own result (its kernels accumulate in the narrow type) and the same
    operator evaluated in float64 on the same narrow inputs, so that a test can place another implementation between them."""
    out = {}
    for case in NARROW_CASES:
        x1, x2, w = narrow_inputs(case)
        n = case["name"]
        out[f"{n}/x1"], out[f"{n}/x2"], out[f"{n}/w"] = npy(x1.float()), npy(x2.float()), npy(w.float())
        for metric in NARROW_METRICS:
            if metric.get("weighted") and x1.dim() == 3:
                continue  # the reference rejects batched weights unless N1 == D (its shape check compares the wrong axis)
            out[f"{n}/{metric['name']}/ref"] = npy(call_metric(T, metric, x1, x2, w if metric.get("weighted") else None).float())
            out[f"{n}/{metric['name']}/f64"] = npy(call_metric(T, metric, x1.double(), x2.double(), w.double() if metric.get("weighted") else None))
    p, q, _ = hausdorff_inputs({"seed": 34, "dtype": torch.float32, "x1": (2, 2, 60, 3), "x2": (2, 3, 45, 3)})
    p, q = p.half(), q.half()
    r = T.directed_hausdorff_distances(p, q)
    out["hd_f16/x1"], out["hd_f16/x2"] = npy(p.float()), npy(q.float())
    out["hd_f16/ref"] = npy(r[0].float())
    out["hd_f16/f64"] = npy(T.directed_hausdorff_distances(p.double(), q.double())[0])
    np.savez_compressed(HERE / "narrow.npz", **out)
    print("narrow.npz", len(out), "arrays")


if __name__ == "__main__":
    torch.set_num_threads(8)
    which = set(sys.argv[1:])
    for name, fn in (("float", float_golden), ("bool", bool_golden), ("hausdorff", hausdorff_golden), ("configs", config_golden),
                     ("extras", extras_golden), ("composed", composed_golden), ("pair_sums", pair_sums_golden),
                     ("jensenshannon", jensenshannon_golden), ("haversine", haversine_golden), ("narrow", narrow_golden)):
        if not which or name in which:
            fn()
