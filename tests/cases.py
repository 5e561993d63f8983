"""Seeded inputs and the metric table shared by the golden generator and the parity tests.

``call_metric(ns, ...)`` works on any namespace that exposes the reference's operator names:
``torch.ops.torchpairwise`` (the reference itself) or the ``torchpairwise_b200`` module.
"""
from __future__ import annotations

import math

import torch

FLOAT_CASES = [
    {"name": "f32_10x8x5", "dtype": torch.float32, "x1": (10, 5), "x2": (8, 5), "seed": 1},
    {"name": "f64_10x8x5", "dtype": torch.float64, "x1": (10, 5), "x2": (8, 5), "seed": 2},
    {"name": "f32_b2_6x5x6", "dtype": torch.float32, "x1": (2, 6, 6), "x2": (2, 5, 6), "seed": 3, "square": True},
    {"name": "f64_b2_6x5x6", "dtype": torch.float64, "x1": (2, 6, 6), "x2": (2, 5, 6), "seed": 4, "square": True},
    {"name": "f32_40x30x70", "dtype": torch.float32, "x1": (40, 70), "x2": (30, 70), "seed": 5},
    {"name": "f32_130x133x36", "dtype": torch.float32, "x1": (130, 36), "x2": (133, 36), "seed": 6, "stride": 3},
    {"name": "f32_b3_20x9x3", "dtype": torch.float32, "x1": (3, 20, 3), "x2": (3, 9, 3), "seed": 7},
    {"name": "f64_33x17x20", "dtype": torch.float64, "x1": (33, 20), "x2": (17, 20), "seed": 8},
]

FLOAT_METRICS = [
    {"name": "euclidean", "fn": "euclidean_distances"},
    {"name": "manhattan", "fn": "manhattan_distances"},
    {"name": "chebyshev", "fn": "chebyshev_distances"},
    {"name": "minkowski_p3", "fn": "minkowski_distances", "kw": {"p": 3.0}},
    {"name": "minkowski_p2.5", "fn": "minkowski_distances", "kw": {"p": 2.5}},
    {"name": "minkowski_p1.5", "fn": "minkowski_distances", "kw": {"p": 1.5}},
    {"name": "minkowski_p0.5", "fn": "minkowski_distances", "kw": {"p": 0.5}},
    {"name": "sqeuclidean", "fn": "sqeuclidean_distances"},
    {"name": "cosine_similarity", "fn": "cosine_similarity"},
    {"name": "cosine", "fn": "cosine_distances"},
    {"name": "correlation", "fn": "correlation_distances"},
    {"name": "linear_kernel", "fn": "linear_kernel"},
    {"name": "wminkowski_p3", "fn": "wminkowski_distances", "kw": {"p": 3.0}, "weighted": True, "needs_square": True},
    {"name": "wminkowski_p1", "fn": "wminkowski_distances", "kw": {"p": 1.0}, "weighted": True, "needs_square": True},
    {"name": "wminkowski_p2", "fn": "wminkowski_distances", "kw": {"p": 2.0}, "weighted": True, "needs_square": True},
    {"name": "wminkowski_p1.7", "fn": "wminkowski_distances", "kw": {"p": 1.7}, "weighted": True, "needs_square": True},
    {"name": "wminkowski_pinf", "fn": "wminkowski_distances", "kw": {"p": math.inf}, "weighted": True, "needs_square": True},
    {"name": "ppminkowski_p3", "fn": "_ppminkowski", "kw": {"p": 3.0}},
    {"name": "ppminkowski_p1", "fn": "_ppminkowski", "kw": {"p": 1.0}},
    {"name": "ppminkowski_p2.5", "fn": "_ppminkowski", "kw": {"p": 2.5}},
    {"name": "ppminkowski_pinf", "fn": "_ppminkowski", "kw": {"p": math.inf}},
    {"name": "ppminkowski_pneginf", "fn": "_ppminkowski", "kw": {"p": -math.inf}},
    {"name": "ppminkowski_p0", "fn": "_ppminkowski", "kw": {"p": 0.0}},
    {"name": "rbf_kernel", "fn": "rbf_kernel"},
    {"name": "rbf_kernel_g0.3", "fn": "rbf_kernel", "kw": {"gamma": 0.3}},
    {"name": "laplacian_kernel", "fn": "laplacian_kernel", "grad": False},  # the reference's own backward fails (in-place on cdist output)
    {"name": "polynomial_kernel", "fn": "polynomial_kernel", "kw": {"degree": 2, "gamma": 0.05, "coef0": 0.5}},
    {"name": "sigmoid_kernel", "fn": "sigmoid_kernel", "kw": {"gamma": 0.02, "coef0": 0.1}},
]


def call_metric(ns, metric, x1, x2, w=None):
    fn = getattr(ns, metric["fn"])
    kw = dict(metric.get("kw", {}))
    if metric.get("weighted"):
        kw["w"] = w
    return fn(x1, x2, **kw)


def float_inputs(case):
    g = torch.Generator().manual_seed(case["seed"])
    dt = case["dtype"]
    x1 = torch.randn(*case["x1"], generator=g, dtype=dt)
    x2 = torch.randn(*case["x2"], generator=g, dtype=dt)
    D = case["x1"][-1]
    wshape = (D,) if len(case["x1"]) == 2 else (case["x1"][0], D)
    w = torch.rand(*wshape, generator=g, dtype=dt) + 0.25
    gshape = case["x1"][:-1] + (case["x2"][-2],)
    grad = torch.randn(*gshape, generator=g, dtype=dt)
    return x1, x2, w, grad


BOOL_CASES = [
    {"name": "bool_10x8x37", "x1": (10, 37), "x2": (8, 37), "seed": 11, "kind": "bool", "p": 0.3},
    {"name": "bool_b2_9x6x70", "x1": (2, 9, 70), "x2": (2, 6, 70), "seed": 12, "kind": "bool", "p": 0.5},
    {"name": "bool_130x135x100", "x1": (130, 100), "x2": (135, 100), "seed": 13, "kind": "bool", "p": 0.1},
    {"name": "bool_20x12x1100", "x1": (20, 1100), "x2": (12, 1100), "seed": 14, "kind": "bool", "p": 0.1},
    {"name": "int64_10x8x5", "x1": (10, 5), "x2": (8, 5), "seed": 15, "kind": "int64"},
    {"name": "int32_b2_7x9x33", "x1": (2, 7, 33), "x2": (2, 9, 33), "seed": 16, "kind": "int32"},
    {"name": "f32_12x11x40", "x1": (12, 40), "x2": (11, 40), "seed": 17, "kind": "float32"},
    {"name": "f64_6x5x7", "x1": (6, 7), "x2": (5, 7), "seed": 18, "kind": "float64"},
    {"name": "uint8_9x4x19", "x1": (9, 19), "x2": (4, 19), "seed": 19, "kind": "uint8"},
]

# boolean metrics take any dtype (cast to bool with a warning); pw{and,or,xor}_sum are bool only
BOOL_METRICS = [
    "hamming_distances", "jaccard_distances", "kulsinski_distances", "kulczynski1_distances",
    "yule_distances", "dice_distances", "rogerstanimoto_distances", "russellrao_distances",
    "sokalmichener_distances", "sokalsneath_distances",
    "pwand_sum", "pwor_sum", "pwxor_sum", "pweq_sum", "pwne_sum", "pweq_mean", "pwne_mean",
]


def bool_inputs(case):
    g = torch.Generator().manual_seed(case["seed"])
    kind = case["kind"]
    if kind == "bool":
        x1 = torch.rand(*case["x1"], generator=g) < case["p"]
        x2 = torch.rand(*case["x2"], generator=g) < case["p"]
        # degenerate rows: all zeros and all ones, so that 0/0 branches are exercised
        x1[..., 0, :] = False
        x2[..., 0, :] = False
        x1[..., 1, :] = True
        x2[..., 1, :] = True
        return x1, x2
    x1 = torch.randint(0, 3, case["x1"], generator=g)
    x2 = torch.randint(0, 3, case["x2"], generator=g)
    dt = getattr(torch, kind)
    return x1.to(dt), x2.to(dt)


HAUSDORFF_CASES = [
    {"name": "hd_f32_b2", "dtype": torch.float32, "x1": (2, 3, 9, 3), "x2": (2, 2, 7, 3), "seed": 21},
    {"name": "hd_f64_b2", "dtype": torch.float64, "x1": (2, 3, 9, 3), "x2": (2, 2, 7, 3), "seed": 22},
    {"name": "hd_f32_unbatched", "dtype": torch.float32, "x1": (3, 9, 3), "x2": (2, 7, 3), "seed": 23},
    {"name": "hd_f32_d2", "dtype": torch.float32, "x1": (2, 50, 2), "x2": (3, 41, 2), "seed": 24},
    {"name": "hd_f32_d5", "dtype": torch.float32, "x1": (2, 30, 5), "x2": (2, 33, 5), "seed": 25},
    {"name": "hd_f32_big", "dtype": torch.float32, "x1": (1, 2, 1500, 3), "x2": (1, 2, 2300, 3), "seed": 26},
    {"name": "hd_f32_grid_ties", "dtype": torch.float32, "x1": (2, 40, 3), "x2": (2, 37, 3), "seed": 27, "grid": True},
]


def hausdorff_inputs(case):
    g = torch.Generator().manual_seed(case["seed"])
    dt = case["dtype"]
    if case.get("grid"):
        # small integer lattice: many exactly tied distances, exercising the tie rules
        x1 = torch.randint(0, 3, case["x1"], generator=g).to(dt)
        x2 = torch.randint(0, 3, case["x2"], generator=g).to(dt) + 0.5
    else:
        x1 = torch.rand(*case["x1"], generator=g, dtype=dt)
        x2 = torch.rand(*case["x2"], generator=g, dtype=dt)
    oshape = case["x1"][:-2] + (case["x2"][-3],)
    grad = torch.randn(*oshape, generator=g, dtype=dt)
    return x1, x2, grad


def config_inputs(name):
    """Row blocks of the five benchmark configurations (a row block of X against all of Y: C2 one batch and 512
    rows, C3 / C4 1024 rows; C1 and C5 whole), generated as the full configurations are (CPU generator, seed 0)
    so that CPU and GPU see identical bits."""
    g = torch.Generator().manual_seed(0)
    if name == "C1":
        return torch.randn(1024, 128, generator=g), torch.randn(2048, 128, generator=g)
    if name == "C2":
        X = torch.randn(1, 512, 256, generator=g)
        Y = torch.randn(1, 4096, 256, generator=g)
        G = torch.randn(1, 512, 4096, generator=g)
        return X, Y, G
    if name == "C3":
        return torch.rand(1024, 1024, generator=g) < 0.1, torch.rand(16384, 1024, generator=g) < 0.1
    if name == "C4":
        return torch.randn(1024, 512, generator=g), torch.randn(16384, 512, generator=g)
    if name == "C5":
        X = torch.rand(64, 8192, 3, generator=g) * 2 - 1
        Y = X + 0.05 * torch.randn(64, 8192, 3, generator=g)
        return X[:, None], Y[:, None]
    raise ValueError(name)


# float16 / bfloat16 inputs through the operators whose reference kernels accumulate in the narrow type itself
NARROW_CASES = [
    {"name": "f16_40x30x70", "dtype": torch.float16, "x1": (40, 70), "x2": (30, 70), "seed": 31},
    {"name": "bf16_40x30x70", "dtype": torch.bfloat16, "x1": (40, 70), "x2": (30, 70), "seed": 32},
    {"name": "f16_b2_33x17x260", "dtype": torch.float16, "x1": (2, 33, 260), "x2": (2, 17, 260), "seed": 33},
]
NARROW_METRICS = [
    {"name": "ppminkowski_p2", "fn": "_ppminkowski", "kw": {"p": 2.0}},
    {"name": "ppminkowski_p3", "fn": "_ppminkowski", "kw": {"p": 3.0}},
    {"name": "sqeuclidean", "fn": "sqeuclidean_distances"},
    {"name": "euclidean", "fn": "euclidean_distances"},
    {"name": "cosine", "fn": "cosine_distances"},
    {"name": "wminkowski_p2", "fn": "_wminkowski", "kw": {"p": 2.0}, "weighted": True},
]


def narrow_inputs(case):
    g = torch.Generator().manual_seed(case["seed"])
    dt = case["dtype"]
    x1 = torch.randn(*case["x1"], generator=g).to(dt)
    x2 = torch.randn(*case["x2"], generator=g).to(dt)
    w = (torch.rand(case["x1"][-1], generator=g) + 0.5).to(dt)
    if len(case["x1"]) == 3:
        w = w.expand(case["x1"][0], -1).contiguous()
    return x1, x2, w
