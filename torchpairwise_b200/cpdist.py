"""``cdist(x1, x2, metric=..., **kwargs)``: the string dispatcher of OPS/cpdist.cpp:149-231.

Same metric names, the same per-metric keyword validation (a keyword the metric does not take
raises ``TypeError`` naming it, OPS/cpdist.cpp:35-79), the same defaults (``p`` defaults to 2) and
the same quirk that ``metric="kulsinski"`` evaluates kulczynski1 (the inline helper at
OPS/pairwise_metrics.h:557-561 calls that functor).  Every metric name of the reference is served.
``pdist``, which the reference declares but does not implement
(OPS/cpdist.cpp:233-246), is the condensed form of ``cdist(x, x)``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor

from . import ops

SUPPORTED_METRICS = [
    "braycurtis", "canberra", "chebyshev", "cityblock", "correlation", "cosine",
    "dice", "directed_hausdorff", "euclidean", "hamming", "haversine", "jaccard",
    "jensenshannon", "kulczynski1", "kulsinski", "l1", "l2", "lp", "linf", "mahalanobis",
    "manhattan", "minkowski", "rogerstanimoto", "russellrao", "seuclidean", "snr",
    "sokalmichener", "sokalsneath", "sqeuclidean", "wminkowski", "yule",
]

# metric -> keyword arguments it accepts (DEFINE_CPDIST_METRIC_SPEC table, OPS/cpdist.cpp:82-147)
_ACCEPTS = {m: () for m in SUPPORTED_METRICS}
_ACCEPTS.update({
    "directed_hausdorff": ("shuffle", "generator"),
    "minkowski": ("p",), "lp": ("p",), "wminkowski": ("w", "p"),
    "seuclidean": ("V",), "mahalanobis": ("VI",), "jensenshannon": ("base",),
})

_SCHEMAS = {
    "minkowski": "(Tensor x1, Tensor? x2=None, float p=2) -> Tensor",
    "lp": "(Tensor x1, Tensor? x2=None, float p=2) -> Tensor",
    "wminkowski": "(Tensor x1, Tensor? x2=None, float p=2, Tensor? w=None) -> Tensor",
    "seuclidean": "(Tensor x1, Tensor? x2=None, Tensor? V=None) -> Tensor",
    "mahalanobis": "(Tensor x1, Tensor? x2=None, Tensor? VI=None) -> Tensor",
    "jensenshannon": "(Tensor x1, Tensor? x2=None, float? base=None) -> Tensor",
    "directed_hausdorff": "(Tensor x1, Tensor? x2=None, *, bool shuffle=False, Generator? generator=None) "
                          "-> (Tensor output, Tensor x1_indices, Tensor x2_indices)",
}

def _check_extra_args(metric: str, **given) -> None:
    bad = [k for k in ("w", "V", "VI", "p", "base", "shuffle", "generator")
           if given.get(k) is not None and k not in _ACCEPTS[metric]]
    if bad:
        schema = _SCHEMAS.get(metric, "(Tensor x1, Tensor? x2=None) -> Tensor")
        raise TypeError(
            f"{metric}_distances was called with incompatible arguments {', '.join(bad)}.\n"
            f"The following signature is supported:\n    torchpairwise::{metric}_distances{schema}\n"
        )


def cdist(x1: Tensor, x2: Tensor, metric: str = "minkowski", *, w: Optional[Tensor] = None,
          V: Optional[Tensor] = None, VI: Optional[Tensor] = None, p: Optional[float] = None,
          base: Optional[float] = None, shuffle: Optional[bool] = None, generator=None) -> Tensor:
    if metric not in SUPPORTED_METRICS:
        raise RuntimeError(f"Got unkown distance metric: {metric}. Supported metrics are [{', '.join(SUPPORTED_METRICS)}]")
    _check_extra_args(metric, w=w, V=V, VI=VI, p=p, base=base, shuffle=shuffle, generator=generator)
    if metric == "directed_hausdorff":
        return ops.directed_hausdorff_distances(x1, x2, shuffle=bool(shuffle) if shuffle is not None else False,
                                                generator=generator)[0]
    if metric in ("minkowski", "lp"):
        return ops.minkowski_distances(x1, x2, 2.0 if p is None else p)
    if metric == "wminkowski":
        return ops.wminkowski_distances(x1, x2, 2.0 if p is None else p, w)
    if metric == "seuclidean":
        return ops.seuclidean_distances(x1, x2, V)
    if metric == "mahalanobis":
        return ops.mahalanobis_distances(x1, x2, VI)
    if metric == "jensenshannon":
        return ops.jensenshannon_distances(x1, x2, base)
    if metric == "kulsinski":
        return ops.kulczynski1_distances(x1, x2)
    if metric == "cosine":
        return ops.cosine_distances(x1, x2)
    return getattr(ops, f"{metric}_distances")(x1, x2)


def pdist(input: Tensor, metric: str = "minkowski", *, w: Optional[Tensor] = None, V: Optional[Tensor] = None,
          VI: Optional[Tensor] = None, p: Optional[float] = None, base: Optional[float] = None,
          shuffle: Optional[bool] = None, generator=None) -> Tensor:
    """Condensed self-distances of ``input`` [N, D] (or [B, N, D]): the upper triangle of
    ``cdist(input, input, metric)`` row by row, shape [.., N (N - 1) / 2], the layout of ``torch.pdist``
    and ``scipy.spatial.distance.pdist``.

    The reference declares this function with the arguments of ``cdist`` and raises "pdist is yet to be
    implemented" (OPS/cpdist.cpp:233-246); its README defines it as ``cdist(x1, x1)`` without the
    duplicated positions.  The L_p metrics run the tile kernel with a condensed epilogue that skips the
    tiles on or below the diagonal (about half of the pairs are evaluated) when no gradient is needed;
    everything else, and every differentiable call, evaluates ``cdist`` and gathers the triangle."""
    from .ops import _FLOAT_CODES, _ROWMIN_METRICS, _abi, _ptr, _require_cuda, _stream, check, lib  # noqa: F401
    if metric not in SUPPORTED_METRICS:
        raise RuntimeError(f"Got unkown distance metric: {metric}. Supported metrics are [{', '.join(SUPPORTED_METRICS)}]")
    _check_extra_args(metric, w=w, V=V, VI=VI, p=p, base=base, shuffle=shuffle, generator=generator)
    if input.dim() not in (2, 3):
        raise RuntimeError("input must be 2D tensor (unbatched) or 3D tensor (batched)")
    _require_cuda(input)
    n = input.size(-2)
    fused = (metric in _ROWMIN_METRICS and w is None and input.dtype in _FLOAT_CODES and input.size(-1) > 0
             and not (input.requires_grad and torch.is_grad_enabled()))
    if fused:
        pp, ex = _ROWMIN_METRICS[metric]
        if pp is None:
            pp = 2.0 if p is None else float(p)
            ex = 1.0 if math.isinf(pp) else (1.0 / pp if pp > 0 else None)
        if ex is not None:
            xc = input.contiguous()
            xb = xc if xc.dim() == 3 else xc.unsqueeze(0)
            out = torch.empty((xb.size(0), n * (n - 1) // 2), dtype=xb.dtype, device=xb.device)
            with torch.cuda.device(xb.device):
                check(lib.tpw_lp_pdist_forward(_FLOAT_CODES[xb.dtype], _ptr(xb), _ptr(out), xb.size(0), n, xb.size(2),
                                               pp, ex, _stream(xb)), "tpw_lp_pdist_forward")
            return out if input.dim() == 3 else out.squeeze(0)
    full = cdist(input, input, metric, w=w, V=V, VI=VI, p=p, base=base, shuffle=shuffle, generator=generator)
    iu = torch.triu_indices(n, n, offset=1, device=input.device)
    return full[..., iu[0], iu[1]]
