"""Row-sharded pairwise distances over the GPUs of one box (one process per GPU).

Every output row ``(b, i, :)`` depends on one row of ``x1`` and all of ``x2``, so the path shards
without any exchange in the data path: ``x1`` is split into contiguous row blocks (batches first
when there are at least as many batches as ranks), ``x2`` is broadcast once from its owner over
NCCL/NVLink into each GPU's own memory, and every rank keeps its output slab.  The only collective
that follows a kernel is the sum of the ``x2`` gradients in the backward pass.  The reference has
no multi-device code at all; this module is an addition around its operators.

The collectives go through ``torch.distributed`` (NCCL on GPUs; the same code runs on gloo for
CPU tests of the partitioning and the gradient reduction).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def split_range(n: int, parts: int) -> List[Tuple[int, int]]:
    """``parts`` contiguous half-open ranges covering ``[0, n)``; the first ``n % parts`` ranges
    are one element longer, trailing ranges may be empty when ``n < parts``."""
    if parts <= 0:
        raise ValueError("parts must be positive")
    base, extra = divmod(max(n, 0), parts)
    out, start = [], 0
    for r in range(parts):
        size = base + (1 if r < extra else 0)
        out.append((start, start + size))
        start += size
    return out


def plan_shards(x1_shape: Tuple[int, ...], world_size: int) -> Tuple[str, List[Tuple[int, int]]]:
    """How ``x1`` ([N1, D] or [B, N1, D]) is cut: ``("batch", ranges)`` when it is batched with at
    least ``world_size`` batches (then ``x2`` is cut the same way and nothing is exchanged),
    otherwise ``("rows", ranges)`` over N1 with ``x2`` replicated."""
    if len(x1_shape) == 3 and x1_shape[0] >= world_size:
        return "batch", split_range(x1_shape[0], world_size)
    rows_dim = 0 if len(x1_shape) == 2 else 1
    return "rows", split_range(x1_shape[rows_dim], world_size)


def local_block(x: Tensor, kind: str, ranges: List[Tuple[int, int]], rank: int, *, is_x2: bool = False) -> Tensor:
    """The slice of ``x`` that ``rank`` works on under ``plan_shards``' plan."""
    lo, hi = ranges[rank]
    if kind == "batch":
        return x[lo:hi]
    if is_x2:
        return x
    return x[lo:hi] if x.dim() == 2 else x[:, lo:hi]


class _ReplicateFromOwner(torch.autograd.Function):
    """Forward: broadcast ``x2`` from ``src`` (every rank passes a buffer of the right shape).
    Backward: all-reduce (sum) of the per-rank partial gradients, so each rank ends up with the
    gradient of the whole job with respect to ``x2``."""

    @staticmethod
    def forward(ctx, x2: Tensor, src: int, group):
        ctx.group = group
        out = x2.detach().clone() if x2.requires_grad else x2.detach()
        dist.broadcast(out, src=src, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        g = grad.contiguous().clone()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None, None


def replicate_x2(x2: Tensor, src: int = 0, group=None) -> Tensor:
    """Broadcast ``x2`` from rank ``src`` into this rank's own memory (differentiable)."""
    return _ReplicateFromOwner.apply(x2, src, group)


def sharded_pairwise(metric: Callable[..., Tensor], x1_local: Tensor, x2: Tensor, *, src: int = 0, group=None,
                     replicate: bool = True, **kwargs) -> Tensor:
    """Distances of this rank's ``x1`` block against all of ``x2``.

    ``metric`` is any pairwise operator of this package (or ``cdist`` with ``metric=...`` in
    ``kwargs``).  With ``replicate=True`` ``x2`` is first broadcast from ``src``; pass ``False``
    when the plan was ``"batch"`` (each rank already holds its own ``x2`` batches).  The result is
    this rank's output slab; slabs are never gathered."""
    if replicate and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        x2 = replicate_x2(x2, src, group)
    return metric(x1_local, x2, **kwargs)


def sharded_pairwise_panels(metric: Callable[..., Tensor], x1_local: Tensor, x2: Tensor, *, src: int = 0, group=None,
                            panels: int = 2, **kwargs) -> List[Tensor]:
    """Distances of this rank's ``x1`` block against all of ``x2``, as ``panels`` column panels
    ``[.., N1_local, N2 / panels]`` (``torch.cat(result, -1)`` is the slab ``sharded_pairwise`` returns).

    ``x2`` (unbatched, ``[N2, D]``, the owner's values on ``src`` and a buffer of the same shape elsewhere) is
    broadcast in ``panels`` row chunks that are all queued at once; the operator runs on chunk c as soon as it
    has landed, while chunk c + 1 is still crossing NVLink, so all but the first chunk of the broadcast hides
    behind the kernels.  Each panel is a dense matrix of its own: the operator is called as it is, with a
    contiguous block of ``x2`` rows.  Forward only (no gradient flows back through the broadcast); ``x2`` holds the
    broadcast values on every rank afterwards."""
    if x2.dim() != 2 or not x2.is_contiguous():
        raise ValueError("sharded_pairwise_panels takes an unbatched, contiguous x2 [N2, D]")
    bounds = [b for b in split_range(x2.size(0), max(1, panels)) if b[1] > b[0]]
    live = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    works = [dist.broadcast(x2[lo:hi], src=src, group=group, async_op=True) for lo, hi in bounds] if live else []
    outs = []
    with torch.no_grad():
        for c, (lo, hi) in enumerate(bounds):
            if live:
                works[c].wait()
            outs.append(metric(x1_local, x2[lo:hi], **kwargs))
    return outs
