"""Forward + backward of a batched pairwise metric whose operands live in pinned host memory.

A [B, N1, N2] upstream gradient is usually far larger than the operands (C2: 1.07 GB against
2 x 16.8 MB), so a step that starts from host buffers is bound by the host-to-device copy unless
the copy of batch chunk c+1 runs while chunk c computes.  ``forward_backward_from_host`` does
exactly that with three streams (copy-in, compute, copy-out); batches are independent, so the
results are identical to one call on the whole batch.  The reference has no such helper (it is
single-stream throughout); this is an addition for callers that feed the GPU from the host.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
from torch import Tensor


_streams = {}


def _side_streams(dev: torch.device):
    """One copy-in and one copy-out stream per device, created once: the caching allocator keeps
    a pool per stream, so fresh streams on every call would mean fresh cudaMallocs on every call."""
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    if key not in _streams:
        _streams[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _streams[key]


def forward_backward_from_host(metric: Callable[..., Tensor], x1_host: Tensor, x2_host: Tensor, grad_host: Tensor,
                               grad_x1_host: Tensor, grad_x2_host: Tensor, device, *, chunk: int = 2,
                               out_host: Optional[Tensor] = None, **kwargs) -> None:
    """``metric(x1, x2, **kwargs).backward(grad)`` batch chunk by batch chunk.

    All tensors are batched ([B, N, D] / [B, N1, N2]) and should be pinned.  Gradients are
    written into ``grad_x1_host`` / ``grad_x2_host`` (and the distances into ``out_host`` when
    given).  Returns after every device-to-host copy has completed."""
    dev = torch.device(device)
    B = x1_host.size(0)
    compute = torch.cuda.current_stream(dev)
    copy_in, copy_out = _side_streams(dev)
    copy_in.wait_stream(compute)
    bounds = [(lo, min(B, lo + chunk)) for lo in range(0, B, chunk)]
    # Copy-in stream: all operand chunks first (small), then the gradient chunks (large), in order.
    xs, ys, gs, x_ready, g_ready = [], [], [], [], []
    with torch.cuda.stream(copy_in):
        for lo, hi in bounds:
            xs.append(x1_host[lo:hi].to(dev, non_blocking=True))
            ys.append(x2_host[lo:hi].to(dev, non_blocking=True))
            ev = torch.cuda.Event()
            ev.record(copy_in)
            x_ready.append(ev)
        for lo, hi in bounds:
            gs.append(grad_host[lo:hi].to(dev, non_blocking=True))
            ev = torch.cuda.Event()
            ev.record(copy_in)
            g_ready.append(ev)
    # Compute stream: every forward needs only its operands, so all forwards run while the gradient is
    # still crossing the bus; each backward starts as soon as its gradient chunk has landed.
    outs = []
    for c in range(len(bounds)):
        compute.wait_event(x_ready[c])
        xs[c].requires_grad_(True)
        ys[c].requires_grad_(True)
        outs.append(metric(xs[c], ys[c], **kwargs))
    for c, (lo, hi) in enumerate(bounds):
        compute.wait_event(g_ready[c])
        outs[c].backward(gs[c])
        done = torch.cuda.Event()
        done.record(compute)
        copy_out.wait_event(done)
        with torch.cuda.stream(copy_out):
            grad_x1_host[lo:hi].copy_(xs[c].grad, non_blocking=True)
            grad_x2_host[lo:hi].copy_(ys[c].grad, non_blocking=True)
            if out_host is not None:
                out_host[lo:hi].copy_(outs[c].detach(), non_blocking=True)
    # the device tensors stay referenced until every stream that touched them has drained
    copy_out.synchronize()
    compute.synchronize()
    del xs, ys, gs, outs
