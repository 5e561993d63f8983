"""Host side of the pairwise path: the reference's operator surface on top of the C ABI.

Names, argument meaning, defaults and error behaviour follow inspiros/torchpairwise v0.3.0
(OPS = torchpairwise/csrc/ops): the public metric functions of OPS/pairwise_metrics.cpp, the
internal ops they are built from (``_ppminkowski``, ``_wminkowski``, ``_directed_hausdorff``,
``pw*_sum`` / ``pw*_mean``, ``prf_div``) and their hand-derived backward passes.  Every function
here takes CUDA tensors and launches the sm_100a kernels of ``libtpw_b200.so`` on the current
stream; nothing falls back to the CPU or to eager PyTorch arithmetic on the [N1, N2] matrix.
"""
from __future__ import annotations

import math
import os
import warnings
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _abi
from ._abi import check, lib

_FLOAT_CODES = {torch.float32: _abi.F32, torch.float64: _abi.F64}

_ENGINE_NAMES = {"auto": _abi.ENGINE_AUTO, "simt": _abi.ENGINE_SIMT_FP32, "tcgen05": _abi.ENGINE_TCGEN05_BF16X3}
_dot_engine = _ENGINE_NAMES.get(os.environ.get("TPW_DOT_ENGINE", "auto").lower(), _abi.ENGINE_AUTO)


def set_dot_engine(name: str) -> None:
    """Engine of the dense-contraction metrics (sqeuclidean, euclidean, cosine, correlation,
    linear kernel) for float32 inputs: "auto" (tensor cores for large problems, CUDA cores
    otherwise), "simt" (always the exact fp32 CUDA-core tile) or "tcgen05" (always the bf16x3
    tensor-core kernel).  float64 always runs on the CUDA cores.  Also settable through the
    environment variable TPW_DOT_ENGINE."""
    global _dot_engine
    if name not in _ENGINE_NAMES:
        raise ValueError(f"engine must be one of {sorted(_ENGINE_NAMES)}")
    _dot_engine = _ENGINE_NAMES[name]


def get_dot_engine() -> str:
    return {v: k for k, v in _ENGINE_NAMES.items()}[_dot_engine]


def _tensor_engine_selected(x1c: Tensor, x2c: Tensor) -> bool:
    """True when the current engine setting sends this float32 problem to the tensor cores."""
    if x1c.dtype != torch.float32 or x1c.size(2) == 0:
        return False
    B, N1, N2, D = x1c.size(0), x1c.size(1), x2c.size(1), x1c.size(2)
    return lib.tpw_dot_metric_scratch_bytes(_abi.F32, _dot_engine, B, N1, N2, D) > 0


# --------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------
def _ptr(t: Optional[Tensor]):
    return None if t is None else t.data_ptr()


def _stream(t: Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*tensors: Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "torchpairwise_b200 runs on CUDA tensors only (no CPU path); got a tensor on "
                f"{t.device}"
            )
    devs = {t.device for t in tensors if t is not None}
    if len(devs) > 1:
        raise RuntimeError(f"Expected all tensors to be on the same device, got {sorted(map(str, devs))}")


def _compute_dtype(dtype: torch.dtype) -> torch.dtype:
    """Half and bfloat16 inputs are computed in float32 and rounded once on the way out."""
    if dtype in (torch.float16, torch.bfloat16):
        return torch.float32
    if dtype in _FLOAT_CODES:
        return dtype
    raise RuntimeError(f"expected a floating point tensor, got {dtype}")


def check_pairwise_inputs(name: str, x1: Tensor, x2: Optional[Tensor] = None, *, boolean: bool = False,
                          sets: bool = False) -> Tuple[Tensor, Tensor]:
    """Rank / feature checks of OPS/pairwise_metrics.h:10-67 (same messages)."""
    lo = 3 if sets else 2
    unbatched = x1.dim() == lo
    if not (unbatched or x1.dim() == lo + 1):
        raise RuntimeError(f"x1 must be {lo}D tensor (unbatched) or {lo + 1}D tensor (batched)")
    if x2 is not None:
        if not (unbatched or x2.dim() == lo + 1):
            raise RuntimeError(f"x2 must be {lo}D tensor (unbatched) or {lo + 1}D tensor (batched)")
        fdim = (lo - 1) if unbatched else lo
        if x2.dim() <= fdim or x1.size(fdim) != x2.size(fdim):
            got2 = x2.size(fdim) if x2.dim() > fdim else "?"
            raise RuntimeError(
                "x1 and x2 must have same number of features. Got: "
                f"x1.size({fdim})={x1.size(fdim)}, x2.size({fdim})={got2}"
            )
    if boolean:
        if x1.dtype != torch.bool or (x2 is not None and x2.dtype != torch.bool):
            warnings.warn(f"Data was converted to {torch.bool} for metric {name}")
        x1b = x1.to(torch.bool)
        return x1b, (x1b if x2 is None else x2.to(torch.bool))
    return x1, (x1 if x2 is None else x2)


def _batched(x1: Tensor, x2: Tensor, what: str):
    """contiguous() + leading batch dimension, as every reference kernel wrapper does
    (e.g. OPS/cuda/ppminkowski_kernel.cu:75-90)."""
    unbatched = x1.dim() == 2
    if not (unbatched or x1.dim() == 3):
        raise RuntimeError("x1 must be 2-D (unbatched) or 3-D (batched) tensor.")
    if not (x2.dim() == x1.dim()):
        raise RuntimeError("x2 must be 2-D (unbatched) or 3-D (batched) tensor.")
    if not unbatched and x1.size(0) != x2.size(0):
        raise RuntimeError("batch_size of x1 and x2 do not match.")
    if x1.size(-1) != x2.size(-1):
        raise RuntimeError("feature dimension of x1 and x2 do not match.")
    if x1.dtype != x2.dtype:
        raise RuntimeError(f"Expected tensor for argument #1 'x1' to have the same type as tensor for argument #2 'x2'; "
                           f"but type {x1.dtype} does not equal {x2.dtype} (while checking arguments for {what})")
    x1c, x2c = x1.contiguous(), x2.contiguous()
    if unbatched:
        x1c, x2c = x1c.unsqueeze(0), x2c.unsqueeze(0)
    return x1c, x2c, unbatched


def _sizes(x1c: Tensor, x2c: Tensor):
    return x1c.size(0), x1c.size(1), x2c.size(1), x1c.size(2)


# --------------------------------------------------------------------------------------------
# raw launches (no autograd)
# --------------------------------------------------------------------------------------------
def _lp_forward_raw(x1c: Tensor, x2c: Tensor, w: Optional[Tensor], p: float, out_exponent: float) -> Tensor:
    B, N1, N2, D = _sizes(x1c, x2c)
    out = torch.empty((B, N1, N2), dtype=x1c.dtype, device=x1c.device)
    if D == 0:
        return out.zero_()
    with torch.cuda.device(x1c.device):
        check(lib.tpw_lp_forward(_FLOAT_CODES[x1c.dtype], _ptr(x1c), _ptr(x2c), _ptr(w), _ptr(out),
                                 B, N1, N2, D, float(p), float(out_exponent), _stream(x1c)), "tpw_lp_forward")
    return out


def _lp_backward_raw(mode: int, grad: Tensor, aux: Optional[Tensor], x1c: Tensor, x2c: Tensor,
                     w: Optional[Tensor], p: float, need1: bool = True, need2: bool = True):
    B, N1, N2, D = _sizes(x1c, x2c)
    if mode == _abi.LP_BWD_CDIST and w is None and math.isinf(p) and p > 0 and (need1 or need2):
        # Chebyshev: find the attaining coordinate of every pair once, then scatter both gradients
        code = _FLOAT_CODES[x1c.dtype]
        nbytes = lib.tpw_chebyshev_backward_scratch_bytes(code, B, N1, N2, D)
        if nbytes > 0:
            g1 = torch.empty_like(x1c) if need1 else None
            g2 = torch.empty_like(x2c) if need2 else None
            scratch = torch.empty((nbytes,), dtype=torch.uint8, device=x1c.device)
            with torch.cuda.device(x1c.device):
                check(lib.tpw_chebyshev_backward_ws(_ptr(grad), _ptr(aux), _ptr(x1c), _ptr(x2c), _ptr(g1), _ptr(g2), _ptr(scratch),
                                                    nbytes, B, N1, N2, D, _stream(x1c)), "tpw_chebyshev_backward_ws")
            return g1, g2
    if w is None and (mode == _abi.LP_BWD_MATMUL or (p == 2.0 and mode in (_abi.LP_BWD_CDIST, _abi.LP_BWD_PPMINKOWSKI))):
        res = _dense_backward_tensor(mode, grad, aux, x1c, x2c, need1, need2)
        if res is not None:
            return res
    g1 = torch.empty_like(x1c) if need1 else None
    g2 = torch.empty_like(x2c) if need2 else None
    _lp_backward_call(mode, grad, aux, x1c, x2c, w, g1, g2, p)
    return g1, g2


def _lp_backward_call(mode: int, grad: Tensor, aux: Optional[Tensor], x1c: Tensor, x2c: Tensor, w: Optional[Tensor],
                      g1: Optional[Tensor], g2: Optional[Tensor], p: float) -> None:
    """``tpw_lp_backward``; with both gradients wanted and a positive scratch query, the one-pass kernel
    (``tpw_lp_backward_ws``: a pair's term is formed once and added to both sums)."""
    B, N1, N2, D = _sizes(x1c, x2c)
    code = _FLOAT_CODES[x1c.dtype]
    with torch.cuda.device(x1c.device):
        nbytes = lib.tpw_lp_backward_scratch_bytes(code, mode, B, N1, N2, D, float(p)) if g1 is not None and g2 is not None else 0
        if nbytes > 0:
            scratch = torch.empty((nbytes,), dtype=torch.uint8, device=x1c.device)
            check(lib.tpw_lp_backward_ws(code, mode, _ptr(grad), _ptr(aux), _ptr(x1c), _ptr(x2c), _ptr(w), _ptr(g1), _ptr(g2),
                                         B, N1, N2, D, float(p), _ptr(scratch), nbytes, _stream(x1c)), "tpw_lp_backward_ws")
        else:
            check(lib.tpw_lp_backward(code, mode, _ptr(grad), _ptr(aux), _ptr(x1c), _ptr(x2c), _ptr(w), _ptr(g1), _ptr(g2),
                                      B, N1, N2, D, float(p), _stream(x1c)), "tpw_lp_backward")


def _bwd_scratch_cap() -> int:
    return int(float(os.environ.get("TPW_BWD_SCRATCH_GB", "8")) * (1 << 30))


def _dense_backward_tensor(mode: int, grad: Tensor, aux: Optional[Tensor], x1c: Tensor, x2c: Tensor,
                           need1: bool, need2: bool, cosine=None):
    """Backward of the p = 2 metrics / the plain gradient products as tensor-core contractions
    (``tpw_dot_backward_ws``), or None when the engine rule keeps the problem on the CUDA cores.

    The split copies of the coefficient matrix take about 8 bytes per element of ``grad``; above
    ``TPW_BWD_SCRATCH_GB`` (default 8) the work is cut into groups of batches, or row blocks of a
    single batch whose grad_x2 contributions are summed in block order (deterministic).

    ``cosine=(epilogue, norm1, norm2)`` runs the whole cosine-family backward instead
    (``tpw_cosine_backward_ws``: ``grad`` is the upstream gradient, ``aux`` the saved forward result)."""
    if x1c.dtype != torch.float32 or not (need1 or need2):
        return None
    B, N1, N2, D = _sizes(x1c, x2c)
    code = _abi.F32
    if lib.tpw_dot_backward_scratch_bytes(code, mode, _dot_engine, B, N1, N2, D) <= 0:
        return None
    eng = _abi.ENGINE_TCGEN05_TF32X3
    cap = _bwd_scratch_cap()
    g1 = torch.empty_like(x1c) if need1 else None
    g2 = torch.empty_like(x2c) if need2 else None
    per_batch = lib.tpw_dot_backward_scratch_bytes(code, mode, eng, 1, N1, N2, D)
    if per_batch <= cap:
        nb = max(1, min(B, cap // per_batch))
        blocks = [(b0, min(B, b0 + nb), 0, N1) for b0 in range(0, B, nb)]
    else:
        rows = N1
        while rows > 256 and lib.tpw_dot_backward_scratch_bytes(code, mode, eng, 1, rows, N2, D) > cap:
            rows = max(256, (rows // 2 + 255) // 256 * 256)
        blocks = [(b, b + 1, r0, min(N1, r0 + rows)) for b in range(B) for r0 in range(0, N1, rows)]
    nbytes = max(lib.tpw_dot_backward_scratch_bytes(code, mode, eng, b1 - b0, r1 - r0, N2, D) for b0, b1, r0, r1 in blocks)
    scratch = torch.empty((nbytes,), dtype=torch.uint8, device=x1c.device)
    part = None
    with torch.cuda.device(x1c.device):
        for b0, b1, r0, r1 in blocks:
            whole = r0 == 0 and r1 == N1
            g1v = None if g1 is None else g1[b0:b1, r0:r1]
            if g2 is None:
                g2v = None
            elif whole or r0 == 0:
                g2v = g2[b0:b1]
            else:
                part = torch.empty_like(g2[b0:b1]) if part is None else part
                g2v = part
            auxv = None if aux is None else aux[b0:b1, r0:r1]
            if cosine is not None:
                epilogue, n1, n2 = cosine
                check(lib.tpw_cosine_backward_ws(epilogue, _ptr(grad[b0:b1, r0:r1]), _ptr(auxv), _ptr(n1[b0:b1, r0:r1]),
                                                 _ptr(n2[b0:b1]), _ptr(x1c[b0:b1, r0:r1]), _ptr(x2c[b0:b1]), _ptr(g1v), _ptr(g2v),
                                                 _ptr(scratch), nbytes, b1 - b0, r1 - r0, N2, D, _stream(x1c)),
                      "tpw_cosine_backward_ws")
            else:
                check(lib.tpw_dot_backward_ws(code, mode, eng, _ptr(grad[b0:b1, r0:r1]), _ptr(auxv), _ptr(x1c[b0:b1, r0:r1]),
                                              _ptr(x2c[b0:b1]), _ptr(g1v), _ptr(g2v), _ptr(scratch), nbytes,
                                              b1 - b0, r1 - r0, N2, D, _stream(x1c)), "tpw_dot_backward_ws")
            if g2 is not None and not (whole or r0 == 0):
                g2[b0:b1] += part
    return g1, g2


def _dot_forward_raw(x1c: Tensor, x2c: Tensor, epilogue: int, engine: Optional[int] = None) -> Tensor:
    engine = _dot_engine if engine is None else engine
    B, N1, N2, D = _sizes(x1c, x2c)
    out = torch.empty((B, N1, N2), dtype=x1c.dtype, device=x1c.device)
    if D == 0:
        # empty contraction: M = 0, norms = 0
        return out.fill_(1.0 if epilogue in (_abi.DOT_COSINE_DIST, _abi.DOT_ONE_MINUS_SIM) else 0.0)
    code = _FLOAT_CODES[x1c.dtype]
    with torch.cuda.device(x1c.device):
        nbytes = lib.tpw_dot_metric_scratch_bytes(code, engine, B, N1, N2, D)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=x1c.device) if nbytes > 0 else None
        check(lib.tpw_dot_metric_forward_ws(code, epilogue, engine, _ptr(x1c), _ptr(x2c), _ptr(out),
                                            _ptr(scratch), nbytes, B, N1, N2, D, _stream(x1c)),
              "tpw_dot_metric_forward_ws")
    return out


def _row_norm(xc: Tensor) -> Tensor:
    B, N, D = xc.shape
    out = torch.empty((B, N), dtype=xc.dtype, device=xc.device)
    with torch.cuda.device(xc.device):
        check(lib.tpw_row_norm(_FLOAT_CODES[xc.dtype], _ptr(xc), _ptr(out), B * N, D, _stream(xc)), "tpw_row_norm")
    return out


def _row_center(xc: Tensor) -> Tensor:
    B, N, D = xc.shape
    out = torch.empty_like(xc)
    with torch.cuda.device(xc.device):
        check(lib.tpw_row_center(_FLOAT_CODES[xc.dtype], _ptr(xc), _ptr(out), B * N, D, _stream(xc)), "tpw_row_center")
    return out


# --------------------------------------------------------------------------------------------
# autograd functions
# --------------------------------------------------------------------------------------------
class _CdistFunction(torch.autograd.Function):
    """at::cdist(x1, x2, p) as called by euclidean / manhattan / minkowski / chebyshev
    (OPS/pairwise_metrics.cpp:30,48,167,305) with ATen's cdist backward formulas."""

    @staticmethod
    def forward(ctx, x1: Tensor, x2: Tensor, p: float):
        in_dtype = x1.dtype
        cdt = _compute_dtype(in_dtype)
        x1c, x2c, unbatched = _batched(x1.to(cdt), x2.to(cdt), "cdist")
        if p == 0:
            out = _cmp_reduce_raw(x1c, x2c, _abi.CMP_NE, _abi.RED_SUM).to(cdt)
        elif math.isinf(p):
            out = _lp_forward_raw(x1c, x2c, None, math.inf, 1.0)
        elif p == 2 and _tensor_engine_selected(x1c, x2c):
            # sqrt(clamp(|x|^2 + |y|^2 - 2 x.y, 0)): the contraction form ATen itself uses for p = 2
            out = _dot_forward_raw(x1c, x2c, _abi.DOT_EUCLIDEAN)
        else:
            out = _lp_forward_raw(x1c, x2c, None, p, 1.0 / p)
        ctx.save_for_backward(x1c, x2c, out)
        ctx.p, ctx.unbatched, ctx.in_dtype = p, unbatched, in_dtype
        res = out.squeeze(0) if unbatched else out
        return res.to(in_dtype)

    @staticmethod
    def backward(ctx, grad):
        x1c, x2c, out = ctx.saved_tensors
        need1, need2 = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if ctx.p == 0:
            g1 = torch.zeros_like(x1c) if need1 else None
            g2 = torch.zeros_like(x2c) if need2 else None
        else:
            g = grad.to(x1c.dtype).contiguous()
            if ctx.unbatched:
                g = g.unsqueeze(0)
            g1, g2 = _lp_backward_raw(_abi.LP_BWD_CDIST, g, out, x1c, x2c, None, ctx.p, need1, need2)
        if ctx.unbatched:
            g1 = None if g1 is None else g1.squeeze(0)
            g2 = None if g2 is None else g2.squeeze(0)
        g1 = None if g1 is None else g1.to(ctx.in_dtype)
        g2 = None if g2 is None else g2.to(ctx.in_dtype)
        return g1, g2, None


class _PPMinkowskiFunction(torch.autograd.Function):
    """PPowerMinkowskiFunction of OPS/autograd/ppminkowski_kernel.cpp:9-46."""

    @staticmethod
    def forward(ctx, x1: Tensor, x2: Tensor, p: float):
        in_dtype = x1.dtype
        cdt = _compute_dtype(in_dtype)
        x1c, x2c, unbatched = _batched(x1.to(cdt), x2.to(cdt), "_ppminkowski_forward")
        if p == 0:
            B, N1, N2, D = _sizes(x1c, x2c)
            out = torch.full((B, N1, N2), float(D), dtype=cdt, device=x1c.device)
        elif p == 2 and _tensor_engine_selected(x1c, x2c):
            out = _dot_forward_raw(x1c, x2c, _abi.DOT_SQEUCLIDEAN)
        else:
            out = _lp_forward_raw(x1c, x2c, None, p, 1.0)
        ctx.save_for_backward(x1c, x2c)
        ctx.p, ctx.unbatched, ctx.in_dtype = p, unbatched, in_dtype
        res = out.squeeze(0) if unbatched else out
        return res.to(in_dtype)

    @staticmethod
    def backward(ctx, grad):
        x1c, x2c = ctx.saved_tensors
        g1, g2 = _ppminkowski_backward_raw(grad, x1c, x2c, ctx.p, ctx.unbatched,
                                           ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        g1 = None if g1 is None else g1.to(ctx.in_dtype)
        g2 = None if g2 is None else g2.to(ctx.in_dtype)
        return g1, g2, None


def _ppminkowski_backward_raw(grad, x1c, x2c, p, unbatched, need1=True, need2=True):
    g = grad.to(x1c.dtype).contiguous()
    if unbatched:
        g = g.unsqueeze(0)
    B, N1, N2, D = _sizes(x1c, x2c)
    if p == 0:
        g1 = torch.zeros_like(x1c) if need1 else None
        g2 = torch.zeros_like(x2c) if need2 else None
    elif math.isinf(p):
        g1 = torch.zeros_like(x1c)
        g2 = torch.zeros_like(x2c)
        with torch.cuda.device(x1c.device):
            check(lib.tpw_lp_inf_backward(_FLOAT_CODES[x1c.dtype], _ptr(g), _ptr(x1c), _ptr(x2c), None,
                                          _ptr(g1), _ptr(g2), None, B, N1, N2, D, int(p < 0), _stream(x1c)),
                  "tpw_lp_inf_backward")
    else:
        g1, g2 = _lp_backward_raw(_abi.LP_BWD_PPMINKOWSKI, g, None, x1c, x2c, None, p, need1, need2)
    if unbatched:
        g1 = None if g1 is None else g1.squeeze(0)
        g2 = None if g2 is None else g2.squeeze(0)
    return g1, g2


class _WMinkowskiFunction(torch.autograd.Function):
    """WeightedMinkowskiFunction of OPS/autograd/wminkowski_kernel.cpp:9-50."""

    @staticmethod
    def forward(ctx, x1: Tensor, x2: Tensor, w: Tensor, p: float):
        in_dtype = x1.dtype
        cdt = _compute_dtype(in_dtype)
        if not (x1.dtype == x2.dtype == w.dtype):
            raise RuntimeError("Expected x1, x2 and w to have the same type (while checking arguments for _wminkowski_forward)")
        x1c, x2c, unbatched = _batched(x1.to(cdt), x2.to(cdt), "_wminkowski_forward")
        if not (unbatched or w.dim() == 2):
            raise RuntimeError("w must be 1-D (unbatched) or 2-D (batched) tensor.")
        if unbatched and w.dim() != 1:
            raise RuntimeError("w must be 1-D (unbatched) or 2-D (batched) tensor.")
        wc = w.to(cdt).contiguous()
        if unbatched:
            wc = wc.unsqueeze(0)
        B, N1, N2, D = _sizes(x1c, x2c)
        if wc.size(0) != B:
            raise RuntimeError("batch_size of x1, x2, and w do not match.")
        # The reference compares w.size(1) with N1 in the batched case (OPS/cuda/wminkowski_kernel.cu:91),
        # which rejects every valid weight vector unless N1 == D; the feature count is what is meant.
        if wc.size(1) != D:
            raise RuntimeError("feature dimension of x1, x2, and w do not match.")
        if p == 0:
            out = torch.full((B, N1, N2), float(D), dtype=cdt, device=x1c.device)
        elif math.isinf(p):
            out = _lp_forward_raw(x1c, x2c, wc, p, 1.0)
        else:
            out = _lp_forward_raw(x1c, x2c, wc, p, 1.0 / p)
        ctx.save_for_backward(x1c, x2c, wc)
        ctx.p, ctx.unbatched, ctx.in_dtype = p, unbatched, in_dtype
        res = out.squeeze(0) if unbatched else out
        return res.to(in_dtype)

    @staticmethod
    def backward(ctx, grad):
        x1c, x2c, wc = ctx.saved_tensors
        g1, g2, gw = _wminkowski_backward_raw(grad, x1c, x2c, wc, ctx.p, ctx.unbatched)
        return g1.to(ctx.in_dtype), g2.to(ctx.in_dtype), gw.to(ctx.in_dtype), None


def _wminkowski_backward_raw(grad, x1c, x2c, wc, p, unbatched):
    g = grad.to(x1c.dtype).contiguous()
    if unbatched:
        g = g.unsqueeze(0)
    B, N1, N2, D = _sizes(x1c, x2c)
    code = _FLOAT_CODES[x1c.dtype]
    g1, g2, gw = torch.zeros_like(x1c), torch.zeros_like(x2c), torch.zeros_like(wc)
    if p != 0 and B * N1 * N2 * D > 0:
        with torch.cuda.device(x1c.device):
            if math.isinf(p):
                check(lib.tpw_lp_inf_backward(code, _ptr(g), _ptr(x1c), _ptr(x2c), _ptr(wc), _ptr(g1), _ptr(g2),
                                              _ptr(gw), B, N1, N2, D, int(p < 0), _stream(x1c)),
                      "tpw_lp_inf_backward")
            else:
                # coefficient S^(1/p-1): the reference's forward kernel with its `backward` flag
                # (OPS/cuda/wminkowski_kernel.cu:16-37 called at :300-320)
                coef = _lp_forward_raw(x1c, x2c, wc, p, 1.0 / p - 1.0)
                _lp_backward_call(_abi.LP_BWD_WMINKOWSKI, g, coef, x1c, x2c, wc, g1, g2, p)
                scratch = torch.empty((B, N1, D), dtype=x1c.dtype, device=x1c.device)
                check(lib.tpw_wminkowski_backward_w(code, _ptr(g), _ptr(coef), _ptr(x1c), _ptr(x2c), _ptr(gw),
                                                    _ptr(scratch), B, N1, N2, D, float(p), _stream(x1c)),
                      "tpw_wminkowski_backward_w")
    if unbatched:
        g1, g2, gw = g1.squeeze(0), g2.squeeze(0), gw.squeeze(0)
    return g1, g2, gw


class _CosineSimilarityFunction(torch.autograd.Function):
    """x1.x2^T / (|x1||x2|^T) with prf_div mode "identity" (OPS/pairwise_metrics.cpp:112-122) and
    the gradient that autograd derives for that composition (norm, outer product, matmul, prf_div:
    OPS/cuda/prf_div_kernel.cu:315-366).  `epilogue` also folds the 1 - S (+clip) of cosine /
    correlation distances (:51-56, :203)."""

    @staticmethod
    def forward(ctx, x1: Tensor, x2: Tensor, epilogue: int):
        in_dtype = x1.dtype
        cdt = _compute_dtype(in_dtype)
        x1c, x2c, unbatched = _batched(x1.to(cdt), x2.to(cdt), "cosine_similarity")
        out = _dot_forward_raw(x1c, x2c, epilogue)
        ctx.save_for_backward(x1c, x2c, out)
        ctx.epilogue, ctx.unbatched, ctx.in_dtype = epilogue, unbatched, in_dtype
        res = out.squeeze(0) if unbatched else out
        return res.to(in_dtype)

    @staticmethod
    def backward(ctx, grad):
        x1c, x2c, out = ctx.saved_tensors
        g = grad.to(x1c.dtype).contiguous()
        if ctx.unbatched:
            g = g.unsqueeze(0)
        B, N1, N2, D = _sizes(x1c, x2c)
        code = _FLOAT_CODES[x1c.dtype]
        n1, n2 = _row_norm(x1c), _row_norm(x2c)
        fused = _dense_backward_tensor(_abi.LP_BWD_MATMUL, g, out, x1c, x2c, True, True, cosine=(ctx.epilogue, n1, n2))
        if fused is not None:
            g1, g2 = fused
        else:
            dM = torch.empty_like(g)
            rowterm = torch.empty((B, N1), dtype=g.dtype, device=g.device)
            colterm = torch.empty((B, N2), dtype=g.dtype, device=g.device)
            with torch.cuda.device(x1c.device):
                check(lib.tpw_cosine_backward_prepare(code, ctx.epilogue, _ptr(g), _ptr(out), _ptr(n1), _ptr(n2),
                                                      _ptr(dM), _ptr(rowterm), _ptr(colterm), B, N1, N2, _stream(x1c)),
                      "tpw_cosine_backward_prepare")
                g1, g2 = _lp_backward_raw(_abi.LP_BWD_MATMUL, dM, None, x1c, x2c, None, 2.0)
                check(lib.tpw_cosine_backward_finish(code, _ptr(g1), _ptr(x1c), _ptr(n1), _ptr(rowterm), B * N1, D, _stream(x1c)),
                      "tpw_cosine_backward_finish")
                check(lib.tpw_cosine_backward_finish(code, _ptr(g2), _ptr(x2c), _ptr(n2), _ptr(colterm), B * N2, D, _stream(x1c)),
                      "tpw_cosine_backward_finish")
        if ctx.unbatched:
            g1, g2 = g1.squeeze(0), g2.squeeze(0)
        return g1.to(ctx.in_dtype), g2.to(ctx.in_dtype), None


class _RowCenterFunction(torch.autograd.Function):
    """x - x.mean(-1, keepdim=True) (OPS/pairwise_metrics.cpp:197-198)."""

    @staticmethod
    def forward(ctx, x: Tensor):
        cdt = _compute_dtype(x.dtype)
        xc = x.to(cdt).contiguous()
        shape = xc.shape
        out = _row_center(xc.reshape(1, -1, shape[-1])).reshape(shape)
        ctx.in_dtype = x.dtype
        return out.to(x.dtype)

    @staticmethod
    def backward(ctx, grad):
        cdt = _compute_dtype(grad.dtype)
        gc = grad.to(cdt).contiguous()
        shape = gc.shape
        return _row_center(gc.reshape(1, -1, shape[-1])).reshape(shape).to(ctx.in_dtype)


class _HausdorffFunction(torch.autograd.Function):
    """DirectedHausdorffDistancesFunction of OPS/autograd/hausdorff_kernel.cpp:9-61.  The
    reference re-runs the forward inside backward with a cloned generator; here the forward
    results are saved instead, which is the same thing without the second pass."""

    @staticmethod
    def forward(ctx, x1: Tensor, x2: Tensor, shuffle: bool, generator):
        if x1.dtype != x2.dtype:
            raise RuntimeError("Expected x1 and x2 to have the same type (while checking arguments for _directed_hausdorff_forward)")
        in_dtype = x1.dtype
        cdt = _compute_dtype(in_dtype)
        unbatched = x1.dim() == 3
        if not (unbatched or x1.dim() == 4):
            raise RuntimeError("x1 must be 3-D (unbatched) or 4-D (batched) tensor.")
        if x2.dim() != x1.dim():
            raise RuntimeError("x2 must be 3-D (unbatched) or 4-D (batched) tensor.")
        if not unbatched and x1.size(0) != x2.size(0):
            raise RuntimeError("batch_size of x1 and x2 do not match.")
        if x1.size(-1) != x2.size(-1):
            raise RuntimeError("feature dimension of x1 and x2 do not match.")
        x1c, x2c = x1.to(cdt).contiguous(), x2.to(cdt).contiguous()
        if unbatched:
            x1c, x2c = x1c.unsqueeze(0), x2c.unsqueeze(0)
        B, N1, M1, D = x1c.shape
        N2, M2 = x2c.size(1), x2c.size(2)
        dev = x1c.device
        out = torch.empty((B, N1, N2), dtype=cdt, device=dev)
        idx1 = torch.empty((B, N1, N2), dtype=torch.int64, device=dev)
        idx2 = torch.empty((B, N1, N2), dtype=torch.int64, device=dev)
        order1 = order2 = None
        if shuffle and B > 0:
            # per batch, x1's permutation then x2's, as OPS/cuda/hausdorff_kernel.cu:158-167 draws them
            order1 = torch.empty((B, M1), dtype=torch.int64, device=dev)
            order2 = torch.empty((B, M2), dtype=torch.int64, device=dev)
            for b in range(B):
                p1 = torch.randperm(M1, generator=generator, device=dev)
                p2 = torch.randperm(M2, generator=generator, device=dev)
                order1[b, p1] = torch.arange(M1, device=dev)
                order2[b, p2] = torch.arange(M2, device=dev)
        with torch.cuda.device(dev):
            nbytes = lib.tpw_hausdorff_scratch_bytes(B, N1, N2, M1)
            scratch = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=dev)
            check(lib.tpw_hausdorff_forward(_FLOAT_CODES[cdt], _ptr(x1c), _ptr(x2c), _ptr(order1), _ptr(order2),
                                            _ptr(out), _ptr(idx1), _ptr(idx2), _ptr(scratch),
                                            B, N1, N2, M1, M2, D, _stream(x1c)), "tpw_hausdorff_forward")
        ctx.save_for_backward(x1c, x2c, out, idx1, idx2)
        ctx.unbatched, ctx.in_dtype = unbatched, in_dtype
        if unbatched:
            out, idx1, idx2 = out.squeeze(0), idx1.squeeze(0), idx2.squeeze(0)
        out = out.to(in_dtype)
        ctx.mark_non_differentiable(idx1, idx2)
        return out, idx1, idx2

    @staticmethod
    def backward(ctx, grad, _g1, _g2):
        x1c, x2c, out, idx1, idx2 = ctx.saved_tensors
        g = grad.to(x1c.dtype).contiguous()
        if ctx.unbatched:
            g = g.unsqueeze(0)
        B, N1, M1, D = x1c.shape
        N2, M2 = x2c.size(1), x2c.size(2)
        g1, g2 = torch.empty_like(x1c), torch.empty_like(x2c)
        with torch.cuda.device(x1c.device):
            check(lib.tpw_hausdorff_backward(_FLOAT_CODES[x1c.dtype], _ptr(g), _ptr(out), _ptr(idx1), _ptr(idx2),
                                             _ptr(x1c), _ptr(x2c), _ptr(g1), _ptr(g2),
                                             B, N1, N2, M1, M2, D, _stream(x1c)), "tpw_hausdorff_backward")
        if ctx.unbatched:
            g1, g2 = g1.squeeze(0), g2.squeeze(0)
        return g1.to(ctx.in_dtype), g2.to(ctx.in_dtype), None, None


class _PRFDivFunction(torch.autograd.Function):
    """PRFDivideFunction of OPS/autograd/prf_div_kernel.cpp:9-52 (same-shape operands)."""

    @staticmethod
    def forward(ctx, x: Tensor, y: Tensor, mode: int):
        if x.shape != y.shape:
            raise RuntimeError("self and other must have the same shape.")
        dt = torch.result_type(x, y)
        if not dt.is_floating_point:
            dt = torch.float32
        cdt = _compute_dtype(dt)
        xc, yc = x.to(cdt).contiguous(), y.to(cdt).contiguous()
        out = torch.empty_like(xc)
        with torch.cuda.device(xc.device):
            check(lib.tpw_prf_div_forward(_FLOAT_CODES[cdt], mode, _ptr(xc), _ptr(yc), _ptr(out), xc.numel(), _stream(xc)),
                  "tpw_prf_div_forward")
        ctx.save_for_backward(xc, yc)
        ctx.mode, ctx.dtypes = mode, (x.dtype, y.dtype)
        return out.to(dt)

    @staticmethod
    def backward(ctx, grad):
        xc, yc = ctx.saved_tensors
        g = grad.to(xc.dtype).contiguous()
        gx = torch.empty_like(xc) if ctx.needs_input_grad[0] else None
        gy = torch.empty_like(yc) if ctx.needs_input_grad[1] else None
        with torch.cuda.device(xc.device):
            check(lib.tpw_prf_div_backward(_FLOAT_CODES[xc.dtype], ctx.mode, _ptr(g), _ptr(xc), _ptr(yc),
                                           _ptr(gx), _ptr(gy), xc.numel(), _stream(xc)), "tpw_prf_div_backward")
        gx = None if gx is None else gx.to(ctx.dtypes[0])
        gy = None if gy is None else gy.to(ctx.dtypes[1])
        return gx, gy, None


# --------------------------------------------------------------------------------------------
# boolean / compare-reduce
# --------------------------------------------------------------------------------------------
def _pack_bool(xb: Tensor):
    """[B, N, D] bool -> (words [B, N, W] int32 view of uint32, popcounts [B, N] int32, W)."""
    B, N, D = xb.shape
    W = max(4, (D + 31) // 32)
    W = (W + 3) // 4 * 4  # 16-byte rows for the TMA path
    words = torch.empty((B, N, W), dtype=torch.int32, device=xb.device)
    pops = torch.empty((B, N), dtype=torch.int32, device=xb.device)
    src = xb.contiguous().view(torch.uint8)
    with torch.cuda.device(xb.device):
        check(lib.tpw_bitpack(_ptr(src), _ptr(words), _ptr(pops), B * N, D, W, _stream(xb)), "tpw_bitpack")
    return words, pops, W


def _bool_metric_raw(x1: Tensor, x2: Tensor, metric: str) -> Tensor:
    """x1, x2 boolean, 2-D or 3-D; float32 result."""
    _require_cuda(x1, x2)
    unbatched = x1.dim() == 2
    if not (unbatched or x1.dim() == 3):
        raise RuntimeError("x1 must be 2-D (unbatched) or 3-D (batched) tensor.")
    if x2.dim() != x1.dim():
        raise RuntimeError("x2 must be 2-D (unbatched) or 3-D (batched) tensor.")
    if not unbatched and x1.size(0) != x2.size(0):
        raise RuntimeError("batch_size of x1 and x2 do not match.")
    if x1.size(-1) != x2.size(-1):
        raise RuntimeError("feature dimension of x1 and x2 do not match.")
    x1c, x2c = (x1.unsqueeze(0), x2.unsqueeze(0)) if unbatched else (x1, x2)
    B, N1, D = x1c.shape
    N2 = x2c.size(1)
    out = torch.empty((B, N1, N2), dtype=torch.float32, device=x1.device)
    if D == 0:
        out.zero_()
        if metric in ("eq_mean", "ne_mean", "kulczynski1", "russellrao", "kulsinski", "dice",
                      "rogerstanimoto", "sokalmichener", "sokalsneath"):
            out.fill_(float("nan"))
    elif out.numel() > 0:
        w1, p1, W = _pack_bool(x1c)
        if x2c is x1c or (x2c.data_ptr() == x1c.data_ptr() and x2c.shape == x1c.shape):
            w2, p2 = w1, p1
        else:
            w2, p2, _ = _pack_bool(x2c)
        with torch.cuda.device(x1.device):
            b1 = x1c.contiguous().view(torch.uint8)
            b2 = b1 if w2 is w1 else x2c.contiguous().view(torch.uint8)
            if lib.tpw_bool_metric_tc_eligible(B, N1, N2, D) and b1.data_ptr() % 16 == 0 and b2.data_ptr() % 16 == 0:
                # large problem: the counts come from the tensor cores (8-bit integer contraction of the 0 / 1 bytes)
                check(lib.tpw_bool_metric_forward_tc(_abi.BOOL_METRICS[metric], _ptr(b1), _ptr(b2), _ptr(p1), _ptr(p2),
                                                     _ptr(out), B, N1, N2, D, _stream(x1)), "tpw_bool_metric_forward_tc")
            else:
                check(lib.tpw_bool_metric_forward(_abi.BOOL_METRICS[metric], _ptr(w1), _ptr(w2), _ptr(p1), _ptr(p2),
                                                  _ptr(out), B, N1, N2, D, W, _stream(x1)), "tpw_bool_metric_forward")
    return out.squeeze(0) if unbatched else out


_CMP_CODES = {torch.float32: _abi.F32, torch.float64: _abi.F64, torch.int32: _abi.I32, torch.int64: _abi.I64}


def _cmp_reduce_raw(x1c: Tensor, x2c: Tensor, op: int, reduction: int) -> Tensor:
    """x1c, x2c batched, same dtype among float32/float64/int32/int64; float32 result."""
    B, N1, N2, D = _sizes(x1c, x2c)
    out = torch.empty((B, N1, N2), dtype=torch.float32, device=x1c.device)
    if D == 0:
        return out.fill_(float("nan") if reduction == _abi.RED_MEAN else 0.0)
    with torch.cuda.device(x1c.device):
        check(lib.tpw_cmp_reduce_forward(_CMP_CODES[x1c.dtype], op, reduction, _ptr(x1c), _ptr(x2c), _ptr(out),
                                         B, N1, N2, D, _stream(x1c)), "tpw_cmp_reduce_forward")
    return out


def _pairwise_compare(x1: Tensor, x2: Tensor, op: int, reduction: int) -> Tensor:
    """pw{eq,ne}_{sum,mean}: any dtype, promoted with result_type, float32 output
    (OPS/cuda/pairwise_binary_kernels.cu:144-220)."""
    _require_cuda(x1, x2)
    common = torch.result_type(x1, x2)
    if common == torch.bool:
        name = ("eq" if op == _abi.CMP_EQ else "ne") + ("_mean" if reduction == _abi.RED_MEAN else "_sum")
        return _bool_metric_raw(x1.to(torch.bool), x2.to(torch.bool), name)
    if common in (torch.float16, torch.bfloat16):
        common = torch.float32  # exact widening keeps every comparison
    elif common in (torch.uint8, torch.int8, torch.int16):
        common = torch.int32
    if common not in _CMP_CODES:
        raise RuntimeError(f"pairwise comparison is not implemented for {common}")
    x1c, x2c, unbatched = _batched(x1.to(common), x2.to(common), "pairwise_binary_reduction_forward")
    out = _cmp_reduce_raw(x1c, x2c, op, reduction)
    return out.squeeze(0) if unbatched else out


def _require_bool(x1: Tensor, x2: Tensor, name: str):
    if torch.result_type(x1, x2) != torch.bool:
        raise RuntimeError(f'"{name}" not implemented for \'{torch.result_type(x1, x2)}\'')


def pwand_sum(x1: Tensor, x2: Tensor) -> Tensor:
    _require_bool(x1, x2, "pairwise_binary_reduction_forward")
    return _bool_metric_raw(x1, x2, "and_sum")


def pwor_sum(x1: Tensor, x2: Tensor) -> Tensor:
    _require_bool(x1, x2, "pairwise_binary_reduction_forward")
    return _bool_metric_raw(x1, x2, "or_sum")


def pwxor_sum(x1: Tensor, x2: Tensor) -> Tensor:
    _require_bool(x1, x2, "pairwise_binary_reduction_forward")
    return _bool_metric_raw(x1, x2, "xor_sum")


def pweq_sum(x1: Tensor, x2: Tensor) -> Tensor:
    return _pairwise_compare(x1, x2, _abi.CMP_EQ, _abi.RED_SUM)


def pwne_sum(x1: Tensor, x2: Tensor) -> Tensor:
    return _pairwise_compare(x1, x2, _abi.CMP_NE, _abi.RED_SUM)


def pweq_mean(x1: Tensor, x2: Tensor) -> Tensor:
    return _pairwise_compare(x1, x2, _abi.CMP_EQ, _abi.RED_MEAN)


def pwne_mean(x1: Tensor, x2: Tensor) -> Tensor:
    return _pairwise_compare(x1, x2, _abi.CMP_NE, _abi.RED_MEAN)


# --------------------------------------------------------------------------------------------
# internal ops of the reference (same names)
# --------------------------------------------------------------------------------------------
def _ppminkowski(x1: Tensor, x2: Tensor, p: float = 2.0) -> Tensor:
    """sum_k |x1 - x2|^p without the root (OPS/ppminkowski.cpp:31-38)."""
    _require_cuda(x1, x2)
    return _PPMinkowskiFunction.apply(x1, x2, float(p))


def _wminkowski(x1: Tensor, x2: Tensor, w: Tensor, p: float = 2.0) -> Tensor:
    """(sum_k w_k |x1 - x2|^p)^(1/p) (OPS/wminkowski.cpp:33-40)."""
    _require_cuda(x1, x2, w)
    return _WMinkowskiFunction.apply(x1, x2, w, float(p))


def _directed_hausdorff(x1: Tensor, x2: Tensor, *, shuffle: bool = False, generator=None):
    _require_cuda(x1, x2)
    return _HausdorffFunction.apply(x1, x2, bool(shuffle), generator)


def prf_div(x: Tensor, y: Tensor, mode: str = "zero") -> Tensor:
    """y != 0 ? x / y : (0 | x) (OPS/prf_div.cpp:359-400, tensor/tensor overload)."""
    if mode not in ("zero", "identity"):
        raise RuntimeError(f"mode must be either zero or identity. Got {mode}")
    _require_cuda(x, y)
    return _PRFDivFunction.apply(x, y, _abi.PRF_IDENTITY if mode == "identity" else _abi.PRF_ZERO)


def _cdist_p(x1: Tensor, x2: Tensor, p: float) -> Tensor:
    _require_cuda(x1, x2)
    if p < 0:
        raise RuntimeError("cdist only supports non-negative p values")
    if x1.dim() == 3 and x2.dim() == 3 and x1.size(0) != x2.size(0):
        raise RuntimeError("batch_size of x1 and x2 do not match.")
    return _CdistFunction.apply(x1, x2, float(p))


# --------------------------------------------------------------------------------------------
# public metrics (OPS/pairwise_metrics.cpp)
# --------------------------------------------------------------------------------------------
def euclidean_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("euclidean_distances", x1, x2)
    return _cdist_p(x1_, x2_, 2.0)


def manhattan_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("manhattan_distances", x1, x2)
    return _cdist_p(x1_, x2_, 1.0)


def chebyshev_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("chebyshev_distances", x1, x2)
    return _cdist_p(x1_, x2_, math.inf)


def minkowski_distances(x1: Tensor, x2: Optional[Tensor] = None, p: float = 2.0) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("minkowski_distances", x1, x2)
    return _cdist_p(x1_, x2_, float(p))


def wminkowski_distances(x1: Tensor, x2: Optional[Tensor] = None, p: float = 2.0, w: Optional[Tensor] = None) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("wminkowski_distances", x1, x2)
    if w is None:
        return _cdist_p(x1_, x2_, float(p))
    return _wminkowski(x1_, x2_, w, p)


def sqeuclidean_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("sqeuclidean_distances", x1, x2)
    return _ppminkowski(x1_, x2_, 2.0)


def cosine_similarity(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("cosine_similarity", x1, x2)
    _require_cuda(x1_, x2_)
    return _CosineSimilarityFunction.apply(x1_, x2_, _abi.DOT_COSINE_SIM)


def cosine_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("cosine_similarity", x1, x2)
    _require_cuda(x1_, x2_)
    return _CosineSimilarityFunction.apply(x1_, x2_, _abi.DOT_COSINE_DIST)


def correlation_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("correlation_distances", x1, x2)
    _require_cuda(x1_, x2_)
    c1 = _RowCenterFunction.apply(x1_)
    c2 = c1 if x2 is None else _RowCenterFunction.apply(x2_)
    return _CosineSimilarityFunction.apply(c1, c2, _abi.DOT_ONE_MINUS_SIM)


def linear_kernel(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("linear_kernel", x1, x2)
    _require_cuda(x1_, x2_)
    return _LinearKernelFunction.apply(x1_, x2_)


class _LinearKernelFunction(torch.autograd.Function):
    """x1 @ x2^T (OPS/pairwise_metrics.cpp:58-65)."""

    @staticmethod
    def forward(ctx, x1, x2):
        in_dtype = x1.dtype
        cdt = _compute_dtype(in_dtype)
        x1c, x2c, unbatched = _batched(x1.to(cdt), x2.to(cdt), "linear_kernel")
        # the raw dot product has no norm to hide bf16 rounding behind: tf32 x 3 with chunked accumulation
        # (as accurate as the fp32 FMA chain) on large problems, the exact fp32 / fp64 tile otherwise
        tensor = _dot_engine != _abi.ENGINE_SIMT_FP32 and _tensor_engine_selected(x1c, x2c)
        out = _dot_forward_raw(x1c, x2c, _abi.DOT_LINEAR, _abi.ENGINE_TCGEN05_TF32X3 if tensor else _abi.ENGINE_SIMT_FP32)
        ctx.save_for_backward(x1c, x2c)
        ctx.unbatched, ctx.in_dtype = unbatched, in_dtype
        return (out.squeeze(0) if unbatched else out).to(in_dtype)

    @staticmethod
    def backward(ctx, grad):
        x1c, x2c = ctx.saved_tensors
        g = grad.to(x1c.dtype).contiguous()
        if ctx.unbatched:
            g = g.unsqueeze(0)
        g1, g2 = _lp_backward_raw(_abi.LP_BWD_MATMUL, g, None, x1c, x2c, None, 2.0)
        if ctx.unbatched:
            g1, g2 = g1.squeeze(0), g2.squeeze(0)
        return g1.to(ctx.in_dtype), g2.to(ctx.in_dtype)


def hamming_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    x1_, x2_ = check_pairwise_inputs("hamming_distances", x1, x2)
    return pwne_mean(x1_, x2_)


def _boolean_metric(name: str, metric: str, x1: Tensor, x2: Optional[Tensor]) -> Tensor:
    x1_, x2_ = check_pairwise_inputs(name, x1, x2, boolean=True)
    return _bool_metric_raw(x1_, x2_, metric)


def jaccard_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return _boolean_metric("jaccard_distances", "jaccard", x1, x2)


def kulsinski_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    warnings.warn("kulsinski_distances is deprecated in SciPy 1.9.0 and might be removed in the future. "
                  "Please use kulczynski1_distances.", DeprecationWarning)
    return _boolean_metric("kulsinski_distances", "kulsinski", x1, x2)


def kulczynski1_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return _boolean_metric("kulczynski1_distances", "kulczynski1", x1, x2)


def yule_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return _boolean_metric("yule_distances", "yule", x1, x2)


def dice_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return _boolean_metric("dice_distances", "dice", x1, x2)


def rogerstanimoto_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return _boolean_metric("rogerstanimoto_distances", "rogerstanimoto", x1, x2)


def russellrao_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return _boolean_metric("russellrao_distances", "russellrao", x1, x2)


def sokalmichener_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return _boolean_metric("sokalmichener_distances", "sokalmichener", x1, x2)


def sokalsneath_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return _boolean_metric("sokalsneath_distances", "sokalsneath", x1, x2)


def directed_hausdorff_distances(x1: Tensor, x2: Optional[Tensor] = None, *, shuffle: bool = False, generator=None):
    x1_, x2_ = check_pairwise_inputs("directed_hausdorff_distances", x1, x2, sets=True)
    return _directed_hausdorff(x1_, x2_, shuffle=shuffle, generator=generator)


# aliases (OPS/pairwise_metrics.cpp:265-270, 411-438)
def cityblock_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return manhattan_distances(x1, x2)


def l1_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return manhattan_distances(x1, x2)


def l2_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return euclidean_distances(x1, x2)


def lp_distances(x1: Tensor, x2: Optional[Tensor] = None, p: float = 2.0) -> Tensor:
    return minkowski_distances(x1, x2, p)


def linf_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    return chebyshev_distances(x1, x2)


# --------------------------------------------------------------------------------------------
# callers on either side of the path: kernel functions, standardised Euclidean, neighbour masks
# (compositions of the operators above, as in the reference; gradients flow through them)
# --------------------------------------------------------------------------------------------
def _default_gamma(x1: Tensor, gamma: Optional[float]) -> float:
    # the reference divides by x1.size(1) whatever the rank (OPS/pairwise_metrics.cpp:76,88,97,108)
    return 1.0 / x1.size(1) if gamma is None else float(gamma)


def polynomial_kernel(x1: Tensor, x2: Optional[Tensor] = None, degree: int = 3, gamma: Optional[float] = None,
                      coef0: float = 1.0) -> Tensor:
    """(gamma <x, y> + coef0)^degree (OPS/pairwise_metrics.cpp:67-78)."""
    return (linear_kernel(x1, x2) * _default_gamma(x1, gamma) + coef0) ** int(degree)


def sigmoid_kernel(x1: Tensor, x2: Optional[Tensor] = None, gamma: Optional[float] = None, coef0: float = 1.0) -> Tensor:
    """tanh(gamma <x, y> + coef0) (OPS/pairwise_metrics.cpp:80-90)."""
    return torch.tanh(linear_kernel(x1, x2) * _default_gamma(x1, gamma) + coef0)


def rbf_kernel(x1: Tensor, x2: Optional[Tensor] = None, gamma: Optional[float] = None) -> Tensor:
    """exp(-gamma |x - y|^2) (OPS/pairwise_metrics.cpp:92-99)."""
    return torch.exp(sqeuclidean_distances(x1, x2) * -_default_gamma(x1, gamma))


def laplacian_kernel(x1: Tensor, x2: Optional[Tensor] = None, gamma: Optional[float] = None) -> Tensor:
    """exp(-gamma |x - y|_1) (OPS/pairwise_metrics.cpp:101-110)."""
    return torch.exp(manhattan_distances(x1, x2) * -_default_gamma(x1, gamma))


def seuclidean_distances(x1: Tensor, x2: Optional[Tensor] = None, V: Optional[Tensor] = None) -> Tensor:
    """sqrt(sum_k (x_k - y_k)^2 / V_k): weighted Minkowski with w = 1/V, p = 2; V defaults to the
    feature variances of x1 (OPS/pairwise_metrics.cpp:245-263)."""
    if x2 is not None and V is None:
        raise RuntimeError("V is required for seuclidean when x2 is passed.")
    x1_, x2_ = check_pairwise_inputs("euclidean_distances", x1, x2)
    if V is None:
        with torch.no_grad():
            V = x1_.var(dim=0 if x1_.dim() == 2 else (0, 1))
    w = prf_div(torch.ones_like(V), V, "identity")  # prf_ldiv(V, 1, "identity"): 1/V, and 1 where V == 0
    return _wminkowski(x1_, x2_, w, 2.0)


class _PairSumFunction(torch.autograd.Function):
    """sum_k term(x1_k, x2_k) for terms that are not functions of the difference alone: _canberra
    (OPS/autograd/canberra_kernel.cpp, kernels OPS/cpu/canberra_kernel.cpp:22-29,85-125) and
    _additive_chi2_kernel (OPS/cpu/additive_chi2_kernel.cpp:22-31,88-131).  Where a term's denominator is 0
    the forward skips it and the backward contributes 0 (the reference's canberra backward divides by it)."""

    @staticmethod
    def forward(ctx, x1: Tensor, x2: Tensor, metric: int):
        in_dtype = x1.dtype
        cdt = _compute_dtype(in_dtype)
        x1c, x2c, unbatched = _batched(x1.to(cdt), x2.to(cdt), "pair_sum")
        B, N1, N2, D = _sizes(x1c, x2c)
        out = torch.empty((B, N1, N2), dtype=cdt, device=x1c.device)
        if D == 0:
            out.zero_()
        else:
            with torch.cuda.device(x1c.device):
                check(lib.tpw_pair_sum_forward(_FLOAT_CODES[cdt], metric, _ptr(x1c), _ptr(x2c), _ptr(out), B, N1, N2, D,
                                               _stream(x1c)), "tpw_pair_sum_forward")
        ctx.save_for_backward(x1c, x2c)
        ctx.metric, ctx.unbatched, ctx.in_dtype = metric, unbatched, in_dtype
        return (out.squeeze(0) if unbatched else out).to(in_dtype)

    @staticmethod
    def backward(ctx, grad):
        x1c, x2c = ctx.saved_tensors
        g = grad.to(x1c.dtype).contiguous()
        if ctx.unbatched:
            g = g.unsqueeze(0)
        B, N1, N2, D = _sizes(x1c, x2c)
        need1, need2 = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        g1 = torch.empty_like(x1c) if need1 else None
        g2 = torch.empty_like(x2c) if need2 else None
        with torch.cuda.device(x1c.device):
            check(lib.tpw_pair_sum_backward(_FLOAT_CODES[x1c.dtype], ctx.metric, _ptr(g), _ptr(x1c), _ptr(x2c), _ptr(g1), _ptr(g2),
                                            B, N1, N2, D, _stream(x1c)), "tpw_pair_sum_backward")
        if ctx.unbatched:
            g1 = None if g1 is None else g1.squeeze(0)
            g2 = None if g2 is None else g2.squeeze(0)
        return (None if g1 is None else g1.to(ctx.in_dtype)), (None if g2 is None else g2.to(ctx.in_dtype)), None


def canberra_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    """sum_k |x1 - x2| / (|x1| + |x2|) (OPS/pairwise_metrics.cpp:317-324)."""
    x1_, x2_ = check_pairwise_inputs("canberra_distances", x1, x2)
    _require_cuda(x1_, x2_)
    return _PairSumFunction.apply(x1_, x2_, _abi.PAIR_CANBERRA)


def _require_non_negative(x1: Tensor, x2: Optional[Tensor], x2_: Tensor) -> None:
    # the reference's check (and message), OPS/pairwise_metrics.cpp:130-131; it synchronises there too
    if not (bool(x1.ge(0).all()) and (x2 is None or bool(x2_.ge(0).all()))):
        raise RuntimeError("All elements of x1 and x2 must be positive")


def additive_chi2_kernel(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    """- sum_k (x1 - x2)^2 / (x1 + x2) on non-negative inputs (OPS/pairwise_metrics.cpp:124-133)."""
    x1_, x2_ = check_pairwise_inputs("additive_chi2_kernel", x1, x2)
    _require_cuda(x1_, x2_)
    _require_non_negative(x1_, x2, x2_)
    return _PairSumFunction.apply(x1_, x2_, _abi.PAIR_ADDITIVE_CHI2)


def chi2_kernel(x1: Tensor, x2: Optional[Tensor] = None, gamma: float = 1.0) -> Tensor:
    """exp(gamma * additive_chi2_kernel(x1, x2)) (OPS/pairwise_metrics.cpp:135-145)."""
    return (additive_chi2_kernel(x1, x2) * gamma).exp()


class _JensenShannonFunction(torch.autograd.Function):
    """f(scale * sum_k (x1 log(x1/m) + x2 log(x2/m))), m = (x1 + x2)/2, with f the identity (_sqjensenshannon,
    OPS/autograd/sqjensenshannon_kernel.cpp, kernels OPS/cpu/sqjensenshannon_kernel.cpp:13-141) or the square
    root that jensenshannon_distances applies in place (OPS/pairwise_metrics.cpp:336), fused into the tile's
    epilogue.  Where the rooted output is 0 the backward contributes 0 (the reference's sqrt backward divides
    by it)."""

    @staticmethod
    def forward(ctx, x1: Tensor, x2: Tensor, scale: float, take_sqrt: bool):
        in_dtype = x1.dtype
        cdt = _compute_dtype(in_dtype)
        x1c, x2c, unbatched = _batched(x1.to(cdt), x2.to(cdt), "_sqjensenshannon")
        B, N1, N2, D = _sizes(x1c, x2c)
        out = torch.empty((B, N1, N2), dtype=cdt, device=x1c.device)
        if D == 0:
            out.zero_()
        else:
            with torch.cuda.device(x1c.device):
                check(lib.tpw_jensenshannon_forward(_FLOAT_CODES[cdt], _ptr(x1c), _ptr(x2c), _ptr(out), B, N1, N2, D,
                                                    float(scale), int(take_sqrt), _stream(x1c)), "tpw_jensenshannon_forward")
        ctx.save_for_backward(x1c, x2c, out if take_sqrt else None)
        ctx.scale, ctx.unbatched, ctx.in_dtype = float(scale), unbatched, in_dtype
        return (out.squeeze(0) if unbatched else out).to(in_dtype)

    @staticmethod
    def backward(ctx, grad):
        x1c, x2c, out = ctx.saved_tensors
        g = grad.to(x1c.dtype).contiguous()
        if ctx.unbatched:
            g = g.unsqueeze(0)
        B, N1, N2, D = _sizes(x1c, x2c)
        need1, need2 = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        g1 = torch.empty_like(x1c) if need1 else None
        g2 = torch.empty_like(x2c) if need2 else None
        if need1 or need2:
            with torch.cuda.device(x1c.device):
                check(lib.tpw_jensenshannon_backward(_FLOAT_CODES[x1c.dtype], _ptr(g), _ptr(out), _ptr(x1c), _ptr(x2c),
                                                     _ptr(g1), _ptr(g2), B, N1, N2, D, ctx.scale, _stream(x1c)),
                      "tpw_jensenshannon_backward")
        if ctx.unbatched:
            g1 = None if g1 is None else g1.squeeze(0)
            g2 = None if g2 is None else g2.squeeze(0)
        return (None if g1 is None else g1.to(ctx.in_dtype)), (None if g2 is None else g2.to(ctx.in_dtype)), None, None


def _js_scale(base: Optional[float]) -> float:
    # output.div_(2 log(base)), or 2 without a base (OPS/cpu/sqjensenshannon_kernel.cpp:75)
    return 0.5 if base is None else 0.5 / math.log(base)


def _sqjensenshannon(x1: Tensor, x2: Tensor, base: Optional[float] = None) -> Tensor:
    """Squared Jensen-Shannon distance of rows that already sum to one (OPS/sqjensenshannon.cpp)."""
    _require_cuda(x1, x2)
    return _JensenShannonFunction.apply(x1, x2, _js_scale(base), False)


def jensenshannon_distances(x1: Tensor, x2: Optional[Tensor] = None, base: Optional[float] = None) -> Tensor:
    """sqrt(_sqjensenshannon(x1 / sum x1, x2 / sum x2, base)) (OPS/pairwise_metrics.cpp:326-337): the rows are
    normalised with plain tensor operations (differentiable), the sum and the root run in one kernel."""
    x1_, x2_ = check_pairwise_inputs("jensenshannon_distances", x1, x2)
    _require_cuda(x1_, x2_)
    n1 = x1_ / x1_.sum(-1, keepdim=True)
    n2 = n1 if x2 is None else x2_ / x2_.sum(-1, keepdim=True)
    return _JensenShannonFunction.apply(n1, n2, _js_scale(base), True)


class _HaversineFunction(torch.autograd.Function):
    """_haversine and its backward (OPS/autograd/haversine_kernel.cpp, kernels OPS/cpu/haversine_kernel.cpp:12-217):
    rows are (latitude, longitude) in radians.  Coincident or antipodal pairs contribute no gradient (the
    reference divides by a zero denominator there)."""

    @staticmethod
    def forward(ctx, x1: Tensor, x2: Tensor):
        in_dtype = x1.dtype
        cdt = _compute_dtype(in_dtype)
        x1c, x2c, unbatched = _batched(x1.to(cdt), x2.to(cdt), "_haversine")
        B, N1, N2, D = _sizes(x1c, x2c)
        if D != 2:
            raise RuntimeError("feature dimension of x1 and x2 must be 2.")
        out = torch.empty((B, N1, N2), dtype=cdt, device=x1c.device)
        with torch.cuda.device(x1c.device):
            check(lib.tpw_haversine_forward(_FLOAT_CODES[cdt], _ptr(x1c), _ptr(x2c), _ptr(out), B, N1, N2, _stream(x1c)),
                  "tpw_haversine_forward")
        ctx.save_for_backward(x1c, x2c)
        ctx.unbatched, ctx.in_dtype = unbatched, in_dtype
        return (out.squeeze(0) if unbatched else out).to(in_dtype)

    @staticmethod
    def backward(ctx, grad):
        x1c, x2c = ctx.saved_tensors
        g = grad.to(x1c.dtype).contiguous()
        if ctx.unbatched:
            g = g.unsqueeze(0)
        B, N1, N2, _ = _sizes(x1c, x2c)
        g1 = torch.empty_like(x1c) if ctx.needs_input_grad[0] else None
        g2 = torch.empty_like(x2c) if ctx.needs_input_grad[1] else None
        if g1 is not None or g2 is not None:
            with torch.cuda.device(x1c.device):
                check(lib.tpw_haversine_backward(_FLOAT_CODES[x1c.dtype], _ptr(g), _ptr(x1c), _ptr(x2c), _ptr(g1), _ptr(g2),
                                                 B, N1, N2, _stream(x1c)), "tpw_haversine_backward")
        if ctx.unbatched:
            g1 = None if g1 is None else g1.squeeze(0)
            g2 = None if g2 is None else g2.squeeze(0)
        return (None if g1 is None else g1.to(ctx.in_dtype)), (None if g2 is None else g2.to(ctx.in_dtype))


def _haversine(x1: Tensor, x2: Tensor) -> Tensor:
    _require_cuda(x1, x2)
    return _HaversineFunction.apply(x1, x2)


def haversine_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    """Great-circle distance on the unit sphere between (latitude, longitude) rows in radians
    (OPS/pairwise_metrics.cpp:33-40)."""
    x1_, x2_ = check_pairwise_inputs("haversine_distances", x1, x2)
    return _haversine(x1_, x2_)


def braycurtis_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    """sum_k |x1 - x2| / sum_k |x1 + x2| (the reference's own kernel, OPS/cpu/braycurtis_kernel.cpp:22-27,
    called at OPS/pairwise_metrics.cpp:308-315): two passes of the L1 tile kernel, the second against
    -x2, and a plain division (0/0 is NaN as in the reference); differentiable through both passes."""
    x1_, x2_ = check_pairwise_inputs("braycurtis_distances", x1, x2)
    _require_cuda(x1_, x2_)
    return _cdist_p(x1_, x2_, 1.0) / _cdist_p(x1_, -x2_, 1.0)


def snr_distances(x1: Tensor, x2: Optional[Tensor] = None) -> Tensor:
    """1 / _snr = sum_k (e_k - mean e)^2 / sum_k (x1_k - mean x1)^2 with e = x2 - x1 (OPS/pairwise_metrics.cpp:401-408,
    OPS/cpu/snr_kernel.cpp:22-34,96).  The deviations of e from its mean are the differences of the centred rows, so
    the numerator is the squared Euclidean distance of the centred rows, taken by the direct-difference kernel: a row
    against itself gives exactly 0 and near-duplicate rows keep their relative accuracy."""
    x1_, x2_ = check_pairwise_inputs("snr_distances", x1, x2)
    _require_cuda(x1_, x2_)
    c1 = x1_ - x1_.mean(-1, keepdim=True)
    c2 = c1 if x2 is None else x2_ - x2_.mean(-1, keepdim=True)
    return _ppminkowski(c1, c2, 2.0) / c1.pow(2).sum(-1, keepdim=True)


def _sqmahalanobis(x1: Tensor, x2: Tensor, VI: Tensor) -> Tensor:
    """(x1 - x2) VI (x1 - x2)^T per pair (OPS/sqmahalanobis.cpp:31-38, OPS/cpu/sqmahalanobis_kernel.cpp:23-31), from
    direct differences.  The form depends on the symmetric part S of VI only.  Where S is positive definite (every
    inverse covariance is) S = L L^T and the form is the squared Euclidean distance of x1 L and x2 L: a sum of
    squares, exactly 0 for a row against itself and accurate for near-duplicate rows.  Otherwise d.e with
    d = x1 - x2, e = d S is taken as (|d/c + c e|^2 - |d/c - c e|^2) / 4, two more direct-difference kernels
    (c balances the two magnitudes).  Differentiable in x1, x2 and VI through both."""
    _require_cuda(x1, x2, VI)
    if not (x1.dtype == x2.dtype == VI.dtype):
        raise RuntimeError("x1, x2 and VI must have the same dtype (while checking arguments for _sqmahalanobis_forward)")
    if x1.dim() not in (2, 3) or x2.dim() != x1.dim() or VI.dim() != x1.dim():
        raise RuntimeError("x1, x2 and VI must all be 2-D (unbatched) or 3-D (batched) tensors.")
    if x1.size(-1) != x2.size(-1) or x1.size(-1) != VI.size(-2) or VI.size(-1) != VI.size(-2):
        raise RuntimeError("feature dimension of x1, x2, and VI do not match.")
    same = x2 is x1
    S = (VI + VI.transpose(-1, -2)) * 0.5
    L, info = torch.linalg.cholesky_ex(S)
    if x1.size(-1) > 0 and bool((info == 0).all()):
        u1 = x1 @ L
        return _ppminkowski(u1, u1 if same else x2 @ L, 2.0)
    e1 = x1 @ S
    e2 = e1 if same else x2 @ S
    with torch.no_grad():
        nx, ne = float(x1.norm()), float(e1.norm())
    c = math.sqrt(nx / ne) if nx > 0 and ne > 0 and math.isfinite(nx / ne) else 1.0
    p1, m1 = x1 / c + e1 * c, x1 / c - e1 * c
    p2, m2 = (p1, m1) if same else (x2 / c + e2 * c, x2 / c - e2 * c)
    return (_ppminkowski(p1, p2, 2.0) - _ppminkowski(m1, m2, 2.0)) * 0.25


def mahalanobis_distances(x1: Tensor, x2: Optional[Tensor] = None, VI: Optional[Tensor] = None) -> Tensor:
    """sqrt((x1 - x2) VI (x1 - x2)^T) (OPS/pairwise_metrics.cpp:272-297); VI defaults to the transposed inverse
    covariance of x1 (no gradient), as there.  See ``_sqmahalanobis`` for how the form is evaluated."""
    if x2 is not None and VI is None:
        raise RuntimeError("VI is required for manhalanobis when x2 is passed.")
    x1_, x2_ = check_pairwise_inputs("mahalanobis_distances", x1, x2)
    _require_cuda(x1_, x2_)
    if VI is None:
        with torch.no_grad():
            VI = torch.linalg.inv(torch.cov(x1_.transpose(-1, -2)) if x1_.dim() == 2 else
                                  torch.stack([torch.cov(xb.transpose(-1, -2)) for xb in x1_])).transpose(-1, -2)
    return _sqmahalanobis(x1_, x2_, VI).sqrt()


def _validate_metric_kwargs(metric: str, kwargs: dict) -> None:
    """The keyword check ``cdist`` applies (OPS/cpdist.cpp:35-79), run before any fused kernel is chosen so that a call
    raises or does not raise whatever the problem size: an unknown metric is a RuntimeError, a keyword the metric
    does not take a TypeError."""
    from .cpdist import SUPPORTED_METRICS, _check_extra_args
    if metric not in SUPPORTED_METRICS:
        raise RuntimeError(f"Got unkown distance metric: {metric}. Supported metrics are [{', '.join(SUPPORTED_METRICS)}]")
    unknown = set(kwargs) - {"w", "V", "VI", "p", "base", "shuffle", "generator"}
    if unknown:
        raise TypeError(f"unexpected keyword argument(s): {', '.join(sorted(unknown))}")
    _check_extra_args(metric, **kwargs)


def radius_neighbors_mask(x1: Tensor, x2: Optional[Tensor] = None, epsilon: float = 0.0, metric: str = "euclidean",
                          **kwargs) -> Tensor:
    """cdist(x1, x2, metric) <= epsilon (OPS/neighbors.cpp:37-58)."""
    from .cpdist import cdist
    x1_, x2_ = check_pairwise_inputs("radius_neighbors_mask", x1, x2)
    if epsilon < 0:
        raise RuntimeError(f"epsilon must be non-negative. Got epsilon={epsilon}")
    _validate_metric_kwargs(metric, kwargs)
    with torch.no_grad():
        if metric in _ROWMIN_METRICS and x1_.is_cuda and set(kwargs) <= {"p"} and x1_.dtype == x2_.dtype \
                and x1_.dtype in _FLOAT_CODES and x1_.size(-1) > 0:
            pp, ex = _ROWMIN_METRICS[metric]
            if pp is None:
                pp = 2.0 if kwargs.get("p") is None else float(kwargs["p"])
                ex = 1.0 if math.isinf(pp) else (1.0 / pp if pp > 0 else None)
            x1c, x2c, unbatched = _batched(x1_, x2_, "radius_neighbors_mask")
            # p = 2 on a large float32 problem is faster as a tensor-core contraction plus a compare pass
            if ex is not None and pp > 0 and not (pp == 2.0 and _tensor_engine_selected(x1c, x2c)):
                B, N1, N2, D = _sizes(x1c, x2c)
                mask = torch.empty((B, N1, N2), dtype=torch.bool, device=x1c.device)
                with torch.cuda.device(x1c.device):
                    check(lib.tpw_lp_radius_mask_forward(_FLOAT_CODES[x1c.dtype], _ptr(x1c), _ptr(x2c), None, _ptr(mask),
                                                         B, N1, N2, D, pp, ex, float(epsilon), _stream(x1c)),
                          "tpw_lp_radius_mask_forward")
                return mask.squeeze(0) if unbatched else mask
        return cdist(x1_, x2_, metric, **kwargs) <= epsilon


def k_neighbors_mask(x1: Tensor, x2: Optional[Tensor] = None, k: int = 1, metric: str = "euclidean", **kwargs) -> Tensor:
    """True at the k + 1 smallest distances of every row (OPS/neighbors.cpp:10-35; the reference keeps
    k + 1 columns, i.e. the point itself plus k neighbours when x2 is x1; unbatched inputs)."""
    from .cpdist import cdist
    x1_, x2_ = check_pairwise_inputs("k_neighbors_mask", x1, x2)
    if k < 0:
        raise RuntimeError(f"k must be non-negative. Got k={k}")
    _validate_metric_kwargs(metric, kwargs)
    with torch.no_grad():
        if (k == 0 and metric in _ROWMIN_METRICS and x1_.dtype == torch.float32 and x2_.dtype == torch.float32
                and x1_.is_cuda and x2_.size(0) > 0 and set(kwargs) <= {"p"}):
            # one column per row: the streaming row minimum, no distance matrix and no sort
            inds = pairwise_argmin_min(x1_, x2_, metric, kwargs.get("p"))[0].unsqueeze(1)
            out = torch.zeros((x1_.size(0), x2_.size(0)), dtype=torch.bool, device=x1_.device)
            return out.scatter_(1, inds, True)
        few = (metric in _ROWMIN_METRICS and set(kwargs) <= {"p"} and kwargs.get("p") in (None, 1.0, 2.0, 3.0, math.inf)
               and x1_.is_cuda and x1_.dtype == torch.float32 and x2_.dtype == torch.float32 and x1_.dim() == 2
               and 0 < x1_.size(-1) <= lib.tpw_lp_topk_max_features() and x1_.size(0) >= 4096
               and 0 < k + 1 <= min(lib.tpw_lp_topk_max_k(), x2_.size(0)) and not os.environ.get("TPW_DISABLE_SMALL_D"))
        if few:
            inds = pairwise_argkmin(x1_, x2_, k + 1, metric, **kwargs)[0]
            out = torch.zeros((x1_.size(0), x2_.size(0)), dtype=torch.bool, device=x1_.device)
            return out.scatter_(1, inds, True)
        if metric in ("euclidean", "l2", "sqeuclidean", "cosine") and not kwargs and x1_.is_cuda and x1_.dtype == torch.float32 \
                and x2_.dtype == torch.float32 and 0 < k + 1 <= min(lib.tpw_dot_topk_max_k(), x2_.size(0)) \
                and _tensor_engine_selected(x1_.unsqueeze(0), x2_.unsqueeze(0)):
            # large problem: the k + 1 nearest rows straight from the tensor-core epilogue, no distance matrix
            inds = pairwise_argkmin(x1_, x2_, k + 1, metric)[0]
            out = torch.zeros((x1_.size(0), x2_.size(0)), dtype=torch.bool, device=x1_.device)
            return out.scatter_(1, inds, True)
        dists = cdist(x1_, x2_, metric, **kwargs)
        # the k + 1 smallest of every row: a partial selection, not the reference's full argsort of each row
        inds = dists.topk(min(k + 1, dists.size(1)), dim=1, largest=False, sorted=False).indices
        out = torch.zeros((x1_.size(0), x2_.size(0)), dtype=torch.bool, device=x1_.device)
        out.scatter_(1, inds, True)
        return out


_ROWMIN_METRICS = {
    # metric -> (p, out_exponent); None = taken from the `p` argument
    "euclidean": (2.0, 0.5), "l2": (2.0, 0.5),
    "sqeuclidean": (2.0, 1.0),
    "manhattan": (1.0, 1.0), "cityblock": (1.0, 1.0), "l1": (1.0, 1.0),
    "chebyshev": (math.inf, 1.0), "linf": (math.inf, 1.0),
    "minkowski": (None, None), "lp": (None, None),
}
# served by the matrix kernel + Tensor.min, or by the tensor-core row-minimum epilogue on large problems
_ROWMIN_DOT_METRICS = {"cosine": _abi.DOT_COSINE_DIST}


def pairwise_argmin_min(x1: Tensor, x2: Optional[Tensor] = None, metric: str = "euclidean",
                        p: Optional[float] = None) -> Tuple[Tensor, Tensor]:
    """For every x1 row, the x2 row at the smallest distance and that distance:
    ``(argmin [.., N1] int64, min [.., N1])``, ties to the smaller index, no gradient.

    float32 inputs stream through the L_p tile kernel, whose epilogue folds each tile into one
    64-bit key per row (warp shuffles, then atomicMin) so the [N1, N2] matrix is never written;
    the values equal ``minkowski_distances(...).min(-1)``. The reference has no such operator: it
    sorts whole rows of the materialised matrix (k_neighbors_mask, OPS/neighbors.cpp:10-35).
    Other floating dtypes take this package's distance kernel followed by ``Tensor.min``.
    """
    if metric in _ROWMIN_DOT_METRICS:
        x1_, x2_ = check_pairwise_inputs("pairwise_argmin_min", x1, x2)
        _require_cuda(x1_, x2_)
        with torch.no_grad():
            x1c, x2c, unbatched = _batched(x1_, x2_, "pairwise_argmin_min")
            B, N1, N2, D = _sizes(x1c, x2c)
            if N2 == 0:
                raise RuntimeError("pairwise_argmin_min: x2 has no rows")
            if x1c.dtype == torch.float32 and D > 0 and _tensor_engine_selected(x1c, x2c):
                mins = torch.empty((B, N1), dtype=torch.float32, device=x1c.device)
                args = torch.empty((B, N1), dtype=torch.int64, device=x1c.device)
                nbytes = lib.tpw_dot_rowmin_scratch_bytes(B, N1, N2, D)
                scratch = torch.empty((nbytes,), dtype=torch.uint8, device=x1c.device)
                with torch.cuda.device(x1c.device):
                    check(lib.tpw_dot_rowmin_forward_ws(_ROWMIN_DOT_METRICS[metric], _ptr(x1c), _ptr(x2c), _ptr(mins), _ptr(args),
                                                        _ptr(scratch), nbytes, B, N1, N2, D, _stream(x1c)), "tpw_dot_rowmin_forward_ws")
            else:
                mins, args = cosine_distances(x1c, x2c).min(dim=-1)
            if unbatched:
                mins, args = mins.squeeze(0), args.squeeze(0)
            return args, mins
    if metric not in _ROWMIN_METRICS:
        raise ValueError(f"pairwise_argmin_min supports {sorted(set(_ROWMIN_METRICS) | set(_ROWMIN_DOT_METRICS))}; got {metric!r}")
    pp, ex = _ROWMIN_METRICS[metric]
    if pp is None:
        pp = 2.0 if p is None else float(p)
        if not pp > 0:
            raise RuntimeError(f"p must be positive. Got p={pp}")
        ex = 1.0 if math.isinf(pp) else 1.0 / pp
    x1_, x2_ = check_pairwise_inputs("pairwise_argmin_min", x1, x2)
    _require_cuda(x1_, x2_)
    with torch.no_grad():
        x1c, x2c, unbatched = _batched(x1_, x2_, "pairwise_argmin_min")
        B, N1, N2, D = _sizes(x1c, x2c)
        if N2 == 0:
            raise RuntimeError("pairwise_argmin_min: x2 has no rows")
        if x1c.dtype != torch.float32 or D == 0:
            dist = _lp_forward_raw(x1c.to(_compute_dtype(x1c.dtype)), x2c.to(_compute_dtype(x2c.dtype)), None, pp, ex)
            mins, args = dist.min(dim=-1)
            mins = mins.to(x1c.dtype)
        elif pp == 2.0 and _tensor_engine_selected(x1c, x2c):
            # large float32 problem: the contraction form on the tensor cores with the row minimum taken in
            # the epilogue (bf16 x 3 rounding: candidates closer than ~1e-5 of the norms may swap)
            mins = torch.empty((B, N1), dtype=torch.float32, device=x1c.device)
            args = torch.empty((B, N1), dtype=torch.int64, device=x1c.device)
            nbytes = lib.tpw_dot_rowmin_scratch_bytes(B, N1, N2, D)
            scratch = torch.empty((nbytes,), dtype=torch.uint8, device=x1c.device)
            with torch.cuda.device(x1c.device):
                check(lib.tpw_dot_rowmin_forward_ws(_abi.DOT_EUCLIDEAN if ex == 0.5 else _abi.DOT_SQEUCLIDEAN, _ptr(x1c), _ptr(x2c),
                                                    _ptr(mins), _ptr(args), _ptr(scratch), nbytes, B, N1, N2, D, _stream(x1c)),
                      "tpw_dot_rowmin_forward_ws")
        else:
            mins = torch.empty((B, N1), dtype=torch.float32, device=x1c.device)
            args = torch.empty((B, N1), dtype=torch.int64, device=x1c.device)
            nbytes = lib.tpw_lp_rowmin_scratch_bytes(B, N1)
            scratch = torch.empty((max(nbytes, 8) // 8,), dtype=torch.int64, device=x1c.device)
            with torch.cuda.device(x1c.device):
                check(lib.tpw_lp_rowmin_forward(_abi.F32, _ptr(x1c), _ptr(x2c), None, _ptr(mins), _ptr(args),
                                                _ptr(scratch), B, N1, N2, D, pp, ex, _stream(x1c)),
                      "tpw_lp_rowmin_forward")
        if unbatched:
            mins, args = mins.squeeze(0), args.squeeze(0)
        return args, mins


def pairwise_argkmin(x1: Tensor, x2: Optional[Tensor] = None, k: int = 1, metric: str = "euclidean",
                     **kwargs) -> Tuple[Tensor, Tensor]:
    """The k nearest x2 rows of every x1 row: ``(indices [.., N1, k] int64, distances [.., N1, k])``,
    ascending by distance, no gradient.  The reference's README lists ``argkmin`` as future work; its
    ``k_neighbors_mask`` sorts every row of the materialised matrix (OPS/neighbors.cpp:10-35).

    Large float32 problems with a Euclidean, squared Euclidean or cosine metric and
    ``k <= tpw_dot_topk_max_k()`` run the tensor-core kernel whose epilogue keeps the k smallest keys
    of each accumulator row in registers (``tpw_dot_topk_forward_ws``; no distance matrix is written).
    float32 L_p metrics (p in 1, 2, 3, inf) on at most ``tpw_lp_topk_max_features()`` features and at least 4096
    query rows run the streaming kernel that keeps one query row and its k best keys per thread
    (``tpw_lp_topk_forward``).  Everything else takes this package's distance kernel followed by a partial selection."""
    from .cpdist import cdist
    if k < 1:
        raise RuntimeError(f"k must be positive. Got k={k}")
    x1_, x2_ = check_pairwise_inputs("pairwise_argkmin", x1, x2)
    _require_cuda(x1_, x2_)
    _validate_metric_kwargs(metric, kwargs)
    if k > x2_.size(-2):
        raise RuntimeError(f"k={k} exceeds the number of x2 rows ({x2_.size(-2)})")
    epilogue = {"euclidean": _abi.DOT_EUCLIDEAN, "l2": _abi.DOT_EUCLIDEAN, "sqeuclidean": _abi.DOT_SQEUCLIDEAN,
                "cosine": _abi.DOT_COSINE_DIST}.get(metric)
    with torch.no_grad():
        if epilogue is not None and not kwargs and x1_.dtype == torch.float32 and x2_.dtype == torch.float32 \
                and x1_.size(-1) > 0 and k <= lib.tpw_dot_topk_max_k():
            x1c, x2c, unbatched = _batched(x1_, x2_, "pairwise_argkmin")
            if _tensor_engine_selected(x1c, x2c):
                B, N1, N2, D = _sizes(x1c, x2c)
                vals = torch.empty((B, N1, k), dtype=torch.float32, device=x1c.device)
                inds = torch.empty((B, N1, k), dtype=torch.int64, device=x1c.device)
                nbytes = lib.tpw_dot_topk_scratch_bytes(k, B, N1, N2, D)
                scratch = torch.empty((nbytes,), dtype=torch.uint8, device=x1c.device)
                with torch.cuda.device(x1c.device):
                    check(lib.tpw_dot_topk_forward_ws(epilogue, k, _ptr(x1c), _ptr(x2c), _ptr(vals), _ptr(inds), _ptr(scratch), nbytes,
                                                      B, N1, N2, D, _stream(x1c)), "tpw_dot_topk_forward_ws")
                return (inds.squeeze(0), vals.squeeze(0)) if unbatched else (inds, vals)
        # few features (point clouds): one x1 row per thread with its k best keys in registers, no distance matrix
        if (metric in _ROWMIN_METRICS and set(kwargs) <= {"p"} and x1_.dtype == torch.float32 and x2_.dtype == torch.float32
                and 0 < x1_.size(-1) <= lib.tpw_lp_topk_max_features() and k <= lib.tpw_lp_topk_max_k()
                and not os.environ.get("TPW_DISABLE_SMALL_D")):
            pp, ex = _ROWMIN_METRICS[metric]
            if pp is None:
                pp = 2.0 if kwargs.get("p") is None else float(kwargs["p"])
                ex = 1.0 if math.isinf(pp) else (1.0 / pp if pp > 0 else None)
            x1c, x2c, unbatched = _batched(x1_, x2_, "pairwise_argkmin")
            B, N1, N2, D = _sizes(x1c, x2c)
            if pp in (1.0, 2.0, 3.0, math.inf) and ex is not None and B * N1 >= 4096:
                vals = torch.empty((B, N1, k), dtype=torch.float32, device=x1c.device)
                inds = torch.empty((B, N1, k), dtype=torch.int64, device=x1c.device)
                with torch.cuda.device(x1c.device):
                    check(lib.tpw_lp_topk_forward(_abi.F32, _ptr(x1c), _ptr(x2c), _ptr(vals), _ptr(inds), B, N1, N2, D, k, pp, ex,
                                                  _stream(x1c)), "tpw_lp_topk_forward")
                return (inds.squeeze(0), vals.squeeze(0)) if unbatched else (inds, vals)
        dist = cdist(x1_, x2_, metric, **kwargs)
        vals, inds = dist.topk(k, dim=-1, largest=False, sorted=True)
        return inds, vals
