"""ctypes binding of ``libtpw_b200.so`` (declared in ``include/tpw_b200.h``).

The library is the product path: there is no CPU or eager-PyTorch fallback.  If the shared
object is missing the import of :data:`lib` fails loudly and tells the caller how to build it.
"""
from __future__ import annotations

import ctypes
import math
import os
from ctypes import c_char_p, c_double, c_int, c_int64, c_void_p, POINTER
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libtpw_b200.so"

# enums of include/tpw_b200.h
TPW_OK = 0
F32, F64, I32, I64 = 0, 1, 2, 3
LP_BWD_CDIST, LP_BWD_PPMINKOWSKI, LP_BWD_WMINKOWSKI, LP_BWD_MATMUL = 0, 1, 2, 3
DOT_LINEAR, DOT_COSINE_SIM, DOT_COSINE_DIST, DOT_ONE_MINUS_SIM, DOT_SQEUCLIDEAN, DOT_EUCLIDEAN = range(6)
PAIR_CANBERRA, PAIR_ADDITIVE_CHI2 = 0, 1
ENGINE_AUTO, ENGINE_SIMT_FP32, ENGINE_TCGEN05_BF16X3, ENGINE_TCGEN05_TF32X3 = 0, 1, 2, 3
CMP_EQ, CMP_NE = 0, 1
RED_SUM, RED_MEAN = 0, 1
PRF_ZERO, PRF_IDENTITY = 0, 1
BOOL_METRICS = {
    "and_sum": 0, "or_sum": 1, "xor_sum": 2, "eq_sum": 3, "ne_sum": 4, "eq_mean": 5, "ne_mean": 6,
    "jaccard": 7, "kulsinski": 8, "kulczynski1": 9, "yule": 10, "dice": 11, "rogerstanimoto": 12,
    "russellrao": 13, "sokalmichener": 14, "sokalsneath": 15,
}

# name -> (restype, argtypes); kept in one table so that tests can check the export list
# against the header.
_P, _I, _L, _D = c_void_p, c_int, c_int64, c_double
SIGNATURES = {
    "tpw_abi_version": (_I, []),
    "tpw_cuda_version": (_I, []),
    "tpw_cuda_arch_flags": (c_char_p, []),
    "tpw_last_error": (c_char_p, []),
    "tpw_device_status": (_I, [POINTER(c_int), _P]),
    "tpw_selftest_bounded_wait": (_I, [_I, _P]),
    "tpw_lp_forward": (_I, [_I, _P, _P, _P, _P, _L, _L, _L, _L, _D, _D, _P]),
    "tpw_lp_rowmin_scratch_bytes": (_L, [_L, _L]),
    "tpw_lp_rowmin_forward": (_I, [_I, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _D, _D, _P]),
    "tpw_lp_topk_max_features": (_I, []),
    "tpw_lp_topk_max_k": (_I, []),
    "tpw_lp_topk_forward": (_I, [_I, _P, _P, _P, _P, _L, _L, _L, _L, _I, _D, _D, _P]),
    "tpw_lp_radius_mask_forward": (_I, [_I, _P, _P, _P, _P, _L, _L, _L, _L, _D, _D, _D, _P]),
    "tpw_lp_pdist_forward": (_I, [_I, _P, _P, _L, _L, _L, _D, _D, _P]),
    "tpw_pair_sum_forward": (_I, [_I, _I, _P, _P, _P, _L, _L, _L, _L, _P]),
    "tpw_pair_sum_backward": (_I, [_I, _I, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P]),
    "tpw_haversine_forward": (_I, [_I, _P, _P, _P, _L, _L, _L, _P]),
    "tpw_haversine_backward": (_I, [_I, _P, _P, _P, _P, _P, _L, _L, _L, _P]),
    "tpw_jensenshannon_forward": (_I, [_I, _P, _P, _P, _L, _L, _L, _L, _D, _I, _P]),
    "tpw_jensenshannon_backward": (_I, [_I, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _D, _P]),
    "tpw_lp_backward": (_I, [_I, _I, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _D, _P]),
    "tpw_lp_backward_scratch_bytes": (_L, [_I, _I, _L, _L, _L, _L, _D]),
    "tpw_lp_backward_ws": (_I, [_I, _I, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _D, _P, _L, _P]),
    "tpw_chebyshev_backward_scratch_bytes": (_L, [_I, _L, _L, _L, _L]),
    "tpw_chebyshev_backward_ws": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P]),
    "tpw_wminkowski_backward_w": (_I, [_I, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _D, _P]),
    "tpw_lp_inf_backward": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _P]),
    "tpw_dot_metric_forward": (_I, [_I, _I, _I, _P, _P, _P, _L, _L, _L, _L, _P]),
    "tpw_dot_metric_scratch_bytes": (_L, [_I, _I, _L, _L, _L, _L]),
    "tpw_dot_rowmin_scratch_bytes": (_L, [_L, _L, _L, _L]),
    "tpw_dot_rowmin_forward_ws": (_I, [_I, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P]),
    "tpw_dot_topk_max_k": (_I, []),
    "tpw_dot_topk_scratch_bytes": (_L, [_L, _L, _L, _L, _L]),
    "tpw_dot_topk_forward_ws": (_I, [_I, _I, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P]),
    "tpw_dot_backward_scratch_bytes": (_L, [_I, _I, _I, _L, _L, _L, _L]),
    "tpw_dot_backward_ws": (_I, [_I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P]),
    "tpw_cosine_backward_ws": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P]),
    "tpw_dot_metric_forward_ws": (_I, [_I, _I, _I, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P]),
    "tpw_row_center": (_I, [_I, _P, _P, _L, _L, _P]),
    "tpw_row_norm": (_I, [_I, _P, _P, _L, _L, _P]),
    "tpw_cosine_backward_prepare": (_I, [_I, _I, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _P]),
    "tpw_cosine_backward_finish": (_I, [_I, _P, _P, _P, _P, _L, _L, _P]),
    "tpw_bitpack": (_I, [_P, _P, _P, _L, _L, _L, _P]),
    "tpw_bool_metric_forward": (_I, [_I, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P]),
    "tpw_bool_metric_tc_eligible": (_I, [_L, _L, _L, _L]),
    "tpw_bool_metric_forward_tc": (_I, [_I, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P]),
    "tpw_cmp_reduce_forward": (_I, [_I, _I, _I, _P, _P, _P, _L, _L, _L, _L, _P]),
    "tpw_hausdorff_scratch_bytes": (_L, [_L, _L, _L, _L]),
    "tpw_hausdorff_forward": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P]),
    "tpw_hausdorff_backward": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P]),
    "tpw_hausdorff_static_max_pairs": (_L, []),
    "tpw_hausdorff_forward_static": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P]),
    "tpw_prf_div_forward": (_I, [_I, _I, _P, _P, _P, _L, _P]),
    "tpw_prf_div_backward": (_I, [_I, _I, _P, _P, _P, _P, _P, _L, _P]),
    "tpw_measure_issue_peak": (_I, [_I, POINTER(c_double)]),
}


class TpwError(RuntimeError):
    """A C-ABI call returned a non-zero tpw_status."""


def _load() -> ctypes.CDLL:
    path = Path(os.environ.get("TPW_B200_LIB", LIB_PATH))
    if not path.exists():
        raise ImportError(
            f"{path} is missing: the CUDA kernel library has not been built. "
            "Run `python torchpairwise_b200/build.py` (needs nvcc); there is no CPU fallback."
        )
    handle = ctypes.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
    return handle


lib = _load()


def check(status: int, what: str = "") -> None:
    """Raise :class:`TpwError` with the library's message unless ``status`` is TPW_OK."""
    if status != TPW_OK:
        msg = lib.tpw_last_error().decode(errors="replace")
        raise TpwError(f"{what or 'tpw call'} failed with status {status}: {msg}")


def device_status(stream_ptr: int = 0) -> int:
    """Synchronise ``stream`` and return (then clear) the device status word; 0 means no kernel
    gave up a bounded wait."""
    code = c_int(0)
    check(lib.tpw_device_status(ctypes.byref(code), c_void_p(stream_ptr)), "tpw_device_status")
    return code.value


def measure_issue_peak(kind: int) -> float:
    """Operations per second of the register-only microbenchmark ``kind`` (0 scalar FFMA, 1 packed
    f32x2 FMA, 2 POPC) on the current device."""
    out = c_double(0.0)
    check(lib.tpw_measure_issue_peak(kind, ctypes.byref(out)), "tpw_measure_issue_peak")
    return out.value


INF = math.inf
