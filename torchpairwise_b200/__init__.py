"""B200 (sm_100a) implementation of torchpairwise's pairwise-reduction hot path.

The module mirrors the reference's Python surface (``torchpairwise/__init__.py`` and
``torchpairwise/ops``): the same function names with the same arguments, backed by hand-written
CUDA kernels behind the C ABI of ``include/tpw_b200.h``.  CUDA tensors only.
"""
from ._abi import LIB_PATH, TpwError, device_status, lib, measure_issue_peak
from .cpdist import cdist, pdist
from .ops import (
    _directed_hausdorff,
    _haversine,
    _ppminkowski,
    _sqjensenshannon,
    _wminkowski,
    additive_chi2_kernel,
    braycurtis_distances,
    canberra_distances,
    chebyshev_distances,
    chi2_kernel,
    cityblock_distances,
    correlation_distances,
    cosine_distances,
    cosine_similarity,
    dice_distances,
    directed_hausdorff_distances,
    euclidean_distances,
    get_dot_engine,
    hamming_distances,
    haversine_distances,
    jaccard_distances,
    jensenshannon_distances,
    k_neighbors_mask,
    kulczynski1_distances,
    kulsinski_distances,
    laplacian_kernel,
    l1_distances,
    l2_distances,
    linear_kernel,
    linf_distances,
    lp_distances,
    mahalanobis_distances,
    manhattan_distances,
    minkowski_distances,
    pairwise_argkmin,
    pairwise_argmin_min,
    polynomial_kernel,
    prf_div,
    pwand_sum,
    pweq_mean,
    pweq_sum,
    pwne_mean,
    pwne_sum,
    pwor_sum,
    pwxor_sum,
    radius_neighbors_mask,
    rbf_kernel,
    rogerstanimoto_distances,
    russellrao_distances,
    set_dot_engine,
    seuclidean_distances,
    sigmoid_kernel,
    snr_distances,
    sokalmichener_distances,
    sokalsneath_distances,
    sqeuclidean_distances,
    wminkowski_distances,
    yule_distances,
)

__version__ = "0.1.0"

TORCH_OPS_LIBRARY = LIB_PATH.parent / "libtpw_b200_torch.so"


def load_torch_ops() -> str:
    """Register the C++ host layer with the torch dispatcher: afterwards
    ``torch.ops.torchpairwise.<op>`` (the reference's own operator names and schemas) runs the
    sm_100a kernels for CUDA tensors.  If the reference extension is installed, load it first: its
    schemas are reused and it keeps serving CPU tensors.  Returns the library path."""
    import torch

    if not TORCH_OPS_LIBRARY.exists():
        raise ImportError(f"{TORCH_OPS_LIBRARY} is missing; run `python torchpairwise_b200/build.py`")
    torch.ops.load_library(str(TORCH_OPS_LIBRARY))
    return str(TORCH_OPS_LIBRARY)


def has_ops() -> bool:
    """torchpairwise.extension.has_ops (extension.py:163-165)."""
    return True


def with_cuda() -> bool:
    """torchpairwise.extension.with_cuda (extension.py:168-175)."""
    return True


def cuda_version() -> int:
    """CUDA runtime version the kernels were compiled with (csrc/torchpairwise.cpp:28-34)."""
    return int(lib.tpw_cuda_version())


def cuda_arch_list():
    """Architectures in the binary (csrc/torchpairwise.cpp:36-52): sm_100a only."""
    return [lib.tpw_cuda_arch_flags().decode()]
