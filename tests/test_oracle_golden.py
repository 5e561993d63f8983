"""The numpy oracle against the golden vectors produced by the reference itself (CPU only)."""
import math

import numpy as np
import pytest

from cases import BOOL_CASES, FLOAT_CASES, FLOAT_METRICS, HAUSDORFF_CASES
from oracle import pairwise_oracle as O

# fp32 tolerance of the parity contract; fp64 is held to 1e-10
TOL = {np.dtype("float32"): dict(rtol=1e-4, atol=1e-5), np.dtype("float64"): dict(rtol=1e-10, atol=1e-10)}


def _oracle_forward(metric, x1, x2, w):
    fn, kw = metric["fn"], metric.get("kw", {})
    p = kw.get("p")
    if fn == "euclidean_distances": return O.cdist(x1, x2, 2.0)
    if fn == "manhattan_distances": return O.cdist(x1, x2, 1.0)
    if fn == "chebyshev_distances": return O.cdist(x1, x2, math.inf)
    if fn == "minkowski_distances": return O.cdist(x1, x2, p)
    if fn == "sqeuclidean_distances": return O.sqeuclidean(x1, x2)
    if fn == "cosine_similarity": return O.cosine_similarity(x1, x2)
    if fn == "cosine_distances": return O.cosine_distances(x1, x2)
    if fn == "correlation_distances": return O.correlation_distances(x1, x2)
    if fn == "linear_kernel": return x1 @ np.swapaxes(x2, -1, -2)
    if fn == "wminkowski_distances": return O.wminkowski(x1, x2, w, p)
    if fn == "_ppminkowski": return O.ppminkowski(x1, x2, p)
    if fn in ("rbf_kernel", "laplacian_kernel", "polynomial_kernel", "sigmoid_kernel"): return getattr(O, fn)(x1, x2, **kw)
    raise KeyError(fn)


def _oracle_backward(metric, g, x1, x2, w):
    fn, kw = metric["fn"], metric.get("kw", {})
    p = kw.get("p")
    if fn == "euclidean_distances": return O.cdist_backward(g, x1, x2, 2.0)
    if fn == "manhattan_distances": return O.cdist_backward(g, x1, x2, 1.0)
    if fn == "chebyshev_distances": return O.cdist_backward(g, x1, x2, math.inf)
    if fn == "minkowski_distances": return O.cdist_backward(g, x1, x2, p)
    if fn == "sqeuclidean_distances": return O.ppminkowski_backward(g, x1, x2, 2.0)
    if fn == "_ppminkowski": return O.ppminkowski_backward(g, x1, x2, p)
    if fn == "wminkowski_distances": return O.wminkowski_backward(g, x1, x2, w, p)
    if fn == "cosine_similarity": return O.cosine_similarity_backward(g, x1, x2)
    if fn == "linear_kernel": return g @ x2, np.swapaxes(g, -1, -2) @ x1
    return None


@pytest.mark.parametrize("case", FLOAT_CASES, ids=lambda c: c["name"])
@pytest.mark.parametrize("metric", FLOAT_METRICS, ids=lambda m: m["name"])
def test_float_metric_matches_reference(golden, case, metric):
    G = golden("float_metrics")
    key = f"{case['name']}/{metric['name']}"
    if key + "/out" not in G.files:
        pytest.skip("the reference rejects this input (batched weights need N1 == D)")
    x1, x2, w, g = (G[f"{case['name']}/{k}"] for k in ("x1", "x2", "w", "g"))
    tol = TOL[x1.dtype]
    st = case.get("stride", 1)
    out = _oracle_forward(metric, x1, x2, w)
    np.testing.assert_allclose(out[..., ::st, ::st], G[key + "/out"], **tol)
    grads = _oracle_backward(metric, g, x1, x2, w) if metric.get("grad", True) else None
    if grads is not None:
        # gradients sum up to N terms of size |g|*|d|^(p-1): scale the absolute floor accordingly
        scale = max(1.0, float(np.abs(G[key + "/gx1"]).max()))
        gtol = dict(rtol=tol["rtol"], atol=tol["atol"] * scale * 10)
        np.testing.assert_allclose(grads[0], G[key + "/gx1"], **gtol)
        np.testing.assert_allclose(grads[1], G[key + "/gx2"], **gtol)
        if metric.get("weighted"):
            np.testing.assert_allclose(grads[2], G[key + "/gw"], **gtol)


_BOOL_FAMILY = ["jaccard", "kulsinski", "kulczynski1", "yule", "dice", "rogerstanimoto", "russellrao",
                "sokalmichener", "sokalsneath"]


@pytest.mark.parametrize("case", BOOL_CASES, ids=lambda c: c["name"])
def test_boolean_family_is_bit_exact(golden, case):
    G = golden("bool_metrics")
    n = case["name"]
    x1, x2 = G[f"{n}/x1"], G[f"{n}/x2"]
    for name in _BOOL_FAMILY:
        ref = G[f"{n}/{name}_distances"]
        got = O.boolean_metric(name, x1 != 0, x2 != 0)
        np.testing.assert_array_equal(got, ref, err_msg=name)  # NaN == NaN in assert_array_equal
        assert got.dtype == np.float32
    np.testing.assert_array_equal(O.hamming(x1, x2), G[f"{n}/hamming_distances"])
    for op in ("eq", "ne"):
        for red in ("sum", "mean"):
            np.testing.assert_array_equal(O.compare_reduce(x1, x2, op, red), G[f"{n}/pw{op}_{red}"])
    if case["kind"] == "bool":
        for op in ("and", "or", "xor"):
            np.testing.assert_array_equal(O.pw_sum(x1, x2, op), G[f"{n}/pw{op}_sum"])


@pytest.mark.parametrize("case", HAUSDORFF_CASES, ids=lambda c: c["name"])
def test_hausdorff_matches_reference(golden, case):
    G = golden("hausdorff")
    n = case["name"]
    x1, x2, g = G[f"{n}/x1"], G[f"{n}/x2"], G[f"{n}/g"]
    out, i1, i2 = O.directed_hausdorff(x1, x2)
    np.testing.assert_array_equal(out, G[f"{n}/out"])  # same arithmetic, same rounding
    np.testing.assert_array_equal(i1, G[f"{n}/idx1"])
    np.testing.assert_array_equal(i2, G[f"{n}/idx2"])
    g1, g2 = O.directed_hausdorff_backward(g, out, i1, i2, x1, x2)
    tol = TOL[x1.dtype]
    np.testing.assert_allclose(g1, G[f"{n}/gx1"], **tol)
    np.testing.assert_allclose(g2, G[f"{n}/gx2"], **tol)


def test_prf_div_modes():
    x = np.array([1.0, 2.0, 0.0, -3.0], dtype=np.float32)
    y = np.array([2.0, 0.0, 0.0, 1.5], dtype=np.float32)
    np.testing.assert_array_equal(O.prf_div(x, y, "zero"), np.array([0.5, 0.0, 0.0, -2.0], dtype=np.float32))
    np.testing.assert_array_equal(O.prf_div(x, y, "identity"), np.array([0.5, 2.0, 0.0, -2.0], dtype=np.float32))
    gs, go = O.prf_div_backward(np.ones_like(x), x, y, "identity")
    np.testing.assert_allclose(gs, [0.5, 1.0, 1.0, 1 / 1.5], rtol=1e-6)
    np.testing.assert_allclose(go, [-0.25, 0.0, 0.0, 3 / 2.25], rtol=1e-6)


def test_extras_match_reference(golden):
    G = golden("extras")
    x1, x2, V = G["x1"], G["x2"], G["V"]
    tol = TOL[x1.dtype]
    np.testing.assert_allclose(O.seuclidean(x1, x2, V), G["seuclidean/out"], **tol)
    np.testing.assert_allclose(O.seuclidean(x1, x1, V), G["seuclidean_self/out"], **tol)
    np.testing.assert_allclose(O.seuclidean(x1, x2, V), G["cdist_seuclidean"], **tol)
    np.testing.assert_array_equal(O.k_neighbors_mask(O.cdist(x1, x2, 2.0), 3), G["k_neighbors_k3"])
    np.testing.assert_array_equal(O.k_neighbors_mask(O.cdist(x1, x1, 1.0), 2), G["k_neighbors_self_k2_manhattan"])
    np.testing.assert_array_equal(O.cdist(x1, x2, 2.0) <= 2.5, G["radius_2.5"])
    np.testing.assert_array_equal(O.cdist(x1, x1, 3.0) <= 3.0, G["radius_self_3_minkowski3"])


def test_composed_metrics_match_reference(golden):
    """braycurtis, snr, mahalanobis: the numpy restatements against the reference's own kernels."""
    G = golden("composed")
    for tag in ("u32", "b64"):
        x1, x2, VI = G[f"{tag}/x1"], G[f"{tag}/x2"], G[f"{tag}/VI"]
        tol = TOL[x1.dtype]
        np.testing.assert_allclose(O.braycurtis(x1, x2), G[f"{tag}/braycurtis_distances/out"], **tol)
        np.testing.assert_allclose(O.braycurtis(x1, x1), G[f"{tag}/braycurtis_distances/self_out"], **tol)
        np.testing.assert_allclose(O.snr_distances(x1, x2), G[f"{tag}/snr_distances/out"], **tol)
        np.testing.assert_allclose(O.snr_distances(x1, x1), G[f"{tag}/snr_distances/self_out"], **tol)
        np.testing.assert_allclose(O.mahalanobis(x1, x2, VI), G[f"{tag}/mahalanobis_distances/out"], **tol)
    np.testing.assert_allclose(O.braycurtis(G["u32/x1"], G["u32/x2"]), G["u32/cdist_braycurtis"], **TOL[np.dtype("float32")])
    big = G["u32/big"]
    VI = np.linalg.inv(np.cov(big.T.astype(np.float64))).T
    np.testing.assert_allclose(O.mahalanobis(big.astype(np.float64), big.astype(np.float64), VI), G["u32/mahalanobis_default_VI"], rtol=1e-3, atol=2e-3)


def test_pair_sum_metrics_match_reference(golden):
    """canberra and the chi-squared kernels: numpy restatements against the reference's own kernels."""
    G = golden("pair_sums")
    for tag in ("u32", "b64", "w32"):
        x1, x2, h1, h2 = G[f"{tag}/x1"], G[f"{tag}/x2"], G[f"{tag}/h1"], G[f"{tag}/h2"]
        tol = TOL[x1.dtype]
        np.testing.assert_allclose(O.canberra(x1, x2), G[f"{tag}/canberra_distances/out"], **tol)
        np.testing.assert_allclose(O.canberra(x1, x1), G[f"{tag}/canberra_distances/self_out"], **tol)
        np.testing.assert_allclose(O.additive_chi2_kernel(h1, h2), G[f"{tag}/additive_chi2_kernel/out"], **tol)
        np.testing.assert_allclose(O.additive_chi2_kernel(h1, h1), G[f"{tag}/additive_chi2_kernel/self_out"], **tol)
        np.testing.assert_allclose(O.chi2_kernel(h1, h2, 0.7), G[f"{tag}/chi2_kernel/out"], **tol)
    np.testing.assert_allclose(O.canberra(G["u32/x1"], G["u32/x2"]), G["u32/cdist_canberra"], **TOL[np.dtype("float32")])


def test_jensenshannon_matches_reference(golden):
    """Jensen-Shannon distance and its squared form: numpy restatement against the reference's kernel."""
    G = golden("jensenshannon")
    for tag in ("u32", "b64", "w32"):
        h1, h2 = G[f"{tag}/h1"], G[f"{tag}/h2"]
        tol = TOL[h1.dtype]
        for name, base in (("nat", None), ("base2", 2.0)):
            np.testing.assert_allclose(O.jensenshannon(h1, h2, base), G[f"{tag}/{name}/out"], **tol)
            n1, n2 = h1 / h1.sum(-1, keepdims=True), h2 / h2.sum(-1, keepdims=True)
            np.testing.assert_allclose(O.sqjensenshannon(n1, n2, base), G[f"{tag}/{name}/sq_out"], **tol)
        self_ref = G[f"{tag}/self_out"]
        assert float(np.abs(np.diagonal(self_ref, axis1=-2, axis2=-1)).max()) == 0.0
    np.testing.assert_allclose(O.jensenshannon(G["u32/h1"], G["u32/h2"], 3.0), G["u32/cdist_base3"], **TOL[np.dtype("float32")])


def test_haversine_matches_reference(golden):
    G = golden("haversine")
    for tag in ("u32", "b64", "w32"):
        x1, x2 = G[f"{tag}/x1"], G[f"{tag}/x2"]
        tol = TOL[x1.dtype]
        np.testing.assert_allclose(O.haversine(x1, x2), G[f"{tag}/out"], **tol)
        np.testing.assert_allclose(O.haversine(x1, x1), G[f"{tag}/self_out"], **tol)
        assert float(np.abs(np.diagonal(G[f"{tag}/self_out"], axis1=-2, axis2=-1)).max()) == 0.0
    np.testing.assert_allclose(O.haversine(G["u32/x1"], G["u32/x2"]), G["u32/cdist"], **TOL[np.dtype("float32")])
