"""CPU restatement (numpy) of the reference algorithms on the pairwise-reduction path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this module; it is the
checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of
``bench.py``.

Each function restates one piece of inspiros/torchpairwise v0.3.0 (OPS = torchpairwise/csrc/ops)
and cites the lines it follows.  Four of the metrics (euclidean, manhattan, chebyshev, minkowski)
are ``at::cdist`` in the reference, and cosine / correlation lean on ``matmul`` and ``norm``: that
arithmetic lives in PyTorch (the reference pins torch>=2.7,<2.8; 2.11.0 is installed here), which
is not part of the reference tree, so those functions restate the published definitions.

Parity pin: the reference has no golden vectors of its own (its single test file only prints
differences).  This oracle is pinned against outputs of the reference itself, built from its own
sources by ``oracle/Makefile`` and run by ``tests/golden/make_golden.py``; the resulting vectors
are committed under ``tests/golden/`` and ``tests/test_oracle_golden.py`` checks every function
here against them.

All functions take and return numpy arrays; inputs are [N, D] or [B, N, D] (point sets:
[N, M, D] or [B, N, M, D]); arithmetic runs in the input dtype unless stated.
"""
from __future__ import annotations

import numpy as np


def _b3(x):
    x = np.asarray(x)
    return (x[None], True) if x.ndim == 2 else (x, False)


def _un(out, unbatched):
    return out[0] if unbatched else out


def _diff(x1, x2):
    """d[b,i,j,k] = x1[b,i,k] - x2[b,j,k]"""
    return x1[:, :, None, :] - x2[:, None, :, :]


# ---- _ppminkowski (OPS/cpu/ppminkowski_kernel.cpp) ------------------------------------------------
def ppminkowski(x1, x2, p=2.0):
    """sum_k |d|^p, no root; +-inf: max / min |d|; p == 0: D.
    OPS/cpu/ppminkowski_kernel.cpp:13-29 (finite), :32-55 (inf), :90-91 (p == 0)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    dt = a.dtype
    if p == 0:
        return _un(np.full((a.shape[0], a.shape[1], b.shape[1]), a.shape[2], dtype=dt), ub)
    ad = np.abs(_diff(a, b))
    if np.isinf(p):
        out = ad.max(-1) if p > 0 else ad.min(-1)
    else:
        out = np.zeros(ad.shape[:-1], dtype=dt)
        for k in range(ad.shape[-1]):  # sequential accumulation over k, as the reference loop
            out += np.power(ad[..., k], dt.type(p))
    return _un(out.astype(dt), ub)


def ppminkowski_backward(grad, x1, x2, p):
    """grad_x1[b,i,k] = sum_j g*p*|d|^(p-1)*sgn(d) and the mirror for x2
    (OPS/cpu/ppminkowski_kernel.cpp:124-169); +-inf: the first extreme coordinate gets g*sgn(d)
    (:171-208); p == 0: zeros (:232)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    g, _ = _b3(grad)
    dt = a.dtype
    d = _diff(a, b)
    if p == 0:
        return _un(np.zeros_like(a), ub), _un(np.zeros_like(b), ub)
    if np.isinf(p):
        ad = np.abs(d)
        ks = ad.argmax(-1) if p > 0 else ad.argmin(-1)  # numpy returns the first extreme, like the strict compare
        sel = np.take_along_axis(d, ks[..., None], -1)[..., 0]
        contrib = g * np.sign(sel)
        onehot = np.zeros_like(d)
        np.put_along_axis(onehot, ks[..., None], 1.0, -1)
        t = contrib[..., None] * onehot
    else:
        t = g[..., None] * dt.type(p) * np.power(np.abs(d), dt.type(p - 1)) * np.sign(d)
    return _un(t.sum(2).astype(dt), ub), _un((-t).sum(1).astype(dt), ub)


# ---- _wminkowski (OPS/cpu/wminkowski_kernel.cpp) --------------------------------------------------
def wminkowski(x1, x2, w, p=2.0):
    """(sum_k w_k |d|^p)^(1/p); +-inf: max / min w_k|d|; p == 0: D.
    OPS/cpu/wminkowski_kernel.cpp:13-33, :36-60, :101-102.  Weights are NOT raised to p."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    ww = np.asarray(w)
    ww = ww[None] if ww.ndim == 1 else ww
    dt = a.dtype
    if p == 0:
        return _un(np.full((a.shape[0], a.shape[1], b.shape[1]), a.shape[2], dtype=dt), ub)
    ad = np.abs(_diff(a, b))
    wb = ww[:, None, None, :]
    if np.isinf(p):
        out = (ad * wb).max(-1) if p > 0 else (ad * wb).min(-1)
    else:
        s = (np.power(ad, dt.type(p)) * wb).sum(-1)
        out = np.power(s, dt.type(1.0 / p))
    return _un(out.astype(dt), ub)


def wminkowski_backward(grad, x1, x2, w, p):
    """OPS/cpu/wminkowski_kernel.cpp:137-211 (finite p; the `output` fed to those kernels is
    S^(1/p-1), computed by the forward kernel with its backward flag, :16-33) and :213-256 (inf)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    g, _ = _b3(grad)
    ww = np.asarray(w)
    ww = ww[None] if ww.ndim == 1 else ww
    dt = a.dtype
    d = _diff(a, b)
    ad = np.abs(d)
    wb = ww[:, None, None, :]
    if p == 0:
        return _un(np.zeros_like(a), ub), _un(np.zeros_like(b), ub), (np.zeros_like(ww)[0] if ub else np.zeros_like(ww))
    if np.isinf(p):
        wd = ad * wb
        ks = wd.argmax(-1) if p > 0 else wd.argmin(-1)
        onehot = np.zeros_like(d)
        np.put_along_axis(onehot, ks[..., None], 1.0, -1)
        sel = np.take_along_axis(d, ks[..., None], -1)[..., 0]
        t = (g * np.sign(sel))[..., None] * onehot * wb
        gw = (g[..., None] * onehot * ad).sum((1, 2))
    else:
        s = (np.power(ad, dt.type(p)) * wb).sum(-1)
        coef = np.power(s, dt.type(1.0 / p - 1.0))
        t = g[..., None] * np.power(ad, dt.type(p - 1)) * wb * coef[..., None] * np.sign(d)
        gw = (g[..., None] * np.power(ad, dt.type(p)) / dt.type(p) * coef[..., None]).sum((1, 2))
    gw = gw.astype(dt)
    return _un(t.sum(2).astype(dt), ub), _un((-t).sum(1).astype(dt), ub), (gw[0] if ub else gw)


# ---- ATen-delegated metrics (definitions; OPS/pairwise_metrics.cpp:30,48,167,305) -----------------
def cdist(x1, x2, p=2.0):
    """torch.cdist semantics: p=0 counts differing coordinates, p=inf is the maximum, otherwise
    (sum |d|^p)^(1/p).  For p=2 this is the direct form; ATen switches to the matmul form
    sqrt(clamp(|x|^2+|y|^2-2xy, 0)) when a side has more than 25 rows, which differs by rounding
    only (and leaves noise of order 1e-2 on the diagonal of self-distances)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    dt = a.dtype
    ad = np.abs(_diff(a, b))
    if p == 0:
        out = (ad != 0).sum(-1).astype(dt)
    elif np.isinf(p):
        out = ad.max(-1)
    elif p == 1:
        out = ad.sum(-1)
    elif p == 2:
        out = np.sqrt((ad * ad).sum(-1))
    else:
        out = np.power(np.power(ad, dt.type(p)).sum(-1), dt.type(1.0 / p))
    return _un(out.astype(dt), ub)


def cdist_backward(grad, x1, x2, p, out=None):
    """ATen's cdist backward: p=1: g*sgn(d); p<2: g*sgn(d)*|d|^(p-1)/o^(p-1) (0 where d == 0 and
    p < 1); p=2: g*d/o; p>2: g*d*|d|^(p-2)/o^(p-1); inf: g*sgn(d)*[|d| == o]; 0 where o == 0."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    g, _ = _b3(grad)
    dt = a.dtype
    d = _diff(a, b)
    ad = np.abs(d)
    o = _b3(cdist(a, b, p))[0] if out is None else _b3(out)[0]
    o4 = o[..., None]
    g4 = g[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        if p == 0:
            t = np.zeros_like(d)
        elif p == 1:
            t = g4 * np.sign(d)
        elif np.isinf(p):
            t = g4 * np.sign(d) * (ad == o4)
        elif p == 2:
            t = np.where(o4 == 0, 0, g4 * d / o4)
        elif p < 2:
            t = np.where(o4 == 0, 0, np.sign(d) * np.power(ad, dt.type(p - 1)) * g4 / np.power(o4, dt.type(p - 1)))
            if p < 1:
                t = np.where(d == 0, 0, t)
        else:
            t = np.where(o4 == 0, 0, d * np.power(ad, dt.type(p - 2)) * g4 / np.power(o4, dt.type(p - 1)))
    t = np.nan_to_num(t, nan=0.0, posinf=0.0, neginf=0.0) if p < 2 and p not in (0, 1) else t
    return _un(t.sum(2).astype(dt), ub), _un((-t).sum(1).astype(dt), ub)


def sqeuclidean(x1, x2):
    """_ppminkowski(x1, x2, 2) (OPS/pairwise_metrics.cpp:181-188)."""
    return ppminkowski(x1, x2, 2.0)


def prf_div(x, y, mode="zero"):
    """y != 0 ? x / y : (0 | x) (OPS/cpu/prf_divide.h:8-16)."""
    x, y = np.asarray(x), np.asarray(y)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = x / y
    return np.where(y != 0, q, x if mode == "identity" else np.zeros_like(x)).astype(np.result_type(x, y))


def prf_div_backward(grad, x, y, mode="zero"):
    """gs = g/o, go = -gs*s/o where o != 0; o == 0: gs = g (identity) or 0, go = 0
    (OPS/cpu/prf_div_kernel.cpp:257-312)."""
    g, x, y = np.asarray(grad), np.asarray(x), np.asarray(y)
    with np.errstate(divide="ignore", invalid="ignore"):
        gs = np.where(y != 0, g / y, g if mode == "identity" else np.zeros_like(g))
        go = np.where(y != 0, -gs * x / y, np.zeros_like(g))
    return gs, go


def cosine_similarity(x1, x2):
    """x1.x2^T / (|x1| |x2|^T) with prf_div "identity" (OPS/pairwise_metrics.cpp:112-122)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    n1 = np.sqrt((a * a).sum(-1, keepdims=True))
    n2 = np.sqrt((b * b).sum(-1, keepdims=True))
    denom = n1 * np.swapaxes(n2, -1, -2)
    m = a @ np.swapaxes(b, -1, -2)
    return _un(prf_div(m, denom, "identity").astype(a.dtype), ub)


def cosine_distances(x1, x2):
    """clip(1 - cosine_similarity, 0, 2) (OPS/pairwise_metrics.cpp:51-56)."""
    s = cosine_similarity(x1, x2)
    return np.clip(s.dtype.type(1) - s, 0, 2).astype(s.dtype)


def correlation_distances(x1, x2):
    """rows centred by their mean, then 1 - cosine_similarity, no clip
    (OPS/pairwise_metrics.cpp:190-204)."""
    a = np.asarray(x1)
    b = np.asarray(x2)
    a = a - a.mean(-1, keepdims=True, dtype=a.dtype)
    b = b - b.mean(-1, keepdims=True, dtype=b.dtype)
    s = cosine_similarity(a, b)
    return (s.dtype.type(1) - s).astype(s.dtype)


def cosine_similarity_backward(grad, x1, x2):
    """Chain rule through matmul, norms, outer product and prf_div "identity"
    (OPS/pairwise_metrics.cpp:118-121 with OPS/cpu/prf_div_kernel.cpp:257-312)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    g, _ = _b3(grad)
    n1 = np.sqrt((a * a).sum(-1, keepdims=True))
    n2 = np.sqrt((b * b).sum(-1, keepdims=True))
    denom = n1 * np.swapaxes(n2, -1, -2)
    m = a @ np.swapaxes(b, -1, -2)
    dm, dden = prf_div_backward(g, m, denom, "identity")
    dn1 = (dden * np.swapaxes(n2, -1, -2)).sum(-1, keepdims=True)
    dn2 = np.swapaxes((dden * n1).sum(-2, keepdims=True), -1, -2)
    with np.errstate(divide="ignore", invalid="ignore"):
        u1 = np.where(n1 != 0, a / n1, 0)
        u2 = np.where(n2 != 0, b / n2, 0)
    g1 = dm @ b + dn1 * u1
    g2 = np.swapaxes(dm, -1, -2) @ a + dn2 * u2
    return _un(g1.astype(a.dtype), ub), _un(g2.astype(a.dtype), ub)


# ---- kernel functions and standardised Euclidean (compositions; OPS/pairwise_metrics.cpp:67-110,245-263)
def _gamma(x1, gamma):
    """Default gamma is 1 / x1.size(1) whatever the rank (OPS/pairwise_metrics.cpp:76,88,97,108)."""
    return 1.0 / np.asarray(x1).shape[1] if gamma is None else gamma


def polynomial_kernel(x1, x2, degree=3, gamma=None, coef0=1.0):
    a, b = np.asarray(x1), np.asarray(x2)
    dt = a.dtype
    return ((a @ np.swapaxes(b, -1, -2) * dt.type(_gamma(a, gamma)) + dt.type(coef0)) ** int(degree)).astype(dt)


def sigmoid_kernel(x1, x2, gamma=None, coef0=1.0):
    a, b = np.asarray(x1), np.asarray(x2)
    dt = a.dtype
    return np.tanh(a @ np.swapaxes(b, -1, -2) * dt.type(_gamma(a, gamma)) + dt.type(coef0)).astype(dt)


def rbf_kernel(x1, x2, gamma=None):
    d = sqeuclidean(x1, x2)
    return np.exp(d * d.dtype.type(-_gamma(x1, gamma))).astype(d.dtype)


def laplacian_kernel(x1, x2, gamma=None):
    d = cdist(x1, x2, 1.0)
    return np.exp(d * d.dtype.type(-_gamma(x1, gamma))).astype(d.dtype)


def seuclidean(x1, x2, V):
    """_wminkowski(x1, x2, 1/V (1 where V == 0), 2) (OPS/pairwise_metrics.cpp:262)."""
    V = np.asarray(V)
    w = prf_div(np.ones_like(V), V, "identity")
    return wminkowski(x1, x2, w, 2.0)


def braycurtis(x1, x2):
    """sum_k |x1 - x2| / sum_k |x1 + x2| (OPS/cpu/braycurtis_kernel.cpp:22-27; 0/0 is NaN as there)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    with np.errstate(divide="ignore", invalid="ignore"):
        out = np.abs(_diff(a, b)).sum(-1) / np.abs(a[:, :, None, :] + b[:, None, :, :]).sum(-1)
    return _un(out.astype(a.dtype), ub)


def snr_distances(x1, x2):
    """1 / _snr with _snr = D var(x1 row, population) / sum_k (e_k - mean(e))^2, e = x2 - x1
    (OPS/cpu/snr_kernel.cpp:22-34,96; OPS/pairwise_metrics.cpp:407)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    e = -_diff(a, b)
    diff_var = ((e - e.mean(-1, keepdims=True)) ** 2).sum(-1)
    x1_var = ((a - a.mean(-1, keepdims=True)) ** 2).sum(-1)[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        out = 1.0 / (x1_var / diff_var)
    return _un(out.astype(a.dtype), ub)


def mahalanobis(x1, x2, VI):
    """sqrt(sum_kl d_k VI[k,l] d_l) (OPS/cpu/sqmahalanobis_kernel.cpp:23-31; sqrt at
    OPS/pairwise_metrics.cpp:296).  VI [D,D] or [B,D,D], not assumed symmetric."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    V = np.asarray(VI)
    V = V[None] if V.ndim == 2 else V
    d = _diff(a, b)
    out = np.sqrt(np.einsum("bijk,bkl,bijl->bij", d, V, d))
    return _un(out.astype(a.dtype), ub)


def canberra(x1, x2):
    """sum_k |x1 - x2| / (|x1| + |x2|), terms with a zero denominator skipped (OPS/cpu/canberra_kernel.cpp:22-29)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    num = np.abs(_diff(a, b))
    den = np.abs(a)[:, :, None, :] + np.abs(b)[:, None, :, :]
    with np.errstate(divide="ignore", invalid="ignore"):
        out = np.where(den != 0, num / den, 0).sum(-1)
    return _un(out.astype(a.dtype), ub)


def additive_chi2_kernel(x1, x2):
    """- sum_k (x1 - x2)^2 / (x1 + x2), terms with a zero denominator skipped (OPS/cpu/additive_chi2_kernel.cpp:22-31)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    d = _diff(a, b)
    nom = a[:, :, None, :] + b[:, None, :, :]
    with np.errstate(divide="ignore", invalid="ignore"):
        out = -np.where(nom != 0, d * d / nom, 0).sum(-1)
    return _un(out.astype(a.dtype), ub)


def chi2_kernel(x1, x2, gamma=1.0):
    """exp(gamma * additive_chi2_kernel) (OPS/pairwise_metrics.cpp:144)."""
    return np.exp(additive_chi2_kernel(x1, x2) * np.asarray(x1).dtype.type(gamma))


def sqjensenshannon(x1, x2, base=None):
    """sum_k rel_entr(x1, m) + rel_entr(x2, m), m = (x1 + x2)/2, divided by 2 log(base) (by 2 without a base)
    (OPS/cpu/sqjensenshannon_kernel.cpp:13-31,75; rel_entr: v log(v/m) for v > 0, 0 at v == 0, OPS/cpu/rel_entr.h:9-18).
    Inputs are non-negative."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    x, y = a[:, :, None, :], b[:, None, :, :]
    m = (x + y) / a.dtype.type(2)
    with np.errstate(divide="ignore", invalid="ignore"):
        tx = np.where(x > 0, x * np.log(x / m), 0)
        ty = np.where(y > 0, y * np.log(y / m), 0)
    out = (tx + ty).sum(-1) / a.dtype.type(2 * np.log(base) if base is not None else 2)
    return _un(out.astype(a.dtype), ub)


def jensenshannon(x1, x2, base=None):
    """sqrt(sqjensenshannon) of the rows scaled to sum one (OPS/pairwise_metrics.cpp:326-337)."""
    a, b = np.asarray(x1), np.asarray(x2)
    return np.sqrt(sqjensenshannon(a / a.sum(-1, keepdims=True), b / b.sum(-1, keepdims=True), base))


def haversine(x1, x2):
    """2 asin(sqrt(sin^2(dlat/2) + cos(lat1) cos(lat2) sin^2(dlon/2))) for (latitude, longitude) rows in radians
    (OPS/cpu/haversine_kernel.cpp:12-27)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    two = a.dtype.type(2)
    dlat = (a[:, :, None, 0] - b[:, None, :, 0]) / two
    dlon = (a[:, :, None, 1] - b[:, None, :, 1]) / two
    val = np.sin(dlat) ** 2 + np.cos(a[:, :, None, 0]) * np.cos(b[:, None, :, 0]) * np.sin(dlon) ** 2
    return _un((two * np.arcsin(np.sqrt(val))).astype(a.dtype), ub)


def k_neighbors_mask(dists, k):
    """True at the k + 1 smallest entries of every row (OPS/neighbors.cpp:29-33)."""
    d = np.asarray(dists)
    idx = np.argsort(d, axis=1, kind="stable")[:, : k + 1]
    out = np.zeros(d.shape, dtype=bool)
    np.put_along_axis(out, idx, True, axis=1)
    return out


# ---- boolean family (OPS/cpu/pairwise_binary_kernels.cpp:28-49 + compositions) -------------------
def _counts(x1, x2):
    a, ub = _b3(np.asarray(x1).astype(bool))
    b, _ = _b3(np.asarray(x2).astype(bool))
    ai = a.astype(np.int64)
    bi = b.astype(np.int64)
    n11 = ai @ np.swapaxes(bi, -1, -2)
    pa = ai.sum(-1)[:, :, None]
    pb = bi.sum(-1)[:, None, :]
    return n11, pa, pb, a.shape[-1], ub


def pw_sum(x1, x2, op):
    """float32 count of op(x1, x2) over features for boolean inputs, op in and/or/xor/eq/ne
    (OPS/cpu/pairwise_binary_kernels.cpp:28-49, float32 output :137-143)."""
    n11, pa, pb, D, ub = _counts(x1, x2)
    nxor = pa + pb - 2 * n11
    val = {"and": n11, "or": pa + pb - n11, "xor": nxor, "ne": nxor, "eq": D - nxor}[op]
    return _un(val.astype(np.float32), ub)


def compare_reduce(x1, x2, op="ne", reduction="mean"):
    """pw{eq,ne}_{sum,mean} on any dtype: float32 sum of the comparison, mean divides by float(D)
    (OPS/cpu/pairwise_binary_kernels.cpp:38-47)."""
    a, ub = _b3(x1)
    b, _ = _b3(x2)
    common = np.result_type(a, b)
    a, b = a.astype(common), b.astype(common)
    cmp = a[:, :, None, :] != b[:, None, :, :]
    if op == "eq":
        cmp = ~cmp
    cnt = cmp.sum(-1).astype(np.float32)
    if reduction == "mean":
        cnt = cnt / np.float32(a.shape[-1])
    return _un(cnt.astype(np.float32), ub)


def hamming(x1, x2):
    """pwne_mean (OPS/pairwise_metrics.cpp:206-213)."""
    return compare_reduce(x1, x2, "ne", "mean")


def boolean_metric(name, x1, x2):
    """The float32 compositions of OPS/pairwise_metrics.cpp:215-243 and :339-399, each
    arithmetic step rounded to float32 in the order the reference evaluates it."""
    f = np.float32
    A = pw_sum(x1, x2, "and")
    X = pw_sum(x1, x2, "xor")
    O = pw_sum(x1, x2, "or")
    E = pw_sum(x1, x2, "eq")
    D = f(np.asarray(x1).shape[-1])
    with np.errstate(divide="ignore", invalid="ignore"):
        if name == "jaccard":            # prf_div(pwxor_sum, pwor_sum)           :221
            return prf_div(X, O, "zero").astype(f)
        if name == "kulsinski":          # (S - and + D) / (S + D)                :232-233
            return (((X - A).astype(f) + D).astype(f) / (X + D).astype(f)).astype(f)
        if name == "kulczynski1":        # and / xor                              :242
            return (A / X).astype(f)
        if name == "yule":               # prf_div(2R, n11*n00 + R), R = n10*n01  :345-346
            a_ = np.asarray(x1).astype(bool)
            b_ = np.asarray(x2).astype(bool)
            n10 = pw_sum(a_, ~b_, "and")
            n01 = pw_sum(~a_, b_, "and")
            n00 = pw_sum(~a_, ~b_, "and")
            half_r = (n10 * n01).astype(f)
            den = ((A * n00).astype(f) + half_r).astype(f)
            return prf_div((f(2) * half_r).astype(f), den, "zero").astype(f)
        if name == "dice":               # R / (2*and + R)                        :355-356
            return (X / ((f(2) * A).astype(f) + X).astype(f)).astype(f)
        if name in ("rogerstanimoto", "sokalmichener"):  # 2R / (eq + 2R)         :365-367, :385-387
            r2 = (f(2) * X).astype(f)
            return (r2 / (E + r2).astype(f)).astype(f)
        if name == "russellrao":         # (D - and) / D                          :376
            return ((D - A).astype(f) / D).astype(f)
        if name == "sokalsneath":        # 2R / (and + 2R)                        :396-398
            r2 = (f(2) * X).astype(f)
            return (r2 / (A + r2).astype(f)).astype(f)
    raise ValueError(name)


# ---- directed Hausdorff (OPS/cpu/hausdorff_kernel.cpp) ------------------------------------------
def directed_hausdorff(x1, x2, order1=None, order2=None):
    """out[b,i,j] = sqrt(max_m min_n |x1[b,i,m]-x2[b,j,n]|^2) with the attaining indices.

    Restates the loop of OPS/cpu/hausdorff_kernel.cpp:20-52 without its early break (the break
    only skips rows that cannot raise the maximum): squared distances are accumulated coordinate
    by coordinate in the input dtype; n* is the first visited n reaching the row minimum (strict
    <, :36), m* the last visited m whose row minimum reaches the running maximum (>=, :42).
    order1/order2 ([B, M] visiting positions) reproduce the shuffled variant (:56-100)."""
    a = np.asarray(x1)
    b = np.asarray(x2)
    ub = a.ndim == 3
    if ub:
        a, b = a[None], b[None]
    B, N1, M1, D = a.shape
    N2, M2 = b.shape[1], b.shape[2]
    dt = a.dtype
    out = np.zeros((B, N1, N2), dtype=dt)
    i1 = np.zeros((B, N1, N2), dtype=np.int64)
    i2 = np.zeros((B, N1, N2), dtype=np.int64)
    for bb in range(B):
        o1 = np.arange(M1) if order1 is None else np.asarray(order1)[bb]
        o2 = np.arange(M2) if order2 is None else np.asarray(order2)[bb]
        for i in range(N1):
            for j in range(N2):
                d = np.zeros((M1, M2), dtype=dt)
                for k in range(D):
                    diff = a[bb, i, :, None, k] - b[bb, j, None, :, k]
                    d = d + diff * diff
                rowmin = d.min(1)
                # first visited n attaining the row minimum
                cand = np.where(d == rowmin[:, None], o2[None, :], M2 + 1)
                npos = cand.min(1)
                cmax = rowmin.max()
                mpos = np.where(rowmin == cmax, o1, -1).max()
                m = int(np.nonzero(o1 == mpos)[0][0])
                n = int(np.nonzero(o2 == npos[m])[0][0])
                out[bb, i, j] = np.sqrt(cmax)
                i1[bb, i, j] = m
                i2[bb, i, j] = n
    if ub:
        return out[0], i1[0], i2[0]
    return out, i1, i2


def directed_hausdorff_backward(grad, out, idx1, idx2, x1, x2):
    """grad_x1[b,i,m*,:] += g*(x1[m*]-x2[n*])/out; grad_x2[b,j,n*,:] -= the same
    (OPS/cpu/hausdorff_kernel.cpp:189-236)."""
    a = np.asarray(x1)
    b = np.asarray(x2)
    ub = a.ndim == 3
    g, o, i1, i2 = np.asarray(grad), np.asarray(out), np.asarray(idx1), np.asarray(idx2)
    if ub:
        a, b, g, o, i1, i2 = a[None], b[None], g[None], o[None], i1[None], i2[None]
    g1 = np.zeros_like(a)
    g2 = np.zeros_like(b)
    B, N1, N2 = o.shape
    with np.errstate(divide="ignore", invalid="ignore"):
        for bb in range(B):
            for i in range(N1):
                for j in range(N2):
                    m, n = i1[bb, i, j], i2[bb, i, j]
                    diff = a[bb, i, m] - b[bb, j, n]
                    g1[bb, i, m] += g[bb, i, j] * diff / o[bb, i, j]
                    g2[bb, j, n] += g[bb, i, j] * (-diff) / o[bb, i, j]
    return (g1[0], g2[0]) if ub else (g1, g2)
