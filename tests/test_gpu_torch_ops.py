"""The C++ host layer: `torch.ops.torchpairwise.*` with the reference's own schemas.

With the reference's CPU build loaded in the same process the very same call goes to the reference
for CPU tensors and to the sm_100a kernels for CUDA tensors, so parity is checked operator by
operator with nothing in between.  Stand-alone registration is checked in a child process.
"""
import math
import subprocess
import sys
import warnings
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref" / "torchpairwise_ref.so"

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    if not REF.exists():
        pytest.skip("oracle/_ref is not built on this machine")
    torch.ops.load_library(str(REF))  # reference first: its schemas are reused
    import torchpairwise_b200
    torchpairwise_b200.load_torch_ops()
    yield torch.ops.torchpairwise
    assert torchpairwise_b200.device_status() == 0


FLOAT_OPS = [
    ("euclidean_distances", {}), ("manhattan_distances", {}), ("chebyshev_distances", {}), ("sqeuclidean_distances", {}),
    ("minkowski_distances", {"p": 3.0}), ("minkowski_distances", {"p": 1.5}), ("cosine_similarity", {}),
    ("cosine_distances", {}), ("correlation_distances", {}), ("l1_distances", {}), ("l2_distances", {}),
    ("lp_distances", {"p": 2.5}), ("linf_distances", {}), ("cityblock_distances", {}),
]


@pytest.mark.parametrize("name,kw", FLOAT_OPS, ids=lambda v: str(v))
@pytest.mark.parametrize("shape", [((37, 19), (23, 19)), ((2, 140, 70), (2, 131, 70))])
def test_same_call_reference_on_cpu_kernels_on_cuda(T, name, kw, shape):
    g = torch.Generator().manual_seed(11)
    x1 = torch.randn(*shape[0], generator=g)
    x2 = torch.randn(*shape[1], generator=g)
    up = torch.randn(*shape[0][:-1], shape[1][-2], generator=g)
    a, b = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True)
    ref = getattr(T, name)(a, b, **kw)
    ref.backward(up)
    c, d = x1.cuda().requires_grad_(True), x2.cuda().requires_grad_(True)
    out = getattr(T, name)(c, d, **kw)
    out.backward(up.cuda())
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-5)
    scale = 10 * max(1.0, float(a.grad.abs().max()))
    torch.testing.assert_close(c.grad.cpu(), a.grad, rtol=1e-4, atol=1e-5 * scale)
    torch.testing.assert_close(d.grad.cpu(), b.grad, rtol=1e-4, atol=1e-5 * scale)


def test_weighted_internal_and_boolean_ops(T):
    g = torch.Generator().manual_seed(12)
    x1, x2 = torch.randn(9, 9, generator=g), torch.randn(7, 9, generator=g)
    w = torch.rand(9, generator=g) + 0.3
    up = torch.randn(9, 7, generator=g)
    for p in (3.0, 1.0, math.inf):
        a, b, ww = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True), w.clone().requires_grad_(True)
        ref = T.wminkowski_distances(a, b, p, ww)
        ref.backward(up)
        c, d, wc = x1.cuda().requires_grad_(True), x2.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
        out = T.wminkowski_distances(c, d, p, wc)
        out.backward(up.cuda())
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-5)
        for got, want in ((c.grad, a.grad), (d.grad, b.grad), (wc.grad, ww.grad)):
            torch.testing.assert_close(got.cpu(), want, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(T._ppminkowski(x1.cuda(), x2.cuda(), 3.0).cpu(), T._ppminkowski(x1, x2, 3.0), rtol=1e-4, atol=1e-5)
    xb, yb = torch.rand(50, 77, generator=g) < 0.3, torch.rand(41, 77, generator=g) < 0.3
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for name in ("hamming", "jaccard", "kulsinski", "kulczynski1", "yule", "dice", "rogerstanimoto", "russellrao",
                     "sokalmichener", "sokalsneath"):
            ref = getattr(T, name + "_distances")(xb, yb)
            out = getattr(T, name + "_distances")(xb.cuda(), yb.cuda()).cpu()
            assert bool(((out == ref) | (out.isnan() & ref.isnan())).all()), name
        for name in ("pwand_sum", "pwor_sum", "pwxor_sum", "pweq_sum", "pwne_sum", "pweq_mean", "pwne_mean"):
            assert torch.equal(getattr(T, name)(xb.cuda(), yb.cuda()).cpu(), getattr(T, name)(xb, yb)), name
        xi, yi = torch.randint(0, 3, (12, 20), generator=g), torch.randint(0, 3, (9, 20), generator=g)
        assert torch.equal(T.hamming_distances(xi.cuda(), yi.cuda()).cpu(), T.hamming_distances(xi, yi))
        assert torch.equal(T.jaccard_distances(xi.cuda(), yi.cuda()).cpu(), T.jaccard_distances(xi, yi))


def test_hausdorff_and_cdist_dispatcher(T):
    g = torch.Generator().manual_seed(13)
    s1, s2 = torch.rand(2, 3, 60, 3, generator=g), torch.rand(2, 2, 45, 3, generator=g)
    up = torch.randn(2, 3, 2, generator=g)
    a, b = s1.clone().requires_grad_(True), s2.clone().requires_grad_(True)
    ref, r1, r2 = T.directed_hausdorff_distances(a, b)
    ref.backward(up)
    c, d = s1.cuda().requires_grad_(True), s2.cuda().requires_grad_(True)
    out, i1, i2 = T.directed_hausdorff_distances(c, d)
    out.backward(up.cuda())
    assert torch.equal(out.cpu(), ref) and torch.equal(i1.cpu(), r1) and torch.equal(i2.cpu(), r2)
    torch.testing.assert_close(c.grad.cpu(), a.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(d.grad.cpu(), b.grad, rtol=1e-4, atol=1e-5)
    x1, x2 = torch.randn(20, 8, generator=g), torch.randn(17, 8, generator=g)
    for metric, kw in (("euclidean", {}), ("minkowski", {"p": 3.0}), ("cosine", {}), ("manhattan", {}), ("sqeuclidean", {}),
                       ("chebyshev", {}), ("correlation", {})):
        torch.testing.assert_close(T.cdist(x1.cuda(), x2.cuda(), metric, **kw).cpu(), T.cdist(x1, x2, metric, **kw),
                                   rtol=1e-4, atol=1e-5)
    assert torch.equal(T.cdist(s1.cuda(), s2.cuda(), "directed_hausdorff").cpu(), ref.detach())
    with pytest.raises(TypeError, match="incompatible arguments p"):
        T.cdist(x1.cuda(), x2.cuda(), "euclidean", p=2.0)
    with pytest.raises(RuntimeError, match="unkown distance metric"):
        T.cdist(x1.cuda(), x2.cuda(), "nope")
    A = torch.randn(8, 8, generator=g)
    VI = A @ A.t() + 0.5 * torch.eye(8)
    torch.testing.assert_close(T.cdist(x1.cuda(), x2.cuda(), "mahalanobis", VI=VI.cuda()).cpu(), T.cdist(x1, x2, "mahalanobis", VI=VI),
                               rtol=1e-4, atol=1e-5)


def test_prf_div_family_and_hausdorff_backward_op(T):
    """Every prf_div / prf_ldiv overload (tensor, Scalar, rScalar, in place) with its gradient, the stand-alone
    backward ops, and __directed_hausdorff_backward: the reference on CPU tensors, these kernels on CUDA tensors."""
    g = torch.Generator().manual_seed(16)
    x = torch.randn(6, 50, generator=g)
    y = torch.randn(6, 50, generator=g)
    x[torch.rand(6, 50, generator=g) < 0.2] = 0
    y[torch.rand(6, 50, generator=g) < 0.3] = 0
    up = torch.randn(6, 50, generator=g)

    def both(fn, *tensors):
        res = []
        for dev in ("cpu", "cuda"):
            leaves = [t.to(dev).clone().requires_grad_(t.is_floating_point()) for t in tensors]
            out = fn(*leaves)
            out.backward(up.to(dev))
            res.append((out.detach().cpu(), [l.grad.cpu() for l in leaves if l.requires_grad]))
        (o_ref, g_ref), (o_got, g_got) = res
        torch.testing.assert_close(o_got, o_ref, rtol=1e-6, atol=0, equal_nan=True)
        for a, b in zip(g_got, g_ref):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-7, equal_nan=True)

    for mode in ("zero", "identity"):
        both(lambda a, b: T.prf_div(a, b, mode), x, y)
        both(lambda a, b: T.prf_ldiv(a, b, mode), x, y)
        for s in (2.5, 0.0):
            both(lambda a: T.prf_div(a, s, mode), x)
            both(lambda a: T.prf_ldiv(a, s, mode), y)
            both(lambda b: T.prf_div(s, b, mode), y)
            both(lambda b: T.prf_ldiv(s, b, mode), x)
        # in place: values, and the input really is overwritten
        for name, args in (("prf_div_", (y,)), ("prf_ldiv_", (y,)), ("prf_div_", (2.0,)), ("prf_ldiv_", (0.0,))):
            outs = []
            for dev in ("cpu", "cuda"):
                a = x.to(dev).clone()
                r = getattr(T, name)(a, *[v.to(dev) if isinstance(v, torch.Tensor) else v for v in args], mode)
                assert r.data_ptr() == a.data_ptr()
                outs.append(a.cpu())
            torch.testing.assert_close(outs[1], outs[0], rtol=1e-6, atol=0, equal_nan=True)
        for name in ("_prf_div_backward", "_prf_ldiv_backward", "_prf_div__backward", "_prf_ldiv__backward"):
            ref = getattr(T, name)(up, x, y, mode)
            got = getattr(T, name)(up.cuda(), x.cuda(), y.cuda(), mode)
            for a, b in zip(got, ref):
                torch.testing.assert_close(a.cpu(), b, rtol=1e-5, atol=1e-7, equal_nan=True)
            torch.testing.assert_close(getattr(T, name)(up.cuda(), x.cuda(), 1.5, mode).cpu(), getattr(T, name)(up, x, 1.5, mode),
                                       rtol=1e-5, atol=1e-7, equal_nan=True)
        for name in ("_prf_div_backward", "_prf_ldiv_backward"):
            torch.testing.assert_close(getattr(T, name)(up.cuda(), 1.5, y.cuda(), mode).cpu(), getattr(T, name)(up, 1.5, y, mode),
                                       rtol=1e-5, atol=1e-7, equal_nan=True)
    xi = torch.randint(-2, 3, (4, 9), generator=g)
    yi = torch.randint(-1, 2, (4, 9), generator=g)
    got, ref = T.prf_div(xi.cuda(), yi.cuda(), "identity"), T.prf_div(xi, yi, "identity")
    assert got.dtype == ref.dtype == torch.float32 and torch.equal(got.cpu(), ref)
    with pytest.raises(RuntimeError, match="mode must be either zero or identity"):
        T.prf_div(x.cuda(), y.cuda(), "nope")
    with pytest.raises(RuntimeError, match="Broadcasting semantic is not implemented"):
        T.prf_div(x.cuda(), y.cuda()[:3], "zero")

    s1, s2 = torch.rand(2, 3, 40, 3, generator=g), torch.rand(2, 2, 33, 3, generator=g)
    gu = torch.randn(2, 3, 2, generator=g)
    r1, r2 = T.__directed_hausdorff_backward(gu, s1, s2)
    g1, g2 = T.__directed_hausdorff_backward(gu.cuda(), s1.cuda(), s2.cuda())
    torch.testing.assert_close(g1.cpu(), r1, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(g2.cpu(), r2, rtol=1e-4, atol=1e-5)


def test_jensenshannon_and_haversine_ops(T):
    """jensenshannon_distances / _sqjensenshannon and haversine_distances / _haversine with their gradients, the
    stand-alone backward ops and the cdist spellings: the reference on CPU tensors, these kernels on CUDA tensors."""
    g = torch.Generator().manual_seed(17)
    h1, h2 = torch.rand(31, 24, generator=g), torch.rand(27, 24, generator=g)
    h1[0, :5] = 0
    h2[1, 3:9] = 0
    up = torch.randn(31, 27, generator=g)
    scale = torch.tensor([math.pi, 2 * math.pi])
    p1, p2 = (torch.rand(31, 2, generator=g) - 0.5) * scale, (torch.rand(27, 2, generator=g) - 0.5) * scale
    n1, n2 = h1 / h1.sum(-1, keepdim=True), h2 / h2.sum(-1, keepdim=True)
    for fn, x1, x2 in ((lambda a, b: T.jensenshannon_distances(a, b, None), h1, h2),
                       (lambda a, b: T.jensenshannon_distances(a, b, 2.0), h1, h2),
                       (lambda a, b: T._sqjensenshannon(a, b, 3.0), n1, n2),
                       (lambda a, b: T.haversine_distances(a, b), p1, p2),
                       (lambda a, b: T._haversine(a, b), p1, p2)):
        res = []
        for dev in ("cpu", "cuda"):
            a, b = x1.detach().clone().to(dev).requires_grad_(True), x2.detach().clone().to(dev).requires_grad_(True)
            out = fn(a, b)
            out.backward(up.to(dev))
            res.append((out.detach().cpu(), a.grad.cpu(), b.grad.cpu()))
        torch.testing.assert_close(res[1][0], res[0][0], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(res[1][1], res[0][1], rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(res[1][2], res[0][2], rtol=1e-4, atol=1e-4)
    for ref, got in ((T.__sqjensenshannon_backward(up, n1, n2, 2.0), T.__sqjensenshannon_backward(up.cuda(), n1.cuda(), n2.cuda(), 2.0)),
                     (T.__haversine_backward(up, p1, p2), T.__haversine_backward(up.cuda(), p1.cuda(), p2.cuda()))):
        for a, b in zip(got, ref):
            torch.testing.assert_close(a.cpu(), b, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(T.cdist(h1.cuda(), h2.cuda(), "jensenshannon", base=2.0).cpu(), T.cdist(h1, h2, "jensenshannon", base=2.0),
                               rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(T.cdist(p1.cuda(), p2.cuda(), "haversine").cpu(), T.cdist(p1, p2, "haversine"), rtol=1e-4, atol=1e-5)
    with pytest.raises(RuntimeError, match="feature dimension of x1 and x2 must be 2"):
        T.haversine_distances(h1.cuda(), h2.cuda())


def test_composed_and_pair_sum_ops(T):
    """canberra, additive_chi2 / chi2, braycurtis, snr and seuclidean through the C++ layer, with gradients, and
    their cdist spellings: the reference on CPU tensors, these kernels on CUDA tensors."""
    g = torch.Generator().manual_seed(18)
    x1, x2 = torch.randn(33, 21, generator=g), torch.randn(26, 21, generator=g)
    h1, h2 = torch.rand(33, 21, generator=g), torch.rand(26, 21, generator=g)
    h1[0, :4] = 0
    h2[2, :6] = 0
    V = torch.rand(21, generator=g) + 0.2
    up = torch.randn(33, 26, generator=g)
    cases = ((lambda a, b: T.canberra_distances(a, b), x1, x2), (lambda a, b: T._canberra(a, b), x1, x2),
             (lambda a, b: T.additive_chi2_kernel(a, b), h1, h2), (lambda a, b: T.chi2_kernel(a, b, 0.7), h1, h2),
             (lambda a, b: T.braycurtis_distances(a, b), x1, x2), (lambda a, b: T.snr_distances(a, b), x1, x2),
             (lambda a, b: T.seuclidean_distances(a, b, V.to(a.device)), x1, x2))
    for fn, u, v in cases:
        res = []
        for dev in ("cpu", "cuda"):
            a, b = u.detach().clone().to(dev).requires_grad_(True), v.detach().clone().to(dev).requires_grad_(True)
            out = fn(a, b)
            out.backward(up.to(dev))
            res.append((out.detach().cpu(), a.grad.cpu(), b.grad.cpu()))
        torch.testing.assert_close(res[1][0], res[0][0], rtol=1e-4, atol=1e-5)
        scale = 10 * max(1.0, float(res[0][1].abs().max()))
        torch.testing.assert_close(res[1][1], res[0][1], rtol=1e-4, atol=1e-5 * scale)
        torch.testing.assert_close(res[1][2], res[0][2], rtol=1e-4, atol=1e-5 * scale)
    torch.testing.assert_close(T.seuclidean_distances(x1.cuda(), None, None).cpu(), T.seuclidean_distances(x1, None, None), rtol=1e-4, atol=1e-5)
    for ref, got in ((T.__canberra_backward(up, x1, x2), T.__canberra_backward(up.cuda(), x1.cuda(), x2.cuda())),
                     (T.__additive_chi2_kernel_backward(up, h1, h2), T.__additive_chi2_kernel_backward(up.cuda(), h1.cuda(), h2.cuda()))):
        for a, b in zip(got, ref):
            torch.testing.assert_close(a.cpu(), b, rtol=1e-4, atol=1e-4)
    for metric, kw in (("canberra", {}), ("braycurtis", {}), ("snr", {}), ("seuclidean", {"V": V})):
        kc = {k: v.cuda() for k, v in kw.items()}
        torch.testing.assert_close(T.cdist(x1.cuda(), x2.cuda(), metric, **kc).cpu(), T.cdist(x1, x2, metric, **kw), rtol=1e-4, atol=1e-5)
    with pytest.raises(RuntimeError, match="must be positive"):
        T.chi2_kernel(x1.cuda(), x2.cuda(), 1.0)


def _both_devices(fn, tensors, up):
    """fn on CPU leaves (the reference) and on CUDA leaves (these kernels): outputs and gradients of every leaf."""
    res = []
    for dev in ("cpu", "cuda"):
        leaves = [t.detach().clone().to(dev).requires_grad_(True) for t in tensors]
        out = fn(*leaves)
        out.backward(up.to(dev))
        res.append((out.detach().cpu(), [l.grad.cpu() for l in leaves]))
    return res


def test_kernel_functions_and_mahalanobis_ops(T):
    """linear / polynomial / sigmoid / rbf / laplacian kernels, mahalanobis_distances, _sqmahalanobis and its stand-alone
    backward op through the C++ layer: the reference on CPU tensors, these kernels on CUDA tensors."""
    g = torch.Generator().manual_seed(19)
    x1, x2 = torch.randn(35, 12, generator=g), torch.randn(29, 12, generator=g)
    up = torch.randn(35, 29, generator=g)
    for fn in (lambda a, b: T.linear_kernel(a, b), lambda a, b: T.polynomial_kernel(a, b, 2, 0.05, 0.5),
               lambda a, b: T.polynomial_kernel(a, b, 3, None, 1.0), lambda a, b: T.sigmoid_kernel(a, b, 0.02, 0.1),
               lambda a, b: T.sigmoid_kernel(a, b, None, 1.0), lambda a, b: T.rbf_kernel(a, b, 0.3), lambda a, b: T.rbf_kernel(a, b, None)):
        (o_ref, g_ref), (o_got, g_got) = _both_devices(fn, (x1, x2), up)
        torch.testing.assert_close(o_got, o_ref, rtol=1e-4, atol=1e-5)
        for a, b in zip(g_got, g_ref):
            torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5 * 10 * max(1.0, float(b.abs().max())))
    # the reference's own backward of laplacian_kernel fails (in-place exp on the output of cdist): forward only
    torch.testing.assert_close(T.laplacian_kernel(x1.cuda(), x2.cuda(), 0.2).cpu(), T.laplacian_kernel(x1, x2, 0.2), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(T.laplacian_kernel(x1.cuda(), None, None).cpu(), T.laplacian_kernel(x1, None, None), rtol=1e-4, atol=1e-5)
    T.laplacian_kernel(x1.cuda().requires_grad_(True), x2.cuda(), 0.2).sum().backward()  # differentiable here

    A = torch.randn(12, 12, generator=g)
    spd = A @ A.t() / 12 + 0.3 * torch.eye(12)
    skew = torch.randn(12, 12, generator=g)
    general = spd + 0.2 * (skew - skew.t())          # not symmetric; its symmetric part is positive definite
    indefinite = spd - 0.8 * torch.eye(12)           # symmetric part has negative eigenvalues: no Cholesky factor
    assert float(torch.linalg.eigvalsh(indefinite).min()) < 0
    for VI in (spd, general, indefinite):
        (o_ref, g_ref), (o_got, g_got) = _both_devices(lambda a, b, v: T._sqmahalanobis(a, b, v), (x1, x2, VI), up)
        torch.testing.assert_close(o_got, o_ref, rtol=1e-4, atol=1e-5 * max(1.0, float(o_ref.abs().max())))
        for a, b in zip(g_got, g_ref):
            torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5 * 10 * max(1.0, float(b.abs().max())))
        ref = T.__sqmahalanobis_backward(up, x1, x2, VI)
        got = T.__sqmahalanobis_backward(up.cuda(), x1.cuda(), x2.cuda(), VI.cuda())
        for a, b in zip(got, ref):
            torch.testing.assert_close(a.cpu(), b, rtol=1e-4, atol=1e-5 * 10 * max(1.0, float(b.abs().max())))
    (o_ref, g_ref), (o_got, g_got) = _both_devices(lambda a, b, v: T.mahalanobis_distances(a, b, v), (x1, x2, spd), up)
    torch.testing.assert_close(o_got, o_ref, rtol=1e-4, atol=1e-5)
    for a, b in zip(g_got, g_ref):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5 * 10 * max(1.0, float(b.abs().max())))
    # x2 = None: the default VI (inverse covariance of x1) and an exactly zero self-distance diagonal, like the reference's
    big = torch.randn(60, 12, generator=g)
    got, ref = T.mahalanobis_distances(big.cuda(), None, None).cpu(), T.mahalanobis_distances(big, None, None)
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-5)
    assert bool((got.diagonal() == 0).all())
    # near-duplicate rows keep their relative accuracy (an expansion into bilinear terms would return rounding noise)
    near = big + 1e-4 * torch.randn(60, 12, generator=g)
    got = T.mahalanobis_distances(big.cuda(), near.cuda(), spd.cuda()).cpu().diagonal()
    ref = T.mahalanobis_distances(big.double(), near.double(), spd.double()).diagonal()
    torch.testing.assert_close(got.double(), ref, rtol=2e-3, atol=0)
    got = T.snr_distances(big.cuda(), near.cuda()).cpu().diagonal()
    ref = T.snr_distances(big.double(), near.double()).diagonal()
    torch.testing.assert_close(got.double(), ref, rtol=2e-3, atol=0)
    with pytest.raises(RuntimeError, match="VI is required"):
        T.mahalanobis_distances(x1.cuda(), x2.cuda(), None)


def test_neighbour_masks_and_pdist_ops(T):
    """k_neighbors_mask / radius_neighbors_mask through the C++ layer equal the reference's masks (its composition is
    cdist + argsort / compare), on small problems and on the shapes that reach the fused kernels; pdist, which the
    reference only declares, returns the upper triangle of the reference's cdist."""
    g = torch.Generator().manual_seed(20)

    def masks_agree(x1, x2, k, metric, **kw):
        ref = T.k_neighbors_mask(x1, x2, k, metric, **kw)
        got = T.k_neighbors_mask(x1.cuda(), None if x2 is None else x2.cuda(), k, metric, **kw).cpu()
        assert got.dtype == torch.bool and got.shape == ref.shape
        assert bool((got.sum(1) == k + 1).all())
        # a row may differ only where two candidates are closer than float32 resolves
        d = T.cdist(x1.double(), (x1 if x2 is None else x2).double(), metric, **kw)
        bad = (got != ref).any(1).nonzero().flatten()
        for i in bad.tolist():
            kth = d[i].sort().values[k]
            assert float((d[i][got[i] != ref[i]] - kth).abs().max()) <= 1e-4 * max(1.0, float(kth)), (metric, i)
        assert bad.numel() <= max(1, x1.size(0) // 500)

    x1, x2 = torch.randn(40, 7, generator=g), torch.randn(33, 7, generator=g)
    for metric, kw in (("euclidean", {}), ("manhattan", {}), ("chebyshev", {}), ("minkowski", {"p": 3.0}), ("cosine", {}),
                       ("sqeuclidean", {}), ("correlation", {})):
        for k in (0, 1, 5):
            masks_agree(x1, x2, k, metric, **kw)
    masks_agree(x1, None, 3, "euclidean")
    pts1, pts2 = torch.randn(4500, 3, generator=g), torch.randn(700, 3, generator=g)
    masks_agree(pts1, pts2, 0, "euclidean")          # streaming row minimum
    masks_agree(pts1, pts2, 7, "euclidean")          # few features: k best keys per thread
    masks_agree(pts1, pts2, 3, "manhattan")
    w1, w2 = torch.randn(2048, 64, generator=g), torch.randn(2048, 64, generator=g)
    masks_agree(w1, w2, 0, "sqeuclidean")            # tensor-core row-minimum epilogue
    masks_agree(w1, w2, 4, "euclidean")              # tensor-core top-k epilogue
    with pytest.raises(RuntimeError, match="k must be non-negative"):
        T.k_neighbors_mask(x1.cuda(), x2.cuda(), -1, "euclidean")
    with pytest.raises(TypeError, match="incompatible arguments p"):
        T.k_neighbors_mask(x1.cuda(), x2.cuda(), 1, "euclidean", p=3.0)

    for a, b in ((x1, x2), (pts1, pts2), (w1[:300], w2[:200])):
        for metric, kw, eps in (("euclidean", {}, None), ("manhattan", {}, None), ("minkowski", {"p": 3.0}, None), ("cosine", {}, None)):
            d = T.cdist(a.double(), b.double(), metric, **kw)
            eps = float(d.median())
            ref = T.radius_neighbors_mask(a, b, eps, metric, **kw)
            got = T.radius_neighbors_mask(a.cuda(), b.cuda(), eps, metric, **kw).cpu()
            clear = (d - eps).abs() > 1e-4 * max(1.0, eps)
            assert got.dtype == torch.bool and torch.equal(got[clear], ref[clear]), metric
            assert torch.equal(got[clear], (d <= eps)[clear])
    with pytest.raises(RuntimeError, match="epsilon must be non-negative"):
        T.radius_neighbors_mask(x1.cuda(), x2.cuda(), -0.5, "euclidean")
    with pytest.raises(TypeError, match="incompatible arguments p"):
        T.radius_neighbors_mask(x1.cuda(), x2.cuda(), 1.0, "manhattan", p=1.0)

    with pytest.raises(NotImplementedError):
        T.pdist(x1, "euclidean")                     # the reference itself
    iu = torch.triu_indices(40, 40, offset=1)
    for metric, kw in (("euclidean", {}), ("manhattan", {}), ("minkowski", {"p": 3.0}), ("chebyshev", {}), ("cosine", {}), ("canberra", {})):
        ref = T.cdist(x1, x1, metric, **kw)[iu[0], iu[1]]
        torch.testing.assert_close(T.pdist(x1.cuda(), metric, **kw).cpu(), ref, rtol=1e-4, atol=1e-5)
    xb = torch.randn(2, 300, 20, generator=g)
    iu = torch.triu_indices(300, 300, offset=1)
    torch.testing.assert_close(T.pdist(xb.cuda(), "manhattan").cpu(), T.cdist(xb, xb, "manhattan")[:, iu[0], iu[1]], rtol=1e-4, atol=1e-5)
    leaf = x1.cuda().requires_grad_(True)
    T.pdist(leaf, "euclidean").sum().backward()      # differentiable calls gather the triangle of cdist
    assert leaf.grad is not None and bool(torch.isfinite(leaf.grad).all())


def test_cpp_layer_agrees_with_python_layer(T):
    import torchpairwise_b200 as tpw
    g = torch.Generator().manual_seed(14)
    x1, x2 = torch.randn(300, 64, generator=g).cuda(), torch.randn(200, 64, generator=g).cuda()
    for name in ("euclidean_distances", "manhattan_distances", "cosine_distances", "correlation_distances", "sqeuclidean_distances"):
        assert torch.equal(getattr(T, name)(x1, x2), getattr(tpw, name)(x1, x2)), name
    assert torch.equal(T.minkowski_distances(x1, x2, 3.0), tpw.minkowski_distances(x1, x2, 3.0))


def test_cpp_layer_dense_backward_on_tensor_cores(T, monkeypatch):
    """Above the engine threshold the C++ autograd nodes of the p = 2 metrics and the cosine family
    run the tcgen05 gradient products, blocked by the same scratch cap, and agree bit for bit with
    the Python layer, which takes the same path."""
    import torchpairwise_b200 as tpw
    from torchpairwise_b200 import _abi
    g = torch.Generator().manual_seed(15)
    x1, x2 = torch.randn(2, 2048, 64, generator=g).cuda(), torch.randn(2, 1100, 64, generator=g).cuda()
    up = torch.randn(2, 2048, 1100, generator=g).cuda()
    assert _abi.lib.tpw_dot_backward_scratch_bytes(_abi.F32, _abi.LP_BWD_MATMUL, _abi.ENGINE_AUTO, 2, 2048, 1100, 64) > 0
    per_batch = _abi.lib.tpw_dot_backward_scratch_bytes(_abi.F32, _abi.LP_BWD_MATMUL, _abi.ENGINE_TCGEN05_TF32X3, 1, 2048, 1100, 64)
    for cap in (None, 0.4 * per_batch / 2 ** 30):
        if cap is not None:
            monkeypatch.setenv("TPW_BWD_SCRATCH_GB", str(cap))   # row blocks inside each batch
        for name in ("sqeuclidean_distances", "euclidean_distances", "cosine_distances", "correlation_distances"):
            grads = []
            for fn in (getattr(T, name), getattr(tpw, name)):
                a, b = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True)
                fn(a, b).backward(up)
                grads.append((a.grad, b.grad))
            assert torch.equal(grads[0][0], grads[1][0]) and torch.equal(grads[0][1], grads[1][1]), name
            a, b = x1.double().requires_grad_(True), x2.double().requires_grad_(True)
            getattr(tpw, name)(a, b).backward(up.double())
            for got, ref in ((grads[0][0], a.grad), (grads[0][1], b.grad)):
                bound = 1e-4 * ref.abs() + 2e-5 * ref.pow(2).mean().sqrt() + 1e-5
                assert float(((got.double() - ref).abs() / bound).max()) <= 1.0, name


def test_stand_alone_registration():
    code = (
        "import torch, torchpairwise_b200 as t\n"
        "t.load_torch_ops()\n"
        "T = torch.ops.torchpairwise\n"
        "x = torch.randn(40, 16, device='cuda', requires_grad=True); y = torch.randn(30, 16, device='cuda')\n"
        "o = T.minkowski_distances(x, y, 3.0); o.sum().backward()\n"
        "assert torch.allclose(o, torch.cdist(x, y, p=3.0), rtol=1e-4, atol=1e-5)\n"
        "assert x.grad.shape == x.shape and torch.isfinite(x.grad).all()\n"
        "assert torch.equal(T.jaccard_distances(x > 0, y > 0), t.jaccard_distances(x > 0, y > 0))\n"
        "assert torch.equal(T.cdist(x, y, 'manhattan'), t.manhattan_distances(x, y))\n"
        "assert T._cuda_version() == t.cuda_version() >= 12000 and T._cuda_arch_flags() == 'sm_100a'\n"
        "assert torch.equal(T.k_neighbors_mask(x, y, 2, 'euclidean'), t.k_neighbors_mask(x, y, 2, 'euclidean'))\n"
        "assert torch.equal(T.pdist(x.detach(), 'manhattan'), t.pdist(x.detach(), 'manhattan'))\n"
        "print('standalone ok')\n"
    )
    r = subprocess.run([sys.executable, "-c", code], cwd=str(ROOT), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "standalone ok" in r.stdout, r.stdout + r.stderr
