"""Parity of the CUDA path with the reference, through the package API (which calls the C ABI).

Three sources of truth, all derived from the reference: the golden vectors it produced
(tests/golden), the numpy oracle that is pinned against those vectors, and -- at the full
benchmark sizes, where neither can run -- size-independent identities of the metrics.
"""
import math
import warnings
import zlib

import numpy as np
import pytest
import torch

from cases import (BOOL_CASES, BOOL_METRICS, FLOAT_CASES, FLOAT_METRICS, HAUSDORFF_CASES, NARROW_CASES, NARROW_METRICS,
                   call_metric, config_inputs)
from oracle import pairwise_oracle as O

pytestmark = pytest.mark.gpu

# the parity contract: fp32 rtol 1e-4 / atol 1e-5, fp64 1e-10, boolean and index outputs bit-exact
TOL = {torch.float32: dict(rtol=1e-4, atol=1e-5), torch.float64: dict(rtol=1e-10, atol=1e-10)}


@pytest.fixture(scope="module")
def tpw():
    import torchpairwise_b200
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    yield torchpairwise_b200
    assert torchpairwise_b200.device_status() == 0, "a kernel gave up a bounded wait"


def cuda(a, requires_grad=False):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.requires_grad_(True) if requires_grad else t


def close(got, ref, tol, scale=1.0, msg=""):
    ref_t = torch.from_numpy(np.asarray(ref))
    torch.testing.assert_close(got.detach().cpu(), ref_t, rtol=tol["rtol"], atol=tol["atol"] * scale,
                               equal_nan=True, msg=lambda m: f"{msg}: {m}")


@pytest.mark.parametrize("case", FLOAT_CASES, ids=lambda c: c["name"])
@pytest.mark.parametrize("metric", FLOAT_METRICS, ids=lambda m: m["name"])
def test_float_metric_golden(tpw, golden, case, metric):
    G = golden("float_metrics")
    key = f"{case['name']}/{metric['name']}"
    n = case["name"]
    weighted_batched = metric.get("weighted") and len(case["x1"]) == 3
    x1, x2 = cuda(G[f"{n}/x1"], True), cuda(G[f"{n}/x2"], True)
    w, g = cuda(G[f"{n}/w"], True), cuda(G[f"{n}/g"])
    tol = TOL[x1.dtype]
    st = case.get("stride", 1)
    out = call_metric(tpw, metric, x1, x2, w)
    if key + "/out" in G.files:
        ref_out = G[key + "/out"]
        has_grad = metric.get("grad", True)
        ref_g1, ref_g2 = (G[key + "/gx1"], G[key + "/gx2"]) if has_grad else (None, None)
        ref_gw = G[key + "/gw"] if metric.get("weighted") else None
    else:
        # batched weights with N1 != D: the reference rejects them (shape-check slip); the oracle
        # restates the same arithmetic
        assert weighted_batched
        p = metric["kw"]["p"]
        ref_out = O.wminkowski(G[f"{n}/x1"], G[f"{n}/x2"], G[f"{n}/w"], p)[..., ::st, ::st]
        ref_g1, ref_g2, ref_gw = O.wminkowski_backward(G[f"{n}/g"], G[f"{n}/x1"], G[f"{n}/x2"], G[f"{n}/w"], p)
    close(out[..., ::st, ::st], ref_out, tol, msg=key + " forward")
    if not metric.get("grad", True):
        return
    out.backward(g)
    scale = 10 * max(1.0, float(np.abs(ref_g1).max()))
    close(x1.grad, ref_g1, tol, scale, key + " grad_x1")
    close(x2.grad, ref_g2, tol, scale, key + " grad_x2")
    if ref_gw is not None:
        close(w.grad, ref_gw, tol, 10 * max(1.0, float(np.abs(ref_gw).max())), key + " grad_w")


@pytest.mark.parametrize("case", BOOL_CASES, ids=lambda c: c["name"])
def test_boolean_metrics_bit_exact(tpw, golden, case):
    G = golden("bool_metrics")
    n = case["name"]
    x1, x2 = cuda(G[f"{n}/x1"]), cuda(G[f"{n}/x2"])
    for name in BOOL_METRICS:
        if f"{n}/{name}" not in G.files:
            with pytest.raises(RuntimeError):
                getattr(tpw, name)(x1, x2)  # pw{and,or,xor}_sum are boolean-only, as in the reference
            continue
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            got = getattr(tpw, name)(x1, x2)
        ref = torch.from_numpy(G[f"{n}/{name}"])
        assert got.dtype == torch.float32
        got_c = got.cpu()
        same = (got_c == ref) | (got_c.isnan() & ref.isnan())
        assert bool(same.all()), f"{n}/{name}: {int((~same).sum())} of {ref.numel()} values differ"


def test_boolean_cast_warns(tpw):
    x = torch.randint(0, 3, (6, 9), device="cuda")
    with pytest.warns(UserWarning, match="converted to torch.bool"):
        tpw.jaccard_distances(x)
    with pytest.warns(DeprecationWarning):
        tpw.kulsinski_distances(x > 0)


@pytest.mark.parametrize("case", HAUSDORFF_CASES, ids=lambda c: c["name"])
def test_hausdorff_golden(tpw, golden, case):
    G = golden("hausdorff")
    n = case["name"]
    x1, x2, g = cuda(G[f"{n}/x1"], True), cuda(G[f"{n}/x2"], True), cuda(G[f"{n}/g"])
    out, i1, i2 = tpw.directed_hausdorff_distances(x1, x2)
    # the squared distances are accumulated with the reference's rounding, so even fp32 agrees exactly
    assert torch.equal(out.detach().cpu(), torch.from_numpy(G[f"{n}/out"]))
    assert torch.equal(i1.cpu(), torch.from_numpy(G[f"{n}/idx1"]))
    assert torch.equal(i2.cpu(), torch.from_numpy(G[f"{n}/idx2"]))
    assert i1.dtype == torch.int64 and not i1.requires_grad
    out.backward(g)
    tol = TOL[x1.dtype]
    close(x1.grad, G[f"{n}/gx1"], tol, msg=n + " grad_x1")
    close(x2.grad, G[f"{n}/gx2"], tol, msg=n + " grad_x2")


@pytest.mark.parametrize("shape", [(1, 1000, 1100, 256), (2, 700, 520, 400), (1, 130, 4100, 1024), (1, 2100, 1300, 144), (1, 300, 900, 1200)])
def test_boolean_tensor_core_counts_equal_popcount_counts(tpw, monkeypatch, shape):
    """The boolean family with the pair counts taken on the tensor cores (8-bit integer contraction of the 0 / 1 bytes)
    returns, for every metric, exactly the bits of the popcount kernel, which the golden vectors pin to the
    reference: ragged row counts, feature counts that are not a multiple of the 128-feature step, batches, a set
    against itself, and degenerate all-zero / all-one rows (the 0/0 branches)."""
    from torchpairwise_b200 import _abi
    b, n1, n2, d = shape
    assert _abi.lib.tpw_bool_metric_tc_eligible(b, n1, n2, d) == 1
    g = torch.Generator().manual_seed(n1 + n2 + d)
    x1 = (torch.rand(b, n1, d, generator=g) < 0.1).cuda()
    x2 = (torch.rand(b, n2, d, generator=g) < 0.3).cuda()
    x1[:, 0] = False
    x2[:, 0] = False
    x1[:, 1] = True
    x2[:, 1] = True
    if b == 1:
        x1, x2 = x1[0], x2[0]
    names = ["hamming", "jaccard", "kulsinski", "kulczynski1", "yule", "dice", "rogerstanimoto", "russellrao", "sokalmichener", "sokalsneath"]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for name in names:
            fn = getattr(tpw, name + "_distances")
            monkeypatch.delenv("TPW_DISABLE_BOOL_TC", raising=False)
            got = fn(x1, x2)
            got_self = fn(x1)
            monkeypatch.setenv("TPW_DISABLE_BOOL_TC", "1")
            ref, ref_self = fn(x1, x2), fn(x1)
            monkeypatch.delenv("TPW_DISABLE_BOOL_TC", raising=False)
            assert bool(((got == ref) | (got.isnan() & ref.isnan())).all()), name
            assert bool(((got_self == ref_self) | (got_self.isnan() & ref_self.isnan())).all()), name + " (self)"
        for name in ("pwand_sum", "pwor_sum", "pwxor_sum", "pweq_sum", "pwne_sum", "pweq_mean", "pwne_mean"):
            fn = getattr(tpw, name)
            got = fn(x1, x2)
            monkeypatch.setenv("TPW_DISABLE_BOOL_TC", "1")
            ref = fn(x1, x2)
            monkeypatch.delenv("TPW_DISABLE_BOOL_TC", raising=False)
            assert torch.equal(got, ref), name
        # the staged tiles leave either through the warp's own stores or through the output's tensor map (the default
        # depends on the metric): both ways write the same bits, ragged last rows and columns included
        for name in ("hamming_distances", "jaccard_distances", "pwand_sum"):
            fn = getattr(tpw, name)
            res = []
            for how in ("plain", "tma"):
                monkeypatch.setenv("TPW_BOOL_TC_STORES", how)
                res.append(fn(x1, x2))
            monkeypatch.delenv("TPW_BOOL_TC_STORES", raising=False)
            assert torch.equal(res[0], res[1]), name
    # against the oracle's integer counts directly
    a, c = (x1, x2) if x1.dim() == 2 else (x1[0], x2[0])
    assert np.array_equal(tpw.jaccard_distances(a, c).cpu().numpy(), O.boolean_metric("jaccard", a.cpu().numpy(), c.cpu().numpy()))
    assert _abi.lib.tpw_bool_metric_tc_eligible(1, 64, 4096, 1024) == 0      # fewer rows than a tile
    assert _abi.lib.tpw_bool_metric_tc_eligible(1, 1000, 1100, 250) == 0     # rows not 16-byte aligned


@pytest.mark.parametrize("d", [1, 3, 4, 7, 8, 11, 16])
def test_hausdorff_fused_loop_equals_exact_loop(tpw, monkeypatch, d):
    """The hot loop that forms squared distances with fused multiply-adds and refines the few rows near the maximum
    returns the same bits -- values and both index tensors -- as evaluating every point pair in the reference's
    separately rounded arithmetic, on continuous clouds, on a cloud against itself (every row minimum is 0), on
    lattice points (most rows tie) and with a caller-chosen visiting order."""
    g = torch.Generator().manual_seed(40 + d)
    clouds = [
        (torch.rand(2, 2, 3000, d, generator=g), torch.rand(2, 3, 2500, d, generator=g)),
        (torch.randint(0, 3, (1, 2, 1300, d), generator=g).float(), torch.randint(0, 3, (1, 2, 1100, d), generator=g).float() + 0.5),
    ]
    same = torch.rand(1, 1, 2100, d, generator=g)
    clouds.append((same, same.clone()))
    for x1, x2 in clouds:
        for shuffle in (False, True):
            res = []
            for exact in (False, True):
                if exact:
                    monkeypatch.setenv("TPW_HAUSDORFF_EXACT_LOOP", "1")
                else:
                    monkeypatch.delenv("TPW_HAUSDORFF_EXACT_LOOP", raising=False)
                gen = torch.Generator(device="cuda").manual_seed(5)
                res.append(tpw.directed_hausdorff_distances(x1.cuda(), x2.cuda(), shuffle=shuffle, generator=gen if shuffle else None))
            monkeypatch.delenv("TPW_HAUSDORFF_EXACT_LOOP", raising=False)
            for a, b in zip(*res):
                assert torch.equal(a, b), (d, shuffle)
            if not shuffle:
                o_ref, i_ref, j_ref = O.directed_hausdorff(x1.numpy(), x2.numpy())
                assert np.array_equal(res[0][0].cpu().numpy(), o_ref)
                assert np.array_equal(res[0][1].cpu().numpy(), i_ref) and np.array_equal(res[0][2].cpu().numpy(), j_ref)


@pytest.mark.parametrize("d", [1, 3, 8, 12])
def test_hausdorff_float64_streamed_equals_one_cta_per_pair(tpw, monkeypatch, d):
    """float64 clouds of up to sixteen coordinates take the streamed kernels (row minima in scratch, one scan per
    set pair); values and both index tensors equal the one-CTA-per-pair kernel's and the oracle's bit for bit,
    also where most rows tie and with a caller-chosen visiting order."""
    g = torch.Generator().manual_seed(70 + d)
    clouds = [
        (torch.rand(2, 2, 1500, d, generator=g, dtype=torch.float64), torch.rand(2, 3, 1200, d, generator=g, dtype=torch.float64)),
        (torch.randint(0, 3, (1, 2, 700, d), generator=g).double(), torch.randint(0, 3, (1, 2, 600, d), generator=g).double() + 0.5),
        (torch.rand(1, 1, 5, d, generator=g, dtype=torch.float64), torch.rand(1, 2, 3, d, generator=g, dtype=torch.float64)),
    ]
    same = torch.rand(1, 1, 900, d, generator=g, dtype=torch.float64)
    clouds.append((same, same.clone()))
    for x1, x2 in clouds:
        for shuffle in (False, True):
            res = []
            for plain in (False, True):
                if plain:
                    monkeypatch.setenv("TPW_HAUSDORFF_PLAIN_F64", "1")
                else:
                    monkeypatch.delenv("TPW_HAUSDORFF_PLAIN_F64", raising=False)
                gen = torch.Generator(device="cuda").manual_seed(5)
                res.append(tpw.directed_hausdorff_distances(x1.cuda(), x2.cuda(), shuffle=shuffle, generator=gen if shuffle else None))
            monkeypatch.delenv("TPW_HAUSDORFF_PLAIN_F64", raising=False)
            for a, b in zip(*res):
                assert torch.equal(a, b), (d, shuffle)
            if not shuffle:
                o_ref, i_ref, j_ref = O.directed_hausdorff(x1.numpy(), x2.numpy())
                assert np.array_equal(res[0][0].cpu().numpy(), o_ref)
                assert np.array_equal(res[0][1].cpu().numpy(), i_ref) and np.array_equal(res[0][2].cpu().numpy(), j_ref)


def test_hausdorff_shuffle_and_cdist(tpw):
    g = torch.Generator().manual_seed(3)
    x1 = torch.rand(2, 3, 40, 3, generator=g).cuda()
    x2 = torch.rand(2, 2, 31, 3, generator=g).cuda()
    ref, r1, r2 = tpw.directed_hausdorff_distances(x1, x2)
    gen = torch.Generator(device="cuda").manual_seed(5)
    out, i1, i2 = tpw.directed_hausdorff_distances(x1, x2, shuffle=True, generator=gen)
    assert torch.equal(out, ref)  # visiting order never changes the value
    # random data has no ties, so the indices agree as well
    assert torch.equal(i1, r1) and torch.equal(i2, r2)
    assert torch.equal(tpw.cdist(x1, x2, "directed_hausdorff"), ref)
    # with exact ties the shuffled indices follow visiting order; the attained distance is still the output
    xi = torch.randint(0, 3, (1, 2, 30, 3), generator=g).float().cuda()
    yi = torch.randint(0, 3, (1, 2, 33, 3), generator=g).float().cuda() + 0.5
    out, i1, i2 = tpw.directed_hausdorff_distances(xi, yi, shuffle=True, generator=gen)
    for i in range(2):
        for j in range(2):
            d = (xi[0, i, i1[0, i, j]] - yi[0, j, i2[0, i, j]]).pow(2).sum().sqrt()
            assert torch.equal(d, out[0, i, j])
    o_ref, _, _ = O.directed_hausdorff(xi.cpu().numpy(), yi.cpu().numpy())
    assert np.array_equal(out.cpu().numpy(), o_ref)


def test_config_shaped_golden(tpw, golden):
    """Row blocks of the benchmark configurations, a block of X against ALL of Y (C2: one batch, 512 rows x 4096 with
    both gradients; C3 / C4: 1024 rows x 16384; C1 and C5 whole), against the reference's outputs.  At these sizes the
    engine rule picks what runs the full configurations: the tensor-core contraction for C4, the tensor-core counts
    for C3, the match-and-scatter backward for chebyshev."""
    from torchpairwise_b200 import _abi
    assert _abi.lib.tpw_dot_metric_scratch_bytes(_abi.F32, _abi.ENGINE_AUTO, 1, 1024, 16384, 512) > 0
    assert _abi.lib.tpw_bool_metric_tc_eligible(1, 1024, 16384, 1024) == 1
    assert _abi.lib.tpw_chebyshev_backward_scratch_bytes(_abi.F32, 1, 512, 4096, 256) > 0
    G = golden("configs")

    def inputs(name):
        ts = config_inputs(name)
        chk = np.array([t.double().sum().item() for t in ts])
        if not np.array_equal(chk, G[f"{name}/checksum"]):
            pytest.skip("this torch build generates different seeded inputs than the one that made the vectors")
        return ts

    tol = TOL[torch.float32]
    X, Y = inputs("C1")
    for name in ("euclidean_distances", "manhattan_distances", "cosine_distances", "chebyshev_distances",
                 "sqeuclidean_distances", "correlation_distances"):
        close(getattr(tpw, name)(X.cuda(), Y.cuda())[::128], G[f"C1/{name}"], tol, msg="C1 " + name)
    X, Y, Gr = inputs("C2")
    for name, fn in (("minkowski3", lambda a, b: tpw.minkowski_distances(a, b, 3.0)),
                     ("chebyshev", lambda a, b: tpw.chebyshev_distances(a, b))):
        a, b = X.cuda().requires_grad_(True), Y.cuda().requires_grad_(True)
        res = fn(a, b)
        res.backward(Gr.cuda())
        close(res[:, ::8, ::16], G[f"C2/{name}/out"], tol, msg="C2 " + name)
        scale = 10 * float(np.abs(G[f"C2/{name}/gx1"]).max())
        close(a.grad[:, ::8], G[f"C2/{name}/gx1"], tol, scale, "C2 grad_x1 " + name)
        close(b.grad[:, ::16], G[f"C2/{name}/gx2"], tol, scale, "C2 grad_x2 " + name)
    X, Y = inputs("C3")
    for name in ("hamming_distances", "jaccard_distances"):
        got = getattr(tpw, name)(X.cuda(), Y.cuda())[::16, ::64].cpu()
        assert torch.equal(got, torch.from_numpy(G[f"C3/{name}"])), name
    X, Y = inputs("C4")
    for name in ("sqeuclidean_distances", "cosine_distances"):
        close(getattr(tpw, name)(X.cuda(), Y.cuda())[::16, ::64], G[f"C4/{name}"], tol, msg="C4 " + name)
    X, Y = inputs("C5")
    a, b = X.cuda().requires_grad_(True), Y.cuda().requires_grad_(True)
    res, i1, i2 = tpw.directed_hausdorff_distances(a, b)
    assert torch.equal(res.detach().cpu(), torch.from_numpy(G["C5/out"]))
    assert torch.equal(i1.cpu(), torch.from_numpy(G["C5/idx1"])) and torch.equal(i2.cpu(), torch.from_numpy(G["C5/idx2"]))
    res.backward(torch.ones_like(res))
    r1 = torch.from_numpy(G["C5/gx1_rows"])
    close(a.grad.cpu()[tuple(r1.t())], G["C5/gx1_vals"], tol, msg="C5 grad_x1")
    assert int((a.grad.abs().sum(-1) != 0).sum()) == r1.shape[0]
    r2 = torch.from_numpy(G["C5/gx2_rows"])
    close(b.grad.cpu()[tuple(r2.t())], G["C5/gx2_vals"], tol, msg="C5 grad_x2")


@pytest.mark.parametrize("p", [1.0, 2.0, 3.0, 2.5, math.inf])
def test_small_problem_backward_kernel_is_bit_identical_to_tile_kernel(tpw, monkeypatch, p):
    """Problems with few 128 x 128 gradient blocks run the backward with one thread per gradient element; it adds the same
    terms in the same order as the tile kernel, so both gradients agree bit for bit (and with the oracle)."""
    from torchpairwise_b200 import _abi
    g = torch.Generator().manual_seed(int(p * 10) if math.isfinite(p) else 77)
    for shape in ((1, 300, 500, 12), (2, 130, 70, 100), (1, 1024, 2048, 128)):
        b, n1, n2, d = shape
        x1, x2 = torch.randn(b, n1, d, generator=g).cuda(), torch.randn(b, n2, d, generator=g).cuda()
        gr = torch.randn(b, n1, n2, generator=g).cuda()
        out = tpw.minkowski_distances(x1, x2, p) if math.isfinite(p) else tpw.chebyshev_distances(x1, x2)
        res = []
        for tile in (False, True):
            if tile:
                monkeypatch.setenv("TPW_DISABLE_SMALL_BWD", "1")
            else:
                monkeypatch.delenv("TPW_DISABLE_SMALL_BWD", raising=False)
            g1, g2 = torch.empty_like(x1), torch.empty_like(x2)
            _abi.check(_abi.lib.tpw_lp_backward(_abi.F32, _abi.LP_BWD_CDIST, gr.data_ptr(), out.data_ptr(), x1.data_ptr(), x2.data_ptr(), None,
                                                g1.data_ptr(), g2.data_ptr(), b, n1, n2, d, p, torch.cuda.current_stream().cuda_stream))
            res.append((g1, g2))
        monkeypatch.delenv("TPW_DISABLE_SMALL_BWD", raising=False)
        assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1]), shape
        r1, r2 = O.cdist_backward(gr.cpu().numpy(), x1.cpu().numpy(), x2.cpu().numpy(), p, out=out.cpu().numpy())
        scale = 10 * max(1.0, float(np.abs(r1).max()))
        close(res[0][0], r1, TOL[torch.float32], scale, "grad_x1")
        close(res[0][1], r2, TOL[torch.float32], scale, "grad_x2")


@pytest.mark.parametrize("mode,p", [("cdist", 1.0), ("cdist", 2.0), ("cdist", 3.0), ("cdist", 2.5), ("pp", 3.0), ("pp", 1.5), ("w", 3.0), ("w", 1.5)])
def test_one_pass_backward(tpw, mode, p):
    """The backward that forms a pair's term once and adds it to both gradient sums (`tpw_lp_backward_ws`) against the
    oracle and against the two-launch kernel, on shapes with ragged row blocks, ragged feature tiles and a ragged
    last stage; bit-reproducible from call to call, and unchanged to rounding when a small scratch forces several
    launches over batch ranges or over row-block ranges (whose sums are then accumulated into grad_x2)."""
    from torchpairwise_b200 import _abi
    lib = _abi.lib
    code = {"cdist": _abi.LP_BWD_CDIST, "pp": _abi.LP_BWD_PPMINKOWSKI, "w": _abi.LP_BWD_WMINKOWSKI}[mode]
    g = torch.Generator().manual_seed(int(p * 10) + len(mode))
    stream = torch.cuda.current_stream().cuda_stream
    for shape in ((10, 1000, 300, 208), (3, 2560, 140, 256), (80, 256, 256, 64)):
        b, n1, n2, d = shape
        x1, x2 = torch.randn(b, n1, d, generator=g).cuda(), torch.randn(b, n2, d, generator=g).cuda()
        gr = torch.randn(b, n1, n2, generator=g).cuda()
        w = (torch.rand(b, d, generator=g) + 0.5).cuda() if mode == "w" else None
        if mode == "cdist":
            aux = tpw.minkowski_distances(x1, x2, p) if p != 1.0 else None
        elif mode == "w":
            aux = (torch.rand(b, n1, n2, generator=g) + 0.5).cuda()
        else:
            aux = None
        ptr = lambda t: None if t is None else t.data_ptr()
        want = lib.tpw_lp_backward_scratch_bytes(_abi.F32, code, b, n1, n2, d, p)
        assert want > 0, shape
        slab = n2 * d * 4
        blocks = (n1 + 255) // 256

        def run(nbytes):
            g1, g2 = torch.full_like(x1, float("nan")), torch.full_like(x2, float("nan"))
            if nbytes is None:
                _abi.check(lib.tpw_lp_backward(_abi.F32, code, ptr(gr), ptr(aux), ptr(x1), ptr(x2), ptr(w), ptr(g1), ptr(g2),
                                               b, n1, n2, d, p, stream))
            else:
                scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
                _abi.check(lib.tpw_lp_backward_ws(_abi.F32, code, ptr(gr), ptr(aux), ptr(x1), ptr(x2), ptr(w), ptr(g1), ptr(g2),
                                                  b, n1, n2, d, p, ptr(scratch), nbytes, stream))
            assert _abi.device_status(stream) == 0
            return g1, g2

        two = run(None)
        one = run(want)
        again = run(want)
        assert torch.equal(one[0], again[0]) and torch.equal(one[1], again[1]), shape
        scale = float(two[0].abs().max()) + float(two[1].abs().max())
        for nbytes in (want, slab * blocks * 2, slab * max(1, blocks - 1), slab):
            res = run(nbytes)
            for a, r in zip(res, two):
                assert not torch.isnan(a).any()
                assert float((a - r).abs().max()) <= 2e-5 * scale, (shape, nbytes)
        # oracle: float64 autograd of the same composite
        a64, b64 = x1.double().requires_grad_(), x2.double().requires_grad_()
        if mode == "cdist":
            torch.cdist(a64, b64, p=p).backward(gr.double())
        elif mode == "pp":
            ((a64[:, :, None, :] - b64[:, None, :, :]).abs() ** p).sum(-1).backward(gr.double())
        else:
            # _wminkowski backward with S^(1/p-1) replaced by the given auxiliary matrix
            (((a64[:, :, None, :] - b64[:, None, :, :]).abs() ** p * w.double()[:, None, None, :]).sum(-1) / p).backward((gr * aux).double())
        s1 = max(1.0, float(a64.grad.abs().max()))
        assert float((one[0].double() - a64.grad).abs().max()) <= 1e-4 * s1, (shape, "grad_x1")
        assert float((one[1].double() - b64.grad).abs().max()) <= 1e-4 * max(1.0, float(b64.grad.abs().max())), (shape, "grad_x2")


@pytest.mark.parametrize("shape", [(1, 70, 50, 16), (2, 129, 67, 36), (1, 64, 64, 70), (2, 200, 333, 300), (1, 300, 130, 257)])
@pytest.mark.parametrize("lattice", [False, True])
def test_chebyshev_backward_match_and_scatter(tpw, shape, lattice):
    """The Chebyshev backward that finds each pair's attaining coordinate once and scatters both gradients against the
    oracle (ATen's rule: every tied coordinate receives the gradient) and, bit for bit, against the dense kernel.
    Lattice-valued inputs have tied maxima in most pairs and take the on-device hand-over to the dense kernel, the
    continuous inputs carry three engineered ties that the scatter kernels resolve themselves; D = 70 is not a
    multiple of 16 bytes (plain loads instead of TMA), D = 300 and 257 span two feature blocks of the scatter."""
    from torchpairwise_b200 import _abi
    b, n1, n2, d = shape
    g = torch.Generator().manual_seed(b * 7 + n1 + n2 + d + int(lattice))
    if lattice:
        x1 = torch.randint(0, 4, (b, n1, d), generator=g).float()
        x2 = torch.randint(0, 4, (b, n2, d), generator=g).float()
        x2[:, 0] = x1[:, 0]                       # one pair at distance 0: no gradient
    else:
        x1, x2 = torch.randn(b, n1, d, generator=g), torch.randn(b, n2, d, generator=g)
        # a few exactly tied maxima (opposite signs, three-way), handled pair by pair inside the scatter kernels
        for r, c, ks, vals in ((0, 0, (1, d - 1), (9.0, -9.0)), (n1 - 1, n2 - 1, (0, 3, d - 2), (-8.5, -8.5, 8.5)), (n1 // 2, 1, (2, 5), (7.0, 7.0))):
            for k, v in zip(ks, vals):
                x2[0, c, k] = 0.0
                x1[0, r, k] = v
    gr = torch.randn(b, n1, n2, generator=g)
    assert _abi.lib.tpw_chebyshev_backward_scratch_bytes(_abi.F32, b, n1, n2, d) == 256 + 4 * b * n1 * n2
    a, c = x1.cuda().requires_grad_(True), x2.cuda().requires_grad_(True)
    out = tpw.chebyshev_distances(a, c)
    out.backward(gr.cuda())
    r1, r2 = O.cdist_backward(gr.numpy(), x1.numpy(), x2.numpy(), math.inf, out=out.detach().cpu().numpy())
    scale = 10 * max(1.0, float(np.abs(r1).max()))
    close(a.grad, r1, TOL[torch.float32], scale, "grad_x1")
    close(c.grad, r2, TOL[torch.float32], scale, "grad_x2")
    # the dense kernel on the same inputs
    d1, d2 = torch.empty_like(a.grad), torch.empty_like(c.grad)
    _abi.check(_abi.lib.tpw_lp_backward(_abi.F32, _abi.LP_BWD_CDIST, gr.cuda().data_ptr(), out.data_ptr(), a.data_ptr(), c.data_ptr(),
                                        None, d1.data_ptr(), d2.data_ptr(), b, n1, n2, d, math.inf,
                                        torch.cuda.current_stream().cuda_stream))
    if lattice:
        assert torch.equal(a.grad, d1) and torch.equal(c.grad, d2)     # the fallback is that kernel
    else:
        torch.testing.assert_close(a.grad, d1, rtol=1e-5, atol=1e-5 * scale)   # same terms, another order of addition
        torch.testing.assert_close(c.grad, d2, rtol=1e-5, atol=1e-5 * scale)
    # run to run reproducible, and one-sided calls leave the other gradient alone
    a2, c2 = x1.cuda().requires_grad_(True), x2.cuda()
    tpw.chebyshev_distances(a2, c2).backward(gr.cuda())
    assert torch.equal(a2.grad, a.grad)
    assert _abi.lib.tpw_chebyshev_backward_scratch_bytes(_abi.F64, b, n1, n2, d) == 0
    assert _abi.lib.tpw_chebyshev_backward_scratch_bytes(_abi.F32, b, n1, n2, 8) == 0


@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 1, 2), (129, 127, 33), (2, 257, 130), (50, 300, 7), (64, 64, 260)])
@pytest.mark.parametrize("p", [1.0, 2.0, 3.0, 2.5, math.inf])
def test_ragged_shapes_vs_oracle(tpw, shape, p):
    n1, n2, d = shape
    g = torch.Generator().manual_seed(n1 * 1000 + n2 * 10 + d)
    x1 = torch.randn(2, n1, d, generator=g)
    x2 = torch.randn(2, n2, d, generator=g)
    gr = torch.randn(2, n1, n2, generator=g)
    a, b = x1.cuda().requires_grad_(True), x2.cuda().requires_grad_(True)
    out = tpw.minkowski_distances(a, b, p)
    ref = O.cdist(x1.numpy(), x2.numpy(), p)
    tol = TOL[torch.float32]
    close(out, ref, tol, msg=f"forward {shape} p={p}")
    out.backward(gr.cuda())
    # the oracle's backward in float64 from the same inputs: the tolerance then only sees our rounding
    g1, g2 = O.cdist_backward(gr.double().numpy(), x1.double().numpy(), x2.double().numpy(), p)
    if math.isinf(p):
        g1, g2 = O.cdist_backward(gr.numpy(), x1.numpy(), x2.numpy(), p, out=out.detach().cpu().numpy())
    scale = 10 * max(1.0, float(np.abs(g1).max()))
    close(a.grad, g1.astype(np.float32), tol, scale, f"grad_x1 {shape} p={p}")
    close(b.grad, g2.astype(np.float32), tol, scale, f"grad_x2 {shape} p={p}")


@pytest.mark.parametrize("d", [1, 3, 4, 7, 8, 13, 16, 17, 31, 32])
@pytest.mark.parametrize("p", [1.0, 2.0, 3.0, math.inf])
def test_few_feature_kernel_vs_oracle_and_tile_kernel(tpw, monkeypatch, d, p):
    """D <= 32 on enough rows and columns takes the streaming few-feature kernel: against the oracle on ragged
    sizes (row count not a multiple of 128, column count odd, so the scalar-store edge is taken), on an
    unaligned-width output, and bit for bit against the tile kernel, which accumulates in the same order."""
    g = torch.Generator().manual_seed(300 + d)
    for n1, n2 in ((131, 1029), (256, 2048)):
        x1, x2 = torch.randn(2, n1, d, generator=g), torch.randn(2, n2, d, generator=g)
        a, b = x1.cuda(), x2.cuda()
        out = tpw.minkowski_distances(a, b, p)
        close(out, O.cdist(x1.numpy(), x2.numpy(), p), TOL[torch.float32], msg=f"few features D={d} p={p} {n1}x{n2}")
        if p == 2.0:
            sq_small = tpw.sqeuclidean_distances(a, b)
            close(sq_small, O.cdist(x1.numpy(), x2.numpy(), 2.0) ** 2, TOL[torch.float32], msg="sqeuclidean")
        monkeypatch.setenv("TPW_DISABLE_SMALL_D", "1")
        tile = tpw.minkowski_distances(a, b, p)
        if p == 2.0:   # the approximate square root of the few-feature kernel is within 1 ulp of the tile kernel's
            assert bool(((out - tile).abs() <= 1.2e-7 * tile.abs()).all())
            assert torch.equal(tpw.sqeuclidean_distances(a, b), sq_small)
        else:
            assert torch.equal(out, tile), f"D={d} p={p} {n1}x{n2}: max diff {float((out - tile).abs().max())}"
        monkeypatch.delenv("TPW_DISABLE_SMALL_D")


@pytest.mark.parametrize("d", [1, 31, 32, 33, 64, 100, 128])
def test_few_words_boolean_kernel_is_bit_exact(tpw, monkeypatch, d):
    """Boolean rows of at most 128 bits on enough rows and columns take the streaming few-words kernel: every
    boolean metric and the pw*_sum / mean counts equal the tile kernel bit for bit (NaN where it has NaN), and
    jaccard / hamming equal the oracle, on ragged sizes and on sizes that take the 128-bit stores."""
    g = torch.Generator().manual_seed(400 + d)
    names = ("hamming", "jaccard", "kulsinski", "kulczynski1", "yule", "dice", "rogerstanimoto", "russellrao",
             "sokalmichener", "sokalsneath")
    for n1, n2 in ((131, 2051), (256, 4096)):
        xb, yb = torch.rand(n1, d, generator=g) < 0.3, torch.rand(n2, d, generator=g) < 0.3
        xb[0] = False   # an empty row: the 0/0 cases of the ratios
        yb[1] = False
        a, b = xb.cuda(), yb.cuda()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            small = {n: getattr(tpw, n + "_distances")(a, b) for n in names}
            small.update({n: getattr(tpw, n)(a, b) for n in ("pwand_sum", "pwor_sum", "pwxor_sum", "pweq_sum", "pwne_mean")})
            monkeypatch.setenv("TPW_DISABLE_SMALL_D", "1")
            tile = {n: getattr(tpw, n + "_distances")(a, b) for n in names}
            tile.update({n: getattr(tpw, n)(a, b) for n in ("pwand_sum", "pwor_sum", "pwxor_sum", "pweq_sum", "pwne_mean")})
            monkeypatch.delenv("TPW_DISABLE_SMALL_D")
        for n in small:
            s_, t_ = small[n], tile[n]
            assert bool(((s_ == t_) | (s_.isnan() & t_.isnan())).all()), (n, d, n1, n2)
        assert np.array_equal(small["jaccard"].cpu().numpy(), O.boolean_metric("jaccard", xb.numpy(), yb.numpy())), d
        assert np.array_equal(small["hamming"].cpu().numpy(), O.hamming(xb.numpy(), yb.numpy())), d


@pytest.mark.parametrize("d", [1, 3, 4, 8, 13, 16, 32])
@pytest.mark.parametrize("metric,p", [("manhattan", None), ("sqeuclidean", None), ("euclidean", None), ("chebyshev", None), ("minkowski", 3.0)])
def test_few_feature_row_minimum(tpw, monkeypatch, d, metric, p):
    """Nearest x2 row on few features (streaming kernel with the x1 rows in registers) against the tile kernel's
    row-minimum epilogue: the same column and the same value (within 1 ulp where the two use different square
    roots), against the matrix written for the same problem (bit-identical), with exact duplicates (ties go to
    the smaller x2 row) and ragged sizes; and against the float64 oracle."""
    g = torch.Generator().manual_seed(500 + d)
    for n1, n2 in ((2051, 131), (2304, 1500)):
        x1, x2 = torch.randn(2, n1, d, generator=g), torch.randn(2, n2, d, generator=g)
        x2[:, 77] = x2[:, 5]          # duplicates: ties
        x1[:, 9] = x2[:, 5]
        a, b = x1.cuda(), x2.cuda()
        arg, mn = tpw.pairwise_argmin_min(a, b, metric, p)
        full = tpw.cdist(a, b, metric, p=p) if p is not None else tpw.cdist(a, b, metric)
        assert torch.equal(full.min(-1).values, mn), (metric, d, n1, n2)
        assert torch.equal(full.gather(-1, arg.unsqueeze(-1))[..., 0], mn)
        assert int(arg[0, 9]) == 5 and float(mn[0, 9]) == 0.0
        monkeypatch.setenv("TPW_DISABLE_SMALL_D", "1")
        arg_t, mn_t = tpw.pairwise_argmin_min(a, b, metric, p)
        monkeypatch.delenv("TPW_DISABLE_SMALL_D")
        assert bool(((mn - mn_t).abs() <= 1.2e-7 * mn_t.abs()).all())
        if metric != "euclidean":
            assert torch.equal(arg, arg_t) and torch.equal(mn, mn_t)
        pp = {"manhattan": 1.0, "sqeuclidean": 2.0, "euclidean": 2.0, "chebyshev": math.inf, "minkowski": 3.0}[metric]
        ref = O.cdist(x1.double().numpy(), x2.double().numpy(), pp)
        ref = ref * ref if metric == "sqeuclidean" else ref
        close(mn.double(), ref.min(-1), TOL[torch.float32], msg="row minimum")
        picked = np.take_along_axis(ref, arg.cpu().numpy()[..., None], -1)[..., 0]
        np.testing.assert_allclose(picked, ref.min(-1), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("d", [1, 2, 3, 4, 7, 8, 12, 16])
@pytest.mark.parametrize("metric,kw,k", [("euclidean", {}, 8), ("sqeuclidean", {}, 1), ("manhattan", {}, 16), ("chebyshev", {}, 5),
                                         ("minkowski", {"p": 3.0}, 3)])
def test_few_feature_k_nearest(tpw, d, metric, kw, k):
    """The streaming k-nearest kernel on few features against a partial selection on the matrix of the same problem:
    the same ascending values bit for bit, valid distinct columns that attain them, exact duplicates resolved to
    the smaller x2 row, ragged sizes, batched inputs; and the neighbour mask built from it."""
    g = torch.Generator().manual_seed(600 + d)
    for shape1, shape2 in (((4099, d), (333, d)), ((2, 2100, d), (2, 1030, d))):
        x1, x2 = torch.randn(*shape1, generator=g), torch.randn(*shape2, generator=g)
        x2[..., 40, :] = x2[..., 7, :]      # a duplicate: ties between columns 7 and 40
        x1[..., 3, :] = x2[..., 7, :]
        a, b = x1.cuda(), x2.cuda()
        inds, vals = tpw.pairwise_argkmin(a, b, k, metric, **kw)
        assert inds.shape == (*shape1[:-1], k) and inds.dtype == torch.int64 and vals.dtype == torch.float32
        full = tpw.cdist(a, b, metric, **kw)
        ref_vals = full.topk(k, dim=-1, largest=False, sorted=True).values
        assert torch.equal(vals, ref_vals), (metric, d)
        assert torch.equal(full.gather(-1, inds), vals)
        assert int((inds.sort(-1).values.diff(dim=-1) == 0).sum()) == 0          # distinct columns
        row = inds[3] if len(shape1) == 2 else inds[0, 3]
        assert int(row[0]) == 7 and (k == 1 or int(row[1]) == 40)
    if metric == "euclidean":
        xs = torch.randn(4200, d, generator=g).cuda()
        mask = tpw.k_neighbors_mask(xs, None, 4, metric)
        assert mask.dtype == torch.bool and bool((mask.sum(-1) == 5).all()) and bool(mask.diagonal().all())
        assert torch.equal(mask, tpw.k_neighbors_mask(xs.double(), None, 4, metric)) or \
            int((mask != tpw.k_neighbors_mask(xs.double(), None, 4, metric)).sum()) <= 8     # float32 / float64 near ties


def test_tma_and_plain_load_paths_agree(tpw):
    """An input whose base address is not 16-byte aligned takes the guarded plain-load path; it
    stages the same layout, so results are bit-identical to the TMA path."""
    g = torch.Generator().manual_seed(9)
    x1 = torch.randn(200, 64, generator=g).cuda()
    x2 = torch.randn(150, 64, generator=g).cuda()
    gr = torch.randn(200, 150, generator=g).cuda()

    def shifted(t):
        buf = torch.empty(t.numel() + 1, device="cuda", dtype=t.dtype)
        view = buf[1:].view(t.shape)
        view.copy_(t)
        assert view.data_ptr() % 16 != 0
        return view

    for p in (1.0, 3.0, math.inf, 2.5):
        a, b = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True)
        o1 = tpw.minkowski_distances(a, b, p)
        o1.backward(gr)
        a2, b2 = shifted(x1).requires_grad_(True), shifted(x2).requires_grad_(True)
        o2 = tpw.minkowski_distances(a2, b2, p)
        o2.backward(shifted(gr))
        assert torch.equal(o1, o2), p
        assert torch.equal(a.grad, a2.grad) and torch.equal(b.grad, b2.grad), p
    xb = torch.rand(70, 300, generator=g).cuda() < 0.2
    assert torch.equal(tpw.jaccard_distances(xb), tpw.jaccard_distances(shifted(xb)))


def test_self_distances_and_empty_inputs(tpw):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(40, 16, generator=g).cuda()
    # x2 = None means (x1, x1); the direct-difference form gives an exactly zero diagonal
    assert torch.equal(tpw.sqeuclidean_distances(x).diagonal(), torch.zeros(40, device="cuda"))
    assert torch.equal(tpw.euclidean_distances(x).diagonal(), torch.zeros(40, device="cuda"))
    assert torch.equal(tpw.manhattan_distances(x), tpw.manhattan_distances(x, x))
    e = torch.empty(0, 16, device="cuda")
    assert tpw.euclidean_distances(e, x).shape == (0, 40)
    assert tpw.euclidean_distances(x, e).shape == (40, 0)
    assert tpw.jaccard_distances(e > 0, x > 0).shape == (0, 40)
    xr = x.clone().requires_grad_(True)
    tpw.minkowski_distances(xr, e, 3.0).sum().backward()
    assert torch.equal(xr.grad, torch.zeros_like(xr))


@pytest.mark.parametrize("case", NARROW_CASES, ids=lambda c: c["name"])
def test_narrow_inputs_between_reference_and_float64(tpw, golden, case):
    """float16 / bfloat16 inputs.  The reference's kernels accumulate in the narrow type; this library widens to float32,
    accumulates there and rounds the result once.  Both are compared with the same operator evaluated in float64 on
    the same narrow inputs: this library's error is at most the reference's plus one rounding of the output type,
    and the two differ by no more than the reference's own accumulation error allows."""
    G = golden("narrow")
    n = case["name"]
    dt = case["dtype"]
    ulp = 2.0 ** -10 if dt == torch.float16 else 2.0 ** -7
    x1, x2, w = cuda(G[f"{n}/x1"]).to(dt), cuda(G[f"{n}/x2"]).to(dt), cuda(G[f"{n}/w"]).to(dt)
    for metric in NARROW_METRICS:
        key = f"{n}/{metric['name']}"
        if key + "/ref" not in G.files:
            continue
        got = call_metric(tpw, metric, x1, x2, w if metric.get("weighted") else None)
        assert got.dtype == dt
        got = got.double().cpu()
        ref, exact = torch.from_numpy(G[key + "/ref"]).double(), torch.from_numpy(G[key + "/f64"])
        scale = exact.abs().clamp_min(1e-2)
        err_got, err_ref = ((got - exact).abs() / scale).max(), ((ref - exact).abs() / scale).max()
        assert float(err_got) <= ulp, (key, float(err_got))                       # one rounding of the output
        assert float(err_got) <= float(err_ref) + ulp, (key, float(err_got), float(err_ref))
        assert float(((got - ref).abs() / scale).max()) <= float(err_ref) + ulp, key


def test_narrow_hausdorff(tpw, golden):
    G = golden("narrow")
    got = tpw.directed_hausdorff_distances(cuda(G["hd_f16/x1"]).half(), cuda(G["hd_f16/x2"]).half())[0]
    assert got.dtype == torch.float16
    exact = torch.from_numpy(G["hd_f16/f64"])
    assert float(((got.double().cpu() - exact).abs() / exact).max()) <= 2.0 ** -10
    ref = torch.from_numpy(G["hd_f16/ref"]).double()
    assert float(((got.double().cpu() - ref).abs() / exact).max()) <= float(((ref - exact).abs() / exact).max()) + 2.0 ** -10


def test_half_precision_inputs(tpw):
    g = torch.Generator().manual_seed(8)
    x1 = torch.randn(33, 24, generator=g).cuda()
    x2 = torch.randn(20, 24, generator=g).cuda()
    for dt in (torch.float16, torch.bfloat16):
        out = tpw.manhattan_distances(x1.to(dt), x2.to(dt))
        assert out.dtype == dt
        ref = tpw.manhattan_distances(x1.to(dt).float(), x2.to(dt).float())
        assert torch.equal(out, ref.to(dt))


def test_cdist_dispatcher(tpw):
    g = torch.Generator().manual_seed(2)
    x1 = torch.randn(12, 6, generator=g).cuda()
    x2 = torch.randn(9, 6, generator=g).cuda()
    assert torch.equal(tpw.cdist(x1, x2), tpw.minkowski_distances(x1, x2, 2.0))
    assert torch.equal(tpw.cdist(x1, x2, "minkowski", p=3.0), tpw.minkowski_distances(x1, x2, 3.0))
    assert torch.equal(tpw.cdist(x1, x2, "manhattan"), tpw.manhattan_distances(x1, x2))
    assert torch.equal(tpw.cdist(x1, x2, "l1"), tpw.cdist(x1, x2, "cityblock"))
    assert torch.equal(tpw.cdist(x1, x2, "linf"), tpw.chebyshev_distances(x1, x2))
    w = torch.rand(6, generator=g).cuda()
    assert torch.equal(tpw.cdist(x1, x2, "wminkowski", w=w, p=3.0), tpw.wminkowski_distances(x1, x2, 3.0, w))
    xb, yb = x1 > 0, x2 > 0
    # the reference's cdist maps "kulsinski" onto kulczynski1
    assert torch.equal(tpw.cdist(xb, yb, "kulsinski"), tpw.kulczynski1_distances(xb, yb), )
    with pytest.raises(TypeError, match="incompatible arguments p"):
        tpw.cdist(x1, x2, "euclidean", p=3.0)
    with pytest.raises(RuntimeError, match="unkown distance metric"):
        tpw.cdist(x1, x2, "nope")
    with pytest.raises(RuntimeError, match="feature dimension of x1 and x2 must be 2"):
        tpw.pdist(x1, "haversine")


def test_gradcheck_float64(tpw):
    g = torch.Generator().manual_seed(6)
    x1 = torch.randn(5, 4, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    x2 = torch.randn(6, 4, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    w = (torch.rand(4, generator=g, dtype=torch.float64) + 0.5).cuda().requires_grad_(True)
    gc = torch.autograd.gradcheck
    assert gc(lambda a, b: tpw.minkowski_distances(a, b, 3.0), (x1, x2))
    assert gc(lambda a, b: tpw.minkowski_distances(a, b, 2.5), (x1, x2))
    assert gc(lambda a, b: tpw.euclidean_distances(a, b), (x1, x2))
    assert gc(lambda a, b: tpw.sqeuclidean_distances(a, b), (x1, x2))
    assert gc(lambda a, b: tpw.cosine_similarity(a, b), (x1, x2))
    assert gc(lambda a, b: tpw.correlation_distances(a, b), (x1, x2))
    assert gc(lambda a, b, c: tpw.wminkowski_distances(a, b, 3.0, c), (x1, x2, w))
    s1 = torch.rand(2, 7, 3, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    s2 = torch.rand(3, 5, 3, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    assert gc(lambda a, b: tpw.directed_hausdorff_distances(a, b)[0], (s1, s2))  # the reference's one real test


def test_full_size_identities(tpw):
    """Benchmark-size runs checked through identities that need no reference run."""
    g = torch.Generator().manual_seed(0)
    # C2: translation invariance of the L_p distances => sum_i grad_x1[i] + sum_j grad_x2[j] = 0
    X = torch.randn(4, 4096, 256, generator=g).cuda().requires_grad_(True)
    Y = torch.randn(4, 4096, 256, generator=g).cuda().requires_grad_(True)
    Gr = torch.randn(4, 4096, 4096, generator=g).cuda()
    for p in (3.0, math.inf):
        X.grad = Y.grad = None
        out = tpw.minkowski_distances(X, Y, p)
        out.backward(Gr)
        resid = X.grad.double().sum(1) + Y.grad.double().sum(1)
        ref_mag = X.grad.double().abs().sum(1) + Y.grad.double().abs().sum(1)
        assert float((resid.abs() / ref_mag).max()) < 1e-5, p
        with torch.no_grad():
            assert torch.equal(tpw.minkowski_distances(Y, X, p), out.transpose(1, 2)), p  # exact symmetry
    del X, Y, Gr, out
    # C3: sum_ij |x_i & y_j| = sum_k colcount_x[k] * colcount_y[k], an integer identity
    Xb = torch.rand(65536, 1024, generator=g).cuda() < 0.1
    Yb = torch.rand(16384, 1024, generator=g).cuda() < 0.1
    n11 = tpw.pwand_sum(Xb, Yb)
    expect = int((Xb.sum(0, dtype=torch.int64) * Yb.sum(0, dtype=torch.int64)).sum())
    assert int(n11.sum(dtype=torch.float64)) == expect
    ham = tpw.hamming_distances(Xb, Yb)
    nx, ny = Xb.sum(1, dtype=torch.float32)[:, None], Yb.sum(1, dtype=torch.float32)[None, :]
    assert torch.equal(ham, (nx + ny - 2 * n11) / 1024.0)  # all operands are exact float32 integers
    jac = tpw.jaccard_distances(Xb, Yb)
    assert float(jac.min()) >= 0.0 and float(jac.max()) <= 1.0
    del Xb, Yb, n11, ham, jac
    # C4: sum_j |x_i - y_j|^2 = N2 |x_i|^2 + sum_j |y_j|^2 - 2 x_i . sum_j y_j
    X = torch.randn(131072, 512, generator=g).cuda()
    Y = torch.randn(16384, 512, generator=g).cuda()
    sq = tpw.sqeuclidean_distances(X, Y)
    lhs = sq.sum(1, dtype=torch.float64)
    Xd, Yd = X.double(), Y.double()
    rhs = 16384 * Xd.pow(2).sum(1) + Yd.pow(2).sum() - 2 * Xd @ Yd.sum(0)
    assert float(((lhs - rhs).abs() / rhs).max()) < 1e-6
    del sq, lhs, rhs, Xd, Yd
    cd = tpw.cosine_distances(X[:32768], Y)
    assert float(cd.min()) >= 0.0 and float(cd.max()) <= 2.0
    close(cd[:64, :64], O.cosine_distances(X[:64].cpu().numpy(), Y[:64].cpu().numpy()), TOL[torch.float32])
    del cd, X, Y
    # C5: the attained pair reproduces the output, and the value does not depend on point order
    P = torch.rand(64, 8192, 3, generator=g) * 2 - 1
    Q = P + 0.05 * torch.randn(64, 8192, 3, generator=g)
    x1, x2 = P[:, None].cuda(), Q[:, None].cuda()
    out, i1, i2 = tpw.directed_hausdorff_distances(x1, x2)
    pick1 = x1[:, 0].gather(1, i1.view(64, 1, 1).expand(64, 1, 3))[:, 0]
    pick2 = x2[:, 0].gather(1, i2.view(64, 1, 1).expand(64, 1, 3))[:, 0]
    d = pick1 - pick2
    dd = ((d[:, 0] * d[:, 0] + d[:, 1] * d[:, 1]) + d[:, 2] * d[:, 2]).sqrt()
    assert torch.equal(dd, out.view(64))
    perm = torch.randperm(8192, generator=g).cuda()
    out2, _, _ = tpw.directed_hausdorff_distances(x1[:, :, perm], x2[:, :, perm.flip(0)])
    assert torch.equal(out, out2)


@pytest.fixture
def tensor_engine(tpw):
    tpw.set_dot_engine("tcgen05")
    yield tpw
    tpw.set_dot_engine("auto")


@pytest.mark.parametrize("shape", [(1, 128, 256, 64), (2, 300, 520, 200), (1, 1, 1, 8), (1, 130, 257, 70), (3, 77, 40, 513)])
def test_tensor_core_engine_vs_oracle(tensor_engine, shape):
    """The bf16x3 tcgen05 kernel against the float64 oracle, at the float32 parity tolerance."""
    tpw = tensor_engine
    B, n1, n2, d = shape
    g = torch.Generator().manual_seed(sum(shape))
    x1 = torch.randn(B, n1, d, generator=g)
    x2 = torch.randn(B, n2, d, generator=g)
    a, b = x1.cuda(), x2.cuda()
    x1d, x2d = x1.double().numpy(), x2.double().numpy()
    tol = TOL[torch.float32]
    close(tpw.sqeuclidean_distances(a, b), O.sqeuclidean(x1d, x2d).astype(np.float32), tol, msg="sqeuclidean")
    close(tpw.euclidean_distances(a, b), O.cdist(x1d, x2d, 2.0).astype(np.float32), tol, msg="euclidean")
    close(tpw.cosine_similarity(a, b), O.cosine_similarity(x1d, x2d).astype(np.float32), tol, msg="cosine_similarity")
    close(tpw.cosine_distances(a, b), O.cosine_distances(x1d, x2d).astype(np.float32), tol, msg="cosine_distances")
    close(tpw.correlation_distances(a, b), O.correlation_distances(x1d, x2d).astype(np.float32), tol, msg="correlation")
    close(tpw.linear_kernel(a, b), (x1d @ np.swapaxes(x2d, -1, -2)).astype(np.float32), tol, d ** 0.5, msg="linear")


def test_tensor_core_engine_details(tensor_engine, golden):
    tpw = tensor_engine
    g = torch.Generator().manual_seed(77)
    x = torch.randn(700, 96, generator=g).cuda()
    # x2 = None: the diagonal of the distance epilogues is exactly zero
    assert torch.equal(tpw.sqeuclidean_distances(x).diagonal(), torch.zeros(700, device="cuda"))
    assert torch.equal(tpw.euclidean_distances(x).diagonal(), torch.zeros(700, device="cuda"))
    # gradients do not depend on which engine produced the forward values beyond its rounding
    a = x.clone().requires_grad_(True)
    y = torch.randn(520, 96, generator=g).cuda().requires_grad_(True)
    gr = torch.randn(700, 520, generator=g).cuda()
    tpw.euclidean_distances(a, y).backward(gr)
    g1, g2 = O.cdist_backward(gr.double().cpu().numpy(), x.double().cpu().numpy(), y.detach().double().cpu().numpy(), 2.0)
    close(a.grad, g1.astype(np.float32), TOL[torch.float32], 10 * float(np.abs(g1).max()), "euclidean grad_x1")
    close(y.grad, g2.astype(np.float32), TOL[torch.float32], 10 * float(np.abs(g2).max()), "euclidean grad_x2")
    # zero rows: cosine similarity keeps the (zero) numerator, distance is 1
    z = x.clone()
    z[5] = 0
    s = tpw.cosine_similarity(z, x)
    assert torch.equal(s[5], torch.zeros(700, device="cuda"))
    # the C4-shaped golden block through the tensor cores
    G = golden("configs")
    X, Y = config_inputs("C4")
    if np.array_equal(np.array([X.double().sum().item(), Y.double().sum().item()]), G["C4/checksum"]):
        for name in ("sqeuclidean_distances", "cosine_distances"):
            close(getattr(tpw, name)(X.cuda(), Y.cuda())[::16, ::64], G[f"C4/{name}"], TOL[torch.float32], msg="C4 " + name)
    # float64 never leaves the CUDA cores
    xd = x.double()
    close(tpw.sqeuclidean_distances(xd[:50], xd[50:90]), O.sqeuclidean(xd[:50].cpu().numpy(), xd[50:90].cpu().numpy()),
          TOL[torch.float64])


def _sum_close(got, ref, msg):
    """Gradients are sums of K signed terms: float32 evaluation orders differ by about 1e-7 * sqrt(K) of
    the typical magnitude, so the absolute slack is tied to the RMS of the reference (plus the
    contract's relative 1e-4 per element)."""
    ref = ref.double()
    bound = 1e-4 * ref.abs() + 2e-5 * ref.pow(2).mean().sqrt() + 1e-5
    err = (got.double() - ref).abs()
    worst = float((err / bound).max())
    assert worst <= 1.0, f"{msg}: max error / bound = {worst:.3f} (max abs error {float(err.max()):.3e})"


DENSE_BWD_OPS = {
    "sqeuclidean": lambda t, a, b: t.sqeuclidean_distances(a, b),
    "euclidean": lambda t, a, b: t.euclidean_distances(a, b),
    "cosine_similarity": lambda t, a, b: t.cosine_similarity(a, b),
    "correlation": lambda t, a, b: t.correlation_distances(a, b),
    "linear_kernel": lambda t, a, b: t.linear_kernel(a, b),
}


@pytest.mark.parametrize("shape", [(1, 300, 520, 96), (2, 257, 1030, 130), (3, 129, 67, 33), (1, 64, 4100, 8), (1, 1, 1, 4)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("op", sorted(DENSE_BWD_OPS))
def test_tensor_core_backward_vs_float64(tensor_engine, shape, op):
    """The tf32x3 tcgen05 gradient products (forced) against the float64 CUDA-core kernels of the same
    operator, next to the float32 CUDA-core result held to the same bound."""
    tpw = tensor_engine
    B, n1, n2, d = shape
    g = torch.Generator().manual_seed(sum(shape) + len(op))
    x1 = torch.randn(B, n1, d, generator=g).cuda()
    x2 = torch.randn(B, n2, d, generator=g).cuda()
    up = torch.randn(B, n1, n2, generator=g).cuda()

    def grads(a, b, u):
        a, b = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
        DENSE_BWD_OPS[op](tpw, a, b).backward(u)
        return a.grad, b.grad

    r1, r2 = grads(x1.double(), x2.double(), up.double())
    t1, t2 = grads(x1, x2, up)
    _sum_close(t1, r1, f"{op} grad_x1 (tensor cores)")
    _sum_close(t2, r2, f"{op} grad_x2 (tensor cores)")
    tpw.set_dot_engine("simt")
    s1, s2 = grads(x1, x2, up)
    tpw.set_dot_engine("tcgen05")
    _sum_close(s1, r1, f"{op} grad_x1 (CUDA cores)")
    _sum_close(s2, r2, f"{op} grad_x2 (CUDA cores)")


@pytest.mark.parametrize("shape", [(2, 300, 520, 200), (1, 130, 257, 70), (1, 64, 64, 4100), (1, 1, 1, 3)], ids=lambda s: "x".join(map(str, s)))
def test_linear_kernel_tf32_forward(tensor_engine, shape):
    """linear_kernel on the tensor cores (tf32x3, chunked accumulation) against float64, held to the
    same bound as the fp32 FMA chain of the CUDA-core tile."""
    tpw = tensor_engine
    B, n1, n2, d = shape
    g = torch.Generator().manual_seed(sum(shape))
    x1, x2 = torch.randn(B, n1, d, generator=g).cuda(), torch.randn(B, n2, d, generator=g).cuda()
    ref = x1.double() @ x2.double().transpose(1, 2)
    _sum_close(tpw.linear_kernel(x1, x2), ref, "linear_kernel (tensor cores)")
    tpw.set_dot_engine("simt")
    _sum_close(tpw.linear_kernel(x1, x2), ref, "linear_kernel (CUDA cores)")
    tpw.set_dot_engine("tcgen05")
    # the kernels built on it
    _sum_close(tpw.polynomial_kernel(x1[0], x2[0], degree=2, gamma=0.01, coef0=1.0),
               (0.01 * ref[0] + 1.0) ** 2, "polynomial_kernel")


def test_tensor_core_backward_blocking_and_abi(tensor_engine, monkeypatch):
    """Scratch-capped blocking (groups of batches, row blocks of one batch) reproduces the single
    call; one-sided gradients; argument checks of the C entry point."""
    tpw = tensor_engine
    from torchpairwise_b200 import _abi
    lib = _abi.lib
    g = torch.Generator().manual_seed(5)
    x1 = torch.randn(3, 600, 64, generator=g).cuda()
    x2 = torch.randn(3, 520, 64, generator=g).cuda()
    up = torch.randn(3, 600, 520, generator=g).cuda()

    def grads(need2=True):
        a, b = x1.clone().requires_grad_(True), x2.clone().requires_grad_(need2)
        tpw.sqeuclidean_distances(a, b).backward(up)
        return a.grad, b.grad

    full1, full2 = grads()
    per_batch = lib.tpw_dot_backward_scratch_bytes(_abi.F32, _abi.LP_BWD_PPMINKOWSKI, _abi.ENGINE_TCGEN05_TF32X3, 1, 600, 520, 64)
    assert per_batch > 8 * 600 * 520   # tf32 high and low copies of the coefficient matrix
    monkeypatch.setenv("TPW_BWD_SCRATCH_GB", str(2.5 * per_batch / 2 ** 30))   # groups of two batches
    b1, b2 = grads()
    assert torch.equal(b1, full1) and torch.equal(b2, full2)
    monkeypatch.setenv("TPW_BWD_SCRATCH_GB", str(0.5 * per_batch / 2 ** 30))   # row blocks of 256 within a batch
    r1, r2 = grads()
    assert torch.equal(r1, full1)
    _sum_close(r2, full2, "row-blocked grad_x2")
    monkeypatch.delenv("TPW_BWD_SCRATCH_GB")
    o1, o2 = grads(need2=False)
    assert o2 is None and torch.equal(o1, full1)
    # C entry point: too little scratch is an error when the engine is forced, a CUDA-core call under AUTO
    nb = lib.tpw_dot_backward_scratch_bytes(_abi.F32, _abi.LP_BWD_MATMUL, _abi.ENGINE_TCGEN05_TF32X3, 3, 600, 520, 64)
    small = torch.empty(1024, dtype=torch.uint8, device="cuda")
    g1, g2 = torch.empty_like(x1), torch.empty_like(x2)
    st = torch.cuda.current_stream().cuda_stream
    args = (up.data_ptr(), None, x1.data_ptr(), x2.data_ptr(), g1.data_ptr(), g2.data_ptr(), small.data_ptr(), 1024, 3, 600, 520, 64, st)
    assert lib.tpw_dot_backward_ws(_abi.F32, _abi.LP_BWD_MATMUL, _abi.ENGINE_TCGEN05_TF32X3, *args) == 1
    assert "scratch" in lib.tpw_last_error().decode()
    assert lib.tpw_dot_backward_ws(_abi.F32, _abi.LP_BWD_WMINKOWSKI, _abi.ENGINE_AUTO, *args) == 1
    assert lib.tpw_dot_backward_ws(_abi.F32, _abi.LP_BWD_MATMUL, _abi.ENGINE_AUTO, *args) == 0
    _sum_close(g1, up.double() @ x2.double(), "AUTO without scratch runs the CUDA-core products")
    assert nb > 0 and lib.tpw_dot_backward_scratch_bytes(_abi.F64, _abi.LP_BWD_MATMUL, _abi.ENGINE_AUTO, 1, 4096, 4096, 512) == 0
    assert lib.tpw_dot_backward_scratch_bytes(_abi.F32, _abi.LP_BWD_MATMUL, _abi.ENGINE_AUTO, 1, 4096, 4096, 512) > 0
    assert lib.tpw_dot_backward_scratch_bytes(_abi.F32, _abi.LP_BWD_MATMUL, _abi.ENGINE_AUTO, 1, 200, 200, 64) == 0
    assert lib.tpw_dot_backward_scratch_bytes(_abi.F32, _abi.LP_BWD_WMINKOWSKI, _abi.ENGINE_TCGEN05_TF32X3, 1, 4096, 4096, 512) == 0


def test_full_size_dense_backward(tpw):
    """A quarter of C4 (X[32768,512], Y[16384,512], 2.1 GB of upstream gradient) through the engine
    rule: the sqeuclidean backward runs as row-blocked tensor-core contractions; checked by
    translation invariance and by float64 evaluation of sampled rows of both gradients."""
    g = torch.Generator().manual_seed(3)
    X = torch.randn(32768, 512, generator=g).cuda().requires_grad_(True)
    Y = torch.randn(16384, 512, generator=g).cuda().requires_grad_(True)
    up = torch.randn(32768, 16384, generator=g).cuda()
    tpw.sqeuclidean_distances(X, Y).backward(up)
    resid = X.grad.double().sum(0) + Y.grad.double().sum(0)
    mag = X.grad.double().abs().sum(0) + Y.grad.double().abs().sum(0)
    assert float((resid.abs() / mag).max()) < 1e-5
    Xd, Yd = X.detach().double(), Y.detach().double()
    rows = torch.arange(0, 32768, 512, device="cuda")
    ud = up[rows].double()
    _sum_close(X.grad[rows], 2 * (Xd[rows] * ud.sum(1, keepdim=True) - ud @ Yd), "C4 quarter grad_x1 rows")
    cols = torch.arange(0, 16384, 256, device="cuda")
    uc = up[:, cols].double()
    _sum_close(Y.grad[cols], 2 * (Yd[cols] * uc.sum(0).unsqueeze(1) - uc.t() @ Xd), "C4 quarter grad_x2 rows")


def test_full_size_neighbour_reductions(tpw):
    """C4-sized nearest-row query (engine rule: tcgen05 row-minimum epilogue, nothing but keys written)
    checked on sampled rows against float64, and a C2-sized fused radius mask against the matrix path."""
    g = torch.Generator().manual_seed(9)
    X = torch.randn(131072, 512, generator=g).cuda()
    Y = torch.randn(16384, 512, generator=g).cuda()
    arg, mn = tpw.pairwise_argmin_min(X, Y, "euclidean")
    rows = torch.arange(0, 131072, 2048, device="cuda")
    ref = torch.cdist(X[rows].double(), Y.double())
    tol = TOL[torch.float32]
    torch.testing.assert_close(mn[rows].double(), ref.min(1).values, rtol=tol["rtol"], atol=tol["atol"])
    picked = ref.gather(1, arg[rows].unsqueeze(1))[:, 0]
    torch.testing.assert_close(picked, ref.min(1).values, rtol=tol["rtol"], atol=tol["atol"])
    assert int(arg.min()) >= 0 and int(arg.max()) < 16384
    del X, Y, ref
    A = torch.randn(4, 4096, 256, generator=g).cuda()
    Bm = torch.randn(4, 4096, 256, generator=g).cuda()
    dist = tpw.chebyshev_distances(A, Bm)
    eps = float(dist[0, :64].median())
    assert torch.equal(tpw.radius_neighbors_mask(A, Bm, eps, "chebyshev"), dist <= eps)


def test_engine_auto_selection(tpw):
    from torchpairwise_b200 import _abi
    lib = _abi.lib
    assert tpw.get_dot_engine() == "auto"
    # small problems and float64 stay on the CUDA cores, large float32 problems go to the tensor cores
    assert lib.tpw_dot_metric_scratch_bytes(_abi.F32, _abi.ENGINE_AUTO, 1, 1024, 2048, 128) > 0
    assert lib.tpw_dot_metric_scratch_bytes(_abi.F32, _abi.ENGINE_AUTO, 1, 100, 100, 16) == 0
    assert lib.tpw_dot_metric_scratch_bytes(_abi.F64, _abi.ENGINE_AUTO, 1, 4096, 4096, 512) == 0
    assert lib.tpw_dot_metric_scratch_bytes(_abi.F32, _abi.ENGINE_SIMT_FP32, 1, 4096, 4096, 512) == 0
    with pytest.raises(ValueError):
        tpw.set_dot_engine("nope")


def test_host_pipeline_matches_single_call(tpw):
    from torchpairwise_b200.host_pipeline import forward_backward_from_host
    g = torch.Generator().manual_seed(21)
    X = torch.randn(5, 200, 64, generator=g).pin_memory()
    Y = torch.randn(5, 150, 64, generator=g).pin_memory()
    G = torch.randn(5, 200, 150, generator=g).pin_memory()
    g1 = torch.empty_like(X).pin_memory()
    g2 = torch.empty_like(Y).pin_memory()
    out = torch.empty_like(G).pin_memory()
    forward_backward_from_host(tpw.minkowski_distances, X, Y, G, g1, g2, "cuda:0", chunk=2, out_host=out, p=3.0)
    a, b = X.cuda().requires_grad_(True), Y.cuda().requires_grad_(True)
    ref = tpw.minkowski_distances(a, b, 3.0)
    ref.backward(G.cuda())
    assert torch.equal(out, ref.detach().cpu())
    assert torch.equal(g1, a.grad.cpu()) and torch.equal(g2, b.grad.cpu())


def test_extras_golden(tpw, golden):
    """seuclidean and the neighbour masks: the callers on either side of the path."""
    G = golden("extras")
    tol = TOL[torch.float32]
    x1, x2, V = cuda(G["x1"], True), cuda(G["x2"], True), cuda(G["V"])
    out = tpw.seuclidean_distances(x1, x2, V)
    close(out, G["seuclidean/out"], tol, msg="seuclidean")
    out.backward(cuda(G["up2"]))
    close(x1.grad, G["seuclidean/gx1"], tol, 10, "seuclidean grad_x1")
    close(x2.grad, G["seuclidean/gx2"], tol, 10, "seuclidean grad_x2")
    x1.grad = None
    out = tpw.seuclidean_distances(x1, None, V)
    close(out, G["seuclidean_self/out"], tol, msg="seuclidean self")
    out.backward(cuda(G["up1"]))
    close(x1.grad, G["seuclidean_self/gx1"], tol, 10, "seuclidean self grad")
    close(tpw.cdist(x1.detach(), x2.detach(), "seuclidean", V=V), G["cdist_seuclidean"], tol, msg="cdist seuclidean")
    # V = None: the feature variances of x1 (the reference intends this; its own call trips on a dangling array ref)
    xd = x1.detach()
    close(tpw.seuclidean_distances(xd), O.seuclidean(G["x1"], G["x1"], G["x1"].var(0, ddof=1)), tol, msg="seuclidean V=None")
    with pytest.raises(RuntimeError, match="V is required"):
        tpw.seuclidean_distances(xd, x2.detach())
    xd2 = x2.detach()
    assert torch.equal(tpw.k_neighbors_mask(xd, xd2, 3).cpu(), torch.from_numpy(G["k_neighbors_k3"]))
    assert torch.equal(tpw.k_neighbors_mask(xd, None, 2, "manhattan").cpu(), torch.from_numpy(G["k_neighbors_self_k2_manhattan"]))
    assert torch.equal(tpw.radius_neighbors_mask(xd, xd2, 2.5).cpu(), torch.from_numpy(G["radius_2.5"]))
    assert torch.equal(tpw.radius_neighbors_mask(xd, None, 3.0, "minkowski", p=3.0).cpu(),
                       torch.from_numpy(G["radius_self_3_minkowski3"]))


ROWMIN_SHAPES = [((130, 7), (257, 7)), ((3, 200, 32), (3, 129, 32)), ((1, 5), (1, 5)), ((2, 300, 96), (2, 40, 96)),
                 ((513, 36), (1000, 36))]
ROWMIN_METRICS = [("euclidean", None, 2.0, 0.5), ("sqeuclidean", None, 2.0, 1.0), ("manhattan", None, 1.0, 1.0),
                  ("chebyshev", None, math.inf, 1.0), ("minkowski", 3.0, 3.0, 1 / 3), ("minkowski", 1.5, 1.5, 1 / 1.5)]


@pytest.mark.parametrize("shapes", ROWMIN_SHAPES, ids=lambda s: "x".join(map(str, s[0])) + "_" + "x".join(map(str, s[1])))
@pytest.mark.parametrize("metric,p,pp,ex", ROWMIN_METRICS, ids=lambda v: str(v))
def test_pairwise_argmin_min_matches_oracle(tpw, shapes, metric, p, pp, ex):
    """The streaming row minimum against min / argmin of the oracle's full matrix (float64 inputs of
    the same float32 values): the value within the float32 contract, and the chosen column's true
    distance equal to the true minimum within the same bound (robust to near ties)."""
    rng = np.random.default_rng(zlib.crc32(repr((shapes, metric, p)).encode()))
    a = rng.standard_normal(shapes[0]).astype(np.float32)
    b = rng.standard_normal(shapes[1]).astype(np.float32)
    ref = O.cdist(a.astype(np.float64), b.astype(np.float64), pp)
    if ex == 1.0 and pp == 2.0:
        ref = ref * ref
    arg, mn = tpw.pairwise_argmin_min(cuda(a), cuda(b), metric, p)
    assert arg.dtype == torch.int64 and mn.dtype == torch.float32
    assert tuple(arg.shape) == shapes[0][:-1] and tuple(mn.shape) == shapes[0][:-1]
    tol = TOL[torch.float32]
    close(mn.double(), ref.min(-1), tol, msg="row minimum")
    picked = np.take_along_axis(ref, arg.cpu().numpy()[..., None], -1)[..., 0]
    np.testing.assert_allclose(picked, ref.min(-1), rtol=tol["rtol"], atol=tol["atol"])
    # the same kernel's full matrix reduces to exactly the same value
    full = tpw.cdist(cuda(a), cuda(b), "minkowski", p=pp) if metric != "sqeuclidean" else None
    if full is not None and not (metric == "euclidean" and tpw.get_dot_engine() != "simt"):
        assert torch.equal(full.min(-1).values, mn)


@pytest.mark.parametrize("shape", [(1, 300, 520, 96), (2, 257, 1030, 130), (1, 128, 256, 64), (1, 5, 3, 8)], ids=lambda s: "x".join(map(str, s)))
def test_pairwise_argmin_min_tensor_cores(tensor_engine, shape):
    """Euclidean / squared Euclidean row minimum in the tcgen05 epilogue (forced) against the float64
    matrix: value within the float32 contract, chosen column attains the minimum within the same bound."""
    tpw = tensor_engine
    B, n1, n2, d = shape
    g = torch.Generator().manual_seed(sum(shape))
    x1, x2 = torch.randn(B, n1, d, generator=g), torch.randn(B, n2, d, generator=g)
    ref = O.cdist(x1.double().numpy(), x2.double().numpy(), 2.0)
    tol = TOL[torch.float32]
    for metric, r in (("euclidean", ref), ("sqeuclidean", ref * ref)):
        arg, mn = tpw.pairwise_argmin_min(x1.cuda(), x2.cuda(), metric)
        assert arg.shape == (B, n1) and arg.dtype == torch.int64
        close(mn.double(), r.min(-1), tol, msg=metric + " row minimum")
        picked = np.take_along_axis(r, arg.cpu().numpy()[..., None], -1)[..., 0]
        np.testing.assert_allclose(picked, r.min(-1), rtol=tol["rtol"], atol=tol["atol"])
        # the matrix the same engine writes has the same row minimum
        full = tpw.euclidean_distances(x1.cuda(), x2.cuda()) if metric == "euclidean" else tpw.sqeuclidean_distances(x1.cuda(), x2.cuda())
        assert torch.equal(full.min(-1).values, mn)
    argc, mnc = tpw.pairwise_argmin_min(x1.cuda(), x2.cuda(), "cosine")
    cd = tpw.cosine_distances(x1.cuda(), x2.cuda())
    assert torch.equal(mnc, cd.min(-1).values)
    assert torch.equal(cd.gather(-1, argc.unsqueeze(-1))[..., 0], mnc)
    close(mnc.double(), O.cosine_distances(x1.double().numpy(), x2.double().numpy()).min(-1), tol, msg="cosine row minimum")


@pytest.mark.parametrize("shape,k", [((1, 300, 520, 96), 1), ((1, 300, 520, 96), 3), ((1, 300, 520, 96), 8), ((1, 300, 520, 96), 16),
                                     ((2, 257, 1030, 130), 5), ((1, 128, 256, 64), 8), ((1, 40, 9, 16), 9), ((1, 700, 2100, 64), 12),
                                     ((1, 260, 4500, 64), 8), ((2, 130, 9000, 72), 16)],   # 18 and 36 column tiles: three column ranges
                         ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else str(v))
def test_pairwise_argkmin_tensor_cores(tensor_engine, shape, k):
    """The k nearest rows from the tcgen05 top-k epilogue (forced) against the float64 matrix: ascending
    values within the float32 contract, distinct valid columns whose true distances are the k smallest
    within the same bound, and agreement with a partial selection on the matrix the same engine writes."""
    tpw = tensor_engine
    B, n1, n2, d = shape
    g = torch.Generator().manual_seed(sum(shape) + k)
    x1, x2 = torch.randn(B, n1, d, generator=g), torch.randn(B, n2, d, generator=g)
    a, b = x1.cuda(), x2.cuda()
    ref = O.cdist(x1.double().numpy(), x2.double().numpy(), 2.0)
    tol = TOL[torch.float32]
    for metric, r, fn in (("euclidean", ref, tpw.euclidean_distances), ("sqeuclidean", ref * ref, tpw.sqeuclidean_distances),
                          ("cosine", O.cosine_distances(x1.double().numpy(), x2.double().numpy()), tpw.cosine_distances)):
        inds, vals = tpw.pairwise_argkmin(a, b, k, metric)
        assert inds.shape == (B, n1, k) and inds.dtype == torch.int64 and vals.dtype == torch.float32
        iv = inds.cpu().numpy()
        assert iv.min() >= 0 and iv.max() < n2
        assert all(len(set(row)) == k for row in iv.reshape(-1, k)), "columns of a row must be distinct"
        assert bool((vals[..., 1:] >= vals[..., :-1]).all())
        want = np.sort(r, axis=-1)[..., :k]
        close(vals.double(), want, tol, msg=f"{metric} k smallest values")
        np.testing.assert_allclose(np.sort(np.take_along_axis(r, iv, -1), -1), want, rtol=tol["rtol"], atol=tol["atol"])
        full = fn(a, b)
        fv = full.topk(k, dim=-1, largest=False, sorted=True).values
        assert torch.equal(fv, vals), metric
        assert torch.equal(full.gather(-1, inds), vals), metric


def test_pairwise_argkmin_other_paths(tpw):
    """Small problems and other metrics take the matrix kernel plus a partial selection; k_neighbors_mask
    on a large problem takes the tensor-core top-k and marks exactly k + 1 columns per row."""
    g = torch.Generator().manual_seed(4)
    x, y = torch.randn(70, 9, generator=g).cuda(), torch.randn(90, 9, generator=g).cuda()
    inds, vals = tpw.pairwise_argkmin(x, y, 4, "manhattan")
    dist = tpw.manhattan_distances(x, y)
    assert torch.equal(vals, dist.topk(4, largest=False).values) and torch.equal(dist.gather(1, inds), vals)
    i64, v64 = tpw.pairwise_argkmin(x.double(), y.double(), 2, "euclidean")
    assert v64.dtype == torch.float64 and i64.shape == (70, 2)
    with pytest.raises(RuntimeError, match="exceeds"):
        tpw.pairwise_argkmin(x, y, 91)
    with pytest.raises(RuntimeError, match="positive"):
        tpw.pairwise_argkmin(x, y, 0)
    X, Y = torch.randn(2048, 128, generator=g).cuda(), torch.randn(3000, 128, generator=g).cuda()   # engine rule: tensor cores
    mask = tpw.k_neighbors_mask(X, Y, 4)
    assert mask.dtype == torch.bool and torch.equal(mask.sum(1), torch.full((2048,), 5, device="cuda"))
    d = tpw.euclidean_distances(X, Y)
    kth = d.topk(5, dim=1, largest=False).values[:, -1:]
    assert bool((d[mask].view(2048, 5) <= kth * (1 + 1e-4) + 1e-5).all())


def test_pairwise_argmin_min_ties_and_edges(tpw):
    """Exact ties go to the smaller x2 row (integer-valued inputs make the distances exact), in a
    tile interior, across the 128-column tile boundary and across batches; other dtypes and the
    k = 0 neighbour mask agree with the matrix path; bad arguments raise."""
    rng = np.random.default_rng(11)
    b = rng.integers(-8, 9, size=(2, 400, 12)).astype(np.float32)
    b[:, 300] = b[:, 17]    # duplicates of row 17 in another column tile
    b[:, 130] = b[:, 17]
    b[:, 129] = b[:, 128]   # duplicates inside one tile
    a = b[:, [17, 128, 5, 399]] + 0.0
    for metric in ("manhattan", "sqeuclidean", "chebyshev"):
        arg, mn = tpw.pairwise_argmin_min(cuda(a), cuda(b), metric)
        ref = O.cdist(a.astype(np.float64), b.astype(np.float64), {"manhattan": 1.0, "sqeuclidean": 2.0, "chebyshev": math.inf}[metric])
        if metric == "sqeuclidean":
            ref = ref * ref
        assert np.array_equal(arg.cpu().numpy(), ref.argmin(-1)), metric   # numpy: first minimum
        assert np.array_equal(mn.cpu().numpy().astype(np.float64), ref.min(-1)), metric
    x = cuda(rng.standard_normal((70, 9)).astype(np.float32))
    y = cuda(rng.standard_normal((90, 9)).astype(np.float32))
    arg64, mn64 = tpw.pairwise_argmin_min(x.double(), y.double(), "euclidean")
    arg32, mn32 = tpw.pairwise_argmin_min(x, y, "euclidean")
    assert mn64.dtype == torch.float64 and torch.equal(arg64, arg32)
    torch.testing.assert_close(mn64.float(), mn32, rtol=1e-5, atol=1e-6)
    argh, mnh = tpw.pairwise_argmin_min(x.half(), y.half(), "manhattan")
    assert mnh.dtype == torch.float16 and argh.shape == arg32.shape
    # self distances: every row finds itself at distance 0
    args, mns = tpw.pairwise_argmin_min(x, None, "manhattan")
    assert torch.equal(args.cpu(), torch.arange(70)) and float(mns.abs().max()) == 0.0
    # k = 0: one True per row, at the nearest x2 row
    mask = tpw.k_neighbors_mask(x, y, 0)
    assert mask.dtype == torch.bool and torch.equal(mask.sum(1).cpu(), torch.ones(70, dtype=torch.int64))
    assert torch.equal(mask.float().argmax(1), arg32)
    assert torch.equal(mask, tpw.k_neighbors_mask(x.double(), y.double(), 0))
    with pytest.raises(ValueError, match="supports"):
        tpw.pairwise_argmin_min(x, y, "jaccard")
    argc, mnc = tpw.pairwise_argmin_min(x, y, "cosine")     # small problem: matrix kernel + min
    cd = tpw.cosine_distances(x, y)
    assert torch.equal(mnc, cd.min(1).values) and torch.equal(cd.gather(1, argc[:, None])[:, 0], mnc)
    with pytest.raises(RuntimeError, match="no rows"):
        tpw.pairwise_argmin_min(x, y[:0])
    with pytest.raises(RuntimeError, match="positive"):
        tpw.pairwise_argmin_min(x, y, "minkowski", -1.0)
    e_arg, e_mn = tpw.pairwise_argmin_min(x[:0], y)
    assert e_arg.shape == (0,) and e_mn.shape == (0,)


@pytest.mark.parametrize("shapes", [((130, 7), (257, 7)), ((3, 200, 32), (3, 144, 32)), ((513, 36), (1008, 36)), ((1, 5), (1, 5)),
                                    # few features on enough rows and columns: the streaming kernel's mask epilogue
                                    ((131, 3), (1029, 3)), ((2, 256, 8), (2, 2048, 8)), ((300, 16), (1026, 16)), ((130, 29), (1031, 29))],
                         ids=lambda s: "x".join(map(str, s[0])) + "_" + "x".join(map(str, s[1])))
def test_radius_mask_fused_equals_compare_pass(tpw, shapes):
    """radius_neighbors_mask through the fused epilogue (one byte per pair, no float matrix) equals
    `distance <= epsilon` on the matrix the same kernel writes, metric by metric and dtype by dtype."""
    rng = np.random.default_rng(zlib.crc32(repr(shapes).encode()))
    a = cuda(rng.standard_normal(shapes[0]).astype(np.float32))
    b = cuda(rng.standard_normal(shapes[1]).astype(np.float32))
    for metric, kw, fn in (("euclidean", {}, tpw.euclidean_distances), ("manhattan", {}, tpw.manhattan_distances),
                           ("chebyshev", {}, tpw.chebyshev_distances), ("sqeuclidean", {}, tpw.sqeuclidean_distances),
                           ("minkowski", {"p": 3.0}, lambda x, y: tpw.minkowski_distances(x, y, 3.0)),
                           ("minkowski", {"p": 1.5}, lambda x, y: tpw.minkowski_distances(x, y, 1.5))):
        for x, y in ((a, b), (a.double(), b.double())):
            dist = fn(x, y)
            eps = float(dist.median())
            mask = tpw.radius_neighbors_mask(x, y, eps, metric, **kw)
            assert mask.dtype == torch.bool and mask.shape == dist.shape
            assert torch.equal(mask, dist <= eps), (metric, kw, x.dtype)
            assert 0 < int(mask.sum()) < mask.numel() or mask.numel() == 1
    assert torch.equal(tpw.radius_neighbors_mask(a, None, 0.0, "manhattan").diagonal(dim1=-2, dim2=-1).all(), torch.tensor(True, device="cuda"))
    with pytest.raises(RuntimeError, match="non-negative"):
        tpw.radius_neighbors_mask(a, b, -1.0)


@pytest.mark.parametrize("n,d", [(2, 3), (5, 1), (129, 7), (300, 64), (515, 33)])
def test_pdist_condensed(tpw, n, d):
    """pdist against scipy.spatial.distance.pdist (the layout and the definitions the reference's README
    points to) in float64, the fused condensed kernel against the gathered triangle of cdist in float32,
    batched inputs, and the gradient through the composition path."""
    from scipy.spatial.distance import pdist as sp_pdist
    rng = np.random.default_rng(n * 1000 + d)
    xn = rng.standard_normal((n, d))
    x64 = cuda(xn)
    m = n * (n - 1) // 2
    for metric, kw, sp_metric, sp_kw in (("euclidean", {}, "euclidean", {}), ("sqeuclidean", {}, "sqeuclidean", {}),
                                         ("cityblock", {}, "cityblock", {}), ("chebyshev", {}, "chebyshev", {}),
                                         ("minkowski", {"p": 3.0}, "minkowski", {"p": 3.0}),
                                         ("minkowski", {"p": 1.5}, "minkowski", {"p": 1.5}),
                                         ("cosine", {}, "cosine", {}), ("correlation", {}, "correlation", {})):
        if metric == "correlation" and d < 2:
            continue
        got = tpw.pdist(x64, metric, **kw)
        assert got.shape == (m,) and got.dtype == torch.float64
        close(got, sp_pdist(xn, sp_metric, **sp_kw), TOL[torch.float64] if metric not in ("cosine", "correlation") else dict(rtol=1e-9, atol=1e-9),
              msg=f"pdist {metric}")
        x32 = x64.float()
        iu = torch.triu_indices(n, n, offset=1, device="cuda")
        tri = tpw.cdist(x32, x32, metric, **kw)[iu[0], iu[1]]
        fused = tpw.pdist(x32, metric, **kw)
        if metric in ("cosine", "correlation"):
            assert torch.equal(fused, tri)
        else:
            close(fused, tri.cpu().numpy(), TOL[torch.float32], msg=f"pdist {metric} float32")
    xb = cuda(rng.standard_normal((3, n, d)).astype(np.float32))
    pb = tpw.pdist(xb, "manhattan")
    assert pb.shape == (3, m)
    for b in range(3):
        assert torch.equal(pb[b], tpw.pdist(xb[b], "manhattan"))
    xb_bool = cuda(rng.random((n, max(d, 8))) < 0.4)
    close(tpw.pdist(xb_bool, "jaccard").double(), sp_pdist(xb_bool.cpu().numpy(), "jaccard"), dict(rtol=1e-6, atol=1e-7), msg="pdist jaccard")
    if n > 2:
        xg = cuda(xn.astype(np.float32), True)
        tpw.pdist(xg, "euclidean").sum().backward()
        xr = torch.from_numpy(xn.astype(np.float32)).requires_grad_(True)
        torch.nn.functional.pdist(xr).sum().backward()
        close(xg.grad, xr.grad.numpy(), TOL[torch.float32], 10, "pdist gradient")


@pytest.mark.parametrize("tag", ["u32", "b64"])
def test_composed_metrics_golden(tpw, golden, tag):
    """braycurtis, snr and mahalanobis (reference kernels of their own, stated here as compositions of the
    path's kernels) against the reference's outputs and gradients."""
    G = golden("composed")
    dt = torch.float32 if tag == "u32" else torch.float64
    tol = TOL[dt]
    up, VI = cuda(G[f"{tag}/up"]), cuda(G[f"{tag}/VI"])
    for name in ("braycurtis_distances", "snr_distances"):
        x1, x2 = cuda(G[f"{tag}/x1"], True), cuda(G[f"{tag}/x2"], True)
        out = getattr(tpw, name)(x1, x2)
        close(out, G[f"{tag}/{name}/out"], tol, msg=name)
        out.backward(up)
        close(x1.grad, G[f"{tag}/{name}/gx1"], tol, 10, name + " grad_x1")
        close(x2.grad, G[f"{tag}/{name}/gx2"], tol, 10, name + " grad_x2")
        close(getattr(tpw, name)(x1.detach()), G[f"{tag}/{name}/self_out"], tol, 10, name + " self")
    x1, x2, v = cuda(G[f"{tag}/x1"], True), cuda(G[f"{tag}/x2"], True), VI.clone().requires_grad_(True)
    out = tpw.mahalanobis_distances(x1, x2, v)
    close(out, G[f"{tag}/mahalanobis_distances/out"], tol, 10, "mahalanobis")
    out.backward(up)
    close(x1.grad, G[f"{tag}/mahalanobis_distances/gx1"], tol, 100, "mahalanobis grad_x1")
    close(x2.grad, G[f"{tag}/mahalanobis_distances/gx2"], tol, 100, "mahalanobis grad_x2")
    close(v.grad, G[f"{tag}/mahalanobis_distances/gVI"], tol, 100, "mahalanobis grad_VI")
    if tag == "u32":
        a, b = x1.detach(), x2.detach()
        close(tpw.cdist(a, b, "braycurtis"), G["u32/cdist_braycurtis"], tol, msg="cdist braycurtis")
        close(tpw.cdist(a, b, "snr"), G["u32/cdist_snr"], tol, msg="cdist snr")
        close(tpw.cdist(a, b, "mahalanobis", VI=VI), G["u32/cdist_mahalanobis"], tol, 10, "cdist mahalanobis")
        big = cuda(G["u32/big"])
        got = tpw.mahalanobis_distances(big)
        # direct differences: the contract tolerance holds (the inverse covariance is computed on the GPU here, on
        # the CPU there, which costs one more digit) and the self-distance diagonal is exactly 0 like the reference's
        torch.testing.assert_close(got.cpu(), torch.from_numpy(G["u32/mahalanobis_default_VI"]), rtol=1e-4, atol=1e-4)
        assert bool((got.diagonal() == 0).all())
        with pytest.raises(RuntimeError, match="VI is required"):
            tpw.mahalanobis_distances(a, b)


@pytest.mark.parametrize("tag", ["u32", "b64", "w32"])
def test_pair_sum_metrics_golden(tpw, golden, tag):
    """canberra_distances, additive_chi2_kernel and chi2_kernel against the reference's outputs and gradients."""
    G = golden("pair_sums")
    dt = torch.float32 if tag != "b64" else torch.float64
    tol = TOL[dt]
    up = cuda(G[f"{tag}/up"])
    for name, k1, k2, kw in (("canberra_distances", "x1", "x2", {}), ("additive_chi2_kernel", "h1", "h2", {}),
                             ("chi2_kernel", "h1", "h2", {"gamma": 0.7})):
        x1, x2 = cuda(G[f"{tag}/{k1}"], True), cuda(G[f"{tag}/{k2}"], True)
        out = getattr(tpw, name)(x1, x2, **kw)
        close(out, G[f"{tag}/{name}/out"], tol, msg=name)
        out.backward(up)
        close(x1.grad, G[f"{tag}/{name}/gx1"], tol, 10, name + " grad_x1")
        close(x2.grad, G[f"{tag}/{name}/gx2"], tol, 10, name + " grad_x2")
        close(getattr(tpw, name)(x1.detach(), **kw), G[f"{tag}/{name}/self_out"], tol, msg=name + " self")
    if tag == "u32":
        a, b = cuda(G["u32/x1"]), cuda(G["u32/x2"])
        close(tpw.cdist(a, b, "canberra"), G["u32/cdist_canberra"], tol, msg="cdist canberra")
        with pytest.raises(RuntimeError, match="must be positive"):
            tpw.chi2_kernel(a, b)
        # a feature that is zero on both sides contributes nothing, forward and backward
        z1, z2 = a.clone(), b.clone()
        z1[:, 3] = 0
        z2[:, 3] = 0
        z1.requires_grad_(True)
        o = tpw.canberra_distances(z1, z2)
        close(o, O.canberra(z1.detach().cpu().numpy(), z2.cpu().numpy()), tol, msg="canberra with a zero feature")
        o.sum().backward()
        assert torch.isfinite(z1.grad).all() and float(z1.grad[:, 3].abs().max()) == 0.0


@pytest.mark.parametrize("tag", ["u32", "b64", "w32"])
def test_jensenshannon_golden(tpw, golden, tag):
    """jensenshannon_distances (fused scale and root) and _sqjensenshannon against the reference's outputs and
    gradients, with and without a base; zero entries on one or both sides; a set against itself."""
    G = golden("jensenshannon")
    dt = torch.float32 if tag != "b64" else torch.float64
    tol = TOL[dt]
    up = cuda(G[f"{tag}/up"])
    for name, base in (("nat", None), ("base2", 2.0)):
        h1, h2 = cuda(G[f"{tag}/h1"], True), cuda(G[f"{tag}/h2"], True)
        out = tpw.jensenshannon_distances(h1, h2, base)
        close(out, G[f"{tag}/{name}/out"], tol, msg="jensenshannon " + name)
        out.backward(up)
        close(h1.grad, G[f"{tag}/{name}/gx1"], tol, 10, "jensenshannon grad_x1 " + name)
        close(h2.grad, G[f"{tag}/{name}/gx2"], tol, 10, "jensenshannon grad_x2 " + name)
        n1 = (h1.detach() / h1.detach().sum(-1, keepdim=True)).requires_grad_(True)
        n2 = (h2.detach() / h2.detach().sum(-1, keepdim=True)).requires_grad_(True)
        sq = tpw._sqjensenshannon(n1, n2, base)
        close(sq, G[f"{tag}/{name}/sq_out"], tol, msg="_sqjensenshannon " + name)
        sq.backward(up)
        close(n1.grad, G[f"{tag}/{name}/sq_gx1"], tol, 10, "_sqjensenshannon grad_x1 " + name)
        close(n2.grad, G[f"{tag}/{name}/sq_gx2"], tol, 10, "_sqjensenshannon grad_x2 " + name)
    h1 = cuda(G[f"{tag}/h1"], True)
    own = tpw.jensenshannon_distances(h1)
    close(own, G[f"{tag}/self_out"], tol, msg="jensenshannon self")
    assert float(own.detach().diagonal(dim1=-2, dim2=-1).abs().max()) == 0.0
    own.sum().backward()           # the zero diagonal contributes nothing instead of dividing by it
    assert torch.isfinite(h1.grad).all()
    if tag == "u32":
        close(tpw.cdist(cuda(G["u32/h1"]), cuda(G["u32/h2"]), "jensenshannon", base=3.0), G["u32/cdist_base3"], tol, msg="cdist base 3")
        with pytest.raises(TypeError, match="incompatible arguments base"):
            tpw.cdist(cuda(G["u32/h1"]), cuda(G["u32/h2"]), "euclidean", base=2.0)


@pytest.mark.parametrize("tag", ["u32", "b64", "w32"])
def test_haversine_golden(tpw, golden, tag):
    """haversine_distances against the reference's outputs and gradients; a set against itself has an exactly
    zero diagonal and finite gradients."""
    G = golden("haversine")
    dt = torch.float32 if tag != "b64" else torch.float64
    tol = TOL[dt]
    x1, x2 = cuda(G[f"{tag}/x1"], True), cuda(G[f"{tag}/x2"], True)
    out = tpw.haversine_distances(x1, x2)
    close(out, G[f"{tag}/out"], tol, msg="haversine")
    out.backward(cuda(G[f"{tag}/up"]))
    # The coefficient 1 / (sqrt(a) sqrt(1 - a)) grows without bound towards coincident and antipodal pairs, and
    # the float32 reference carries its own rounding there (its float32 and float64 gradients differ by 5e-4 on
    # these inputs).  Each term is therefore allowed a few float32 roundings of its own magnitude:
    # |grad - ref| <= rtol |ref| + atol + 4e-6 sum |g| / (sqrt(a) sqrt(1 - a)) over the reduced index.
    ref64 = O.haversine(G[f"{tag}/x1"].astype(np.float64), G[f"{tag}/x2"].astype(np.float64))
    a64 = np.sin(ref64 / 2) ** 2
    amp = np.abs(G[f"{tag}/up"].astype(np.float64)) / np.maximum(np.sqrt(a64 * (1 - a64)), 1e-300)
    eps = 4e-6 if dt == torch.float32 else 1e-14
    for got, key, axis in ((x1.grad, "gx1", -1), (x2.grad, "gx2", -2)):
        ref = G[f"{tag}/{key}"].astype(np.float64)
        bound = tol["rtol"] * np.abs(ref) + tol["atol"] + eps * amp.sum(axis)[..., None]
        err = np.abs(got.cpu().numpy().astype(np.float64) - ref)
        assert (err <= bound).all(), ("haversine " + key, float((err / bound).max()))
    y = cuda(G[f"{tag}/x1"], True)
    own = tpw.haversine_distances(y)
    close(own, G[f"{tag}/self_out"], tol, msg="haversine self")
    assert float(own.detach().diagonal(dim1=-2, dim2=-1).abs().max()) == 0.0
    own.sum().backward()
    assert torch.isfinite(y.grad).all()
    if tag == "u32":
        close(tpw.cdist(x1.detach(), x2.detach(), "haversine"), G["u32/cdist"], tol, msg="cdist haversine")
        with pytest.raises(RuntimeError, match="feature dimension of x1 and x2 must be 2"):
            tpw.haversine_distances(torch.zeros(4, 3, device="cuda"))


def test_jensenshannon_and_haversine_edge_cases(tpw):
    """Empty operands, batched inputs and narrow dtypes (widened to float32 on entry, rounded once on exit)."""
    z = torch.zeros(0, 2, device="cuda", requires_grad=True)
    y = torch.rand(5, 2, device="cuda", requires_grad=True)
    out = tpw.haversine_distances(z, y)
    assert out.shape == (0, 5)
    out.sum().backward()
    assert z.grad.shape == (0, 2) and float(y.grad.abs().max()) == 0.0
    h = torch.rand(0, 7, device="cuda")
    assert tpw.jensenshannon_distances(h, torch.rand(4, 7, device="cuda")).shape == (0, 4)
    g = torch.Generator().manual_seed(71)
    hb1, hb2 = torch.rand(3, 20, 11, generator=g).cuda(), torch.rand(3, 17, 11, generator=g).cuda()
    full = tpw.jensenshannon_distances(hb1, hb2, 2.0)
    for b in range(3):
        assert torch.equal(full[b], tpw.jensenshannon_distances(hb1[b], hb2[b], 2.0))
    pb1, pb2 = (torch.rand(3, 20, 2, generator=g) - 0.5).cuda(), (torch.rand(3, 17, 2, generator=g) - 0.5).cuda()
    fullh = tpw.haversine_distances(pb1, pb2)
    for b in range(3):
        assert torch.equal(fullh[b], tpw.haversine_distances(pb1[b], pb2[b]))
    for dt, tol in ((torch.float16, 2e-3), (torch.bfloat16, 2e-2)):
        o = tpw.jensenshannon_distances(hb1.to(dt), hb2.to(dt))
        assert o.dtype == dt
        ref = tpw.jensenshannon_distances(hb1.to(dt).float(), hb2.to(dt).float())
        assert float((o.float() - ref).abs().max()) <= tol
        o = tpw.haversine_distances(pb1.to(dt), pb2.to(dt))
        assert o.dtype == dt
        assert float((o.float() - tpw.haversine_distances(pb1.to(dt).float(), pb2.to(dt).float())).abs().max()) <= tol


def test_haversine_large_identities(tpw):
    """At a size no CPU loop finishes quickly: symmetry, the triangle inequality through a third set, the range
    [0, pi], and the backward of sum(out) against a float64 run of the same kernels."""
    g = torch.Generator().manual_seed(70)
    scale = torch.tensor([math.pi, 2 * math.pi])
    x1 = ((torch.rand(3001, 2, generator=g) - 0.5) * scale).cuda()
    x2 = ((torch.rand(2050, 2, generator=g) - 0.5) * scale).cuda()
    d12, d21 = tpw.haversine_distances(x1, x2), tpw.haversine_distances(x2, x1)
    assert torch.equal(d12, d21.t())
    assert float(d12.min()) >= 0.0 and float(d12.max()) <= math.pi + 1e-6
    x3 = x2[:64]
    via = (tpw.haversine_distances(x1, x3).unsqueeze(1) + tpw.haversine_distances(x2, x3).unsqueeze(0)).min(-1).values
    assert bool((d12 <= via + 2e-3).all())   # nearly antipodal pairs are ill-conditioned in float32 (asin near 1)
    # gradients on one octant of the sphere: no pair is close to antipodal, where the coefficient is unbounded
    x1, x2 = x1.abs() * 0.45, x2.abs() * 0.45
    a, b = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True)
    tpw.haversine_distances(a, b).sum().backward()
    c, d = x1.double().requires_grad_(True), x2.double().requires_grad_(True)
    tpw.haversine_distances(c, d).sum().backward()
    for got, ref in ((a.grad, c.grad), (b.grad, d.grad)):
        bound = 1e-4 * ref.abs() + 1e-3 * ref.abs().median()   # sums over thousands of pairs, some nearly antipodal
        assert bool(((got.double() - ref).abs() <= bound).all())


def test_bounded_wait_reports_instead_of_hanging(tpw):
    """A wait that can never complete gives up after its budget, leaves a code in the device status
    word and leaves the context usable (no trap, no fault, no endless loop)."""
    import time
    from torchpairwise_b200 import _abi
    assert tpw.device_status() == 0
    t0 = time.perf_counter()
    _abi.check(_abi.lib.tpw_selftest_bounded_wait(50, torch.cuda.current_stream().cuda_stream))
    code = tpw.device_status()  # synchronises, reads and clears
    dt = time.perf_counter() - t0
    assert code == (15 << 16) | 1
    assert 0.04 < dt < 5.0, dt   # 50 ms of waiting plus launch, module load and the status read-back
    assert tpw.device_status() == 0  # cleared
    x = torch.randn(64, 32, device="cuda")
    assert torch.isfinite(tpw.euclidean_distances(x)).all()  # the context still works
    assert _abi.lib.tpw_selftest_bounded_wait(0, None) == 1  # argument check


def test_layout_and_size_edges(tpw):
    g = torch.Generator().manual_seed(33)
    base1 = torch.randn(24, 50, generator=g).cuda()
    base2 = torch.randn(24, 41, generator=g).cuda()
    # non-contiguous views are made contiguous, as the reference's wrappers do
    x1, x2 = base1.t(), base2.t()          # [50, 24], [41, 24] with strides (1, 50)
    assert not x1.is_contiguous()
    ref = O.cdist(x1.cpu().numpy(), x2.cpu().numpy(), 3.0)
    close(tpw.minkowski_distances(x1, x2, 3.0), ref, TOL[torch.float32], msg="non-contiguous")
    close(tpw.cosine_distances(x1[::2], x2[::3]), O.cosine_distances(x1[::2].cpu().numpy(), x2[::3].cpu().numpy()),
          TOL[torch.float32], msg="strided rows")
    # more than 65535 row tiles in one launch, ragged last tile, D not a multiple of four
    xa = torch.randn(70001, 3, generator=g).cuda()
    xb = torch.randn(130, 3, generator=g).cuda()
    out = tpw.manhattan_distances(xa, xb)
    pick = torch.tensor([0, 1, 127, 128, 65535, 65536, 70000])
    close(out[pick.cuda()], O.cdist(xa[pick.cuda()].cpu().numpy(), xb.cpu().numpy(), 1.0), TOL[torch.float32], msg="many tiles")
    xbool = torch.rand(70001, 40, generator=g).cuda() < 0.4
    ybool = torch.rand(130, 40, generator=g).cuda() < 0.4
    jac = tpw.jaccard_distances(xbool, ybool)
    assert np.array_equal(jac[pick.cuda()].cpu().numpy(), O.boolean_metric("jaccard", xbool[pick.cuda()].cpu().numpy(), ybool.cpu().numpy()))
    # zero features: empty sums
    z1, z2 = torch.empty(5, 0, device="cuda"), torch.empty(4, 0, device="cuda")
    assert torch.equal(tpw.manhattan_distances(z1, z2), torch.zeros(5, 4, device="cuda"))
    assert torch.equal(tpw.cosine_distances(z1, z2), torch.ones(5, 4, device="cuda"))
    # mixed dtypes promote as torch.result_type does before comparing (hamming on non-boolean data)
    a8 = torch.randint(0, 3, (9, 13), generator=g).to(torch.int8).cuda()
    f32 = torch.randint(0, 3, (7, 13), generator=g).float().cuda()
    assert np.array_equal(tpw.hamming_distances(a8, f32).cpu().numpy(), O.hamming(a8.cpu().numpy(), f32.cpu().numpy()))
    # dtype and device mismatches are errors, as in the reference
    with pytest.raises(RuntimeError):
        tpw.sqeuclidean_distances(base1, base2.double()[:, :50])
    with pytest.raises(RuntimeError, match="same number of features"):
        tpw.euclidean_distances(base1, base2)
    with pytest.raises(RuntimeError, match="batch_size"):
        tpw.euclidean_distances(torch.randn(2, 4, 3, device="cuda"), torch.randn(3, 4, 3, device="cuda"))
