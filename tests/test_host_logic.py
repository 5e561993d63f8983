"""Host-side behaviour that needs no GPU: input checks, the cdist dispatcher's keyword validation,
the shard planner, and the differentiable broadcast over two gloo ranks."""
import os
import socket
import warnings

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import torchpairwise_b200 as tpw
from torchpairwise_b200 import ops, sharding


def test_cpu_tensors_are_rejected_loudly():
    x = torch.randn(4, 3)
    for fn in (tpw.euclidean_distances, tpw.manhattan_distances, tpw.cosine_distances, tpw.sqeuclidean_distances,
               tpw.hamming_distances, tpw.correlation_distances):
        with pytest.raises(RuntimeError, match="CUDA tensors only"):
            fn(x)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with pytest.raises(RuntimeError, match="CUDA tensors only"):
            tpw.jaccard_distances(x)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        tpw.directed_hausdorff_distances(torch.rand(2, 5, 3))


def test_check_pairwise_inputs_messages():
    with pytest.raises(RuntimeError, match="x1 must be 2D tensor \\(unbatched\\) or 3D tensor \\(batched\\)"):
        ops.check_pairwise_inputs("euclidean_distances", torch.randn(3))
    with pytest.raises(RuntimeError, match="same number of features. Got: x1.size\\(1\\)=4, x2.size\\(1\\)=5"):
        ops.check_pairwise_inputs("euclidean_distances", torch.randn(3, 4), torch.randn(2, 5))
    with pytest.raises(RuntimeError, match="x2 must be 2D tensor"):
        ops.check_pairwise_inputs("euclidean_distances", torch.randn(2, 3, 4), torch.randn(3, 4))
    with pytest.raises(RuntimeError, match="x1 must be 3D tensor \\(unbatched\\) or 4D tensor \\(batched\\)"):
        ops.check_pairwise_inputs("directed_hausdorff_distances", torch.randn(3, 4), sets=True)
    a, b = ops.check_pairwise_inputs("euclidean_distances", torch.randn(3, 4))
    assert a is b
    with pytest.warns(UserWarning, match="converted to torch.bool for metric jaccard_distances"):
        a, b = ops.check_pairwise_inputs("jaccard_distances", torch.randint(0, 2, (3, 4)), boolean=True)
    assert a.dtype == torch.bool and a is b


def test_cdist_keyword_validation():
    x = torch.randn(3, 4)
    with pytest.raises(TypeError, match="euclidean_distances was called with incompatible arguments p"):
        tpw.cdist(x, x, "euclidean", p=2.0)
    with pytest.raises(TypeError, match="incompatible arguments w, V"):
        tpw.cdist(x, x, "minkowski", w=x[0], V=x[0], p=3.0)
    with pytest.raises(TypeError, match="shuffle"):
        tpw.cdist(x, x, "hamming", shuffle=True)
    with pytest.raises(RuntimeError, match="Got unkown distance metric: foo"):
        tpw.cdist(x, x, "foo")
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        tpw.cdist(x[:, :2], x[:, :2], "haversine")
    with pytest.raises(TypeError, match="incompatible arguments base"):
        tpw.cdist(x, x, "haversine", base=2.0)
    # pdist validates like cdist, then needs a CUDA tensor (the reference only has a stub that raises)
    with pytest.raises(TypeError, match="incompatible arguments p"):
        tpw.pdist(x, "euclidean", p=2.0)
    with pytest.raises(RuntimeError, match="Got unkown distance metric: foo"):
        tpw.pdist(x, "foo")
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        tpw.pdist(x)
    # valid keywords get past validation and then hit the device check
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        tpw.cdist(x, x, "minkowski", p=3.0)


def test_prf_div_mode_check():
    with pytest.raises(RuntimeError, match="mode must be either zero or identity"):
        tpw.prf_div(torch.ones(2), torch.ones(2), "nope")


def test_split_range_and_plan():
    assert sharding.split_range(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert sharding.split_range(2, 4) == [(0, 1), (1, 2), (2, 2), (2, 2)]
    assert sharding.split_range(0, 2) == [(0, 0), (0, 0)]
    for n in (0, 1, 7, 131072, 131073):
        for w in (1, 2, 4, 8):
            r = sharding.split_range(n, w)
            assert r[0][0] == 0 and r[-1][1] == n and all(a[1] == b[0] for a, b in zip(r, r[1:]))
            assert max(b - a for a, b in r) - min(b - a for a, b in r) <= 1
    assert sharding.plan_shards((16, 4096, 256), 8) == ("batch", sharding.split_range(16, 8))
    assert sharding.plan_shards((2, 4096, 256), 8) == ("rows", sharding.split_range(4096, 8))
    assert sharding.plan_shards((131072, 512), 8) == ("rows", sharding.split_range(131072, 8))
    x = torch.arange(24.).view(2, 6, 2)
    kind, ranges = sharding.plan_shards(tuple(x.shape), 4)
    assert kind == "rows"
    assert torch.equal(torch.cat([sharding.local_block(x, kind, ranges, r) for r in range(4)], 1), x)
    assert sharding.local_block(x, kind, ranges, 1, is_x2=True) is x


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _sharded_worker(rank, world, port, n1, n2, d):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        x1 = torch.randn(n1, d, generator=g, dtype=torch.float64)
        x2 = torch.randn(n2, d, generator=g, dtype=torch.float64)
        up = torch.randn(n1, n2, generator=g, dtype=torch.float64)
        kind, ranges = sharding.plan_shards((n1, d), world)
        lo, hi = ranges[rank]
        a = sharding.local_block(x1, kind, ranges, rank).clone().requires_grad_(True)
        # only rank 0 owns x2; the others pass a buffer of the right shape
        b = (x2.clone() if rank == 0 else torch.zeros_like(x2)).requires_grad_(True)
        # torch.cdist stands in for the CUDA operator: this test is about the plumbing around it
        out = sharding.sharded_pairwise(lambda u, v: torch.cdist(u, v, p=1.0), a, b, src=0)
        assert out.shape == (hi - lo, n2)
        full = torch.cdist(x1, x2, p=1.0)
        assert torch.allclose(out, full[lo:hi])
        out.backward(up[lo:hi])
        xr, yr = x1.clone().requires_grad_(True), x2.clone().requires_grad_(True)
        torch.cdist(xr, yr, p=1.0).backward(up)
        assert torch.allclose(a.grad, xr.grad[lo:hi])
        assert torch.allclose(b.grad, yr.grad), "grad_x2 must be the sum over all row blocks"
        # the same slab as column panels, x2 broadcast in row chunks that are queued at once
        for panels in (1, 2, 3, 7):
            buf = x2.clone() if rank == 0 else torch.zeros_like(x2)
            parts = sharding.sharded_pairwise_panels(lambda u, v: torch.cdist(u, v, p=1.0), a.detach(), buf, src=0, panels=panels)
            assert len(parts) == min(panels, n2) and torch.allclose(torch.cat(parts, -1), full[lo:hi])
            assert torch.equal(buf, x2), "every rank holds the broadcast x2 afterwards"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n1", [9, 2])
def test_row_sharding_over_two_gloo_ranks(n1):
    mp.spawn(_sharded_worker, args=(2, _free_port(), n1, 5, 3), nprocs=2, join=True)
