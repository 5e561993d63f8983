"""Row sharding over the GPUs of one box, on hardware: one process per GPU over NCCL (started as child processes with
torch.distributed.run), every rank comparing its slab and its gradients with the one-GPU result of the same
operator.  Skipped on a box with a single GPU; the partition logic and the gradient all-reduce are also covered on
CPU with gloo (tests/test_host_logic.py)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["TPW_ROOT"])
import torchpairwise_b200 as tpw
from torchpairwise_b200 import sharding

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=dev)
tpw.load_torch_ops()
T = torch.ops.torchpairwise

def worst(x):
    t = torch.tensor([float(x)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())

g = torch.Generator().manual_seed(5)
# forward only, unbatched: rows of x1 over the ranks, x2 broadcast from rank 0 (every other rank starts from zeros)
X = torch.randn(1000, 96, generator=g).to(dev)
Y = torch.randn(700, 96, generator=g).to(dev)
kind, ranges = sharding.plan_shards(tuple(X.shape), world)
assert kind == "rows"
lo, hi = ranges[rank]
for name, fn, exact in (("sqeuclidean", T.sqeuclidean_distances, True), ("manhattan", T.manhattan_distances, True),
                        ("cosine", T.cosine_distances, True)):
    y_in = Y if rank == 0 else torch.zeros_like(Y)
    slab = sharding.sharded_pairwise(fn, X[lo:hi].contiguous(), y_in, src=0)
    full = fn(X, Y)
    err = (slab - full[lo:hi]).abs().max() if slab.numel() else 0.0
    assert worst(err) <= 1e-5 * float(full.abs().max()), (name, float(err))
# boolean metric, bit-exact
xb, yb = X > 0.3, Y > 0.3
slab = sharding.sharded_pairwise(T.jaccard_distances, xb[lo:hi].contiguous(), yb if rank == 0 else torch.zeros_like(yb), src=0)
assert worst((slab != T.jaccard_distances(xb, yb)[lo:hi]).sum()) == 0
# forward + backward, batched with fewer batches than ranks: x2 gradient partials are all-reduced
nb = 1
X1 = torch.randn(nb, 600, 64, generator=g).to(dev)
X2 = torch.randn(nb, 500, 64, generator=g).to(dev)
G = torch.randn(nb, 600, 500, generator=g).to(dev)
kind, ranges = sharding.plan_shards(tuple(X1.shape), world)
lo, hi = ranges[rank]
for fn, kw in ((T.minkowski_distances, {"p": 3.0}), (T.chebyshev_distances, {}), (T.euclidean_distances, {})):
    x1l = sharding.local_block(X1, kind, ranges, rank).contiguous().requires_grad_(True)
    x2l = (X2.clone() if rank == 0 else torch.zeros_like(X2)).requires_grad_(True)
    out = sharding.sharded_pairwise(fn, x1l, x2l, src=0, **kw)
    out.backward(sharding.local_block(G, kind, ranges, rank).contiguous())
    a, b = X1.clone().requires_grad_(True), X2.clone().requires_grad_(True)
    full = fn(a, b, **kw)
    full.backward(G)
    scale = 10 * max(1.0, float(b.grad.abs().max()))
    e1 = (x1l.grad - a.grad[:, lo:hi]).abs().max() if x1l.numel() else 0.0
    e2 = (x2l.grad - b.grad).abs().max()
    assert worst(e1) <= 1e-5 * scale and worst(e2) <= 1e-5 * scale, (str(fn), float(e1), float(e2))
assert tpw.device_status() == 0
dist.barrier()
dist.destroy_process_group()
if rank == 0:
    print("sharded ok", world)
'''


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_slabs_and_gradients_match_one_gpu(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, TPW_ROOT=str(ROOT), NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), str(script)],
                       cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and f"sharded ok {world}" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
