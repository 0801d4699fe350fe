"""MLP 784-256-128-10 on synthetic data: three SGD steps on the CPU, the same steps with
two local DDP ranks, then a checkpoint round trip.

    python examples/mlp_checkpoint.py
"""
import os
import sys
import tempfile

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
import orthon_b200.distributed as dist  # noqa: E402
from orthon_b200.models import MLP  # noqa: E402


def batch(step, rank=0, n=64):
    rng = np.random.default_rng(1000 * step + rank)
    return ob.from_numpy(rng.standard_normal((n, 784)).astype(np.float32)), [int(v) for v in rng.integers(0, 10, n)]


def single(steps=3):
    ob.manual_seed(0)
    model = MLP()
    opt = ob.optim.SGD(model.parameters(), lr=0.01)
    out = []
    for s in range(steps):
        x, y = batch(s)
        out.append(ob.training.train_step(model, x, y, ob.cross_entropy, opt))
    return model, opt, out


def ddp_worker(rank, steps):
    ob.manual_seed(0)
    model = MLP()
    ddp = dist.DDP(model, bucket_size_mb=25)
    opt = ob.optim.SGD(model.parameters(), lr=0.01)
    losses = []
    for s in range(steps):
        x, y = batch(s, rank, 32)
        ddp.zero_grad()
        loss = ob.cross_entropy(ddp(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses, next(iter(model.parameters())).tolist()[:4]


def main():
    model, opt, metrics = single()
    print("single process:", [round(m["loss"], 4) for m in metrics])
    results = dist.spawn(ddp_worker, args=(3,), nprocs=2, backend="local")
    print("local DDP (2 ranks):", [[round(v, 4) for v in r[0]] for r in results])
    assert results[0][1] == results[1][1], "replicas diverged"
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "mlp.ckpt")
        ob.save_checkpoint(path, model, opt, {"steps": 3})
        ob.manual_seed(1)
        clone = MLP()
        clone_opt = ob.optim.SGD(clone.parameters(), lr=1.0)
        meta = ob.load_checkpoint(path, clone, clone_opt)
        same = all(a.tolist() == b.tolist() for a, b in zip(model.parameters(), clone.parameters()))
        print("checkpoint round trip:", meta, "identical parameters:", same, "lr:", clone_opt.get_lr())
        assert same and clone_opt.get_lr() == 0.01


if __name__ == "__main__":
    main()
