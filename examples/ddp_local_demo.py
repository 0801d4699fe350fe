"""Two CPU ranks train one Linear(2, 1) with explicit gradient synchronisation over the local
multiprocessing backend, and the result is checked against the same steps on the full batch in
one process.

    python examples/ddp_local_demo.py

Each rank sees one of two samples; the loss is the mean squared error.  DDP is built with
`sync_grads=False`, so the gradients are averaged where the script says so
(`all_reduce_gradients()` between `backward()` and `step()`).  Averaging the two per-rank
gradients equals the gradient of the two-sample mean, hence the comparison.
(reference project: examples/ddp_local_demo.py:21-82)
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
import orthon_b200.distributed as dist  # noqa: E402

STEPS = 3
LR = 0.05
INPUTS = np.asarray([[1.0, 2.0], [3.0, 4.0]], dtype=np.float32)
TARGETS = np.asarray([[1.5], [3.5]], dtype=np.float32)


def fixed_model():
    model = ob.nn.Linear(2, 1)
    weight, bias = list(model.parameters())
    weight.fill_(0.25)
    bias.fill_(0.1)
    return model


def flat_params(model):
    return [float(v) for p in model.parameters() for v in p.tolist()]


def mse(model, x, negated_target):
    diff = model(x) + negated_target
    return ob.mean(diff * diff)


def worker(rank):
    model = fixed_model()
    ddp = dist.DistributedDataParallel(model, sync_grads=False)
    optimizer = ob.optim.SGD(ddp.parameters(), lr=LR)
    x = ob.from_numpy(INPUTS[rank:rank + 1])
    t = ob.from_numpy(-TARGETS[rank:rank + 1])
    losses = []
    for _ in range(STEPS):
        loss = mse(ddp, x, t)
        losses.append(float(loss.item()))
        loss.backward()
        ddp.all_reduce_gradients()
        optimizer.step()
        optimizer.zero_grad()
    return {"rank": rank, "losses": losses, "final_params": flat_params(model)}


def single_process():
    model = fixed_model()
    optimizer = ob.optim.SGD(model.parameters(), lr=LR)
    x, t = ob.from_numpy(INPUTS), ob.from_numpy(-TARGETS)
    for _ in range(STEPS):
        loss = mse(model, x, t)
        loss.backward()
        optimizer.step()
        optimizer.zero_grad()
    return flat_params(model)


def main():
    results = dist.spawn(worker, nprocs=2, backend="local")
    for r in results:
        print(f"rank {r['rank']}: losses=[{', '.join(f'{v:.6f}' for v in r['losses'])}] "
              f"final_params=[{', '.join(f'{v:.6f}' for v in r['final_params'])}]")
    expected = single_process()
    worst = max(abs(a - b) for r in results for a, b in zip(r["final_params"], expected))
    print(f"full-batch single process: [{', '.join(f'{v:.6f}' for v in expected)}]  max difference {worst:.2e}")
    if results[0]["final_params"] != results[1]["final_params"] or worst > 1e-6:
        raise RuntimeError("replicas diverged from the full-batch run")
    return worst


if __name__ == "__main__":
    main()
