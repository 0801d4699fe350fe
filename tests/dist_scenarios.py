"""More worker functions for the multi-process CPU tests (local backend)."""
import numpy as np


def facade(rank):
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    out = {"rank": dist.get_rank(), "world": dist.get_world_size(), "init": dist.is_initialized()}
    t = ob.from_numpy(np.full([5], float(rank + 1), dtype=np.float32))
    work = dist.all_reduce(t, async_op=True)
    work.wait()
    out["async_done"] = bool(work.is_completed())
    out["sum"] = t.tolist()
    b = ob.from_numpy(np.arange(4, dtype=np.float32) + 10 * rank)
    dist.broadcast(b, src=1)
    out["bcast"] = b.tolist()
    dist.barrier()
    try:
        dist.init_process_group("local")
    except RuntimeError as exc:
        out["double_init"] = str(exc)
    return out


def _tiny(seed):
    import orthon_b200 as ob
    ob.manual_seed(seed)
    return ob.nn.Sequential(ob.nn.Linear(6, 8), ob.nn.ReLU(), ob.nn.Linear(8, 3))


def accumulation(rank):
    """Two backward passes before one step: gradients accumulate locally and the synchronised
    gradient is the average over ranks of the accumulated sums."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    model = _tiny(3)
    ddp = dist.DDP(model, sync_grads=False)
    rng = np.random.default_rng(50 + rank)
    ddp.zero_grad()
    for _ in range(2):
        x = ob.from_numpy(rng.standard_normal((4, 6)).astype(np.float32))
        y = [int(v) for v in rng.integers(0, 3, 4)]
        ob.cross_entropy(ddp(x), y).backward()
    local = [np.asarray(p.grad.tolist()) for p in model.parameters()]
    ddp.all_reduce_gradients()
    ddp.wait_for_gradient_sync()
    synced = [np.asarray(p.grad.tolist()) for p in model.parameters()]
    return [g.tolist() for g in local], [g.tolist() for g in synced]


class _Tied:
    pass


def tied_parameters(rank):
    """A weight used twice is one owner: reduced once, replicas stay identical."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    from orthon_b200 import nn

    class Tied(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(9, 5)
            self.out = nn.Linear(5, 5)

        def forward(self, ids):
            h = self.out(self.emb(ids).mean(1))
            return h @ self.emb.weight.transpose(0, 1)

    ob.manual_seed(5)
    model = Tied()
    ddp = dist.DDP(model)
    opt = ob.optim.SGD(model.parameters(), lr=0.1)
    rng = np.random.default_rng(70 + rank)
    for _ in range(3):
        ids = ob.from_numpy(rng.integers(0, 9, size=(4, 3)).astype(np.int64))
        ddp.zero_grad()
        ob.cross_entropy(ddp(ids), [int(v) for v in rng.integers(0, 9, 4)]).backward()
        opt.step()
    return len(list(model.parameters())), np.concatenate([np.asarray(p.tolist()) for p in model.parameters()]).tolist()


def amp_inf_on_one_rank(rank):
    """Rank 1 produces a non-finite gradient in step 1: every rank skips that update and halves
    the scale; the other steps apply normally and replicas stay identical."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    model = _tiny(7)
    ddp = dist.DDP(model, sync_grads=False)
    opt = ob.amp.MixedPrecisionOptimizer(ddp, ob.optim.Adam, lr=1e-2)
    scaler = ob.amp.GradScaler(init_scale=64.0)
    rng = np.random.default_rng(90 + rank)
    trace = []
    for step in range(3):
        x = ob.from_numpy(rng.standard_normal((4, 6)).astype(np.float32))
        y = [int(v) for v in rng.integers(0, 3, 4)]
        opt.zero_grad()
        loss = ob.cross_entropy(ddp(x), y)
        if step == 1 and rank == 1:
            loss = loss * float("inf")
        before = np.concatenate([np.asarray(p.tolist()) for p in model.parameters()])
        scaler.scale(loss).backward()
        scaler.step(opt)
        skipped = scaler.found_inf
        scaler.update()
        after = np.concatenate([np.asarray(p.tolist()) for p in model.parameters()])
        trace.append((bool(skipped), float(scaler.scale_factor), bool(np.array_equal(before, after))))
    return trace, np.concatenate([np.asarray(p.tolist()) for p in model.parameters()]).tolist()


def partially_used_parameter(rank):
    """Rank 1 never touches the second head: it contributes zeros and receives the average."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    from orthon_b200 import nn

    class TwoHeads(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(4, 3)
            self.b = nn.Linear(4, 3)

        def forward(self, x, use_b):
            y = self.a(x)
            return y + self.b(x) if use_b else y

    ob.manual_seed(9)
    model = TwoHeads()
    ddp = dist.DDP(model)
    x = ob.from_numpy(np.random.default_rng(3).standard_normal((2, 4)).astype(np.float32))
    ddp.zero_grad()
    ddp(x, rank == 0).sum().backward()
    gb = model.b.weight.grad
    return None if gb is None else np.asarray(gb.tolist()).tolist(), np.asarray(model.a.weight.grad.tolist()).tolist()


def lifecycle(rank):
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    t = ob.from_numpy(np.ones([2], dtype=np.float32))
    dist.all_reduce(t)
    dist.destroy_process_group()
    after = dist.is_initialized()
    try:
        dist.all_reduce(t)
        err = None
    except RuntimeError as exc:
        err = str(exc)
    return t.tolist(), after, err
