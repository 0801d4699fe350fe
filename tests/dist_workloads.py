"""Worker functions for multi-process tests (importable by spawned children)."""
import numpy as np


def _device(backend, rank):
    return "cpu" if backend == "local" else f"cuda:{rank}"


def collectives(rank, backend):
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    from orthon_b200 import _C
    dev = _device(backend, rank)
    ws = dist.get_world_size()
    out = {}
    for n in (1, 7, 1000, 300_000):
        t = _C.from_numpy(np.full([n], float(rank + 1), dtype=np.float32))
        t = t if dev == "cpu" else t.to(dev)
        dist.all_reduce(t)
        out[f"sum{n}"] = (t.tolist()[0], t.tolist()[-1])
    b = _C.from_numpy(np.arange(12, dtype=np.float32).reshape(3, 4) * (rank + 1))
    b = b if dev == "cpu" else b.to(dev)
    dist.broadcast(b, src=ws - 1)
    out["bcast"] = b.tolist()
    dist.barrier()
    if dev != "cpu":
        h = _C.from_numpy(np.full([4096], 0.5 * (rank + 1), dtype=np.float32), "bfloat16").to(dev)
        dist.all_reduce(h)
        out["bf16"] = h.tolist()[:2]
    return out


def _make_model(seed, dtype, dev):
    import orthon_b200 as ob
    ob.manual_seed(seed)
    m = ob.nn.Sequential(ob.nn.Linear(24, 32), ob.nn.ReLU(), ob.nn.Linear(32, 16), ob.nn.ReLU(), ob.nn.Linear(16, 5))
    if dtype != "float32":
        m.cast(dtype)
    if dev != "cpu":
        m.to(dev)
    return m


def _batch(step, rank, dev, dtype="float32"):
    from orthon_b200 import _C
    rng = np.random.default_rng(1000 * step + rank)
    x = _C.from_numpy(rng.standard_normal((8, 24)).astype(np.float32), dtype)
    y = _C.from_numpy(rng.integers(0, 5, 8).astype(np.int64))
    return (x, y) if dev == "cpu" else (x.to(dev), y.to(dev))


def ddp_sgd_trace(rank, backend, steps, bucket_mb):
    """Plain DDP + SGD; returns final flat parameters and the loss trace."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    dev = _device(backend, rank)
    model = _make_model(11, "float32", dev)
    ddp = dist.DDP(model, bucket_size_mb=bucket_mb)
    opt = ob.optim.SGD(model.parameters(), lr=0.05)
    losses = []
    for step in range(steps):
        x, y = _batch(step, rank, dev)
        ddp.zero_grad()
        loss = ob.cross_entropy(ddp(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    flat = np.concatenate([p.numpy().reshape(-1) for p in model.parameters()])
    return flat.tolist(), losses, type(ddp._reducer).__name__


def amp_ddp_trace(rank, backend, steps, dtype, fused, use_scaler):
    """AMP + DDP(sync_grads=False) + Adam; returns final master values and losses."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    dev = _device(backend, rank)
    model = _make_model(13, dtype, dev)
    ddp = dist.DDP(model, sync_grads=False, bucket_size_mb=1)
    opt = ob.amp.MixedPrecisionOptimizer(ddp, ob.optim.Adam, fused=fused, lr=1e-2)
    scaler = ob.amp.GradScaler(init_scale=128.0, enabled=use_scaler)
    losses = []
    for step in range(steps):
        x, y = _batch(step, rank, dev, dtype)
        opt.zero_grad()
        loss = ob.cross_entropy(ddp(x), y)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        losses.append(loss.item())
    ob.cuda_synchronize() if dev != "cpu" else None
    masters = np.concatenate([s.master.numpy().reshape(-1) for s in opt._states])
    model_vals = np.concatenate([p.numpy().astype(np.float32).reshape(-1) for p in model.parameters()])
    return masters.tolist(), model_vals.tolist(), losses, opt._inner._t


def single_process_reference(world, steps, dtype="float32", optimizer="sgd", lr=0.05):
    """Same math in one process: gradients averaged over the per-rank batches by hand."""
    import orthon_b200 as ob
    model = _make_model(11 if optimizer == "sgd" else 13, "float32", "cpu")
    params = list(model.parameters())
    opt = ob.optim.SGD(params, lr=lr) if optimizer == "sgd" else ob.optim.Adam(params, lr=lr)
    for step in range(steps):
        sums = None
        for rank in range(world):
            x, y = _batch(step, rank, "cpu")
            for p in params:
                p.zero_grad()
            ob.cross_entropy(model(x), y).backward()
            g = [p.grad.numpy().copy() for p in params]
            sums = g if sums is None else [a + b for a, b in zip(sums, g)]
        for p, g in zip(params, sums):
            p.set_grad(ob.from_numpy((g / world).astype(np.float32)))
        opt.step()
    return np.concatenate([p.numpy().reshape(-1) for p in params])


def nvls_reduce(rank, backend, dtype, n):
    """Kernel-level check of the in-switch (multimem) reducer against the peer-load reducer on
    the same multicast-bound region.  Returns {"skipped": reason} where NVLS is unavailable."""
    import os
    os.environ["ORTHON_NVLS"] = "1"
    import orthon_b200.distributed as dist
    from orthon_b200 import _C
    from orthon_b200.distributed import group as _group
    be = _group.active().backend
    ws = dist.get_world_size()
    dev = f"cuda:{rank}"
    esz = 4 if dtype == "float32" else 2
    flag_bytes = (_C._PEER_FLAG_BYTES + 255) & ~255
    region = be.allocate_symmetric(n * esz + n * 4 + flag_bytes, multicast=True)
    if region.mc is None:
        return {"skipped": "no multicast mapping on this box"}
    grads = list(region.ptrs)
    staging = [p + n * esz for p in region.ptrs]
    flags = [p + n * esz + n * 4 for p in region.ptrs]
    grad_t = _C._tensor_from_ptr(region.local, [n], dtype, rank)
    status, found = be.status_tensors()
    rng = np.random.default_rng(7)
    base = rng.standard_normal(n).astype(np.float32)
    out = {}

    def fill():
        grad_t._copy_flat_range_from(0, _C.from_numpy(base * (rank + 1), dtype).to(dev), 0, n)
        _C.cuda_synchronize()
        dist.barrier()

    for name, mc in (("nvls", region.mc), ("peer", 0)):
        fill()
        _C._peer_reduce(rank, ws, rank, grads, staging, flags, n, dtype, be.next_epoch(), 1.0 / ws, "average", False,
                        status=status, found_inf=found, stream_kind=0, mc_grads=mc)
        _C.cuda_synchronize()
        dist.barrier()
        out[name] = np.asarray(grad_t.tolist(), dtype=np.float32)
    # Fused Adam through the NVLS variant: one step from zero state.
    fill()
    master = _C._zeros_on([n], "float32", dev)
    m, v = _C._zeros_on([n], "float32", dev), _C._zeros_on([n], "float32", dev)
    model = None if dtype == "float32" else _C._zeros_on([n], dtype, dev)
    _C._peer_reduce(rank, ws, rank, grads, staging, flags, n, dtype, be.next_epoch(), 1.0 / ws, "adam", False,
                    master=master, m=m, v=v, model=model,
                    hyper=dict(lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, bias_c1=0.1, bias_c2=0.001),
                    status=status, found_inf=found, stream_kind=0, mc_grads=region.mc)
    _C.cuda_synchronize()
    be.check_status()
    dist.barrier()
    expect = base * sum(r + 1 for r in range(ws)) / ws
    return {"nvls": out["nvls"].tolist(), "peer": out["peer"].tolist(), "expect": expect.tolist(),
            "master": master.tolist(), "found_inf": int(found.tolist()[0])}


# ------------------------------------------------------------------ peer-path scenarios (GPU ranks)
def _small_model(seed, dev, dtype="float32"):
    import orthon_b200 as ob
    ob.manual_seed(seed)
    m = ob.nn.Sequential(ob.nn.Linear(6, 8), ob.nn.ReLU(), ob.nn.Linear(8, 3))
    if dtype != "float32":
        m.cast(dtype)
    return m.to(dev) if dev != "cpu" else m


def _flat_params(model):
    return np.concatenate([p.numpy().astype(np.float32).reshape(-1) for p in model.parameters()])


def accumulation_explicit_sync(rank, backend):
    """Two backward passes, then one explicit synchronisation: the result is the average over
    ranks of the locally accumulated sums (the wrapper was built with sync_grads=False)."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    dev = _device(backend, rank)
    model = _small_model(3, dev)
    ddp = dist.DDP(model, sync_grads=False, bucket_size_mb=1)
    rng = np.random.default_rng(50 + rank)
    ddp.zero_grad()
    for _ in range(2):
        x = ob.from_numpy(rng.standard_normal((4, 6)).astype(np.float32)).to(dev)
        y = ob.from_numpy(rng.integers(0, 3, 4).astype(np.int64)).to(dev)
        ob.cross_entropy(ddp(x), y).backward()
    local = [p.grad.numpy().copy() for p in model.parameters()]
    ddp.all_reduce_gradients()
    ddp.wait_for_gradient_sync()
    synced = [p.grad.numpy().copy() for p in model.parameters()]
    return [g.tolist() for g in local], [g.tolist() for g in synced], type(ddp._reducer).__name__


def amp_accumulation(rank, backend, fused):
    """AMP + GradScaler with two micro-batches per step.  'reduce' accumulates locally and
    averages in step(); 'overlap' and 'update' reduce inside backward and must refuse the
    second backward.  Returns the final masters, or the refusal text."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    dev = _device(backend, rank)
    model = _small_model(21, dev)
    ddp = dist.DDP(model, sync_grads=False, bucket_size_mb=1)
    opt = ob.amp.MixedPrecisionOptimizer(ddp, ob.optim.Adam, fused=fused, lr=1e-2)
    scaler = ob.amp.GradScaler(init_scale=8.0, enabled=fused != "update")
    refused = None
    for step in range(2):
        opt.zero_grad()
        for micro in range(2):
            rng = np.random.default_rng(1000 * step + 10 * micro + rank)
            x = ob.from_numpy(rng.standard_normal((4, 6)).astype(np.float32)).to(dev)
            y = ob.from_numpy(rng.integers(0, 3, 4).astype(np.int64)).to(dev)
            try:
                scaler.scale(ob.cross_entropy(ddp(x), y) * 0.5).backward()
            except RuntimeError as exc:
                refused = str(exc)
                break
        if refused:
            break
        scaler.step(opt)
        scaler.update()
    ob.cuda_synchronize()
    dist.barrier()
    return refused, _flat_params(model).tolist()


def amp_accumulation_reference(world):
    """The same two steps of two micro-batches in one process (gradients averaged by hand)."""
    import orthon_b200 as ob
    model = _small_model(21, "cpu")
    params = list(model.parameters())
    opt = ob.optim.Adam(params, lr=1e-2)
    for step in range(2):
        total = [np.zeros(tuple(p.shape), dtype=np.float32) for p in params]
        for rank in range(world):
            for micro in range(2):
                rng = np.random.default_rng(1000 * step + 10 * micro + rank)
                x = ob.from_numpy(rng.standard_normal((4, 6)).astype(np.float32))
                y = [int(v) for v in rng.integers(0, 3, 4)]
                for p in params:
                    p.zero_grad()
                (ob.cross_entropy(model(x), y) * 0.5).backward()
                total = [t + p.grad.numpy() for t, p in zip(total, params)]
        for p, g in zip(params, total):
            p.set_grad(ob.from_numpy((g / world).astype(np.float32)))
        opt.step()
    return _flat_params(model)


def amp_inf_on_last_rank(rank, backend, fused):
    """The last rank overflows in step 1: every rank must skip that update, halve the scale and
    stay bit-identical."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    dev = _device(backend, rank)
    ws = dist.get_world_size()
    model = _small_model(7, dev)
    ddp = dist.DDP(model, sync_grads=False, bucket_size_mb=1)
    opt = ob.amp.MixedPrecisionOptimizer(ddp, ob.optim.Adam, fused=fused, lr=1e-2)
    scaler = ob.amp.GradScaler(init_scale=64.0)
    rng = np.random.default_rng(90 + rank)
    trace = []
    for step in range(3):
        x = ob.from_numpy(rng.standard_normal((4, 6)).astype(np.float32)).to(dev)
        y = ob.from_numpy(rng.integers(0, 3, 4).astype(np.int64)).to(dev)
        opt.zero_grad()
        loss = ob.cross_entropy(ddp(x), y)
        if step == 1 and rank == ws - 1:
            loss = loss * float("inf")
        before = _flat_params(model)
        scaler.scale(loss).backward()
        scaler.step(opt)
        skipped = scaler.found_inf
        scaler.update()
        trace.append((bool(skipped), float(scaler.scale_factor), bool(np.array_equal(before, _flat_params(model)))))
    return trace, _flat_params(model).tolist()


def found_inf_in_a_late_block(rank, backend, n):
    """Kernel level: one non-finite value near the end of the last rank's bucket (an element that
    a high-numbered thread block reduces) must raise the found-inf word on every rank."""
    import orthon_b200.distributed as dist
    from orthon_b200 import _C
    from orthon_b200.distributed import group as _group
    be = _group.active().backend
    ws = dist.get_world_size()
    dev = f"cuda:{rank}"
    flag_bytes = (_C._PEER_FLAG_BYTES + 255) & ~255
    region = be.allocate_symmetric(n * 4 + n * 4 + flag_bytes)
    grads, staging = list(region.ptrs), [p + n * 4 for p in region.ptrs]
    flags = [p + 8 * n for p in region.ptrs]
    grad_t = _C._tensor_from_ptr(region.local, [n], "float32", rank)
    status, found = be.status_tensors()
    out = {}
    for name, poison in (("clean", False), ("poisoned", True)):
        host = np.full([n], float(rank + 1), dtype=np.float32)
        if poison and rank == ws - 1:
            host[n - 3] = np.inf
        grad_t._copy_flat_range_from(0, _C.from_numpy(host).to(dev), 0, n)
        _C.cuda_synchronize()
        dist.barrier()
        blocks = _C._peer_reduce(rank, ws, rank, grads, staging, flags, n, "float32", be.next_epoch(), 1.0 / ws, "average", False,
                                 status=status, found_inf=found, stream_kind=0)
        _C.cuda_synchronize()
        code, hit = be.read_words()
        out[name] = (int(code), bool(hit), int(blocks), float(grad_t.tolist()[0]))
        found.fill_(0.0)
        dist.barrier()
    return out


def participation(rank, backend, case):
    """Rank-divergent participation on the default (non-overlapped) schedule.
    case 'partial': only rank 0 uses head b -> idle ranks contribute zeros, all get the average.
    case 'unused' : nobody uses head b -> its gradient stays None everywhere.
    case 'invalid': the optimizer update is fused into the reduction and rank 0 has no gradient
                    for head b -> no rank applies the step and every rank is told."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    from orthon_b200 import nn
    dev = _device(backend, rank)

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
    if dev != "cpu":
        model.to(dev)
    ddp = dist.DDP(model, sync_grads=False, bucket_size_mb=1)
    x = ob.from_numpy(np.random.default_rng(3).standard_normal((2, 4)).astype(np.float32))
    x = x if dev == "cpu" else x.to(dev)
    error, unchanged = None, None
    if case == "invalid":
        opt = ob.amp.MixedPrecisionOptimizer(ddp, ob.optim.SGD, fused="update", lr=0.5)
        before = _flat_params(model)
        opt.zero_grad()
        ddp(x, rank != 0).sum().backward()
        try:
            opt.step()
            ddp.wait_for_gradient_sync()
        except RuntimeError as exc:
            error = str(exc)
        ob.cuda_synchronize()
        unchanged = bool(np.array_equal(before, _flat_params(model)))
    else:
        ddp.zero_grad()
        ddp(x, case == "partial" and rank == 0).sum().backward()
        try:
            ddp.all_reduce_gradients()
            ddp.wait_for_gradient_sync()
        except RuntimeError as exc:
            error = str(exc)
    dist.barrier()
    gb = model.b.weight.grad
    return {"error": error, "b": None if gb is None else gb.numpy().tolist(), "unchanged": unchanged,
            "a": None if error else model.a.weight.grad.numpy().tolist(), "reducer": type(ddp._reducer).__name__}


def missing_peer(rank, backend):
    """Rank 0 launches a bucket that no other rank ever launches, with a wait budget of 100 ms and
    without multicast.  Its kernel must come back, the status word must name the entry barrier
    and the group must stay failed; the other ranks, which were between steps, shut down normally."""
    import orthon_b200.distributed as dist
    from orthon_b200 import _C
    from orthon_b200.distributed import group as _group
    group = _group.active()
    be = group.backend
    ws = dist.get_world_size()
    n = 1 << 16
    flag_bytes = (_C._PEER_FLAG_BYTES + 255) & ~255
    region = be.allocate_symmetric(n * 4 + n * 4 + flag_bytes)
    out = {"rank": rank}
    dist.barrier()
    if rank == 0:
        status, found = be.status_tensors()
        _C._peer_reduce(rank, ws, rank, list(region.ptrs), [p + 4 * n for p in region.ptrs], [p + 8 * n for p in region.ptrs], n,
                        "float32", be.next_epoch(), 1.0, "average", False, status=status, found_inf=found, stream_kind=0,
                        wait_ms=100.0)
        _C.cuda_synchronize()  # returns: the wait is bounded
        try:
            be.check_status()
            out["first"] = None
        except RuntimeError as exc:
            out["first"] = str(exc)
        try:
            group.barrier()
            out["second"] = None
        except RuntimeError as exc:
            out["second"] = str(exc)
    return out
