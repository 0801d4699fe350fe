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
    from orthon_b200.distributed import _state
    be = _state.get_active().backend
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
