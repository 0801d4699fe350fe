"""Worker functions of the DDP runtime contract tests (local backend, CPU ranks).  Every
function returns plain Python values so the parent can compare ranks with each other and with a
closed-form expectation."""
import numpy as np


def T(values, dtype="float32"):
    import orthon_b200 as ob
    return ob.from_numpy(np.asarray(values, dtype=np.float32), dtype)


def show(t):
    return None if t is None else (t.dtype, tuple(t.shape), [round(float(v), 6) for v in t.tolist()])


def _three(dtype="float32"):
    """Parameters a, b and an `unused` one; forward(active, factor) -> nested container whose
    first leaf is a scalar loss = factor * sum(coef * p) over the active parameters."""
    import orthon_b200 as ob
    from orthon_b200 import nn

    class Three(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Parameter(T([1.0, 2.0, 3.0, 4.0], dtype))
            self.b = nn.Parameter(T([1.0, 2.0], dtype))
            self.unused = nn.Parameter(T([5.0], dtype))
            self.register_buffer("rank_buffer", T([0.0]))
            self.last_output = None

        def forward(self, active, factor):
            terms = []
            if active in ("a", "all"):
                terms.append((self.a * T([1.0, 2.0, 3.0, 5.0], dtype)).sum())
            if active in ("b", "all"):
                terms.append((self.b * T([2.0, -1.0], dtype)).sum())
            if not terms:  # a graph that reaches no parameter
                free = T([0.0], dtype)
                free.requires_grad_(True)
                terms.append((free * 1.0).sum())
            total = terms[0]
            for extra in terms[1:]:
                total = total + extra
            self.last_output = {"nested": [(total * factor, "tag")], "aux": 3}
            return self.last_output

    return Three()


def _ddp(model, options):
    import orthon_b200.distributed as dist
    return dist.DDP(model, sync_grads=not options.get("manual", False), bucket_size_mb=options.get("bucket"),
                    overlap_grad_sync=options.get("overlap", False))


def training_modes(rank, options):
    """Four backward passes with rank-divergent participation; records every parameter's gradient
    after each pass, checks that a second synchronisation changes nothing."""
    import orthon_b200.distributed as dist
    model = _three()
    ddp = _ddp(model, options)
    out = []
    for it in range(4):
        active = ("a" if rank == 0 else "b") if it < 2 else ("a" if it == 2 else "none")
        result = ddp(active, 2.0 + 4.0 * rank)
        assert result is model.last_output
        result["nested"][0][0].backward(retain_graph=(it == 0))
        if options.get("manual"):
            ddp.all_reduce_gradients()
        before = [show(p.grad) for p in model.parameters()]
        ddp.wait_for_gradient_sync()
        ddp.all_reduce_gradients()     # nothing new since the last synchronisation: a no-op
        assert [show(p.grad) for p in model.parameters()] == before
        out.append(before)
    return out, ddp._reducer.diagnostics(), type(ddp._reducer).__name__


def rejected_profile(rank, kind):
    """Rank 0 holds a gradient the reducer cannot average; every rank must raise after exactly one
    control collective and no data collective, and the group stays usable."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    from orthon_b200 import nn
    from orthon_b200.distributed import group as G
    dtype = {"low-precision": "float16", "backend-dtype": "float64"}[kind]
    calls = []
    backend = G.active().backend
    real_all_reduce = backend.all_reduce

    def counting(tensor, op="sum", async_op=False):
        calls.append(tuple(tensor.shape))
        return real_all_reduce(tensor, op=op, async_op=async_op)

    backend.all_reduce = counting
    if kind == "backend-dtype":
        def only_float32(dt):
            if dt != "float32":
                raise RuntimeError("this transport averages float32 gradients only")
        backend._validate_gradient_dtype = only_float32
    model = nn.Module()
    model.weight = nn.Parameter(ob.cast(T([1.0, 2.0]), dtype))
    ddp = dist.DDP(model, sync_grads=False, bucket_size_mb=1.0)
    if rank == 0:
        model.weight.set_grad(ob.cast(T([3.0, 4.0]), dtype))
    before = show(model.weight.grad)
    calls.clear()
    try:
        ddp.all_reduce_gradients()
        message = None
    except RuntimeError as exc:
        message = str(exc)
    after = show(model.weight.grad)
    diag = ddp._reducer.diagnostics()
    value = T([rank + 1.0, 2.0])
    dist.all_reduce(value)
    return {"message": message, "unchanged": before == after, "control_shapes": calls[:-1], "diag": diag, "sum": value.tolist()}


def descriptor_mismatch(rank, kind):
    import orthon_b200.distributed as dist
    value = T([rank + 1.0, 3.0], "float64" if (kind == "dtype" and rank) else "float32")
    if kind == "shape" and rank:
        value = T([rank + 1.0])
    before = show(value)
    try:
        if kind == "collective" and rank:
            dist.broadcast(value)
        elif kind == "barrier" and rank:
            dist.barrier()
        elif kind == "source":
            dist.broadcast(value, src=rank)
        else:
            dist.all_reduce(value)
        first = None
    except RuntimeError as exc:
        first = str(exc)
    try:
        dist.barrier()
        second = None
    except RuntimeError as exc:
        second = str(exc)
    return {"first": first, "second": second, "unchanged": show(value) == before}


def preflight_rejections(rank):
    """Calls that must be refused before they enter the collective sequence: the group stays in
    step and the next valid collective works."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    value = T([rank + 1.0, 2.0])
    refused = []
    for name, call in (("op", lambda: dist.all_reduce(value, op="mean")),
                       ("src", lambda: dist.broadcast(value, src=dist.get_world_size())),
                       ("negative src", lambda: dist.broadcast(value, src=-1)),
                       ("strided", lambda: dist.all_reduce(T([[1.0, 2.0], [3.0, 4.0]]).transpose(0, 1))),
                       ("bfloat16", lambda: dist.all_reduce(ob.cast(T([1.0]), "bfloat16"))),
                       ("bool reduction", lambda: dist.all_reduce(ob.cast(T([1.0]), "bool")))):
        try:
            call()
        except (RuntimeError, NotImplementedError, ValueError):
            refused.append(name)
    dist.all_reduce(value)
    flag = ob.cast(T([float(rank)]), "bool")
    dist.broadcast(flag, src=1)
    return refused, value.tolist(), flag.tolist()


def failing_worker(rank):
    import orthon_b200.distributed as dist
    if rank == dist.get_world_size() - 1:
        raise ValueError("worker failure injected by the test")
    dist.barrier()
    raise AssertionError("a collective returned although a rank had failed")


def absent_rank(rank):
    """Rank 1 never joins the collective.  Rank 0, on a transport with a 0.4 s budget, gets a
    timeout (not a hang), and the failure is sticky."""
    import time
    from orthon_b200.distributed import group as G
    from orthon_b200.distributed.local_backend import LocalBackend
    store = G.active().backend._store
    if rank == 1:
        time.sleep(1.0)   # stays away from the collective; leaves between steps
        return "absent"
    handle = G.GroupHandle(LocalBackend(0, 2, store, timeout=0.4))
    started = time.monotonic()
    try:
        handle.all_reduce(T([1.0]))
        first = None
    except RuntimeError as exc:
        first = str(exc)
    waited = time.monotonic() - started
    try:
        handle.barrier()
        second = None
    except RuntimeError as exc:
        second = str(exc)
    return {"first": first, "second": second, "waited": waited}


def zero_grad_with_outstanding_work(rank):
    """An asynchronous bucket that has not been waited for makes zero_grad() refuse."""
    import orthon_b200.distributed as dist
    from orthon_b200.distributed import group as G
    model = _three()
    ddp = dist.DDP(model, sync_grads=False, bucket_size_mb=1.0, overlap_grad_sync=False)
    ddp._reducer.overlap = True   # explicit synchronisation with asynchronous launches
    model.a.set_grad(T([1.0, 1.0, 1.0, 1.0]))
    model.b.set_grad(T([1.0, 1.0]))
    # Hold back the completion: the reducer sees a Work that is not finished yet.
    backend = G.active().backend
    real = backend.all_reduce
    held = []

    def lazy(tensor, op="sum", async_op=False):
        if not async_op or tuple(tensor.shape) == (3, 3):
            return real(tensor, op=op, async_op=async_op)
        real(tensor, op=op, async_op=False)
        work = G.Work(wait=lambda: True, probe=lambda: False)
        held.append(work)
        return work

    backend.all_reduce = lazy
    reducer = ddp._reducer
    original_wait = reducer.wait
    reducer.wait = lambda: None          # synchronize() returns with the bucket still outstanding
    ddp.all_reduce_gradients()
    reducer.wait = original_wait
    outstanding = reducer.diagnostics()["outstanding"]
    try:
        ddp.zero_grad()
        refused = None
    except RuntimeError as exc:
        refused = str(exc)
    ddp.wait_for_gradient_sync()
    ddp.zero_grad()
    return {"outstanding": outstanding, "refused": refused, "after": reducer.diagnostics()["outstanding"],
            "grads_cleared": all(p.grad is None for p in model.parameters())}


def reinitialise(rank):
    """destroy_process_group() then a second group on the same store: old handles stay dead, the
    new group works, sequence numbers start over."""
    import orthon_b200.distributed as dist
    from orthon_b200.distributed import group as G
    old = G.active()
    store = old.backend._store
    v = T([1.0, 1.0])
    dist.all_reduce(v)
    dist.destroy_process_group()
    dist.destroy_process_group()   # idempotent
    states = [dist.is_initialized()]
    try:
        old.all_reduce(v)
        stale = None
    except RuntimeError as exc:
        stale = str(exc)
    try:
        dist.get_rank()
        no_group = None
    except RuntimeError as exc:
        no_group = str(exc)
    backend = dist.init_process_group("local", rank=rank, world_size=2, store=store)
    states.append(dist.is_initialized())
    w = T([rank + 1.0])
    dist.all_reduce(w)
    return {"first": v.tolist(), "states": states, "stale": stale, "no_group": no_group, "second": w.tolist(),
            "returned_backend": type(backend).__name__, "rank": backend.rank}


def strided_gradient(rank, dtype):
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    from orthon_b200 import nn
    model = nn.Module()
    model.weight = nn.Parameter(ob.cast(T([[1.0, 2.0], [3.0, 4.0]]), dtype))
    ddp = dist.DDP(model, sync_grads=False, bucket_size_mb=1.0)
    g = ob.cast(T([[2.0 + 4.0 * rank, 4.0], [6.0, 8.0]]), dtype)
    if rank == 0:
        g = g.transpose(0, 1)       # logical value [[2, 6], [4, 8]], strided storage
    model.weight.set_grad(g)
    ddp.all_reduce_gradients()
    return show(model.weight.grad), bool(model.weight.grad.is_contiguous)


def owners_sharing_storage(rank):
    """Two parameters that are views of the same bytes are two owners with two gradients."""
    import orthon_b200.distributed as dist
    from orthon_b200 import nn
    model = nn.Module()
    base = T([1.0, 2.0])
    alias = base.reshape([2])        # a view taken before either becomes a parameter: its own autograd identity
    model.a = nn.Parameter(base)
    model.b = nn.Parameter(alias)
    assert model.a is not model.b
    ddp = dist.DDP(model, bucket_size_mb=0.000001, overlap_grad_sync=True)
    ((model.a * (2.0 + 4.0 * rank)).sum() + (model.b * (10.0 + 4.0 * rank)).sum()).backward()
    return len(list(ddp.parameters())), model.a.grad.tolist(), model.b.grad.tolist()


def unused_parameter_state(rank):
    """A parameter no rank uses never receives a gradient, its Adam moments are never created and
    weight decay does not touch it; buffers are not broadcast."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    model = _three()
    model.rank_buffer.fill_(float(rank))
    ddp = dist.DDP(model, bucket_size_mb=1.0, overlap_grad_sync=True)
    opt = ob.optim.Adam(ddp.parameters(), lr=0.1, weight_decay=0.2)
    for _ in range(3):
        opt.zero_grad()
        ddp("a", 2.0 + 4.0 * rank)["nested"][0][0].backward()
        opt.step()
    state = opt.state_dict()
    index = [id(p) for p in ddp.parameters()].index(id(model.unused))
    return {"unused": model.unused.tolist(), "grad": show(model.unused.grad), "m": show(state["m"][index]),
            "v": show(state["v"][index]), "buffer": model.rank_buffer.tolist(), "a": model.a.tolist()}


def manual_gradients(rank):
    """Gradients set by hand; repeated synchronisation without new gradients is a no-op; an
    in-place change makes the gradient new again."""
    import orthon_b200.distributed as dist
    model = _three()
    ddp = dist.DDP(model, sync_grads=False)
    model.a.set_grad(T([2.0 + 4.0 * rank] * 4))
    ddp.all_reduce_gradients()
    first = show(model.a.grad)
    ddp.all_reduce_gradients()
    ddp.wait_for_gradient_sync()
    ddp.wait_for_gradient_sync()
    same = show(model.a.grad) == first
    model.a.grad.mul_(2.0 + rank)   # rank 0: x2, rank 1: x3
    ddp.all_reduce_gradients()
    return first, same, show(model.a.grad), show(model.unused.grad)


def amp_rounds(rank, mode):
    """Three AMP rounds with hand-set gradients on different parameters per rank.  'enabled':
    rank 1 overflows in the second cycle; 'disabled' / 'direct': no scaling."""
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    from orthon_b200 import nn
    model = nn.Module()
    model.a = nn.Parameter(T([10.0]))
    model.b = nn.Parameter(T([20.0]))
    model.unused = nn.Parameter(T([30.0]))
    ddp = dist.DDP(model, sync_grads=False)
    opt = ob.amp.MixedPrecisionOptimizer(ddp, ob.optim.SGD, lr=0.25)
    scaler = ob.amp.GradScaler(enabled=(mode != "disabled"), init_scale=4.0)
    rounds = []
    for it in range(3):
        opt.zero_grad()
        scale = scaler.scale_factor if mode == "enabled" else 1.0
        if rank == 0:
            model.a.set_grad(T([4.0 * scale]))
        else:
            model.b.set_grad(T([8.0 * scale]))
        if it == 1 and mode == "enabled" and rank == 1:
            model.b.set_grad(T([float("inf")]))
        if mode == "direct":
            opt.step()
        else:
            scaler.step(opt)
            scaler.update()
        rounds.append({"params": [p.tolist()[0] for p in model.parameters()], "scale": scaler.scale_factor})
    return rounds
