"""Mixed-precision optimizer wrapper: float16/bfloat16 model owners are optimised through
detached float32 masters; float32 owners are their own masters.

Each step transfers gradients to the masters as float32 (unscaling and checking them for
inf/NaN with a single device flag read for the whole model), optionally averages the master
gradients across ranks, runs the inner optimizer and refreshes the low-precision model copies.
With the built-in Adam/SGD the master update and the model refresh are one fused kernel per
parameter.  Module transforms (`to`, `cast`, `half`, ...) are reconciled lazily because the
Python owners keep their identity.
(reference project: python/orthon/amp/optimizer.py:48-284)"""
from .. import _C
from .._state import PreparedLoad, commit_prepared

_LOW = {"float16", "bfloat16"}
_OK = _LOW | {"float32"}


def _no_grad():
    import orthon_b200 as ob
    return ob.no_grad()


class _State:
    __slots__ = ("parameter", "model_dtype", "master", "model_device")

    def __init__(self, parameter, model_dtype, master, model_device):
        self.parameter, self.model_dtype, self.master, self.model_device = parameter, model_dtype, master, model_device


def _check_param(p):
    if not isinstance(p, _C.Tensor):
        raise TypeError("AMP model parameters must be Tensor owners")
    if p.dtype not in _OK:
        raise ValueError("AMP model parameters must be float32/float16/bfloat16")


def _new_master(value, device):
    with _no_grad():
        m = value.to(device)  # always an independent copy
        if m.dtype != "float32":
            m = _C.cast(m, "float32")
    m.requires_grad_(True)
    return m


def _check_sync(p, master):
    if tuple(p.shape) != tuple(master.shape) or p.device != master.device:
        raise ValueError("AMP master shape/device must match model owner")
    if master.dtype != "float32" or p.dtype not in _OK:
        raise ValueError("AMP synchronization requires an FP32 master")
    if not p.is_contiguous or not master.is_contiguous:
        raise RuntimeError("AMP synchronization requires contiguous tensors")


class MixedPrecisionOptimizer:
    def __init__(self, model, optimizer_cls, fused="auto", bucket_size_mb=None, **optimizer_kwargs):
        """`fused` selects how the step is scheduled when the gradients can live in flat buckets
        (one CUDA device, one dtype; across ranks: the peer-memory transport):

        * "reduce" / "auto": gradients accumulate locally over any number of backward passes;
          `step()` averages every bucket with one fused kernel and applies one fused update per
          bucket.  Works with a GradScaler.
        * "overlap": each bucket is averaged from the autograd hooks while backward is still
          running; `step()` applies the update.  Works with a GradScaler.  Exactly one backward
          per `zero_grad()`: a second one raises.
        * "update": the optimizer update itself runs inside the reduction kernel during backward
          (no GradScaler: there is no point at which a step could be skipped).  One backward per
          `zero_grad()`, as above.
        * False keeps the per-parameter path.

        `bucket_size_mb` sizes the flat buckets when the optimizer builds them itself (a plain
        module on one GPU; a DistributedDataParallel wrapper brings its own)."""
        if fused not in ("auto", "reduce", "overlap", "update", False):
            raise ValueError("fused must be 'auto', 'reduce', 'overlap', 'update' or False")
        check = getattr(model, "_validate_master_gradient_sync", None)
        if check is not None:
            check()
        from ..distributed import group as dstate
        self._group = dstate.active() if dstate.is_active() else None
        self._ddp = model if hasattr(model, "_reducer") else None
        self._peer = None
        self._pending_inv_scale = None
        params = tuple(model.parameters())
        for p in params:
            _check_param(p)
        self._bucket_size_mb = bucket_size_mb
        if fused is not False and self._try_init_fused(model, params, optimizer_cls, fused, optimizer_kwargs):
            return
        self._states = tuple(_State(p, p.dtype, p if p.dtype == "float32" else _new_master(p, p.device), p.device)
                             for p in params)
        self._factory, self._kwargs = optimizer_cls, dict(optimizer_kwargs)
        self._inner = optimizer_cls((s.master for s in self._states), **optimizer_kwargs)

    # ------------------------------------------------------------ fused path
    def _try_init_fused(self, model, params, optimizer_cls, fused, kwargs):
        from ..optim import SGD, Adam
        from ..optim.adam import _Moments
        from ..parallel.peer_reducer import PeerReducer
        from ..parallel.peer_reducer import LocalFlatReducer
        if optimizer_cls not in (Adam, SGD) or not params:
            return False
        reducer = getattr(model, "_reducer", None)
        if reducer is None and not hasattr(model, "_reducer"):
            # Plain module on one GPU: flat local buckets, same fused update schedule.
            named = [(n, p) for n, p in sorted(model.named_parameters(), key=lambda e: e[0])] if hasattr(model, "named_parameters") \
                else [(str(i), p) for i, p in enumerate(params)]
            seen, owners = set(), []
            for n, p in named:
                if id(p) not in seen:
                    seen.add(id(p))
                    owners.append((n, p))
            if any(not p.requires_grad for _, p in owners) or not LocalFlatReducer.eligible(owners):
                return False
            reducer = LocalFlatReducer(owners, self._bucket_size_mb)
            for _, p in owners:
                p._register_post_accumulate_grad_hook(lambda r=reducer, k=id(p): r.mark(k))
        if not isinstance(reducer, PeerReducer):
            return False
        if {id(p) for p in params} != {id(p) for _, p in reducer.parameters}:
            return False  # frozen parameters: keep the general path
        low = params[0].dtype in _LOW
        masters = dict(zip((id(p) for _, p in reducer.parameters), reducer.flatten_state(want_masters=low)))
        self._states = tuple(_State(p, p.dtype, masters[id(p)] if low else p, p.device) for p in params)
        self._factory, self._kwargs = optimizer_cls, dict(kwargs)
        self._inner = optimizer_cls((s.master for s in self._states), **kwargs)
        self._kind = "adam" if optimizer_cls is Adam else "sgd"
        if self._kind == "adam":
            moments = dict(zip((id(p) for _, p in reducer.parameters), reducer.flat_moments()))
            for s, b in zip(self._states, self._inner._bindings):
                b.state = _Moments(*moments[id(s.parameter)])
        by_master = {id(s.parameter): s.master for s in self._states}
        reducer.set_decay_segments(lambda p: self._inner._weight_decay if self._inner._should_decay(by_master[id(p)]) else 0.0)
        self._peer = reducer
        if fused in ("overlap", "update"):
            reducer.overlap = True          # launch from the hooks, during backward
            reducer.single_backward = True  # nothing synchronises at the end of backward: guard the cycle
        if fused == "update":
            reducer.mode = self._kind
            reducer.hyper = self._fused_hyper
            reducer.on_first_launch = self._begin_fused_step
        return True

    def _begin_fused_step(self):
        if self._kind == "adam":
            self._inner._t += 1

    def _fused_hyper(self, grad_scale=1.0):
        o = self._inner
        h = {"lr": float(o._lr), "weight_decay": 0.0, "grad_scale": float(grad_scale)}
        if self._kind == "adam":
            h.update(beta1=float(o._beta1), beta2=float(o._beta2), eps=float(o._eps),
                     bias_c1=1.0 - o._beta1 ** o._t, bias_c2=1.0 - o._beta2 ** o._t)
        return h

    def _fused_step(self, grad_scale=1.0):
        peer = self._peer
        peer.synchronize()
        if peer.mode == "average":
            self._begin_fused_step()
            peer.local_update(self._kind, self._fused_hyper(grad_scale))

    # -------------------------------------------------------- reconciliation
    def _prepare_states(self):
        fresh, copies, changed = [], [], False
        for s in self._states:
            p, master = s.parameter, s.master
            _check_param(p)
            if tuple(p.shape) != tuple(master.shape):
                raise ValueError("AMP transformed parameter shape differs from master")
            if p.dtype == "float32":
                if s.model_dtype in _LOW:  # model was promoted: carry the master values over
                    if master.device != p.device:
                        master = _new_master(master, p.device)
                    _check_sync(p, master)
                    copies.append((p, master))
                master = p
            elif s.model_dtype == "float32":
                master = _new_master(p, p.device)
            elif master.device != p.device:
                master = _new_master(master, p.device)
            if p.dtype in _LOW:
                _check_sync(p, master)
            if master is not s.master or p.dtype != s.model_dtype or p.device != s.model_device:
                changed = True
            fresh.append(_State(p, p.dtype, master, p.device))
        return tuple(fresh), copies, changed

    def _publish(self, states, copies, changed):
        if changed:
            self._inner._rebind_parameters(s.master for s in states)
            with _no_grad():
                for p, master in copies:
                    _C._amp_copy_master_to_model_(p, master)
            self._states = states

    def _reconcile(self):
        self._publish(*self._prepare_states())

    # ----------------------------------------------------------------- steps
    def zero_grad(self):
        if self._peer is not None:
            self._peer.reset()
        for s in self._states:
            s.parameter.zero_grad()
            if s.master is not s.parameter:
                s.master.zero_grad()

    def _transfer_gradients(self, inv_scale=None):
        states, copies, changed = self._prepare_states()
        grads = tuple(s.parameter.grad for s in states)
        for s, g in zip(states, grads):
            if g is None:
                continue
            if tuple(g.shape) != tuple(s.parameter.shape) or g.device != s.parameter.device:
                raise ValueError("AMP gradient shape/device must match model owner")
            if g.dtype not in _OK:
                raise ValueError("AMP gradients must be float32/float16/bfloat16")
        out, found_inf, flag = [], False, None
        with _no_grad():
            for s, g in zip(states, grads):
                if g is not None:
                    if inv_scale is not None and g.device.is_cuda():
                        if flag is None:
                            flag = _C._zeros_on([1], "int32", str(g.device))
                        g = _C._amp_unscale_into(g, float(inv_scale), flag)  # no host sync per tensor
                    else:
                        if g.dtype != "float32":
                            g = _C.cast(g, "float32")
                        elif s.model_dtype == "float32":
                            g = g.to(g.device)
                        if inv_scale is not None:
                            g = g * inv_scale
                            found_inf |= not _C.isfinite_all(g)
                    if g.requires_grad or not g.is_leaf:
                        g = g.to(g.device)
                out.append(g)
            if flag is not None:
                found_inf |= bool(flag.tolist()[0])
        self._publish(states, copies, changed)
        for s, g in zip(self._states, out):
            if g is None:
                s.master.zero_grad()
            else:
                s.master.set_grad(g)
        return found_inf

    def _unscale_and_check(self, inv_scale):
        if self._peer is not None:
            if self._peer.mode != "average":
                raise RuntimeError("GradScaler needs MixedPrecisionOptimizer(fused='reduce') or fused='overlap': "
                                   "an update that runs inside backward cannot be skipped")
            self._peer.synchronize()
            self._pending_inv_scale = float(inv_scale)
            return self._peer.found_inf()  # scaled, averaged gradients: same verdict on every rank
        return self._transfer_gradients(inv_scale)

    def step(self):
        if self._peer is not None:
            self._fused_step()
            return
        self._transfer_gradients()
        self._step_prepared()

    def sync_to_model(self):
        if self._peer is not None:
            with _no_grad():
                for b in self._peer.buckets:
                    if b.master_flat is not b.param_flat:
                        _C._amp_copy_master_to_model_(b.param_flat, b.master_flat)
            return
        self._reconcile()
        with _no_grad():
            for s in self._states:
                if s.master is not s.parameter:
                    _C._amp_copy_master_to_model_(s.parameter, s.master)

    def _agree_on_overflow(self, local):
        """The overflow verdict of this cycle, identical on every rank.  The peer-memory reducer
        exchanges the found-inf word inside its reduction kernel, so its verdict already is;
        otherwise the ranks add up a one-element flag."""
        from ..distributed import group as dstate
        if self._group is not None:
            self._group.ensure_open()
        group = self._group if self._group is not None else (dstate.active() if dstate.is_active() else None)
        if group is None or group.world_size == 1 or self._peer is not None or not self._states:
            return bool(local)
        flag = _C._full_on([1], 1.0 if local else 0.0, "float32", str(self._states[0].master.device))
        group.all_reduce(flag, op="sum")
        return float(flag.tolist()[0]) > 0.0

    def _all_reduce_master_grads(self):
        from ..distributed import group as dstate
        from ..parallel.reducer import reduce_master_gradients
        if self._group is None and dstate.is_active():
            self._group = dstate.active()
        if self._group is None:
            return
        self._group.ensure_open()
        if self._group.world_size > 1:
            reduce_master_gradients(tuple(s.master for s in self._states), self._group)

    def _step_prepared(self):
        if self._peer is not None:
            scale, self._pending_inv_scale = (self._pending_inv_scale or 1.0), None
            self._begin_fused_step()
            self._peer.local_update(self._kind, self._fused_hyper(scale))
            return
        self._all_reduce_master_grads()
        fused = getattr(self._inner, "_step_with_model_copies", None)
        if fused is not None:
            fused([None if s.master is s.parameter else s.parameter for s in self._states])
        else:
            self._inner.step()
            self.sync_to_model()

    def get_lr(self):
        return self._inner.get_lr()

    def set_lr(self, lr):
        self._inner.set_lr(lr)

    # ----------------------------------------------------------------- state
    def state_dict(self):
        if self._peer is None:
            self._reconcile()
        return {"version": 1, "orig_dtypes": [s.model_dtype for s in self._states],
                "masters": [s.master for s in self._states], "inner": self._inner.state_dict()}

    def load_state_dict(self, state, map_location=None):
        commit_prepared([self._prepare_load_state_dict(state, map_location)])

    def _prepare_load_state_dict(self, state, map_location=None, placement=None):
        if type(state.get("version")) is not int or state["version"] != 1:
            raise RuntimeError("MixedPrecisionOptimizer: unsupported state version")
        dtypes, masters, inner_state = list(state["orig_dtypes"]), list(state["masters"]), state["inner"]
        if len(dtypes) != len(self._states) or len(masters) != len(self._states):
            raise ValueError("MixedPrecisionOptimizer state parameter count mismatch")
        target = _C.Device(map_location) if isinstance(map_location, str) else map_location
        if target is not None and not isinstance(target, _C.Device):
            raise TypeError("AMP map_location must be a device string or Device")
        devices = tuple(placement(s.parameter) if placement else s.parameter.device for s in self._states)
        for cur, dt, master, dev in zip(self._states, dtypes, masters, devices):
            p = cur.parameter
            _check_param(p)
            if dt != p.dtype:
                raise ValueError("MixedPrecisionOptimizer dtype mismatch")
            if not isinstance(master, _C.Tensor):
                raise TypeError("AMP saved masters must be Tensor values")
            if tuple(master.shape) != tuple(p.shape):
                raise ValueError("MixedPrecisionOptimizer master shape mismatch")
            if target is not None and target != dev:
                raise ValueError("AMP map_location conflicts with bound model device")
            if p.dtype in _LOW and not p.is_contiguous and dev == p.device:
                raise RuntimeError("AMP synchronization requires contiguous tensors")
        fresh = tuple(_State(s.parameter, dt, s.parameter if dt == "float32" else _new_master(master, dev), dev)
                      for s, dt, master, dev in zip(self._states, dtypes, masters, devices))
        temp = self._factory((s.master for s in fresh), **self._kwargs)
        where = {id(s.master): dev for s, dev in zip(fresh, devices)}
        prep = getattr(temp, "_prepare_load_state_dict", None)
        if prep is not None:
            prep(inner_state, map_location=target, placement=lambda p: where[id(p)]).commit()
        else:
            temp.load_state_dict(inner_state, map_location=target)
        copies, old_values = [], []
        with _no_grad():
            for s in fresh:
                if s.master is s.parameter:
                    continue
                p = s.parameter if s.parameter.device == s.model_device else s.parameter.to(s.model_device)
                _check_sync(p, s.master)
                copies.append((s.parameter, s.master))
                old_values.append(_new_master(s.parameter, s.parameter.device))
        before = (self._states, self._inner)
        done = []

        def commit():
            with _no_grad():
                for i, (p, master) in enumerate(copies):
                    done.append(i)
                    _C._amp_copy_master_to_model_(p, master)
            self._states, self._inner = fresh, temp

        def rollback():
            self._states, self._inner = before
            with _no_grad():
                for i in reversed(done):
                    p, _ = copies[i]
                    v = old_values[i]
                    if v.device != p.device:
                        v = v.to(p.device)
                    _C._amp_copy_master_to_model_(p, v)
                done.clear()

        return PreparedLoad(commit, rollback)
