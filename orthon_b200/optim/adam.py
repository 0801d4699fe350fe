"""Adam with bias correction by a global step count, epsilon outside the square root and
decoupled weight decay (skipping 1-D parameters unless ``decay_bias``).  Moments are created
lazily in pairs.  The whole per-parameter update is one fused kernel:

    m += (b1-1) m + (1-b1) g ;  v += (b2-1) v + (1-b2) g² ;
    p += -lr*wd*p ;  p += -(lr/bc1) * m / (sqrt(v/bc2) + eps)

(reference project: python/orthon/optim/adam.py:90-266)"""
import os

from .. import _C
from .._state import PreparedLoad, commit_prepared
from ._binding import Binding, capture_bindings, no_grad


class _Moments:
    __slots__ = ("m", "v")

    def __init__(self, m, v):
        self.m, self.v = m, v


def _check_profile(p, device=None):
    device = p.device if device is None else device
    if p.dtype not in ("float32", "float64") or (device.is_cuda() and p.dtype != "float32"):
        raise RuntimeError("bare Adam supports CPU float32/float64 and CUDA float32")


def _as_device(location):
    if location is None or isinstance(location, _C.Device):
        return location
    if not isinstance(location, str):
        raise TypeError("Adam map_location must be a device string or Device")
    try:
        return _C.Device(location)
    except (RuntimeError, ValueError) as exc:
        raise ValueError(f"invalid Adam map_location: {location!r}") from exc


def _adopt(moments, p, device=None):
    if tuple(moments.m.shape) != tuple(p.shape) or tuple(moments.v.shape) != tuple(p.shape):
        raise ValueError("Adam moment shape does not match bound parameter")
    out = []
    for t in (moments.m, moments.v):
        c = t.to(p.device if device is None else device)
        if c.dtype != p.dtype:
            c = _C.cast(c, p.dtype)
        out.append(c)
    return _Moments(*out)


class Adam:
    def __init__(self, params, lr=0.001, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, decay_bias=False):
        self._bindings = capture_bindings(params)
        self._lr = lr
        self._beta1, self._beta2 = betas
        self._eps, self._weight_decay, self._decay_bias = eps, weight_decay, decay_bias
        self._t = 0

    def get_lr(self):
        return self._lr

    def set_lr(self, lr):
        self._lr = lr

    def _should_decay(self, p):
        return self._weight_decay != 0.0 and p.requires_grad and (self._decay_bias or len(p.shape) > 1)

    def zero_grad(self):
        for b in self._bindings:
            if b.parameter.grad is not None:
                b.parameter.zero_grad()

    def step(self):
        self._step_impl(None)

    def _step_with_model_copies(self, models):
        """AMP bridge: `models[i]` (or None) is the low-precision copy of parameter i, refreshed
        by the same kernel that updates the float32 master."""
        self._step_impl(list(models))

    def _step_impl(self, models):
        debug = os.environ.get("ORTHON_DEBUG_ADAM") == "1"
        with no_grad():
            self._t += 1  # advances even when no parameter has a gradient
            bc1 = 1.0 - self._beta1 ** self._t
            bc2 = 1.0 - self._beta2 ** self._t
            for i, b in enumerate(self._bindings):
                p = b.parameter
                g = p.grad
                if g is None:
                    continue
                _check_profile(p)
                st = b.state
                if st is None:
                    st = _Moments(_C._zeros_on(list(p.shape), p.dtype, str(p.device)),
                                  _C._zeros_on(list(p.shape), p.dtype, str(p.device)))
                    b.state = st
                elif any(tuple(t.shape) != tuple(p.shape) or t.dtype != p.dtype or t.device != p.device for t in (st.m, st.v)):
                    st = _adopt(st, p)
                    b.state = st
                wd = self._weight_decay if self._should_decay(p) else 0.0
                target = p if p.is_contiguous else p.contiguous()
                model = None if models is None else models[i]
                fused_model = model if (model is not None and model.is_contiguous and target is p) else None
                _C._adam_step_(target, st.m, st.v, g.contiguous(), fused_model, float(self._lr), float(self._beta1),
                               float(self._beta2), float(self._eps), float(wd), bc1, bc2, 1.0)
                if target is not p:
                    p._copy_data_(target)
                if model is not None and fused_model is None:
                    _C._amp_copy_master_to_model_(model, p)
                if debug:
                    import sys
                    print(f"[adam] param {i} shape={tuple(p.shape)} t={self._t}", file=sys.stderr)

    def state_dict(self):
        return {
            "lr": self._lr, "betas": (self._beta1, self._beta2), "eps": self._eps,
            "weight_decay": self._weight_decay, "decay_bias": self._decay_bias, "t": self._t,
            "m": [None if b.state is None else b.state.m for b in self._bindings],
            "v": [None if b.state is None else b.state.v for b in self._bindings],
        }

    def load_state_dict(self, state, map_location=None):
        commit_prepared([self._prepare_load_state_dict(state, map_location)])

    def _prepare_load_state_dict(self, state, map_location=None, placement=None):
        lr, (b1, b2), eps, t = state["lr"], state["betas"], state["eps"], state["t"]
        wd, db = state.get("weight_decay", 0.0), state.get("decay_bias", False)
        ms, vs = list(state["m"]), list(state["v"])
        target = _as_device(map_location)
        devices = tuple(placement(b.parameter) if placement else b.parameter.device for b in self._bindings)
        if len(ms) != len(self._bindings) or len(vs) != len(self._bindings):
            raise ValueError("Adam optimizer state parameter count mismatch")
        for b, m, v, dev in zip(self._bindings, ms, vs, devices):
            p = b.parameter
            if target is not None and target != dev:
                raise ValueError("Adam map_location conflicts with bound parameter device")
            if (m is None) != (v is None):
                raise ValueError("Adam moments must be initialized together")
            if m is None:
                continue
            if not isinstance(m, _C.Tensor) or not isinstance(v, _C.Tensor):
                raise TypeError("Adam moments must be Tensor values or both None")
            if tuple(m.shape) != tuple(p.shape) or tuple(v.shape) != tuple(p.shape):
                raise ValueError("Adam moment shape does not match bound parameter")
            _check_profile(p, dev)
        with no_grad():
            fresh = tuple(Binding(b.parameter, None if m is None else _adopt(_Moments(m, v), b.parameter, dev))
                          for b, m, v, dev in zip(self._bindings, ms, vs, devices))
        before = (self._lr, self._beta1, self._beta2, self._eps, self._weight_decay, self._decay_bias, self._t, self._bindings)

        def commit():
            (self._lr, self._beta1, self._beta2, self._eps, self._weight_decay, self._decay_bias, self._t,
             self._bindings) = (lr, b1, b2, eps, wd, db, t, fresh)

        def rollback():
            (self._lr, self._beta1, self._beta2, self._eps, self._weight_decay, self._decay_bias, self._t,
             self._bindings) = before

        return PreparedLoad(commit, rollback)

    def _rebind_parameters(self, params):
        fresh = capture_bindings(params)
        if len(fresh) != len(self._bindings):
            raise ValueError("Adam rebind parameter count mismatch")
        for old, new in zip(self._bindings, fresh):
            if tuple(old.parameter.shape) != tuple(new.parameter.shape):
                raise ValueError("Adam rebind parameter shape mismatch")
            if old.state is not None:
                _check_profile(new.parameter)
        with no_grad():
            self._bindings = tuple(Binding(n.parameter, None if o.state is None else _adopt(o.state, n.parameter))
                                   for o, n in zip(self._bindings, fresh))
