"""Plain SGD with optional decoupled weight decay; one fused kernel per parameter.
(reference project: python/orthon/optim/sgd.py:7-83)"""
from .. import _C
from .._state import PreparedLoad, commit_prepared
from ._binding import capture_bindings, no_grad


class SGD:
    def __init__(self, params, lr: float, weight_decay=0.0, decay_bias=False):
        self._bindings = capture_bindings(params)
        self._lr, self._weight_decay, self._decay_bias = lr, weight_decay, decay_bias

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
        """AMP bridge: refreshes the low-precision copies in the update kernel."""
        self._step_impl(list(models))

    def _step_impl(self, models):
        with no_grad():
            for i, b in enumerate(self._bindings):
                p = b.parameter
                model = None if models is None else models[i]
                g = p.grad
                if g is None:
                    continue
                wd = self._weight_decay if self._should_decay(p) else 0.0
                if p.is_contiguous and g.is_contiguous and p.dtype in ("float32", "float64") and not (
                        p.device.is_cuda() and p.dtype != "float32"):
                    fused_model = model if (model is not None and model.is_contiguous) else None
                    _C._sgd_step_(p, g, fused_model, float(self._lr), float(wd), 1.0)
                    if model is not None and fused_model is None:
                        _C._amp_copy_master_to_model_(model, p)
                else:
                    if wd:
                        p.add_(p, alpha=-self._lr * wd)
                    p.add_(g, alpha=-self._lr)
                    if model is not None:
                        _C._amp_copy_master_to_model_(model, p)

    def state_dict(self):
        return {"lr": self._lr, "weight_decay": self._weight_decay, "decay_bias": self._decay_bias}

    def load_state_dict(self, state, map_location=None):
        commit_prepared([self._prepare_load_state_dict(state, map_location)])

    def _prepare_load_state_dict(self, state, map_location=None, placement=None):
        lr = state["lr"]
        wd, db = state.get("weight_decay", 0.0), state.get("decay_bias", False)
        if placement is not None and map_location is not None:
            for b in self._bindings:
                if map_location != placement(b.parameter):
                    raise ValueError("SGD map_location conflicts with bound parameter device")
        before = (self._lr, self._weight_decay, self._decay_bias)

        def commit():
            self._lr, self._weight_decay, self._decay_bias = lr, wd, db

        def rollback():
            self._lr, self._weight_decay, self._decay_bias = before

        return PreparedLoad(commit, rollback)

    def _rebind_parameters(self, params):
        fresh = capture_bindings(params)
        if len(fresh) != len(self._bindings):
            raise ValueError("SGD rebind parameter count mismatch")
        if any(tuple(o.parameter.shape) != tuple(n.parameter.shape) for o, n in zip(self._bindings, fresh)):
            raise ValueError("SGD rebind parameter shape mismatch")
        self._bindings = fresh
