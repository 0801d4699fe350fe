"""Dynamic loss scaling.  One optimizer per update cycle; the scale adapts inside ``step``:
a non-finite gradient anywhere (on any rank) skips the update and multiplies the scale by
``backoff_factor``; ``growth_interval`` consecutive finite steps multiply it by ``growth_factor``.
(reference project: python/orthon/amp/grad_scaler.py:31-138)"""


def _real(value, name, ok):
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise TypeError(f"GradScaler: {name} must be a real number")
    value = float(value)
    if value != value or value in (float("inf"), float("-inf")) or not ok(value):
        raise ValueError(f"GradScaler: invalid {name}")
    return value


def _integer(value, name, minimum=0):
    if isinstance(value, bool) or not isinstance(value, int):
        raise TypeError(f"GradScaler: {name} must be an integer")
    if value < minimum:
        raise ValueError(f"GradScaler: {name} must be at least {minimum}")
    return value


def _boolean(value, name):
    if not isinstance(value, bool):
        raise TypeError(f"GradScaler: {name} must be a bool")
    return value


class GradScaler:
    def __init__(self, init_scale=1024.0, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000, enabled=True):
        self._scale = _real(init_scale, "scale", lambda x: x > 0)
        self._growth_factor = _real(growth_factor, "growth_factor", lambda x: x > 1)
        self._backoff_factor = _real(backoff_factor, "backoff_factor", lambda x: 0 < x < 1)
        self._growth_interval = _integer(growth_interval, "growth_interval", 1)
        self._enabled = _boolean(enabled, "enabled")
        self._unscaled = False
        self._found_inf = False
        self._growth_tracker = 0
        self._cycle_optimizer = None

    scale_factor = property(lambda self: self._scale)
    enabled = property(lambda self: self._enabled)
    found_inf = property(lambda self: self._found_inf)

    def scale(self, loss):
        return loss * self._scale if self._enabled else loss

    def _check_cycle(self, optimizer):
        if self._cycle_optimizer is not None and self._cycle_optimizer is not optimizer:
            raise RuntimeError("GradScaler controls one optimizer per update cycle")
        if self._unscaled and self._cycle_optimizer is None:
            raise RuntimeError("GradScaler restored an unscaled cycle; call update() first")

    def unscale_(self, mp_optimizer):
        if not self._enabled:
            return
        self._check_cycle(mp_optimizer)
        if self._unscaled:
            return
        found = mp_optimizer._unscale_and_check(1.0 / self._scale)
        self._cycle_optimizer = mp_optimizer  # only a successful preparation binds the cycle
        self._found_inf = found
        self._unscaled = True

    def _agree_on_found_inf(self, mp_optimizer):
        from .. import distributed as dist
        from .. import _C
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return self._found_inf
        device = mp_optimizer._amp_collective_device()
        if device is None:
            return self._found_inf
        flag = _C._full_on([1], 1.0 if self._found_inf else 0.0, "float32", str(device))
        dist.all_reduce(flag, op="sum")
        return float(flag.tolist()[0]) > 0.0

    def step(self, mp_optimizer):
        if not self._enabled:
            mp_optimizer.step()
            return
        self._check_cycle(mp_optimizer)
        if not self._unscaled:
            self.unscale_(mp_optimizer)
        self._found_inf = self._agree_on_found_inf(mp_optimizer)
        if self._found_inf:
            self._scale *= self._backoff_factor
            self._growth_tracker = 0
        else:
            mp_optimizer._step_prepared()
            self._growth_tracker += 1
            if self._growth_tracker >= self._growth_interval:
                self._scale *= self._growth_factor
                self._growth_tracker = 0
        self._unscaled = False

    def update(self):
        self._unscaled = False
        self._found_inf = False
        self._cycle_optimizer = None

    def state_dict(self):
        return {"version": 1, "scale": self._scale, "growth_factor": self._growth_factor,
                "backoff_factor": self._backoff_factor, "growth_interval": self._growth_interval,
                "enabled": self._enabled, "unscaled": self._unscaled, "found_inf": self._found_inf,
                "growth_tracker": self._growth_tracker}

    def load_state_dict(self, state):
        if type(state.get("version")) is not int or state["version"] != 1:
            raise RuntimeError("GradScaler: unsupported state version")
        scale = _real(state["scale"], "scale", lambda x: x > 0)
        growth = _real(state["growth_factor"], "growth_factor", lambda x: x > 1)
        backoff = _real(state["backoff_factor"], "backoff_factor", lambda x: 0 < x < 1)
        interval = _integer(state["growth_interval"], "growth_interval", 1)
        enabled = _boolean(state["enabled"], "enabled")
        unscaled = _boolean(state.get("unscaled", False), "unscaled")
        found = _boolean(state.get("found_inf", False), "found_inf")
        tracker = _integer(state.get("growth_tracker", 0), "growth_tracker")
        if tracker >= interval:
            raise ValueError("GradScaler: growth_tracker must be below growth_interval")
        self._scale, self._growth_factor, self._backoff_factor = scale, growth, backoff
        self._growth_interval, self._enabled = interval, enabled
        self._unscaled, self._found_inf, self._growth_tracker = unscaled, found, tracker
        self._cycle_optimizer = None
