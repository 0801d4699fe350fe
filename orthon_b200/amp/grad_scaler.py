"""Dynamic loss scaling.

A scaler drives update cycles of one MixedPrecisionOptimizer:

    scaler.scale(loss).backward()      # gradients carry the factor `scale_factor`
    scaler.unscale_(opt)               # optional, idempotent within a cycle
    scaler.step(opt)                   # skip or apply; the schedule adapts HERE
    scaler.update()                    # closes the cycle

The verdict "some gradient was non-finite" belongs to the optimizer, not to the scaler: the
optimizer's `_unscale_and_check` returns the local verdict and its `_agree_on_overflow` makes it
the same on every rank.  With the peer-memory reducer that agreement is already part of the fused
reduction kernel (the found-inf word is exchanged with the gradients), so no extra collective is
issued; otherwise it is a one-element all-reduce.  A skipped step multiplies the scale by
`backoff_factor`; `growth_interval` applied steps in a row multiply it by `growth_factor`.
(reference project: python/orthon/amp/grad_scaler.py:31-138)"""
import math

# name -> (kind, admissible, state-dict default or None when the key is mandatory)
_FIELDS = {
    "scale": ("real", lambda x: x > 0.0, None),
    "growth_factor": ("real", lambda x: x > 1.0, None),
    "backoff_factor": ("real", lambda x: 0.0 < x < 1.0, None),
    "growth_interval": ("count", lambda n: n >= 1, None),
    "enabled": ("flag", None, None),
    "unscaled": ("flag", None, False),
    "found_inf": ("flag", None, False),
    "growth_tracker": ("count", lambda n: n >= 0, 0),
}


def _checked(name, value):
    kind, admissible, _ = _FIELDS[name]
    if kind == "flag":
        if type(value) is not bool:
            raise TypeError(f"GradScaler: {name} must be a bool")
        return value
    if type(value) is bool or not isinstance(value, (int,) if kind == "count" else (int, float)):
        raise TypeError(f"GradScaler: {name} must be " + ("an integer" if kind == "count" else "a real number"))
    if kind == "real":
        value = float(value)
        if not math.isfinite(value) or not admissible(value):
            raise ValueError(f"GradScaler: invalid {name}")
    elif not admissible(value):
        raise ValueError(f"GradScaler: {name} must be at least {1 if name == 'growth_interval' else 0}")
    return value


class _Schedule:
    """The adaptive part: current scale and the count of applied steps since the last change."""

    __slots__ = ("scale", "growth_factor", "backoff_factor", "growth_interval", "growth_tracker")

    def __init__(self, scale, growth_factor, backoff_factor, growth_interval, growth_tracker=0):
        self.scale, self.growth_factor, self.backoff_factor = scale, growth_factor, backoff_factor
        self.growth_interval, self.growth_tracker = growth_interval, growth_tracker
        if growth_tracker >= growth_interval:
            raise ValueError("GradScaler: growth_tracker must be below growth_interval")

    def record(self, overflowed):
        if overflowed:
            self.scale *= self.backoff_factor
            self.growth_tracker = 0
            return
        self.growth_tracker += 1
        if self.growth_tracker == self.growth_interval:
            self.scale *= self.growth_factor
            self.growth_tracker = 0


class GradScaler:
    def __init__(self, init_scale=1024.0, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000, enabled=True):
        self._schedule = _Schedule(_checked("scale", init_scale), _checked("growth_factor", growth_factor),
                                   _checked("backoff_factor", backoff_factor), _checked("growth_interval", growth_interval))
        self._enabled = _checked("enabled", enabled)
        self._open_cycle(None, unscaled=False, overflow=False)

    # ------------------------------------------------------------------ cycle
    def _open_cycle(self, owner, unscaled, overflow):
        self._owner, self._unscaled, self._overflow = owner, unscaled, overflow

    def _admit(self, optimizer):
        """A cycle belongs to the first optimizer that was unscaled in it.  A restored state
        that says "unscaled" without an owner can only be closed by update()."""
        if self._owner is None:
            if self._unscaled:
                raise RuntimeError("GradScaler restored an unscaled cycle; call update() first")
        elif self._owner is not optimizer:
            raise RuntimeError("GradScaler controls one optimizer per update cycle")

    @property
    def scale_factor(self):
        return self._schedule.scale

    @property
    def enabled(self):
        return self._enabled

    @property
    def found_inf(self):
        return self._overflow

    # -------------------------------------------------------------------- API
    def scale(self, loss):
        if not self._enabled:
            return loss
        return loss * self._schedule.scale

    def unscale_(self, mp_optimizer):
        if not self._enabled:
            return
        self._admit(mp_optimizer)
        if not self._unscaled:
            verdict = mp_optimizer._unscale_and_check(1.0 / self._schedule.scale)
            self._open_cycle(mp_optimizer, unscaled=True, overflow=bool(verdict))  # bound only after success

    def step(self, mp_optimizer):
        if not self._enabled:
            return mp_optimizer.step()
        self.unscale_(mp_optimizer)
        agree = getattr(mp_optimizer, "_agree_on_overflow", None)
        self._overflow = bool(agree(self._overflow)) if agree is not None else self._overflow
        if not self._overflow:
            mp_optimizer._step_prepared()
        self._schedule.record(self._overflow)
        self._unscaled = False
        return None

    def update(self):
        self._open_cycle(None, unscaled=False, overflow=False)

    # ------------------------------------------------------------------ state
    def state_dict(self):
        s = self._schedule
        return {"version": 1, "scale": s.scale, "growth_factor": s.growth_factor, "backoff_factor": s.backoff_factor,
                "growth_interval": s.growth_interval, "enabled": self._enabled, "unscaled": self._unscaled,
                "found_inf": self._overflow, "growth_tracker": s.growth_tracker}

    def load_state_dict(self, state):
        if type(state.get("version")) is not int or state["version"] != 1:
            raise RuntimeError("GradScaler: unsupported state version")
        seen = {}
        for name, (_, _, default) in _FIELDS.items():
            seen[name] = _checked(name, state[name] if default is None else state.get(name, default))
        schedule = _Schedule(seen["scale"], seen["growth_factor"], seen["backoff_factor"], seen["growth_interval"],
                             seen["growth_tracker"])  # validated as a whole before anything is replaced
        self._schedule, self._enabled = schedule, seen["enabled"]
        self._open_cycle(None, unscaled=seen["unscaled"], overflow=seen["found_inf"])


__all__ = ["GradScaler"]
