"""Optimizer and mixed-precision contracts: the update formulas against closed-form NumPy over
a grid of hyper-parameters, decay rules, lazy state, atomic state loads, master ownership, the
GradScaler schedule and its state validation.
(reference project: tests/spec/optim/*, tests/spec/amp/*, tests/python/test_adam_parity.py,
test_grad_scaler.py)"""
import itertools

import numpy as np
import pytest

import orthon_b200 as ob
from orthon_b200 import nn


def T(a, dtype=None, grad=True):
    x = ob.from_numpy(np.asarray(a, dtype=np.float32), dtype)
    if grad:
        x.requires_grad_(True)
    return x


def G(a, dtype=None):
    return T(a, dtype, grad=False)


# ------------------------------------------------------------------------ Adam
def adam_reference(p, grads, lr, b1, b2, eps, wd, decay):
    p = p.astype(np.float64).copy()
    m, v = np.zeros_like(p), np.zeros_like(p)
    for t, g in enumerate(grads, start=1):
        g = g.astype(np.float64)
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        mhat, vhat = m / (1 - b1 ** t), v / (1 - b2 ** t)
        if decay:
            p = p - lr * wd * p
        p = p - lr * mhat / (np.sqrt(vhat) + eps)           # eps outside the square root
    return p


@pytest.mark.parametrize("lr,betas,eps,wd", list(itertools.product([1e-3, 0.1], [(0.9, 0.999), (0.5, 0.9), (0.0, 0.5)], [1e-8, 1e-2], [0.0, 0.1])))
def test_adam_matches_the_closed_form(lr, betas, eps, wd):
    rng = np.random.default_rng(int(lr * 1e4) + int(betas[0] * 10) + int(wd * 10))
    w0, b0 = rng.standard_normal((3, 2)).astype(np.float32), rng.standard_normal(2).astype(np.float32)
    w, b = T(w0), T(b0)
    opt = ob.optim.Adam([w, b], lr=lr, betas=betas, eps=eps, weight_decay=wd)
    gw = [rng.standard_normal((3, 2)).astype(np.float32) for _ in range(4)]
    gb = [rng.standard_normal(2).astype(np.float32) for _ in range(4)]
    for a, c in zip(gw, gb):
        w.set_grad(G(a))
        b.set_grad(G(c))
        opt.step()
    assert np.allclose(np.asarray(w.tolist()).reshape(3, 2), adam_reference(w0, gw, lr, *betas, eps, wd, True), rtol=2e-5, atol=1e-6)
    assert np.allclose(np.asarray(b.tolist()), adam_reference(b0, gb, lr, *betas, eps, wd, False), rtol=2e-5, atol=1e-6)   # 1-D: no decay


def test_adam_decay_bias_extends_decay_to_one_dimensional_parameters():
    b0 = np.array([1.0, -2.0], dtype=np.float32)
    b = T(b0)
    opt = ob.optim.Adam([b], lr=0.1, weight_decay=0.5, decay_bias=True)
    g = [np.ones(2, dtype=np.float32)] * 2
    for x in g:
        b.set_grad(G(x))
        opt.step()
    assert np.allclose(b.tolist(), adam_reference(b0, g, 0.1, 0.9, 0.999, 1e-8, 0.5, True), rtol=1e-5)


def test_adam_time_advances_without_gradients_and_moments_stay_lazy():
    a, b = T([1.0, 2.0]), T([3.0])
    opt = ob.optim.Adam([a, b], lr=0.1)
    opt.step()
    opt.step()
    state = opt.state_dict()
    assert state["t"] == 2 and state["m"] == [None, None] and state["v"] == [None, None]
    a.set_grad(G([1.0, 1.0]))
    opt.step()
    state = opt.state_dict()
    assert state["t"] == 3 and state["m"][0] is not None and state["v"][0] is not None and state["m"][1] is None
    # bias correction uses the global step count (3), not the count of steps that had a gradient
    m = 0.1
    v = 0.001
    want = 1.0 - 0.1 * (m / (1 - 0.9 ** 3)) / (np.sqrt(v / (1 - 0.999 ** 3)) + 1e-8)
    assert np.allclose(a.tolist(), [want, want + 1.0], rtol=1e-5)
    assert b.tolist() == [3.0]


@pytest.mark.parametrize("cls", [ob.optim.Adam, ob.optim.SGD])
def test_optimizers_capture_owners_once_and_keep_them_alive(cls):
    p = T([1.0])
    with pytest.raises(ValueError, match="duplicate"):
        cls([p, p], lr=0.1)
    with pytest.raises(TypeError):
        cls([p, 3.0], lr=0.1)
    opt = cls((q for q in [T([1.0]), T([2.0])]), lr=0.1)          # a generator is consumed once, owners are retained
    assert len(opt._bindings) == 2
    import gc
    gc.collect()
    assert [b.parameter.tolist() for b in opt._bindings] == [[1.0], [2.0]]


@pytest.mark.parametrize("cls", [ob.optim.Adam, ob.optim.SGD])
def test_zero_grad_set_lr_and_get_lr(cls):
    p = T([1.0])
    opt = cls([p], lr=0.5)
    p.set_grad(G([1.0]))
    opt.zero_grad()
    assert p.grad is None
    opt.set_lr(0.25)
    assert opt.get_lr() == 0.25


# ------------------------------------------------------------------------- SGD
@pytest.mark.parametrize("lr,wd,decay_bias", list(itertools.product([0.1, 1.0], [0.0, 0.5], [False, True])))
def test_sgd_matches_the_closed_form(lr, wd, decay_bias):
    w0, b0 = np.array([[1.0, -2.0], [0.5, 4.0]], dtype=np.float32), np.array([1.0, 2.0], dtype=np.float32)
    w, b = T(w0), T(b0)
    opt = ob.optim.SGD([w, b], lr=lr, weight_decay=wd, decay_bias=decay_bias)
    gw, gb = np.full((2, 2), 0.5, dtype=np.float32), np.array([1.0, -1.0], dtype=np.float32)
    for _ in range(3):
        w.set_grad(G(gw))
        b.set_grad(G(gb))
        opt.step()
    ew, eb = w0.astype(np.float64), b0.astype(np.float64)
    for _ in range(3):
        ew = ew - lr * wd * ew - lr * gw
        eb = (eb - lr * wd * eb if decay_bias else eb) - lr * gb
    assert np.allclose(np.asarray(w.tolist()).reshape(2, 2), ew, rtol=1e-5, atol=1e-6)
    assert np.allclose(b.tolist(), eb, rtol=1e-5, atol=1e-6)


def test_sgd_skips_parameters_without_gradients():
    a, b = T([1.0]), T([2.0])
    opt = ob.optim.SGD([a, b], lr=0.5, weight_decay=0.5)
    a.set_grad(G([2.0]))
    opt.step()
    assert b.tolist() == [2.0] and a.tolist() != [1.0]


@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_optimizers_work_in_the_parameter_dtype(dtype):
    for cls in (ob.optim.SGD, ob.optim.Adam):
        p = ob.cast(G([1.0, 2.0]), dtype)
        p.requires_grad_(True)
        opt = cls([p], lr=0.1)
        p.set_grad(ob.cast(G([1.0, 1.0]), dtype))
        opt.step()
        assert p.dtype == dtype and p.tolist()[0] < 1.0


# ---------------------------------------------------------------- state loads
def _trained_adam():
    p, q = T([[1.0, 2.0]]), T([3.0])
    opt = ob.optim.Adam([p, q], lr=0.05, betas=(0.8, 0.9), eps=1e-6, weight_decay=0.01)
    p.set_grad(G([[1.0, -1.0]]))
    opt.step()
    return opt, (p, q)


def test_adam_state_dict_layout():
    opt, _ = _trained_adam()
    s = opt.state_dict()
    assert set(s) >= {"lr", "betas", "eps", "weight_decay", "t", "m", "v"}
    assert s["t"] == 1 and tuple(s["betas"]) == (0.8, 0.9) and s["lr"] == 0.05
    assert s["m"][1] is None and s["v"][1] is None and s["m"][0].shape == (1, 2)


def test_adam_state_round_trip_continues_identically():
    opt, (p, q) = _trained_adam()
    p2, q2 = T(np.asarray(p.tolist()).reshape(1, 2)), T(q.tolist())
    opt2 = ob.optim.Adam([p2, q2], lr=9.9)
    opt2.load_state_dict(opt.state_dict())
    for o, (a, b) in ((opt, (p, q)), (opt2, (p2, q2))):
        a.set_grad(G([[0.5, 0.5]]))
        b.set_grad(G([1.0]))
        o.step()
    assert p.tolist() == p2.tolist() and q.tolist() == q2.tolist()
    assert opt2.state_dict()["m"][0]._buffer_id != opt.state_dict()["m"][0]._buffer_id      # loaded state is a copy


@pytest.mark.parametrize("mutate,error", [
    (lambda s: s["m"].pop(), ValueError),
    (lambda s: s["m"].__setitem__(0, None), ValueError),                    # m without v
    (lambda s: s["m"].__setitem__(0, ob.from_numpy(np.zeros((2, 2), dtype=np.float32))), ValueError),
    (lambda s: s["v"].__setitem__(0, "text"), TypeError),
    (lambda s: s["v"].__setitem__(0, None), ValueError),                    # v without m
    (lambda s: s["m"].append(None), ValueError),
])
def test_adam_state_loads_are_atomic(mutate, error):
    source, _ = _trained_adam()
    state = dict(source.state_dict())
    state["m"], state["v"] = list(state["m"]), list(state["v"])
    mutate(state)
    target, (p, q) = _trained_adam()
    before = (target.get_lr(), target._t, target.state_dict()["m"][0].tolist())
    with pytest.raises(error):
        target.load_state_dict(state)
    assert (target.get_lr(), target._t, target.state_dict()["m"][0].tolist()) == before


def test_sgd_state_round_trip():
    p = T([1.0])
    a = ob.optim.SGD([p], lr=0.3, weight_decay=0.1, decay_bias=True)
    b = ob.optim.SGD([T([1.0])], lr=7.0)
    b.load_state_dict(a.state_dict())
    assert b.get_lr() == 0.3 and b.state_dict() == a.state_dict()


# ------------------------------------------------------------------------- AMP
def _amp_model(dtype):
    ob.manual_seed(4)
    m = nn.Sequential(nn.Linear(3, 4), nn.Tanh(), nn.Linear(4, 2))
    if dtype != "float32":
        m.cast(dtype)
    return m


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
def test_masters_are_float32_and_float32_owners_are_their_own_masters(dtype):
    m = _amp_model(dtype)
    opt = ob.amp.MixedPrecisionOptimizer(m, ob.optim.SGD, lr=0.1)
    state = opt.state_dict()
    assert state["version"] == 1 and state["orig_dtypes"] == [dtype] * 4
    for p, master in zip(m.parameters(), state["masters"]):
        assert master.dtype == "float32" and master.shape == p.shape
        assert (master is p) == (dtype == "float32")
        if dtype != "float32":
            assert master._buffer_id != p._buffer_id and not master.grad and master.is_leaf


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_a_step_updates_masters_in_float32_and_refreshes_the_model_copy(dtype):
    m = _amp_model(dtype)
    opt = ob.amp.MixedPrecisionOptimizer(m, ob.optim.SGD, lr=2 ** -10)
    p = next(iter(m.parameters()))
    master = opt.state_dict()["masters"][0]
    before = np.asarray(master.tolist())
    g = np.ones(p.shape, dtype=np.float32)
    for _ in range(3):
        opt.zero_grad()
        p.set_grad(ob.cast(G(g), dtype))
        opt.step()
    after = np.asarray(opt.state_dict()["masters"][0].tolist())
    assert np.allclose(after, before - 3 * 2 ** -10, atol=1e-7)            # three tiny updates accumulate in the master
    rounded = ob.cast(ob.cast(opt.state_dict()["masters"][0], dtype), "float32").tolist()
    assert ob.cast(p, "float32").tolist() == rounded                          # the model holds the rounded master


def test_amp_rejects_unsupported_owners_and_ddp_with_automatic_sync():
    with pytest.raises(ValueError):
        ob.amp.MixedPrecisionOptimizer(nn.Sequential(nn.Linear(2, 2)).cast("float64"), ob.optim.SGD, lr=0.1)

    class FakeDdp:
        def parameters(self):
            return iter([])

        def _validate_master_gradient_sync(self):
            raise ValueError("MixedPrecisionOptimizer requires DDP(sync_grads=False)")

    with pytest.raises(ValueError, match="sync_grads=False"):
        ob.amp.MixedPrecisionOptimizer(FakeDdp(), ob.optim.SGD, lr=0.1)
    with pytest.raises(ValueError, match="fused"):
        ob.amp.MixedPrecisionOptimizer(_amp_model("float32"), ob.optim.SGD, fused="sometimes", lr=0.1)


def test_module_transforms_are_reconciled_lazily():
    m = _amp_model("float32")
    opt = ob.amp.MixedPrecisionOptimizer(m, ob.optim.SGD, lr=0.5)
    owners = [id(p) for p in m.parameters()]
    m.half()
    assert [id(p) for p in m.parameters()] == owners
    p = next(iter(m.parameters()))
    p.set_grad(ob.cast(G(np.ones(p.shape)), "float16"))
    opt.step()
    state = opt.state_dict()
    assert state["orig_dtypes"] == ["float16"] * 4 and state["masters"][0].dtype == "float32"
    m.float()
    opt.step()
    state = opt.state_dict()
    assert state["orig_dtypes"] == ["float32"] * 4 and state["masters"][0] is p                # promoted: the owner is its master again


def test_amp_state_round_trip_and_validation():
    m = _amp_model("bfloat16")
    opt = ob.amp.MixedPrecisionOptimizer(m, ob.optim.Adam, lr=0.01)
    for p in m.parameters():
        p.set_grad(ob.cast(G(np.ones(p.shape)), "bfloat16"))
    opt.step()
    state = opt.state_dict()
    m2 = _amp_model("bfloat16")
    opt2 = ob.amp.MixedPrecisionOptimizer(m2, ob.optim.Adam, lr=9.0)
    opt2.load_state_dict(state)
    assert [a.tolist() for a in opt2.state_dict()["masters"]] == [a.tolist() for a in state["masters"]]
    assert [p.tolist() for p in m2.parameters()] == [p.tolist() for p in m.parameters()]
    assert opt2.get_lr() == 0.01
    for bad, error in ((dict(state, version=2), RuntimeError), (dict(state, orig_dtypes=["float32"] * 4), ValueError),
                       (dict(state, masters=state["masters"][:2]), ValueError), (dict(state, masters=["x"] * 4), TypeError)):
        before = [p.tolist() for p in m2.parameters()]
        with pytest.raises(error):
            opt2.load_state_dict(bad)
        assert [p.tolist() for p in m2.parameters()] == before


# ------------------------------------------------------------------ GradScaler
class CountingOptimizer:
    """Stands in for a MixedPrecisionOptimizer: reports a scripted overflow verdict."""

    def __init__(self, verdicts):
        self.verdicts, self.unscaled_with, self.steps, self.plain_steps = list(verdicts), [], 0, 0

    def _unscale_and_check(self, inv_scale):
        self.unscaled_with.append(inv_scale)
        return self.verdicts.pop(0)

    def _step_prepared(self):
        self.steps += 1

    def step(self):
        self.plain_steps += 1


@pytest.mark.parametrize("verdicts,scales,steps", [
    ([False, False, False, False], [8.0, 16.0, 16.0, 32.0], 4),            # grows every second clean step
    ([True, False, False, True], [4.0, 4.0, 8.0, 4.0], 2),
    ([False, True, False, False], [8.0, 4.0, 4.0, 8.0], 3),                # an overflow resets the growth count
    ([True, True, True, True], [4.0, 2.0, 1.0, 0.5], 0),
])
def test_scale_schedule(verdicts, scales, steps):
    scaler = ob.amp.GradScaler(init_scale=8.0, growth_interval=2)
    opt = CountingOptimizer(verdicts)
    seen = []
    for _ in range(4):
        scaler.step(opt)
        seen.append(scaler.scale_factor)
        scaler.update()
    assert seen == scales and opt.steps == steps


def test_unscale_is_idempotent_within_a_cycle_and_binds_one_optimizer():
    scaler = ob.amp.GradScaler(init_scale=4.0)
    a, b = CountingOptimizer([False, False]), CountingOptimizer([False])
    scaler.unscale_(a)
    scaler.unscale_(a)
    assert a.unscaled_with == [0.25]
    with pytest.raises(RuntimeError, match="one optimizer per update cycle"):
        scaler.unscale_(b)
    with pytest.raises(RuntimeError, match="one optimizer per update cycle"):
        scaler.step(b)
    scaler.step(a)
    assert a.steps == 1 and a.unscaled_with == [0.25]
    scaler.update()
    scaler.step(b)
    assert b.steps == 1


def test_found_inf_is_visible_until_update():
    scaler = ob.amp.GradScaler(init_scale=4.0)
    scaler.step(CountingOptimizer([True]))
    assert scaler.found_inf and scaler.scale_factor == 2.0
    scaler.update()
    assert not scaler.found_inf


def test_a_disabled_scaler_is_transparent():
    scaler = ob.amp.GradScaler(enabled=False)
    opt = CountingOptimizer([])
    loss = G([2.0])
    assert scaler.scale(loss) is loss
    scaler.unscale_(opt)
    scaler.step(opt)
    scaler.update()
    assert opt.plain_steps == 1 and opt.steps == 0 and opt.unscaled_with == [] and not scaler.enabled


def test_scale_multiplies_the_loss_and_the_gradient_carries_the_factor():
    x = T([1.0, 2.0])
    scaler = ob.amp.GradScaler(init_scale=16.0)
    scaler.scale((x * x).sum()).backward()
    assert x.grad.tolist() == [32.0, 64.0]


@pytest.mark.parametrize("kwargs", [dict(init_scale=0.0), dict(init_scale=-1.0), dict(init_scale=float("inf")), dict(init_scale="big"),
                                     dict(init_scale=True), dict(growth_factor=1.0), dict(growth_factor=0.5), dict(backoff_factor=1.0),
                                     dict(backoff_factor=0.0), dict(growth_interval=0), dict(growth_interval=2.5), dict(growth_interval=True),
                                     dict(enabled=1), dict(enabled=None)])
def test_scaler_rejects_bad_arguments(kwargs):
    with pytest.raises((ValueError, TypeError)):
        ob.amp.GradScaler(**kwargs)


def test_scaler_state_round_trip():
    scaler = ob.amp.GradScaler(init_scale=8.0, growth_factor=3.0, backoff_factor=0.25, growth_interval=5)
    scaler.step(CountingOptimizer([False]))
    state = scaler.state_dict()
    assert state == {"version": 1, "scale": 8.0, "growth_factor": 3.0, "backoff_factor": 0.25, "growth_interval": 5, "enabled": True,
                     "unscaled": False, "found_inf": False, "growth_tracker": 1}
    other = ob.amp.GradScaler()
    other.load_state_dict(state)
    assert other.state_dict() == state


@pytest.mark.parametrize("patch,error", [
    (dict(version=2), RuntimeError), (dict(version="1"), RuntimeError), (dict(scale=0.0), ValueError), (dict(scale="x"), TypeError),
    (dict(growth_factor=1.0), ValueError), (dict(backoff_factor=1.5), ValueError), (dict(growth_interval=0), ValueError),
    (dict(growth_tracker=5), ValueError), (dict(growth_tracker=-1), ValueError), (dict(enabled="yes"), TypeError),
    (dict(found_inf=1), TypeError), (dict(unscaled=None), TypeError),
])
def test_scaler_state_is_validated_as_a_whole(patch, error):
    scaler = ob.amp.GradScaler(init_scale=8.0, growth_interval=5)
    good = scaler.state_dict()
    with pytest.raises(error):
        scaler.load_state_dict(dict(good, **patch))
    assert scaler.state_dict() == good


def test_a_restored_unscaled_cycle_must_be_closed_first():
    scaler = ob.amp.GradScaler()
    scaler.load_state_dict(dict(scaler.state_dict(), unscaled=True, found_inf=True))
    with pytest.raises(RuntimeError, match="call update"):
        scaler.step(CountingOptimizer([False]))
    scaler.update()
    scaler.step(CountingOptimizer([False]))


def test_real_overflow_skips_the_step_and_halves_the_scale():
    """float16 compute does not exist on the CPU backend, so the gradients are set by hand: one
    of them carries an infinity, as a float16 backward pass that overflowed would leave it."""
    m = _amp_model("float16")
    opt = ob.amp.MixedPrecisionOptimizer(m, ob.optim.SGD, lr=0.1)
    scaler = ob.amp.GradScaler(init_scale=2.0 ** 20)
    before = [p.tolist() for p in m.parameters()]
    for i, p in enumerate(m.parameters()):
        g = np.ones(p.shape, dtype=np.float32)
        if i == 2:
            g.reshape(-1)[0] = np.inf
        p.set_grad(ob.cast(G(g), "float16"))
    scaler.step(opt)
    assert scaler.found_inf and scaler.scale_factor == 2.0 ** 19
    assert [p.tolist() for p in m.parameters()] == before
    scaler.update()
    opt.zero_grad()
    for p in m.parameters():
        p.set_grad(ob.cast(G(np.full(p.shape, 2.0 ** 19)), "float16") if False else ob.cast(G(np.full(p.shape, 1024.0)), "float16"))
    scaler.step(opt)                                       # finite: applied, unscaled by 2^-19
    assert not scaler.found_inf
    first = next(iter(m.parameters()))
    assert first.tolist() != before[0]
