"""Module, optimizer and AMP contracts.
(reference project: tests/spec/nn/*, tests/spec/optim/*, tests/spec/amp/*)"""
import numpy as np
import pytest
import torch

import orthon_b200 as ob
from orthon_b200 import _C, nn


def t(a, dtype=None):
    return ob.from_numpy(np.asarray(a, dtype=np.float32), dtype)


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(4, 8)
        self.act = nn.ReLU()
        self.fc2 = nn.Linear(8, 3)
        self.register_buffer("steps", ob.cast(ob.zeros([1]), "int64"))
        self.register_buffer("scratch", ob.zeros([2]), persistent=False)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


def test_registration_rules_and_traversal():
    m = Net()
    names = [n for n, _ in m.named_parameters()]
    assert names == ["fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"]
    assert list(m.state_dict()) == ["steps", "fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"]
    assert [n for n, _ in m.named_buffers()] == ["steps", "scratch"]
    with pytest.raises(KeyError):
        m.register_buffer("fc1", ob.zeros([1]))
    with pytest.raises(KeyError):
        m.steps = nn.Linear(1, 1)  # buffer slots keep their role
    with pytest.raises(ValueError):
        m.register_buffer("a.b", ob.zeros([1]))
    m.tied = nn.Parameter(m.fc1.weight)  # tie
    assert len(list(m.parameters())) == 4 and len(list(m.named_parameters())) == 5
    m.eval()
    assert not m.fc1.training
    m.train()
    assert m.act.training


def test_parameter_identity_survives_transforms():
    m = Net()
    w = m.fc1.weight
    (m(t(np.ones((2, 4)))).sum()).backward()
    assert w.grad is not None
    m.cast("float64")
    assert m.fc1.weight is w and w.dtype == "float64" and w.grad is None and w.requires_grad
    assert m.steps.dtype == "int64"  # integer buffers keep their dtype
    m.float()
    assert w.dtype == "float32"


def test_load_state_dict_is_atomic():
    a, b = Net(), Net()
    state = dict(b.state_dict())
    a.load_state_dict(state)
    assert a.fc2.weight.tolist() == b.fc2.weight.tolist()
    before = a.fc1.weight.tolist()
    bad = dict(state)
    bad["fc1.weight"] = ob.from_numpy(np.full((4, 8), 5.0, dtype=np.float32))
    bad["fc2.weight"] = ob.zeros([1, 1])  # wrong shape, later in the walk
    with pytest.raises(ValueError, match="size mismatch"):
        a.load_state_dict(bad)
    assert a.fc1.weight.tolist() == before
    with pytest.raises(KeyError, match="Missing keys"):
        a.load_state_dict({"fc1.weight": state["fc1.weight"]})


def test_layers_forward_shapes_and_modes():
    x = t(np.random.default_rng(0).standard_normal((2, 3, 8, 8)))
    y = nn.Sequential(nn.Conv2d(3, 4, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2), nn.Flatten(), nn.Linear(64, 5))(x)
    assert y.shape == (2, 5)
    d = nn.Dropout(0.5, seed=3)
    a = d(t(np.ones(1000)))
    assert 300 < sum(1 for v in a.tolist() if v == 0.0) < 700 and max(a.tolist()) == 2.0
    d.eval()
    assert d(t(np.ones(4))).tolist() == [1, 1, 1, 1]
    blk = nn.TransformerEncoderBlock(16, 4)
    z = blk(t(np.random.default_rng(1).standard_normal((2, 5, 16))), is_causal=True)
    assert z.shape == (2, 5, 16)
    emb = nn.Embedding(10, 4, padding_idx=0)
    assert emb([[1, 0]]).shape == (1, 2, 4) and emb.weight.tolist()[:4] == [0.0] * 4


def test_dropout_mask_is_splitmix64_stream():
    p, seed, n = 0.25, 12345, 64
    mask = _C.dropout(t(np.ones(n)), p, seed).tolist()

    def splitmix(x):
        x = (x + 0x9E3779B97F4A7C15) & (2 ** 64 - 1)
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & (2 ** 64 - 1)
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & (2 ** 64 - 1)
        return x ^ (x >> 31)

    expect = [(1.0 / (1.0 - p)) if (splitmix(seed + i) >> 40) / 16777216.0 >= p else 0.0 for i in range(n)]
    assert np.allclose(mask, expect)


def test_batchnorm_matches_torch():
    rng = np.random.default_rng(2)
    X = rng.standard_normal((6, 3, 4, 4))
    bn, tbn = nn.BatchNorm2d(3), torch.nn.BatchNorm2d(3)
    y = bn(t(X))
    ty = tbn(torch.tensor(X, dtype=torch.float32))
    assert np.allclose(y.numpy(), ty.detach().numpy(), atol=1e-4)
    assert np.allclose(bn.running_var.numpy(), tbn.running_var.numpy(), atol=1e-5)
    bn.eval(), tbn.eval()
    assert np.allclose(bn(t(X)).numpy(), tbn(torch.tensor(X, dtype=torch.float32)).detach().numpy(), atol=1e-4)


@pytest.mark.parametrize("wd", [0.0, 0.1])
def test_adam_matches_formula_and_torch(wd):
    rng = np.random.default_rng(3)
    W0, G = rng.standard_normal((3, 4)), [rng.standard_normal((3, 4)) for _ in range(4)]
    w = t(W0)
    w.requires_grad_(True)
    opt = ob.optim.Adam([w], lr=1e-2, weight_decay=wd)
    tw = torch.tensor(W0, dtype=torch.float32, requires_grad=True)
    topt = torch.optim.AdamW([tw], lr=1e-2, weight_decay=wd, eps=1e-8)
    for g in G:
        w.set_grad(t(g))
        opt.step()
        tw.grad = torch.tensor(g, dtype=torch.float32)
        topt.step()
    assert np.allclose(w.numpy(), tw.detach().numpy(), atol=2e-5)
    st = opt.state_dict()
    assert st["t"] == 4 and st["m"][0].shape == (3, 4)
    opt2 = ob.optim.Adam([w], lr=1.0)
    opt2.load_state_dict(st)
    assert opt2.get_lr() == 1e-2 and opt2._t == 4
    with pytest.raises(ValueError):
        ob.optim.Adam([w, w])
    b = t(np.ones(4))
    b.requires_grad_(True)
    o3 = ob.optim.Adam([b], lr=0.1, weight_decay=0.5)
    assert not o3._should_decay(b)  # 1-D parameters skip decay


def test_sgd_and_global_step_without_grads():
    w = t([1.0, 2.0])
    w.requires_grad_(True)
    w.set_grad(t([0.5, 0.5]))
    ob.optim.SGD([w], lr=0.1).step()
    assert np.allclose(w.tolist(), [0.95, 1.95])
    a = ob.optim.Adam([t([1.0]).requires_grad_(True)])
    a.step()
    assert a._t == 1


def test_grad_scaler_schedule():
    s = ob.amp.GradScaler(init_scale=8.0, growth_interval=2)

    class Fake:
        def __init__(self):
            self.inf, self.steps = False, 0

        def _unscale_and_check(self, inv):
            return self.inf

        def _step_prepared(self):
            self.steps += 1

        def _amp_collective_device(self):
            return None

    o = Fake()
    for _ in range(2):
        s.step(o)
        s.update()
    assert s.scale_factor == 16.0 and o.steps == 2
    o.inf = True
    s.step(o)
    assert s.found_inf and s.scale_factor == 8.0 and o.steps == 2
    s.update()
    st = s.state_dict()
    s2 = ob.amp.GradScaler()
    s2.load_state_dict(st)
    assert s2.scale_factor == 8.0
    with pytest.raises(RuntimeError):
        s.unscale_(o)
        s.step(Fake())


def test_mixed_precision_optimizer_cpu():
    ob.manual_seed(0)
    m = nn.Sequential(nn.Linear(4, 4), nn.ReLU(), nn.Linear(4, 2))
    opt = ob.amp.MixedPrecisionOptimizer(m, ob.optim.Adam, lr=1e-2)
    scaler = ob.amp.GradScaler(init_scale=128.0)
    x, y = t(np.ones((3, 4))), [0, 1, 0]
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = ob.cross_entropy(m(x), y)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    st = opt.state_dict()
    assert st["version"] == 1 and st["orig_dtypes"] == ["float32"] * 4
    # an injected inf skips the step and backs the scale off
    opt.zero_grad()
    loss = ob.cross_entropy(m(x), y)
    scaler.scale(loss).backward()
    with ob.no_grad():
        next(iter(m.parameters())).grad.fill_(float("inf"))
    before = next(iter(m.parameters())).tolist()
    scaler.step(opt)
    assert scaler.found_inf and scaler.scale_factor == 64.0 and next(iter(m.parameters())).tolist() == before


def test_fused_mlp_matches_composed_linears():
    """_mlp_gelu (one node, GELU gradient inside the input-gradient GEMM) against two linears."""
    import numpy as np
    from orthon_b200 import _C
    rng = np.random.default_rng(3)
    x_np = rng.standard_normal((5, 7, 12)).astype(np.float32)
    w1_np, b1_np = rng.standard_normal((12, 20)).astype(np.float32) * 0.3, rng.standard_normal(20).astype(np.float32)
    w2_np, b2_np = rng.standard_normal((20, 12)).astype(np.float32) * 0.3, rng.standard_normal(12).astype(np.float32)

    def run(fused):
        ts = [_C.from_numpy(a) for a in (x_np, w1_np, b1_np, w2_np, b2_np)]
        for t in ts:
            t.requires_grad_(True)
        x, w1, b1, w2, b2 = ts
        if fused:
            y = _C._mlp_gelu(x, w1, b1, w2, b2, x)
        else:
            y = _C.linear(_C.linear(x, w1, b1, "gelu"), w2, b2, "none", x)
        (y * y).sum().backward()
        return [np.asarray(y.tolist())] + [np.asarray(t.grad.tolist()) for t in ts]

    for a, b in zip(run(True), run(False)):
        assert np.allclose(a, b, rtol=1e-5, atol=1e-5)


def test_functional_reductions_and_max_returns_values():
    import numpy as np
    import orthon_b200.functional as F
    from orthon_b200 import _C
    x = _C.from_numpy(np.asarray([[1.0, 5.0, 2.0], [7.0, 0.0, 3.0]], dtype=np.float32))
    assert F.sum(x).item() == 18.0 and np.allclose(F.mean(x, 1).tolist(), [8.0 / 3, 10.0 / 3], rtol=1e-6)
    m = F.max(x, 1)
    assert isinstance(m, _C.Tensor) and m.tolist() == [5.0, 7.0]  # values only; indices come from argmax
    assert F.argmax(x, 1).tolist() == [1, 0] and F.max(x).item() == 7.0
    assert np.allclose(F.exp(x).tolist(), np.exp([1, 5, 2, 7, 0, 3]), rtol=1e-6)


def test_diagnostics_pool_switches():
    from orthon_b200 import _diagnostics as diag
    assert diag.memory_pool_enabled() in (True, False)
    before = diag.memory_pool_max_cached_bytes()
    diag.memory_pool_set_max_cached_bytes(1 << 20)
    assert diag.memory_pool_max_cached_bytes() == 1 << 20
    diag.memory_pool_set_max_cached_bytes(before)
    stats = diag.memory_pool_stats()
    assert {"current_bytes", "peak_bytes", "cached_bytes"} <= set(stats)
    assert isinstance(diag.dispatch_kernels(), (list, tuple, dict))


def test_conv2d_backward_entry_point_matches_autograd_and_skips_the_input_gradient_on_request():
    """`_C._conv2d_backward` is the formula the autograd node runs; benchmarks call it directly."""
    import numpy as np
    import torch
    from orthon_b200 import _C
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 3, 7, 6)).astype(np.float32)
    w = rng.standard_normal((4, 3, 3, 3)).astype(np.float32)
    g = rng.standard_normal((2, 4, 4, 3)).astype(np.float32)   # stride 2, padding 1
    dx, dw, db = _C._conv2d_backward(_C.from_numpy(g), _C.from_numpy(x), _C.from_numpy(w), True, 2, 2, 1, 1, True)
    tx, tw = torch.tensor(x, requires_grad=True), torch.tensor(w, requires_grad=True)
    tb = torch.zeros(4, requires_grad=True)
    torch.nn.functional.conv2d(tx, tw, tb, stride=2, padding=1).backward(torch.tensor(g))
    assert np.allclose(dx.numpy(), tx.grad.numpy(), atol=1e-4)
    assert np.allclose(dw.numpy(), tw.grad.numpy(), atol=1e-4)
    assert np.allclose(db.numpy(), tb.grad.numpy(), atol=1e-4)
    none_dx, dw2, no_bias = _C._conv2d_backward(_C.from_numpy(g), _C.from_numpy(x), _C.from_numpy(w), False, 2, 2, 1, 1, False)
    assert none_dx is None and no_bias is None
    assert np.allclose(dw2.numpy(), dw.numpy())
