"""Autograd engine contracts and gradient checks against PyTorch.
(reference project: tests/spec/autograd/*, tests/cpp/test_autograd_engine.cpp)"""
import numpy as np
import pytest
import torch

import orthon_b200 as ob


def t(a, grad=True, dtype=None):
    x = ob.from_numpy(np.asarray(a, dtype=np.float32), dtype)
    if grad:
        x.requires_grad_(True)
    return x


def tt(a):
    return torch.tensor(np.asarray(a, dtype=np.float32), requires_grad=True)


def close(a, b, tol=1e-5):
    assert np.allclose(a.numpy(), b.detach().numpy().reshape(a.numpy().shape), atol=tol, rtol=tol)


def test_chain_and_branches_match_torch():
    rng = np.random.default_rng(0)
    A, B, C = rng.standard_normal((4, 5)), rng.standard_normal((5, 3)), rng.standard_normal((3,))
    a, b, c = t(A), t(B), t(C)
    y = ((a @ b + c).tanh() * (a @ b).sigmoid()).sum() + (a * a).mean()
    y.backward()
    ta, tb, tc = tt(A), tt(B), tt(C)
    ty = ((ta @ tb + tc).tanh() * (ta @ tb).sigmoid()).sum() + (ta * ta).mean()
    ty.backward()
    close(a.grad, ta.grad)
    close(b.grad, tb.grad)
    close(c.grad, tc.grad)


@pytest.mark.parametrize("op", ["relu", "sigmoid", "tanh", "gelu", "exp", "sqrt", "reciprocal", "neg", "log"])
def test_unary_gradients(op):
    x0 = np.random.default_rng(1).uniform(0.5, 2.0, size=(3, 4))
    x = t(x0)
    getattr(x, op)().sum().backward()
    tx = tt(x0)
    f = {"gelu": torch.nn.functional.gelu, "neg": torch.neg}.get(op) or getattr(torch, op)
    f(tx).sum().backward()
    close(x.grad, tx.grad)


def test_views_slices_index_and_transpose_backward():
    X = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    x = t(X)
    y = x.transpose(1, 2).contiguous().reshape([2, 12]).slice(1, 2, 9)
    (y * y).sum().backward()
    tx = tt(X)
    ty = tx.transpose(1, 2).contiguous().reshape(2, 12)[:, 2:9]
    (ty * ty).sum().backward()
    close(x.grad, tx.grad)
    z = t(X)
    (z[1] * 3.0).sum().backward()
    assert z.grad.tolist()[:12] == [0.0] * 12 and z.grad.tolist()[12:] == [3.0] * 12


def test_max_softmax_losses_embedding():
    rng = np.random.default_rng(2)
    L = rng.standard_normal((6, 7))
    tgt = rng.integers(0, 7, 6)
    x = t(L)
    ob.cross_entropy(x, tgt.tolist()).backward()
    tx = tt(L)
    torch.nn.functional.cross_entropy(tx, torch.tensor(tgt)).backward()
    close(x.grad, tx.grad)
    x2, tx2 = t(L), tt(L)
    ob.nll_loss(x2.log_softmax(-1), tgt.tolist(), "sum").backward()
    torch.nn.functional.nll_loss(tx2.log_softmax(-1), torch.tensor(tgt), reduction="sum").backward()
    close(x2.grad, tx2.grad)
    x3, tx3 = t(L), tt(L)
    (x3.softmax(0) * x3).sum().backward()
    (tx3.softmax(0) * tx3).sum().backward()
    close(x3.grad, tx3.grad)
    x4, tx4 = t(L), tt(L)
    v = x4.max(1)
    v.sum().backward()
    tx4.max(1).values.sum().backward()
    close(x4.grad, tx4.grad)
    W = rng.standard_normal((10, 4))
    w, tw = t(W), tt(W)
    idx = np.array([[1, 1, 3], [9, 0, 1]])
    ob.embedding(ob.from_numpy(idx.astype(np.int64)), w).sum().backward()
    torch.nn.functional.embedding(torch.tensor(idx), tw).sum().backward()
    close(w.grad, tw.grad)


def test_conv_pool_layernorm_attention_gradients():
    rng = np.random.default_rng(3)
    X, W, B = rng.standard_normal((2, 3, 7, 7)), rng.standard_normal((4, 3, 3, 3)), rng.standard_normal(4)
    x, w, b = t(X), t(W), t(B)
    y = ob.maxpool2d(ob.conv2d(x, w, b, 2, 2, 1, 1).relu(), 2, 2, 2, 2)
    y.sum().backward()
    tx, tw, tb = tt(X), tt(W), tt(B)
    ty = torch.nn.functional.max_pool2d(torch.nn.functional.conv2d(tx, tw, tb, stride=2, padding=1).relu(), 2, 2)
    ty.sum().backward()
    close(x.grad, tx.grad), close(w.grad, tw.grad), close(b.grad, tb.grad)
    Z, G, Bt = rng.standard_normal((5, 8)), rng.standard_normal(8), rng.standard_normal(8)
    z, g, bt = t(Z), t(G), t(Bt)
    (ob.layer_norm(z, 8, g, bt) * z).sum().backward()
    tz, tg, tbt = tt(Z), tt(G), tt(Bt)
    (torch.nn.functional.layer_norm(tz, (8,), tg, tbt) * tz).sum().backward()
    close(z.grad, tz.grad, 1e-4), close(g.grad, tg.grad, 1e-4), close(bt.grad, tbt.grad, 1e-4)
    Q, K, V = (rng.standard_normal((2, 2, 5, 4)) for _ in range(3))
    q, k, v = t(Q), t(K), t(V)
    ob.scaled_dot_product_attention(q, k, v, is_causal=True).sum().backward()
    tq, tk, tv = tt(Q), tt(K), tt(V)
    torch.nn.functional.scaled_dot_product_attention(tq, tk, tv, is_causal=True).sum().backward()
    close(q.grad, tq.grad, 1e-4), close(k.grad, tk.grad, 1e-4), close(v.grad, tv.grad, 1e-4)


def test_accumulation_retain_graph_and_freed_graph():
    x = t([1.0, 2.0])
    y = (x * x).sum()
    y.backward(retain_graph=True)
    y.backward()
    assert x.grad.tolist() == [4.0, 8.0]
    with pytest.raises(RuntimeError, match="Cannot call backward twice on a freed graph"):
        y.backward()
    x.zero_grad()
    assert x.grad is None


def test_saved_tensor_version_check():
    x = t([1.0, 2.0])
    w = t([3.0, 4.0], grad=False)
    y = (x * w).sum()
    w.fill_(0.0)
    with pytest.raises(RuntimeError, match="was modified in-place after it was saved for backward"):
        y.backward()
    assert x.grad is None  # nothing was published


def test_grad_is_independent_leaf_and_hooks_and_finalizers():
    x = t([1.0, 2.0, 3.0])
    calls = []
    x._register_post_accumulate_grad_hook(lambda: calls.append("hook"))
    x._register_backward_finalizer(7, lambda: calls.append("fin"))
    x._register_backward_finalizer(7, lambda: calls.append("fin"))  # same key: once
    (x + x).sum().backward()
    assert calls == ["hook", "fin"]
    g = x.grad
    assert g.is_leaf and not g.requires_grad and g.tolist() == [2.0, 2.0, 2.0]
    g2 = x.grad
    assert g2._buffer_id == g._buffer_id


def test_no_grad_nonscalar_root_and_integer_cast_cuts_graph():
    x = t([1.0, 2.0])
    with ob.no_grad():
        y = x * 2.0
    assert not y.requires_grad
    (x * 3.0).backward()  # non-scalar root: seed of ones
    assert x.grad.tolist() == [3.0, 3.0]
    z = ob.cast(x, "int32")
    assert not z.requires_grad
    with pytest.raises(RuntimeError):
        y.backward()


def test_deep_chain_does_not_recurse():
    x = t([1.0])
    y = x
    for _ in range(4096):
        y = y + 1.0
    y.backward()
    assert x.grad.tolist() == [1.0]


def test_unused_branch_and_shared_subexpression():
    a, b = t([2.0]), t([5.0])
    s = a * b
    unused = s * 10.0  # noqa: F841
    (s + s * s).backward()
    assert a.grad.tolist() == [5.0 + 2 * 10.0 * 5.0]
    assert b.grad.tolist() == [2.0 + 2 * 10.0 * 2.0]
