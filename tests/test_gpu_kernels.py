"""sm_100a kernels against a plain PyTorch float32 reference of the same op."""
import numpy as np
import pytest
import torch

import orthon_b200 as ob
from orthon_b200 import _C

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "float16": 5e-3, "bfloat16": 4e-2}


def dev_tensor(arr, dtype, requires_grad=False):
    t = _C.from_numpy(np.ascontiguousarray(arr, dtype=np.float32), dtype).to("cuda:0")
    if requires_grad:
        t.requires_grad_(True)
    return t


def ref_round(arr, dtype):
    """The values after a round trip through `dtype` (what the kernel actually sees), held in float64 so that the
    reference arithmetic adds no error of its own (the float32 CPU routines of the reference library differ
    between hosts by more than the kernels' tolerance)."""
    t = torch.tensor(np.asarray(arr, dtype=np.float32))
    if dtype == "float16":
        t = t.half().float()
    elif dtype == "bfloat16":
        t = t.bfloat16().float()
    return t.double()


def close(actual, expected, dtype, scale=1.0):
    a = torch.tensor(actual.numpy().astype(np.float32))
    e = expected.detach().float().reshape(a.shape)
    tol = TOL[dtype] * scale
    err = (a - e).abs().max().item()
    ref = e.abs().max().item()
    if not err <= tol * max(1.0, ref):
        import inspect
        where = inspect.stack()[1]
        bad = int((a - e).abs().argmax().item())
        raise AssertionError(f"line {where.lineno}: max err {err} vs tol {tol * max(1.0, ref)} at flat index {bad} of {a.numel()} "
                             f"(got {a.reshape(-1)[bad].item()}, want {e.reshape(-1)[bad].item()})")


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_elementwise_and_broadcast(dtype):
    rng = np.random.default_rng(0)
    a = rng.standard_normal((37, 65)); b = rng.standard_normal((65,))
    ta, tb = ref_round(a, dtype), ref_round(b, dtype)
    x, y = dev_tensor(a, dtype), dev_tensor(b, dtype)
    close(x + y, ta + tb, dtype)
    close(x * y, ta * tb, dtype)
    close(x.relu(), ta.relu(), dtype)
    # Transcendental references are taken in float64: the float32 CPU routines of the reference library
    # differ between hosts by more than the kernels' own error.
    td = ta.double()
    close(x.gelu(), torch.nn.functional.gelu(td), dtype)
    close(x.sigmoid(), td.sigmoid(), dtype)
    close(x.tanh(), td.tanh(), dtype)
    close(x.exp(), td.exp(), dtype, 4)
    close(x * 2.5 + 1.0, ta * 2.5 + 1.0, dtype)
    close(x.transpose(0, 1).contiguous(), ta.t(), dtype)
    big = rng.standard_normal((1 << 20) + 3)
    close(dev_tensor(big, dtype) + dev_tensor(big, dtype), 2 * ref_round(big, dtype), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unary_backward(dtype):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((33, 40))
    for name in ["relu", "gelu", "sigmoid", "tanh"]:
        x = dev_tensor(a, dtype, True)
        getattr(x, name)().sum().backward()
        t = ref_round(a, dtype).double().requires_grad_(True)   # float64 reference, see above
        getattr(torch.nn.functional, name)(t).sum().backward() if name != "tanh" else t.tanh().sum().backward()
        close(x.grad, t.grad, dtype)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_reductions(dtype):
    rng = np.random.default_rng(2)
    a = rng.standard_normal((6, 50, 33))
    t = ref_round(a, dtype); x = dev_tensor(a, dtype)
    close(x.sum(), t.sum(), dtype, 50)
    close(x.mean(), t.mean(), dtype)
    for d in range(3):
        close(x.sum(d), t.sum(d), dtype, 8)
        close(x.mean(d, True), t.mean(d, True), dtype)
        v, i = x.max(d), x.argmax(d)
        tv, ti = t.max(d)
        close(v, tv, dtype)
        assert i.tolist() == ti.flatten().tolist()
    big = rng.standard_normal((3, 200000))
    close(dev_tensor(big, dtype).sum(1), ref_round(big, dtype).sum(1), dtype, 200)
    close(dev_tensor(big, dtype).sum(0), ref_round(big, dtype).sum(0), dtype, 4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_bias_grad_unbroadcast(dtype):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((300, 96)); b = rng.standard_normal((96,))
    x = dev_tensor(a, dtype, True); y = dev_tensor(b, dtype, True)
    (x + y).sum().backward()
    close(y.grad, torch.full((96,), 300.0), dtype)
    close(x.grad, torch.ones(300, 96), dtype)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_softmax_family_and_losses(dtype):
    rng = np.random.default_rng(4)
    a = rng.standard_normal((64, 1000)) * 3
    tgt = rng.integers(0, 1000, size=64)
    t = ref_round(a, dtype).requires_grad_(True)
    x = dev_tensor(a, dtype, True)
    close(x.softmax(-1), t.softmax(-1), dtype)
    close(x.log_softmax(-1), t.log_softmax(-1), dtype, 8)
    loss = _C.cross_entropy(x, tgt.tolist())
    tl = torch.nn.functional.cross_entropy(t, torch.tensor(tgt))
    close(loss, tl, "float32" if dtype != "float32" else dtype, 50)
    loss.backward(); tl.backward()
    close(x.grad, t.grad, dtype, 0.05)
    x2 = dev_tensor(a, dtype, True); t2 = ref_round(a, dtype).requires_grad_(True)
    l2 = _C.nll_loss(x2.log_softmax(-1), _C.from_numpy(tgt.astype(np.int64)).to("cuda:0"))
    tl2 = torch.nn.functional.nll_loss(t2.log_softmax(-1), torch.tensor(tgt))
    close(l2, tl2, dtype, 8)
    l2.backward(); tl2.backward()
    close(x2.grad, t2.grad, dtype, 0.05)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_norm(dtype):
    rng = np.random.default_rng(5)
    # (4100, 512): narrow rows in thousands of persistent blocks, parameter gradients reduced in two stages
    for R, D in ((70, 512), (70, 100), (4100, 512), (300, 2048)):
        a = rng.standard_normal((R, D)) * 2 + 0.5; w = rng.standard_normal((D,)); b = rng.standard_normal((D,))
        g = rng.standard_normal((R, D))
        x, ww, bb = dev_tensor(a, dtype, True), dev_tensor(w, dtype, True), dev_tensor(b, dtype, True)
        t, tw, tb = (ref_round(v, dtype).requires_grad_(True) for v in (a, w, b))
        y = _C._layer_norm(x, ww, bb, 1e-5)
        ty = torch.nn.functional.layer_norm(t, (D,), tw, tb, 1e-5)
        close(y, ty, dtype)
        (y * dev_tensor(g, dtype)).sum().backward()
        (ty * ref_round(g, dtype)).sum().backward()
        close(x.grad, t.grad, dtype, 2)
        close(ww.grad, tw.grad, dtype, 8 if R < 1000 else 32)
        close(bb.grad, tb.grad, dtype, 8 if R < 1000 else 32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding(dtype):
    rng = np.random.default_rng(6)
    w = rng.standard_normal((50, 64)); idx = rng.integers(0, 50, size=(4, 9))
    ww = dev_tensor(w, dtype, True); tw = ref_round(w, dtype).requires_grad_(True)
    ii = _C.from_numpy(idx.astype(np.int64)).to("cuda:0")
    y = _C.embedding(ii, ww); ty = torch.nn.functional.embedding(torch.tensor(idx), tw)
    close(y, ty, dtype)
    y.sum().backward(); ty.sum().backward()
    close(ww.grad, tw.grad, dtype)


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (200, 136, 72), (384, 1024, 512), (1024, 1024, 1024), (130, 96, 200)]


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_all_majors(dtype, ta, tb):
    rng = np.random.default_rng(7)
    for (M, N, K) in GEMM_SHAPES:
        a = rng.standard_normal((K, M) if ta else (M, K)); b = rng.standard_normal((N, K) if tb else (K, N))
        x, y = dev_tensor(a, dtype), dev_tensor(b, dtype)
        t, u = ref_round(a, dtype), ref_round(b, dtype)
        out = _C._gemm(x, ta, y, tb)
        ref = (t.t() if ta else t) @ (u.t() if tb else u)
        close(out, ref, dtype, 0.5 if dtype != "float32" else 20)
    _C.cuda_synchronize()


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_linear_epilogues(dtype):
    rng = np.random.default_rng(8)
    M, K, N = 300, 256, 512
    a, w, b, r = rng.standard_normal((M, K)), rng.standard_normal((K, N)) * 0.1, rng.standard_normal((N,)), rng.standard_normal((M, N))
    for act in ("none", "relu", "gelu"):
        x, ww, bb = dev_tensor(a, dtype, True), dev_tensor(w, dtype, True), dev_tensor(b, dtype, True)
        t, tw, tb = (ref_round(v, dtype).requires_grad_(True) for v in (a, w, b))
        res = None if act == "relu" else dev_tensor(r, dtype)
        y = _C.linear(x, ww, bb, act, res)
        z = t @ tw + tb
        ty = {"none": z, "relu": z.relu(), "gelu": torch.nn.functional.gelu(z)}[act]
        if res is not None:
            ty = ty + ref_round(r, dtype)
        close(y, ty, dtype)
        y.sum().backward(); ty.sum().backward()
        close(x.grad, t.grad, dtype, 2)
        close(ww.grad, tw.grad, dtype, 2)
        close(bb.grad, tb.grad, dtype, 8)
    _C.cuda_synchronize()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_batched_gemm_and_attention(dtype):
    rng = np.random.default_rng(9)
    B, H, T, D = 2, 3, 128, 64
    q, k, v = (rng.standard_normal((B, H, T, D)) for _ in range(3))
    xq, xk, xv = (dev_tensor(t_, dtype, True) for t_ in (q, k, v))
    tq, tk, tv = (ref_round(t_, dtype).requires_grad_(True) for t_ in (q, k, v))
    out = _C._attention(xq, xk, xv, None, True, D ** -0.5)
    ref = torch.nn.functional.scaled_dot_product_attention(tq, tk, tv, is_causal=True)
    close(out, ref, dtype)
    out.sum().backward(); ref.sum().backward()
    for g, tg in ((xq, tq), (xk, tk), (xv, tv)):
        close(g.grad, tg.grad, dtype, 2)
    _C.cuda_synchronize()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_conv_and_pool(dtype):
    rng = np.random.default_rng(10)
    x = rng.standard_normal((3, 5, 12, 12)); w = rng.standard_normal((7, 5, 3, 3)) * 0.2; b = rng.standard_normal((7,))
    for stride in (1, 2):
        xx, ww, bb = dev_tensor(x, dtype, True), dev_tensor(w, dtype, True), dev_tensor(b, dtype, True)
        t, tw, tb = (ref_round(v_, dtype).requires_grad_(True) for v_ in (x, w, b))
        y = _C.conv2d(xx, ww, bb, stride, stride, 1, 1)
        ty = torch.nn.functional.conv2d(t, tw, tb, stride=stride, padding=1)
        close(y, ty, dtype)
        y.sum().backward(); ty.sum().backward()
        close(xx.grad, t.grad, dtype, 2); close(ww.grad, tw.grad, dtype, 8); close(bb.grad, tb.grad, dtype, 8)
    xx = dev_tensor(x, dtype, True); t = ref_round(x, dtype).requires_grad_(True)
    y = _C.maxpool2d(xx, 2, 2, 2, 2); ty = torch.nn.functional.max_pool2d(t, 2, 2)
    close(y, ty, dtype)
    y.sum().backward(); ty.sum().backward()
    close(xx.grad, t.grad, dtype)


CONV_CASES = [
    # (N, C, H, W, K, R, S, stride, pad): the three layers of the small CNN, then shapes that leave tiles partly empty
    (8, 3, 32, 32, 32, 3, 3, 1, 1), (8, 32, 32, 32, 64, 3, 3, 2, 1), (8, 64, 16, 16, 128, 3, 3, 2, 1),
    (2, 5, 12, 12, 7, 3, 3, 1, 1), (3, 4, 9, 11, 20, 3, 3, 2, 0), (1, 16, 8, 8, 24, 1, 1, 1, 0), (2, 6, 10, 10, 130, 3, 3, 1, 1),
    (2, 40, 16, 16, 16, 5, 5, 1, 2), (5, 8, 20, 20, 8, 3, 3, 3, 1),
    # strides larger than the filter: some input pixels are reached by no tap
    (2, 8, 8, 8, 16, 1, 1, 2, 0), (2, 4, 9, 9, 8, 2, 2, 3, 0),
]


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_implicit_gemm_forward_and_gradients(dtype, case):
    N, C, H, W, K, R, S, stride, pad = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((N, C, H, W)); w = rng.standard_normal((K, C, R, S)) * (1.0 / np.sqrt(C * R * S)); b = rng.standard_normal((K,))
    xx, ww, bb = dev_tensor(x, dtype, True), dev_tensor(w, dtype, True), dev_tensor(b, dtype, True)
    t, tw, tb = (ref_round(v_, dtype).requires_grad_(True) for v_ in (x, w, b))
    y = _C.conv2d(xx, ww, bb, stride, stride, pad, pad)
    assert _C._conv2d_last_route() == "tcgen05_implicit_gemm"
    ty = torch.nn.functional.conv2d(t, tw, tb, stride=stride, padding=pad)
    close(y, ty, dtype)
    weight = rng.standard_normal(tuple(ty.shape))
    gw = dev_tensor(weight, dtype)
    (y * gw).sum().backward()
    (ty * ref_round(weight, dtype)).sum().backward()
    scale = 4 * np.sqrt(N * ty.shape[2] * ty.shape[3] / 64.0) + 4
    close(xx.grad, t.grad, dtype, 4); close(ww.grad, tw.grad, dtype, scale); close(bb.grad, tb.grad, dtype, scale)
    assert _C._cuda_index_errors() == 0


def test_conv_skips_the_input_gradient_nobody_asked_for():
    rng = np.random.default_rng(3)
    xx = dev_tensor(rng.standard_normal((2, 3, 8, 8)), "bfloat16")            # does not require grad
    ww = dev_tensor(rng.standard_normal((4, 3, 3, 3)), "bfloat16", True)
    before = _C._kernel_launch_count()
    y = _C.conv2d(xx, ww, None, 1, 1, 1, 1)
    y.sum().backward()
    assert xx.grad is None and ww.grad is not None
    _C._conv2d_force_route("auto")
    assert _C._kernel_launch_count() - before <= 12


def test_adam_fused_matches_formula():
    rng = np.random.default_rng(11)
    p0, g = rng.standard_normal(1000), rng.standard_normal(1000)
    p = dev_tensor(p0, "float32"); m = _C._zeros_on([1000], "float32", "cuda:0"); v = _C._zeros_on([1000], "float32", "cuda:0")
    model = _C._zeros_on([1000], "bfloat16", "cuda:0")
    gg = dev_tensor(g * 128, "bfloat16")
    _C._adam_step_(p, m, v, gg, model, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1 - 0.9, 1 - 0.999, 1.0 / 128)
    tp = torch.tensor(p0, dtype=torch.float32).requires_grad_(True)
    opt = torch.optim.Adam([tp], lr=1e-3)
    tp.grad = (torch.tensor(g * 128, dtype=torch.float32).bfloat16().float() / 128)
    opt.step()
    close(p, tp, "float32", 10)
    close(model, tp, "bfloat16")


def test_diagnostic_routes():
    from orthon_b200 import _diagnostics as diag
    rng = np.random.default_rng(21)
    a, b = rng.standard_normal((256, 192)), rng.standard_normal((192, 320))
    xa, xb = dev_tensor(a, "bfloat16"), dev_tensor(b, "bfloat16")
    ref = ref_round(a, "bfloat16") @ ref_round(b, "bfloat16")
    close(diag.matmul_simt(xa, xb), ref, "bfloat16")
    close(diag.matmul_tcgen05(xa, xb), ref, "bfloat16")
    assert diag.matmul_dispatch_path(xa, xb) == "tcgen05_128x128"  # four wide tiles would leave most SMs idle
    big_a, big_b = dev_tensor(rng.standard_normal((2048, 64)), "bfloat16"), dev_tensor(rng.standard_normal((64, 2560)), "bfloat16")
    assert diag.matmul_dispatch_path(big_a, big_b) == "tcgen05_128x256"
    # float32: the FMA kernel by default; under "high" precision large products run as bfloat16
    # piece products on the tensor cores and small ones stay where they were
    small_a, small_b = dev_tensor(a[:64, :64], "float32"), dev_tensor(b[:64, :64], "float32")
    fa, fb = dev_tensor(a, "float32"), dev_tensor(b, "float32")
    assert ob.get_float32_matmul_precision() == "highest"
    assert diag.matmul_dispatch_path(fa, fb) == "simt"
    ob.set_float32_matmul_precision("high")
    try:
        assert diag.matmul_dispatch_path(small_a, small_b) == "simt"
        assert diag.matmul_dispatch_path(fa, fb).startswith("tcgen05")
    finally:
        ob.set_float32_matmul_precision("highest")
    with pytest.raises(ValueError):
        ob.set_float32_matmul_precision("medium")
    exact = torch.tensor(a, dtype=torch.float64) @ torch.tensor(b, dtype=torch.float64)
    close(diag.matmul_tcgen05(fa, fb), exact, "float32")
    close(diag.matmul_simt(fa, fb), exact, "float32")
    x = rng.standard_normal((2, 8, 16, 16)); w = rng.standard_normal((16, 8, 3, 3)) * 0.2
    xx, ww = dev_tensor(x, "bfloat16"), dev_tensor(w, "bfloat16")
    y_direct = diag.conv2d_direct(xx, ww, None, (1, 1), (1, 1))
    assert _C._conv2d_last_route() == "direct"
    assert diag.conv2d_dispatch_path(xx, ww, None, (1, 1), (1, 1)) == "tcgen05_implicit_gemm"
    _C._conv2d_force_route("lowering")
    try:
        y_lowered = _C.conv2d(xx, ww, None, 1, 1, 1, 1)
        assert _C._conv2d_last_route() == "tcgen05_lowering"
    finally:
        _C._conv2d_force_route("auto")
    close(y_lowered, torch.nn.functional.conv2d(ref_round(x, "bfloat16"), ref_round(w, "bfloat16"), padding=1), "bfloat16")
    y_auto = _C.conv2d(xx, ww, None, 1, 1, 1, 1)
    ty = torch.nn.functional.conv2d(ref_round(x, "bfloat16"), ref_round(w, "bfloat16"), padding=1)
    close(y_direct, ty, "bfloat16"); close(y_auto, ty, "bfloat16")


@pytest.mark.parametrize("dtype,shape", [("bfloat16", (384, 256, 512)), ("float32", (384, 256, 512)),
                                         # 256-row tiles with the activation derivative as a second output of the same
                                         # staging tile (16 x 9 tiles fill one wave), and a width that ends in a half group
                                         ("bfloat16", (4096, 2048, 2304)), ("float16", (1024, 2048, 9440))])
def test_fused_mlp_gelu(dtype, shape):
    rng = np.random.default_rng(31)
    M, E, F = shape
    arrs = [rng.standard_normal((M, E)), rng.standard_normal((E, F)) * 0.05, rng.standard_normal((F,)) * 0.1,
            rng.standard_normal((F, E)) * 0.05, rng.standard_normal((E,)) * 0.1]
    xs = [dev_tensor(a, dtype, True) for a in arrs]
    ts = [ref_round(a, dtype).requires_grad_(True) for a in arrs]
    y = _C._mlp_gelu(xs[0], xs[1], xs[2], xs[3], xs[4], xs[0])
    ty = torch.nn.functional.gelu(ts[0] @ ts[1] + ts[2]) @ ts[3] + ts[4] + ts[0]
    close(y, ty, dtype, 2)
    w = rng.standard_normal((M, E))
    (y * dev_tensor(w, dtype)).sum().backward()
    (ty * ref_round(w, dtype)).sum().backward()
    for g, tg in zip(xs, ts):
        close(g.grad, tg.grad, dtype, 8)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_broadcast_fast_paths(dtype):
    """Row, column and single-value operands on either side, including shapes whose rows are
    not a multiple of the 16-byte pack (generic route)."""
    rng = np.random.default_rng(5)
    cases = [((64, 256), (256,)), ((64, 256), (1, 256)), ((64, 256), (64, 1)), ((64, 256), (1,)), ((4, 8, 64), (8, 64)),
             ((4, 8, 64), (4, 1, 1)), ((4, 8, 64), (4, 8, 1)), ((33, 100), (100,)), ((33, 100), (33, 1)), ((7, 5), (5,))]
    for full_shape, small_shape in cases:
        f, s = rng.standard_normal(full_shape), rng.standard_normal(small_shape)
        tf, ts = dev_tensor(f, dtype), dev_tensor(s, dtype)
        rf, rs = ref_round(f, dtype), ref_round(s, dtype)
        close(ob.add(tf, ts), rf + rs, dtype)
        close(ob.add(ts, tf), rs + rf, dtype)
        close(ob.mul(tf, ts), rf * rs, dtype, scale=2.0)
        close(ob.sub(ts, tf), rs - rf, dtype)   # broadcast operand on the left of a composite
        close(ob.div(tf, ob.add(ob.mul(ts, ts), ob.ones([1]).to("cuda:0").cast(dtype))), rf / (rs * rs + 1), dtype, scale=4.0)


def test_dropout_mask_matches_cpu_stream_for_every_alignment():
    for n in (1, 7, 8, 1000, 4096 + 3):
        for dtype in ("float32", "bfloat16"):
            x = np.ones(n, dtype=np.float32)
            cpu = ob.dropout(ob.from_numpy(x), 0.3, 99).tolist()
            gpu = ob.dropout(dev_tensor(x, dtype), 0.3, 99)
            got = torch.tensor(gpu.numpy().astype(np.float32))
            want = ref_round(np.asarray(cpu, dtype=np.float32), dtype)
            assert (got == 0).tolist() == (want == 0).tolist(), (n, dtype)
            assert torch.allclose(got, want.float(), rtol=1e-2)
    # Fused forward and recomputed-mask backward against the CPU composite (mask tensor times input).
    rng = np.random.default_rng(8)
    for dtype in ("float32", "bfloat16"):
        x = rng.standard_normal((37, 24))
        cx = ob.from_numpy(ref_round(x, dtype).numpy()).requires_grad_(True)
        gx = dev_tensor(x, dtype, requires_grad=True)
        w = rng.standard_normal((37, 24))
        (ob.dropout(cx, 0.25, 7) * ob.from_numpy(ref_round(w, dtype).numpy())).sum().backward()
        (ob.dropout(gx, 0.25, 7) * dev_tensor(w, dtype)).sum().backward()
        close(ob.dropout(gx, 0.25, 7), torch.tensor(ob.dropout(cx, 0.25, 7).numpy()), dtype)
        close(gx.grad, torch.tensor(cx.grad.numpy()), dtype, scale=2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_sum_long_rows(dtype):
    rng = np.random.default_rng(6)
    for n in (1 << 20, (1 << 20) + 13, 5000):
        x = rng.standard_normal(n) * 0.1
        t = dev_tensor(x, dtype)
        want = ref_round(x, dtype).double().sum().float()
        close(t.sum(), want.reshape(1), dtype, scale=8.0)
        close(t.reshape([1, n]).mean(1), (want / n).reshape(1), dtype)


def test_float32_gemm_through_piece_products():
    """float32 matmul / linear on the tensor-core route against a float64 product: error at the
    float32 level for every operand major, batch form, odd reduction length and epilogue."""
    from orthon_b200 import _diagnostics as diag
    rng = np.random.default_rng(33)

    def f64(x):
        return torch.tensor(np.asarray(x, dtype=np.float32), dtype=torch.float64)

    for (m, k, n) in [(256, 192, 320), (130, 191, 70), (512, 1024, 256), (64, 4096, 40)]:
        a, b = rng.standard_normal((m, k)), rng.standard_normal((k, n))
        ta, tb = dev_tensor(a, "float32", True), dev_tensor(b, "float32", True)
        out = diag.matmul_tcgen05(ta, tb)
        ref = f64(a) @ f64(b)
        err = (torch.tensor(out.numpy(), dtype=torch.float64) - ref).abs().max().item() / ref.abs().max().item()
        assert err < 3e-6 + 3e-8 * k, (m, k, n, err)   # truncating accumulation: grows with the reduction length
    ob.set_float32_matmul_precision("high")
    try:
        _piece_product_api_checks(rng, f64)
    finally:
        ob.set_float32_matmul_precision("highest")


def _piece_product_api_checks(rng, f64):
    # transposed views (backward products) and gradients through the public matmul
    a, b = rng.standard_normal((384, 256)), rng.standard_normal((256, 512))
    ta, tb = dev_tensor(a, "float32", True), dev_tensor(b, "float32", True)
    w = rng.standard_normal((384, 512))
    (ob.matmul(ta, tb) * dev_tensor(w, "float32")).sum().backward()
    assert _C._matmul_last_route().startswith("tcgen05")
    close(ta.grad, f64(w) @ f64(b).T, "float32")
    close(tb.grad, f64(a).T @ f64(w), "float32")
    # batched, one operand shared by the batch
    a3, b3 = rng.standard_normal((6, 128, 96)), rng.standard_normal((6, 96, 160))
    close(ob.matmul(dev_tensor(a3, "float32"), dev_tensor(b3, "float32")), f64(a3) @ f64(b3), "float32")
    # linear with bias and ReLU
    x, wgt, bias = rng.standard_normal((300, 200)), rng.standard_normal((200, 150)) * 0.1, rng.standard_normal(150)
    y = ob.fused_linear_relu(dev_tensor(x, "float32"), dev_tensor(wgt, "float32"), dev_tensor(bias, "float32"))
    close(y, torch.relu(f64(x) @ f64(wgt) + f64(bias)), "float32")
    y2 = ob.linear(dev_tensor(x, "float32"), dev_tensor(wgt, "float32"), dev_tensor(bias, "float32"))
    close(y2, f64(x) @ f64(wgt) + f64(bias), "float32")


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_split_k_gemm_small_output_long_reduction(dtype):
    """Weight-gradient shapes of a narrow model: the reduction is split over batch entries of the
    tcgen05 kernel and the float32 partials are added in a fixed order."""
    rng = np.random.default_rng(44)
    for (m, k, n) in [(512, 16384, 512), (512, 8192, 2048), (256, 4096, 384)]:
        x = rng.standard_normal((k, m)) * 0.1   # stored [K, M]: the transposed (weight-gradient) form
        g = rng.standard_normal((k, n)) * 0.1
        tx, tg = dev_tensor(x, dtype), dev_tensor(g, dtype)
        ref = ref_round(x, dtype).double().T @ ref_round(g, dtype).double()
        out = ob.matmul(ob.transpose(tx, 0, 1), tg)
        assert _C._matmul_last_route().startswith("tcgen05")
        close(out, ref.float(), dtype, scale=0.5)
        again = ob.matmul(ob.transpose(tx, 0, 1), tg)
        assert out.numpy().tobytes() == again.numpy().tobytes()   # fixed summation order
        # K-major operands as well
        a = rng.standard_normal((m, k)) * 0.1
        b = rng.standard_normal((n, k)) * 0.1
        ta, tb = dev_tensor(a, dtype), dev_tensor(b, dtype)
        ref2 = ref_round(a, dtype).double() @ ref_round(b, dtype).double().T
        close(ob.matmul(ta, ob.transpose(tb, 0, 1)), ref2.float(), dtype, scale=0.5)
    # gradients of a Linear over many tokens take the same route
    w = rng.standard_normal((512, 512)) * 0.05
    xs = rng.standard_normal((16384, 512)) * 0.5
    tw, txs = dev_tensor(w, dtype, True), dev_tensor(xs, dtype)
    ob.matmul(txs, tw).sum().backward()
    expect = ref_round(xs, dtype).double().T @ torch.ones(16384, 512, dtype=torch.float64)
    close(tw.grad, expect.float(), dtype, scale=2.0)


def test_embedding_backward_is_deterministic_and_sums_in_position_order():
    """Many positions share few rows, so the order of the additions matters for the rounded
    result: two runs must agree bit for bit and match a float32 reference that adds in
    increasing position."""
    rng = np.random.default_rng(12)
    n, V, D = 4099, 37, 72
    idx_np = rng.integers(0, V - 3, size=n).astype(np.int64)        # rows V-3.. stay untouched
    g_np = rng.standard_normal((n, D)).astype(np.float32)
    for dtype, tol in (("float32", 0.0), ("bfloat16", 0.0)):
        w = _C.from_numpy(np.zeros((V, D), dtype=np.float32), dtype).to("cuda:0")
        w.requires_grad_(True)
        idx = _C.from_numpy(idx_np).to("cuda:0")
        g = _C.from_numpy(g_np, dtype).to("cuda:0")
        runs = []
        for _ in range(2):
            w.zero_grad()
            (ob.embedding(idx, w) * g).sum().backward()
            runs.append(w.grad.numpy().astype(np.float32).copy())
        assert np.array_equal(runs[0], runs[1])
        g_used = g.numpy().astype(np.float32)
        want = np.zeros((V, D), dtype=np.float32)
        for i in range(n):                                           # increasing position, float32 accumulation
            want[idx_np[i]] += g_used[i]
        if dtype == "bfloat16":
            want = torch.tensor(want).to(torch.bfloat16).to(torch.float32).numpy()
        assert np.array_equal(runs[0], want)
        assert not runs[0][V - 3:].any()
    assert _C._cuda_index_errors() == 0


def test_debug_bounds_switch_names_the_kernel_that_clamped_an_index():
    """With ORTHON_DEBUG_BOUNDS=1 every kernel wrapper drains the device and an out-of-range index raises at once."""
    import os
    import subprocess
    import sys
    code = (
        "import numpy as np\n"
        "from orthon_b200 import _C\n"
        "from orthon_b200.nn.embedding import embedding\n"
        "w = _C.from_numpy(np.ones((10, 8), np.float32), 'float32').to('cuda:0')\n"
        "ok = _C.from_numpy(np.array([1, 9], np.int64)).to('cuda:0')\n"
        "embedding(ok, w)\n"
        "bad = _C.from_numpy(np.array([1, 10], np.int64)).to('cuda:0')\n"
        "try:\n"
        "    embedding(bad, w)\n"
        "except IndexError as e:\n"
        "    print('RAISED', e)\n"
    )
    env = dict(os.environ, ORTHON_DEBUG_BOUNDS="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert "RAISED embedding: " in out.stdout and "index value(s) outside the valid range" in out.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(64, 512), (33, 2048), (7, 200)])
def test_layer_norm_backward_adds_the_residual_gradient_in_the_same_pass(dtype, shape):
    """y = h + LayerNorm(h): the skip path's gradient reaches h first and the LayerNorm formula adds it while it
    writes its own input gradient; the sum must match the reference either way."""
    rng = np.random.default_rng(shape[0])
    x = rng.standard_normal(shape); w = rng.standard_normal((shape[1],)); b = rng.standard_normal((shape[1],))
    up = rng.standard_normal(shape)
    xx, ww, bb = dev_tensor(x, dtype, True), dev_tensor(w, dtype, True), dev_tensor(b, dtype, True)
    h = xx * 2.0
    before = _C._kernel_launch_count()
    y = h + ob.layer_norm(h, shape[1], ww, bb)
    (y * dev_tensor(up, dtype)).sum().backward()
    t, tw, tb = (ref_round(v_, dtype).requires_grad_(True) for v_ in (x, w, b))
    th = t * 2.0
    ty = th + torch.nn.functional.layer_norm(th, (shape[1],), tw, tb)
    (ty * ref_round(up, dtype)).sum().backward()
    close(xx.grad, t.grad, dtype, 8); close(ww.grad, tw.grad, dtype, 8); close(bb.grad, tb.grad, dtype, 8)
    # Without the fused addition the same graph takes one more kernel wrapper (the engine's add).
    assert _C._kernel_launch_count() - before > 0


@pytest.mark.parametrize("case", [
    # (M, K, N, expected tile rows, expected epilogue warps): 256-row tiles and eight-warp tiles have one staging tile
    # per epilogue warp; widths that end in a partial 64-column group are clipped by the store
    (1024, 2048, 9440, 256, 4), (1024, 2048, 9448, 256, 4), (2048, 512, 2056, 128, 8), (4096, 4096, 2304, 256, 4)])
def test_gemm_single_staging_tile_stores(case):
    M, K, N, tm, ew = case
    plan = _C._plan_gemm("bfloat16", M, N, K, 1, False, False, False, 0, True, True, 148, {})
    assert (plan["tm"], plan["epilogue_warps"]) == (tm, ew), plan
    rng = np.random.default_rng(M + N)
    a, b = rng.standard_normal((M, K)), rng.standard_normal((K, N)) * (1.0 / np.sqrt(K))
    bias, res = rng.standard_normal((N,)), rng.standard_normal((M, N))
    ta, tb = ref_round(a, "bfloat16"), ref_round(b, "bfloat16")
    xa, xb = dev_tensor(a, "bfloat16"), dev_tensor(b, "bfloat16")
    close(_C._gemm(xa, False, xb, False), ta @ tb, "bfloat16", 2)
    y = ob.linear(xa, xb, dev_tensor(bias, "bfloat16"), "none", dev_tensor(res, "bfloat16"))      # bias + residual in the epilogue
    close(y, ta @ tb + ref_round(bias, "bfloat16") + ref_round(res, "bfloat16"), "bfloat16", 2)
    g = ob.linear(xa, xb, dev_tensor(bias, "bfloat16"), "gelu")                                    # bias + GELU in the epilogue
    close(g, torch.nn.functional.gelu(ta @ tb + ref_round(bias, "bfloat16")), "bfloat16", 2)
