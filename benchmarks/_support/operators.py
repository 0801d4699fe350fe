"""Operator micro-benchmark case tables, one family per function.

A case is `Case(name, shape, build)`, where `build(ctx)` returns `(fn, torch_fn_or_None,
work)`: `fn` runs the operator once through the public API, `torch_fn` the same operator in
PyTorch on the same device (comparison arm and correctness oracle), and `work` is a dict with
`bytes` and / or `flops` per call for the derived rates.  Families: matmul, conv2d, fusion,
softmax_ce, elementwise, reductions, dropout, nn, memory_pool, no_grad.
(reference project: benchmarks/_support/operators.py:17-184)
"""
import dataclasses

import numpy as np

import orthon_b200 as ob


@dataclasses.dataclass
class Context:
    device: str
    dtype: str
    quick: bool
    seed: int = 0

    def __post_init__(self):
        self.rng = np.random.default_rng(self.seed)
        try:
            import torch
            self.torch = torch
            # The comparison arm computes float32 in float32: no TF32 in its convolutions or products.
            torch.backends.cudnn.allow_tf32 = False
            torch.backends.cuda.matmul.allow_tf32 = False
        except ImportError:
            self.torch = None

    @property
    def cuda(self):
        return self.device.startswith("cuda")

    @property
    def esz(self):
        return {"float32": 4, "float64": 8, "float16": 2, "bfloat16": 2}[self.dtype]

    def array(self, *shape, scale=1.0):
        return (self.rng.standard_normal(shape) * scale).astype(np.float32)

    def tensor(self, array, grad=False, dtype=None):
        dtype = dtype or self.dtype
        if dtype in ("float16", "bfloat16") and not self.cuda:
            raise ValueError("16-bit compute runs on CUDA only")
        t = ob.from_numpy(np.ascontiguousarray(array.astype(np.float64 if dtype == "float64" else np.float32)))
        t = t.to(self.device)
        if dtype in ("float16", "bfloat16"):
            t = ob.cast(t, dtype)
        if grad:
            t.requires_grad_(True)
        return t

    def ttensor(self, array, grad=False, dtype=None):
        if self.torch is None:
            return None
        torch = self.torch
        dt = {"float32": torch.float32, "float64": torch.float64, "float16": torch.float16, "bfloat16": torch.bfloat16}[dtype or self.dtype]
        t = torch.from_numpy(np.ascontiguousarray(array)).to(self.device).to(dt)
        return t.requires_grad_(True) if grad else t


@dataclasses.dataclass
class Case:
    name: str
    shape: object
    build: object
    mode: str = "forward"
    cuda_only: bool = False
    compare: bool = True  # False where the two arms cannot agree element by element (random masks)


def _mm_cases(ctx):
    sizes = [128, 256] if ctx.quick else ([256, 512, 1024] + ([2048, 4096, 8192] if ctx.cuda else []))
    cases = []
    for n in sizes:
        def build(ctx, n=n):
            a, b = ctx.array(n, n, scale=0.05), ctx.array(n, n, scale=0.05)
            ta, tb = ctx.tensor(a), ctx.tensor(b)
            pa, pb = ctx.ttensor(a), ctx.ttensor(b)
            return (lambda: ob.matmul(ta, tb)), (None if pa is None else (lambda: pa @ pb)), {"flops": 2.0 * n ** 3}
        cases.append(Case(f"matmul_{n}", [n, n, n], build))

    def build_bwd(ctx, n=sizes[-1] if ctx.quick else 1024):
        a, b = ctx.array(n, n, scale=0.05), ctx.array(n, n, scale=0.05)
        ta, tb = ctx.tensor(a, True), ctx.tensor(b, True)
        pa, pb = ctx.ttensor(a, True), ctx.ttensor(b, True)

        def fn():
            ta.zero_grad(); tb.zero_grad()
            ob.matmul(ta, tb).sum().backward()

        def tfn():
            pa.grad = pb.grad = None
            (pa @ pb).sum().backward()
        return fn, (None if pa is None else tfn), {"flops": 6.0 * n ** 3}
    cases.append(Case("matmul_fwd_bwd", "square", build_bwd, mode="forward+backward"))

    def build_batched(ctx):
        bsz, m, k, n = (4, 64, 32, 64) if ctx.quick else (64, 256, 64, 256)
        a, b = ctx.array(bsz, m, k, scale=0.1), ctx.array(bsz, k, n, scale=0.1)
        ta, tb, pa, pb = ctx.tensor(a), ctx.tensor(b), ctx.ttensor(a), ctx.ttensor(b)
        return (lambda: ob.matmul(ta, tb)), (None if pa is None else (lambda: pa @ pb)), {"flops": 2.0 * bsz * m * k * n}
    cases.append(Case("matmul_batched", "batched", build_batched))
    return cases


def _conv_cases(ctx):
    shapes = [((2, 3, 16, 16), (8, 3, 3, 3), 1, 1)] if ctx.quick else [
        ((32, 3, 32, 32), (32, 3, 3, 3), 1, 1), ((32, 32, 32, 32), (64, 32, 3, 3), 2, 1), ((32, 64, 16, 16), (128, 64, 3, 3), 2, 1)]
    cases = []
    for xs, ws, stride, pad in shapes:
        for mode in ("forward", "forward+backward"):
            def build(ctx, xs=xs, ws=ws, stride=stride, pad=pad, mode=mode):
                x, w, b = ctx.array(*xs), ctx.array(*ws, scale=0.1), ctx.array(ws[0], scale=0.1)
                grad = mode != "forward"
                tx, tw, tb = ctx.tensor(x, grad), ctx.tensor(w, grad), ctx.tensor(b, grad)
                px, pw, pb = ctx.ttensor(x, grad), ctx.ttensor(w, grad), ctx.ttensor(b, grad)
                oh = (xs[2] + 2 * pad - ws[2]) // stride + 1
                flops = 2.0 * xs[0] * ws[0] * oh * oh * ws[1] * ws[2] * ws[3] * (3 if grad else 1)

                def fn():
                    out = ob.conv2d(tx, tw, tb, stride, stride, pad, pad)
                    if grad:
                        for t in (tx, tw, tb):
                            t.zero_grad()
                        out.sum().backward()
                    return out

                def tfn():
                    out = ctx.torch.nn.functional.conv2d(px, pw, pb, stride=stride, padding=pad)
                    if grad:
                        px.grad = pw.grad = pb.grad = None
                        out.sum().backward()
                    return out
                return fn, (None if px is None else tfn), {"flops": flops}
            cases.append(Case(f"conv2d_{xs[1]}to{ws[0]}_s{stride}", [list(xs), list(ws)], build, mode=mode))
    return cases


def _fusion_cases(ctx):
    m, k, n = (64, 64, 64) if ctx.quick else (1024, 1024, 1024)

    def build_fused(ctx):
        x, w, b = ctx.array(m, k, scale=0.1), ctx.array(k, n, scale=0.1), ctx.array(n, scale=0.1)
        tx, tw, tb, px, pw, pb = ctx.tensor(x), ctx.tensor(w), ctx.tensor(b), ctx.ttensor(x), ctx.ttensor(w), ctx.ttensor(b)
        return (lambda: ob.fused_linear_relu(tx, tw, tb)), (None if px is None else (lambda: ctx.torch.relu(px @ pw + pb))), {"flops": 2.0 * m * k * n}

    def build_composed(ctx):
        x, w, b = ctx.array(m, k, scale=0.1), ctx.array(k, n, scale=0.1), ctx.array(n, scale=0.1)
        tx, tw, tb = ctx.tensor(x), ctx.tensor(w), ctx.tensor(b)
        return (lambda: ob.relu(ob.add(ob.matmul(tx, tw), tb))), None, {"flops": 2.0 * m * k * n}
    return [Case("fused_linear_relu", [m, k, n], build_fused), Case("composed_linear_relu", [m, k, n], build_composed)]


def _softmax_ce_cases(ctx):
    rows, cols = (64, 100) if ctx.quick else (4096, 8192)

    def build_softmax(ctx):
        x = ctx.array(rows, cols)
        tx, px = ctx.tensor(x), ctx.ttensor(x)
        return (lambda: ob.softmax(tx, 1)), (None if px is None else (lambda: ctx.torch.softmax(px, 1))), {"bytes": 2.0 * rows * cols * ctx.esz}

    def build_log_softmax(ctx):
        x = ctx.array(rows, cols)
        tx, px = ctx.tensor(x), ctx.ttensor(x)
        return (lambda: ob.log_softmax(tx, 1)), (None if px is None else (lambda: ctx.torch.log_softmax(px, 1))), {"bytes": 2.0 * rows * cols * ctx.esz}

    def build_ce(ctx):
        x = ctx.array(rows, cols)
        y = ctx.rng.integers(0, cols, rows)
        tx, px = ctx.tensor(x, True), ctx.ttensor(x, True)
        ty = ob.from_numpy(y.astype(np.int64)).to(ctx.device)
        py = None if px is None else ctx.torch.from_numpy(y).to(ctx.device)

        def fn():
            tx.zero_grad()
            loss = ob.cross_entropy(tx, ty)
            loss.backward()
            return loss

        def tfn():
            px.grad = None
            loss = ctx.torch.nn.functional.cross_entropy(px.float(), py)
            loss.backward()
            return loss
        return fn, (None if px is None else tfn), {"bytes": 3.0 * rows * cols * ctx.esz}
    return [Case("softmax_rows", [rows, cols], build_softmax), Case("log_softmax_rows", [rows, cols], build_log_softmax),
            Case("cross_entropy_fwd_bwd", [rows, cols], build_ce, mode="forward+backward")]


def _elementwise_cases(ctx):
    rows, cols = (64, 256) if ctx.quick else (8192, 8192)
    n = rows * cols

    def binary(op, top, rhs_shape):
        def build(ctx):
            a, b = ctx.array(rows, cols), ctx.array(*rhs_shape)
            ta, tb, pa, pb = ctx.tensor(a), ctx.tensor(b), ctx.ttensor(a), ctx.ttensor(b)
            moved = (2 * n + int(np.prod(rhs_shape))) * ctx.esz
            return (lambda: op(ta, tb)), (None if pa is None else (lambda: top(pa, pb))), {"bytes": float(moved)}
        return build

    def unary(op, top):
        def build(ctx):
            a = ctx.array(rows, cols)
            ta, pa = ctx.tensor(a), ctx.ttensor(a)
            return (lambda: op(ta)), (None if pa is None else (lambda: top(pa))), {"bytes": 2.0 * n * ctx.esz}
        return build

    t = ctx.torch
    cases = [Case("add_same_shape", [rows, cols], binary(ob.add, (lambda a, b: a + b), (rows, cols))),
             Case("add_row_broadcast", [rows, cols], binary(ob.add, (lambda a, b: a + b), (cols,))),
             Case("mul_same_shape", [rows, cols], binary(ob.mul, (lambda a, b: a * b), (rows, cols))),
             Case("relu", [rows, cols], unary(ob.relu, (lambda a: t.relu(a)))),
             Case("gelu", [rows, cols], unary(ob.gelu, (lambda a: t.nn.functional.gelu(a)))),
             Case("tanh", [rows, cols], unary(ob.tanh, (lambda a: t.tanh(a)))),
             Case("exp", [rows, cols], unary(ob.exp, (lambda a: t.exp(a))))]
    if ctx.cuda and ctx.dtype == "float32":
        cases.append(Case("cast_f32_to_bf16", [rows, cols], unary((lambda a: ob.cast(a, "bfloat16")), (lambda a: a.to(t.bfloat16))), cuda_only=True))
    return cases


def _reduction_cases(ctx):
    rows, cols = (64, 256) if ctx.quick else (8192, 8192)

    def red(op, top):
        def build(ctx):
            a = ctx.array(rows, cols)
            ta, pa = ctx.tensor(a), ctx.ttensor(a)
            return (lambda: op(ta)), (None if pa is None else (lambda: top(pa))), {"bytes": float(rows * cols * ctx.esz)}
        return build
    return [Case("sum_all", [rows, cols], red((lambda a: a.sum()), (lambda a: a.sum()))),
            Case("sum_dim0", [rows, cols], red((lambda a: a.sum(0)), (lambda a: a.sum(0)))),
            Case("sum_dim1", [rows, cols], red((lambda a: a.sum(1)), (lambda a: a.sum(1)))),
            Case("mean_dim1", [rows, cols], red((lambda a: a.mean(1)), (lambda a: a.mean(1)))),
            Case("max_dim1", [rows, cols], red((lambda a: a.max(1)), (lambda a: a.max(1).values))),
            Case("argmax_dim1", [rows, cols], red((lambda a: a.argmax(1)), (lambda a: a.argmax(1))))]


def _dropout_cases(ctx):
    n = 4096 if ctx.quick else 1 << 24

    def build(ctx):
        a = ctx.array(n)
        ta, pa = ctx.tensor(a, dtype="float32"), ctx.ttensor(a, dtype="float32")
        return (lambda: ob.dropout(ta, 0.1, 1234)), (None if pa is None else (lambda: ctx.torch.nn.functional.dropout(pa, 0.1))), {"bytes": 8.0 * n}
    return [Case("dropout_p0.1", [n], build, compare=False)]


def _nn_cases(ctx):
    rows, width = (32, 64) if ctx.quick else (8192, 2048)
    t = ctx.torch

    def build_ln(ctx):
        x, g, b = ctx.array(rows, width), ctx.array(width), ctx.array(width)
        tx, tg, tb, px, pg, pb = ctx.tensor(x), ctx.tensor(g), ctx.tensor(b), ctx.ttensor(x), ctx.ttensor(g), ctx.ttensor(b)
        return (lambda: ob.layer_norm(tx, [width], tg, tb, 1e-5)), (None if px is None else (lambda: t.nn.functional.layer_norm(px, (width,), pg, pb, 1e-5))), {"bytes": 2.0 * rows * width * ctx.esz}

    def build_emb(ctx):
        vocab = 512 if ctx.quick else 32000
        w = ctx.array(vocab, width)
        idx = ctx.rng.integers(0, vocab, rows)
        tw, pw = ctx.tensor(w), ctx.ttensor(w)
        ti = ob.from_numpy(idx.astype(np.int64)).to(ctx.device)
        pi = None if pw is None else t.from_numpy(idx).to(ctx.device)
        return (lambda: ob.embedding(ti, tw)), (None if pw is None else (lambda: t.nn.functional.embedding(pi, pw))), {"bytes": 2.0 * rows * width * ctx.esz}

    def build_attn(ctx):
        b, h, s, d = (1, 2, 32, 16) if ctx.quick else (4, 16, 1024, 128)
        q, k, v = (ctx.array(b * h, s, d, scale=0.5) for _ in range(3))
        tq, tk, tv = ctx.tensor(q), ctx.tensor(k), ctx.tensor(v)
        pq, pk, pv = ctx.ttensor(q), ctx.ttensor(k), ctx.ttensor(v)
        return (lambda: ob.scaled_dot_product_attention(tq, tk, tv)), (None if pq is None else (lambda: t.nn.functional.scaled_dot_product_attention(pq, pk, pv))), {"flops": 4.0 * b * h * s * s * d}
    return [Case("layer_norm", [rows, width], build_ln), Case("embedding_gather", [rows, width], build_emb),
            Case("attention_unfused_api", "b,h,s,d", build_attn)]


def _memory_pool_cases(ctx):
    n = 1 << 12 if ctx.quick else 1 << 20

    def build(enabled):
        def inner(ctx):
            def fn():
                was = ob._C._memory_pool_enabled()
                ob._C._memory_pool_set_enabled(enabled)
                try:
                    for _ in range(8):
                        ob.zeros([n]).to(ctx.device)
                finally:
                    ob._C._memory_pool_set_enabled(was)
            return fn, None, {}
        return inner
    return [Case("alloc_cycle_pool_on", [8, n], build(True)), Case("alloc_cycle_pool_off", [8, n], build(False))]


def _no_grad_cases(ctx):
    width = 64 if ctx.quick else 1024

    def build(grad):
        def inner(ctx):
            x = ctx.tensor(ctx.array(128, width))
            ws = [ctx.tensor(ctx.array(width, width, scale=0.03), True) for _ in range(4)]

            def forward():
                h = x
                for w in ws:
                    h = ob.relu(ob.matmul(h, w))
                return h

            def fn():
                if grad:
                    return forward()
                with ob.no_grad():
                    return forward()
            return fn, None, {"flops": 8.0 * 128 * width * width}
        return inner
    return [Case("mlp_forward_grad_mode", [128, width], build(True)), Case("mlp_forward_no_grad", [128, width], build(False))]


FAMILIES = {"matmul": _mm_cases, "conv2d": _conv_cases, "fusion": _fusion_cases, "softmax_ce": _softmax_ce_cases,
            "elementwise": _elementwise_cases, "reductions": _reduction_cases, "dropout": _dropout_cases, "nn": _nn_cases,
            "memory_pool": _memory_pool_cases, "no_grad": _no_grad_cases}


def to_numpy(value):
    """Result of either arm as a float64 array (None when it is not a tensor)."""
    if isinstance(value, ob.Tensor):
        t = value
        if t.dtype in ("float16", "bfloat16"):
            t = ob.cast(t, "float32")
        return np.asarray(t.to("cpu").tolist(), dtype=np.float64).reshape(t.shape)
    if hasattr(value, "detach"):
        return value.detach().double().cpu().numpy()
    return None


TOLERANCE = {"float64": 1e-10, "float32": 2e-4, "float16": 2e-2, "bfloat16": 8e-2}


def check(ours, theirs, dtype):
    """'matched' / 'mismatch(<max relative error>)' / 'not-compared'."""
    a, b = to_numpy(ours), to_numpy(theirs)
    if a is None or b is None or a.size != b.size:
        return "not-compared"
    b = b.reshape(a.shape)
    scale = max(1.0, float(np.abs(b).max()))
    err = float(np.abs(a - b).max()) / scale
    return "matched" if err <= TOLERANCE[dtype] else f"mismatch({err:.2e})"
