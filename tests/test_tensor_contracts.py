"""Tensor contracts checked case by case against NumPy on the CPU backend: all 81 cast pairs,
broadcasting, reductions with the extrema policy, slices and integer indexing (values, aliasing
and gradients), scalar arithmetic in every operand order, shape operations and versioning.
(reference project: tests/spec/tensor/*, tests/python/test_cast.py, test_slice_autograd.py,
test_index_autograd.py, test_scalar_arithmetic.py, test_max_argmax.py, test_inplace_versioning.py)"""
import itertools

import numpy as np
import pytest

import orthon_b200 as ob

DTYPES = ["float32", "float64", "float16", "bfloat16", "int32", "int64", "uint8", "int8", "bool"]
NP = {"float32": np.float32, "float64": np.float64, "float16": np.float16, "int32": np.int32, "int64": np.int64,
      "uint8": np.uint8, "int8": np.int8, "bool": np.bool_}


def T(a, dtype=None, grad=False):
    x = ob.from_numpy(np.asarray(a, dtype=np.float32), dtype)
    if grad:
        x.requires_grad_(True)
    return x


def arr(t):
    return np.asarray(t.tolist(), dtype=np.float64).reshape(t.shape)


def _bf16(values):
    """float32 -> bfloat16 -> float32 with round-to-nearest-even, by bit arithmetic."""
    bits = np.asarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32)


# ------------------------------------------------------------------------ cast
@pytest.mark.parametrize("src,dst", list(itertools.product(DTYPES, DTYPES)))
def test_cast_pair(src, dst):
    # Values every dtype can hold exactly after the first conversion (bool collapses to 0 / 1).
    base = np.array([0.0, 1.0, 2.0, 3.0, 100.0, 0.0, 7.0, 1.0], dtype=np.float32)
    first = ob.cast(ob.from_numpy(base), src)
    out = ob.cast(first, dst)
    assert out.dtype == dst and out.shape == first.shape
    expect = (base != 0).astype(np.float32) if src == "bool" else base
    expect = (expect != 0).astype(np.float32) if dst == "bool" else expect
    assert ob.cast(out, "float32").tolist() == expect.tolist()
    if src == dst:
        assert out._impl_id == first._impl_id          # a same-dtype cast of a contiguous tensor is the same value
    else:
        assert out._buffer_id != first._buffer_id


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("value", [1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65504.0, 1e-8, -0.0, 3.14159265, 1e5, float("inf"), -float("inf")])
def test_low_precision_rounding_is_nearest_even(dtype, value):
    got = ob.cast(ob.cast(T([value]), dtype), "float32").tolist()[0]
    with np.errstate(over="ignore"):
        want = float(np.float32(value).astype(np.float16)) if dtype == "float16" else float(_bf16([value])[0])
    assert got == want or (np.isnan(got) and np.isnan(want))
    assert np.signbit(got) == np.signbit(want)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32", "float64"])
def test_nan_survives_casts(dtype):
    x = ob.cast(T([float("nan"), 1.0]), dtype)
    back = ob.cast(x, "float64").tolist()
    assert np.isnan(back[0]) and back[1] == 1.0
    assert not ob.isfinite_all(x)


# ---------------------------------------------------------------- broadcasting
SHAPES = [((3, 4), (3, 4)), ((3, 4), (4,)), ((3, 4), (1, 4)), ((3, 4), (3, 1)), ((3, 1), (1, 4)), ((2, 3, 4), (3, 4)),
          ((2, 3, 4), (2, 1, 4)), ((1,), (5,)), ((5,), (1,)), ((2, 1, 1), (1, 3, 1)), ((0, 3), (1, 3)), ((4, 1), (0,) + ())]


@pytest.mark.parametrize("op", ["add", "mul", "sub", "div"])
@pytest.mark.parametrize("sa,sb", SHAPES[:-1])
def test_broadcast_binary_matches_numpy(op, sa, sb):
    rng = np.random.default_rng(hash((op, sa, sb)) % 2 ** 32)
    a, b = rng.uniform(0.5, 2.0, sa).astype(np.float32), rng.uniform(0.5, 2.0, sb).astype(np.float32)
    got = getattr(ob, op)(T(a), T(b))
    want = {"add": np.add, "mul": np.multiply, "sub": np.subtract, "div": np.divide}[op](a, b)
    assert got.shape == want.shape
    assert np.allclose(arr(got), want, rtol=1e-6)


@pytest.mark.parametrize("sa,sb", [((3, 4), (3,)), ((2, 3), (3, 2)), ((2, 3, 4), (2, 4)), ((5,), (4,))])
def test_incompatible_shapes_are_rejected(sa, sb):
    with pytest.raises(Exception):
        ob.add(T(np.zeros(sa)), T(np.zeros(sb)))


@pytest.mark.parametrize("sa,sb", SHAPES[:10])
def test_broadcast_gradients_reduce_back_to_the_operand_shape(sa, sb):
    rng = np.random.default_rng(5)
    a, b = T(rng.standard_normal(sa), grad=True), T(rng.standard_normal(sb), grad=True)
    (a * b).sum().backward()
    ga = np.broadcast_to(arr(b), np.broadcast_shapes(sa, sb))
    gb = np.broadcast_to(arr(a), np.broadcast_shapes(sa, sb))

    def unbroadcast(g, shape):
        while g.ndim > len(shape):
            g = g.sum(0)
        for i, n in enumerate(shape):
            if n == 1 and g.shape[i] != 1:
                g = g.sum(i, keepdims=True)
        return g

    assert a.grad.shape == tuple(sa) and b.grad.shape == tuple(sb)
    assert np.allclose(arr(a.grad), unbroadcast(ga, sa), atol=1e-5)
    assert np.allclose(arr(b.grad), unbroadcast(gb, sb), atol=1e-5)


# ------------------------------------------------------------------ reductions
@pytest.mark.parametrize("shape", [(5,), (3, 4), (2, 3, 4), (1, 6), (4, 1, 2)])
@pytest.mark.parametrize("op", ["sum", "mean", "max", "argmax"])
@pytest.mark.parametrize("keepdim", [False, True])
def test_reduce_every_dim(shape, op, keepdim):
    rng = np.random.default_rng(len(shape) * 17)
    a = rng.permutation(int(np.prod(shape))).reshape(shape).astype(np.float32)  # distinct values: argmax is unambiguous
    x = T(a)
    for dim in [None] + list(range(-len(shape), len(shape))):
        got = getattr(x, op)(dim, keepdim) if dim is not None else getattr(x, op)(None, keepdim)
        if op == "argmax":
            want = np.argmax(a) if dim is None else np.argmax(a, axis=dim)
            if keepdim:
                want = np.asarray(want).reshape([1] * len(shape)) if dim is None else np.expand_dims(want, dim)
            assert got.dtype == "int64"
        else:
            fn = {"sum": np.sum, "mean": np.mean, "max": np.max}[op]
            want = fn(a, axis=dim, keepdims=keepdim)
        want = np.asarray(want, dtype=np.float64)
        if want.ndim == 0:
            want = want.reshape([1] * (len(shape) if keepdim else 1)) if keepdim else want.reshape([1])
        assert tuple(got.shape) == want.shape, (dim, got.shape, want.shape)
        assert np.allclose(arr(got), want, rtol=1e-6)


@pytest.mark.parametrize("values,index", [([1.0, 5.0, 5.0, 2.0], 1), ([float("nan"), 9.0], 0), ([3.0, float("nan"), float("nan")], 1),
                                          ([-np.inf, -np.inf], 0), ([2.0, np.inf, np.inf], 1), ([7.0], 0)])
def test_extrema_policy_first_maximum_and_first_nan_win(values, index):
    x = T(values)
    assert x.argmax().tolist() == [index]
    top = x.max().tolist()[0]
    assert (np.isnan(top) and np.isnan(values[index])) or top == values[index]


@pytest.mark.parametrize("shape,dim", [((3, 4), 0), ((3, 4), 1), ((2, 3, 4), 1), ((2, 3, 4), None)])
def test_max_backward_routes_the_gradient_to_the_first_maximum(shape, dim):
    a = np.zeros(shape, dtype=np.float32)
    a[...] = 1.0                                         # all equal: the first index along the reduced extent wins
    x = T(a, grad=True)
    x.max(dim).sum().backward()
    g = arr(x.grad)
    if dim is None:
        want = np.zeros(shape)
        want.reshape(-1)[0] = 1.0
    else:
        want = np.zeros(shape)
        index = [slice(None)] * len(shape)
        index[dim] = 0
        want[tuple(index)] = 1.0
    assert np.array_equal(g, want)


def test_reductions_of_empty_tensors_are_rejected():
    for op in ("sum", "mean", "max", "argmax"):
        with pytest.raises(Exception):
            getattr(ob.zeros([0, 3]), op)()


# ------------------------------------------------------------- slice and index
SLICES = [((6,), 0, 0, 6), ((6,), 0, 2, 5), ((6,), 0, 5, 6), ((6,), 0, 3, 3), ((4, 5), 0, 1, 3), ((4, 5), 1, 0, 2),
          ((4, 5), 1, 4, 5), ((4, 5), -1, 1, 4), ((2, 3, 4), 1, 1, 3), ((2, 3, 4), 2, 0, 1), ((2, 3, 4), -3, 1, 2),
          ((2, 3, 4), 0, 0, 2)]


@pytest.mark.parametrize("shape,dim,start,end", SLICES)
def test_slice_is_a_view_with_the_expected_values(shape, dim, start, end):
    a = np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)
    x = T(a)
    s = x.slice(dim, start, end)
    index = [slice(None)] * len(shape)
    index[dim] = slice(start, end)
    want = a[tuple(index)]
    assert tuple(s.shape) == want.shape
    assert np.array_equal(arr(s), want)
    assert s._buffer_id == x._buffer_id
    if want.size:
        s.fill_(-1.0)                                    # writes through to the base
        a[tuple(index)] = -1.0
        assert np.array_equal(arr(x), a)


@pytest.mark.parametrize("shape,dim,start,end", SLICES)
def test_slice_backward_scatters_into_zeros(shape, dim, start, end):
    x = T(np.arange(int(np.prod(shape))).reshape(shape), grad=True)
    s = x.slice(dim, start, end)
    if s.numel == 0:
        pytest.skip("an empty slice has nothing to differentiate")
    (s * s).sum().backward()
    a = arr(x.detach())
    want = np.zeros(shape)
    index = [slice(None)] * len(shape)
    index[dim] = slice(start, end)
    want[tuple(index)] = 2 * a[tuple(index)]
    assert np.array_equal(arr(x.grad), want)


@pytest.mark.parametrize("shape,dim,start,end", [((4,), 0, -1, 2), ((4,), 0, 3, 2), ((4,), 0, 0, 5), ((4,), 1, 0, 1), ((4,), -2, 0, 1),
                                                  ((2, 3), 2, 0, 1)])
def test_invalid_slices_are_rejected(shape, dim, start, end):
    with pytest.raises(Exception):
        T(np.zeros(shape)).slice(dim, start, end)


def test_overlapping_slices_accumulate_their_gradients():
    x = T(np.arange(6.0), grad=True)
    (x.slice(0, 0, 4).sum() + x.slice(0, 2, 6).sum() * 3.0).backward()
    assert x.grad.tolist() == [1.0, 1.0, 4.0, 4.0, 3.0, 3.0]


@pytest.mark.parametrize("shape,indices", [((5,), (2,)), ((5,), (-1,)), ((3, 4), (1,)), ((3, 4), (2, 3)), ((3, 4), (-1, -4)),
                                            ((2, 3, 4), (1,)), ((2, 3, 4), (1, 2)), ((2, 3, 4), (0, 1, 3)), ((2, 3, 4), (-2, -3, -4))])
def test_integer_indexing_values_views_and_gradients(shape, indices):
    a = np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)
    x = T(a, grad=True)
    v = x
    for i in indices:
        v = v[i]
    want = a[indices]
    assert np.array_equal(arr(v).reshape(np.shape(want)), want)
    assert v._buffer_id == x._buffer_id
    (v * 2.0).sum().backward()
    g = np.zeros(shape)
    g[indices] = 2.0
    assert np.array_equal(arr(x.grad), g)


@pytest.mark.parametrize("shape,index", [((3,), 3), ((3,), -4), ((2, 3), 2)])
def test_out_of_range_index_is_rejected(shape, index):
    with pytest.raises(Exception):
        T(np.zeros(shape))[index]


# ----------------------------------------------------------- scalar arithmetic
@pytest.mark.parametrize("dtype", ["float32", "float64"])
@pytest.mark.parametrize("form", ["t+s", "s+t", "t-s", "s-t", "t*s", "s*t", "t/s", "s/t", "-t"])
def test_scalar_forms_value_and_gradient(dtype, form):
    a = np.array([[1.0, 2.0], [4.0, 8.0]], dtype=np.float64)
    x = ob.cast(T(a), dtype)
    x.requires_grad_(True)
    s = 2.5
    y = {"t+s": lambda: x + s, "s+t": lambda: s + x, "t-s": lambda: x - s, "s-t": lambda: s - x, "t*s": lambda: x * s,
         "s*t": lambda: s * x, "t/s": lambda: x / s, "s/t": lambda: s / x, "-t": lambda: -x}[form]()
    want = {"t+s": a + s, "s+t": s + a, "t-s": a - s, "s-t": s - a, "t*s": a * s, "s*t": s * a, "t/s": a / s, "s/t": s / a,
            "-t": -a}[form]
    grad = {"t+s": 1 + 0 * a, "s+t": 1 + 0 * a, "t-s": 1 + 0 * a, "s-t": -1 + 0 * a, "t*s": s + 0 * a, "s*t": s + 0 * a,
            "t/s": 1 / s + 0 * a, "s/t": -s / a ** 2, "-t": -1 + 0 * a}[form]
    assert y.dtype == dtype
    assert np.allclose(arr(y), want, rtol=1e-6)
    y.sum().backward()
    assert x.grad.dtype == dtype
    assert np.allclose(arr(x.grad), grad, rtol=1e-5)


@pytest.mark.parametrize("other", ["text", None, [1.0, 2.0], object(), np.ones(2, dtype=np.float32), True, np.float32(1.5), np.int64(4)])
def test_foreign_operands_are_not_coerced(other):
    x = T([1.0, 2.0])
    for op in (lambda: x + other, lambda: other + x, lambda: x * other, lambda: other * x, lambda: x - other, lambda: x / other):
        with pytest.raises(TypeError):
            op()


@pytest.mark.parametrize("value", [3, 2.5, np.float64(1.5), -0.0, 10 ** 6])
def test_python_numbers_are_accepted_as_scalars(value):
    x = T([1.0, 2.0])
    assert np.allclose(arr(x * value), np.array([1.0, 2.0]) * float(value))
    assert np.allclose(arr(value + x), np.array([1.0, 2.0]) + float(value))


# --------------------------------------------------------------- shape changes
@pytest.mark.parametrize("shape,d0,d1", [((2, 3), 0, 1), ((2, 3), 1, 0), ((2, 3, 4), 0, 2), ((2, 3, 4), -1, -2), ((2, 3, 4), 1, 1),
                                          ((5,), 0, 0)])
def test_transpose_is_a_view_and_round_trips_gradients(shape, d0, d1):
    a = np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)
    x = T(a, grad=True)
    y = x.transpose(d0, d1)
    assert np.array_equal(arr(y), np.swapaxes(a, d0, d1)) and y._buffer_id == x._buffer_id
    w = np.arange(y.numel, dtype=np.float32).reshape(y.shape)
    (y * T(w)).sum().backward()
    assert np.array_equal(arr(x.grad), np.swapaxes(w, d0, d1))


@pytest.mark.parametrize("shape,new", [((6,), (2, 3)), ((2, 3), (3, 2)), ((2, 3), (-1,)), ((2, 3, 4), (6, -1)), ((2, 3, 4), (2, -1, 2)),
                                        ((1,), ()), ((0, 3), (3, 0))])
def test_reshape_infers_one_extent_and_shares_storage(shape, new):
    a = np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)
    x = T(a)
    y = x.reshape(list(new))
    assert np.array_equal(arr(y), a.reshape(new))
    assert y._buffer_id == x._buffer_id


@pytest.mark.parametrize("shape,new", [((6,), (4,)), ((6,), (-1, -1)), ((6,), (4, -1)), ((0,), (-1, 0))])
def test_impossible_reshapes_are_rejected(shape, new):
    with pytest.raises(Exception):
        T(np.zeros(shape)).reshape(list(new))


@pytest.mark.parametrize("shape,start,end,want", [((2, 3, 4), 0, -1, (24,)), ((2, 3, 4), 1, 2, (2, 12)), ((2, 3, 4), 0, 1, (6, 4)),
                                                   ((2, 3, 4), 2, 2, (2, 3, 4)), ((5,), 0, 0, (5,))])
def test_flatten_ranges(shape, start, end, want):
    assert T(np.zeros(shape)).flatten(start, end).shape == want


# ------------------------------------------------------------------ versioning
WRITES = {
    "fill_": lambda t: t.fill_(2.0),
    "add_": lambda t: t.add_(T(np.ones(t.shape)), alpha=2.0),
    "mul_": lambda t: t.mul_(3.0),
    "set_item": lambda t: t.set_item(0, 9.0),
    "_copy_data_": lambda t: t._copy_data_(T(np.zeros(t.shape))),
    "_copy_flat_range_from": lambda t: t._copy_flat_range_from(0, T(np.zeros(2)), 0, 2),
    "same value fill": lambda t: t.fill_(t.tolist()[0]),
}


@pytest.mark.parametrize("name", sorted(WRITES))
def test_every_logical_write_bumps_the_buffer_version_once(name):
    t = T(np.ones(4))
    view = t.reshape([2, 2])
    before = t._storage_version
    WRITES[name](t)
    assert t._storage_version == before + 1
    assert view._storage_version == t._storage_version   # aliases share the generation


@pytest.mark.parametrize("name", sorted(WRITES))
def test_a_write_after_saving_invalidates_backward(name):
    x = T(np.ones(4) * 2.0, grad=True)
    y = (x * x).sum()                                    # MulNode saved x
    with ob.no_grad():
        WRITES[name](x)
    with pytest.raises(RuntimeError, match="modified in-place after it was saved"):
        y.backward()
    assert x.grad is None                                # nothing was committed


@pytest.mark.parametrize("op", ["reshape", "transpose", "slice", "contiguous", "detach", "index"])
def test_metadata_operations_never_bump_the_version(op):
    t = T(np.arange(6.0).reshape(2, 3))
    before = t._storage_version
    {"reshape": lambda: t.reshape([3, 2]), "transpose": lambda: t.transpose(0, 1), "slice": lambda: t.slice(1, 0, 2),
     "contiguous": lambda: t.contiguous(), "detach": lambda: t.detach(), "index": lambda: t[1]}[op]()
    assert t._storage_version == before
