"""The allocation-free sum entry point, called the way its intended users call it: through
the exported C symbol with raw device pointers.

Those users are hosts that cannot call cudaMalloc at that moment (their own stream capture is
open, or they run under a fixed device-memory budget), so the entry point keeps its block
partials in a static device array.  The check: its result equals the regular `sum` operator's
(which draws scratch from the caching pool) within the float32 reduction tolerance used by the
other reduction tests, on two consecutive calls with different sizes, so that partials left in
the shared array by the first call cannot leak into the second.  Also: oversize requests are
refused with a message, and nothing is allocated from the library's pool by the calls.

Named test_zz_* so it is collected last: if it fails under `-x`, every other test has run.
"""
import ctypes

import numpy as np
import pytest

from orthon_b200 import _C

pytestmark = pytest.mark.gpu

MAX_ELEMENTS = 1 << 30


def _entry():
    lib = ctypes.CDLL(_C.__file__)
    fn = lib.orthon_sum_f32_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_ulong]
    return fn


def _call(fn, x, out):
    err = ctypes.create_string_buffer(256)
    stream = _C._cuda_stream_handle(0)  # same stream as the tensors' producers and readers
    code = fn(x._data_ptr, int(x.numel), out._data_ptr, stream, err, 256)
    return code, err.value.decode()


def test_no_alloc_sum_matches_pool_backed_sum_twice():
    fn = _entry()
    rng = np.random.default_rng(42)
    out = _C._empty_on([1], "float32", "cuda:0")
    for n in (3_000_003, 70_001):  # two calls in a row; the second uses fewer scratch slots
        host = rng.standard_normal(n).astype(np.float32)
        x = _C.from_numpy(host).to("cuda:0")
        expected = x.sum().tolist()[0]  # existing entry point (scratch from the pool)
        before = _C._memory_pool_stats()["total_requests"]
        code, message = _call(fn, x, out)
        after = _C._memory_pool_stats()["total_requests"]
        assert code == 0, message
        assert after == before, "the allocation-free entry point touched the memory pool"
        got = out.tolist()[0]
        scale = max(1.0, float(np.abs(host).sum()))
        assert abs(got - expected) <= 2e-5 * 50 * max(1.0, abs(expected)) + 1e-7 * scale, (n, got, expected)
        assert abs(got - float(host.astype(np.float64).sum())) <= 1e-6 * scale


def test_no_alloc_sum_edge_cases():
    """The branches the main test does not reach: an input that is not 16-byte aligned (element
    by element instead of four at a time), an empty input, and a size large enough that the
    number of partials hits its ceiling of 1024 and every block walks several chunks."""
    fn = _entry()
    rng = np.random.default_rng(7)
    out = _C._empty_on([1], "float32", "cuda:0")
    host = rng.standard_normal(100_001).astype(np.float32)
    x = _C.from_numpy(host).to("cuda:0")
    shifted = _C._view_flat(x, 1, [100_000])                 # starts 4 bytes past a 16-byte boundary
    assert shifted._data_ptr % 16 == 4
    code, message = _call(fn, shifted, out)
    assert code == 0, message
    want = float(host[1:].astype(np.float64).sum())
    assert abs(out.tolist()[0] - want) <= 1e-6 * float(np.abs(host).sum())
    err = ctypes.create_string_buffer(256)
    out.fill_(5.0)
    code = fn(x._data_ptr, 0, out._data_ptr, _C._cuda_stream_handle(0), err, 256)   # n = 0: the sum of nothing
    assert code == 0 and out.tolist()[0] == 0.0
    n = 4096 * 1024 * 2 + 13                                   # more than 1024 chunks of 4096 elements
    big = rng.standard_normal(n).astype(np.float32)
    xb = _C.from_numpy(big).to("cuda:0")
    code, message = _call(fn, xb, out)
    assert code == 0, message
    assert abs(out.tolist()[0] - float(big.astype(np.float64).sum())) <= 1e-6 * float(np.abs(big).sum())


def test_no_alloc_sum_rejects_bad_requests():
    fn = _entry()
    out = _C._empty_on([1], "float32", "cuda:0")
    x = _C._zeros_on([16], "float32", "cuda:0")
    err = ctypes.create_string_buffer(256)
    code = fn(x._data_ptr, MAX_ELEMENTS + 1, out._data_ptr, _C._cuda_stream_handle(0), err, 256)
    assert code == 2 and b"exceed" in err.value
    code = fn(x._data_ptr, -1, out._data_ptr, _C._cuda_stream_handle(0), err, 256)
    assert code == 1
    code = fn(None, 4, out._data_ptr, _C._cuda_stream_handle(0), err, 256)
    assert code == 1
    code, message = _call(fn, x, out)  # still usable afterwards
    assert code == 0 and out.tolist()[0] == 0.0
