"""Private observations for tests and benchmarks; nothing here is part of the public API.

Memory-pool switches and counters, and route control for the two operators that have more than
one implementation on the GPU: matmul (the tcgen05 tile kernel or the SIMT kernel) and conv2d
(lowering onto the tcgen05 GEMM or the direct kernels).  Forced routes bypass the planner and are
for measurement and parity checks only.
(reference project: python/orthon/_diagnostics.py:8-39)"""
import contextlib

from . import _C

memory_pool_set_enabled = _C._memory_pool_set_enabled
memory_pool_enabled = _C._memory_pool_enabled
memory_pool_set_max_cached_bytes = _C._memory_pool_set_max_cached_bytes
memory_pool_max_cached_bytes = _C._memory_pool_max_cached_bytes
memory_pool_stats = _C._memory_pool_stats
memory_pool_reset_stats = _C._memory_pool_reset_stats
memory_pool_reset_peak = _C._memory_pool_reset_peak
memory_pool_clear_cache = _C._memory_pool_clear
memory_pool_scratch_stats = _C._scratch_pool_stats
kernel_launch_count = _C._kernel_launch_count
dispatch_kernels = _C._dispatch_kernels
dispatch_resolve = _C._dispatch_resolve


@contextlib.contextmanager
def _forced(setter, route):
    setter(route)
    try:
        yield
    finally:
        setter("auto")


def matmul_simt(a, b):
    """a @ b through the SIMT kernel (exact float32 accumulation order of the fallback)."""
    with _forced(_C._matmul_force_route, "simt"):
        return _C.matmul(a, b)


def matmul_tcgen05(a, b):
    """a @ b through the tcgen05 kernel; raises if the operands cannot take that route."""
    with _forced(_C._matmul_force_route, "tcgen05"):
        return _C.matmul(a, b)


def matmul_dispatch_path(a, b):
    """Name of the route the planner picks for a @ b (runs the product once)."""
    _C.matmul(a, b)
    return _C._matmul_last_route()


def conv2d_direct(x, w, b=None, stride=(1, 1), padding=(0, 0)):
    """conv2d through the direct kernels regardless of dtype."""
    with _forced(_C._conv2d_force_route, "direct"):
        return _C.conv2d(x, w, b, stride[0], stride[1], padding[0], padding[1])


def conv2d_dispatch_path(x, w, b=None, stride=(1, 1), padding=(0, 0)):
    _C.conv2d(x, w, b, stride[0], stride[1], padding[0], padding[1])
    return _C._conv2d_last_route()
