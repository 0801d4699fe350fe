"""Lightweight tracing: named ranges with CUDA-event device times, off unless enabled.

    enable_tracing(True)
    with trace_range("bucket 3"):
        ...
    for name, ms in collected_ranges(): ...
"""
from contextlib import contextmanager

_enabled = False
_ranges = []


def enable_tracing(on=True):
    global _enabled
    _enabled = bool(on)
    _ranges.clear()


@contextmanager
def trace_range(name, device=0):
    if not _enabled:
        yield
        return
    from .. import _C
    if _C.cuda_available():
        start = _C.CudaEvent.record(device)
        yield
        stop = _C.CudaEvent.record(device)
        _ranges.append((name, start, stop))
    else:
        import time
        t0 = time.perf_counter()
        yield
        _ranges.append((name, None, (time.perf_counter() - t0) * 1e3))


def collected_ranges():
    out = []
    for name, start, stop in _ranges:
        out.append((name, stop if start is None else stop.elapsed_ms_since(start)))
    return out
