"""Lightweight tracing: named ranges with CUDA-event device times, off unless enabled.

    enable_tracing(True)                 # or ORTHON_TRACE=1 in the environment
    with trace_range("bucket 3", device, stream_kind=1):
        ...
    for name, ms in collected_ranges(): ...
    for name, stream, start_ms, end_ms in timeline(): ...   # offsets from the first recorded event

The reducers wrap every bucket launch (communication stream) and the optimizers every step in a
range, so with tracing on a training step yields a timeline that shows which reductions ran
beside the backward pass and which were left for its tail.  Ranges cost two event records each and
nothing when tracing is off.  With ORTHON_NVTX=1 every range is also an NVTX range on the calling
thread, for a profiler that is attached to the process (no events are recorded for that alone).
"""
import os
from contextlib import contextmanager

_enabled = os.environ.get("ORTHON_TRACE", "0") not in ("", "0")
_nvtx = os.environ.get("ORTHON_NVTX", "0") not in ("", "0")
_ranges = []


def enable_tracing(on=True):
    global _enabled
    _enabled = bool(on)
    _ranges.clear()


def tracing_enabled():
    return _enabled


@contextmanager
def trace_range(name, device=0, stream_kind=0):
    if _nvtx:
        from .. import _C
        _C._nvtx_push(str(name))
        try:
            with _event_range(name, device, stream_kind):
                yield
        finally:
            _C._nvtx_pop()
    else:
        with _event_range(name, device, stream_kind):
            yield


@contextmanager
def _event_range(name, device, stream_kind):
    if not _enabled:
        yield
        return
    from .. import _C
    if _C.cuda_available():
        start = _C.CudaEvent.record(device, stream_kind)
        try:
            yield
        finally:
            _ranges.append((name, stream_kind, start, _C.CudaEvent.record(device, stream_kind)))
    else:
        import time
        t0 = time.perf_counter()
        try:
            yield
        finally:
            _ranges.append((name, stream_kind, None, (time.perf_counter() - t0) * 1e3))


def collected_ranges():
    """(name, duration in ms) of every finished range, in completion order."""
    out = []
    for name, _, start, stop in _ranges:
        out.append((name, stop if start is None else stop.elapsed_ms_since(start)))
    return out


def timeline():
    """(name, stream kind, start ms, end ms) relative to the earliest recorded range start.
    Waits for the device."""
    rows = [r for r in _ranges if r[2] is not None]
    if not rows:
        return []
    for _, _, _, stop in rows:
        stop.synchronize()
    base = rows[0][2]
    offsets = [(name, kind, start.elapsed_ms_since(base), stop.elapsed_ms_since(base)) for name, kind, start, stop in rows]
    shift = min(o[2] for o in offsets)
    return [(name, kind, a - shift, b - shift) for name, kind, a, b in offsets]


def clear_ranges():
    _ranges.clear()
