"""Wall-clock and device timers shared by the benchmark scripts.

Host timer (`measure`, `measure_pair`): warm-up calls, then an inner repeat count chosen so that
one sample lasts about `target_ms` (capped by `cap_ms`), then `samples` samples; two
implementations are sampled alternately (A B A B ...) so that drift hits both.  Each sample
ends with `sync()` (a device synchronisation for CUDA work, nothing for the CPU).  Reported:
median, quartiles and inter-quartile range of the per-call time in milliseconds.
(reference project: benchmarks/_support/timing.py:8-137 - 25 warm-up calls, 11 samples, 40 ms
target, 500 ms cap)

Device timer (`measure_device`): CUDA events on the launching stream around every call, an L2
flush before each timed call, warm-up first.
"""
import dataclasses
import statistics
import time


@dataclasses.dataclass(frozen=True)
class TimingConfig:
    warmup: int = 25
    samples: int = 11
    target_ms: float = 40.0
    cap_ms: float = 500.0

    def __post_init__(self):
        if self.warmup < 0 or self.samples < 1 or self.target_ms <= 0 or self.cap_ms < self.target_ms:
            raise ValueError("invalid timing configuration")

    @staticmethod
    def quick():
        return TimingConfig(warmup=3, samples=3, target_ms=5.0, cap_ms=50.0)


def quartiles(values):
    """Median-of-halves quartiles (the median itself excluded from both halves when n is odd)."""
    ordered = sorted(values)
    n = len(ordered)
    if n == 1:
        return ordered[0], ordered[0], ordered[0]
    half = n // 2
    lower, upper = ordered[:half], ordered[half + (n % 2):]
    return statistics.median(lower), statistics.median(ordered), statistics.median(upper)


@dataclasses.dataclass(frozen=True)
class Statistics:
    samples_ms: tuple
    inner: int

    def as_dict(self):
        q1, med, q3 = quartiles(self.samples_ms)
        return {"median": med, "q1": q1, "q3": q3, "iqr": q3 - q1, "min": min(self.samples_ms), "max": max(self.samples_ms),
                "samples": len(self.samples_ms), "inner": self.inner, "units": "ms"}

    @property
    def median(self):
        return statistics.median(self.samples_ms)


def _batch_ms(fn, inner, sync):
    sync()
    start = time.perf_counter()
    for _ in range(inner):
        fn()
    sync()
    return (time.perf_counter() - start) * 1e3 / inner


def _estimate_ms(fn, sync, trials=3):
    return min(_batch_ms(fn, 1, sync) for _ in range(trials))


def choose_inner(estimate_ms, config):
    """Repeat count so that one sample lasts about target_ms and never more than cap_ms."""
    if estimate_ms <= 0:
        return 1000
    inner = max(1, int(config.target_ms / estimate_ms))
    while inner > 1 and inner * estimate_ms > config.cap_ms:
        inner //= 2
    return min(inner, 100000)


def measure(fn, sync=lambda: None, config=TimingConfig()):
    for _ in range(config.warmup):
        fn()
    sync()
    inner = choose_inner(_estimate_ms(fn, sync), config)
    return Statistics(tuple(_batch_ms(fn, inner, sync) for _ in range(config.samples)), inner)


def measure_pair(fn_a, fn_b, sync_a=lambda: None, sync_b=lambda: None, config=TimingConfig()):
    """Both callables with the same inner count, sampled alternately."""
    for _ in range(config.warmup):
        fn_a()
        fn_b()
    sync_a()
    sync_b()
    inner = choose_inner(max(_estimate_ms(fn_a, sync_a), _estimate_ms(fn_b, sync_b)), config)
    a, b = [], []
    for _ in range(config.samples):
        a.append(_batch_ms(fn_a, inner, sync_a))
        b.append(_batch_ms(fn_b, inner, sync_b))
    return Statistics(tuple(a), inner), Statistics(tuple(b), inner)


def comparison(stats_a, stats_b):
    """Ratio of medians and a verdict that only claims a difference when the inter-quartile
    ranges do not overlap."""
    da, db = stats_a.as_dict(), stats_b.as_dict()
    ratio = da["median"] / db["median"] if db["median"] > 0 else float("inf")
    if da["q3"] < db["q1"]:
        verdict = "a-faster"
    elif db["q3"] < da["q1"]:
        verdict = "b-faster"
    else:
        verdict = "indistinguishable"
    return {"ratio_a_over_b": ratio, "verdict": verdict}


def measure_device(fn, device=0, warmup=5, iters=20, flush_l2=True):
    """Per-call device time from CUDA events on the launching stream."""
    from orthon_b200 import _C

    for _ in range(warmup):
        fn()
    _C.cuda_synchronize()
    samples = []
    for _ in range(iters):
        if flush_l2:
            _C._flush_l2(device)
        start = _C.CudaEvent.record(device)
        fn()
        stop = _C.CudaEvent.record(device)
        samples.append(stop.elapsed_ms_since(start))
    _C.cuda_synchronize()
    return Statistics(tuple(samples), 1)


def time_cuda(fn, warmup=5, iters=20, flush_l2=True, device=0):
    """`measure_device` as a plain dict of milliseconds (median, min, max, sample count)."""
    stats = measure_device(fn, device=device, warmup=warmup, iters=iters, flush_l2=flush_l2)
    return {"median_ms": stats.median, "min_ms": min(stats.samples_ms), "max_ms": max(stats.samples_ms), "samples": len(stats.samples_ms)}
