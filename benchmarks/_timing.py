"""Device timing helpers shared by the benchmark scripts: CUDA events on the launching
stream, warm-up iterations first, an L2 flush between timed iterations, median of samples."""
import statistics

import orthon_b200 as ob
from orthon_b200 import _C


def time_cuda(fn, warmup=5, iters=20, flush_l2=True, device=0):
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
    return {"median_ms": statistics.median(samples), "min_ms": min(samples), "max_ms": max(samples), "samples": len(samples)}
