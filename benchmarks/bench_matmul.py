"""Square matmul sweep (M = N = K) for the tcgen05 GEMM, with a relative-error check against
a float32 torch reference on the smaller sizes.

    python benchmarks/bench_matmul.py --dtype bfloat16 --sizes 512 1024 2048 4096 8192
    python benchmarks/bench_matmul.py --sustained 4 --shapes 8192x8192x8192 8192x6144x2048 --torch

`--sustained S` runs each product back to back for S seconds (no L2 flush, no idle gaps), which is
the regime of a training step: the GPU sits at its power cap and the clock, not the issue rate,
decides the throughput.  Shapes are MxNxK; the SM clock is sampled during the loop.
"""
import argparse
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks._support.timing import time_cuda  # noqa: E402
from orthon_b200 import _C  # noqa: E402


def _loop(fn, sync, record, seconds, flops):
    """Launches `fn` back to back in chunks of 20 for `seconds`; returns TFLOP/s over the whole span."""
    import time
    for _ in range(10):
        fn()
    sync()
    start = record()
    t0, n = time.perf_counter(), 0
    while time.perf_counter() - t0 < seconds:
        for _ in range(20):
            fn()
        n += 20
        sync()
    ms = record(start)
    return flops * n / (ms * 1e-3) / 1e12, n


def sustained(args):
    from orthon_b200.utils import ClockSampler
    rng = np.random.default_rng(0)
    rows = []
    for shape in args.shapes:
        m, n, k = (int(v) for v in shape.lower().split("x"))
        a = _C.from_numpy(rng.standard_normal((m, k)).astype(np.float32), args.dtype).to("cuda:0")
        b = _C.from_numpy(rng.standard_normal((k, n)).astype(np.float32), args.dtype).to("cuda:0")

        def record(start=None):
            ev = _C.CudaEvent.record(0)
            if start is None:
                return ev
            ev.synchronize()
            return ev.elapsed_ms_since(start)

        with ClockSampler(0) as clocks:
            tflops, launches = _loop(lambda: _C._gemm(a, False, b, False), _C.cuda_synchronize, record, args.sustained, 2.0 * m * n * k)
        row = {"shape": shape, "dtype": args.dtype, "seconds": args.sustained, "launches": launches, "tflops_sustained": tflops,
               "sm_mhz": clocks.result["sm_mhz"], "power_w": clocks.result["power_w"], "reasons": clocks.result["reasons"]}
        if args.torch:
            import torch
            dt = {"bfloat16": torch.bfloat16, "float16": torch.float16}[args.dtype]
            x = torch.randn(m, k, device="cuda", dtype=dt)
            y = torch.randn(k, n, device="cuda", dtype=dt)
            out = torch.empty(m, n, device="cuda", dtype=dt)

            def trecord(start=None):
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                if start is None:
                    return ev
                ev.synchronize()
                return start.elapsed_time(ev)

            with ClockSampler(0) as tclocks:
                ttf, _ = _loop(lambda: torch.matmul(x, y, out=out), torch.cuda.synchronize, trecord, args.sustained, 2.0 * m * n * k)
            row["cublas_tflops_sustained"] = ttf
            row["cublas_sm_mhz"] = tclocks.result["sm_mhz"]
            row["cublas_power_w"] = tclocks.result["power_w"]
        rows.append(row)
        print(json.dumps(row), flush=True)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--sizes", type=int, nargs="+", default=[512, 1024, 2048, 4096, 8192])
    ap.add_argument("--layouts", nargs="+", default=["nn", "nt", "tn"])
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--torch", action="store_true", help="also time torch.matmul (cuBLAS) on the same shapes")
    ap.add_argument("--sustained", type=float, default=0.0, help="seconds of back-to-back launches per shape")
    ap.add_argument("--shapes", nargs="+", default=["8192x8192x8192"], help="MxNxK products for --sustained")
    args = ap.parse_args()
    if args.sustained > 0:
        return sustained(args)
    rng = np.random.default_rng(0)
    rows = []
    for n in args.sizes:
        a_np = rng.standard_normal((n, n)).astype(np.float32)
        b_np = rng.standard_normal((n, n)).astype(np.float32)
        a = _C.from_numpy(a_np, args.dtype).to("cuda:0")
        b = _C.from_numpy(b_np, args.dtype).to("cuda:0")
        for layout in args.layouts:
            ta, tb = layout[0] == "t", layout[1] == "t"
            stats = time_cuda(lambda: _C._gemm(a, ta, b, tb))
            row = {"n": n, "dtype": args.dtype, "layout": layout, **stats,
                   "tflops": 2.0 * n ** 3 / (stats["median_ms"] * 1e-3) / 1e12}
            if args.check and n <= 2048:
                import torch
                ta_ = torch.tensor(a.numpy().astype(np.float32)).cuda()
                tb_ = torch.tensor(b.numpy().astype(np.float32)).cuda()
                ref = (ta_.t() if ta else ta_).double() @ (tb_.t() if tb else tb_).double()
                out = torch.tensor(_C._gemm(a, ta, b, tb).numpy().astype(np.float32)).cuda().double()
                row["rel_err"] = float((out - ref).norm() / ref.norm())
            if args.torch:
                import torch
                dt = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[args.dtype]
                x = torch.randn(n, n, device="cuda", dtype=dt); y = torch.randn(n, n, device="cuda", dtype=dt)
                for _ in range(5):
                    x @ y
                torch.cuda.synchronize()
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                ts = []
                for _ in range(20):
                    _C._flush_l2(0); _C.cuda_synchronize()
                    ev[0].record(); x @ y; ev[1].record(); torch.cuda.synchronize()
                    ts.append(ev[0].elapsed_time(ev[1]))
                ts.sort()
                row["cublas_tflops"] = 2.0 * n ** 3 / (ts[len(ts) // 2] * 1e-3) / 1e12
            rows.append(row)
            print(json.dumps(row), flush=True)
    return rows


if __name__ == "__main__":
    main()
