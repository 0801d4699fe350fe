"""Convolution kernels one by one: forward, input gradient and weight gradient of a conv2d layer,
timed on the device for the implicit-GEMM route and for the unfold + GEMM lowering, optionally
beside torch (cuDNN) on the same shapes.

    python benchmarks/bench_conv.py                       # the three layers of the small CNN
    python benchmarks/bench_conv.py --shapes 128x64x56x56x64x3x3x1x1 --torch

A shape is NxCxHxWxKxRxSxstridexpad.  Each kernel is launched `--inner` times back to back between
two CUDA events (the launches queue up, so the figure is the kernel's own throughput and not the
host's launch rate); the median of `--samples` such spans is reported per launch, in microseconds.
The layer's tensors are a few megabytes, so they stay in the L2 between launches, as they do in a
training step, where the producer of an activation has just written it.
"""
import argparse
import json
import os
import statistics
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from orthon_b200 import _C  # noqa: E402

SMALL_CNN = ["128x3x32x32x32x3x3x1x1", "128x32x32x32x64x3x3x2x1", "128x64x16x16x128x3x3x2x1"]


def span_us(fn, inner, samples, warmup=3):
    for _ in range(warmup):
        fn()
    _C.cuda_synchronize()
    spans = []
    for _ in range(samples):
        start = _C.CudaEvent.record(0)
        for _ in range(inner):
            fn()
        stop = _C.CudaEvent.record(0)
        stop.synchronize()
        spans.append(stop.elapsed_ms_since(start) * 1e3 / inner)
    return statistics.median(spans)


def torch_span_us(fn, inner, samples, warmup=3):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    spans = []
    for _ in range(samples):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(inner):
            fn()
        b.record()
        torch.cuda.synchronize()
        spans.append(a.elapsed_time(b) * 1e3 / inner)
    return statistics.median(spans)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", nargs="+", default=SMALL_CNN)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--inner", type=int, default=50)
    ap.add_argument("--samples", type=int, default=7)
    ap.add_argument("--routes", nargs="+", default=["auto", "lowering"])
    ap.add_argument("--torch", action="store_true")
    args = ap.parse_args()
    rng = np.random.default_rng(0)
    for shape in args.shapes:
        N, C, H, W, K, R, S, stride, pad = (int(v) for v in shape.lower().split("x"))
        OH, OW = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
        flops = 2.0 * N * OH * OW * K * C * R * S
        x = _C.from_numpy(rng.standard_normal((N, C, H, W)).astype(np.float32), args.dtype).to("cuda:0")
        w = _C.from_numpy((rng.standard_normal((K, C, R, S)) / np.sqrt(C * R * S)).astype(np.float32), args.dtype).to("cuda:0")
        b = _C.from_numpy(rng.standard_normal((K,)).astype(np.float32), args.dtype).to("cuda:0")
        gy = _C.from_numpy(rng.standard_normal((N, K, OH, OW)).astype(np.float32), args.dtype).to("cuda:0")
        row = {"shape": shape, "dtype": args.dtype, "gflop": flops / 1e9}
        for route in args.routes:
            _C._conv2d_force_route(route)
            fwd = span_us(lambda: _C.conv2d(x, w, b, stride, stride, pad, pad), args.inner, args.samples)
            row[f"{route}_route"] = _C._conv2d_last_route()
            if row[f"{route}_route"] == "tcgen05_implicit_gemm":
                row["forward_launch"] = dict(zip(("grid", "shared_bytes", "ring_slots", "ctas_per_sm"), _C._conv2d_last_launch()))
            both = span_us(lambda: _C._conv2d_backward(gy, x, w, True, stride, stride, pad, pad, True), args.inner, args.samples)
            wonly = span_us(lambda: _C._conv2d_backward(gy, x, w, True, stride, stride, pad, pad, False), args.inner, args.samples)
            row[f"{route}_us"] = {"forward": fwd, "input_grad": both - wonly, "weight_and_bias_grad": wonly}
        _C._conv2d_force_route("auto")
        if args.torch:
            import torch
            dt = {"bfloat16": torch.bfloat16, "float16": torch.float16}[args.dtype]
            tx = torch.randn(N, C, H, W, device="cuda", dtype=dt)
            tw = torch.randn(K, C, R, S, device="cuda", dtype=dt)
            tb = torch.randn(K, device="cuda", dtype=dt)
            tg = torch.randn(N, K, OH, OW, device="cuda", dtype=dt)
            torch.backends.cudnn.benchmark = True
            conv = torch.nn.functional.conv2d
            grad = torch.ops.aten.convolution_backward
            geom = dict(bias_sizes=[K], stride=[stride, stride], padding=[pad, pad], dilation=[1, 1], transposed=False,
                        output_padding=[0, 0], groups=1)
            row["torch_us"] = {
                "forward": torch_span_us(lambda: conv(tx, tw, tb, stride=stride, padding=pad), args.inner, args.samples),
                "input_grad": torch_span_us(lambda: grad(tg, tx, tw, output_mask=[True, False, False], **geom), args.inner, args.samples),
                "weight_and_bias_grad": torch_span_us(lambda: grad(tg, tx, tw, output_mask=[False, True, True], **geom), args.inner, args.samples),
            }
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
