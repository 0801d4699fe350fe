"""Times the GEMM shapes of one transformer block (forward, input-gradient and weight-gradient
forms, plus the batched attention products) with the tcgen05 kernel.

    python benchmarks/bench_gemm_shapes.py --tokens 8192 --d-model 2048 --ffn 8192 --heads 16 --seq 1024
    python benchmarks/bench_gemm_shapes.py --sustained 1.5 --pair-modes 0 1 2 --skip-attention

`--sustained S` launches every case back to back for S seconds instead of sampling isolated
launches: the GPU then sits at its power cap, as it does inside a training step.  `--pair-modes`
repeats every case under the given CTA-pair settings of the planner (0 off, 1 256 x 256 pair
tiles, 2 512 x 256 pair tiles).
"""
import argparse
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks._support.timing import time_cuda  # noqa: E402
from orthon_b200 import _C  # noqa: E402


def rand(shape, dtype):
    rng = np.random.default_rng(0)
    return _C.from_numpy(rng.standard_normal(shape).astype(np.float32), dtype).to("cuda:0")


def sustained_ms(fn, seconds):
    """Mean duration of one launch over `seconds` of back-to-back launches (device time)."""
    import time
    for _ in range(5):
        fn()
    _C.cuda_synchronize()
    start = _C.CudaEvent.record(0)
    t0, n = time.perf_counter(), 0
    while time.perf_counter() - t0 < seconds:
        for _ in range(20):
            fn()
        n += 20
        _C.cuda_synchronize()
    stop = _C.CudaEvent.record(0)
    stop.synchronize()
    return stop.elapsed_ms_since(start) / n


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--sustained", type=float, default=0.0)
    ap.add_argument("--pair-modes", type=int, nargs="+", default=None)
    ap.add_argument("--skip-attention", action="store_true")
    a = ap.parse_args()
    M, E, F = a.tokens, a.d_model, a.ffn
    cases = []
    for name, k, n in (("qkv", E, 3 * E), ("proj", E, E), ("fc1", E, F), ("fc2", F, E), ("head", E, a.vocab)):
        x, w, g = rand((M, k), a.dtype), rand((k, n), a.dtype), rand((M, n), a.dtype)
        cases.append((f"{name}.fwd  [{M}x{k}]@[{k}x{n}]", 2.0 * M * k * n, lambda x=x, w=w: _C._gemm(x, False, w, False)))
        cases.append((f"{name}.dgrad g@Wt", 2.0 * M * k * n, lambda g=g, w=w: _C._gemm(g, False, w, True)))
        cases.append((f"{name}.wgrad xt@g", 2.0 * M * k * n, lambda x=x, g=g: _C._gemm(x, True, g, False)))
    if not a.skip_attention:
        B, H, T, D = M // a.seq, a.heads, a.seq, E // a.heads
        q, k_, v = rand((B, H, T, D), a.dtype), rand((B, H, T, D), a.dtype), rand((B, H, T, D), a.dtype)
        p = rand((B, H, T, T), a.dtype)
        cases.append((f"attn.scores q@kt [{B*H}x{T}x{D}]", 2.0 * B * H * T * T * D, lambda: _C._gemm(q, False, k_, True)))
        cases.append(("attn.pv p@v", 2.0 * B * H * T * T * D, lambda: _C._gemm(p, False, v, False)))
        cases.append(("attn.dv pt@do", 2.0 * B * H * T * T * D, lambda: _C._gemm(p, True, v, False)))
        cases.append(("attn.dq ds@k", 2.0 * B * H * T * T * D, lambda: _C._gemm(p, False, k_, False)))
    for mode in (a.pair_modes or [None]):
        if mode is not None:
            _C._set_gemm_pair_mode(mode)
        total_ms = 0.0
        for name, flops, fn in cases:
            if a.sustained > 0:
                ms = sustained_ms(fn, a.sustained)
            else:
                ms = time_cuda(fn, warmup=3, iters=10)["median_ms"]
            total_ms += ms
            print(json.dumps({"case": name, "pair_mode": mode, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1)}), flush=True)
        print(json.dumps({"pair_mode": mode, "total_ms": total_ms, "sustained": a.sustained}), flush=True)


if __name__ == "__main__":
    main()
