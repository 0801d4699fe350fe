"""Fused tcgen05 attention (packed qkv, causal) forward and backward timings.

    python benchmarks/bench_attention.py --batch 8 --heads 16 --seq 1024 --head-dim 128 [--torch]

FLOPs counted: forward 4*B*H*T*T*D, backward 10*B*H*T*T*D (the five matrix products of the
textbook formulation), both halved under the causal mask.  Times are CUDA-event medians with the
L2 flushed before each sample.  ORTHON_ATTENTION=composed times the GEMM + softmax composition.
"""
import argparse
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks._support.timing import time_cuda  # noqa: E402
from orthon_b200 import _C  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--no-causal", action="store_true")
    ap.add_argument("--torch", action="store_true", help="also time torch scaled_dot_product_attention (library kernel)")
    a = ap.parse_args()
    B, H, T, D = a.batch, a.heads, a.seq, a.head_dim
    E = H * D
    causal = not a.no_causal
    rng = np.random.default_rng(0)
    qkv = _C.from_numpy(rng.standard_normal((B, T, 3 * E)).astype(np.float32), a.dtype).to("cuda:0")
    qkv.requires_grad_(True)
    dout = _C.from_numpy(rng.standard_normal((B, T, E)).astype(np.float32), a.dtype).to("cuda:0")
    scale = D ** -0.5
    frac = 0.5 if causal else 1.0
    fwd_flops, bwd_flops = 4.0 * B * H * T * T * D * frac, 10.0 * B * H * T * T * D * frac

    def fwd():
        with_no_grad = _C.set_grad_enabled(False)
        out = _C._attention_qkv(qkv, H, None, causal, scale)
        _C.set_grad_enabled(True)
        return out

    def fwd_bwd():
        out = _C._attention_qkv(qkv, H, None, causal, scale)
        (out * dout).sum().backward()
        qkv.zero_grad()

    t_f = time_cuda(fwd, warmup=3, iters=10)["median_ms"]
    t_fb = time_cuda(fwd_bwd, warmup=3, iters=10)["median_ms"]
    row = {"shape": [B, H, T, D], "dtype": a.dtype, "causal": causal, "fused": bool(_C._attention_qkv_fused(qkv, H)),
           "fwd_ms": t_f, "fwd_tflops": fwd_flops / t_f / 1e9, "fwd_bwd_ms": t_fb,
           "note": "fwd_bwd includes the elementwise mul/sum that seeds the gradient"}
    if a.torch:
        import torch
        tq = torch.randn(B, H, T, D, device="cuda", dtype=getattr(torch, a.dtype), requires_grad=True)
        tk, tv = torch.randn_like(tq, requires_grad=True), torch.randn_like(tq, requires_grad=True)
        tdo = torch.randn_like(tq)

        def timed(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            ts = []
            for _ in range(10):
                _C._flush_l2(0)
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record(); fn(); e.record(); torch.cuda.synchronize()
                ts.append(s.elapsed_time(e))
            return sorted(ts)[len(ts) // 2]
        f = lambda: torch.nn.functional.scaled_dot_product_attention(tq, tk, tv, is_causal=causal)  # noqa: E731

        def fb():
            o = f()
            o.backward(tdo)
        row["torch_sdpa_fwd_ms"] = timed(lambda: f().detach())
        row["torch_sdpa_fwd_bwd_ms"] = timed(fb)
    print(json.dumps(row))


if __name__ == "__main__":
    main()
