"""Runs each hand-written kernel family once or twice on a small case (operands larger than the
126 MB L2 where the op is bandwidth-bound, a few hundred MB in total) so that one profiler
capture can cover them:

    python benchmarks/profile_kernels.py                       # plain run (prints CUDA-event times)
    ncu --set full --clock-control none -k regex:<kernel> -c 2 -o out python benchmarks/profile_kernels.py --only <family>

Families: layernorm, xent, adam, elementwise, reduce, dropout, embedding, attention, conv, maxpool.
"""
import argparse
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
from orthon_b200 import _C  # noqa: E402

DEV = "cuda:0"


def rand(shape, dtype="bfloat16", grad=False, scale=1.0, seed=0):
    rng = np.random.default_rng(seed)
    t = _C.from_numpy((rng.standard_normal(shape) * scale).astype(np.float32), dtype).to(DEV)
    if grad:
        t.requires_grad_(True)
    return t


def timed(name, fn, bytes_moved=None, flops=None, reps=3):
    fn()
    _C.cuda_synchronize()
    best = None
    for _ in range(reps):
        _C._flush_l2(0)
        s = _C.CudaEvent.record(0)
        fn()
        e = _C.CudaEvent.record(0)
        _C.cuda_synchronize()
        ms = e.elapsed_ms_since(s)
        best = ms if best is None else min(best, ms)
    row = {"case": name, "ms": round(best, 4)}
    if bytes_moved:
        row["gb_per_s"] = round(bytes_moved / best / 1e6, 1)
    if flops:
        row["tflops"] = round(flops / best / 1e9, 1)
    print(json.dumps(row), flush=True)


def fam_layernorm():
    R, D = 32768, 2048
    x = rand((R, D), grad=True)
    w, b = rand((D,), grad=True, seed=1), rand((D,), grad=True, seed=2)
    g = rand((R, D), seed=3)
    with ob.no_grad():
        timed("layernorm_fwd [32768x2048] bf16", lambda: _C._layer_norm(x, w, b, 1e-5), bytes_moved=2 * R * D * 2)

    def fb():
        y = _C._layer_norm(x, w, b, 1e-5)
        (y * g).sum().backward()
        x.zero_grad(); w.zero_grad(); b.zero_grad()
    timed("layernorm_fwd+bwd (+mul,sum seed)", fb)


def fam_xent():
    R, V = 8192, 32000
    logits = rand((R, V), grad=True)
    tgt = _C.from_numpy(np.random.default_rng(0).integers(0, V, R).astype(np.int64)).to(DEV)

    def fb():
        loss = ob.cross_entropy(logits, tgt)
        loss.backward()
        logits.zero_grad()
    timed("softmax_xent fwd+bwd [8192x32000] bf16", fb, bytes_moved=3 * R * V * 2)


def fam_adam():
    n = 64 << 20
    p = rand((n,), "float32", scale=0.02)
    m = _C._zeros_on([n], "float32", DEV)
    v = _C._zeros_on([n], "float32", DEV)
    g = rand((n,), "bfloat16", seed=1)
    model = _C._zeros_on([n], "bfloat16", DEV)
    timed("adam fused (fp32 master/m/v, bf16 grad+model) 64M", lambda: _C._adam_step_(p, m, v, g, model, 1e-3, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001, 1.0),
          bytes_moved=n * (12 + 12 + 2 + 2))


def fam_elementwise():
    n = 128 << 20
    a, b = rand((n,)), rand((n,), seed=1)
    with ob.no_grad():
        timed("add bf16 128M", lambda: a + b, bytes_moved=3 * n * 2)
        timed("gelu bf16 128M", lambda: a.gelu(), bytes_moved=2 * n * 2)
        timed("cast bf16->f32 128M", lambda: a.cast("float32"), bytes_moved=n * 6)


def fam_reduce():
    R, C = 65536, 2048
    x = rand((R, C))
    with ob.no_grad():
        timed("sum(dim=0) [65536x2048] bf16 (bias-gradient shape)", lambda: x.sum(0), bytes_moved=R * C * 2)
        timed("sum(dim=1) [65536x2048] bf16", lambda: x.sum(1), bytes_moved=R * C * 2)
        timed("max(dim=1) [65536x2048] bf16", lambda: x.max(1), bytes_moved=R * C * 2)
        timed("sum(all) 128M bf16", lambda: x.sum(), bytes_moved=R * C * 2)


def fam_dropout():
    n = 128 << 20
    x = rand((n,))
    with ob.no_grad():
        timed("dropout p=0.1 bf16 128M", lambda: _C.dropout(x, 0.1, 1234), bytes_moved=2 * n * 2)


def fam_embedding():
    V, D, N = 32000, 2048, 65536
    w = rand((V, D), grad=True, scale=0.02)
    idx = _C.from_numpy(np.random.default_rng(0).integers(0, V, N).astype(np.int64)).to(DEV)

    def fb():
        y = _C.embedding(idx, w)
        y.sum().backward()
        w.zero_grad()
    timed("embedding gather+scatter [65536 x 2048] bf16", fb)


def fam_attention():
    B, H, T, D = 8, 16, 1024, 128
    qkv = rand((B, T, 3 * H * D), grad=True)
    dout = rand((B, T, H * D), seed=1)
    fl = 4.0 * B * H * T * T * D * 0.5
    with ob.no_grad():
        timed("flash_fwd causal [8,16,1024,128] bf16", lambda: _C._attention_qkv(qkv, H, None, True, D ** -0.5), flops=fl)

    def fb():
        out = _C._attention_qkv(qkv, H, None, True, D ** -0.5)
        (out * dout).sum().backward()
        qkv.zero_grad()
    timed("flash fwd+bwd (+mul,sum seed)", fb, flops=3.5 * fl)


def fam_conv():
    x = rand((256, 64, 32, 32), grad=True)
    w = rand((128, 64, 3, 3), grad=True, scale=0.05)
    b = rand((128,), grad=True)
    fl = 2.0 * 256 * 128 * 32 * 32 * 64 * 9
    with ob.no_grad():
        timed("conv2d 3x3 s1 p1 [256,64,32,32]->128 bf16 fwd", lambda: _C.conv2d(x, w, b, 1, 1, 1, 1), flops=fl)

    def fb():
        y = _C.conv2d(x, w, b, 1, 1, 1, 1)
        y.sum().backward()
        x.zero_grad(); w.zero_grad(); b.zero_grad()
    timed("conv2d fwd+bwd", fb, flops=3 * fl)


def fam_maxpool():
    x = rand((256, 64, 64, 64), "float32", grad=True)

    def fb():
        y = _C.maxpool2d(x, 2, 2, 2, 2)
        y.sum().backward()
        x.zero_grad()
    timed("maxpool2d 2x2 fwd+bwd [256,64,64,64] f32", fb)


FAMILIES = {"layernorm": fam_layernorm, "xent": fam_xent, "adam": fam_adam, "elementwise": fam_elementwise,
            "reduce": fam_reduce, "dropout": fam_dropout, "embedding": fam_embedding, "attention": fam_attention,
            "conv": fam_conv, "maxpool": fam_maxpool}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", nargs="*", default=None)
    a = ap.parse_args()
    for name, fn in FAMILIES.items():
        if a.only and name not in a.only:
            continue
        fn()
        _C._memory_pool_clear()


if __name__ == "__main__":
    main()
