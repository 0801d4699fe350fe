"""Timeline of one training step of the causal LM: where the forward, the backward and the
optimizer step sit on the compute stream, and when each gradient bucket's fused reduction (or
update) ran on the communication stream.

    python benchmarks/trace_step.py --model 1p3b                                   # one GPU
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \\
        benchmarks/trace_step.py --model 1p3b                                      # DDP, peer transport

Prints one JSON document (rank 0): the phases, every bucket range, and how much of the bucket
time fell inside the backward pass.  Uses the tracing ranges of orthon_b200.utils (CUDA events on
the stream a range belongs to), so nothing runs under a profiler.
"""
import argparse
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1p3b", choices=["1p3b", "tiny"])
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--fused", default="update", choices=["update", "overlap", "reduce"])
    args = ap.parse_args()
    import orthon_b200 as ob
    import orthon_b200.distributed as dist
    from orthon_b200 import _C
    from orthon_b200.models import LM_1P3B, TINY_LM, CausalLM
    from orthon_b200.utils import clear_ranges, enable_tracing, timeline, trace_range

    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    cfg, batch, seq = (LM_1P3B, 8, 1024) if args.model == "1p3b" else (TINY_LM, 32, 512)
    device = f"cuda:{local}"
    if world > 1:
        dist.init_process_group("p2p", rank=rank, world_size=world, device=local)
    ob.manual_seed(1234)
    model = CausalLM(cfg)
    model.cast("bfloat16").to(device)
    wrapped = dist.DDP(model, sync_grads=False, bucket_size_mb=25) if world > 1 else model
    opt = ob.amp.MixedPrecisionOptimizer(wrapped, ob.optim.Adam, fused=args.fused, lr=3e-4)
    rng = np.random.default_rng(100 + rank)
    tok = rng.integers(0, cfg.vocab_size, size=(batch, seq + 1), dtype=np.int64)
    ids = _C.from_numpy(np.ascontiguousarray(tok[:, :-1])).to(device)
    tgt = _C.from_numpy(np.ascontiguousarray(tok[:, 1:]).reshape(-1)).to(device)

    def step(traced):
        opt.zero_grad()
        with trace_range("forward", local):
            loss = _C.cross_entropy(wrapped(ids), tgt)
        with trace_range("backward", local):
            loss.backward()
        with trace_range("optimizer.step", local):
            opt.step()

    for _ in range(args.warmup):
        step(False)
    _C.cuda_synchronize()
    if world > 1:
        dist.barrier()
    enable_tracing(True)
    clear_ranges()
    step(True)
    _C.cuda_synchronize()
    rows = timeline()
    enable_tracing(False)
    phases = {name: (a, b) for name, kind, a, b in rows if kind == 0 and name in ("forward", "backward", "optimizer.step")}
    buckets = [(name, a, b) for name, kind, a, b in rows if kind == 1]
    b0, b1 = phases["backward"]
    inside = sum(max(0.0, min(b, b1) - max(a, b0)) for _, a, b in buckets)
    total = sum(b - a for _, a, b in buckets)
    doc = {"model": args.model, "world": world, "fused": args.fused,
           "phases_ms": {k: [round(v[0], 3), round(v[1], 3)] for k, v in phases.items()},
           "step_ms": round(max(v[1] for v in phases.values()) - min(v[0] for v in phases.values()), 3),
           "buckets": len(buckets), "bucket_ms_total": round(total, 3), "bucket_ms_inside_backward": round(inside, 3),
           "last_bucket_end_after_backward_ms": round(max((b for _, _, b in buckets), default=b1) - b1, 3),
           "bucket_ranges_ms": [[name, round(a, 3), round(b, 3)] for name, a, b in buckets]}
    if rank == 0:
        print(json.dumps(doc), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
