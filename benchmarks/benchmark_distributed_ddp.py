"""Data-parallel training-step benchmark: one MLP trained by N ranks, gradient synchronisation
in three modes, next to the same step on a single rank, in float32 and under AMP.

    python benchmarks/benchmark_distributed_ddp.py --nprocs 2                      # CPU ranks, local backend
    python -m orthon_b200.distributed.run --nproc_per_node 2 --backend p2p \
        benchmarks/benchmark_distributed_ddp.py --device cuda --amp bfloat16       # one rank per GPU
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 \
        benchmarks/benchmark_distributed_ddp.py --device cuda --backend nccl

Modes: `blocking` (one all-reduce per parameter after backward), `bucketed` (greedy buckets of
`--bucket-mb`, reduced after backward), `overlap` (buckets launched from the gradient hooks
while backward is still running); with `--amp` there is one mode, `amp_ddp` (DDP with
sync_grads=False, master gradients reduced by MixedPrecisionOptimizer).  Model: MLP `--width` x `--depth` (default 1024 x 4, the
AMP comparison of the reference uses 2048 -> 4096 x 4 -> 1024 with batch 1024: `--preset amp`).
Without a launcher environment the script spawns `--nprocs` CPU ranks itself.  Times are wall
clock per step between barriers, the maximum over ranks.
(reference project: benchmarks/benchmark_distributed_ddp.py:13-154, bench_ddp_vs_single.py,
bench_amp_ddp_vs_fp32_ddp.py:84-156)
"""
import argparse
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
import orthon_b200.distributed as dist  # noqa: E402
from benchmarks._support import results  # noqa: E402
from orthon_b200 import _C, models  # noqa: E402

MODES = {"blocking": dict(bucket_size_mb=None, overlap_grad_sync=False),
         "bucketed": dict(bucket_size_mb=25, overlap_grad_sync=False),
         "overlap": dict(bucket_size_mb=25, overlap_grad_sync=True)}


def layer_sizes(args):
    if args.preset == "amp":
        return (2048, 4096, 4096, 4096, 4096, 1024), 1024
    return (args.width,) * (args.depth + 1) + (10,), args.batch


def run_mode(mode, args, rank, world, device):
    """Median step time (ms) of this rank, first and last loss."""
    sizes, batch = layer_sizes(args)
    ob.manual_seed(0)
    model = models.MLP(sizes)
    if args.amp:
        model.cast(args.amp)
    model.to(device)
    wrapped = model
    if mode != "single":
        if mode == "amp_ddp":
            wrapped = dist.DistributedDataParallel(model, sync_grads=False, bucket_size_mb=args.bucket_mb)
        else:
            kwargs = dict(MODES[mode])
            if kwargs["bucket_size_mb"] is not None:
                kwargs["bucket_size_mb"] = args.bucket_mb
            wrapped = dist.DistributedDataParallel(model, **kwargs)
    if args.amp:
        optimizer = ob.amp.MixedPrecisionOptimizer(wrapped, ob.optim.Adam, lr=1e-3)
        scaler = ob.amp.GradScaler(init_scale=128.0, enabled=(args.amp == "float16"))
    else:
        optimizer, scaler = ob.optim.Adam(model.parameters(), lr=1e-3), None
    rng = np.random.default_rng(100 + rank)
    x = ob.from_numpy(rng.standard_normal((batch, sizes[0])).astype(np.float32)).to(device)
    if args.amp:
        x = ob.cast(x, args.amp)
    y = _C.from_numpy(rng.integers(0, sizes[-1], batch).astype(np.int64)).to(device)
    cuda = device.startswith("cuda")

    def sync():
        if cuda:
            ob.cuda_synchronize()
        if mode != "single" and world > 1:
            dist.barrier()

    def step():
        optimizer.zero_grad()
        loss = ob.cross_entropy(wrapped(x), y)
        if scaler is None:
            loss.backward()
            optimizer.step()
        else:
            scaler.scale(loss).backward()
            scaler.step(optimizer)
            scaler.update()
        return loss

    first = float(step().item())
    for _ in range(args.warmup):
        step()
    samples = []
    for _ in range(args.steps):
        sync()
        t0 = time.perf_counter()
        step()
        sync()
        samples.append((time.perf_counter() - t0) * 1e3)
    last = float(step().item())
    return float(np.median(samples)), first, last


def worker(rank, args_dict):
    args = argparse.Namespace(**args_dict)
    world = dist.get_world_size() if dist.is_initialized() else 1
    device = f"cuda:{int(os.environ.get('LOCAL_RANK', rank))}" if args.device.startswith("cuda") else "cpu"
    rows = {}
    # Under AMP the optimizer reduces the float32 master gradients itself (DDP is built with
    # sync_grads=False), so the three synchronisation modes collapse into one.
    modes = ["amp_ddp"] if args.amp else [m for m in MODES if args.mode in ("all", m)]
    for mode in ["single"] + modes:
        ms, first, last = run_mode(mode, args, rank, world, device)
        if world > 1:
            t = ob.from_numpy(np.asarray([ms if r == rank else 0.0 for r in range(world)], dtype=np.float32)).to(device)
            dist.all_reduce(t)
            ms = max(t.to("cpu").tolist())
        rows[mode] = {"ms": ms, "first_loss": first, "last_loss": last}
    return rows


def report(rows, args, world):
    sizes, batch = layer_sizes(args)
    single = rows["single"]["ms"]
    cases = []
    for mode, r in rows.items():
        n = 1 if mode == "single" else world
        stats = {"median": r["ms"], "q1": r["ms"], "q3": r["ms"], "iqr": 0.0, "min": r["ms"], "max": r["ms"], "samples": args.steps,
                 "inner": 1, "units": "ms"}
        cases.append(results.case_result(f"ddp/{mode}", stats, shape=[batch, list(sizes)], implementation="orthon", device=args.device,
                                         dtype=args.amp or "float32", mode=mode, ranks=n, examples_per_s=batch * n / (r["ms"] / 1e3),
                                         step_time_vs_single=r["ms"] / single, first_loss=r["first_loss"], last_loss=r["last_loss"],
                                         correctness="loss-decreased" if r["last_loss"] < r["first_loss"] else "loss-not-decreased"))
    doc = results.document("distributed_ddp", cases, {"world_size": world, "backend": args.backend, "bucket_mb": args.bucket_mb,
                                                      "steps": args.steps, "warmup": args.warmup, "preset": args.preset})
    results.emit(doc, args.output or None)
    for c in cases:
        print(f"    {c['mode']:<9} ranks={c['ranks']} {c['examples_per_s']:.0f} examples/s, step time x{c['step_time_vs_single']:.2f} of single")
    return doc


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--mode", default="all", choices=["all"] + list(MODES))
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--backend", default="", help="local (spawned CPU ranks), p2p or nccl (launched ranks)")
    ap.add_argument("--nprocs", type=int, default=2, help="CPU ranks to spawn when no launcher environment is present")
    ap.add_argument("--amp", default="", choices=["", "float16", "bfloat16"])
    ap.add_argument("--preset", default="", choices=["", "amp"])
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--depth", type=int, default=4)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--output", default="")
    args = ap.parse_args(argv)
    if args.amp and not args.device.startswith("cuda"):
        raise SystemExit("AMP needs --device cuda")
    launched = "RANK" in os.environ and "WORLD_SIZE" in os.environ
    if launched:
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        backend = args.backend or os.environ.get("ORTHON_DISTRIBUTED_BACKEND") or ("p2p" if args.device.startswith("cuda") else "local")
        args.backend = backend
        if world > 1:
            kwargs = {"device": int(os.environ.get("LOCAL_RANK", rank))} if backend in ("p2p", "nccl") else {}
            dist.init_process_group(backend, rank=rank, world_size=world, **kwargs)
        rows = worker(rank, vars(args))
        doc = report(rows, args, world) if rank == 0 else None
        if world > 1:
            dist.destroy_process_group()
        return doc
    if args.device.startswith("cuda"):
        raise SystemExit("start one rank per GPU with `python -m orthon_b200.distributed.run --nproc_per_node N ...`")
    args.backend = "local"
    out = dist.spawn(worker, args=(vars(args),), nprocs=args.nprocs, backend="local")
    return report(out[0], args, args.nprocs)


if __name__ == "__main__":
    main()
