"""The smaller headline configurations, for this framework and for the unmodified reference.

    python benchmarks/bench_configs.py --config mlp_cpu [--impl reference]
    python benchmarks/bench_configs.py --config cnn --steps 30 --warmup 5 [--impl reference]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_configs.py --config cnn

mlp_cpu  MLP 784-256-128-10 (Linear/ReLU), float32, batch 64, SGD lr 0.01 on the CPU: three
         steps single-process, three steps as 2-rank local DDP, then a checkpoint save / load
         round trip; reports ms per step and the largest parameter difference after reload.
cnn      Small CNN (conv3x3 3-32 s1, 32-64 s2, 64-128 s2, ReLU, spatial mean, Linear 128-10),
         bf16 AMP with a disabled GradScaler, Adam lr 1e-3, 128 images per GPU, DDP when
         launched with several ranks; reports images/s (device time, max over ranks).

Both arms build the model through the public nn API of the package under test.  Inputs are
synthetic: pixels iid U[0,1] normalised to mean 0 / std 1, labels uniform in [0, 10).
"""
import argparse
import json
import os
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def load_framework(impl):
    """Returns (package, distributed module, from_numpy) of the arm under test."""
    if impl == "reference":
        ref = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref, "orthon")):
            raise RuntimeError("baseline/_ref/orthon is missing (reference not installed)")
        sys.path.insert(0, ref)
        import orthon as fw
        import orthon.distributed as dist
        return fw, dist, fw.from_numpy
    import orthon_b200 as fw
    import orthon_b200.distributed as dist
    return fw, dist, fw._C.from_numpy


# ------------------------------------------------------------------ mlp_cpu
def build_mlp(fw):
    nn = fw.nn
    return nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 10))


def mlp_steps(fw, from_numpy, model, rank, steps=3):
    opt = fw.optim.SGD(model.parameters(), lr=0.01)
    rng = np.random.default_rng(10 + rank)
    times, losses = [], []
    for _ in range(steps):
        x = from_numpy(rng.standard_normal((64, 784)).astype(np.float32))
        y = [int(v) for v in rng.integers(0, 10, 64)]
        t0 = time.perf_counter()
        opt.zero_grad()
        loss = fw.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        losses.append(float(loss.item()))
        times.append((time.perf_counter() - t0) * 1e3)
    return times, losses, opt


def _mlp_ddp_worker(rank, impl, out_dir):
    fw, dist, from_numpy = load_framework(impl)
    fw.manual_seed(0)
    model = build_mlp(fw)
    wrapped = dist.DistributedDataParallel(model)
    times, losses, _ = mlp_steps(fw, from_numpy, wrapped, rank)
    flat = np.concatenate([np.asarray(p.tolist(), dtype=np.float64) for p in model.parameters()])
    np.save(os.path.join(out_dir, f"params_{rank}.npy"), flat)
    with open(os.path.join(out_dir, f"times_{rank}.json"), "w") as f:
        json.dump({"times": times, "losses": losses}, f)


def run_mlp_cpu(args):
    fw, dist, from_numpy = load_framework(args.impl)
    fw.manual_seed(0)
    model = build_mlp(fw)
    times, losses, opt = mlp_steps(fw, from_numpy, model, 0)
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "mlp.ckpt")
        t0 = time.perf_counter()
        fw.save_checkpoint(path, model, opt)
        save_ms = (time.perf_counter() - t0) * 1e3
        before = np.concatenate([np.asarray(p.tolist(), dtype=np.float64) for p in model.parameters()])
        fw.manual_seed(1)
        clone = build_mlp(fw)
        clone_opt = fw.optim.SGD(clone.parameters(), lr=0.5)
        t0 = time.perf_counter()
        fw.load_checkpoint(path, clone, clone_opt)
        load_ms = (time.perf_counter() - t0) * 1e3
        after = np.concatenate([np.asarray(p.tolist(), dtype=np.float64) for p in clone.parameters()])
        size = os.path.getsize(path)
        dist.spawn(_mlp_ddp_worker, args=(args.impl, tmp), nprocs=2, backend="local")
        p0, p1 = np.load(os.path.join(tmp, "params_0.npy")), np.load(os.path.join(tmp, "params_1.npy"))
        with open(os.path.join(tmp, "times_0.json")) as f:
            ddp = json.load(f)
    print(json.dumps({
        "config": "mlp_cpu", "impl": args.impl, "single_ms_per_step": float(np.median(times)), "single_losses": losses,
        "ddp2_ms_per_step": float(np.median(ddp["times"])), "ddp2_losses_rank0": ddp["losses"],
        "ddp2_replica_max_abs_diff": float(np.abs(p0 - p1).max()), "checkpoint_bytes": size, "checkpoint_save_ms": save_ms,
        "checkpoint_load_ms": load_ms, "checkpoint_roundtrip_max_abs_diff": float(np.abs(before - after).max()),
        "restored_lr": clone_opt.get_lr(),
    }))


# ---------------------------------------------------------------------- cnn
def build_cnn(fw):
    nn = fw.nn

    class SmallCNN(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = nn.Conv2d(3, 32, 3, stride=1, padding=1)
            self.conv2 = nn.Conv2d(32, 64, 3, stride=2, padding=1)
            self.conv3 = nn.Conv2d(64, 128, 3, stride=2, padding=1)
            self.head = nn.Linear(128, 10)

        def forward(self, x):
            h = self.conv1(x).relu()
            h = self.conv2(h).relu()
            h = self.conv3(h).relu()
            return self.head(h.mean(3).mean(2))

    return SmallCNN()


def run_cnn(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    fw, dist, from_numpy = load_framework(args.impl)
    device = f"cuda:{local}"
    batch = 128
    if world > 1:
        if args.impl == "reference":
            store = f"/tmp/orthon_ref_store_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}"
            os.makedirs(store, exist_ok=True)
            os.environ["ORTHON_NCCL_STORE_DIR"] = store
            dist.init_process_group("nccl", rank=rank, world_size=world, device=local)
        else:
            dist.init_process_group("p2p", rank=rank, world_size=world, device=local)
    fw.manual_seed(0)
    model = build_cnn(fw)
    model.cast("bfloat16")
    model.to(device)
    wrapped = dist.DistributedDataParallel(model, sync_grads=False) if world > 1 else model
    opt = fw.amp.MixedPrecisionOptimizer(wrapped, fw.optim.Adam, lr=1e-3)
    scaler = fw.amp.GradScaler(enabled=False)
    rng = np.random.default_rng(rank)

    def make_arrays():
        px = rng.uniform(0, 1, size=(batch, 3, 32, 32)).astype(np.float32)
        px = (px - px.mean()) / px.std()
        return px, rng.integers(0, 10, batch)

    def upload(px, labels):
        """Host arrays -> device tensors through the public API (what a data loader hands over)."""
        if args.impl == "ours":
            x = fw.cast(from_numpy(px).to(device), "bfloat16")
            return x, from_numpy(labels.astype(np.int64)).to(device)
        return fw.cast(from_numpy(px), "bfloat16").to(device), [int(v) for v in labels]

    def make_batch():
        return upload(*make_arrays())

    def loss_of(x, y):
        logits = wrapped(x)
        if args.impl == "reference":
            logits = fw.cast(logits, "float32")  # the reference's cross-entropy kernel is float32-only
        return fw.cross_entropy(logits, y)

    def step(x, y):
        opt.zero_grad()
        loss = loss_of(x, y)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        return loss

    def sync():
        fw.cuda_synchronize()
        if world > 1:
            dist.barrier()

    x, y = make_batch()
    for _ in range(args.warmup):
        step(x, y)
    sync()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(x, y)
    sync()
    dev_s = time.perf_counter() - t0
    # End to end: the batches exist as host arrays (a loader's output); every step uploads its own
    # batch and reads the loss back.
    host_batches = [make_arrays() for _ in range(args.steps)]
    sync()
    t0 = time.perf_counter()
    last = None
    for px, labels in host_batches:
        x, y = upload(px, labels)
        last = float(step(x, y).item())
    sync()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        rows = np.zeros((world, 2), dtype=np.float32)
        rows[rank] = [dev_s, e2e_s]
        t = from_numpy(rows).to(device)
        dist.all_reduce(t)
        vals = np.asarray(t.to("cpu").tolist()).reshape(world, 2)
        dev_s, e2e_s = float(vals[:, 0].max()), float(vals[:, 1].max())
    images = batch * world * args.steps
    if rank == 0:
        print(json.dumps({
            "metric": "ddp_train_images_per_s", "config": "small-cnn bf16 AMP (scaler disabled), Adam, 128 images/GPU",
            "impl": args.impl, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "value": images / dev_s,
            "unit": "images/s", "ms_per_step": dev_s / args.steps * 1e3,
            "timing": "wall clock between device synchronisations (same for both arms), max over ranks",
            "e2e": {"value": images / e2e_s, "unit": "images/s", "last_loss": last},
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", choices=["mlp_cpu", "cnn"], required=True)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    try:
        (run_mlp_cpu if args.config == "mlp_cpu" else run_cnn)(args)
    except Exception as exc:  # noqa: BLE001
        if args.impl != "reference":
            raise
        print(json.dumps({"impl": "reference", "config": args.config, "unavailable": f"{type(exc).__name__}: {exc}"[:400]}))


if __name__ == "__main__":
    main()
