"""Small CNN on synthetic 3x32x32 images, bf16 AMP with a disabled GradScaler, DDP over every
visible GPU through the peer-memory transport.

    python -m orthon_b200.distributed.run --nproc_per_node 2 --backend p2p examples/ddp_cnn_amp.py
    python examples/ddp_cnn_amp.py            # single GPU
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
import orthon_b200.distributed as dist  # noqa: E402
from orthon_b200 import _C  # noqa: E402
from orthon_b200.models import SmallCNN  # noqa: E402


def main(steps=10, batch=128):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = f"cuda:{local}"
    if world > 1:
        dist.init_process_group()
    ob.manual_seed(0)
    model = SmallCNN()
    model.cast("bfloat16").to(device)
    wrapped = dist.DDP(model, sync_grads=False, bucket_size_mb=25) if world > 1 else model
    opt = ob.amp.MixedPrecisionOptimizer(wrapped, ob.optim.Adam, lr=1e-3)
    scaler = ob.amp.GradScaler(enabled=False)
    rng = np.random.default_rng(rank)
    for step in range(steps):
        pixels = rng.uniform(0, 1, size=(batch, 3, 32, 32)).astype(np.float32)
        pixels = (pixels - pixels.mean()) / pixels.std()
        x = _C.from_numpy(pixels, "bfloat16").to(device)
        y = _C.from_numpy(rng.integers(0, 10, batch).astype(np.int64)).to(device)
        opt.zero_grad()
        loss = ob.cross_entropy(wrapped(x), y)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        if rank == 0:
            print(f"step {step} loss {loss.item():.4f}")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
