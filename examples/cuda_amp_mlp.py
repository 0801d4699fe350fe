"""float16 mixed precision on one GPU: an MLP cast to float16, FP32 master weights in
MixedPrecisionOptimizer, dynamic loss scaling with GradScaler(init_scale=128); one step is fed a
deliberately huge loss to show the skipped update and the scale back-off.

    python examples/cuda_amp_mlp.py          # needs a CUDA device
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
from orthon_b200 import nn  # noqa: E402


def main(device="cuda:0", steps=8):
    ob.manual_seed(0)
    model = nn.Sequential(nn.Linear(64, 128), nn.ReLU(), nn.Linear(128, 10))
    model.cast("float16")
    model.to(device)
    opt = ob.amp.MixedPrecisionOptimizer(model, ob.optim.Adam, lr=1e-3)
    scaler = ob.amp.GradScaler(init_scale=128.0, growth_interval=4)
    rng = np.random.default_rng(0)
    for step in range(steps):
        x = ob.from_numpy(rng.standard_normal((32, 64)).astype(np.float32)).to(device).cast("float16")
        y = ob.from_numpy(rng.integers(0, 10, 32).astype(np.int64)).to(device)
        opt.zero_grad()
        loss = ob.cross_entropy(model(x).cast("float32"), y)
        if step == 3:
            loss = loss * 1e6  # overflows float16 gradients: the step is skipped, the scale halves
        scaler.scale(loss).backward()
        scaler.step(opt)
        print(f"step {step} loss {loss.item():.4f} scale {scaler.scale_factor:g} skipped {scaler.found_inf}")
        scaler.update()


if __name__ == "__main__":
    main()
