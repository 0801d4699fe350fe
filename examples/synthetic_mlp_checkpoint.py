"""Checkpoint and resume: an MLP trained with Adam on one synthetic batch is saved after
`--steps`, training continues for `--resume-steps`, and a fresh model restored from the file
and trained for the same extra steps must end at the same parameters (difference <= 1e-5).

    python examples/synthetic_mlp_checkpoint.py --resume-smoke

The file holds the parameters, Adam's moments and step count, and the metadata dictionary; it
does not hold gradients, the training / evaluation mode or any random state.
(reference project: examples/synthetic_mlp_checkpoint.py:15-129)
"""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
from orthon_b200 import nn  # noqa: E402


def make_model(hidden):
    ob.manual_seed(7)
    return nn.Sequential(nn.Linear(8, hidden), nn.Tanh(), nn.Linear(hidden, 1))


def make_batch(batch_size):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((batch_size, 8)).astype(np.float32)
    y = np.sin(x.sum(axis=1, keepdims=True)).astype(np.float32)
    return ob.from_numpy(x), ob.from_numpy(-y)


def loss_fn(model, batch):
    x, negated_target = batch
    diff = model(x) + negated_target
    return ob.mean(diff * diff)


def train_steps(model, optimizer, batch, steps):
    losses = []
    for _ in range(steps):
        optimizer.zero_grad()
        loss = loss_fn(model, batch)
        loss.backward()
        optimizer.step()
        losses.append(float(loss.item()))
    return losses


def flat_params(model):
    return np.asarray([v for p in model.parameters() for v in p.tolist()], dtype=np.float64)


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--resume-steps", type=int, default=3)
    ap.add_argument("--batch-size", type=int, default=16)
    ap.add_argument("--hidden", type=int, default=16)
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--checkpoint", default="examples/results/synthetic_mlp_checkpoint.ckpt")
    ap.add_argument("--resume-smoke", action="store_true", help="check that resumed training matches continuous training")
    ap.add_argument("--keep-checkpoint", action="store_true")
    return ap.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    os.makedirs(os.path.dirname(os.path.abspath(args.checkpoint)), exist_ok=True)
    batch = make_batch(args.batch_size)
    model = make_model(args.hidden)
    optimizer = ob.optim.Adam(model.parameters(), lr=args.lr)
    initial = float(loss_fn(model, batch).item())
    first = train_steps(model, optimizer, batch, args.steps)
    ob.save_checkpoint(args.checkpoint, model, optimizer, {"steps": args.steps, "loss": first[-1]})
    print(f"saved checkpoint: {args.checkpoint} initial_loss={initial:.6f} step_loss={first[-1]:.6f}")
    if not args.resume_smoke:
        return None
    continuous = train_steps(model, optimizer, batch, args.resume_steps)
    resumed = make_model(args.hidden)
    resumed_optimizer = ob.optim.Adam(resumed.parameters(), lr=args.lr * 10)  # overwritten by the load
    metadata = ob.load_checkpoint(args.checkpoint, resumed, resumed_optimizer)
    resumed_losses = train_steps(resumed, resumed_optimizer, batch, args.resume_steps)
    diff = float(np.abs(flat_params(model) - flat_params(resumed)).max())
    print(f"resume smoke: metadata={metadata} continuous_loss={continuous[-1]:.6f} "
          f"resumed_loss={resumed_losses[-1]:.6f} max_param_diff={diff:.3e}")
    if not args.keep_checkpoint:
        os.remove(args.checkpoint)
    if diff > 1e-5:
        raise RuntimeError(f"resume mismatch: max_param_diff={diff:.3e}")
    return diff


if __name__ == "__main__":
    main()
