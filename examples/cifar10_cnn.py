"""Two CNNs for 3x32x32 images on CIFAR-10 (or a synthetic stand-in): a small two-convolution
network with max pooling and a six-convolution mini-VGG.

    python examples/cifar10_cnn.py --model small --channels 8 --hidden 64 --epochs 1
    python examples/cifar10_cnn.py --model minivgg --device cuda --batch-size 128 --synthetic \
        --train-limit 4096 --test-limit 1024 --lr-schedule cosine --epochs 3

CIFAR-10 is read from the binary-version batches (`cifar-10-batches-bin/data_batch_1..5.bin`,
`test_batch.bin`: one label byte and 3072 pixel bytes per record) under `--data-dir`; nothing is
downloaded and nothing is unpickled.  Without them, or with `--synthetic`, ten fixed random image
prototypes plus noise are used.  `--augment` applies random
horizontal flips and 4-pixel shifts.  Schedules: none, step (multiply by `--lr-gamma` at the
listed epochs) and cosine (to `--min-lr`).
(reference project: examples/cifar10_cnn.py:18-327)
"""
import argparse
import json
import math
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
from orthon_b200 import nn  # noqa: E402

MEAN = np.array([0.4914, 0.4822, 0.4465], dtype=np.float32).reshape(1, 3, 1, 1)
STD = np.array([0.2470, 0.2435, 0.2616], dtype=np.float32).reshape(1, 3, 1, 1)


class _Classifier(nn.Module):
    """Convolutional features, flatten, two-layer head; parameters optionally shrunk at start."""

    def __init__(self, features, flat_features, hidden, init_scale):
        super().__init__()
        self.features = features
        self.classifier = nn.Sequential(nn.Linear(flat_features, hidden), nn.ReLU(), nn.Linear(hidden, 10))
        self._flat_features = flat_features
        if init_scale != 1.0:
            with ob.no_grad():
                for p in self.parameters():
                    p.mul_(init_scale)

    def forward(self, x):
        return self.classifier(self.features(x).reshape([x.shape[0], self._flat_features]))


def small_cnn(hidden, channels=16, init_scale=0.5):
    features = nn.Sequential(
        nn.Conv2d(3, channels, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2),
        nn.Conv2d(channels, channels, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2))
    return _Classifier(features, channels * 8 * 8, hidden, init_scale)


def mini_vgg(hidden, base_channels=32, init_scale=0.5):
    layers, c_in = [], 3
    for width in (base_channels, base_channels * 2, base_channels * 4):
        layers += [nn.Conv2d(c_in, width, 3, padding=1), nn.ReLU(), nn.Conv2d(width, width, 3, padding=1), nn.ReLU(),
                   nn.MaxPool2d(2)]
        c_in = width
    return _Classifier(nn.Sequential(*layers), c_in * 4 * 4, hidden, init_scale)


def make_model(args):
    if args.model == "small":
        return small_cnn(args.hidden, args.channels, args.init_scale)
    return mini_vgg(args.hidden, args.vgg_base_channels, args.init_scale)


def load_cifar(data_dir):
    root = os.path.join(data_dir, "cifar-10-batches-bin")
    if not os.path.isdir(root):
        return None

    def read(name):
        records = np.fromfile(os.path.join(root, name), dtype=np.uint8).reshape(-1, 3073)
        return records[:, 1:].reshape(-1, 3, 32, 32), records[:, 0].astype(np.int64)

    train = [read(f"data_batch_{i}.bin") for i in range(1, 6)]
    tx, ty = np.concatenate([t[0] for t in train]), np.concatenate([t[1] for t in train])
    vx, vy = read("test_batch.bin")
    return tx, ty, vx, vy


def synthetic_images(n_train, n_test, seed):
    rng = np.random.default_rng(seed)
    coarse = rng.uniform(0, 255, size=(10, 3, 8, 8))
    prototypes = np.repeat(np.repeat(coarse, 4, axis=2), 4, axis=3)

    def draw(n):
        labels = rng.integers(0, 10, n)
        images = np.clip(prototypes[labels] + rng.normal(0, 40, size=(n, 3, 32, 32)), 0, 255).astype(np.uint8)
        return images, labels.astype(np.int64)

    return (*draw(n_train), *draw(n_test))


def normalise(images):
    return ((images.astype(np.float32) / 255.0) - MEAN) / STD


def augment(images, rng):
    out = np.empty_like(images)
    padded = np.pad(images, ((0, 0), (0, 0), (4, 4), (4, 4)), mode="constant")
    for i in range(len(images)):
        dy, dx = rng.integers(0, 9, 2)
        crop = padded[i, :, dy:dy + 32, dx:dx + 32]
        out[i] = crop[:, :, ::-1] if rng.random() < 0.5 else crop
    return out


def apply_lr_schedule(optimizer, args, epoch, step_epochs):
    """`epoch` counts from 1.  Returns the learning rate in force for that epoch."""
    if args.lr_schedule == "step" and epoch in step_epochs:
        optimizer.set_lr(optimizer.get_lr() * args.lr_gamma)
    elif args.lr_schedule == "cosine":
        progress = (epoch - 1) / max(1, args.epochs - 1)
        optimizer.set_lr(args.min_lr + 0.5 * (args.lr - args.min_lr) * (1.0 + math.cos(math.pi * progress)))
    return optimizer.get_lr()


def parse_step_epochs(text):
    epochs = {int(part) for part in text.split(",") if part.strip()}
    if any(e <= 0 for e in epochs):
        raise ValueError("--lr-step-epochs values must be positive")
    return epochs


def run_epoch(model, x, y, optimizer, args, rng, train):
    order = rng.permutation(len(x)) if (train and not args.disable_shuffle) else np.arange(len(x))
    outputs = []
    for start in range(0, len(order), args.batch_size):
        sel = order[start:start + args.batch_size]
        images = x[sel]
        if train and args.augment:
            images = augment(images, rng)
        bx = ob.from_numpy(np.ascontiguousarray(normalise(images))).to(args.device)
        if train:
            out = ob.training.train_step(model, bx, y[sel], ob.cross_entropy, optimizer)
        else:
            with ob.no_grad():
                out = ob.training.eval_step(model, bx, y[sel], ob.cross_entropy)
        if not math.isfinite(out["loss"]):
            raise RuntimeError(f"non-finite loss {out['loss']} in {'training' if train else 'evaluation'}")
        outputs.append(out)
    return ob.training.weighted_metric_average(outputs)


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--data-dir", default="data")
    ap.add_argument("--output", default="")
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--model", choices=["small", "minivgg"], default="small")
    ap.add_argument("--hidden", type=int, default=64)
    ap.add_argument("--channels", type=int, default=8)
    ap.add_argument("--vgg-base-channels", type=int, default=32)
    ap.add_argument("--init-scale", type=float, default=0.5)
    ap.add_argument("--lr", type=float, default=0.001)
    ap.add_argument("--adam-eps", type=float, default=1e-8)
    ap.add_argument("--adam-beta1", type=float, default=0.9)
    ap.add_argument("--adam-beta2", type=float, default=0.999)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--decay-bias", action="store_true")
    ap.add_argument("--optimizer", choices=["adam", "sgd"], default="adam")
    ap.add_argument("--augment", action="store_true")
    ap.add_argument("--lr-schedule", choices=["none", "step", "cosine"], default="none")
    ap.add_argument("--lr-step-epochs", default="")
    ap.add_argument("--lr-gamma", type=float, default=0.1)
    ap.add_argument("--min-lr", type=float, default=0.0)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--disable-shuffle", action="store_true")
    ap.add_argument("--train-limit", type=int, default=0)
    ap.add_argument("--test-limit", type=int, default=0)
    ap.add_argument("--synthetic", action="store_true")
    return ap.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    ob.manual_seed(args.seed)
    data = None if args.synthetic else load_cifar(args.data_dir)
    source = "cifar10"
    if data is None:
        source = "synthetic"
        data = synthetic_images(args.train_limit or 512, args.test_limit or 128, args.seed)
    tx, ty, vx, vy = data
    if args.train_limit:
        tx, ty = tx[:args.train_limit], ty[:args.train_limit]
    if args.test_limit:
        vx, vy = vx[:args.test_limit], vy[:args.test_limit]
    model = make_model(args)
    model.to(args.device)
    if args.optimizer == "adam":
        optimizer = ob.optim.Adam(model.parameters(), lr=args.lr, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_eps,
                                  weight_decay=args.weight_decay, decay_bias=args.decay_bias)
    else:
        optimizer = ob.optim.SGD(model.parameters(), lr=args.lr, weight_decay=args.weight_decay, decay_bias=args.decay_bias)
    step_epochs = parse_step_epochs(args.lr_step_epochs)
    rng = np.random.default_rng(args.seed)
    history = []
    start = time.perf_counter()
    for epoch in range(1, args.epochs + 1):
        lr = apply_lr_schedule(optimizer, args, epoch, step_epochs)
        train = run_epoch(model, tx, ty, optimizer, args, rng, True)
        test = run_epoch(model, vx, vy, optimizer, args, rng, False)
        history.append({"epoch": epoch, "lr": lr, "train": train, "test": test})
        print(f"epoch {epoch} lr {lr:.6g}: train loss {train['loss']:.4f} acc {train['accuracy']:.3f} | "
              f"test loss {test['loss']:.4f} acc {test['accuracy']:.3f}")
    result = {"example": "cifar10_cnn", "data": source, "model": args.model, "device": args.device, "history": history,
              "seconds": time.perf_counter() - start}
    if args.output:
        os.makedirs(os.path.dirname(os.path.abspath(args.output)), exist_ok=True)
        with open(args.output, "w") as f:
            json.dump(result, f, indent=2)
    return result


if __name__ == "__main__":
    main()
