"""MLP 784-hidden-10 on MNIST (or on a synthetic stand-in with the same shapes).

    python examples/mnist_mlp.py --epochs 1 --hidden 128 --optimizer adam
    python examples/mnist_mlp.py --synthetic --train-limit 2048 --test-limit 512 --device cuda

The images are read from the four IDX files of the original distribution
(`train-images-idx3-ubyte[.gz]`, ...) under `--data-dir`; nothing is downloaded.  With
`--synthetic`, or when the files are absent, ten fixed random prototypes plus noise stand in for
the digits so the script stays runnable on a machine without the dataset.  Results (per-epoch
loss / accuracy, wall time) are written as JSON to `--output`.
(reference project: examples/mnist_mlp.py:25-165)
"""
import argparse
import gzip
import json
import os
import struct
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
from orthon_b200 import nn  # noqa: E402


def read_idx(path):
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rb") as f:
        magic = struct.unpack(">I", f.read(4))[0]
        rank = magic & 0xFF
        dims = struct.unpack(">" + "I" * rank, f.read(4 * rank))
        return np.frombuffer(f.read(), dtype=np.uint8).reshape(dims)


def find_idx(data_dir, stem):
    for root in (data_dir, os.path.join(data_dir, "MNIST", "raw")):
        for name in (stem, stem + ".gz"):
            path = os.path.join(root, name)
            if os.path.exists(path):
                return path
    return None


def load_mnist(data_dir):
    stems = ["train-images-idx3-ubyte", "train-labels-idx1-ubyte", "t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte"]
    paths = [find_idx(data_dir, s) for s in stems]
    if any(p is None for p in paths):
        return None
    tx, ty, vx, vy = (read_idx(p) for p in paths)

    def norm(images):
        return ((images.reshape(len(images), -1).astype(np.float32) / 255.0) - 0.1307) / 0.3081

    return norm(tx), ty.astype(np.int64), norm(vx), vy.astype(np.int64)


def synthetic_digits(n_train, n_test, seed):
    rng = np.random.default_rng(seed)
    prototypes = rng.standard_normal((10, 784)).astype(np.float32)

    def draw(n):
        labels = rng.integers(0, 10, n)
        return (prototypes[labels] + 0.8 * rng.standard_normal((n, 784))).astype(np.float32), labels.astype(np.int64)

    return (*draw(n_train), *draw(n_test))


def make_model(hidden):
    return nn.Sequential(nn.Linear(784, hidden), nn.ReLU(), nn.Linear(hidden, 10))


def make_optimizer(name, params, lr):
    return ob.optim.Adam(params, lr=lr) if name == "adam" else ob.optim.SGD(params, lr=lr)


def batches(x, y, batch_size, order=None):
    index = np.arange(len(x)) if order is None else order
    for start in range(0, len(index), batch_size):
        sel = index[start:start + batch_size]
        yield x[sel], y[sel]


def run_epoch(model, x, y, optimizer, batch_size, device, rng):
    outputs = []
    for bx, by in batches(x, y, batch_size, rng.permutation(len(x))):
        outputs.append(ob.training.train_step(model, ob.from_numpy(bx).to(device), by, ob.cross_entropy, optimizer))
    return ob.training.weighted_metric_average(outputs)


def evaluate(model, x, y, batch_size, device):
    with ob.no_grad():
        outputs = [ob.training.eval_step(model, ob.from_numpy(bx).to(device), by, ob.cross_entropy)
                   for bx, by in batches(x, y, batch_size)]
    return ob.training.weighted_metric_average(outputs)


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--data-dir", default="data")
    ap.add_argument("--output", default="")
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=128)
    ap.add_argument("--lr", type=float, default=0.001)
    ap.add_argument("--optimizer", choices=["adam", "sgd"], default="adam")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--train-limit", type=int, default=0, help="use only the first N training images (0 = all)")
    ap.add_argument("--test-limit", type=int, default=0)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--synthetic", action="store_true")
    return ap.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    ob.manual_seed(args.seed)
    data = None if args.synthetic else load_mnist(args.data_dir)
    source = "mnist"
    if data is None:
        source = "synthetic"
        data = synthetic_digits(args.train_limit or 4096, args.test_limit or 1024, args.seed)
    tx, ty, vx, vy = data
    if args.train_limit:
        tx, ty = tx[:args.train_limit], ty[:args.train_limit]
    if args.test_limit:
        vx, vy = vx[:args.test_limit], vy[:args.test_limit]
    model = make_model(args.hidden)
    model.to(args.device)
    optimizer = make_optimizer(args.optimizer, model.parameters(), args.lr)
    rng = np.random.default_rng(args.seed)
    history = []
    start = time.perf_counter()
    for epoch in range(args.epochs):
        train = run_epoch(model, tx, ty, optimizer, args.batch_size, args.device, rng)
        test = evaluate(model, vx, vy, args.batch_size, args.device)
        history.append({"epoch": epoch + 1, "train": train, "test": test})
        print(f"epoch {epoch + 1}: train loss {train['loss']:.4f} acc {train['accuracy']:.3f} | "
              f"test loss {test['loss']:.4f} acc {test['accuracy']:.3f}")
    result = {"example": "mnist_mlp", "data": source, "device": args.device, "hidden": args.hidden,
              "optimizer": args.optimizer, "lr": args.lr, "batch_size": args.batch_size, "history": history,
              "seconds": time.perf_counter() - start}
    if args.output:
        os.makedirs(os.path.dirname(os.path.abspath(args.output)), exist_ok=True)
        with open(args.output, "w") as f:
            json.dump(result, f, indent=2)
    return result


if __name__ == "__main__":
    main()
