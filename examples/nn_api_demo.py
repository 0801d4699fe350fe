"""Tour of the nn API on the CPU: explicit registries, tied parameters, buffers, train/eval,
dtype and device transforms that keep Parameter identity, state_dict round trip with rollback on a
bad load, and a MiniVGG-style CNN (Conv2d, BatchNorm2d, MaxPool2d, Flatten, Dropout).

    python examples/nn_api_demo.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
from orthon_b200 import nn  # noqa: E402


class MiniVGG(nn.Module):
    def __init__(self, classes=10):
        super().__init__()
        self.features = nn.Sequential(
            nn.Conv2d(3, 8, 3, padding=1), nn.BatchNorm2d(8), nn.ReLU(), nn.MaxPool2d(2),
            nn.Conv2d(8, 16, 3, padding=1), nn.BatchNorm2d(16), nn.ReLU(), nn.MaxPool2d(2))
        self.classifier = nn.Sequential(nn.Flatten(), nn.Dropout(0.25), nn.Linear(16 * 8 * 8, classes))

    def forward(self, x):
        return self.classifier(self.features(x))


class Tied(nn.Module):
    """Input and output projections share one weight matrix (counted once by parameters())."""

    def __init__(self, vocab=12, dim=6):
        super().__init__()
        self.emb = nn.Embedding(vocab, dim)
        self.register_buffer("calls", ob.zeros([1]))

    def forward(self, ids):
        h = self.emb(ids).mean(1)
        return h @ self.emb.weight.transpose(0, 1)


def main():
    ob.manual_seed(0)
    net = MiniVGG()
    names = [n for n, _ in net.named_parameters()]
    print(len(names), "parameters, e.g.", names[:3], "| buffers:", [n for n, _ in net.named_buffers()][:2])
    x = ob.from_numpy(np.random.default_rng(0).standard_normal((4, 3, 32, 32)).astype(np.float32))
    net.train()
    loss = ob.cross_entropy(net(x), [1, 2, 3, 4])
    loss.backward()
    net.eval()
    print("train loss", round(loss.item(), 4), "| eval logits row 0:", [round(v, 3) for v in net(x).tolist()[:3]])

    first = next(iter(net.parameters()))
    net.cast("float64")
    assert next(iter(net.parameters())) is first and first.dtype == "float64"  # identity survives the transform
    net.cast("float32")

    state = net.state_dict()
    other = MiniVGG()
    other.load_state_dict(state)
    bad = dict(state)
    bad.pop(next(iter(bad)))
    try:
        other.load_state_dict(bad)
    except (KeyError, RuntimeError, ValueError) as exc:
        print("rejected incomplete state:", type(exc).__name__)
    other.eval()
    assert other(x).tolist() == net(x).tolist()  # the failed load changed nothing

    tied = Tied()
    assert len(list(tied.parameters())) == 1
    ids = ob.from_numpy(np.asarray([[1, 2, 3], [4, 5, 6]], dtype=np.int64))
    tied(ids).sum().backward()
    print("tied weight gradient norm", round(float((tied.emb.weight.grad * tied.emb.weight.grad).sum().item()) ** 0.5, 4))


if __name__ == "__main__":
    main()
