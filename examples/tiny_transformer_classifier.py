"""Sequence classification with a small pre-LayerNorm transformer encoder: token + position
embeddings, two encoder blocks, mean pooling, linear head.  Synthetic task: the label is the
most frequent of four marker tokens in the sequence.  Runs on the CPU by default.

    python examples/tiny_transformer_classifier.py [--device cuda:0] [--steps 60]
"""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
from orthon_b200 import nn  # noqa: E402


class Classifier(nn.Module):
    def __init__(self, vocab=32, seq=16, dim=32, heads=4, layers=2, classes=4):
        super().__init__()
        self.tok = nn.Embedding(vocab, dim)
        self.pos = nn.Embedding(seq, dim)
        self.blocks = nn.Sequential(*[nn.TransformerEncoderBlock(dim, heads, 4 * dim) for _ in range(layers)])
        self.norm = nn.LayerNorm(dim)
        self.head = nn.Linear(dim, classes)
        self.seq = seq

    def forward(self, ids, positions):
        x = self.tok(ids) + self.pos(positions)
        x = self.norm(self.blocks(x))
        return self.head(x.mean(1))


def make_batch(rng, n, seq, vocab, classes, device):
    ids = rng.integers(classes, vocab, size=(n, seq))
    labels = rng.integers(0, classes, n)
    for i, c in enumerate(labels):  # plant the label's marker token five times
        ids[i, rng.choice(seq, 5, replace=False)] = c
    pos = np.tile(np.arange(seq), (n, 1))
    to = (lambda a: ob.from_numpy(a.astype(np.int64)).to(device))
    return to(ids), to(pos), [int(v) for v in labels]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--steps", type=int, default=60)
    a = ap.parse_args()
    ob.manual_seed(0)
    model = Classifier()
    model.to(a.device)
    opt = ob.optim.Adam(model.parameters(), lr=3e-3)
    rng = np.random.default_rng(0)
    for step in range(a.steps):
        ids, pos, y = make_batch(rng, 32, 16, 32, 4, a.device)
        opt.zero_grad()
        logits = model(ids, pos)
        loss = ob.cross_entropy(logits, y)
        loss.backward()
        opt.step()
        if step % 10 == 0 or step == a.steps - 1:
            print(f"step {step:3d} loss {loss.item():.4f} acc {ob.training.classification_accuracy(logits, y):.2f}")
    return float(loss.item())


if __name__ == "__main__":
    main()
