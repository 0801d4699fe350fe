"""Bag-of-embeddings text classifier on a synthetic two-topic corpus: Embedding, mean over the
sequence, Dropout, Linear; trained with SGD, evaluated with the training helpers, then saved and
reloaded through the checkpoint format.

    python examples/tiny_text_classifier.py
"""
import os
import sys
import tempfile

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
from orthon_b200 import nn  # noqa: E402


class BagOfEmbeddings(nn.Module):
    def __init__(self, vocab=50, dim=16, classes=2):
        super().__init__()
        self.emb = nn.Embedding(vocab, dim)
        self.drop = nn.Dropout(0.1)
        self.out = nn.Linear(dim, classes)

    def forward(self, ids):
        return self.out(self.drop(self.emb(ids).mean(1)))


def corpus(rng, n, seq=12, vocab=50):
    labels = rng.integers(0, 2, n)
    ids = np.where(labels[:, None] == 0, rng.integers(0, vocab // 2, (n, seq)), rng.integers(vocab // 2, vocab, (n, seq)))
    noise = rng.random((n, seq)) < 0.2
    ids = np.where(noise, rng.integers(0, vocab, (n, seq)), ids)
    return ob.from_numpy(ids.astype(np.int64)), [int(v) for v in labels]


def main():
    ob.manual_seed(0)
    rng = np.random.default_rng(0)
    model = BagOfEmbeddings()
    opt = ob.optim.SGD(model.parameters(), lr=0.5)
    for epoch in range(15):
        x, y = corpus(rng, 64)
        m = ob.training.train_step(model, x, y, ob.cross_entropy, opt)
    evals = [ob.training.eval_step(model, *corpus(rng, 32), ob.cross_entropy) for _ in range(4)]
    summary = ob.training.weighted_metric_average(evals)
    print("train loss", round(m["loss"], 4), "eval", {k: round(v, 4) for k, v in summary.items()})
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "text.ckpt")
        ob.save_checkpoint(path, model, opt)
        clone = BagOfEmbeddings()
        ob.load_checkpoint(path, clone)
        clone.eval(); model.eval()
        x, _ = corpus(rng, 8)
        assert clone(x).tolist() == model(x).tolist()
    return summary["accuracy"]


if __name__ == "__main__":
    main()
