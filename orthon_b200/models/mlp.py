"""MLP 784 -> 256 -> 128 -> 10 with ReLU (reference project: examples/mnist_mlp.py)."""
from .. import nn


class MLP(nn.Module):
    def __init__(self, sizes=(784, 256, 128, 10)):
        super().__init__()
        layers = []
        for i in range(len(sizes) - 1):
            layers.append(nn.Linear(sizes[i], sizes[i + 1]))
            if i + 2 < len(sizes):
                layers.append(nn.ReLU())
        self.net = nn.Sequential(*layers)

    def forward(self, x):
        return self.net(x)
