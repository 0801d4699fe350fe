"""Activation modules (reference project: python/orthon/nn/activations.py)."""
from .. import _C
from .module import Module


class ReLU(Module):
    def forward(self, x):
        return _C.relu(x)


class Sigmoid(Module):
    def forward(self, x):
        return _C.sigmoid(x)


class Tanh(Module):
    def forward(self, x):
        return _C.tanh(x)


class LeakyReLU(Module):
    def __init__(self, negative_slope: float = 0.01):
        super().__init__()
        self.negative_slope = float(negative_slope)

    def forward(self, x):
        return _C.leaky_relu(x, self.negative_slope)


class GELU(Module):
    """Exact (erf) GELU."""

    def forward(self, x):
        return _C.gelu(x)
