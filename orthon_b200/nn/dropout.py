"""Inverted dropout with a stateless splitmix64 mask: element i of call c uses
splitmix64(seed + c * 0x9E3779B97F4A7C15 + i), identical on CPU and CUDA.
(reference project: python/orthon/nn/dropout.py:9-31)"""
from .. import _C
from .._random import randbits
from .module import Module

_GOLDEN = 0x9E3779B97F4A7C15
_MASK64 = (1 << 64) - 1


class Dropout(Module):
    def __init__(self, p: float = 0.5, seed=None):
        super().__init__()
        if p < 0.0 or p >= 1.0:
            raise ValueError("Dropout p must be in [0, 1)")
        self.p = float(p)
        self.seed = int(seed) if seed is not None else randbits(64)
        self._counter = 0

    def _next_seed(self):
        seed = (self.seed + self._counter * _GOLDEN) & _MASK64
        self._counter += 1
        return seed

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        return _C.dropout(x, self.p, self._next_seed())
