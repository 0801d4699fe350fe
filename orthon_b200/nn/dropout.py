"""Inverted dropout whose mask is a pure function of (seed, call number, element index).

The mask of element i in the c-th training call of a module is drawn from
splitmix64(seed + c * 0x9E3779B97F4A7C15 + i): nothing is stored between forward and backward
(the CUDA kernel recomputes the mask from the per-call seed), and the CPU and CUDA kernels agree
bit for bit.  (reference project: python/orthon/nn/dropout.py:9-31)"""
from .. import _C
from .._random import randbits
from .module import Module


class _CallSeeds:
    """The per-call seed stream of one module: seed + n * golden ratio, modulo 2^64."""

    STEP = 0x9E3779B97F4A7C15
    WRAP = 1 << 64

    def __init__(self, base):
        self.base = int(base) % self.WRAP
        self.calls = 0

    def take(self):
        value = (self.base + self.calls * self.STEP) % self.WRAP
        self.calls += 1
        return value


class Dropout(Module):
    def __init__(self, p: float = 0.5, seed=None):
        super().__init__()
        if not 0.0 <= p < 1.0:
            raise ValueError("Dropout p must be in [0, 1)")
        self.p = float(p)
        self._seeds = _CallSeeds(randbits(64) if seed is None else seed)

    # The reference exposes the base seed and the call counter as attributes; keep both readable.
    @property
    def seed(self):
        return self._seeds.base

    @property
    def _counter(self):
        return self._seeds.calls

    def _next_seed(self):
        return self._seeds.take()

    def forward(self, x):
        active = self.training and self.p > 0.0
        return _C.dropout(x, self.p, self._seeds.take()) if active else x
