"""Embedding lookup (reference project: python/orthon/nn/embedding.py:10-68)."""
import math

import numpy as np

from .. import _C
from .._random import uniform_array
from .module import Module, Parameter


def _as_indices(values, device):
    if isinstance(values, _C.Tensor):
        return values
    t = _C.from_numpy(np.ascontiguousarray(np.asarray(values, dtype=np.int64)))
    return t.to(device) if device is not None and device.is_cuda() else t


def embedding(indices, weight, padding_idx=None):
    return _C.embedding(_as_indices(indices, weight.device), weight)


class Embedding(Module):
    def __init__(self, num_embeddings, embedding_dim, padding_idx=None, device=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim = int(num_embeddings), int(embedding_dim)
        if self.num_embeddings <= 0:
            raise ValueError("num_embeddings must be positive")
        if self.embedding_dim <= 0:
            raise ValueError("embedding_dim must be positive")
        if padding_idx is not None:
            padding_idx = int(padding_idx)
            if padding_idx < 0:
                padding_idx += self.num_embeddings
            if not 0 <= padding_idx < self.num_embeddings:
                raise ValueError("padding_idx must be within num_embeddings")
        self.padding_idx = padding_idx
        bound = 1.0 / math.sqrt(self.num_embeddings)
        table = uniform_array((self.num_embeddings, self.embedding_dim), -bound, bound)
        if padding_idx is not None:
            table[padding_idx] = 0.0
        w = _C.from_numpy(table)
        if device is not None:
            w = w.to(device)
        self.weight = Parameter(w)

    def forward(self, input):  # noqa: A002 - keyword name of the reference API
        indices = input
        return embedding(indices, self.weight, self.padding_idx)
