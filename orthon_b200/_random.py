"""Process-local random stream used for module initialisation and default dropout seeds.

``manual_seed`` only resets this stream: Python's ``random``, NumPy, PyTorch and device
state are untouched, and existing tensors never change.
(reference project: python/orthon/_random.py:10-30)
"""
import random as _random

import numpy as _np

_stream = _random.Random()


def manual_seed(seed):
    _stream.seed(int(seed))


def uniform(low, high):
    return _stream.uniform(low, high)


def randbits(bits):
    return _stream.getrandbits(bits)


def uniform_array(shape, low, high):
    """Vectorised draw: one 64-bit value from the stream seeds a NumPy generator, so large
    parameters initialise in O(1) Python calls while staying reproducible under manual_seed."""
    gen = _np.random.default_rng(_stream.getrandbits(64))
    return gen.uniform(low, high, size=shape).astype(_np.float32)


def normal_array(shape, std):
    gen = _np.random.default_rng(_stream.getrandbits(64))
    return (gen.standard_normal(size=shape) * std).astype(_np.float32)
