"""Functional forms of composite operators.
(reference project: python/orthon/functional/math.py:39-96, functional/shape.py)"""
import math as _math

from .. import _C
from .._random import randbits as _randbits


def layer_norm(tensor, normalized_shape, weight=None, bias=None, eps=1e-5):
    """Normalises the last dimension with one fused kernel (mean / rstd kept for backward)."""
    if isinstance(normalized_shape, int):
        normalized_shape = (normalized_shape,)
    normalized_shape = tuple(int(v) for v in normalized_shape)
    if len(normalized_shape) != 1:
        raise ValueError("layer_norm normalises the last dimension only")
    if tensor.shape[-1] != normalized_shape[0]:
        raise ValueError(
            f"layer_norm: normalized_shape {normalized_shape} does not match input shape {tuple(tensor.shape)}")
    return _C._layer_norm(tensor, weight, bias, float(eps))


def causal_mask(length, dtype="float32", device="cpu", fill=-1e9):
    """Additive [T, T] mask with `fill` above the diagonal."""
    import numpy as np
    m = np.triu(np.full((length, length), fill, dtype=np.float32), k=1)
    t = _C.from_numpy(m, dtype)
    return t if str(device) == "cpu" else t.to(device)


def scaled_dot_product_attention(q, k, v, mask=None, dropout_p=0.0, training=True, is_causal=False, seed=None):
    """softmax(q kᵀ / sqrt(d) + mask) v for [N, T, D] or [B, H, T, D] operands.

    The score scaling, additive mask, optional in-kernel causal mask and softmax are one
    kernel; scores stay in the operand dtype instead of a float32 [B·H, T, T] tensor."""
    if not 0.0 <= dropout_p < 1.0:
        raise ValueError("dropout_p must be in [0, 1)")
    scale = 1.0 / _math.sqrt(q.shape[-1])
    p = float(dropout_p) if training else 0.0
    if p > 0.0 and seed is None:
        seed = _randbits(64)
    return _C._attention(q, k, v, mask, bool(is_causal), scale, p, int(seed or 0))


def flatten(tensor, start_dim=0, end_dim=-1):
    return tensor.flatten(start_dim, end_dim)


from .._C import (  # noqa: E402,F401
    relu, sigmoid, tanh, leaky_relu, gelu, softmax, log_softmax, cross_entropy, nll_loss,
    dropout, embedding, conv2d, maxpool2d, linear, fused_linear_relu, matmul,
)


def exp(x):
    return x.exp()


def sum(x, dim=None, keepdim=False):  # noqa: A001 - mirrors the tensor method
    return x.sum(dim, keepdim)


def mean(x, dim=None, keepdim=False):
    return x.mean(dim, keepdim)


def max(x, dim=None, keepdim=False):  # noqa: A001
    return x.max(dim, keepdim)


def argmax(x, dim=None, keepdim=False):
    return x.argmax(dim, keepdim)
