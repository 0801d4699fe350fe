"""Fully connected layers.  The weight is stored [in_features, out_features] and the whole
layer (GEMM + bias + optional activation) is one tcgen05 kernel launch on CUDA.
(reference project: python/orthon/nn/linear.py:8-43)"""
import math

from .. import _C
from .._random import uniform_array
from .module import Module, Parameter


def kaiming_uniform(shape, fan_in):
    bound = math.sqrt(6.0 / fan_in)
    return _C.from_numpy(uniform_array(tuple(shape), -bound, bound))


class Linear(Module):
    def __init__(self, in_features, out_features, bias=True):
        super().__init__()
        self.in_features, self.out_features = int(in_features), int(out_features)
        self.weight = Parameter(kaiming_uniform((self.in_features, self.out_features), self.in_features))
        if bias:
            self.bias = Parameter(_C.zeros([self.out_features]))
        else:
            self.bias = None

    def forward(self, x):
        return _C.linear(x, self.weight, self.bias)


class FusedLinearReLU(Module):
    """relu(x @ W + b) with the activation applied in the GEMM epilogue."""

    def __init__(self, in_features, out_features):
        super().__init__()
        self.weight = Parameter(kaiming_uniform((int(in_features), int(out_features)), int(in_features)))
        self.bias = Parameter(_C.zeros([int(out_features)]))

    def forward(self, x):
        return _C.fused_linear_relu(x, self.weight, self.bias)
