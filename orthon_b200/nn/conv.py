"""Conv2d and MaxPool2d over NCHW tensors.
(reference project: python/orthon/nn/conv2d.py:8-61, python/orthon/nn/pooling.py:5-27)"""
from .. import _C
from .linear import kaiming_uniform
from .module import Module, Parameter


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


class Conv2d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, bias=True):
        super().__init__()
        kh, kw = _pair(kernel_size)
        self._stride, self._padding = _pair(stride), _pair(padding)
        self._use_bias = bool(bias)
        self._out_channels = int(out_channels)
        self.weight = Parameter(kaiming_uniform((int(out_channels), int(in_channels), kh, kw), int(in_channels) * kh * kw))
        if bias:
            self.bias = Parameter(_C.zeros([int(out_channels)]))

    def forward(self, x):
        (sh, sw), (ph, pw) = self._stride, self._padding
        return _C.conv2d(x, self.weight, self.bias if self._use_bias else None, sh, sw, ph, pw)


class MaxPool2d(Module):
    def __init__(self, kernel_size, stride=None, padding=0):
        super().__init__()
        self.kernel_size = _pair(kernel_size)
        self.stride = self.kernel_size if stride is None else _pair(stride)
        self.padding = _pair(padding)

    def forward(self, x):
        (kh, kw), (sh, sw), (ph, pw) = self.kernel_size, self.stride, self.padding
        return _C.maxpool2d(x, kh, kw, sh, sw, ph, pw)
