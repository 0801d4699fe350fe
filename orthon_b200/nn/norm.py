"""LayerNorm (one fused kernel each way) and BatchNorm1d/2d (running statistics as buffers).
(reference project: python/orthon/nn/layernorm.py:34-90, python/orthon/nn/batchnorm.py:17-143)"""
from .. import _C
from ..functional import layer_norm
from .module import Module, Parameter


def _no_grad():
    import orthon_b200 as ob
    return ob.no_grad()


class LayerNorm(Module):
    def __init__(self, normalized_shape, eps=1e-5, elementwise_affine=True, device=None):
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(int(v) for v in normalized_shape)
        if len(self.normalized_shape) != 1 or self.normalized_shape[0] <= 0:
            raise ValueError("LayerNorm normalises one positive trailing dimension")
        self.eps = float(eps)
        self.elementwise_affine = bool(elementwise_affine)
        if self.elementwise_affine:
            w, b = _C.ones(list(self.normalized_shape)), _C.zeros(list(self.normalized_shape))
            if device is not None:
                w, b = w.to(device), b.to(device)
            self.weight, self.bias = Parameter(w), Parameter(b)

    def forward(self, x):
        w = self.weight if self.elementwise_affine else None
        b = self.bias if self.elementwise_affine else None
        return layer_norm(x, self.normalized_shape, weight=w, bias=b, eps=self.eps)


def _mean_over(t, dims):
    for d in sorted(dims, reverse=True):
        t = t.mean(d, True)
    return t


class _BatchNorm(Module):
    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True):
        super().__init__()
        self.num_features, self.eps = int(num_features), float(eps)
        self.momentum, self.affine = float(momentum), bool(affine)
        if affine:
            self.weight = Parameter(_C.ones([self.num_features]))
            self.bias = Parameter(_C.zeros([self.num_features]))
        self.register_buffer("running_mean", _C.zeros([self.num_features]))
        self.register_buffer("running_var", _C.ones([self.num_features]))

    def _axes(self, ndim):
        raise NotImplementedError

    def _stat_shape(self, ndim):
        raise NotImplementedError

    def _snapshot(self, stat, like):
        with _no_grad():
            out = stat.reshape([self.num_features]).to(like.device)
            if out.dtype != like.dtype:
                out = _C.cast(out, like.dtype)
        return out

    def forward(self, x):
        if x.shape[1] != self.num_features:
            raise ValueError(f"expected {self.num_features} channels, got {x.shape[1]}")
        shape = list(self._stat_shape(x.ndim))
        if self.training:
            dims = self._axes(x.ndim)
            count = 1
            for d in dims:
                count *= int(x.shape[d])
            if count < 2:
                raise ValueError(f"Expected more than 1 value per channel when training, got input size {list(x.shape)}")
            mean = _mean_over(x, dims)
            centered = x - mean
            var = _mean_over(centered * centered, dims)  # biased variance normalises
            bm, bv = self._snapshot(mean, self.running_mean), self._snapshot(var, self.running_var)
            keep = 1.0 - self.momentum
            with _no_grad():  # the running variance tracks the unbiased estimate
                self.running_mean = self.running_mean * keep + bm * self.momentum
                self.running_var = self.running_var * keep + (bv * (count / (count - 1))) * self.momentum
        else:
            mean, var = self.running_mean.reshape(shape), self.running_var.reshape(shape)
            centered = x - mean
        y = centered * _C.reciprocal(_C.sqrt(var + self.eps))
        if self.affine:
            y = y * self.weight.reshape(shape) + self.bias.reshape(shape)
        return y


class BatchNorm1d(_BatchNorm):
    def _axes(self, ndim):
        if ndim not in (2, 3):
            raise ValueError("BatchNorm1d expects [N, C] or [N, C, L] input")
        return (0,) if ndim == 2 else (0, 2)

    def _stat_shape(self, ndim):
        return (1, self.num_features) if ndim == 2 else (1, self.num_features, 1)


class BatchNorm2d(_BatchNorm):
    def _axes(self, ndim):
        if ndim != 4:
            raise ValueError("BatchNorm2d expects [N, C, H, W] input")
        return (0, 2, 3)

    def _stat_shape(self, ndim):
        return (1, self.num_features, 1, 1)
