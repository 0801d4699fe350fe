"""Pointwise activation modules: parameter-free wrappers around the native operators.

Each class names the operator it applies; `_Pointwise.forward` looks it up once per call, so a
new activation is one line.  GELU is the exact (erf) form, like the native kernel.
(reference project: python/orthon/nn/activations.py)"""
from .. import _C
from .module import Module


class _Pointwise(Module):
    """Applies `_C.<operator>` element by element; subclasses set `operator` (and `arguments()` when the
    operator takes more than the tensor)."""

    operator = None

    def arguments(self):
        return ()

    def forward(self, tensor):
        return getattr(_C, self.operator)(tensor, *self.arguments())

    def __repr__(self):
        inner = ", ".join(repr(a) for a in self.arguments())
        return f"{type(self).__name__}({inner})"


def _pointwise(class_name, operator, doc):
    return type(class_name, (_Pointwise,), {"operator": operator, "__doc__": doc, "__module__": __name__})


ReLU = _pointwise("ReLU", "relu", "max(x, 0)")
Sigmoid = _pointwise("Sigmoid", "sigmoid", "1 / (1 + exp(-x))")
Tanh = _pointwise("Tanh", "tanh", "Hyperbolic tangent.")
GELU = _pointwise("GELU", "gelu", "x * Phi(x) with the exact normal CDF (erf), not the tanh approximation.")


class LeakyReLU(_Pointwise):
    """x for x > 0, negative_slope * x otherwise."""

    operator = "leaky_relu"

    def __init__(self, negative_slope: float = 0.01):
        super().__init__()
        self.negative_slope = float(negative_slope)

    def arguments(self):
        return (self.negative_slope,)


__all__ = ["ReLU", "Sigmoid", "Tanh", "LeakyReLU", "GELU"]
