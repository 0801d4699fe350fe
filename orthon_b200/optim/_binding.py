"""Parameter capture shared by the optimizers: strong references to the Python owners, one
binding per owner, duplicates rejected.  (reference project: python/orthon/optim/_binding.py)"""
from .. import _C


class Binding:
    __slots__ = ("parameter", "state")

    def __init__(self, parameter, state=None):
        self.parameter = parameter
        self.state = state


def capture_bindings(params):
    owners = list(params)
    seen = set()
    for i, p in enumerate(owners):
        if not isinstance(p, _C.Tensor):
            raise TypeError(f"optimizer parameter {i} must be a Tensor")
        if id(p) in seen:
            raise ValueError(f"duplicate optimizer parameter owner at index {i}")
        seen.add(id(p))
    return tuple(Binding(p) for p in owners)


def no_grad():
    import orthon_b200 as ob
    return ob.no_grad()
