"""Sequential and Flatten (reference project: python/orthon/nn/{sequential,flatten}.py)."""
from .module import Module


class Sequential(Module):
    def __init__(self, *modules):
        super().__init__()
        for i, m in enumerate(modules):
            self._register_module(str(i), m)

    def __len__(self):
        return len(self._modules)

    def __getitem__(self, i):
        return list(self._modules.values())[i]

    def __iter__(self):
        return iter(self._modules.values())

    def forward(self, x):
        for m in self._modules.values():
            x = m(x)
        return x


class Flatten(Module):
    def __init__(self, start_dim: int = 1, end_dim: int = -1):
        super().__init__()
        self.start_dim, self.end_dim = int(start_dim), int(end_dim)

    def forward(self, x):
        return x.flatten(self.start_dim, self.end_dim)
