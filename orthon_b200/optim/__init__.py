"""Optimizers (reference project: python/orthon/optim/__init__.py)."""
from .sgd import SGD  # noqa: F401
from .adam import Adam  # noqa: F401
