"""Explicit mixed precision (reference project: python/orthon/amp/__init__.py)."""
from .grad_scaler import GradScaler  # noqa: F401
from .optimizer import MixedPrecisionOptimizer  # noqa: F401
