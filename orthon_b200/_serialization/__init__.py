"""Pickle-free ``ml-runtime-checkpoint`` v1 container (format spec: the reference project's
docs/checkpoint_format.md)."""
