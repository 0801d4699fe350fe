"""Checkpoint files: thin entry points over the one serializer (`_serialization.service`).

`save_checkpoint` / `load_checkpoint` handle a model, an optimizer and free-form metadata in one
archive; `save_state_dict` / `load_state_dict` are the model-only spellings.  The format is
`ml-runtime-checkpoint` version 1 (see docs/checkpoint_format.md).
(reference project: python/orthon/checkpoint.py:12-29)"""
from ._serialization import service
from ._serialization.format import FORMAT_ID, FORMAT_VERSION

__all__ = ["FORMAT_ID", "FORMAT_VERSION", "save_checkpoint", "load_checkpoint", "save_state_dict", "load_state_dict"]


def save_checkpoint(path, model=None, optimizer=None, metadata=None):
    """Writes the archive atomically; returns what the serializer returns (the path written)."""
    return service.save_checkpoint(path, model, optimizer, metadata)


def load_checkpoint(path, model=None, optimizer=None, map_location=None):
    """Validates the whole archive, then restores model and optimizer as one transaction."""
    return service.load_checkpoint(path, model, optimizer, map_location)


def save_state_dict(model, path):
    service.save_checkpoint(path, model, None, None)


def load_state_dict(model, path, map_location=None):
    service.load_checkpoint(path, model, None, map_location)
