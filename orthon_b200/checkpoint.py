"""File APIs over the single v1 serializer.
(reference project: python/orthon/checkpoint.py:12-29)"""
from ._serialization.format import FORMAT_ID, FORMAT_VERSION  # noqa: F401
from ._serialization import service as _service


def save_checkpoint(path, model=None, optimizer=None, metadata=None):
    return _service.save_checkpoint(path, model, optimizer, metadata)


def load_checkpoint(path, model=None, optimizer=None, map_location=None):
    return _service.load_checkpoint(path, model, optimizer, map_location)


def save_state_dict(model, path):
    save_checkpoint(path, model=model)


def load_state_dict(model, path, map_location=None):
    load_checkpoint(path, model=model, map_location=map_location)
