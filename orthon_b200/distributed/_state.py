"""The process-wide active group (reference project: python/orthon/distributed/_state.py)."""
_active = None


def set_active(group):
    global _active
    _active = group


def get_active():
    if _active is None:
        raise RuntimeError("distributed process group is not initialized")
    return _active


def clear_active():
    global _active
    _active = None


def is_initialized():
    return _active is not None
