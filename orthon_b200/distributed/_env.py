"""Launcher-style environment defaults: RANK, WORLD_SIZE, LOCAL_RANK, LOCAL_WORLD_SIZE and
ORTHON_DISTRIBUTED_BACKEND.  (reference project: python/orthon/distributed/_env.py:17-51)"""
import os

BACKEND_ENV = "ORTHON_DISTRIBUTED_BACKEND"
_DEVICE_BACKENDS = ("nccl", "p2p")


def _int_or_none(environ, name):
    raw = environ.get(name)
    if raw is None or raw == "":
        return None
    try:
        return int(raw)
    except ValueError:
        raise ValueError(f"{name} must be an integer, got {raw!r}") from None


def rank_config_from_env(environ=None):
    environ = os.environ if environ is None else environ
    return {"rank": _int_or_none(environ, "RANK"), "world_size": _int_or_none(environ, "WORLD_SIZE"),
            "local_rank": _int_or_none(environ, "LOCAL_RANK"), "local_world_size": _int_or_none(environ, "LOCAL_WORLD_SIZE"),
            "backend": environ.get(BACKEND_ENV)}


def apply_env_defaults(backend, kwargs, environ=None):
    cfg = rank_config_from_env(environ)
    backend = backend if backend is not None else cfg["backend"]
    if backend is None:
        raise ValueError(f"distributed backend must be provided explicitly or via {BACKEND_ENV}")
    out = dict(kwargs)
    for key in ("rank", "world_size"):
        if out.get(key) is None and cfg[key] is not None:
            out[key] = cfg[key]
    if backend in _DEVICE_BACKENDS and out.get("device") is None and cfg["local_rank"] is not None:
        out["device"] = cfg["local_rank"]
    return backend, out


__all__ = ["apply_env_defaults", "rank_config_from_env"]
