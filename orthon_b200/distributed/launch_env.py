"""What a launcher tells a rank through the environment: RANK, WORLD_SIZE, LOCAL_RANK,
LOCAL_WORLD_SIZE and ORTHON_DISTRIBUTED_BACKEND.  `init_process_group` uses it to fill in
arguments the caller left out.  (reference project: python/orthon/distributed/_env.py:17-51)"""
import os
from dataclasses import dataclass
from typing import Optional

BACKEND_ENV = "ORTHON_DISTRIBUTED_BACKEND"
DEVICE_BACKENDS = frozenset({"nccl", "p2p"})  # transports that bind one GPU per rank
_INTEGER_FIELDS = (("rank", "RANK"), ("world_size", "WORLD_SIZE"), ("local_rank", "LOCAL_RANK"),
                   ("local_world_size", "LOCAL_WORLD_SIZE"))


@dataclass(frozen=True)
class LaunchEnvironment:
    rank: Optional[int] = None
    world_size: Optional[int] = None
    local_rank: Optional[int] = None
    local_world_size: Optional[int] = None
    backend: Optional[str] = None

    @classmethod
    def read(cls, environ=None):
        source = os.environ if environ is None else environ
        values = {}
        for field, variable in _INTEGER_FIELDS:
            text = source.get(variable)
            if text in (None, ""):
                continue
            try:
                values[field] = int(text)
            except ValueError:
                raise ValueError(f"{variable} must be an integer, got {text!r}") from None
        return cls(backend=source.get(BACKEND_ENV), **values)

    def complete(self, backend, kwargs):
        """(backend, kwargs) with the gaps filled from the environment.  Explicit arguments win;
        a device-bound backend defaults its device to the local rank."""
        chosen = self.backend if backend is None else backend
        if chosen is None:
            raise ValueError(f"distributed backend must be provided explicitly or via {BACKEND_ENV}")
        filled = dict(kwargs)
        defaults = {"rank": self.rank, "world_size": self.world_size}
        if chosen in DEVICE_BACKENDS:
            defaults["device"] = self.local_rank
        for key, value in defaults.items():
            if filled.get(key) is None and value is not None:
                filled[key] = value
        return chosen, filled


def rank_config_from_env(environ=None):
    env = LaunchEnvironment.read(environ)
    return {"rank": env.rank, "world_size": env.world_size, "local_rank": env.local_rank,
            "local_world_size": env.local_world_size, "backend": env.backend}


def apply_env_defaults(backend, kwargs, environ=None):
    return LaunchEnvironment.read(environ).complete(backend, kwargs)


__all__ = ["LaunchEnvironment", "apply_env_defaults", "rank_config_from_env", "BACKEND_ENV"]
