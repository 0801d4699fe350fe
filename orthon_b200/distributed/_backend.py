"""Transport extension point: the Backend interface and the name -> factory registry.
Built-ins: "local" (host processes over a shared store), "nccl" (NCCL through the native
process group) and "p2p" (peer-memory kernels over NVLink with NCCL for generic collectives).
(reference project: python/orthon/distributed/_backend.py:8-113)"""
from abc import ABC, abstractmethod


class _TransportFailure(RuntimeError):
    """A collective entered its ordering sequence and failed; the group is poisoned."""


class Backend(ABC):
    @property
    @abstractmethod
    def rank(self):
        ...

    @property
    @abstractmethod
    def world_size(self):
        ...

    @abstractmethod
    def all_reduce(self, tensor, op="sum", async_op=False):
        ...

    @abstractmethod
    def broadcast(self, tensor, src=0, async_op=False):
        ...

    @abstractmethod
    def barrier(self):
        ...

    @abstractmethod
    def shutdown(self):
        ...


_BACKENDS = {}


def register_backend(name, factory):
    if not isinstance(name, str) or not name:
        raise ValueError("backend name must be a non-empty string")
    if not callable(factory):
        raise TypeError("backend factory must be callable")
    _BACKENDS[name] = factory


def get_backend_factory(name):
    if name not in _BACKENDS:
        known = ", ".join(sorted(_BACKENDS)) or "<none>"
        raise ValueError(f"unknown distributed backend: {name!r}; available backends: {known}")
    return _BACKENDS[name]


class _SingleRankBackend(Backend):
    def __init__(self, *args, **kwargs):
        self._closed = False

    def _open(self):
        if self._closed:
            raise RuntimeError("single-rank backend has been shut down")

    rank = property(lambda self: 0)
    world_size = property(lambda self: 1)

    def all_reduce(self, tensor, op="sum", async_op=False):
        self._open()
        if async_op:
            from .work import _CompletedWork
            return _CompletedWork()
        return tensor

    def broadcast(self, tensor, src=0, async_op=False):
        self._open()
        if src != 0:
            raise ValueError("single-rank backend only supports src=0")
        if async_op:
            from .work import _CompletedWork
            return _CompletedWork()
        return tensor

    def barrier(self):
        self._open()

    def shutdown(self):
        self._closed = True


def _local_factory(**kw):
    from .local_backend import LocalBackend
    if kw.get("store") is None:
        # Launched ranks (no spawn parent to hand over a store): the launcher's file store or a
        # MASTER_ADDR / MASTER_PORT rendezvous.
        from .store import store_from_env
        kw["store"] = store_from_env(kw.get("rank"), kw.get("world_size"))
    return LocalBackend(**kw)


def _nccl_factory(**kw):
    from .nccl_backend import NcclBackend
    return NcclBackend(**kw)


def _p2p_factory(**kw):
    from .p2p_backend import PeerBackend
    return PeerBackend(**kw)


register_backend("local", _local_factory)
register_backend("nccl", _nccl_factory)
register_backend("p2p", _p2p_factory)

__all__ = ["Backend", "_SingleRankBackend", "_BACKENDS", "register_backend", "get_backend_factory"]
