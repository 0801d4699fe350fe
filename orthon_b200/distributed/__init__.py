"""Distributed facade: process-group lifecycle, collectives, `spawn`, DDP.
(reference project: python/orthon/distributed/__init__.py:14-88)"""
from . import _state
from ._backend import Backend, register_backend, get_backend_factory, _SingleRankBackend  # noqa: F401
from ._env import apply_env_defaults, rank_config_from_env  # noqa: F401
from ._process_group import _ProcessGroup
from .work import Work  # noqa: F401


def init_process_group(backend=None, **kwargs):
    """Creates the process-wide group.  Missing rank / world_size / device come from the
    launcher environment; `backend` may come from ORTHON_DISTRIBUTED_BACKEND."""
    if _state.is_initialized():
        raise RuntimeError("distributed process group is already initialized")
    backend, kwargs = apply_env_defaults(backend, kwargs)
    transport = get_backend_factory(backend)(**kwargs)
    _state.set_active(_ProcessGroup(transport))


def destroy_process_group():
    if not _state.is_initialized():
        return
    group = _state.get_active()
    try:
        group.shutdown()
    finally:
        _state.clear_active()


def is_initialized():
    return _state.is_initialized()


def get_rank():
    return _state.get_active().rank


def get_world_size():
    return _state.get_active().world_size


def barrier():
    return _state.get_active().barrier()


def all_reduce(tensor, op="sum", async_op=False):
    return _state.get_active().all_reduce(tensor, op=op, async_op=async_op)


def broadcast(tensor, src=0, async_op=False):
    return _state.get_active().broadcast(tensor, src=src, async_op=async_op)


def spawn(fn, args=(), nprocs=2, backend="local"):
    from .local_backend import spawn as _spawn
    return _spawn(fn, args=args, nprocs=nprocs, backend=backend)


from ..parallel.ddp import DistributedDataParallel, DDP  # noqa: E402,F401

__all__ = ["init_process_group", "destroy_process_group", "is_initialized", "get_rank", "get_world_size", "barrier",
           "all_reduce", "broadcast", "spawn", "Backend", "register_backend", "Work", "DistributedDataParallel", "DDP"]
