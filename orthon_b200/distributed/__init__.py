"""Distributed facade: process-group lifecycle, collectives, `spawn`, DDP.

One group is active per process.  `init_process_group` builds the transport named by `backend`
(arguments the caller leaves out come from the launcher environment), wraps it in a
`GroupHandle` and returns the transport, as the reference does
(python/orthon/distributed/__init__.py:14-88).
"""
from . import group as _group
from .group import Backend, Work, register_backend, get_backend_factory  # noqa: F401
from .launch_env import LaunchEnvironment, apply_env_defaults, rank_config_from_env  # noqa: F401


def init_process_group(backend=None, **kwargs):
    if _group.is_active():
        raise RuntimeError("distributed process group is already initialized")
    name, arguments = LaunchEnvironment.read().complete(backend, kwargs)
    transport = get_backend_factory(name)(**arguments)
    _group.activate(_group.GroupHandle(transport))
    return transport


def destroy_process_group():
    if _group.is_active():
        handle = _group.active()
        try:
            handle.shutdown()
        finally:
            _group.deactivate()


def is_initialized():
    return _group.is_active()


def get_rank():
    return _group.active().rank


def get_world_size():
    return _group.active().world_size


def barrier():
    return _group.active().barrier()


def all_reduce(tensor, op="sum", async_op=False):
    return _group.active().all_reduce(tensor, op=op, async_op=async_op)


def broadcast(tensor, src=0, async_op=False):
    return _group.active().broadcast(tensor, src=src, async_op=async_op)


def spawn(fn, args=(), nprocs=2, backend="local"):
    from .local_backend import spawn as _spawn
    return _spawn(fn, args=args, nprocs=nprocs, backend=backend)


from ..parallel.ddp import DistributedDataParallel, DDP  # noqa: E402,F401

__all__ = ["init_process_group", "destroy_process_group", "is_initialized", "get_rank", "get_world_size", "barrier",
           "all_reduce", "broadcast", "spawn", "Backend", "register_backend", "Work", "DistributedDataParallel", "DDP"]
