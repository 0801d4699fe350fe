"""NCCL transport: the native process group (one communicator, one communication stream)
behind the Backend interface.  The unique id travels through a rendezvous store: the shared
multiprocessing store handed over by `spawn`, a directory named by ORTHON_STORE_DIR (set by the
launcher), or torch.distributed's TCPStore under a torchrun-style environment.
(reference project: python/orthon/distributed/nccl_backend.py:16-201)"""
import importlib.util
import os

from .. import _C
from .group import Backend, Work, _TransportFailure
from .store import ManagerStore, Store, store_from_env

RENDEZVOUS_TIMEOUT_SECONDS = 60.0
_SUPPORTED = ("float32", "float16", "bfloat16")


def _bundled_nccl():
    """Path of the NCCL that ships with the installed torch wheel, if any (newer than the system one)."""
    try:
        spec = importlib.util.find_spec("nvidia.nccl")
    except (ImportError, ValueError):
        return ""
    if spec is None or not spec.submodule_search_locations:
        return ""
    for base in spec.submodule_search_locations:
        cand = os.path.join(base, "lib", "libnccl.so.2")
        if os.path.exists(cand):
            return cand
    return ""


def _NativeWork(native):
    """Public handle over the native process group's Work (event-backed, polls the communicator)."""
    return Work(wait=native.wait, probe=native.is_completed)


class NcclBackend(Backend):
    def __init__(self, rank=None, world_size=None, device=None, store=None, fake=False):
        if rank is None or world_size is None:
            raise ValueError("nccl backend requires rank and world_size")
        if world_size < 1 or not 0 <= rank < world_size:
            raise ValueError("rank must be in [0, world_size)")
        if not fake:
            # The copy that ships with the Python environment goes first: a process that later
            # imports PyTorch (the MASTER_ADDR rendezvous store does) must not already hold an
            # older system libnccl under the same soname.
            path = _bundled_nccl()
            if path:
                _C._nccl_load(path)
            if not _C.nccl_enabled():
                raise RuntimeError("this build cannot load NCCL")
        self._rank, self._world = int(rank), int(world_size)
        self._device = int(rank if device is None else device)
        if not fake and self._device >= _C.cuda_device_count():
            raise ValueError(f"nccl backend: cuda:{self._device} is not visible")
        if store is None:
            self._store = store_from_env(self._rank, self._world)
        else:
            self._store = store if isinstance(store, Store) else ManagerStore(store)
        self._generation = self._store.add(f"nccl/generation/{self._rank}", 1) - 1
        self._xseq = 0
        uid_key = f"nccl/uid/{self._generation}"
        if self._rank == 0:
            uid = bytes(128) if fake else _C._nccl_unique_id()
            self._store.set(uid_key, uid)
        self._store.wait_for([uid_key], RENDEZVOUS_TIMEOUT_SECONDS)
        uid = self._store.get(uid_key)
        self._group = _C._NcclGroup(self._rank, self._world, self._device, uid, fake)
        self._closed = False

    rank = property(lambda self: self._rank)
    world_size = property(lambda self: self._world)
    device = property(lambda self: self._device)

    def _open(self):
        if self._closed:
            raise RuntimeError("nccl backend has been shut down")

    def _check(self, tensor):
        if not tensor.device.is_cuda():
            raise RuntimeError("nccl collectives require CUDA tensors")
        if tensor.device.index != self._device:
            raise RuntimeError(f"tensor is on {tensor.device} but this rank owns cuda:{self._device}")
        if not tensor.is_contiguous:
            raise RuntimeError("nccl collectives require contiguous tensors")
        if tensor.dtype not in _SUPPORTED:
            raise RuntimeError(f"nccl collectives support {_SUPPORTED}, got {tensor.dtype}")

    def _run(self, fn, *args, async_op=False):
        try:
            work = fn(*args)
        except (ValueError, TypeError):
            raise
        except RuntimeError as exc:
            if "failed" in str(exc):
                raise _TransportFailure(str(exc)) from exc
            raise
        if async_op:
            return _NativeWork(work)
        try:
            work.wait()
        except RuntimeError as exc:
            raise _TransportFailure(str(exc)) from exc
        return None

    def all_reduce(self, tensor, op="sum", async_op=False):
        self._open()
        if op != "sum":
            raise NotImplementedError("nccl backend only supports all_reduce op='sum'")
        self._check(tensor)
        out = self._run(self._group.all_reduce, tensor, async_op=async_op)
        return out if async_op else tensor

    def broadcast(self, tensor, src=0, async_op=False):
        self._open()
        if not 0 <= src < self._world:
            raise ValueError("broadcast src must be in [0, world_size)")
        self._check(tensor)
        out = self._run(self._group.broadcast, tensor, src, async_op=async_op)
        return out if async_op else tensor

    def barrier(self):
        self._open()
        try:
            self._group.barrier()
        except RuntimeError as exc:
            raise _TransportFailure(str(exc)) from exc

    def exchange_objects(self, value: bytes):
        """All-gather of one bytes value per rank through the rendezvous store."""
        prefix = f"nccl/x/{self._generation}/{self._xseq}"
        self._xseq += 1
        self._store.set(f"{prefix}/r{self._rank}", value)
        keys = [f"{prefix}/r{r}" for r in range(self._world)]
        self._store.wait_for(keys, RENDEZVOUS_TIMEOUT_SECONDS)
        out = [self._store.get(k) for k in keys]
        if self._store.add(f"{prefix}/leave", 1) == self._world:
            for k in keys + [f"{prefix}/leave"]:
                self._store.delete(k)
        return out

    def _validate_gradient_dtype(self, dtype):
        if dtype not in _SUPPORTED:
            raise RuntimeError(f"nccl gradient synchronization supports {_SUPPORTED}, got {dtype}")

    def shutdown(self):
        if self._closed:
            return
        self._closed = True
        self._group.shutdown()


__all__ = ["NcclBackend"]
