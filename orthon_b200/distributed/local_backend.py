"""Host multiprocessing transport and the `spawn` supervisor.

Every collective is an all-gather of (descriptor, payload bytes) through the shared store
followed by a local reduction in rank order, so every rank computes bit-identical results.
Ranks that disagree on the descriptor (kind, shape, dtype, source) abort the whole group; all
waits are bounded (30 s) and an abort raised by one rank or by the supervisor reaches the
others on their next poll.
(reference project: python/orthon/distributed/local_backend.py:13-234)"""
import json
import multiprocessing as mp
import struct
import traceback

import numpy as np

from . import group as _group
from .group import Backend, Work, _TransportFailure
from .store import ManagerStore, Store, StoreTimeout

COLLECTIVE_TIMEOUT_SECONDS = 30.0
_NP = {"float32": np.float32, "float64": np.float64, "float16": np.float16, "int32": np.int32, "int64": np.int64,
       "uint8": np.uint8, "int8": np.int8, "bool": np.bool_}


def _pack(descriptor, payload):
    head = json.dumps(descriptor).encode()
    return struct.pack("<I", len(head)) + head + (payload or b"")


def _unpack(blob):
    (n,) = struct.unpack("<I", blob[:4])
    return json.loads(blob[4:4 + n].decode()), blob[4 + n:]


class LocalBackend(Backend):
    def __init__(self, rank: int, world_size: int, store, timeout=COLLECTIVE_TIMEOUT_SECONDS):
        if world_size < 1:
            raise ValueError("world_size must be >= 1")
        if rank < 0 or rank >= world_size:
            raise ValueError("rank must be in [0, world_size)")
        if store is None:
            raise ValueError("local backend requires a shared multiprocessing store")
        self._rank, self._world = int(rank), int(world_size)
        self._store = store if isinstance(store, Store) else ManagerStore(store)
        self._timeout = float(timeout)
        self._seq, self._closed, self._failure = 0, False, None
        # A per-rank generation keeps a re-initialised group away from stale keys.
        self._gen = self._store.add(f"generation/{self._rank}", 1) - 1

    rank = property(lambda self: self._rank)
    world_size = property(lambda self: self._world)

    def _open(self):
        if self._closed:
            raise RuntimeError("local distributed backend has been shut down")
        if self._failure is not None:
            raise _TransportFailure("local distributed backend failed: " + self._failure)

    @staticmethod
    def _check(tensor, reduction):
        if not tensor.is_contiguous:
            raise RuntimeError("local collectives require contiguous tensors")
        ok = {"float32", "float64", "float16", "int32", "int64", "uint8", "int8"} | (set() if reduction else {"bool"})
        if tensor.dtype not in ok:
            raise RuntimeError(f"local collective does not support dtype {tensor.dtype}")

    def _fail(self, message):
        self._failure = str(message)
        raise _TransportFailure(self._failure)

    def _gather(self, descriptor, payload):
        """Returns the payload bytes of every rank, in rank order."""
        prefix = f"g{self._gen}/c{self._seq}"
        abort_key = f"g{self._gen}/abort"
        self._seq += 1
        self._store.set(f"{prefix}/r{self._rank}", _pack(descriptor, payload))
        keys = [f"{prefix}/r{r}" for r in range(self._world)]
        try:
            aborted = self._store.wait_for(keys, self._timeout, abort_keys=("spawn:abort", abort_key))
        except StoreTimeout:
            message = f"timed out waiting for local collective {prefix}"
            self._store.set(abort_key, message.encode())
            self._fail(message)
        if aborted is not None:
            self._fail(aborted.decode() if isinstance(aborted, bytes) else str(aborted))
        parts = [_unpack(self._store.get(k)) for k in keys]
        descriptors = [d for d, _ in parts]
        if any(d != descriptor for d in descriptors):
            message = f"local collective mismatch at sequence {self._seq - 1}: {descriptors}"
            self._store.set(abort_key, message.encode())
            self._fail(message)
        if self._store.add(f"{prefix}/leave", 1) == self._world:  # last one out cleans up
            for k in keys + [f"{prefix}/leave"]:
                self._store.delete(k)
        return [p for _, p in parts]

    @staticmethod
    def _bytes_of(tensor):
        from .. import _C
        return _C._tensor_to_bytes(tensor)

    @staticmethod
    def _write_back(tensor, data):
        import orthon_b200 as ob
        from .. import _C
        src = _C._tensor_from_bytes(data, list(tensor.shape), tensor.dtype)
        if tensor.device.is_cuda():
            src = src.to(tensor.device)
        with ob.no_grad():
            tensor._copy_flat_range_from(0, src.reshape([-1]) if src.ndim != 1 else src, 0, int(tensor.numel))

    def all_reduce(self, tensor, op="sum", async_op=False):
        self._open()
        if op != "sum":
            raise NotImplementedError("local backend only supports all_reduce op='sum'")
        self._check(tensor, True)
        desc = ["all_reduce", list(tensor.shape), tensor.dtype, None]
        parts = self._gather(desc, self._bytes_of(tensor))
        total = np.frombuffer(parts[0], dtype=_NP[tensor.dtype]).copy()
        for p in parts[1:]:
            total += np.frombuffer(p, dtype=_NP[tensor.dtype])
        self._write_back(tensor, total.tobytes())
        return Work() if async_op else tensor

    def broadcast(self, tensor, src=0, async_op=False):
        self._open()
        if src < 0 or src >= self._world:
            raise ValueError("broadcast src must be in [0, world_size)")
        self._check(tensor, False)
        desc = ["broadcast", list(tensor.shape), tensor.dtype, src]
        parts = self._gather(desc, self._bytes_of(tensor) if self._rank == src else b"")
        self._write_back(tensor, parts[src])
        return Work() if async_op else tensor

    def barrier(self):
        self._open()
        self._gather(["barrier", [], None, None], b"")

    def exchange_objects(self, value: bytes):
        self._open()
        return self._gather(["objects", [], None, None], value)

    def shutdown(self):
        self._closed = True


def create_store(ctx=None):
    ctx = ctx or mp.get_context("spawn")
    return ManagerStore.create(ctx)


def _abort(handles, message):
    ManagerStore(handles).set("spawn:abort", message.encode())


def _worker(rank, world_size, backend, handles, fn, args, results, errors):
    import orthon_b200.distributed as dist
    try:
        kwargs = dict(backend=backend, rank=rank, world_size=world_size, store=handles)
        if backend in ("nccl", "p2p"):
            kwargs["device"] = rank
        dist.init_process_group(**kwargs)
        results[rank] = fn(rank, *args)
    except BaseException:
        text = traceback.format_exc()
        errors[rank] = text
        _abort(handles, f"rank {rank} failed: {text}")
        raise
    finally:
        dist.destroy_process_group()


def spawn(fn, args=(), nprocs=2, backend="local"):
    """Runs `fn(rank, *args)` in `nprocs` fresh processes, returns the rank-ordered results.
    The first failing worker aborts the shared store; survivors are terminated, then killed."""
    if nprocs < 1:
        raise ValueError("nprocs must be >= 1")
    if _group.is_active():
        raise RuntimeError("cannot spawn while distributed is already initialized")
    ctx = mp.get_context("spawn")
    manager, handles = create_store(ctx)
    procs = []
    try:
        results, errors = manager.list([None] * nprocs), manager.dict()
        for rank in range(nprocs):
            p = ctx.Process(target=_worker, args=(rank, nprocs, backend, handles, fn, args, results, errors))
            p.start()
            procs.append(p)
        while any(p.is_alive() for p in procs):
            if errors or any(p.exitcode not in (None, 0) for p in procs):
                break
            for p in procs:
                p.join(timeout=0.05)
        failed = dict(errors)
        bad = [(r, p.exitcode) for r, p in enumerate(procs) if p.exitcode not in (None, 0)]
        if failed or bad:
            lines = [f"rank {r} failed:\n{tb}" for r, tb in sorted(failed.items())]
            lines += [f"rank {r} exited with code {code}" for r, code in bad]
            raise RuntimeError("local distributed spawn failed\n" + "\n".join(lines))
        return list(results)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=2)
            if p.is_alive():
                p.kill()
                p.join(timeout=2)
        manager.shutdown()


__all__ = ["LocalBackend", "create_store", "spawn"]
