"""Rendezvous stores shared by the host-side transports: a key -> bytes map with an atomic
counter and bounded waits.  ManagerStore lives in a multiprocessing manager (used by `spawn`),
FileStore in a directory (used by the launcher, reference project:
python/orthon/distributed/nccl_backend.py:154-177), TorchStore wraps torch.distributed's
TCPStore when a torchrun-style MASTER_ADDR/MASTER_PORT environment is present."""
import os
import time


class StoreTimeout(RuntimeError):
    pass


class Store:
    def set(self, key, value: bytes):
        raise NotImplementedError

    def get(self, key):
        """bytes, or None when the key is absent."""
        raise NotImplementedError

    def add(self, key, amount=1) -> int:
        raise NotImplementedError

    def delete(self, key):
        raise NotImplementedError

    def wait_for(self, keys, timeout, abort_keys=()):
        """Blocks until every key exists.  Returns the abort value if an abort key shows up first."""
        deadline = time.monotonic() + timeout
        pause = 0.0005
        while True:
            for ak in abort_keys:
                v = self.get(ak)
                if v is not None:
                    return v
            if all(self.get(k) is not None for k in keys):
                return None
            if time.monotonic() > deadline:
                raise StoreTimeout("timed out waiting for " + ", ".join(keys))
            time.sleep(pause)
            pause = min(pause * 1.5, 0.02)


class ManagerStore(Store):
    def __init__(self, handles):
        self._cond, self._values = handles["condition"], handles["values"]

    @staticmethod
    def create(ctx):
        manager = ctx.Manager()
        return manager, {"condition": manager.Condition(), "values": manager.dict()}

    def set(self, key, value):
        with self._cond:
            self._values[key] = value
            self._cond.notify_all()

    def get(self, key):
        return self._values.get(key)

    def add(self, key, amount=1):
        with self._cond:
            v = int(self._values.get(key, 0)) + amount
            self._values[key] = v
            self._cond.notify_all()
            return v

    def delete(self, key):
        with self._cond:
            self._values.pop(key, None)

    def wait_for(self, keys, timeout, abort_keys=()):
        deadline = time.monotonic() + timeout
        with self._cond:
            while True:
                for ak in abort_keys:
                    v = self._values.get(ak)
                    if v is not None:
                        return v
                if all(k in self._values for k in keys):
                    return None
                left = deadline - time.monotonic()
                if left <= 0:
                    raise StoreTimeout("timed out waiting for " + ", ".join(keys))
                self._cond.wait(timeout=min(left, 0.1))


class FileStore(Store):
    """One file per key, written to a temporary name and renamed so readers never see a torn value."""

    def __init__(self, directory):
        self._dir = directory
        os.makedirs(directory, exist_ok=True)

    def _path(self, key):
        return os.path.join(self._dir, key.replace("/", "__"))

    def set(self, key, value):
        tmp = self._path(key) + f".tmp{os.getpid()}"
        with open(tmp, "wb") as f:
            f.write(value if isinstance(value, bytes) else str(value).encode())
        os.replace(tmp, self._path(key))

    def get(self, key):
        try:
            with open(self._path(key), "rb") as f:
                return f.read()
        except FileNotFoundError:
            return None

    def add(self, key, amount=1):
        import fcntl
        lock = self._path(key) + ".lock"
        with open(lock, "a+") as lf:
            fcntl.flock(lf, fcntl.LOCK_EX)
            cur = self.get(key)
            v = (int(cur) if cur else 0) + amount
            self.set(key, str(v).encode())
            fcntl.flock(lf, fcntl.LOCK_UN)
        return v

    def delete(self, key):
        try:
            os.unlink(self._path(key))
        except FileNotFoundError:
            pass


class TorchStore(Store):
    """torch.distributed.TCPStore as plumbing (rank 0 hosts it)."""

    def __init__(self, host, port, rank, world_size, timeout=60.0):
        from datetime import timedelta
        import torch.distributed as dist
        self._store = dist.TCPStore(host, int(port), world_size, is_master=(rank == 0),
                                    timeout=timedelta(seconds=timeout), wait_for_workers=False)

    def set(self, key, value):
        self._store.set(key, value if isinstance(value, bytes) else str(value).encode())

    def get(self, key):
        if not self._store.check([key]):
            return None
        return bytes(self._store.get(key))

    def add(self, key, amount=1):
        return int(self._store.add(key, amount))

    def delete(self, key):
        try:
            self._store.delete_key(key)
        except Exception:  # noqa: BLE001
            pass


_PROCESS_STORES = {}


def store_from_env(rank, world_size, environ=None):
    """ORTHON_STORE_DIR (set by the launcher) wins; otherwise a torchrun-style rendezvous."""
    environ = os.environ if environ is None else environ
    directory = environ.get("ORTHON_STORE_DIR") or environ.get("ORTHON_NCCL_STORE_DIR")
    if directory:
        return FileStore(directory)
    host, port = environ.get("MASTER_ADDR"), environ.get("MASTER_PORT")
    if host and port:
        # A second port keeps clear of the launcher's own rendezvous store.  The connection (and on
        # rank 0 the server) lives as long as the process: a group that is destroyed and created
        # again finds the same store, told apart by the generation counters the backends keep in
        # it, and a rank that is already rejoining never talks to a server that is being torn down.
        key = (host, int(port) + 17, int(rank), int(world_size))
        if key not in _PROCESS_STORES:
            _PROCESS_STORES[key] = TorchStore(*key)
        return _PROCESS_STORES[key]
    raise RuntimeError("no rendezvous available: set ORTHON_STORE_DIR or MASTER_ADDR/MASTER_PORT, or pass store=")
