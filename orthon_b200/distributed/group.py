"""Core objects of the distributed package, in one place.

* `Work`           completion handle of one collective.  Concrete: it is built from up to three
                   callables (wait, probe, on_failure), so a transport never has to subclass it
                   and a finished collective is simply `Work()`.
* `Backend`        the transport extension point (rank, world_size, all_reduce, broadcast,
                   barrier, shutdown) and the registry that maps names to factories.
* `GroupHandle`    what DDP, AMP and the facade hold on to: it owns the group's lifetime (open /
                   shut down), its failure state (a transport failure is sticky: every later use
                   is refused) and the access to the backend's rendezvous store.
* the active handle of the process (`activate`, `active`, `deactivate`, `is_active`).

Contracts follow the reference project's python/orthon/distributed/{_backend,_process_group,
_state,work}.py; the structure is this package's own.
"""
from abc import ABC, abstractmethod


class _TransportFailure(RuntimeError):
    """A collective entered its ordering sequence and failed: the ranks are no longer in step."""


class Work:
    """Handle of an asynchronous collective.

    `wait()` blocks until the collective is done and returns True; `is_completed()` never blocks.
    Once either has observed completion the handle is settled and forgets its callables, so the
    transport objects behind them can be released.  An exception from the transport is reported
    to `on_failure` (the owning group poisons itself) and re-raised.
    """

    __slots__ = ("_wait", "_probe", "_on_failure", "_settled")

    def __init__(self, wait=None, probe=None, on_failure=None):
        self._wait, self._probe, self._on_failure = wait, probe, on_failure
        self._settled = wait is None and probe is None

    def _settle(self):
        self._settled, self._wait, self._probe, self._on_failure = True, None, None, None

    def _guarded(self, call):
        try:
            return call()
        except Exception as exc:  # noqa: BLE001
            if self._on_failure is not None:
                self._on_failure(str(exc))
            raise

    def wait(self):
        if not self._settled:
            if self._wait is not None:
                self._guarded(self._wait)
            self._settle()
        return True

    def is_completed(self):
        if self._settled:
            return True
        if self._probe is None:
            return False
        if self._guarded(self._probe):
            self._settle()
            return True
        return False

    def watched_by(self, on_failure):
        """The same collective, reporting transport errors to `on_failure` as well."""
        if self._settled:
            return self
        return Work(self._wait, self._probe, on_failure)


class Backend(ABC):
    """Transport interface.  `all_reduce` / `broadcast` work in place and return the tensor, or a
    `Work` when `async_op` is true; `shutdown` is idempotent."""

    @property
    @abstractmethod
    def rank(self):
        """This process's rank in [0, world_size)."""

    @property
    @abstractmethod
    def world_size(self):
        """Number of ranks of the group."""

    @abstractmethod
    def all_reduce(self, tensor, op="sum", async_op=False):
        """Element-wise reduction over all ranks, result on every rank."""

    @abstractmethod
    def broadcast(self, tensor, src=0, async_op=False):
        """Every rank receives rank `src`'s values."""

    @abstractmethod
    def barrier(self):
        """Returns once every rank has entered."""

    @abstractmethod
    def shutdown(self):
        """Releases the transport; further collectives are refused."""


class BackendRegistry:
    """Name -> factory table.  A factory is called with the keyword arguments of
    `init_process_group` (rank, world_size, device, store, ...) and returns a Backend."""

    def __init__(self):
        self._factories = {}

    def register(self, name, factory):
        if not isinstance(name, str) or not name:
            raise ValueError("backend name must be a non-empty string")
        if not callable(factory):
            raise TypeError("backend factory must be callable")
        self._factories[name] = factory

    def lookup(self, name):
        factory = self._factories.get(name)
        if factory is None:
            listed = ", ".join(sorted(self._factories)) or "<none>"
            raise ValueError(f"unknown distributed backend: {name!r}; available backends: {listed}")
        return factory

    def names(self):
        return tuple(sorted(self._factories))


backends = BackendRegistry()
register_backend = backends.register
get_backend_factory = backends.lookup


class _SingleRankBackend(Backend):
    """World of one: every collective is the identity."""

    rank, world_size = 0, 1

    def __init__(self, *unused, **also_unused):
        self._down = False

    def _collective(self, tensor, async_op):
        if self._down:
            raise RuntimeError("single-rank backend has been shut down")
        return Work() if async_op else tensor

    def all_reduce(self, tensor, op="sum", async_op=False):
        return self._collective(tensor, async_op)

    def broadcast(self, tensor, src=0, async_op=False):
        if src != 0:
            raise ValueError("single-rank backend only supports src=0")
        return self._collective(tensor, async_op)

    def barrier(self):
        self._collective(None, False)

    def shutdown(self):
        self._down = True


class GroupHandle:
    """A process group as its users see it.  States: open -> (failed) -> shut down.

    * open: collectives are forwarded to the backend;
    * failed: a `_TransportFailure` escaped from the backend or from one of its `Work` handles;
      the reason is kept and every later collective raises "distributed process group failed";
    * shut down: `shutdown()` ran (once); every later use raises.
    Objects that captured the handle (DDP, AMP optimizers) therefore notice a torn-down or broken
    group even if a new group has been initialised since.
    """

    def __init__(self, backend):
        self._backend = backend
        self.rank, self.world_size = backend.rank, backend.world_size
        self._down = False
        self._failure = None

    backend = property(lambda self: self._backend)
    failure = property(lambda self: self._failure)

    def poison(self, reason):
        if self._failure is None:
            self._failure = str(reason)

    def ensure_open(self):
        if self._down:
            raise RuntimeError("distributed process group has been shut down")
        if self._failure is not None:
            raise RuntimeError("distributed process group failed: " + self._failure)

    def _collective(self, method, *args, async_op=None, **kwargs):
        self.ensure_open()
        if async_op is not None:
            kwargs["async_op"] = async_op
        try:
            result = method(*args, **kwargs)
        except _TransportFailure as exc:
            self.poison(exc)
            raise
        if async_op and isinstance(result, Work):
            return result.watched_by(self.poison)
        return result

    def all_reduce(self, tensor, op="sum", async_op=False):
        return self._collective(self._backend.all_reduce, tensor, op=op, async_op=bool(async_op))

    def broadcast(self, tensor, src=0, async_op=False):
        return self._collective(self._backend.broadcast, tensor, src=src, async_op=bool(async_op))

    def barrier(self):
        return self._collective(self._backend.barrier)

    def validate_gradient_dtype(self, dtype):
        """Backends may restrict the gradient dtypes they can average (hook `_validate_gradient_dtype`)."""
        check = getattr(self._backend, "_validate_gradient_dtype", None)
        if check is not None:
            check(dtype)

    def exchange_objects(self, value):
        """All-gather of one small bytes value per rank through the backend's rendezvous store."""
        self.ensure_open()
        return self._backend.exchange_objects(value)

    def shutdown(self):
        if self._down:
            return None
        self._down = True
        return self._backend.shutdown()


_current = None


def activate(handle):
    global _current
    _current = handle


def deactivate():
    global _current
    _current = None


def is_active():
    return _current is not None


def active():
    if _current is None:
        raise RuntimeError("distributed process group is not initialized")
    return _current


def _builtin(module, cls, needs_store=False):
    def factory(**kwargs):
        import importlib
        backend_cls = getattr(importlib.import_module(module, __package__), cls)
        if needs_store and kwargs.get("store") is None:
            # Launched ranks have no spawn parent to hand over a store: use the launcher's file
            # store or a MASTER_ADDR / MASTER_PORT rendezvous.
            from .store import store_from_env
            kwargs["store"] = store_from_env(kwargs.get("rank"), kwargs.get("world_size"))
        return backend_cls(**kwargs)
    return factory


register_backend("local", _builtin(".local_backend", "LocalBackend", needs_store=True))
register_backend("nccl", _builtin(".nccl_backend", "NcclBackend"))
register_backend("p2p", _builtin(".p2p_backend", "PeerBackend"))

__all__ = ["Backend", "BackendRegistry", "GroupHandle", "Work", "backends", "register_backend", "get_backend_factory",
           "activate", "deactivate", "active", "is_active"]
