"""Lifetime / failure wrapper captured by DDP and AMP: a group that was shut down or whose
transport failed rejects every further call.
(reference project: python/orthon/distributed/_process_group.py:5-68)"""
from ._backend import _TransportFailure
from .work import Work


class _TransportWork(Work):
    def __init__(self, work, group):
        self._work, self._group = work, group

    def _forward(self, name):
        try:
            return getattr(self._work, name)()
        except Exception as exc:  # noqa: BLE001
            self._group._failure = str(exc)
            raise

    def wait(self):
        return self._forward("wait")

    def is_completed(self):
        return self._forward("is_completed")


class _ProcessGroup:
    def __init__(self, backend):
        self._backend = backend
        self.rank, self.world_size = backend.rank, backend.world_size
        self._closed, self._failure = False, None

    @property
    def backend(self):
        return self._backend

    def ensure_open(self):
        if self._closed:
            raise RuntimeError("distributed process group has been shut down")
        if self._failure is not None:
            raise RuntimeError("distributed process group failed: " + self._failure)

    def _call(self, name, *args, **kwargs):
        self.ensure_open()
        try:
            result = getattr(self._backend, name)(*args, **kwargs)
        except _TransportFailure as exc:
            self._failure = str(exc)
            raise
        return _TransportWork(result, self) if kwargs.get("async_op") else result

    def all_reduce(self, tensor, op="sum", async_op=False):
        return self._call("all_reduce", tensor, op=op, async_op=async_op)

    def broadcast(self, tensor, src=0, async_op=False):
        return self._call("broadcast", tensor, src=src, async_op=async_op)

    def barrier(self):
        return self._call("barrier")

    def validate_gradient_dtype(self, dtype):
        check = getattr(self._backend, "_validate_gradient_dtype", None)
        if check is not None:
            check(dtype)

    def exchange_objects(self, obj):
        """All-gather of small picklable-free values (bytes/str/int) through the backend's store."""
        self.ensure_open()
        return self._backend.exchange_objects(obj)

    def shutdown(self):
        if self._closed:
            return None
        self._closed = True
        return self._backend.shutdown()
