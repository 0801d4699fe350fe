"""DistributedDataParallel: replicated parameters, averaged gradients.

The wrapper owns one gradient synchroniser for the trainable parameters of a module (unique
owners, sorted by name so every rank agrees on the order) and wires it into autograd with two
callbacks: a per-parameter post-accumulate hook that reports "this parameter has its gradient"
and one keyed backward finalizer that runs the synchroniser once per backward pass.

Which synchroniser is chosen follows from where the parameters live:

* parameters of one dtype on one CUDA device under the peer-memory transport get the
  PeerReducer: their gradients live inside symmetric buckets and one fused kernel per bucket
  averages them over NVLink.  `overlap_grad_sync=True` launches a bucket from the hooks while
  backward is still running; otherwise all buckets are launched by the finalizer (or by
  `all_reduce_gradients()` when `sync_grads=False`), with the participation consensus carried in
  the kernel's entry barrier;
* everything else gets the generic Reducer (any backend, control all-reduce, packing).

Parameters are broadcast from `src` at construction; buffers are not.
(reference project: python/orthon/distributed/ddp.py:7-119)"""
import weakref

from ..distributed import group as _group
from .peer_reducer import PeerReducer
from .reducer import Reducer

_MODULE_API = ("named_parameters", "state_dict", "load_state_dict")


def _check_options(sync_grads, bucket_size_mb, overlap_grad_sync):
    if overlap_grad_sync:
        if not sync_grads:
            raise ValueError("overlap_grad_sync=True requires sync_grads=True")
        if bucket_size_mb is None:
            raise ValueError("overlap_grad_sync=True requires bucket_size_mb to be provided")
    if bucket_size_mb is not None and int(float(bucket_size_mb) * 1024 * 1024) < 1:
        raise ValueError("bucket_size_mb must be positive when provided")


def _trainable_owners(module):
    """(name, parameter) pairs: each trainable Python owner once, in sorted-name order."""
    if hasattr(module, "named_parameters"):
        pairs = sorted(module.named_parameters(), key=lambda pair: pair[0])
    else:
        pairs = [(str(index), p) for index, p in enumerate(module.parameters())]
        pairs.sort(key=lambda pair: pair[0])
    unique = {}
    for name, p in pairs:
        if p.requires_grad:
            unique.setdefault(id(p), (name, p))
    return list(unique.values())


class _AutogradLink:
    """Callbacks handed to autograd.  They hold the reducer weakly: a wrapper that was dropped
    leaves hooks behind on the parameters, and those must turn into no-ops."""

    def __init__(self, reducer):
        self._reducer = weakref.ref(reducer)
        self.key = id(reducer)

    def finalize(self):
        reducer = self._reducer()
        if reducer is not None:
            reducer.synchronize()

    def marker(self, parameter):
        owner, ref = id(parameter), self._reducer

        def mark():
            reducer = ref()
            if reducer is not None:
                reducer.mark(owner)

        return mark


class DistributedDataParallel:
    def __init__(self, module, src=0, sync_grads=True, bucket_size_mb=None, overlap_grad_sync=False):
        _check_options(sync_grads, bucket_size_mb, overlap_grad_sync)
        self.module = module
        self._sync_grads = bool(sync_grads)
        group = _group.active()
        owners = _trainable_owners(module)
        for _, parameter in owners:
            group.broadcast(parameter, src=src)
        if PeerReducer.eligible(owners, group):
            self._reducer = PeerReducer(owners, group, bucket_size_mb, overlap=bool(overlap_grad_sync))
        else:
            self._reducer = Reducer(owners, group, bucket_size_mb, bool(overlap_grad_sync))
        self._link = _AutogradLink(self._reducer)
        for _, parameter in owners:
            parameter._register_post_accumulate_grad_hook(self._link.marker(parameter))
            if self._sync_grads:
                parameter._register_backward_finalizer(self._link.key, self._link.finalize)

    # The finalizer is also keyed on the outputs, so a backward pass that reaches no parameter
    # of this rank still takes part in the synchronisation.
    def _attach_outputs(self, output):
        if not self._sync_grads:
            return
        pending = [output]
        while pending:
            value = pending.pop()
            if isinstance(value, dict):
                pending.extend(value.values())
            elif isinstance(value, (tuple, list)):
                pending.extend(value)
            elif hasattr(value, "_register_backward_finalizer") and value.requires_grad:
                value._register_backward_finalizer(self._link.key, self._link.finalize)

    def __call__(self, *args, **kwargs):
        self._reducer.group.ensure_open()
        output = self.module(*args, **kwargs)
        self._attach_outputs(output)
        return output

    forward = __call__

    # ------------------------------------------------------------ module API
    def parameters(self):
        return self.module.parameters()

    def __getattr__(self, name):
        # Only reached for names the wrapper does not define itself.
        if name in _MODULE_API:
            module = self.__dict__.get("module")
            if module is None or not hasattr(module, name):
                raise AttributeError(f"{type(module).__name__} has no {name}()")
            return getattr(module, name)
        raise AttributeError(f"{type(self).__name__!r} object has no attribute {name!r}")

    def train(self):
        switch = getattr(self.module, "train", None)
        return self if switch is None else switch()

    def eval(self):
        switch = getattr(self.module, "eval", None)
        return self if switch is None else switch()

    # ------------------------------------------------------- gradient control
    def zero_grad(self):
        self._reducer.reset()  # raises while asynchronous reductions are outstanding
        clear = getattr(self.module, "zero_grad", None)
        if clear is not None:
            return clear()
        for parameter in self.parameters():
            parameter.zero_grad()

    def all_reduce_gradients(self):
        self._reducer.synchronize()

    def wait_for_gradient_sync(self):
        self._reducer.group.ensure_open()
        self._reducer.wait()

    def _validate_master_gradient_sync(self):
        if self._sync_grads:
            raise ValueError("MixedPrecisionOptimizer requires DDP(sync_grads=False)")


DDP = DistributedDataParallel
__all__ = ["DistributedDataParallel", "DDP"]
