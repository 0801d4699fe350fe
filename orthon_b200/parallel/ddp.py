"""DistributedDataParallel: replicated parameters, averaged gradients.

Construction captures the active group, takes the unique trainable parameters in sorted-name
order, broadcasts them from `src`, and registers a post-accumulate hook per parameter (marks
it used) plus one keyed backward finalizer (runs the reducer once per backward, after every
leaf gradient is committed).  Buffers are not broadcast.
(reference project: python/orthon/distributed/ddp.py:7-119)"""
import weakref

from ..distributed import _state
from .peer_reducer import PeerReducer
from .reducer import Reducer


class DistributedDataParallel:
    def __init__(self, module, src=0, sync_grads=True, bucket_size_mb=None, overlap_grad_sync=False):
        self.module = module
        self._sync_grads = bool(sync_grads)
        if overlap_grad_sync and not sync_grads:
            raise ValueError("overlap_grad_sync=True requires sync_grads=True")
        if overlap_grad_sync and bucket_size_mb is None:
            raise ValueError("overlap_grad_sync=True requires bucket_size_mb to be provided")
        if bucket_size_mb is not None and int(float(bucket_size_mb) * 1024 * 1024) < 1:
            raise ValueError("bucket_size_mb must be positive when provided")
        group = _state.get_active()
        if hasattr(module, "named_parameters"):
            named = list(module.named_parameters())
        else:
            named = [(str(i), p) for i, p in enumerate(module.parameters())]
        owners, seen = [], set()
        for name, p in sorted(named, key=lambda item: item[0]):
            if id(p) not in seen and p.requires_grad:
                seen.add(id(p))
                owners.append((name, p))
        for _, p in owners:
            group.broadcast(p, src=src)
        if PeerReducer.eligible(owners, group):
            # Buckets become the gradient storage; reduction starts from the leaf hooks.
            self._reducer = PeerReducer(owners, group, bucket_size_mb, overlap=True)
        else:
            self._reducer = Reducer(owners, group, bucket_size_mb, bool(overlap_grad_sync))
        ref = weakref.ref(self._reducer)

        def finalize():
            r = ref()
            if r is not None:
                r.synchronize()

        self._finalizer, self._finalizer_key = finalize, id(self._reducer)
        for _, p in owners:

            def used(owner=id(p), ref=ref):
                r = ref()
                if r is not None:
                    r.mark(owner)

            p._register_post_accumulate_grad_hook(used)
            if self._sync_grads:
                p._register_backward_finalizer(self._finalizer_key, finalize)

    def _attach_outputs(self, output):
        if not self._sync_grads:
            return
        if isinstance(output, (tuple, list)):
            for v in output:
                self._attach_outputs(v)
        elif isinstance(output, dict):
            for v in output.values():
                self._attach_outputs(v)
        elif hasattr(output, "_register_backward_finalizer") and output.requires_grad:
            output._register_backward_finalizer(self._finalizer_key, self._finalizer)

    def __call__(self, *args, **kwargs):
        self._reducer.group.ensure_open()
        out = self.module(*args, **kwargs)
        self._attach_outputs(out)
        return out

    def forward(self, *args, **kwargs):
        return self(*args, **kwargs)

    def parameters(self):
        return self.module.parameters()

    def _delegate(self, name, *args, **kwargs):
        if not hasattr(self.module, name):
            raise AttributeError(f"{type(self.module).__name__} has no {name}()")
        return getattr(self.module, name)(*args, **kwargs)

    def named_parameters(self, *a, **k):
        return self._delegate("named_parameters", *a, **k)

    def state_dict(self, *a, **k):
        return self._delegate("state_dict", *a, **k)

    def load_state_dict(self, *a, **k):
        return self._delegate("load_state_dict", *a, **k)

    def train(self):
        return self.module.train() if hasattr(self.module, "train") else self

    def eval(self):
        return self.module.eval() if hasattr(self.module, "eval") else self

    def zero_grad(self):
        self._reducer.reset()
        if hasattr(self.module, "zero_grad"):
            return self.module.zero_grad()
        for p in self.parameters():
            p.zero_grad()

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
