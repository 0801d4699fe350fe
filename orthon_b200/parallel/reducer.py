"""Gradient reducer: participation consensus, bucketing and averaging.

Generic path (any transport).  `synchronize()`:
  1. waits for outstanding asynchronous buckets;
  2. builds three rows per parameter -- used this step, packable into a flat float buffer,
     gradient profile valid -- and sums them over ranks with ONE control all-reduce;
  3. raises on every rank if any rank reported an invalid profile (no data collective ran);
  4. zero-fills gradients of parameters that some other rank used (globally unused ones stay
     without a gradient);
  5. per bucket: packs the gradients into one flat buffer, all-reduces it (asynchronously when
     overlap is on), scales by 1/world_size and copies back; non-packable entries are reduced
     one tensor at a time.
Buckets are filled greedily in sorted-name order up to `bucket_size_mb`.

Peer-memory path (CUDA + "p2p" transport): see `PeerReducer` in peer_reducer.py, where the
buckets ARE the gradient storage and one fused kernel per bucket does the reduction, the
unscale / inf check, the averaging and the optimizer update.
(reference project: python/orthon/distributed/_reducer.py:10-171)"""
import numpy as np

from .. import _C

_ELEMENT_BYTES = {"float32": 4, "float64": 8, "float16": 2, "bfloat16": 2}
_REJECTED = ("DDP gradient synchronization rejected an invalid gradient profile "
             "on one or more ranks (dtype, shape, device, or backend support)")


def _no_grad():
    import orthon_b200 as ob
    return ob.no_grad()


def _stamp(p):
    g = p.grad
    return None if g is None else (g._impl_id, g._storage_version)


def make_buckets(entries, bucket_size_mb):
    """Greedy fill in the given order; a bucket closes when the next tensor would overflow it."""
    limit = int(float(bucket_size_mb) * 1024 * 1024)
    if limit < 1:
        raise ValueError("bucket_size_mb must be positive when provided")
    buckets, cur, size = [], [], 0
    for entry in entries:
        p = entry[1]
        nbytes = int(p.numel) * _ELEMENT_BYTES.get(p.dtype, 1)
        if cur and size + nbytes > limit:
            buckets.append(cur)
            cur, size = [], 0
        cur.append(entry)
        size += nbytes
    if cur:
        buckets.append(cur)
    return buckets


class Reducer:
    def __init__(self, parameters, group, bucket_size_mb=None, overlap=False):
        self.parameters = tuple(parameters)  # (name, tensor)
        self.group = group
        self.overlap = bool(overlap)
        self.pending = set()
        self.synced = {id(p): None for _, p in self.parameters}
        self.outstanding = []
        self.launch_count = 0
        self.buckets = None if bucket_size_mb is None else make_buckets(self.parameters, bucket_size_mb)

    def diagnostics(self):
        return {"buckets": len(self.buckets or ()), "outstanding": len(self.outstanding), "async_launches": self.launch_count}

    def mark(self, owner_id):
        self.pending.add(owner_id)

    def reset(self):
        if self.outstanding:
            raise RuntimeError("DDP has pending asynchronous gradient synchronization; "
                               "call wait_for_gradient_sync() before zero_grad()")
        self.pending.clear()
        self.synced = {id(p): None for _, p in self.parameters}
        self.launch_count = 0

    # ---------------------------------------------------------------- profile
    def _valid(self, p, g):
        if g is None:
            return True
        if g.dtype not in _ELEMENT_BYTES:
            return False
        # Averaging scales the gradient in place in its own dtype: the CPU backend does that for
        # float32 / float64 only, the CUDA backend for float32 / float16 / bfloat16.
        if g.dtype not in (("float32", "float16", "bfloat16") if g.device.is_cuda() else ("float32", "float64")):
            return False
        try:
            self.group.validate_gradient_dtype(g.dtype)
        except (RuntimeError, ValueError, NotImplementedError):
            return False
        if tuple(g.shape) != tuple(p.shape) or g.device != p.device or g.dtype != p.dtype:
            return False
        return not (g.dtype == "float64" and g.device.is_cuda())

    def _control_rows(self):
        used, packable, valid = [], [], []
        for _, p in self.parameters:
            g = p.grad
            valid.append(float(self._valid(p, g)))
            used.append(float(id(p) in self.pending or (g is not None and _stamp(p) != self.synced[id(p)])))
            packable.append(float(g is None or (g.dtype == p.dtype and g.is_contiguous)))
        if self.buckets is not None:
            index = {id(p): i for i, (_, p) in enumerate(self.parameters)}
            for bucket in self.buckets:
                first = bucket[0][1]
                if any(p.device != first.device or p.dtype != first.dtype for _, p in bucket):
                    for _, p in bucket:
                        packable[index[id(p)]] = 0.0
        return used, packable, valid

    # ------------------------------------------------------------ synchronize
    def synchronize(self):
        self.group.ensure_open()
        self.wait()
        if not self.parameters:
            return
        ws = self.group.world_size
        rows = self._control_rows()
        with _no_grad():
            control = _C.from_numpy(np.asarray(rows, dtype=np.float32))
            device = self.parameters[0][1].device
            if device.is_cuda():
                control = control.to(device)
            self.group.all_reduce(control)  # the single control collective
            agreed = np.asarray(control.tolist(), dtype=np.float64).reshape(3, -1)
            if np.any(agreed[2] != ws):
                raise RuntimeError(_REJECTED)
            active = {id(p) for i, (_, p) in enumerate(self.parameters) if agreed[0, i] > 0}
            packable = {id(p) for i, (_, p) in enumerate(self.parameters) if agreed[1, i] == ws}
            for _, p in self.parameters:
                if id(p) in active and p.grad is None:
                    p.set_grad(_C._zeros_on(list(p.shape), p.dtype, str(p.device)))
            groups = self.buckets if self.buckets is not None else [[e] for e in self.parameters]
            for bucket in groups:
                live = [(p, p.grad) for _, p in bucket if id(p) in active]
                if not live:
                    continue
                pack = (self.buckets is not None and all(id(p) in packable for p, _ in live)
                        and all(g.device == live[0][1].device for _, g in live))
                if pack:
                    self._reduce_packed(live)
                else:
                    for p, g in live:
                        payload = g if g.is_contiguous else _C.contiguous(g)
                        self.group.all_reduce(payload)
                        payload.mul_(1.0 / ws)
                        if payload is not g:
                            p.set_grad(payload)
            self.wait()
        self.pending.clear()
        self.synced = {id(p): _stamp(p) for _, p in self.parameters}

    def _reduce_packed(self, live):
        total = sum(int(g.numel) for _, g in live)
        first = live[0][1]
        flat = _C._empty_on([total], first.dtype, str(first.device))
        offset = 0
        for _, g in live:
            flat._copy_flat_range_from(offset, g.reshape([-1]), 0, int(g.numel))
            offset += int(g.numel)
        if self.overlap:
            work = self.group.all_reduce(flat, async_op=True)
            self.outstanding.append((work, flat, live))
            self.launch_count += 1
        else:
            self.group.all_reduce(flat)
            self._scatter(flat, live)

    def _scatter(self, flat, live):
        flat.mul_(1.0 / self.group.world_size)
        offset = 0
        for p, g in live:
            cur = p.grad
            if cur is None or cur._impl_id != g._impl_id:
                raise RuntimeError("DDP gradient changed before asynchronous bucket synchronization completed")
            g.reshape([-1])._copy_flat_range_from(0, flat, offset, int(g.numel))
            offset += int(g.numel)

    def wait(self):
        with _no_grad():
            for work, flat, live in self.outstanding:
                work.wait()
                self._scatter(flat, live)
        self.outstanding.clear()


def reduce_master_gradients(parameters, group):
    """Averages freshly prepared FP32 master gradients (AMP path)."""
    reducer = Reducer([(str(i), p) for i, p in enumerate(parameters)], group)
    reducer.pending.update(id(p) for _, p in reducer.parameters if p.grad is not None)
    reducer.synchronize()


_Reducer = Reducer
_reduce_master_gradients = reduce_master_gradients
