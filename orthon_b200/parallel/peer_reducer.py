"""Peer-memory reducer: the gradient buckets ARE the gradient storage.

Every parameter's `.grad` is a view into a symmetric bucket that all ranks map.  The autograd
engine writes a parameter's gradient into its slot as soon as its last consumer has run and
fires the parameter's hook.  One fused kernel per bucket then averages the bucket in place
("average") or also applies the FP32-master Adam/SGD update and refreshes the low-precision
parameters ("adam" / "sgd"): no pack/unpack copies, no NCCL call, no separate scale / unscale /
inf-check / optimizer kernels.

Two schedules:

* at synchronisation (default): `synchronize()` launches every bucket, in bucket order, on every
  rank.  The kernel's entry barrier carries the participation consensus of the reference's control
  all-reduce (python/orthon/distributed/_reducer.py:61-113): one usage bit per parameter and an
  "invalid local gradient profile" bit.  A parameter without a gradient on this rank contributes
  zeros and receives the average if any rank used it, and keeps `grad is None` if no rank did; an
  invalid profile on any rank leaves every bucket untouched on every rank and raises the
  reference's rejection.  Gradients accumulate locally across backward calls until then.
* from the leaf hooks (`overlap=True`): a bucket is queued on the communication stream the moment
  its last gradient has been written, so reduction (and the fused update) overlaps the rest of
  backward.  This needs every rank to produce the same gradients in the same order; a rank that
  skips a bucket makes its peers' bounded waits run out, which surfaces as the group's sticky
  failure.  Under `single_backward` (set by the AMP wrapper, where nothing synchronises at the
  end of backward) a second backward before `reset()` raises instead of mixing averaged and
  local gradients.

Buckets of at least NVLS_MIN_BYTES go through the in-switch (multimem) variant of the kernel
when the group has at least ORTHON_NVLS_MIN_WORLD ranks (4 unless set) and the backend could bind
the buckets to an NVLink multicast object; everything else uses the one-shot / two-shot peer-load
variants.
"""
import os

from .. import _C
from ..utils.tracing import trace_range
from .reducer import _ELEMENT_BYTES, make_buckets

MAX_BUCKET_ENTRIES = 32 * _C._PEER_USAGE_WORDS if hasattr(_C, "_PEER_USAGE_WORDS") else 2048


def _no_grad():
    import orthon_b200 as ob
    return ob.no_grad()


def _align(n, a):
    return (n + a - 1) // a * a


def _split_long(groups, limit):
    for entries in groups:
        for i in range(0, len(entries), limit):
            yield entries[i:i + limit]


class _Bucket:
    __slots__ = ("entries", "offsets", "n", "dtype", "grads", "staging", "flags", "grad_flat", "seen", "launched",
                 "param_flat", "master_flat", "m_flat", "v_flat", "seg", "seg_host", "mc", "flag_words")

    def full_usage(self):
        k = len(self.entries)
        return [0xFFFFFFFF if k >= 32 * (w + 1) else (1 << (k - 32 * w)) - 1 for w in range((k + 31) // 32)]


class PeerReducer:
    # One-shot (every rank reads every copy) pays while (world - 1) x bucket stays small.  Measured
    # crossover against the two-shot kernel: 512 KB at 2 ranks, about 32 KB at 4, 16 KB at 8.
    ONESHOT_BYTES_BY_WORLD = {1: 512 << 10, 2: 512 << 10, 3: 32 << 10, 4: 32 << 10}
    ONESHOT_BYTES_LARGE_WORLD = 16 << 10
    # In-switch reduction (multimem) moves S bytes per GPU and direction instead of 2 S (w-1)/w.
    # Measured on NVLink 5 / NVSwitch, 1 GB buckets, bus GB/s: 2 GPUs 392 against 683 for peer loads;
    # 4 GPUs 686 against 651 (and the 1.3 B step 83.1 against 84.4 ms); 8 GPUs 830 against 625 (step
    # 82.7 against 85.0 ms), ahead from 8 KB buckets on at both sizes.  So groups of 4 ranks and more
    # use it wherever the box could bind the buckets to a multicast object; ORTHON_NVLS_MIN_WORLD
    # moves the threshold (0 turns it off), ORTHON_NVLS=0 never binds.
    NVLS_MIN_BYTES = int(os.environ.get("ORTHON_NVLS_MIN_BYTES", 8 << 10))  # smaller buckets use peer loads
    NVLS_MIN_WORLD = int(os.environ.get("ORTHON_NVLS_MIN_WORLD", 4))
    # Block size of launches that run beside a backward pass: small enough to share an SM with a
    # persistent GEMM CTA (see csrc/cuda/peer_reducer.cu).
    OVERLAP_THREADS = int(os.environ.get("ORTHON_PEER_OVERLAP_THREADS", 512))
    OVERLAP_CTAS = int(os.environ.get("ORTHON_PEER_OVERLAP_CTAS", 0))  # 0 = one per SM
    SIDE_STREAM_UPDATE = os.environ.get("ORTHON_UPDATE_SIDE_STREAM", "1") != "0"  # single device: update beside backward

    @staticmethod
    def eligible(parameters, group):
        backend = getattr(group, "backend", None)
        if not getattr(backend, "supports_peer_reduce", False) or not parameters:
            return False
        first = parameters[0][1]
        return all(p.device.is_cuda() and p.device == first.device and p.dtype == first.dtype and p.is_contiguous
                   and p.dtype in ("float32", "float16", "bfloat16") for _, p in parameters)

    @classmethod
    def choose_variant(cls, world, nbytes, has_multicast):
        """Which kernel reduces a bucket of `nbytes` across `world` ranks: "in_switch" (multimem
        through the NVSwitch), "one_shot" (every rank reads every copy) or "two_shot"
        (reduce-scatter by peer loads, all-gather by peer stores)."""
        if has_multicast and nbytes >= cls.NVLS_MIN_BYTES and 0 < cls.NVLS_MIN_WORLD <= world:
            return "in_switch"
        if nbytes <= cls.ONESHOT_BYTES_BY_WORLD.get(world, cls.ONESHOT_BYTES_LARGE_WORLD):
            return "one_shot"
        return "two_shot"

    def __init__(self, parameters, group, bucket_size_mb=None, overlap=False):
        self.parameters = tuple(parameters)
        self.group = group
        self.backend = group.backend
        self.overlap = bool(overlap)
        self.single_backward = False
        self.world, self.rank, self.device = group.world_size, group.rank, self.backend.device
        self.dev = f"cuda:{self.device}"
        self.mode = "average"          # or "adam" / "sgd" once an optimizer is attached in update mode
        self.hyper = None              # callable -> dict, consulted at launch time
        self.on_first_launch = None    # optimizer step counter hook
        self.launch_count = 0
        self._step_open = False
        self._cycle_closed = False
        self._bucket_of = {}
        dtype = self.parameters[0][1].dtype
        esz = _ELEMENT_BYTES[dtype]
        groups = _split_long(make_buckets(self.parameters, 25 if bucket_size_mb is None else bucket_size_mb), MAX_BUCKET_ENTRIES)
        self.buckets = []
        grad_bytes = stage_bytes = 0
        for entries in groups:
            b = _Bucket()
            b.entries, b.offsets, off = entries, [], 0
            for _, p in entries:
                b.offsets.append(off)
                off = _align(off + int(p.numel), 8)
            b.n, b.dtype, b.seen, b.launched = off, dtype, set(), False
            b.param_flat = b.master_flat = b.m_flat = b.v_flat = b.seg = None
            self.buckets.append(b)
            grad_bytes += _align(b.n * esz, 256)
            stage_bytes += _align(b.n * 4, 256)
        flag_bytes = _align(_C._PEER_FLAG_BYTES, 256)
        use_nvls = 0 < self.NVLS_MIN_WORLD <= self.world
        region = self.backend.allocate_symmetric(grad_bytes + stage_bytes + flag_bytes * len(self.buckets), multicast=use_nvls)
        g_off, s_off, f_off = 0, grad_bytes, grad_bytes + stage_bytes
        for i, b in enumerate(self.buckets):
            b.grads = [ptr + g_off for ptr in region.ptrs]
            b.staging = [ptr + s_off for ptr in region.ptrs]
            b.flags = [ptr + f_off for ptr in region.ptrs]
            b.mc = (region.mc + g_off) if getattr(region, "mc", None) else 0
            b.grad_flat = _C._tensor_from_ptr(b.grads[self.rank], [b.n], dtype, self.device)
            b.flag_words = _C._tensor_from_ptr(b.flags[self.rank], [_C._PEER_FLAG_BYTES // 4], "int32", self.device)
            g_off += _align(b.n * esz, 256)
            s_off += _align(b.n * 4, 256)
            f_off += flag_bytes
            for (name, p), off in zip(b.entries, b.offsets):
                p._set_grad_slot(_C._view_flat(b.grad_flat, off, list(p.shape)))
                self._bucket_of[id(p)] = i
        self._region = region

    # ------------------------------------------------------------- diagnostics
    def diagnostics(self):
        return {"buckets": len(self.buckets), "outstanding": sum(1 for b in self.buckets if b.launched),
                "async_launches": self.launch_count, "mode": self.mode}

    # ------------------------------------------------------------------- hooks
    def mark(self, owner_id):
        i = self._bucket_of.get(owner_id)
        if i is None:
            return
        b = self.buckets[i]
        if self.overlap and self.single_backward and (b.launched or self._cycle_closed):
            raise RuntimeError(
                "this optimizer reduces gradients inside backward: a second backward() before zero_grad() would add local "
                "gradients to averaged ones (or apply the update twice); call zero_grad() first, or build the optimizer "
                "with fused='reduce' to accumulate gradients over several backward passes")
        b.seen.add(owner_id)
        if self.overlap and not b.launched and len(b.seen) >= len(b.entries):
            self._launch(i, b.full_usage(), beside_backward=True)

    def _launch(self, i, usage, invalid=False, beside_backward=False):
        b = self.buckets[i]
        if not self._step_open:
            self._step_open = True
            if self.on_first_launch is not None:
                self.on_first_launch()
        hyper = self.hyper() if (self.hyper is not None and self.mode != "average") else {}
        scale = hyper.pop("grad_scale", 1.0) / self.world
        if b.seg is not None and self.mode != "average":
            hyper["seg_end"], hyper["seg_wd"] = b.seg
        nbytes = b.n * _ELEMENT_BYTES[b.dtype]
        variant = self.choose_variant(self.world, nbytes, bool(b.mc))
        in_switch, oneshot = variant == "in_switch", variant == "one_shot"
        status, found_inf = self.backend.status_tensors()
        _C._stream_fence(self.device, 0, 1)  # communication stream waits for the gradients
        fused = self.mode != "average"
        with trace_range(f"peer_reduce bucket {i}", self.device, 1):
            _C._peer_reduce(self.rank, self.world, self.device, b.grads, b.staging, b.flags, b.n, b.dtype,
                            self.backend.next_epoch(), scale, self.mode, oneshot,
                            master=b.master_flat if fused else None, m=b.m_flat if self.mode == "adam" else None,
                            v=b.v_flat if self.mode == "adam" else None,
                            model=b.param_flat if (fused and b.param_flat is not None and b.master_flat is not b.param_flat) else None,
                            hyper=hyper, status=status, found_inf=found_inf, stream_kind=1,
                            mc_grads=b.mc if in_switch else 0,
                            ctas=self.OVERLAP_CTAS if beside_backward else 0,
                            threads=self.OVERLAP_THREADS if beside_backward else 512,
                            wait_ms=self.backend.wait_ms, invalid=bool(invalid), usage=usage)
        b.launched = True
        self.launch_count += 1

    # ------------------------------------------------------------ step control
    def _local_profile(self, b):
        """Usage bits of this rank for bucket `b`, the parameters without a local gradient, and
        whether a hand-assigned gradient disagrees with its parameter (shape, dtype or device)."""
        usage, idle, invalid = [0] * ((len(b.entries) + 31) // 32), [], False
        for k, ((name, p), off) in enumerate(zip(b.entries, b.offsets)):
            g = p.grad
            slot = _C._view_flat(b.grad_flat, off, list(p.shape))
            if g is None:
                slot.fill_(0.0)
                idle.append((p, slot))
                continue
            usage[k // 32] |= 1 << (k % 32)
            if g._data_ptr != slot._data_ptr:  # a gradient assigned by hand
                if tuple(g.shape) != tuple(p.shape) or g.dtype != p.dtype or g.device != p.device:
                    invalid = True
                    continue
                slot._copy_data_(g)
                p.set_grad(slot)
        if self.mode != "average" and idle:
            invalid = True  # the fused update needs a gradient for every parameter
        return usage, idle, invalid

    def synchronize(self):
        """Launches whatever has not been launched yet and orders the compute stream after the
        communication stream.  Waits for the device only when this rank has parameters without a
        gradient (it then has to learn whether any other rank used them)."""
        self.group.ensure_open()
        self.backend.poll_status()
        idle_by_bucket, rejected = [], None
        with _no_grad():
            for i, b in enumerate(self.buckets):
                if b.launched:
                    continue
                usage, idle, invalid = self._local_profile(b)
                if invalid and rejected is None:
                    rejected = next((name for (name, p) in b.entries if p.grad is None), b.entries[0][0])
                self._launch(i, usage, invalid=invalid)
                if idle:
                    idle_by_bucket.append((b, idle))
            _C._stream_fence(self.device, 1, 0)
            if idle_by_bucket and rejected is None:
                base = _C._PEER_USAGE_WORD_OFFSET
                for b, idle in idle_by_bucket:
                    words = b.flag_words.tolist()  # synchronises: the union of every rank's usage bits
                    index = {id(p): k for k, (_, p) in enumerate(b.entries)}
                    for p, slot in idle:
                        k = index[id(p)]
                        if (words[base + k // 32] & 0xFFFFFFFF) >> (k % 32) & 1:
                            p.set_grad(slot)
                self.backend.check_status()
        for b in self.buckets:
            b.seen, b.launched = set(), False
        self._step_open = False
        self._cycle_closed = self.single_backward
        if rejected is not None:
            _C.cuda_synchronize()
            self.backend._status.fill_(0.0)
            if self.mode != "average":
                raise RuntimeError(f"fused optimizer update needs a gradient for every parameter; '{rejected}' has none "
                                   "(no rank applied this step)")
            raise RuntimeError(self.backend.INVALID_PROFILE)

    def wait(self):
        """Orders the compute stream after the communication stream and checks the kernels' error word."""
        _C._stream_fence(self.device, 1, 0)
        self.backend.check_status()

    def reset(self):
        for b in self.buckets:
            b.seen, b.launched = set(), False
        self._step_open = False
        self._cycle_closed = False
        self.launch_count = 0

    def found_inf(self, clear=True):
        """True when any reduced gradient since the last clear was non-finite: one device read,
        which also checks the kernels' error word."""
        code, hit = self.backend.read_words()
        self.backend._judge(code)
        if hit and clear:
            self.backend.status_tensors()[1].fill_(0.0)
        return hit

    # --------------------------------------------------------- optimizer state
    def flatten_state(self, want_masters):
        """Moves every parameter into one flat buffer per bucket (identity preserved) and, when
        the parameters are low precision, creates flat float32 masters.  Returns, per parameter
        in `self.parameters` order, (master view or None)."""
        masters = {}
        with _no_grad():
            for b in self.buckets:
                b.param_flat = _C._zeros_on([b.n], b.dtype, self.dev)
                if want_masters:
                    b.master_flat = _C._zeros_on([b.n], "float32", self.dev)
                else:
                    b.master_flat = b.param_flat
                for (name, p), off in zip(b.entries, b.offsets):
                    view = _C._view_flat(b.param_flat, off, list(p.shape))
                    view._copy_data_(p)
                    p._rebind_model_value_(view)
                    p.requires_grad_(True)
                    if want_masters:
                        mv = _C._view_flat(b.master_flat, off, list(p.shape))
                        mv._copy_data_(p)  # casts to float32
                        mv.requires_grad_(True)
                        masters[id(p)] = mv
        return [masters.get(id(p)) for _, p in self.parameters]

    def flat_moments(self):
        """Flat zeroed Adam moments per bucket; returns per-parameter (m view, v view)."""
        out = {}
        for b in self.buckets:
            b.m_flat = _C._zeros_on([b.n], "float32", self.dev)
            b.v_flat = _C._zeros_on([b.n], "float32", self.dev)
            for (name, p), off in zip(b.entries, b.offsets):
                out[id(p)] = (_C._view_flat(b.m_flat, off, list(p.shape)), _C._view_flat(b.v_flat, off, list(p.shape)))
        return [out[id(p)] for _, p in self.parameters]

    def set_decay_segments(self, decay_of):
        """`decay_of(param) -> weight decay` ; builds the per-bucket segment tables the kernel searches."""
        import numpy as np
        for b in self.buckets:
            ends, wds = [], []
            for i, ((name, p), off) in enumerate(zip(b.entries, b.offsets)):
                end = b.offsets[i + 1] if i + 1 < len(b.offsets) else b.n
                ends.append(end)
                wds.append(float(decay_of(p)))
            if any(w != 0.0 for w in wds):
                b.seg = (_C.from_numpy(np.asarray(ends, dtype=np.int64)).to(self.dev),
                         _C.from_numpy(np.asarray(wds, dtype=np.float32)).to(self.dev))
            else:
                b.seg = None

    def local_update(self, kind, hyper):
        """Applies the optimizer bucket by bucket from the (already averaged) gradients: one
        fused kernel per bucket.  Used when the update may not run inside backward (GradScaler)."""
        with _no_grad():
            for b in self.buckets:
                model = b.param_flat if b.master_flat is not b.param_flat else None
                if kind == "adam":
                    _C._adam_step_(b.master_flat, b.m_flat, b.v_flat, b.grad_flat, model, hyper["lr"], hyper["beta1"],
                                   hyper["beta2"], hyper["eps"], hyper.get("weight_decay", 0.0), hyper["bias_c1"],
                                   hyper["bias_c2"], hyper.get("grad_scale", 1.0))
                else:
                    _C._sgd_step_(b.master_flat, b.grad_flat, model, hyper["lr"], hyper.get("weight_decay", 0.0),
                                  hyper.get("grad_scale", 1.0))


class LocalFlatReducer(PeerReducer):
    """Single-process sibling of PeerReducer: the same flat gradient / parameter / master /
    moment buckets and the same hook-driven schedule, without peers.  In update mode each
    bucket's fused optimizer kernel is queued on the second stream as soon as the bucket's last
    gradient has been written, in blocks small enough to share the SMs with the GEMMs of the
    backward pass, so the (memory-bound) update of late layers hides behind the (tensor-bound)
    backward of early layers."""

    def __init__(self, parameters, bucket_size_mb=None):
        self.parameters = tuple(parameters)
        self.group, self.backend = None, None
        self.overlap, self.single_backward = True, True
        first = self.parameters[0][1]
        self.world, self.rank, self.device = 1, 0, first.device.index
        self.dev = f"cuda:{self.device}"
        self.mode, self.hyper, self.on_first_launch = "average", None, None
        self.launch_count, self._step_open, self._cycle_closed, self._bucket_of = 0, False, False, {}
        self.buckets = []
        self._flag = _C._zeros_on([1], "int32", self.dev)
        for entries in make_buckets(self.parameters, 25 if bucket_size_mb is None else bucket_size_mb):
            b = _Bucket()
            b.entries, b.offsets, off = entries, [], 0
            for _, p in entries:
                b.offsets.append(off)
                off = _align(off + int(p.numel), 8)
            b.n, b.dtype, b.seen, b.launched = off, first.dtype, set(), False
            b.param_flat = b.master_flat = b.m_flat = b.v_flat = b.seg = None
            b.grads = b.staging = b.flags = None
            b.grad_flat = _C._zeros_on([b.n], first.dtype, self.dev)
            for (name, p), o in zip(b.entries, b.offsets):
                p._set_grad_slot(_C._view_flat(b.grad_flat, o, list(p.shape)))
                self._bucket_of[id(p)] = len(self.buckets)
            self.buckets.append(b)

    @staticmethod
    def eligible(parameters):
        if not parameters:
            return False
        first = parameters[0][1]
        return all(p.device.is_cuda() and p.device == first.device and p.dtype == first.dtype and p.is_contiguous
                   and p.dtype in ("float32", "float16", "bfloat16") for _, p in parameters)

    def mark(self, owner_id):
        if self.mode == "average":
            return  # nothing to do before step(): gradients simply accumulate in their slots
        super().mark(owner_id)

    def _launch(self, i, usage=None, invalid=False, beside_backward=False):
        b = self.buckets[i]
        if not self._step_open:
            self._step_open = True
            if self.on_first_launch is not None:
                self.on_first_launch()
        if self.mode != "average":
            if b.seg is not None:
                raise RuntimeError("per-parameter weight decay needs fused='reduce' on a single device")
            beside_backward = beside_backward and self.SIDE_STREAM_UPDATE
            if beside_backward:
                _C._stream_fence(self.device, 0, 1)  # the second stream waits for the gradients
            self._update_bucket(b, self.mode, self.hyper(), side_stream=beside_backward)
        b.launched = True
        self.launch_count += 1

    def _update_bucket(self, b, kind, h, side_stream=False):
        model = b.param_flat if b.master_flat is not b.param_flat else None
        stream, threads = (1, 256) if side_stream else (0, 0)
        with _no_grad(), trace_range(f"optimizer bucket {kind}", self.device, stream):
            if kind == "adam":
                _C._adam_step_(b.master_flat, b.m_flat, b.v_flat, b.grad_flat, model, h["lr"], h["beta1"], h["beta2"], h["eps"],
                               h.get("weight_decay", 0.0), h["bias_c1"], h["bias_c2"], h.get("grad_scale", 1.0), stream, threads)
            else:
                _C._sgd_step_(b.master_flat, b.grad_flat, model, h["lr"], h.get("weight_decay", 0.0), h.get("grad_scale", 1.0),
                              stream, threads)

    def synchronize(self):
        with _no_grad():
            for i, b in enumerate(self.buckets):
                if b.launched:
                    continue
                for (name, p), off in zip(b.entries, b.offsets):
                    g = p.grad
                    slot = _C._view_flat(b.grad_flat, off, list(p.shape))
                    if g is None:
                        if self.mode != "average":
                            raise RuntimeError(f"fused optimizer update needs a gradient for every parameter; '{name}' has none")
                        slot.fill_(0.0)
                        p.set_grad(slot)
                    elif g._data_ptr != slot._data_ptr:
                        slot._copy_data_(g)
                        p.set_grad(slot)
                self._launch(i)
        if self.mode != "average":
            _C._stream_fence(self.device, 1, 0)
        for b in self.buckets:
            b.seen, b.launched = set(), False
        self._step_open = False
        self._cycle_closed = self.mode != "average"

    def wait(self):
        return None

    def found_inf(self, clear=True):
        for b in self.buckets:
            _C._isfinite_into(b.grad_flat, self._flag)
        hit = bool(self._flag.tolist()[0])
        if hit and clear:
            self._flag.fill_(0.0)
        return hit

    def local_update(self, kind, hyper):
        for b in self.buckets:
            if b.seg is not None:
                # Weight decay differs per parameter: update parameter by parameter inside the bucket.
                self._update_segments(b, kind, hyper)
            else:
                self._update_bucket(b, kind, hyper)

    def _update_segments(self, b, kind, h):
        ends, wds = b.seg_host
        start = 0
        with _no_grad():
            for end, wd in zip(ends, wds):
                n = end - start
                sl = lambda t: None if t is None else _C._view_flat(t, start, [n])  # noqa: E731
                model = sl(b.param_flat) if b.master_flat is not b.param_flat else None
                if kind == "adam":
                    _C._adam_step_(sl(b.master_flat), sl(b.m_flat), sl(b.v_flat), sl(b.grad_flat), model, h["lr"], h["beta1"],
                                   h["beta2"], h["eps"], wd, h["bias_c1"], h["bias_c2"], h.get("grad_scale", 1.0))
                else:
                    _C._sgd_step_(sl(b.master_flat), sl(b.grad_flat), model, h["lr"], wd, h.get("grad_scale", 1.0))
                start = end

    def set_decay_segments(self, decay_of):
        for b in self.buckets:
            ends, wds = [], []
            for i, ((name, p), off) in enumerate(zip(b.entries, b.offsets)):
                ends.append(b.offsets[i + 1] if i + 1 < len(b.offsets) else b.n)
                wds.append(float(decay_of(p)))
            b.seg = (ends, wds) if any(w != 0.0 for w in wds) else None
            b.seg_host = (ends, wds)
