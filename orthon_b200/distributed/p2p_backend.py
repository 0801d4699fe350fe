"""Peer-memory transport for one node of NVLink/NVSwitch-connected GPUs.

Collectives on tensors run as the peer-memory reduction kernel over a symmetric staging region
that every rank maps from every other rank (CUDA IPC): no NCCL call is made for all_reduce,
broadcast or barrier; tensors larger than the staging region go through it in chunks.
The DDP gradient path does not go through these generic collectives at all: PeerReducer keeps
the gradients inside symmetric buckets and launches the fused kernel on them directly.  Those
buckets are cuMemCreate allocations shared through file descriptors and, where the devices
support NVLink multicast, bound to one multicast object (`region.mc`) so the kernel can reduce
and broadcast inside the NVSwitch (`multimem`); ORTHON_NVLS=0 keeps to plain peer mappings.
"""
import json
import os
import time
import socket

from .. import _C
from .group import Backend, Work, _TransportFailure
from .nccl_backend import RENDEZVOUS_TIMEOUT_SECONDS
from .store import ManagerStore, Store, store_from_env

STAGING_BYTES = 64 << 20
_ESIZE = {"float32": 4, "float16": 2, "bfloat16": 2}


def _no_grad():
    import orthon_b200 as ob
    return ob.no_grad()


class SymmetricRegion:
    """`ptrs[r]` is rank r's copy of the region as mapped into this process."""

    def __init__(self, nbytes, ptrs, rank, mc=None):
        self.nbytes, self.ptrs, self.rank = nbytes, ptrs, rank
        self.mc = mc  # multicast (NVLS) mapping of all copies, or None

    @property
    def local(self):
        return self.ptrs[self.rank]


class PeerBackend(Backend):
    supports_peer_reduce = True

    def __init__(self, rank=None, world_size=None, device=None, store=None):
        if rank is None or world_size is None:
            raise ValueError("p2p backend requires rank and world_size")
        if not 1 <= world_size <= _C._PEER_MAX_RANKS or not 0 <= rank < world_size:
            raise ValueError(f"p2p backend supports 1..{_C._PEER_MAX_RANKS} ranks on one node")
        self._rank, self._world = int(rank), int(world_size)
        self._device = int(rank if device is None else device)
        if self._device >= _C.cuda_device_count():
            raise ValueError(f"p2p backend: cuda:{self._device} is not visible")
        self._store = store_from_env(self._rank, self._world) if store is None else (
            store if isinstance(store, Store) else ManagerStore(store))
        self._generation = self._store.add(f"p2p/generation/{self._rank}", 1) - 1
        self._xseq = 0
        self._closed, self._failure = False, None
        self._dev = f"cuda:{self._device}"
        # Device words the kernels report into: [0] first error code of a bounded wait, [1] "a
        # reduced gradient was non-finite", [2] the same for generic collectives (kept apart so that
        # an overflow in an unrelated all_reduce never makes a GradScaler skip a step).
        self._words = _C._zeros_on([4], "int32", self._dev)
        self._status = _C._view_flat(self._words, 0, [1])
        self._found_inf = _C._view_flat(self._words, 1, [1])
        self._coll_inf = _C._view_flat(self._words, 2, [1])
        self._host_words = _C._pinned_empty([4], "int32")
        self._host_words._copy_data_(_C.zeros([4], "int32"))
        self._poll_event = None
        self.wait_ms = float(os.environ.get("ORTHON_PEER_WAIT_MS", 2000.0))  # budget of every device-side flag wait
        self._epoch = 0
        # One symmetric region: [staging grads | float32 staging | flags].
        self._stage = self.allocate_symmetric(STAGING_BYTES * 2 + _C._PEER_FLAG_BYTES)
        self._nccl = None
        self._vmm = None  # decided collectively on first use

    rank = property(lambda self: self._rank)
    world_size = property(lambda self: self._world)
    device = property(lambda self: self._device)

    # ---------------------------------------------------------------- plumbing
    def _open(self):
        if self._closed:
            raise RuntimeError("p2p backend has been shut down")
        if self._failure is not None:
            raise _TransportFailure("p2p backend failed: " + self._failure)

    def exchange_objects(self, value: bytes):
        prefix = f"p2p/x/{self._generation}/{self._xseq}"
        self._xseq += 1
        self._store.set(f"{prefix}/r{self._rank}", value)
        keys = [f"{prefix}/r{r}" for r in range(self._world)]
        self._store.wait_for(keys, RENDEZVOUS_TIMEOUT_SECONDS)
        out = [self._store.get(k) for k in keys]
        if self._store.add(f"{prefix}/leave", 1) == self._world:
            for k in keys + [f"{prefix}/leave"]:
                self._store.delete(k)
        return out

    def allocate_symmetric(self, nbytes, multicast=False):
        """Collective: every rank allocates `nbytes` (zeroed) and maps everybody else's copy.

        With `multicast=True` the copies are additionally bound to one NVLink multicast object
        when every rank's device and driver support it (`region.mc` is then the multicast
        pointer); otherwise `region.mc` is None and only the peer mappings exist."""
        if multicast and self._world > 1 and self._vmm_enabled():
            try:
                region = self._allocate_vmm(int(nbytes))
            except (OSError, RuntimeError, ValueError):
                region = None  # descriptor exchange or driver call failed here: use the IPC path
                self._vmm = False
            if not self._agree(region is not None):
                region = None
            if region is not None:
                return region
        nbytes = (int(nbytes) + 255) & ~255
        ptr, handle = _C._peer_alloc(nbytes, self._device)
        handles = self.exchange_objects(handle)
        ptrs = [ptr if r == self._rank else _C._peer_open(handles[r], self._device) for r in range(self._world)]
        self.exchange_objects(b"mapped")  # nobody touches a region before everyone has mapped it
        return SymmetricRegion(nbytes, ptrs, self._rank)

    # ------------------------------------------------- shareable allocations
    def _agree(self, ok):
        """True only if every rank reports success (keeps the ranks on the same code path)."""
        return all(v == b"ok" for v in self.exchange_objects(b"ok" if ok else b"no"))

    def _vmm_enabled(self):
        if self._vmm is None:
            want = os.environ.get("ORTHON_NVLS", "1") != "0"
            caps = _C._vmm_supported(self._device) if want else {"fd_handles": False, "multicast": False}
            self._vmm = self._agree(bool(caps["fd_handles"]) and bool(caps["multicast"]))
        return self._vmm

    def _exchange_fds(self, fds):
        """All-gather of file descriptors through a Unix socket owned by rank 0 (SCM_RIGHTS).
        Returns, for every rank, this process's duplicates of that rank's descriptors."""
        tag = f"p2p/fd/{self._generation}/{self._xseq}"
        self._xseq += 1
        if self._rank == 0:
            name = f"\0orthon-b200-fd-{os.getpid()}-{self._generation}-{self._xseq}".encode()
            srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            srv.settimeout(RENDEZVOUS_TIMEOUT_SECONDS)
            srv.bind(name)
            srv.listen(self._world)
            self._store.set(tag, name.hex().encode())
            gathered, conns = {0: list(fds)}, []
            try:
                for _ in range(self._world - 1):
                    conn, _ = srv.accept()
                    conn.settimeout(RENDEZVOUS_TIMEOUT_SECONDS)
                    msg, got, _, _ = socket.recv_fds(conn, 256, 16)
                    head = json.loads(msg.decode())
                    if len(got) != head["n"]:
                        raise RuntimeError("file-descriptor exchange: truncated message")
                    gathered[int(head["rank"])] = list(got)
                    conns.append(conn)
                counts = [len(gathered[r]) for r in range(self._world)]
                flat = [fd for r in range(self._world) for fd in gathered[r]]
                for conn in conns:
                    socket.send_fds(conn, [json.dumps({"counts": counts}).encode()], flat)
                    conn.recv(1)  # the peer has received its duplicates
            finally:
                for conn in conns:
                    conn.close()
                srv.close()
                self._store.delete(tag)
            return [gathered[r] for r in range(self._world)]
        self._store.wait_for([tag], RENDEZVOUS_TIMEOUT_SECONDS)
        name = bytes.fromhex(self._store.get(tag).decode())
        cli = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        cli.settimeout(RENDEZVOUS_TIMEOUT_SECONDS)
        try:
            cli.connect(name)
            socket.send_fds(cli, [json.dumps({"rank": self._rank, "n": len(fds)}).encode()], list(fds))
            msg, got, _, _ = socket.recv_fds(cli, 1024, 16 * self._world)
            counts = json.loads(msg.decode())["counts"]
            cli.send(b"k")
        finally:
            cli.close()
        if len(got) != sum(counts):
            raise RuntimeError("file-descriptor exchange: truncated reply")
        out, pos = [], 0
        for c in counts:
            out.append(list(got[pos:pos + c]))
            pos += c
        return out

    def _allocate_vmm(self, nbytes):
        """cuMemCreate allocation per rank, mapped on every rank and bound to a multicast object.
        Returns None (on every rank) if any step is unavailable, so the caller can fall back."""
        dev, world, rank = self._device, self._world, self._rank
        grans = self.exchange_objects(str(_C._vmm_granularity(dev, world, True)).encode())
        gran = max(int(g) for g in grans)
        size = (nbytes + gran - 1) // gran * gran
        mine, mc_id, err = None, None, None
        own_fds = []
        try:
            mine = _C._vmm_alloc(size, gran, dev)  # (id, ptr, fd)
            own_fds.append(mine[2])
            if rank == 0:
                mc_id, mc_fd = _C._mc_create(world, size, dev)
                own_fds.append(mc_fd)
        except RuntimeError as exc:
            err = exc
        if not self._agree(err is None):
            for fd in own_fds:
                _C._close_fd(fd)
            self._vmm = False
            return None
        every = self._exchange_fds(own_fds)
        ptrs, ok = [], True
        try:
            for r in range(world):
                ptrs.append(mine[1] if r == rank else _C._vmm_import(every[r][0], size, gran, dev)[1])
            if rank != 0:
                mc_id = _C._mc_import(every[0][1], size, dev)
            _C._mc_add_device(mc_id, dev)
        except RuntimeError:
            ok = False
        finally:
            for fd in set(fd for row in every for fd in row) | set(own_fds):
                _C._close_fd(fd)
        if not self._agree(ok):  # also the "every device has been added" barrier
            self._vmm = False
            return None
        mc_ptr = None
        try:
            mc_ptr = _C._mc_bind_map(mc_id, mine[0], gran, dev)
        except RuntimeError:
            ok = False
        if not self._agree(ok):
            mc_ptr = None  # peer mappings stay usable; only the multicast view is dropped
        return SymmetricRegion(size, ptrs, rank, mc=mc_ptr)

    def next_epoch(self):
        self._epoch += 1
        return self._epoch

    INVALID_PROFILE = ("DDP gradient synchronization rejected an invalid gradient profile "
                       "on one or more ranks (dtype, shape, device, or backend support)")

    def _judge(self, code):
        """Turns a status code into the exception it stands for.  A wait that ran out poisons
        the group (the ranks are no longer in step); a rejected gradient profile does not: every
        rank left that bucket untouched, in step."""
        if not code:
            return
        self._status.fill_(0.0)
        if code == _C._PEER_ERR_INVALID_PROFILE:
            raise RuntimeError(self.INVALID_PROFILE)
        self._failure = f"peer kernel wait timed out (code {code})"
        raise _TransportFailure("p2p backend failed: " + self._failure)

    def read_words(self):
        """One device read (synchronises the compute stream): (status code, gradient found-inf)."""
        status, found, _, _ = self._words.tolist()
        return int(status), bool(found)

    def check_status(self):
        """Reads the device error word (synchronises); a timeout poisons the group."""
        self._open()
        self._judge(self.read_words()[0])

    def poll_status(self):
        """Checks the error word without waiting for the device: looks at the copy queued by the
        previous call if it has landed, then queues a fresh copy behind the work issued so far.
        A failure therefore surfaces one call late, on steps that never synchronise."""
        self._open()
        if self._poll_event is not None and self._poll_event.ready():
            self._poll_event = None
            self._judge(int(self._host_words.tolist()[0]))
        if self._poll_event is None:
            _C._copy_d2h_async(self._host_words, self._words)
            self._poll_event = _C.CudaEvent.record(self._device)

    def status_tensors(self):
        return self._status, self._found_inf

    # ------------------------------------------------------------- collectives
    def _peer_sum(self, tensor):
        """In-place sum over ranks through the symmetric staging region (compute stream).

        Tensors larger than the staging region go through it chunk by chunk, so no size falls
        back to another transport."""
        n = int(tensor.numel)
        esz = _ESIZE[tensor.dtype]
        flat = tensor.reshape([-1])
        cap = (STAGING_BYTES // esz) & ~7
        off = 0
        while off < n:
            m = min(cap, n - off)
            self._peer_sum_chunk(flat, off, m, tensor.dtype, esz)
            off += m
        return True

    def _peer_sum_chunk(self, flat, off, n, dtype, esz):
        padded = (n + 7) & ~7
        stage = _C._tensor_from_ptr(self._stage.local, [padded], dtype, self._device)
        if padded != n:
            stage.fill_(0.0)
        stage._copy_flat_range_from(0, flat, off, n)
        grads = list(self._stage.ptrs)
        staging = [p + STAGING_BYTES for p in self._stage.ptrs]
        flags = [p + 2 * STAGING_BYTES for p in self._stage.ptrs]
        _C._peer_reduce(self._rank, self._world, self._device, grads, staging, flags, padded, dtype, self.next_epoch(),
                        1.0, "average", padded * esz <= (1 << 20), status=self._status, found_inf=self._coll_inf,
                        stream_kind=0, wait_ms=self.wait_ms)
        flat._copy_flat_range_from(off, stage, 0, n)

    def _fallback(self):
        if self._nccl is None:
            from .nccl_backend import NcclBackend
            self._nccl = NcclBackend(self._rank, self._world, self._device, self._store)
        return self._nccl

    def _check(self, tensor):
        if not tensor.device.is_cuda() or tensor.device.index != self._device:
            raise RuntimeError(f"p2p collectives require tensors on cuda:{self._device}")
        if not tensor.is_contiguous:
            raise RuntimeError("p2p collectives require contiguous tensors")
        if tensor.dtype not in _ESIZE:
            raise RuntimeError(f"p2p collectives support {tuple(_ESIZE)}, got {tensor.dtype}")

    def all_reduce(self, tensor, op="sum", async_op=False):
        self._open()
        if op != "sum":
            raise NotImplementedError("p2p backend only supports all_reduce op='sum'")
        self._check(tensor)
        with _no_grad():
            if self._world > 1 and not self._peer_sum(tensor):
                return self._fallback().all_reduce(tensor, op=op, async_op=async_op)
        return Work() if async_op else tensor

    def broadcast(self, tensor, src=0, async_op=False):
        self._open()
        if not 0 <= src < self._world:
            raise ValueError("broadcast src must be in [0, world_size)")
        self._check(tensor)
        with _no_grad():
            if self._world > 1:
                # Non-source ranks contribute zeros, so the sum is the source's value.
                if self._rank != src:
                    tensor.fill_(0.0)
                if not self._peer_sum(tensor):
                    return self._fallback().broadcast(tensor, src=src, async_op=async_op)
        return Work() if async_op else tensor

    def barrier(self):
        self._open()
        if self._world > 1:
            token = _C._zeros_on([8], "float32", self._dev)
            self._peer_sum(token)
            _C.cuda_synchronize()
            self.check_status()

    def _validate_gradient_dtype(self, dtype):
        if dtype not in _ESIZE:
            raise RuntimeError(f"p2p gradient synchronization supports {tuple(_ESIZE)}, got {dtype}")

    def shutdown(self):
        if self._closed:
            return
        self._closed = True
        try:
            _C.cuda_synchronize()
            code = self.read_words()[0]
            if code and self._failure is None:
                self._failure = f"peer kernel reported code {code} before shutdown"
        except RuntimeError:
            pass
        if self._nccl is not None:
            self._nccl.shutdown()
        # Wait until every rank has stopped using the mappings before tearing them down.
        try:
            self.exchange_objects(b"bye")
            # Rank 0 may host the rendezvous store: it leaves last, once every rank has finished
            # reading (bounded wait).
            done = f"p2p/bye/{self._generation}"
            self._store.add(done, 1)
            if self._rank == 0:
                deadline = time.monotonic() + 5.0
                while self._store.add(done, 0) < self._world and time.monotonic() < deadline:
                    time.sleep(0.01)
        except Exception:  # noqa: BLE001
            pass
        _C._vmm_release_all()
        _C._peer_release_all()


__all__ = ["PeerBackend", "SymmetricRegion"]
