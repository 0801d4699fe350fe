"""CPU backend: results do not depend on the worker count, strided operands need no packing,
and forked children get their own worker pool."""
import os
import subprocess
import sys

import numpy as np

import orthon_b200 as ob

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r"""
import hashlib, sys
import numpy as np
sys.path.insert(0, %r)
import orthon_b200 as ob
rng = np.random.default_rng(0)
a = ob.from_numpy(rng.standard_normal((300, 257)).astype(np.float32))
b = ob.from_numpy(rng.standard_normal((257, 190)).astype(np.float32))
a.requires_grad_(True); b.requires_grad_(True)
y = ob.linear(a @ b, ob.from_numpy(rng.standard_normal((190, 64)).astype(np.float32)), None, "gelu")
y.sum().backward()
h = hashlib.sha256()
for t in (y, a.grad, b.grad):
    h.update(np.asarray(t.tolist(), dtype=np.float32).tobytes())
print(h.hexdigest())
"""


def _digest(threads):
    env = dict(os.environ, ORTHON_CPU_THREADS=str(threads))
    out = subprocess.run([sys.executable, "-c", SCRIPT % ROOT], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr
    return out.stdout.strip().splitlines()[-1]


def test_results_are_identical_for_any_worker_count():
    assert _digest(1) == _digest(3) == _digest(8)


def test_strided_operands_match_packed_ones():
    rng = np.random.default_rng(1)
    a_np = rng.standard_normal((64, 48)).astype(np.float32)
    b_np = rng.standard_normal((48, 80)).astype(np.float32)
    a, b = ob.from_numpy(a_np), ob.from_numpy(b_np)
    at = ob.from_numpy(np.ascontiguousarray(a_np.T)).transpose(0, 1)   # strided view equal to a
    bt = ob.from_numpy(np.ascontiguousarray(b_np.T)).transpose(0, 1)   # strided view equal to b
    want = np.asarray((a @ b).tolist())
    for x, y in ((at, b), (a, bt), (at, bt)):
        assert np.array_equal(np.asarray((x @ y).tolist()), want) or np.allclose(np.asarray((x @ y).tolist()), want, rtol=1e-5, atol=1e-5)
    assert np.allclose(want.reshape(64, 80), a_np @ b_np, rtol=1e-4, atol=1e-4)


def _child(rank):
    rng = np.random.default_rng(rank)
    a = ob.from_numpy(rng.standard_normal((128, 128)).astype(np.float32))
    return float((a @ a).sum().item())


def test_spawned_workers_use_the_backend_after_the_parent_did():
    a = ob.from_numpy(np.ones((256, 256), dtype=np.float32))
    assert (a @ a).sum().item() == 256.0 ** 3  # starts the parent's worker pool
    import orthon_b200.distributed as dist
    res = dist.spawn(_child, nprocs=2, backend="local")
    assert len(res) == 2 and all(np.isfinite(v) for v in res)
