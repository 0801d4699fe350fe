"""Multi-GPU checks of the peer-memory transport and the fused reducer, at 2, 4 and 8 ranks of
one box (each size runs where that many GPUs are visible).
(reference project: tests/python/test_distributed_nccl.py:19-61,418-784)"""
import os

import numpy as np
import pytest

import orthon_b200 as ob
import orthon_b200.distributed as dist

import dist_workloads as W

pytestmark = pytest.mark.gpu


def _gpus():
    try:
        return ob.cuda_device_count()
    except Exception:  # noqa: BLE001
        return 0


def _worlds(*sizes):
    return [pytest.param(n, marks=pytest.mark.skipif(_gpus() < n, reason=f"needs {n} GPUs")) for n in sizes]


WORLDS = _worlds(2, 4, 8)


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("backend", ["p2p", "nccl"])
def test_collectives(backend, world):
    res = dist.spawn(W.collectives, args=(backend,), nprocs=world, backend=backend)
    total = float(world * (world + 1) // 2)
    for r in res:
        for n in (1, 7, 1000, 300_000):
            assert r[f"sum{n}"] == (total, total)
        assert r["bcast"] == (np.arange(12, dtype=np.float32).reshape(3, 4) * world).reshape(-1).tolist()
        assert r["bf16"] == [0.5 * total, 0.5 * total]


@pytest.mark.parametrize("world", WORLDS)
def test_peer_ddp_matches_single_process(world):
    res = dist.spawn(W.ddp_sgd_trace, args=("p2p", 3, 0.001), nprocs=world, backend="p2p")
    ref = W.single_process_reference(world, 3)
    assert res[0][2] == "PeerReducer"
    for flat, _, _ in res:
        assert np.allclose(np.asarray(flat), ref, atol=2e-5)
    assert all(r[0] == res[0][0] for r in res)  # bit-identical replicas


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("fused", ["update", "reduce", "overlap"])
def test_peer_amp_fused_adam(fused, world):
    res = dist.spawn(W.amp_ddp_trace, args=("p2p", 3, "float32", fused, False), nprocs=world, backend="p2p")
    ref = W.single_process_reference(world, 3, optimizer="adam", lr=1e-2)
    for masters, model_vals, losses, t in res:
        assert t == 3
        assert np.allclose(np.asarray(masters), ref, atol=5e-5)
    assert all(r[0] == res[0][0] for r in res)


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("dtype,fused", [("bfloat16", "reduce"), ("float16", "overlap")])
def test_peer_amp_low_precision_with_scaler(dtype, fused, world):
    res = dist.spawn(W.amp_ddp_trace, args=("p2p", 4, dtype, fused, True), nprocs=world, backend="p2p")
    ref = W.single_process_reference(world, 4, optimizer="adam", lr=1e-2)
    for masters, model_vals, losses, t in res:
        assert t == 4
        assert np.allclose(np.asarray(masters), ref, atol=0.05)
        assert np.allclose(np.asarray(model_vals), np.asarray(masters), atol=0.02)
    assert all(r[0] == res[0][0] for r in res)


@pytest.mark.parametrize("world", WORLDS)
def test_accumulation_then_explicit_sync(world):
    res = dist.spawn(W.accumulation_explicit_sync, args=("p2p",), nprocs=world, backend="p2p")
    assert res[0][2] == "PeerReducer"
    want = [sum(np.asarray(r[0][k]) for r in res) / world for k in range(len(res[0][0]))]
    for _, synced, _ in res:
        for got, expect in zip(synced, want):
            assert np.allclose(np.asarray(got), expect, atol=1e-6)


@pytest.mark.parametrize("world", _worlds(2))
def test_amp_accumulation_modes(world):
    ref = W.amp_accumulation_reference(world)
    refused, values = dist.spawn(W.amp_accumulation, args=("p2p", "reduce"), nprocs=world, backend="p2p")[0]
    assert refused is None
    assert np.allclose(np.asarray(values), ref, atol=5e-5)
    for fused in ("overlap", "update"):
        res = dist.spawn(W.amp_accumulation, args=("p2p", fused), nprocs=world, backend="p2p")
        for refused, _ in res:
            assert refused is not None and "zero_grad" in refused


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("fused", ["reduce", "overlap"])
def test_amp_skips_on_every_rank_when_one_rank_overflows(fused, world):
    res = dist.spawn(W.amp_inf_on_last_rank, args=("p2p", fused), nprocs=world, backend="p2p")
    for trace, _ in res:
        assert [t[0] for t in trace] == [False, True, False]
        assert [t[1] for t in trace] == [64.0, 32.0, 32.0]
        assert [t[2] for t in trace] == [False, True, False]
    assert all(r[1] == res[0][1] for r in res)


@pytest.mark.parametrize("world", WORLDS)
def test_found_inf_reaches_every_rank_from_a_late_block(world):
    n = 1 << 22
    res = dist.spawn(W.found_inf_in_a_late_block, args=("p2p", n), nprocs=world, backend="p2p")
    mean = (world + 1) / 2
    for r in res:
        code, hit, blocks, first = r["clean"]
        assert (code, hit) == (0, False) and blocks > 1 and first == mean
        code, hit, blocks, first = r["poisoned"]
        assert (code, hit) == (0, True) and first == mean


@pytest.mark.parametrize("world", _worlds(2, 4))
def test_participation_consensus(world):
    x = np.random.default_rng(3).standard_normal((2, 4)).astype(np.float32)
    res = dist.spawn(W.participation, args=("p2p", "partial"), nprocs=world, backend="p2p")
    assert res[0]["reducer"] == "PeerReducer"
    want = np.tile(x.sum(0)[:, None], (1, 3)) / world
    for r in res:
        assert r["error"] is None
        assert np.allclose(np.asarray(r["b"]).reshape(4, 3), want, atol=1e-6)
    res = dist.spawn(W.participation, args=("p2p", "unused"), nprocs=world, backend="p2p")
    for r in res:
        assert r["error"] is None and r["b"] is None and r["a"] is not None
    res = dist.spawn(W.participation, args=("p2p", "invalid"), nprocs=world, backend="p2p")
    assert "needs a gradient for every parameter" in res[0]["error"]          # the rank that lacks the gradient
    for r in res[1:]:
        assert "rejected an invalid gradient profile" in r["error"]           # everybody else is told
    assert all(r["unchanged"] for r in res)                                   # and nobody applied the step


@pytest.mark.parametrize("world", _worlds(2))
def test_a_rank_that_never_joins_times_out_into_a_sticky_failure(world, monkeypatch):
    monkeypatch.setenv("ORTHON_NVLS", "0")
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    res = dist.spawn(W.missing_peer, args=("p2p",), nprocs=world, backend="p2p")
    first = res[0]
    assert first["first"] is not None and "code 11" in first["first"]
    assert first["second"] is not None and "failed" in first["second"]


@pytest.mark.parametrize("world", _worlds(2, 4, 8))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_nvls_reducer_matches_peer_reducer(dtype, world):
    n = 3 * (1 << 18) + 64  # not a multiple of the per-rank slice granularity
    res = dist.spawn(W.nvls_reduce, args=("p2p", dtype, n), nprocs=world, backend="p2p")
    if "skipped" in res[0]:
        pytest.skip(res[0]["skipped"])
    tol = 1e-6 if dtype == "float32" else 2e-2
    for r in res:
        expect = np.asarray(r["expect"], dtype=np.float32)
        assert np.allclose(np.asarray(r["nvls"]), expect, atol=tol, rtol=tol)
        assert np.allclose(np.asarray(r["peer"]), expect, atol=tol, rtol=tol)
        assert r["found_inf"] == 0
        # One Adam step from zero moments moves every weight by -lr * sign(g) (bias-corrected).
        g = expect
        step = np.asarray(r["master"], dtype=np.float32)
        nz = np.abs(g) > 1e-2
        assert np.allclose(step[nz], -1e-2 * np.sign(g[nz]), atol=2e-4)
    assert all(r["nvls"] == res[0]["nvls"] for r in res)  # every rank holds the same bits


def test_bounded_wait_runs_out_on_one_gpu():
    """One GPU plays rank 0 of a two-rank group whose second rank does not exist: the 'peer'
    buffers are this GPU's own memory, which nobody writes.  With a budget of 2 ms the entry
    barrier gives up, the kernel returns with status 11 and leaves the data alone."""
    from orthon_b200 import _C
    n = 1 << 14
    dev = "cuda:0"
    mine, fake = _C._zeros_on([n], "float32", dev), _C._zeros_on([n], "float32", dev)
    mine.fill_(3.0)
    stage = [_C._zeros_on([n], "float32", dev) for _ in range(2)]
    flags = [_C._zeros_on([_C._PEER_FLAG_BYTES // 4], "int32", dev) for _ in range(2)]
    status, found = _C._zeros_on([1], "int32", dev), _C._zeros_on([1], "int32", dev)
    _C._peer_reduce(0, 2, 0, [mine._data_ptr, fake._data_ptr], [s._data_ptr for s in stage], [f._data_ptr for f in flags], n,
                    "float32", 1, 0.5, "average", False, status=status, found_inf=found, stream_kind=0, wait_ms=2.0)
    ob.cuda_synchronize()
    assert status.tolist() == [11]
    assert found.tolist() == [0]
    assert set(mine.tolist()) == {3.0}
