"""Multi-GPU checks of the peer-memory transport and the fused reducer (2 GPUs of one box)."""
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


needs2 = pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")


@needs2
@pytest.mark.parametrize("backend", ["p2p", "nccl"])
def test_collectives(backend):
    res = dist.spawn(W.collectives, args=(backend,), nprocs=2, backend=backend)
    for r in res:
        for n in (1, 7, 1000, 300_000):
            assert r[f"sum{n}"] == (3.0, 3.0)
        assert r["bcast"] == (np.arange(12, dtype=np.float32) * 2).tolist()
        assert r["bf16"] == [1.5, 1.5]


@needs2
def test_peer_ddp_matches_single_process():
    res = dist.spawn(W.ddp_sgd_trace, args=("p2p", 3, 0.001), nprocs=2, backend="p2p")
    ref = W.single_process_reference(2, 3)
    assert res[0][2] == "PeerReducer"
    for flat, _, _ in res:
        assert np.allclose(np.asarray(flat), ref, atol=2e-5)
    assert res[0][0] == res[1][0]  # bit-identical replicas


@needs2
@pytest.mark.parametrize("fused", ["update", "reduce"])
def test_peer_amp_fused_adam(fused):
    res = dist.spawn(W.amp_ddp_trace, args=("p2p", 3, "float32", fused, False), nprocs=2, backend="p2p")
    ref = W.single_process_reference(2, 3, optimizer="adam", lr=1e-2)
    for masters, model_vals, losses, t in res:
        assert t == 3
        assert np.allclose(np.asarray(masters), ref, atol=5e-5)
    assert res[0][0] == res[1][0]


@needs2
def test_peer_amp_bf16_with_scaler():
    res = dist.spawn(W.amp_ddp_trace, args=("p2p", 4, "bfloat16", "reduce", True), nprocs=2, backend="p2p")
    ref = W.single_process_reference(2, 4, optimizer="adam", lr=1e-2)
    for masters, model_vals, losses, t in res:
        assert t == 4
        assert np.allclose(np.asarray(masters), ref, atol=0.05)
        assert np.allclose(np.asarray(model_vals), np.asarray(masters), atol=0.02)
    assert res[0][0] == res[1][0]


@needs2
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_nvls_reducer_matches_peer_reducer(dtype):
    n = 3 * (1 << 18) + 64  # not a multiple of the per-rank slice granularity
    res = dist.spawn(W.nvls_reduce, args=("p2p", dtype, n), nprocs=2, backend="p2p")
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
    assert res[0]["nvls"] == res[1]["nvls"]  # every rank holds the same bits
