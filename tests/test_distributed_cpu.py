"""Host-side distributed logic with the local multiprocessing transport (no GPU)."""
import numpy as np
import pytest

import orthon_b200.distributed as dist

import dist_workloads as W


def test_local_collectives():
    res = dist.spawn(W.collectives, args=("local",), nprocs=2, backend="local")
    for r in res:
        assert r["sum1000"] == (3.0, 3.0)
        assert r["bcast"] == (np.arange(12, dtype=np.float32) * 2).tolist()


@pytest.mark.parametrize("bucket_mb", [None, 0.001, 25])
def test_local_ddp_matches_single_process(bucket_mb):
    res = dist.spawn(W.ddp_sgd_trace, args=("local", 3, bucket_mb), nprocs=2, backend="local")
    ref = W.single_process_reference(2, 3)
    assert res[0][2] == "Reducer"
    for flat, _, _ in res:
        assert np.allclose(np.asarray(flat), ref, atol=2e-5)
    assert res[0][0] == res[1][0]


def test_local_amp_ddp():
    res = dist.spawn(W.amp_ddp_trace, args=("local", 3, "float32", "auto", True), nprocs=2, backend="local")
    ref = W.single_process_reference(2, 3, optimizer="adam", lr=1e-2)
    for masters, _, _, t in res:
        assert t == 3
        assert np.allclose(np.asarray(masters), ref, atol=5e-5)


def _boom(rank):
    if rank == 1:
        raise ValueError("injected failure on rank 1")
    import orthon_b200.distributed as d
    d.barrier()
    return rank


def test_spawn_reports_worker_failure():
    with pytest.raises(RuntimeError, match="local distributed spawn failed"):
        dist.spawn(_boom, nprocs=2, backend="local")


def _mismatch(rank):
    import orthon_b200 as ob_
    import orthon_b200.distributed as d
    t = ob_.zeros([4 if rank == 0 else 5])
    d.all_reduce(t)


def test_descriptor_mismatch_aborts_group():
    with pytest.raises(RuntimeError, match="mismatch"):
        dist.spawn(_mismatch, nprocs=2, backend="local")


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_rendezvous_store_outlives_a_group_so_it_can_be_created_again():
    """torchrun-style rendezvous: the store of a process is created once and found again by the next group."""
    from orthon_b200.distributed import store as store_mod
    env = {"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(_free_port())}
    first = store_mod.store_from_env(0, 1, environ=env)
    first.set("generation/0/key", b"a")
    second = store_mod.store_from_env(0, 1, environ=env)
    assert second is first
    assert second.get("generation/0/key") == b"a"
    assert second.add("p2p/generation/0", 1) == 1 and second.add("p2p/generation/0", 1) == 2
    other = store_mod.store_from_env(0, 1, environ={"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(_free_port())})
    assert other is not first


def test_store_directory_wins_over_the_rendezvous_address(tmp_path):
    from orthon_b200.distributed import store as store_mod
    env = {"ORTHON_STORE_DIR": str(tmp_path), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "1"}
    s = store_mod.store_from_env(0, 2, environ=env)
    assert isinstance(s, store_mod.FileStore)
    s.set("k", b"v")
    assert store_mod.store_from_env(1, 2, environ=env).get("k") == b"v"


def test_no_rendezvous_information_is_an_error():
    from orthon_b200.distributed import store as store_mod
    with pytest.raises(RuntimeError, match="no rendezvous available"):
        store_mod.store_from_env(0, 1, environ={})
