"""DDP runtime contracts on live CPU ranks (local backend): training modes with rank-divergent
participation, rejected gradient profiles, descriptor mismatches, preflight refusals, worker
failure, a rank that never joins, outstanding asynchronous work, group re-initialisation,
strided and shared-storage gradients, unused parameters, AMP rounds.
(reference project: tests/spec/distributed/workloads.py:199-590, cases.py:6-11)"""
import numpy as np
import pytest

import orthon_b200.distributed as dist

import dist_runtime as R

MODES = [pytest.param({"manual": True}, id="manual"), pytest.param({}, id="automatic"),
         pytest.param({"bucket": 0.000001}, id="bucket-small"), pytest.param({"bucket": 1.0}, id="bucket-large"),
         pytest.param({"bucket": 0.000001, "overlap": True}, id="overlap-small"),
         pytest.param({"bucket": 1.0, "overlap": True}, id="overlap-large")]
CA, CB = np.array([1.0, 2.0, 3.0, 5.0]), np.array([2.0, -1.0])


def _g(entry):
    return None if entry is None else np.asarray(entry[2])


@pytest.mark.parametrize("options", MODES)
def test_training_modes_average_what_each_rank_contributed(options):
    (r0, diag0, kind), (r1, _, _) = dist.spawn(R.training_modes, args=(options,), nprocs=2, backend="local")
    assert kind == "Reducer"
    assert r0 == r1                                     # replicas see identical gradients after every pass
    # Factors 2 (rank 0) and 6 (rank 1); gradients accumulate because nothing calls zero_grad.
    expect = [
        (CA * 1.0, CB * 3.0),      # pass 0: rank 0 used a (2 CA), rank 1 used b (6 CB); idle ranks contribute zeros
        (CA * 2.0, CB * 6.0),      # pass 1: (CA + 2 CA, CA) -> 2 CA ; (3 CB, 3 CB + 6 CB) -> 6 CB
        (CA * 6.0, CB * 6.0),      # pass 2: both use a: (2 CA + 2 CA, 2 CA + 6 CA) -> 6 CA ; b untouched
        (CA * 6.0, CB * 6.0),      # pass 3: the graph reaches no parameter
    ]
    for got, (want_a, want_b) in zip(r0, expect):
        a, b, unused = (_g(e) for e in got)
        assert np.allclose(a, want_a) and np.allclose(b, want_b) and unused is None
    assert diag0["outstanding"] == 0
    if options.get("overlap"):
        assert diag0["async_launches"] >= 1
    else:
        assert diag0["async_launches"] == 0


@pytest.mark.parametrize("kind", ["low-precision", "backend-dtype"])
def test_rejected_gradient_profile_raises_on_every_rank_before_any_data_moves(kind):
    res = dist.spawn(R.rejected_profile, args=(kind,), nprocs=2, backend="local")
    for r in res:
        assert r["message"] is not None and "invalid gradient profile" in r["message"]
        assert r["unchanged"]
        assert r["control_shapes"] == [(3, 1)]            # one control collective, zero data collectives
        assert r["diag"]["async_launches"] == 0 and r["diag"]["outstanding"] == 0
        assert r["sum"] == [3.0, 4.0]                     # the group is still in step


@pytest.mark.parametrize("kind", ["shape", "dtype", "collective", "barrier", "source"])
def test_descriptor_mismatch_fails_the_group_on_every_rank(kind):
    res = dist.spawn(R.descriptor_mismatch, args=(kind,), nprocs=2, backend="local")
    for r in res:
        assert r["first"] is not None and "mismatch" in r["first"]
        assert r["second"] is not None and "failed" in r["second"]
        assert r["unchanged"]


def test_invalid_collectives_are_refused_before_they_enter_the_sequence():
    res = dist.spawn(R.preflight_rejections, nprocs=2, backend="local")
    for refused, total, flag in res:
        assert refused == ["op", "src", "negative src", "strided", "bfloat16", "bool reduction"]
        assert total == [3.0, 4.0]
        assert flag == [1.0] or flag == [True]


def test_a_failing_worker_aborts_the_others_and_spawn_reports_it():
    with pytest.raises(RuntimeError) as info:
        dist.spawn(R.failing_worker, nprocs=3, backend="local")
    text = str(info.value)
    assert text.startswith("local distributed spawn failed")
    assert "worker failure injected by the test" in text and "rank 2 failed" in text


def test_a_rank_that_never_joins_becomes_a_bounded_sticky_failure():
    res = dist.spawn(R.absent_rank, nprocs=2, backend="local")
    r = res[0]
    assert res[1] == "absent"
    assert r["first"] is not None and "timed out" in r["first"]
    assert 0.3 <= r["waited"] < 5.0
    assert r["second"] is not None and "failed" in r["second"]


def test_zero_grad_refuses_while_asynchronous_work_is_outstanding():
    for r in dist.spawn(R.zero_grad_with_outstanding_work, nprocs=2, backend="local"):
        assert r["outstanding"] >= 1
        assert r["refused"] is not None and "wait_for_gradient_sync" in r["refused"]
        assert r["after"] == 0 and r["grads_cleared"]


def test_group_can_be_destroyed_and_initialised_again():
    res = dist.spawn(R.reinitialise, nprocs=2, backend="local")
    for rank, r in enumerate(res):
        assert r["first"] == [2.0, 2.0] and r["second"] == [3.0]
        assert r["states"] == [False, True]
        assert r["stale"] is not None and "shut down" in r["stale"]
        assert r["no_group"] is not None and "not initialized" in r["no_group"]
        assert r["returned_backend"] == "LocalBackend" and r["rank"] == rank


@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_strided_gradients_are_averaged_by_value(dtype):
    res = dist.spawn(R.strided_gradient, args=(dtype,), nprocs=2, backend="local")
    # rank 0's logical gradient is [[2, 6], [4, 8]], rank 1's [[6, 4], [6, 8]]
    want = [4.0, 5.0, 5.0, 8.0]
    for shown, _ in res:
        assert shown[0] == dtype and shown[1] == (2, 2) and shown[2] == want


def test_views_of_one_buffer_are_distinct_owners():
    for count, ga, gb in dist.spawn(R.owners_sharing_storage, nprocs=2, backend="local"):
        assert count == 2 and ga == [4.0, 4.0] and gb == [12.0, 12.0]


def test_globally_unused_parameter_keeps_no_gradient_and_no_optimizer_state():
    res = dist.spawn(R.unused_parameter_state, nprocs=2, backend="local")
    for rank, r in enumerate(res):
        assert r["unused"] == [5.0] and r["grad"] is None and r["m"] is None and r["v"] is None
        assert r["buffer"] == [float(rank)]               # buffers are not broadcast
    assert res[0]["a"] == res[1]["a"]


def test_manual_gradients_and_repeated_synchronisation():
    res = dist.spawn(R.manual_gradients, nprocs=2, backend="local")
    for first, same, final, unused in res:
        assert first[2] == [4.0] * 4 and same and unused is None
        assert final[2] == [10.0] * 4                     # (2 * 4 + 3 * 4) / 2


@pytest.mark.parametrize("mode", ["enabled", "disabled", "direct"])
def test_amp_rounds_with_rank_local_gradients(mode):
    res = dist.spawn(R.amp_rounds, args=(mode,), nprocs=2, backend="local")
    assert res[0] == res[1]
    rounds = res[0]
    # a gets 4/2 per applied round, b gets 8/2, lr 0.25; unused never moves
    if mode == "enabled":
        assert [r["scale"] for r in rounds] == [4.0, 2.0, 2.0]
        assert rounds[0]["params"] == [9.5, 19.0, 30.0]
        assert rounds[1]["params"] == [9.5, 19.0, 30.0]   # skipped on both ranks
        assert rounds[2]["params"] == [9.0, 18.0, 30.0]
    else:
        assert [r["params"] for r in rounds] == [[9.5, 19.0, 30.0], [9.0, 18.0, 30.0], [8.5, 17.0, 30.0]]


def test_reducer_variant_follows_the_measured_crossovers():
    """Which kernel reduces a bucket is a pure function of the group size, the bucket size and whether the
    buckets could be bound to a multicast object."""
    from orthon_b200.parallel.peer_reducer import PeerReducer as R
    KB, MB = 1 << 10, 1 << 20
    # two ranks: peer loads at every size, one-shot up to 512 KB
    assert R.choose_variant(2, 25 * MB, True) == "two_shot"
    assert R.choose_variant(2, 512 * KB, True) == "one_shot"
    assert R.choose_variant(2, 512 * KB + 2, False) == "two_shot"
    # four and eight ranks: in-switch from 8 KB on when the box has multicast
    for world in (4, 8):
        assert R.choose_variant(world, 25 * MB, True) == "in_switch"
        assert R.choose_variant(world, 8 * KB, True) == "in_switch"
        assert R.choose_variant(world, 4 * KB, True) == "one_shot"
        assert R.choose_variant(world, 25 * MB, False) == "two_shot"
    # without multicast the one-shot limit shrinks with the group
    assert R.choose_variant(4, 32 * KB, False) == "one_shot" and R.choose_variant(4, 64 * KB, False) == "two_shot"
    assert R.choose_variant(8, 16 * KB, False) == "one_shot" and R.choose_variant(8, 32 * KB, False) == "two_shot"
    assert R.choose_variant(6, 16 * KB, False) == "one_shot"
    assert R.choose_variant(3, 32 * KB, False) == "one_shot"


def test_reducer_variant_thresholds_can_be_moved(monkeypatch):
    from orthon_b200.parallel.peer_reducer import PeerReducer as R
    monkeypatch.setattr(R, "NVLS_MIN_WORLD", 0)
    assert R.choose_variant(8, 1 << 26, True) == "two_shot"
    monkeypatch.setattr(R, "NVLS_MIN_WORLD", 2)
    assert R.choose_variant(2, 1 << 26, True) == "in_switch"
    monkeypatch.setattr(R, "NVLS_MIN_BYTES", 1 << 27)
    assert R.choose_variant(2, 1 << 26, True) == "two_shot"
