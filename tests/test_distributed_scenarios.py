"""Distributed behaviour on the local (multi-process CPU) backend: facade, accumulation, tied
parameters, AMP with a non-finite gradient on one rank, partially used parameters, lifecycle."""
import numpy as np

import orthon_b200.distributed as dist

import dist_scenarios as S


def test_facade_collectives_and_double_init():
    res = dist.spawn(S.facade, nprocs=2, backend="local")
    for rank, r in enumerate(res):
        assert (r["rank"], r["world"], r["init"]) == (rank, 2, True)
        assert r["sum"] == [3.0] * 5 and r["async_done"]
        assert r["bcast"] == [10.0, 11.0, 12.0, 13.0]
        assert "already" in r["double_init"].lower() or "initialized" in r["double_init"].lower()


def test_gradient_accumulation_then_explicit_sync():
    res = dist.spawn(S.accumulation, nprocs=2, backend="local")
    (l0, s0), (l1, s1) = res
    for a, b, sa, sb in zip(l0, l1, s0, s1):
        want = (np.asarray(a) + np.asarray(b)) / 2
        assert np.allclose(np.asarray(sa), want, atol=1e-6) and np.allclose(np.asarray(sb), want, atol=1e-6)


def test_tied_parameters_are_one_owner():
    res = dist.spawn(S.tied_parameters, nprocs=2, backend="local")
    assert res[0][0] == res[1][0] == 3  # embedding weight, linear weight, linear bias
    assert res[0][1] == res[1][1]


def test_amp_skips_on_every_rank_when_one_rank_overflows():
    res = dist.spawn(S.amp_inf_on_one_rank, nprocs=2, backend="local")
    for trace, _ in res:
        assert [t[0] for t in trace] == [False, True, False]
        assert [t[1] for t in trace] == [64.0, 32.0, 32.0]
        assert [t[2] for t in trace] == [False, True, False]  # parameters unchanged only in the skipped step
    assert res[0][1] == res[1][1]


def test_partially_used_parameter_gets_the_average():
    res = dist.spawn(S.partially_used_parameter, nprocs=2, backend="local")
    gb0, ga0 = res[0]
    gb1, ga1 = res[1]
    assert gb0 is not None and gb1 is not None
    assert np.allclose(np.asarray(gb0), np.asarray(gb1))
    assert np.allclose(np.asarray(ga0), np.asarray(ga1))
    # rank 1 contributed zeros for the unused head: the average is half of rank 0's gradient
    x = np.random.default_rng(3).standard_normal((2, 4)).astype(np.float32)
    want = np.tile(x.sum(0)[:, None], (1, 3)) / 2
    assert np.allclose(np.asarray(gb0).reshape(4, 3), want, atol=1e-6)


def test_group_lifecycle():
    res = dist.spawn(S.lifecycle, nprocs=2, backend="local")
    for values, after, err in res:
        assert values == [2.0, 2.0] and after is False and err is not None
