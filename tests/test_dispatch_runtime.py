"""Dispatcher / registry, fake-CUDA runtime seams and native process-group ordering (host only).
(reference project: tests/cpp/test_dispatcher.cpp, test_async_runtime.cpp, test_distributed_runtime.cpp)"""
import pytest

import orthon_b200 as ob
from orthon_b200 import _C


def test_registry_contents_and_resolution():
    ks = _C._dispatch_kernels()
    ops = {k["op"] for k in ks}
    for name in ("add", "mul", "matmul", "linear", "conv2d", "layer_norm", "cross_entropy", "embedding", "adam_step"):
        assert name in ops
    assert "sub" not in ops and "div" not in ops  # composite operators own no kernels
    assert _C._dispatch_resolve("matmul", "cuda:0", "bfloat16") == "sm100_gemm_tc05_bf16"
    assert _C._dispatch_resolve("matmul", "cpu", "float32") == "cpu_matmul_f32"
    assert _C._dispatch_resolve("matmul", "cpu", "bfloat16") is None
    assert _C._dispatch_resolve("softmax", "cuda:0", "float16") == "sm100_softmax_f16"
    names = [(k["op"], k["backend"], tuple(k["dtypes"]), k["layouts"]) for k in ks]
    assert len(names) == len(set(names))


def test_unsupported_dtype_message_and_trace():
    a = ob.cast(ob.ones([2, 2]), "bfloat16")
    with pytest.raises(RuntimeError, match="unsupported dtype bfloat16 on cpu"):
        a @ a
    with pytest.raises(ValueError, match="dtype mismatch"):
        ob.ones([2]) + ob.cast(ob.ones([2]), "float64")
    seen = []
    _C._set_dispatch_trace(lambda op, kernel: seen.append((op, kernel)))
    try:
        ob.ones([2]) + ob.ones([2])
    finally:
        _C._set_dispatch_trace(None)
    assert ("add", "cpu_add_f32") in seen


@pytest.fixture
def fake_cuda():
    _C._testing_use_fake_cuda(2)
    _C._testing_fake_clear()
    yield
    _C._memory_pool_clear()
    _C._testing_use_fake_cuda(0)


def test_fake_group_orders_streams_and_never_host_waits_on_drop(fake_cuda):
    g = _C._NcclGroup(0, 2, 0, bytes(128), True)
    t = _C._empty_on([16], "float32", "cuda:0")
    v0 = t._storage_version
    _C._testing_fake_clear()
    w = g.all_reduce(t)
    log = _C._testing_fake_log()
    kinds = [e.split(":")[0] for e in log]
    assert kinds == ["record", "stream_wait", "all_reduce", "record", "stream_wait"]
    assert t._storage_version == v0 + 1  # counted as a write at enqueue time
    del w
    assert not any(e.startswith("host_wait") for e in _C._testing_fake_log())
    w2 = g.broadcast(t, 1)
    assert w2.wait() is True
    assert any(e.startswith("host_wait") for e in _C._testing_fake_log())
    g.shutdown()
    with pytest.raises(RuntimeError, match="shut down"):
        g.all_reduce(t)


def test_fake_group_validation_does_not_poison_and_failure_is_sticky(fake_cuda):
    g = _C._NcclGroup(1, 2, 1, bytes(128), True)
    with pytest.raises(Exception):
        g.all_reduce(ob.ones([4]))  # CPU tensor: preflight only
    with pytest.raises(Exception):
        g.all_reduce(_C._empty_on([4], "int32", "cuda:1"))
    with pytest.raises(Exception):
        g.all_reduce(_C._empty_on([4], "float32", "cuda:0"))  # wrong device
    t = _C._empty_on([4], "float32", "cuda:1")
    g.all_reduce(t).wait()
    _C._testing_fake_fail(True, False)
    with pytest.raises(RuntimeError, match="failed"):
        g.all_reduce(t)
    _C._testing_fake_fail(False, False)
    with pytest.raises(RuntimeError, match="failed"):
        g.all_reduce(t)  # sticky
    assert _C._testing_fake_log().count("abort") == 1
    with pytest.raises(Exception):
        _C._NcclGroup(2, 2, 0, bytes(128), True)


def test_async_error_surfaces_on_wait(fake_cuda):
    g = _C._NcclGroup(0, 1, 0, bytes(128), True)
    t = _C._empty_on([4], "float16", "cuda:0")
    w = g.all_reduce(t)
    _C._testing_fake_fail(False, True)
    with pytest.raises(RuntimeError, match="async error"):
        w.wait()
    with pytest.raises(RuntimeError, match="failed"):
        g.ensure_open()


def test_pool_reuse_with_fake_devices(fake_cuda):
    a = _C._empty_on([1024], "float32", "cuda:1")
    ptr = a._data_ptr
    del a
    b = _C._empty_on([1024], "float32", "cuda:1")
    assert b._data_ptr == ptr
    c = _C._empty_on([1024], "float32", "cuda:0")
    assert c._data_ptr != ptr
    with pytest.raises(RuntimeError, match="not available"):
        _C._empty_on([1], "float32", "cuda:5")


def test_env_defaults_and_backend_registry(monkeypatch):
    from orthon_b200.distributed import launch_env as _env, get_backend_factory, register_backend
    env = {"RANK": "3", "WORLD_SIZE": "8", "LOCAL_RANK": "3", "ORTHON_DISTRIBUTED_BACKEND": "nccl"}
    backend, kw = _env.apply_env_defaults(None, {}, env)
    assert backend == "nccl" and kw == {"rank": 3, "world_size": 8, "device": 3}
    with pytest.raises(ValueError):
        _env.apply_env_defaults(None, {}, {})
    with pytest.raises(ValueError, match="RANK must be an integer"):
        _env.rank_config_from_env({"RANK": "x"})
    with pytest.raises(ValueError, match="unknown distributed backend"):
        get_backend_factory("nope")
    register_backend("mine", lambda **kw: None)
    assert get_backend_factory("mine") is not None


def test_function_style_nccl_entry_points_drive_the_same_group(fake_cuda):
    """`_nccl_all_reduce_sum(group, t)` and friends are the spelling Orthon's private bindings use; they act on the
    same group object as the methods."""
    g = _C._NcclGroup(0, 2, 0, bytes(128), True)
    t = _C._empty_on([8], "float32", "cuda:0")
    _C._testing_fake_clear()
    w = _C._nccl_all_reduce_sum_async(g, t)
    assert isinstance(w, _C._NcclWork) and w.wait() is True
    _C._nccl_all_reduce_sum(g, t)
    _C._nccl_broadcast(g, t, 1)
    assert _C._nccl_broadcast_async(g, t, 0).wait() is True
    kinds = [e.split(":")[0] for e in _C._testing_fake_log()]
    assert kinds.count("all_reduce") == 2 and kinds.count("broadcast") == 2
    assert callable(_C._nccl_barrier)     # a one-float all-reduce on the device: exercised on real GPUs only
    with pytest.raises(Exception):
        _C._nccl_broadcast(g, t, 2)
    _C._nccl_shutdown(g)
    with pytest.raises(RuntimeError, match="shut down"):
        _C._nccl_all_reduce_sum(g, t)


def test_nccl_init_without_the_library_or_a_device_fails_with_a_reason():
    if _C.cuda_enabled() and _C.cuda_available():
        pytest.skip("a real device is present")
    with pytest.raises(Exception):
        _C._nccl_init(bytes(128), 0, 1, 0)
