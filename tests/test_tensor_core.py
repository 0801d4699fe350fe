"""Tensor / Buffer / Layout contracts: aliasing, versioning, dtypes, devices, broadcasting.
(reference project: tests/spec/tensor/*, tests/cpp/test_tensor_core.cpp, test_float_formats.cpp)"""
import numpy as np
import pytest

import orthon_b200 as ob
from orthon_b200 import _C


def t(a, dtype=None, grad=False):
    x = ob.from_numpy(np.asarray(a, dtype=np.float32), dtype)
    if grad:
        x.requires_grad_(True)
    return x


def test_views_share_buffer_and_write_through():
    a = t(np.arange(12).reshape(3, 4))
    v = a.transpose(0, 1)
    s = a.slice(0, 1, 3)
    r = a.reshape([4, 3])
    assert v._buffer_id == a._buffer_id == s._buffer_id == r._buffer_id
    assert v.shape == (4, 3) and v.strides == (1, 4) and not v.is_contiguous
    assert s.storage_offset == 4
    s.fill_(-1.0)
    assert a.tolist()[4:] == [-1.0] * 8
    a[0][0].fill_(7.0)
    assert r.tolist()[0] == 7.0 and v.tolist()[0] == 7.0


def test_version_bumps_once_per_logical_write():
    a = t(np.zeros(6))
    v0 = a._storage_version
    a.fill_(1.0)
    a.add_(a, alpha=0.5)
    a.mul_(2.0)
    a.set_item(0, 3.0)
    a._copy_data_(t(np.ones(6)))
    assert a._storage_version == v0 + 5
    _ = a.reshape([2, 3]).transpose(0, 1)  # metadata ops never bump
    assert a._storage_version == v0 + 5


def test_to_always_copies_and_same_dtype_cast_is_identity():
    a = t(np.arange(4))
    b = a.to("cpu")
    assert b._buffer_id != a._buffer_id
    assert a.cast("float32")._impl_id == a._impl_id
    assert a.contiguous()._impl_id == a._impl_id
    arr = np.arange(4, dtype=np.float32)
    c = ob.from_numpy(arr)
    arr[0] = 100
    assert c.tolist()[0] == 0.0  # from_numpy snapshots


def test_layout_validation():
    with pytest.raises(Exception):
        ob.zeros([2, -1])
    a = t(np.arange(6).reshape(2, 3))
    with pytest.raises(Exception):
        a.transpose(0, 1).reshape([6])  # reshape needs contiguous
    assert a.transpose(0, 1).contiguous().reshape([6]).tolist() == [0, 3, 1, 4, 2, 5]
    with pytest.raises(Exception):
        a.slice(1, 2, 5)
    assert a.flatten().shape == (6,)
    assert ob.zeros([0, 3]).numel == 0 and ob.zeros([0, 3]).numel() == 0


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16", "int32", "int64", "uint8", "int8", "bool"])
def test_all_dtypes_roundtrip_and_cast(dtype):
    src = np.array([0, 1, 2, 3, 100], dtype=np.float32)
    x = ob.cast(ob.from_numpy(src), dtype)
    assert x.dtype == dtype
    back = ob.cast(x, "float32").tolist()
    expect = [0.0, 1.0, 1.0, 1.0, 1.0] if dtype == "bool" else [0.0, 1.0, 2.0, 3.0, 100.0]
    assert back == expect
    raw = _C._tensor_to_bytes(x)
    y = _C._tensor_from_bytes(raw, list(x.shape), dtype)
    assert _C._tensor_to_bytes(y) == raw


def test_float_format_rounding():
    vals = np.array([1.0 + 2 ** -9, 1.0 + 3 * 2 ** -9, 65504.0, 1e-8, np.inf], dtype=np.float32)
    h = ob.cast(ob.from_numpy(vals), "float16").numpy()
    assert np.array_equal(h, vals.astype(np.float16))
    import torch
    b = ob.cast(ob.from_numpy(vals), "bfloat16").numpy()
    assert np.array_equal(b, torch.tensor(vals).bfloat16().float().numpy())
    nan = ob.cast(ob.from_numpy(np.array([np.nan], dtype=np.float32)), "bfloat16").numpy()
    assert np.isnan(nan[0])


def test_device_parsing():
    assert str(ob.Device("cpu")) == "cpu" and str(ob.Device("cuda")) == "cuda:0" and ob.Device("cuda:3").index == 3
    for bad in ("gpu", "cuda:", "cuda:-1", "cuda:x", "CPU", ""):
        with pytest.raises(Exception):
            ob.Device(bad)
    assert ob.Device("cpu") == "cpu" and ob.zeros([1]).device.is_cpu()


def test_broadcasting_and_scalars():
    a, b = t(np.arange(6).reshape(2, 3)), t([10, 20, 30])
    assert (a + b).tolist() == [10, 21, 32, 13, 24, 35]
    assert (a * t(np.ones((2, 1)) * 2)).tolist() == [0, 2, 4, 6, 8, 10]
    assert (2 - a).tolist() == [2, 1, 0, -1, -2, -3]
    assert (a / 2).tolist() == [0, 0.5, 1, 1.5, 2, 2.5]
    assert (1 / (a + 1)).tolist()[1] == 0.5
    with pytest.raises(Exception):
        a + t(np.ones(4))
    assert a.__add__("x") is NotImplemented
    z = ob.zeros([0, 3]) + t([1, 2, 3])
    assert z.shape == (0, 3)


def test_reductions_and_extrema_policy():
    a = t([[1, 5, 5], [np.nan, 2, np.nan]])
    v, i = a.max(1), a.argmax(1)
    assert v.tolist()[0] == 5 and i.tolist() == [1, 0]  # first max, first NaN wins
    assert np.isnan(v.tolist()[1])
    assert a.slice(0, 0, 1).sum().tolist() == [11.0]
    assert t(np.arange(6).reshape(2, 3)).mean(0).tolist() == [1.5, 2.5, 3.5]
    assert t(np.arange(6).reshape(2, 3)).sum(1, True).shape == (2, 1)
    assert t([3, 9, 2]).argmax().tolist() == [1]
    with pytest.raises(Exception):
        ob.zeros([0]).sum()


def test_inplace_overlap_and_grad_rules():
    a = t(np.arange(8))
    with pytest.raises(Exception):
        a.slice(0, 0, 6).add_(a.slice(0, 2, 8))
    a.add_(a, alpha=1.0)
    assert a.tolist()[3] == 6.0
    p = t([1, 2], grad=True)
    p.add_(p)  # a leaf is a plain value: in-place writes bump its version and record nothing
    p.fill_(3.0)
    p.set_item(1, 4.0)
    assert p.tolist() == [3, 4] and p.is_leaf and p.requires_grad
    h = p * 2.0
    with pytest.raises(RuntimeError, match="autograd history"):
        h.mul_(2.0)
    with ob.no_grad():
        h.mul_(2.0)
    assert h.tolist() == [12, 16]


def test_getitem_setitem_and_scalar_access():
    a = t(np.arange(6).reshape(2, 3))
    assert a[1].tolist() == [3, 4, 5] and a[1, 2].item() == 5.0 and a[-1][0].item() == 3.0
    a[0] = 9.0
    assert a.tolist()[:3] == [9, 9, 9]
    assert a.get_item([1, 1]) == 4.0
    with pytest.raises(Exception):
        a[5]
    with pytest.raises(TypeError):
        a[0.5]


def test_memory_pool_stats_and_reuse():
    _C._memory_pool_clear()
    s0 = _C._memory_pool_stats()
    x = ob.zeros([1000])
    del x
    y = ob.zeros([1000])
    s1 = _C._memory_pool_stats()
    assert s1["reused_blocks"] >= s0["reused_blocks"] + 1
    assert s1["peak_bytes"] >= s1["current_bytes"] > 0
    del y
    _C._memory_pool_set_enabled(False)
    assert not _C._memory_pool_enabled()
    z = ob.zeros([10])
    del z
    _C._memory_pool_set_enabled(True)
