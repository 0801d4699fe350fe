"""Host-side plan of the implicit-GEMM convolution launches: the index arithmetic the kernel
relies on, checked without a GPU.  (reference project: the kernel selectors of
src/backends/cuda/conv2d_cuda.cu and tests/spec/nn/test_conv2d.py play this role there)"""
import itertools

import numpy as np
import pytest

from orthon_b200 import _C

SMALL_CNN = [(128, 3, 32, 32, 32, 3, 3, 1, 1), (128, 32, 32, 32, 64, 3, 3, 2, 1), (128, 64, 16, 16, 128, 3, 3, 2, 1)]
ODD = [(2, 5, 12, 12, 7, 3, 3, 1, 1), (3, 4, 9, 11, 20, 3, 3, 2, 0), (1, 16, 8, 8, 24, 1, 1, 1, 0), (2, 6, 10, 10, 130, 3, 3, 1, 1),
       (2, 40, 16, 16, 16, 5, 5, 1, 2), (5, 8, 20, 20, 8, 3, 3, 3, 1), (2, 8, 8, 8, 16, 1, 1, 2, 0), (2, 4, 9, 9, 8, 2, 2, 3, 0),
       (4, 300, 14, 14, 96, 3, 3, 1, 1), (1, 3, 224, 224, 64, 7, 7, 2, 3), (2, 8, 5, 40, 8, 1, 9, 1, 4)]


def plan(which, case, sms=148):
    N, C, H, W, K, R, S, stride, pad = case
    return _C._plan_conv(which, N, C, H, W, K, R, S, stride, stride, pad, pad, sms)


@pytest.mark.parametrize("case", SMALL_CNN + ODD)
@pytest.mark.parametrize("which", ["forward", "input_gradient", "weight_gradient"])
def test_ring_and_grid_fit_the_sm(which, case):
    p = plan(which, case)
    if not p["eligible"]:
        assert which == "weight_gradient"
        return
    assert 2 <= p["stages"] <= 4
    assert p["stage_bytes"] % 1024 == 0 and p["gather_bytes"] % 1024 == 0
    assert p["smem_bytes"] == p["stages"] * p["stage_bytes"] + 1280
    assert p["smem_bytes"] <= 227 * 1024
    assert p["ctas_per_sm"] in (1, 2)
    assert p["ctas_per_sm"] * (p["smem_bytes"] + 1024) <= 227 * 1024 or p["ctas_per_sm"] == 1
    assert p["ctas_per_sm"] * p["tmem_cols"] <= 512
    assert p["tmem_cols"] >= p["bn"] and p["tmem_cols"] & (p["tmem_cols"] - 1) == 0 and p["tmem_cols"] >= 32
    assert p["bn"] % 16 == 0 and 16 <= p["bn"] <= 256
    assert 1 <= p["grid"] <= 148 * p["ctas_per_sm"] and p["grid"] <= p["items"]
    # the operands of one ring slot: 64 taps x 128 pixels gathered (or bn rows x 64 pixels), bn (or 128) rows by TMA
    if which == "weight_gradient":
        assert p["gather_bytes"] >= p["bn"] * 128 and p["stage_bytes"] == p["gather_bytes"] + 16384
    else:
        assert p["gather_bytes"] == 16384 and p["stage_bytes"] >= 16384 + p["bn"] * 128


@pytest.mark.parametrize("case", SMALL_CNN + ODD)
def test_forward_tiles_cover_every_output_pixel_and_channel(case):
    N, C, H, W, K, R, S, stride, pad = case
    p = plan("forward", case)
    assert p["eligible"]
    OH, OW = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
    assert (p["out_h"], p["out_w"]) == (OH, OW)
    assert p["rows_total"] == C * R * S
    assert p["tiles_m"] * 128 >= N * OH * OW > (p["tiles_m"] - 1) * 128
    assert p["tiles_n"] * p["bn"] >= K > (p["tiles_n"] - 1) * p["bn"]
    assert p["items"] == p["tiles_m"] * p["tiles_n"]
    assert p["weight_ld"] % 8 == 0 and 0 <= p["weight_ld"] - C * R * S < 8
    assert p["pad_weights"] == (C * R * S % 8 != 0)
    assert p["fast"] == (OW % 8 == 0 and S <= 8)


@pytest.mark.parametrize("case", SMALL_CNN + ODD)
def test_stride_classes_partition_pixels_and_taps(case):
    """Every input pixel belongs to exactly one class, every filter tap to the classes that can see it, and the
    (class, tap) pairs reproduce the direct formula oh = (ih + ph - r) / sh exactly."""
    N, C, H, W, K, R, S, stride, pad = case
    p = plan("input_gradient", case)
    assert p["eligible"] and p["classes"] == stride * stride == len(p["stride_classes"])
    owner = np.full((H, W), -1)
    for z, c in enumerate(p["stride_classes"]):
        assert (c["a"], c["b"]) == divmod(z, stride)
        rows, cols = range(c["a"], H, stride), range(c["b"], W, stride)
        assert (c["ha"], c["wb"]) == (len(rows), len(cols))
        for ih in rows:
            for iw in cols:
                assert owner[ih, iw] == -1
                owner[ih, iw] = z
        taps_r = [r for r in range(R) if (c["a"] + pad - r) % stride == 0]
        taps_s = [s for s in range(S) if (c["b"] + pad - s) % stride == 0]
        assert taps_r == [c["ra0"] + stride * i for i in range(c["ra"])]
        assert taps_s == [c["sb0"] + stride * i for i in range(c["sb"])]
        for i, ih in enumerate(rows):
            for ri, r in enumerate(taps_r):
                assert (ih + pad - r) % stride == 0 and (ih + pad - r) // stride == i + c["qa"] - ri
        for j, iw in enumerate(cols):
            for si, s in enumerate(taps_s):
                assert (iw + pad - s) // stride == j + c["qb"] - si
    assert (owner >= 0).all()
    biggest = max(c["ha"] * c["wb"] for c in p["stride_classes"])
    assert p["tiles_m"] * 128 >= N * biggest
    assert p["stride_classes"][0]["ha"] * p["stride_classes"][0]["wb"] == biggest
    taps_max = max(c["ra"] * c["sb"] for c in p["stride_classes"])
    assert p["weight_ld"] % 8 == 0 and p["weight_ld"] >= K * taps_max
    assert p["zero_fill"] == (stride > R or stride > S)
    assert p["zero_fill"] == any(c["ra"] * c["sb"] == 0 and c["ha"] * c["wb"] > 0 for c in p["stride_classes"])
    assert p["fast"] == (W % (8 * stride) == 0 and S <= 8)
    if p["fast"]:
        assert all(c["wb"] % 8 == 0 for c in p["stride_classes"])
    assert p["items"] == p["tiles_m"] * p["tiles_n"] * p["classes"]


@pytest.mark.parametrize("case", SMALL_CNN + ODD)
@pytest.mark.parametrize("sms", [1, 16, 148])
def test_weight_gradient_slices_cover_the_reduction_once(case, sms):
    N, C, H, W, K, R, S, stride, pad = case
    p = plan("weight_gradient", case, sms)
    OH, OW = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
    P = OH * OW
    if K > 128 or P % 8:
        assert not p["eligible"] and ("128" in p["why"] or "8 pixels" in p["why"])
        return
    assert p["eligible"]
    rows = C * R * S + 1
    assert p["rows_total"] == rows
    assert p["tiles_n"] * p["bn"] >= rows and p["ldp"] == p["tiles_n"] * p["bn"] and p["bn"] <= 256
    assert p["kb_total"] == N * ((P + 63) // 64)
    assert p["splits"] * p["kb_per_split"] >= p["kb_total"] > (p["splits"] - 1) * p["kb_per_split"]
    assert p["items"] == p["tiles_n"] * p["splits"]
    assert p["items"] <= max(p["tiles_n"], sms * p["ctas_per_sm"])     # one wave unless a single slice per tile is already more
    assert p["splits"] <= (p["kb_total"] + 3) // 4                      # no more than one slice per four blocks of 64 pixels


def test_small_cnn_layers_take_the_row_uniform_gather_with_two_ctas_per_sm():
    for case in SMALL_CNN:
        for which in ("forward", "input_gradient", "weight_gradient"):
            p = plan(which, case)
            assert p["eligible"] and p["fast"], (which, case, p["text"])
            if which != "weight_gradient" or p["bn"] <= 64:
                assert p["ctas_per_sm"] == 2, (which, case, p["text"])


def test_invalid_geometry_and_large_tensors_are_refused_with_a_reason():
    assert _C._plan_conv("forward", 1, 1, 2, 2, 1, 3, 3, 1, 1, 0, 0)["why"] == "invalid geometry"
    assert _C._plan_conv("forward", 0, 1, 8, 8, 1, 3, 3)["why"] == "invalid geometry"
    huge = _C._plan_conv("forward", 4096, 1024, 32, 32, 8, 1, 1)
    assert not huge["eligible"] and "32 bits" in huge["why"]
    with pytest.raises(ValueError):
        _C._plan_conv("sideways", 1, 1, 8, 8, 1, 3, 3)


def test_plan_text_names_the_pass_and_the_gather():
    text = plan("input_gradient", SMALL_CNN[1])["text"]
    assert text.startswith("input gradient bn32") and "classes 4" in text and "row-uniform gather" in text
    assert "per-element gather" in plan("forward", ODD[1])["text"]
    assert plan("weight_gradient", ODD[3])["text"].startswith("not eligible")
