"""Routes of the matmul planner, checked without a GPU: the planner is a pure function of the
problem and of its options.  (reference project: tests/cpp/test_matmul_planner.cpp,
tests/spec/operators/test_matmul_planner_routes.py)"""
import pytest

from orthon_b200 import _C


def plan(dtype="bfloat16", m=8192, n=8192, k=8192, **kw):
    options = kw.pop("options", {})
    return _C._plan_gemm(dtype, m, n, k, options=options, **kw)


# ---------------------------------------------------------------------- float32
def test_float32_is_exact_fma_by_default():
    p = plan("float32", 4096, 4096, 4096)
    assert p["route"] == "simt128" and (p["bn"], p["tm"]) == (128, 128)


@pytest.mark.parametrize("m,n,k,route", [
    (64, 64, 64, "simt64"),          # small: parallelism over tile size
    (128, 128, 128, "simt64"),       # short reduction does not amortise the large tile
    (4096, 4096, 200, "simt64"),
    (2048, 2048, 256, "simt128"),    # fills 148 SMs at least once
    (1024, 1024, 256, "simt64"),     # 64 large tiles < 148 SMs
])
def test_float32_tile_choice(m, n, k, route):
    assert plan("float32", m, n, k)["route"] == route


def test_float32_high_precision_uses_the_tensor_cores_for_large_products_only():
    high = {"float32_precision": 1}
    assert plan("float32", 1024, 1024, 1024, options=high)["route"] == "tcgen05_float32"
    assert plan("float32", 64, 64, 64, options=high)["route"] == "simt64"
    assert plan("float32", 1024, 1024, 1024, residual=True, options=high)["route"] in ("simt64", "simt128")
    assert plan("float32", 1024, 1024, 1024, preact=True, options=high)["route"] in ("simt64", "simt128")
    assert plan("float32", 1024, 1024, 1024, act=3, options=high)["route"] in ("simt64", "simt128")
    assert plan("float32", 1024, 128, 1024, options=high)["bn"] == 128
    assert plan("float32", 1024, 129, 1024, options=high)["bn"] == 256
    assert plan("float32", 1024, 1024, 1024, options={"float32_precision": 1, "float32_split_min": 1 << 40})["route"] == "simt64"
    assert plan("float32", 2048, 2048, 1024, tcgen05=False, options=high)["route"] == "simt128"


def test_forced_routes_for_float32():
    assert plan("float32", 64, 64, 64, options={"force_route": 2})["route"] == "tcgen05_float32"
    assert plan("float32", 4096, 4096, 4096, options={"force_route": 1, "float32_precision": 1})["route"] == "simt128"
    with pytest.raises(RuntimeError, match="cannot take the tcgen05 route"):
        plan("float32", 64, 64, 64, residual=True, options={"force_route": 2})


# ------------------------------------------------------------------ 16-bit types
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_tiny_products_stay_off_the_tensor_cores(dtype):
    assert plan(dtype, 32, 32, 32)["route"] == "simt64"
    assert plan(dtype, 64, 64, 64)["route"] == "tcgen05"  # 2^18 multiply-adds is the boundary
    assert plan(dtype, 32, 32, 32, options={"force_route": 2})["route"] == "tcgen05"


def test_operands_tma_cannot_describe_fall_back():
    assert plan(m=1024, n=1024, k=1024, tma_ok=False)["route"] == "simt64"
    assert plan(m=4096, n=4096, k=1024, tma_ok=False)["route"] == "simt128"
    assert plan(m=1024, n=1024, k=1024, tcgen05=False)["route"] == "simt64"
    with pytest.raises(RuntimeError, match="cannot take the tcgen05 route"):
        plan(m=1024, n=1024, k=1024, tma_ok=False, options={"force_route": 2})
    assert plan(m=1024, n=1024, k=1024, options={"force_route": 1})["route"] == "simt64"


@pytest.mark.parametrize("n,sq,bn", [(512, 512, 128), (1024, 1024, 128), (2048, 2048, 256), (4096, 4096, 256)])
def test_square_sizes_pick_the_tile_width_that_fills_the_sms(n, sq, bn):
    p = plan(m=sq, n=n, k=sq)
    assert p["route"] == "tcgen05" and p["bn"] == bn


def test_narrow_outputs_use_narrow_tiles():
    assert plan(m=8192, n=128, k=1024)["bn"] == 128
    assert plan(m=16384, n=129, k=1024)["bn"] == 256   # 128 wide tiles: narrow ones would not fit in one wave anyway
    assert plan(m=8192, n=129, k=1024)["bn"] == 128    # 64 wide tiles would leave most SMs idle
    assert plan(m=8192, n=8192, k=1024, options={"force_bn": 128})["bn"] == 128
    assert plan(m=512, n=512, k=512, options={"force_bn": 256})["bn"] == 256


@pytest.mark.parametrize("name,m,n,k,tm", [
    ("qkv forward", 8192, 6144, 2048, 256),
    ("projection forward", 8192, 2048, 2048, 256),
    ("fc2 forward", 8192, 2048, 8192, 256),
    ("vocabulary head", 8192, 32000, 2048, 256),
    ("projection weight gradient", 2048, 2048, 8192, 128),
    ("fc1 weight gradient", 2048, 8192, 8192, 256),
    ("short reduction", 8192, 8192, 1024, 128),
])
def test_tall_tiles_on_transformer_shapes(name, m, n, k, tm):
    p = plan(m=m, n=n, k=k)
    assert p["route"] == "tcgen05" and p["bn"] == 256 and p["tm"] == tm, (name, p)


def test_tall_tiles_respect_their_conditions():
    assert plan(m=8192, n=8192, k=2048, preact=True, act=4)["tm"] == 256   # a second output goes through the same staging tile
    assert plan(m=8192, n=8192, k=2048, preact=True, options={"tall_preact": False})["tm"] == 128
    assert plan(m=256, n=8192, k=8192)["tm"] == 128                        # fewer than 512 rows
    assert plan(m=8192, n=8192, k=2047)["tm"] == 128
    assert plan(m=8192, n=8192, k=1024, options={"tall_min_k": 1024})["tm"] == 256
    assert plan(m=8192, n=8192, k=8192, options={"force_tm": 128})["tm"] == 128
    assert plan(m=256, n=512, k=512, options={"force_tm": 256, "force_bn": 256})["tm"] == 256


def test_eight_epilogue_warps_for_short_reductions():
    assert plan(m=8192, n=8192, k=1024)["epilogue_warps"] == 8
    assert plan(m=8192, n=8192, k=1025)["epilogue_warps"] == 4
    assert plan(m=8192, n=8192, k=512, preact=True)["epilogue_warps"] == 4
    assert plan(m=8192, n=8192, k=2048, options={"ew8_max_k": 2048, "tall_min_k": 4096})["epilogue_warps"] == 8
    assert plan(m=8192, n=128, k=512)["epilogue_warps"] == 4               # narrow tile


def test_split_k_for_small_outputs_with_long_reductions():
    p = plan(m=512, n=512, k=16384)
    assert p["route"] == "tcgen05_split_k" and p["splits"] == 16 and p["bn"] == 256
    assert plan(m=512, n=512, k=16384, options={"splitk": False})["route"] == "tcgen05"
    assert plan(m=512, n=512, k=16384, bias=True)["route"] == "tcgen05"      # the second pass has no epilogue
    assert plan(m=512, n=512, k=16384, batch=2)["route"] == "tcgen05"
    assert plan(m=512, n=512, k=2048)["route"] == "tcgen05"                   # reduction too short
    assert plan(m=512, n=510, k=16384)["route"] == "tcgen05"                  # the second pass stores four values at a time
    assert plan(m=2048, n=2048, k=16384)["route"] == "tcgen05"                # 128 tiles already fill the SMs
    assert plan(m=256, n=256, k=8192)["splits"] == 16                         # a slice keeps at least 512 elements of K
    assert plan(m=256, n=256, k=4096)["splits"] == 8


def test_cta_pairs_where_tall_tiles_fill_their_waves_badly():
    p = plan(m=2048, n=6144, k=8192)     # 192 tiles of 256 x 256: 65 % of two waves
    assert p["route"] == "tcgen05_pair" and (p["tm"], p["bn"]) == (128, 256)
    assert plan(m=2048, n=6144, k=8192, options={"pair_mode": 0})["route"] == "tcgen05"
    assert plan(m=2048, n=6144, k=2048)["route"] == "tcgen05"                 # short reduction
    assert plan(m=2048, n=2048, k=8192)["route"] == "tcgen05"                 # 64 pair tiles: fewer than the 74 pairs of SMs
    assert plan(m=2048, n=8192, k=8192)["route"] == "tcgen05"                 # tall tiles fill 86 %: kept


def test_cta_pairs_only_on_request():
    assert plan(m=8192, n=8192, k=8192)["route"] == "tcgen05"
    p = plan(m=8192, n=8192, k=8192, options={"pair_mode": 1})
    assert p["route"] == "tcgen05_pair" and (p["tm"], p["bn"], p["epilogue_warps"]) == (128, 256, 4)
    p = plan(m=8192, n=8192, k=2048, options={"pair_mode": 1})
    assert p["epilogue_warps"] == 8
    p = plan(m=8192, n=8192, k=8192, options={"pair_mode": 2})
    assert p["route"] == "tcgen05_pair" and (p["tm"], p["bn"]) == (256, 256)
    assert plan(m=256, n=8192, k=8192, options={"pair_mode": 2})["tm"] == 128   # fewer than 512 rows: 256-row pair tile
    assert plan(m=128, n=8192, k=8192, bias=True, options={"pair_mode": 1})["route"] == "tcgen05"   # one row block: nothing to pair
    assert plan(m=8192, n=128, k=8192, bias=True, options={"pair_mode": 1})["route"] == "tcgen05"   # narrow tile
    assert plan(m=8192, n=8192, k=8192, options={"pair_mode": 0})["route"] == "tcgen05"


def test_plan_text_names_route_tile_and_reason():
    text = plan(m=8192, n=8192, k=8192)["text"]
    assert text.startswith("tcgen05 256x256 ew4") and "(" in text
    assert "splits 16" in plan(m=512, n=512, k=16384)["text"]
    assert plan(m=8192, n=8192, k=8192, options={"pair_mode": 2})["text"].startswith("tcgen05_pair 512x256")


def test_options_come_from_the_environment(monkeypatch):
    for name, value in (("ORTHON_FLOAT32_MATMUL", "high"), ("ORTHON_GEMM_BN", "128"), ("ORTHON_GEMM_TM", "256"),
                        ("ORTHON_GEMM_TALL_MIN_K", "512"), ("ORTHON_GEMM_EW8_MAX_K", "64"), ("ORTHON_GEMM_SPLITK", "0"),
                        ("ORTHON_GEMM_PAIR", "2"), ("ORTHON_GEMM_PAIR_EW8_MAX_K", "128"), ("ORTHON_GEMM_F32_SPLIT_MIN", "77"),
                        ("ORTHON_GEMM_TALL_PREACT", "0")):
        monkeypatch.setenv(name, value)
    o = _C._gemm_plan_options_from_environment()
    assert o == {"float32_precision": 1, "float32_split_min": 77, "force_bn": 128, "force_tm": 256, "tall_min_k": 512,
                 "ew8_max_k": 64, "splitk": False, "pair_mode": 2, "pair_ew8_max_k": 128, "tall_preact": False}
    for name in ("ORTHON_FLOAT32_MATMUL", "ORTHON_GEMM_BN", "ORTHON_GEMM_TM", "ORTHON_GEMM_TALL_MIN_K", "ORTHON_GEMM_EW8_MAX_K",
                 "ORTHON_GEMM_SPLITK", "ORTHON_GEMM_PAIR", "ORTHON_GEMM_PAIR_EW8_MAX_K", "ORTHON_GEMM_F32_SPLIT_MIN"):
        monkeypatch.delenv(name)
    o = _C._gemm_plan_options_from_environment()
    assert o["float32_precision"] == 0 and o["pair_mode"] == -1 and o["splitk"] is True and o["tall_min_k"] == 2048
