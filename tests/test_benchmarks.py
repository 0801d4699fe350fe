"""Benchmark tooling: timer arithmetic, result-document schema and a quick run of each script."""
import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from benchmarks._support import results, timing  # noqa: E402


def test_quartiles_and_statistics():
    assert timing.quartiles([5.0]) == (5.0, 5.0, 5.0)
    assert timing.quartiles([1, 2, 3, 4]) == (1.5, 2.5, 3.5)
    assert timing.quartiles([7, 1, 3, 5, 9]) == (2.0, 5, 8.0)  # the median is in neither half
    d = timing.Statistics((4.0, 1.0, 3.0, 2.0), 10).as_dict()
    assert (d["median"], d["iqr"], d["min"], d["max"], d["samples"], d["inner"], d["units"]) == (2.5, 2.0, 1.0, 4.0, 4, 10, "ms")


def test_inner_count_targets_sample_length_and_respects_cap():
    cfg = timing.TimingConfig(warmup=0, samples=1, target_ms=40.0, cap_ms=500.0)
    assert timing.choose_inner(0.1, cfg) == 400
    assert timing.choose_inner(100.0, cfg) == 1
    assert timing.choose_inner(0.0, cfg) == 1000
    tight = timing.TimingConfig(warmup=0, samples=1, target_ms=40.0, cap_ms=40.0)
    assert timing.choose_inner(30.0, tight) == 1
    with pytest.raises(ValueError):
        timing.TimingConfig(samples=0)
    with pytest.raises(ValueError):
        timing.TimingConfig(target_ms=10, cap_ms=5)


def test_measure_counts_calls_and_syncs():
    calls, syncs = [], []
    cfg = timing.TimingConfig(warmup=2, samples=3, target_ms=0.001, cap_ms=1.0)
    stats = timing.measure(lambda: calls.append(1), lambda: syncs.append(1), cfg)
    assert len(stats.samples_ms) == 3 and stats.inner >= 1
    assert len(calls) >= 2 + 3 + 3 * stats.inner  # warm-up, estimate trials, samples
    assert len(syncs) >= 1 + 2 * 3


def test_measure_pair_alternates():
    order = []
    cfg = timing.TimingConfig(warmup=0, samples=3, target_ms=1e-9, cap_ms=1.0)  # inner count 1
    a, b = timing.measure_pair(lambda: order.append("a"), lambda: order.append("b"), config=cfg)
    assert a.inner == b.inner == 1
    assert order[-6:] == ["a", "b", "a", "b", "a", "b"]


def test_comparison_verdict_needs_disjoint_quartiles():
    fast, slow = timing.Statistics((1.0, 1.1, 1.2), 1), timing.Statistics((2.0, 2.1, 2.2), 1)
    assert timing.comparison(fast, slow)["verdict"] == "a-faster"
    assert timing.comparison(slow, fast)["verdict"] == "b-faster"
    assert timing.comparison(fast, timing.Statistics((0.9, 1.1, 1.3), 1))["verdict"] == "indistinguishable"
    assert timing.comparison(fast, slow)["ratio_a_over_b"] == pytest.approx(1.1 / 2.1)


def test_result_document_round_trip_and_strict_json(tmp_path):
    stats = timing.Statistics((1.0, 2.0, 3.0), 4)
    case = results.case_result("x/y", stats, shape=[2, 3], implementation="orthon", device="cpu", tflops=1.5)
    doc = results.document("unit", [case], {"k": 1}, environment={"git_commit": "abc", "git_dirty": False})
    path = tmp_path / "sub" / "doc.json"
    results.write_json(str(path), doc)
    loaded = results.load(str(path))
    assert loaded["schema"] == "orthon-b200-benchmark" and loaded["schema_version"] == 1 and loaded["cases"][0]["median"] == 2.0
    with pytest.raises(ValueError):
        results.write_json(str(path), {"bad": float("nan")})
    other = tmp_path / "other.json"
    other.write_text(json.dumps({"schema": "something-else", "schema_version": 1}))
    with pytest.raises(ValueError):
        results.load(str(other))


def test_provenance_names_the_loaded_extension():
    from benchmarks._support.environment import provenance

    prov = provenance()
    assert prov["extension_path"].endswith(".so") and prov["package"] == "orthon_b200" and prov["logical_cpu_count"] >= 1
    assert prov["cuda_enabled"] in (True, False)


def test_operator_benchmark_quick_run_matches_pytorch(tmp_path):
    from benchmarks import benchmark_ops

    out = tmp_path / "ops.json"
    doc = benchmark_ops.main(["--family", "all", "--device", "cpu", "--quick", "--output", str(out)])
    names = {c["name"].split("/")[0] for c in doc["cases"]}
    assert names == {"matmul", "conv2d", "fusion", "softmax_ce", "elementwise", "reductions", "dropout", "nn", "memory_pool", "no_grad"}
    bad = [c["name"] for c in doc["cases"] if c["correctness"].startswith("mismatch")]
    assert not bad, bad
    assert sum(c["correctness"] == "matched" for c in doc["cases"]) >= 20
    from benchmarks import report_benchmarks

    text = report_benchmarks.main([str(out)])
    assert "| matmul/matmul_128 | orthon | cpu | float32 | forward |" in text


def test_pytorch_comparison_emits_both_arms():
    from benchmarks import compare_pytorch

    doc = compare_pytorch.main(["--family", "reductions", "--device", "cpu", "--quick"])
    impls = [c["implementation"] for c in doc["cases"]]
    assert impls.count("orthon") == impls.count("torch") == 6
    assert all(c["verdict"] in ("orthon-faster", "torch-faster", "indistinguishable") for c in doc["cases"] if c["implementation"] == "orthon")


def test_training_benchmark_quick_run_with_checkpoint_overhead():
    from benchmarks import benchmark_training

    doc = benchmark_training.main(["--workload", "tiny_mlp", "--device", "cpu", "--quick", "--checkpoint-overhead"])
    names = [c["name"] for c in doc["cases"]]
    assert names == ["train_step/tiny_mlp", "checkpoint_save/tiny_mlp", "checkpoint_load/tiny_mlp"]
    assert doc["cases"][0]["correctness"] == "loss-decreased" and doc["cases"][1]["file_bytes"] > 0


def test_ddp_benchmark_spawns_cpu_ranks():
    from benchmarks import benchmark_distributed_ddp

    doc = benchmark_distributed_ddp.main(["--nprocs", "2", "--width", "32", "--depth", "2", "--batch", "16", "--steps", "2", "--warmup", "1"])
    modes = [c["mode"] for c in doc["cases"]]
    assert modes == ["single", "blocking", "bucketed", "overlap"]
    assert all(c["correctness"] == "loss-decreased" for c in doc["cases"])
    assert [c["ranks"] for c in doc["cases"]] == [1, 2, 2, 2]


def test_ddp_benchmark_under_the_launcher_with_local_backend():
    """Launched ranks have no spawn parent: the local backend takes its store from the launcher."""
    import subprocess

    cmd = [sys.executable, "-m", "orthon_b200.distributed.run", "--nproc_per_node", "2", "--backend", "local",
           os.path.join(ROOT, "benchmarks", "benchmark_distributed_ddp.py"), "--width", "32", "--depth", "2", "--batch", "16",
           "--steps", "2", "--warmup", "1", "--mode", "bucketed"]
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "ddp/bucketed" in out.stdout and "ranks=2" in out.stdout


GPU_SCRIPTS = ["bench_matmul.py", "bench_gemm_shapes.py", "bench_attention.py", "bench_conv.py", "bench_reducer.py",
               "bench_configs.py", "trace_step.py", "profile_kernels.py"]


@pytest.mark.parametrize("script", GPU_SCRIPTS)
def test_gpu_benchmark_scripts_parse_their_arguments_without_a_device(script):
    """Every benchmark script imports and documents its options on a machine without a GPU (`--help` exits 0);
    each one also explains itself in a module docstring that gives at least one command line."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "benchmarks", script)
    out = subprocess.run([sys.executable, path, "--help"], capture_output=True, text=True, cwd=root, timeout=300)
    assert out.returncode == 0, out.stderr[-400:]
    assert "usage" in out.stdout.lower()
    source = open(path).read()
    assert source.lstrip().startswith('"""') and "python " in source.split('"""')[1]


def test_bench_py_help_names_both_arms_and_the_bucket_option():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--help"], capture_output=True, text=True, cwd=root, timeout=300)
    assert out.returncode == 0, out.stderr[-400:]
    for word in ("--gpus", "--steps", "--warmup", "--impl", "--bucket-mb", "--no-anchor", "reference"):
        assert word in out.stdout
