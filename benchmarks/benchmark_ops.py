"""Operator micro-benchmarks through the public API.

    python benchmarks/benchmark_ops.py --family elementwise --device cuda --dtype bfloat16
    python benchmarks/benchmark_ops.py --family all --device cpu --quick --output results/ops_cpu.json

Families: matmul, conv2d, fusion, softmax_ce, elementwise, reductions, dropout, nn,
memory_pool, no_grad (or `all`).  Every case is timed with the shared host timer (warm-up,
adaptive repeat count, 11 samples, median and inter-quartile range; a device synchronisation
closes each sample on CUDA) and, where a `bytes` or `flops` figure is known, reported as GB/s
or TFLOP/s.  When PyTorch is importable each result is also checked against it.
(reference project: benchmarks/benchmark_ops.py, bench_elementwise.py, bench_reductions.py,
bench_softmax_cross_entropy.py, benchmark_conv2d.py, benchmark_dropout.py, benchmark_fusion.py,
benchmark_memory_pool.py, benchmark_no_grad.py, bench_matmul.py)
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks._support import cli, operators, results, timing  # noqa: E402


def run_family(family, ctx, config, compare=True):
    out = []
    sync = cli.sync_for(ctx.device)
    for case in operators.FAMILIES[family](ctx):
        if case.cuda_only and not ctx.cuda:
            continue
        fn, torch_fn, work = case.build(ctx)
        correctness = "not-compared"
        if compare and case.compare and torch_fn is not None:
            correctness = operators.check(fn(), torch_fn(), ctx.dtype)
        stats = timing.measure(fn, sync, config)
        extra = {}
        seconds = stats.median / 1e3
        if work.get("bytes"):
            extra["gbytes_per_s"] = work["bytes"] / seconds / 1e9
        if work.get("flops"):
            extra["tflops"] = work["flops"] / seconds / 1e12
        out.append(results.case_result(f"{family}/{case.name}", stats, shape=case.shape, implementation="orthon", device=ctx.device,
                                       dtype=ctx.dtype, mode=case.mode, correctness=correctness, **extra))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--family", default="all", choices=["all"] + sorted(operators.FAMILIES))
    ap.add_argument("--no-compare", action="store_true", help="skip the PyTorch correctness check")
    cli.add_options(ap)
    args = ap.parse_args(argv)
    ctx = operators.Context(args.device, args.dtype, args.quick, args.seed)
    config = cli.timing_config(args)
    families = sorted(operators.FAMILIES) if args.family == "all" else [args.family]
    cases = []
    for family in families:
        cases += run_family(family, ctx, config, compare=not args.no_compare)
    doc = results.document("operators", cases, {"families": families, "device": args.device, "dtype": args.dtype, "quick": args.quick,
                                                "timer": config.__dict__})
    results.emit(doc, args.output or None)
    return doc


if __name__ == "__main__":
    main()
