"""Side-by-side timing against PyTorch: every operator case that has a PyTorch arm is sampled
alternately (A B A B ...) with the same repeat count, so that clock drift hits both.

    python benchmarks/compare_pytorch.py --family matmul --device cuda --dtype bfloat16
    python benchmarks/compare_pytorch.py --family all --device cpu --quick

Each case gets two rows (implementation `orthon` and `torch`) and a verdict that claims a
difference only when the inter-quartile ranges do not overlap.  The comparison says nothing
about which library kernels PyTorch chose; it is a reference point, not a target.
(reference project: benchmarks/compare_pytorch.py, benchmarks/_support/comparison_cases.py:110-437)
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks._support import cli, operators, results, timing  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--family", default="all", choices=["all"] + sorted(operators.FAMILIES))
    cli.add_options(ap)
    args = ap.parse_args(argv)
    ctx = operators.Context(args.device, args.dtype, args.quick, args.seed)
    if ctx.torch is None:
        raise SystemExit("PyTorch is not importable: nothing to compare against")
    ctx.torch.manual_seed(args.seed)
    config = cli.timing_config(args)
    sync_a, sync_b = cli.sync_for(args.device), cli.torch_sync_for(args.device)
    families = sorted(operators.FAMILIES) if args.family == "all" else [args.family]
    cases = []
    for family in families:
        for case in operators.FAMILIES[family](ctx):
            if case.cuda_only and not ctx.cuda:
                continue
            fn, torch_fn, _ = case.build(ctx)
            if torch_fn is None:
                continue
            correctness = operators.check(fn(), torch_fn(), args.dtype) if case.compare else "not-compared"
            a, b = timing.measure_pair(fn, torch_fn, sync_a, sync_b, config)
            verdict = timing.comparison(a, b)
            name = f"{family}/{case.name}"
            cases.append(results.case_result(name, a, shape=case.shape, implementation="orthon", device=args.device, dtype=args.dtype,
                                             mode=case.mode, correctness=correctness, ratio_vs_torch=verdict["ratio_a_over_b"],
                                             verdict=verdict["verdict"].replace("a-", "orthon-").replace("b-", "torch-")))
            cases.append(results.case_result(name, b, shape=case.shape, implementation="torch", device=args.device, dtype=args.dtype,
                                             mode=case.mode, correctness="oracle"))
    doc = results.document("compare_pytorch", cases, {"families": families, "device": args.device, "dtype": args.dtype,
                                                      "quick": args.quick, "timer": config.__dict__})
    results.emit(doc, args.output or None)
    return doc


if __name__ == "__main__":
    main()
