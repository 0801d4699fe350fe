"""Summarise benchmark result documents as one Markdown table per document.

    python benchmarks/report_benchmarks.py results/*.json [--output report.md]

Reads the documents written by the benchmark scripts (`--output`), checks the schema, and
prints name / implementation / device / dtype / mode / median / inter-quartile range, the
derived rate where the case has one, and the correctness status.
(reference project: benchmarks/report_benchmarks.py, benchmarks/_support/reporting.py:8-24)
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks._support import results  # noqa: E402


def rate_of(case):
    for key, unit in (("tflops", "TFLOP/s"), ("gbytes_per_s", "GB/s"), ("examples_per_s", "examples/s")):
        if isinstance(case.get(key), (int, float)):
            return f"{case[key]:.4g} {unit}"
    return ""


def render(doc, source):
    prov = doc["provenance"]
    lines = [f"## {doc['benchmark']} ({os.path.basename(source)})", "",
             f"commit `{prov.get('git_commit')}` dirty={prov.get('git_dirty')} gpu=`{prov.get('gpu')}` cpu=`{prov.get('cpu')}` "
             f"at {prov.get('timestamp_utc')}", "",
             "| case | impl | device | dtype | mode | median ms | IQR ms | rate | correctness |", "|---|---|---|---|---|---|---|---|---|"]
    for c in doc["cases"]:
        lines.append(f"| {c['name']} | {c['implementation']} | {c['device']} | {c['dtype']} | {c['mode']} | {c['median']:.5f} | "
                     f"{c['iqr']:.5f} | {rate_of(c)} | {c['correctness']} |")
    return "\n".join(lines) + "\n"


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("paths", nargs="+")
    ap.add_argument("--output", default="")
    args = ap.parse_args(argv)
    text = "\n".join(render(results.load(p), p) for p in args.paths)
    if args.output:
        with open(args.output, "w", encoding="utf-8") as f:
            f.write(text)
    else:
        print(text)
    return text


if __name__ == "__main__":
    main()
