"""The one writer of benchmark result documents (strict UTF-8 JSON, no NaN literals).

Document: {"schema": "orthon-b200-benchmark", "schema_version": 1, "benchmark", "mode",
"provenance", "config", "cases": [...]}; a case carries its name, shape, implementation,
device, dtype, mode, correctness status and the timer's statistics.
(reference project: benchmarks/_support/results.py:7-37)
"""
import json
import os

from .environment import provenance

SCHEMA = "orthon-b200-benchmark"
SCHEMA_VERSION = 1


def case_result(name, stats, *, shape, implementation, device, dtype="float32", mode="forward", correctness="not-compared",
                notes="", **extra):
    body = stats.as_dict() if hasattr(stats, "as_dict") else dict(stats)
    return {"name": name, "shape": shape, "implementation": implementation, "device": device, "dtype": dtype, "mode": mode,
            "correctness": correctness, "notes": notes, **body, **extra}


def document(benchmark, cases, config, *, mode="benchmark", environment=None):
    return {"schema": SCHEMA, "schema_version": SCHEMA_VERSION, "benchmark": benchmark, "mode": mode,
            "provenance": provenance() if environment is None else environment, "config": config, "cases": cases}


def write_json(path, payload):
    text = json.dumps(payload, indent=2, allow_nan=False, ensure_ascii=False) + "\n"
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w", encoding="utf-8") as f:
        f.write(text)


def load(path):
    with open(path, encoding="utf-8") as f:
        payload = json.load(f)
    if payload.get("schema") != SCHEMA or payload.get("schema_version") != SCHEMA_VERSION:
        raise ValueError(f"{path}: not a {SCHEMA} v{SCHEMA_VERSION} document")
    return payload


def emit(payload, path=None):
    print(f"{payload['benchmark']} mode={payload['mode']}")
    for c in payload["cases"]:
        extra = "".join(f" {k}={c[k]:.4g}" for k in ("gbytes_per_s", "tflops", "ratio_vs_torch") if isinstance(c.get(k), (int, float)))
        print(f"  {c['name']:<34} {c['implementation']:<8} {c['device']:<5} {c['dtype']:<9} median={c['median']:.5f} "
              f"iqr={c['iqr']:.5f} {c['units']} correctness={c['correctness']}{extra}")
    if path:
        write_json(path, payload)
