"""Reference arm of bench.py: drives the UNMODIFIED reference package installed under
baseline/_ref through its own public API (filled in by reference_lm.py)."""
import json


def run(args):
    try:
        from baseline.reference_lm import run_reference_lm
    except Exception as exc:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"reference harness failed to import: {exc}"}))
        return
    run_reference_lm(args)
