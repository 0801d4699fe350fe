"""Native test layer: builds `build/ob_native_tests` from tests/cpp and the extension's objects
and runs it (core value types, memory pool and tokens over a fake CUDA seam, registry and
dispatcher rules, CPU operators, autograd engine)."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_native_suite_passes():
    import build

    exe = build.build_native_tests()
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    tail = out.stdout[-4000:] + out.stderr[-2000:]
    assert out.returncode == 0, tail
    m = re.search(r"native tests: (\d+) run, (\d+) failed", out.stdout)
    assert m and int(m.group(1)) >= 150 and int(m.group(2)) == 0, tail


def test_native_runner_filters_and_reports_failures():
    import build

    exe = build.build_native_tests()
    out = subprocess.run([str(exe), "layout_contiguity"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "native tests: 1 run, 0 failed" in out.stdout
