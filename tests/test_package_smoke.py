"""Runs the plain-script smoke test in a fresh interpreter."""
import os
import subprocess
import sys


def test_package_smoke_script():
    script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "smoke", "package_smoke.py")
    out = subprocess.run([sys.executable, script], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "package smoke ok" in out.stdout
