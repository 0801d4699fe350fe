"""Tracing ranges: off by default, host-timed on the CPU, NVTX ranges behind a switch."""
import importlib
import os
import subprocess
import sys

import orthon_b200.utils.tracing as tracing

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_ranges_cost_nothing_and_record_nothing_when_tracing_is_off():
    tracing.enable_tracing(False)
    with tracing.trace_range("idle"):
        pass
    assert tracing.collected_ranges() == []


def test_enabled_ranges_are_collected_in_completion_order():
    tracing.enable_tracing(True)
    try:
        with tracing.trace_range("outer"):
            with tracing.trace_range("inner"):
                pass
        names = [name for name, _ in tracing.collected_ranges()]
        assert names == ["inner", "outer"]
        assert all(ms >= 0.0 for _, ms in tracing.collected_ranges())
    finally:
        tracing.enable_tracing(False)


def test_enable_tracing_clears_earlier_ranges():
    tracing.enable_tracing(True)
    with tracing.trace_range("first"):
        pass
    tracing.enable_tracing(True)
    assert tracing.collected_ranges() == []
    tracing.enable_tracing(False)


def test_a_range_survives_an_exception_in_its_body():
    tracing.enable_tracing(True)
    try:
        try:
            with tracing.trace_range("failing"):
                raise ValueError("body failed")
        except ValueError:
            pass
        assert [name for name, _ in tracing.collected_ranges()] == ["failing"]
    finally:
        tracing.enable_tracing(False)


def test_nvtx_switch_opens_and_closes_ranges_without_a_profiler_attached():
    code = ("from orthon_b200 import _C\n"
            "from orthon_b200.utils.tracing import trace_range, collected_ranges\n"
            "with trace_range('step'):\n"
            "    with trace_range('bucket 0'):\n"
            "        pass\n"
            "assert collected_ranges() == []\n"      # NVTX alone records no events
            "assert _C._nvtx_pop() < 0\n"            # nothing left on the thread's range stack
            "print('balanced')\n")
    env = dict(os.environ, ORTHON_NVTX="1", ORTHON_TRACE="0")
    out = subprocess.run([sys.executable, "-c", code], env=env, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert "balanced" in out.stdout


def test_environment_switch_turns_tracing_on_at_import():
    code = ("from orthon_b200.utils.tracing import tracing_enabled\n"
            "print(tracing_enabled())\n")
    out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, ORTHON_TRACE="1"), cwd=ROOT, capture_output=True,
                         text=True, timeout=300)
    assert out.stdout.strip() == "True"
    importlib.reload(tracing)
