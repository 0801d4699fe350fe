"""The CPU examples run end to end (small step counts) and reach their stated outcomes."""
import importlib.util
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(f"example_{name}", os.path.join(ROOT, "examples", f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_transformer_classifier_learns(monkeypatch):
    monkeypatch.setattr(sys, "argv", ["x", "--steps", "40"])
    assert _load("tiny_transformer_classifier").main() < 0.5


def test_text_classifier_and_checkpoint():
    assert _load("tiny_text_classifier").main() > 0.8


def test_nn_api_demo_runs():
    _load("nn_api_demo").main()
