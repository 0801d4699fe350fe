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


def test_mnist_mlp_on_synthetic_digits(tmp_path):
    out = tmp_path / "mnist.json"
    result = _load("mnist_mlp").main(["--synthetic", "--train-limit", "512", "--test-limit", "128", "--epochs", "2",
                                      "--output", str(out)])
    assert result["data"] == "synthetic" and result["history"][-1]["test"]["accuracy"] > 0.9
    assert out.exists()


def test_mnist_idx_reader_round_trip(tmp_path):
    import gzip
    import struct

    import numpy as np

    images = np.arange(2 * 28 * 28, dtype=np.uint8).reshape(2, 28, 28)
    path = tmp_path / "train-images-idx3-ubyte.gz"
    with gzip.open(path, "wb") as f:
        f.write(struct.pack(">IIII", 0x00000803, 2, 28, 28) + images.tobytes())
    assert (_load("mnist_mlp").read_idx(str(path)) == images).all()


def test_cifar_cnn_both_models_step_and_schedule(tmp_path):
    mod = _load("cifar10_cnn")
    small = mod.main(["--synthetic", "--train-limit", "32", "--test-limit", "16", "--batch-size", "8", "--epochs", "2",
                      "--lr-schedule", "step", "--lr-step-epochs", "2", "--augment"])
    assert [h["lr"] for h in small["history"]] == [0.001, 0.0001]
    assert small["history"][1]["train"]["loss"] < small["history"][0]["train"]["loss"] + 0.5
    vgg = mod.main(["--synthetic", "--model", "minivgg", "--vgg-base-channels", "4", "--hidden", "16", "--train-limit", "16",
                    "--test-limit", "8", "--batch-size", "8", "--lr-schedule", "cosine", "--epochs", "2"])
    assert vgg["history"][-1]["lr"] == 0.0 and vgg["model"] == "minivgg"


def test_cifar_binary_reader(tmp_path):
    import numpy as np

    root = tmp_path / "cifar-10-batches-bin"
    root.mkdir()
    rng = np.random.default_rng(0)
    for name in [f"data_batch_{i}.bin" for i in range(1, 6)] + ["test_batch.bin"]:
        rec = rng.integers(0, 256, size=(3, 3073), dtype=np.uint8)
        rec[:, 0] = [1, 5, 9]
        rec.tofile(root / name)
    tx, ty, vx, vy = _load("cifar10_cnn").load_cifar(str(tmp_path))
    assert tx.shape == (15, 3, 32, 32) and vx.shape == (3, 3, 32, 32) and ty[:3].tolist() == [1, 5, 9] and vy.tolist() == [1, 5, 9]


def test_ddp_local_demo_matches_full_batch(monkeypatch):
    # The workers are started by name, so the module must be importable under its own name.
    monkeypatch.syspath_prepend(os.path.join(ROOT, "examples"))
    monkeypatch.setenv("PYTHONPATH", os.path.join(ROOT, "examples") + os.pathsep + os.environ.get("PYTHONPATH", ""))
    import ddp_local_demo

    assert ddp_local_demo.main() <= 1e-6


def test_synthetic_checkpoint_resume(tmp_path):
    assert _load("synthetic_mlp_checkpoint").main(["--resume-smoke", "--checkpoint", str(tmp_path / "s.ckpt")]) <= 1e-5
    assert not (tmp_path / "s.ckpt").exists()
