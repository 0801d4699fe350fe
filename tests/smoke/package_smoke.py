"""Plain-script smoke test of the installed package: runs without pytest and with torch, triton
and pickle made unusable, so any hidden dependency on them fails loudly.

    python tests/smoke/package_smoke.py
"""
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
for forbidden in ("torch", "triton", "pytest"):
    sys.modules[forbidden] = None  # importing it now raises ImportError

import pickle  # noqa: E402


def _fatal(*_a, **_k):
    raise AssertionError("pickle entry point used")


pickle.dump = pickle.dumps = pickle.load = pickle.loads = _fatal

import numpy as np  # noqa: E402

import orthon_b200 as ob  # noqa: E402


def main():
    a = ob.from_numpy(np.arange(6, dtype=np.float32).reshape(2, 3))
    b = ob.ones([3])
    a.requires_grad_(True)
    y = ((a + b) * 2.0) @ ob.from_numpy(np.eye(3, dtype=np.float32))
    assert y.tolist() == [2.0, 4.0, 6.0, 8.0, 10.0, 12.0]
    y.sum().backward()
    assert a.grad.tolist() == [2.0] * 6
    v = a.detach().reshape([3, 2])
    v.fill_(7.0)
    assert a.tolist() == [7.0] * 6  # views share the buffer

    ob.manual_seed(0)
    model = ob.nn.Sequential(ob.nn.Linear(4, 8), ob.nn.ReLU(), ob.nn.Linear(8, 2))
    opt = ob.optim.Adam(model.parameters(), lr=1e-2)
    x = ob.from_numpy(np.random.default_rng(0).standard_normal((5, 4)).astype(np.float32))
    first = None
    for _ in range(5):
        opt.zero_grad()
        loss = ob.cross_entropy(model(x), [0, 1, 0, 1, 0])
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < first

    with tempfile.TemporaryDirectory() as d:
        p1, p2 = os.path.join(d, "a.ckpt"), os.path.join(d, "b.ckpt")
        ob.save_checkpoint(p1, model, opt, {"note": "smoke"})
        ob.save_checkpoint(p2, model, opt, {"note": "smoke"})
        raw1, raw2 = open(p1, "rb").read(), open(p2, "rb").read()
        assert raw1 == raw2 and raw1[:2] == b"PK"  # deterministic, ZIP container
        clone = ob.nn.Sequential(ob.nn.Linear(4, 8), ob.nn.ReLU(), ob.nn.Linear(8, 2))
        meta = ob.load_checkpoint(p1, clone)
        assert clone(x).tolist() == model(x).tolist()
        bad = os.path.join(d, "bad.ckpt")
        with open(bad, "wb") as f:
            f.write(b"\x80\x04not a checkpoint")
        try:
            ob.load_checkpoint(bad, clone)
        except Exception as exc:  # noqa: BLE001
            assert str(exc).startswith("checkpoint: "), str(exc)
        else:
            raise AssertionError("a pickle stream was accepted")
    print("package smoke ok", meta if isinstance(meta, dict) else "")


if __name__ == "__main__":
    main()
