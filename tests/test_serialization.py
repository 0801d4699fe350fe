"""ml-runtime-checkpoint v1: determinism, bit exactness, validation, atomicity, transactions.
(reference project: tests/spec/serialization/*, tests/python/test_checkpoint_format.py)"""
import json
import pickle
import zipfile

import numpy as np
import pytest

import orthon_b200 as ob
from orthon_b200 import _C, nn


def model():
    ob.manual_seed(5)
    return nn.Sequential(nn.Linear(3, 4), nn.ReLU(), nn.Linear(4, 2))


def test_roundtrip_and_byte_identical(tmp_path):
    m = model()
    opt = ob.optim.Adam(m.parameters(), lr=0.01)
    ob.cross_entropy(m(ob.ones([2, 3])), [0, 1]).backward()
    opt.step()
    p1, p2 = tmp_path / "a.ckpt", tmp_path / "b.ckpt"
    meta = {"epoch": 3, "lr": float("inf"), "tags": ("x", [1, 2.5, None, True])}
    ob.save_checkpoint(p1, m, opt, meta)
    ob.save_checkpoint(p2, m, opt, meta)
    assert p1.read_bytes() == p2.read_bytes()
    m2 = model()
    for p in m2.parameters():
        with ob.no_grad():
            p.fill_(0.0)
    opt2 = ob.optim.Adam(m2.parameters(), lr=1.0)
    got = ob.load_checkpoint(p1, m2, opt2)
    assert got == meta
    assert [p.tolist() for p in m2.parameters()] == [p.tolist() for p in m.parameters()]
    assert opt2._t == 1 and opt2.get_lr() == 0.01
    assert opt2.state_dict()["m"][0].tolist() == opt.state_dict()["m"][0].tolist()
    with zipfile.ZipFile(p1) as zf:
        names = zf.namelist()
        assert names[0] == "manifest.json" and names[1] == "tensors/000000.bin"
        assert zf.getinfo("tensors/000000.bin").compress_type == zipfile.ZIP_STORED
        manifest = json.loads(zf.read("manifest.json"))
        assert manifest["format"] == "ml-runtime-checkpoint" and manifest["format_version"] == 1


def test_bit_exact_payloads_including_nan_payload(tmp_path):
    raw = np.array([0x7F800001, 0x80000000, 0x7FC00000, 0x3F800000], dtype=np.uint32).view(np.float32)

    class Holder:
        def __init__(self, t):
            self.t = t

        def state_dict(self):
            return {"w": self.t}

        def load_state_dict(self, state, map_location=None):
            self.t = state["w"]

    h = Holder(ob.from_numpy(raw))
    ob.save_checkpoint(tmp_path / "n.ckpt", h)
    h2 = Holder(None)
    ob.load_checkpoint(tmp_path / "n.ckpt", h2)
    assert _C._tensor_to_bytes(h2.t) == raw.tobytes()


def test_rejects_pickle_garbage_and_tampering(tmp_path):
    p = tmp_path / "x.ckpt"
    p.write_bytes(pickle.dumps({"version": 1}))
    with pytest.raises(RuntimeError, match="^checkpoint: .*pickle"):
        ob.load_checkpoint(p)
    p.write_bytes(b"hello")
    with pytest.raises(RuntimeError, match="^checkpoint: "):
        ob.load_checkpoint(p)
    m = model()
    ob.save_checkpoint(p, m)
    data = bytearray(p.read_bytes())
    # flip one payload byte: stored payloads sit uncompressed in the file
    with zipfile.ZipFile(p) as zf:
        info = zf.getinfo("tensors/000000.bin")
        off = info.header_offset + 30 + len(info.filename)
    data[off + 3] ^= 0xFF
    p.write_bytes(bytes(data))
    before = [q.tolist() for q in m.parameters()]
    with pytest.raises(Exception):
        ob.load_checkpoint(p, m)
    assert [q.tolist() for q in m.parameters()] == before


def test_manifest_validation(tmp_path):
    def write(manifest_text, extra=()):
        p = tmp_path / "m.ckpt"
        with zipfile.ZipFile(p, "w") as zf:
            zf.writestr("manifest.json", manifest_text)
            for name, data in extra:
                zf.writestr(name, data)
        return p

    good = {"format": "ml-runtime-checkpoint", "format_version": 1,
            "sections": {"model": None, "optimizer": None, "metadata": {"k": "dict", "v": []}}}
    assert ob.load_checkpoint(write(json.dumps(good))) == {}
    for text, pat in [
        (json.dumps(dict(good, format_version=2)), "format_version"),
        (json.dumps(dict(good, format="other")), "format"),
        ('{"format":"ml-runtime-checkpoint","format":"x","format_version":1,"sections":{}}', "duplicate"),
        (json.dumps(good).replace("[]", "[NaN]"), "literal"),
    ]:
        with pytest.raises(RuntimeError, match="^checkpoint: "):
            ob.load_checkpoint(write(text))
    with pytest.raises(TypeError, match="unsupported value type"):
        ob.save_checkpoint(tmp_path / "bad.ckpt", metadata={"x": object()})
    assert not (tmp_path / "bad.ckpt").exists() and not list(tmp_path.glob("*.tmp"))


def test_failed_optimizer_prepare_leaves_model_untouched(tmp_path):
    m = model()
    opt = ob.optim.Adam(m.parameters())
    ob.save_checkpoint(tmp_path / "c.ckpt", m, opt)
    other = nn.Sequential(nn.Linear(3, 4), nn.ReLU(), nn.Linear(4, 2))
    before = [q.tolist() for q in other.parameters()]
    wrong_opt = ob.optim.Adam(list(other.parameters())[:2])  # parameter count mismatch
    with pytest.raises(ValueError, match="count mismatch"):
        ob.load_checkpoint(tmp_path / "c.ckpt", other, wrong_opt)
    assert [q.tolist() for q in other.parameters()] == before


def test_training_resume_equality(tmp_path):
    def run(steps, resume_at=None):
        m = model()
        opt = ob.optim.Adam(m.parameters(), lr=0.05)
        rng = np.random.default_rng(9)
        out = []
        for s in range(steps):
            x = ob.from_numpy(rng.standard_normal((4, 3)).astype(np.float32))
            y = list(rng.integers(0, 2, 4))
            if resume_at is not None and s == resume_at:
                ob.save_checkpoint(tmp_path / "r.ckpt", m, opt, {"s": s})
                m, opt = model(), None
                opt = ob.optim.Adam(m.parameters(), lr=123.0)
                ob.load_checkpoint(tmp_path / "r.ckpt", m, opt)
            opt.zero_grad()
            loss = ob.cross_entropy(m(x), y)
            loss.backward()
            opt.step()
            out.append(loss.item())
        return out

    assert np.allclose(run(6), run(6, resume_at=3), atol=1e-6)
