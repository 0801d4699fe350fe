"""Checkpoint archive integrity and restore transactions, one corruption per case: every
malformed archive is refused with the uniform "checkpoint: " error before any recipient is
touched; restores are staged (model, then optimizer) and rolled back in reverse order.
(reference project: tests/spec/serialization/test_whole_archive_integrity.py,
test_restore_transaction.py, test_checkpoint_validation.py, test_checkpoint_failure_atomicity.py)"""
import hashlib
import io
import json
import os
import zipfile

import numpy as np
import pytest

import orthon_b200 as ob
from orthon_b200 import nn
from orthon_b200._serialization.format import FORMAT_ID


def small_model(seed=3):
    ob.manual_seed(seed)
    return nn.Sequential(nn.Linear(2, 3), nn.ReLU(), nn.Linear(3, 2))


def values(model):
    return [p.tolist() for p in model.parameters()]


PAYLOAD = np.arange(4, dtype=np.float32).tobytes()
TENSOR = {"k": "tensor", "shape": [4], "dtype": "float32", "nbytes": 16, "sha256": hashlib.sha256(PAYLOAD).hexdigest(),
          "payload": "tensors/000000.bin"}


def manifest(model=None, optimizer=None, metadata=None, **top):
    doc = {"format": FORMAT_ID, "format_version": 1,
           "sections": {"model": model, "optimizer": optimizer, "metadata": metadata or {"k": "dict", "v": []}}}
    doc.update(top)
    return doc


def write(path, manifest_obj, members=(), manifest_bytes=None, compression=zipfile.ZIP_STORED, manifest_name="manifest.json"):
    with zipfile.ZipFile(path, "w") as zf:
        data = manifest_bytes if manifest_bytes is not None else json.dumps(manifest_obj).encode()
        zf.writestr(manifest_name, data)
        for name, blob in members:
            zf.writestr(zipfile.ZipInfo(name), blob, compress_type=compression)
    return path


def model_section(tensor=None):
    return {"k": "dict", "v": [["w", dict(TENSOR if tensor is None else tensor)]]}


# -------------------------------------------------------------- whole archive
def test_a_minimal_handwritten_archive_loads(tmp_path):
    p = write(tmp_path / "ok.ckpt", manifest(model=model_section()), [("tensors/000000.bin", PAYLOAD)])

    class Sink:
        def load_state_dict(self, state, map_location=None):
            self.state = state

        def state_dict(self):
            return {}

    sink = Sink()
    assert ob.load_checkpoint(p, sink) == {}
    assert sink.state["w"].tolist() == [0.0, 1.0, 2.0, 3.0]


@pytest.mark.parametrize("name,blob", [
    ("empty file", b""), ("text", b"not an archive"), ("pickle protocol 2", b"\x80\x02}q\x00."), ("pickle protocol 5", b"\x80\x05\x95"),
    ("truncated zip", b"PK\x03\x04" + b"\x00" * 10), ("gzip", b"\x1f\x8b\x08\x00"),
])
def test_files_that_are_not_archives_are_refused_by_their_header(tmp_path, name, blob):
    p = tmp_path / "x.ckpt"
    p.write_bytes(blob)
    with pytest.raises(RuntimeError, match="^checkpoint: "):
        ob.load_checkpoint(p)


def test_missing_file_and_bad_path_types(tmp_path):
    with pytest.raises((FileNotFoundError, OSError)):
        ob.load_checkpoint(tmp_path / "absent.ckpt")
    with pytest.raises(TypeError):
        ob.load_checkpoint(123)
    with pytest.raises(TypeError):
        ob.save_checkpoint(None, small_model())


MANIFEST_FAULTS = [
    ("no manifest", dict(manifest_name="other.json"), "manifest.json is missing"),
    ("not utf-8", dict(manifest_bytes=b"\xff\xfe{}"), "not UTF-8"),
    ("not json", dict(manifest_bytes=b"{format:"), "not valid JSON"),
    ("json array", dict(manifest_bytes=b"[]"), "unknown container format"),
    ("wrong format id", dict(top=dict(format="another-format")), "unknown container format"),
    ("version 2", dict(top=dict(format_version=2)), "format_version"),
    ("version as text", dict(top=dict(format_version="1")), "format_version"),
    ("version as bool", dict(top=dict(format_version=True)), "format_version"),
    ("version as float", dict(top=dict(format_version=1.0)), "format_version"),
    ("sections missing", dict(top=dict(sections=None)), "sections are malformed"),
    ("extra section", dict(top=dict(sections={"model": None, "optimizer": None, "metadata": {"k": "dict", "v": []}, "x": None})), "sections are malformed"),
    ("section missing", dict(top=dict(sections={"model": None, "metadata": {"k": "dict", "v": []}})), "sections are malformed"),
    ("duplicate field", dict(manifest_bytes=b'{"format":"ml-runtime-checkpoint","format":"ml-runtime-checkpoint","format_version":1,"sections":{}}'), "duplicate JSON field"),
    ("bare NaN", dict(manifest_bytes=json.dumps(manifest()).replace('"v": []', '"v": [NaN]').encode()), "non-standard JSON literal"),
    ("bare Infinity", dict(manifest_bytes=json.dumps(manifest()).replace('"v": []', '"v": [-Infinity]').encode()), "non-standard JSON literal"),
    ("nesting too deep", dict(manifest_bytes=(b'{"format":"ml-runtime-checkpoint","format_version":1,"sections":' + b"[" * 200 + b"]" * 200 + b"}")), "too deep"),
]


@pytest.mark.parametrize("label,how,message", MANIFEST_FAULTS, ids=[f[0] for f in MANIFEST_FAULTS])
def test_manifest_faults_are_refused(tmp_path, label, how, message):
    kwargs = {k: v for k, v in how.items() if k != "top"}
    p = write(tmp_path / "m.ckpt", manifest(**how.get("top", {})), **kwargs)
    with pytest.raises(RuntimeError, match="^checkpoint: .*" + message):
        ob.load_checkpoint(p)


def test_oversized_manifest_is_refused(tmp_path):
    big = json.dumps(manifest(metadata={"k": "dict", "v": [["pad", {"k": "str", "v": "x" * (9 << 20)}]]})).encode()
    with pytest.raises(RuntimeError, match="^checkpoint: .*size limit"):
        ob.load_checkpoint(write(tmp_path / "big.ckpt", None, manifest_bytes=big))


def test_duplicate_member_names_are_refused(tmp_path):
    p = tmp_path / "dup.ckpt"
    with zipfile.ZipFile(p, "w") as zf:
        zf.writestr("manifest.json", json.dumps(manifest()))
        with pytest.warns(UserWarning):
            zf.writestr("manifest.json", json.dumps(manifest()))
    with pytest.raises(RuntimeError, match="^checkpoint: .*duplicate archive member"):
        ob.load_checkpoint(p)


TENSOR_FAULTS = [
    ("payload missing", {}, (), "is missing"),
    ("payload name outside tensors/", {"payload": "weights.bin"}, (("weights.bin", PAYLOAD),), "invalid payload name"),
    ("payload name with traversal", {"payload": "tensors/../x.bin"}, (), "invalid payload name"),
    ("payload name not a string", {"payload": 7}, (), "invalid payload name"),
    ("size differs from record", {"nbytes": 12, "shape": [3]}, (("tensors/000000.bin", PAYLOAD),), "expected 12"),
    ("byte count contradicts shape", {"nbytes": 16, "shape": [5]}, (("tensors/000000.bin", PAYLOAD),), "byte count does not match"),
    ("checksum mismatch", {"sha256": "0" * 64}, (("tensors/000000.bin", PAYLOAD),), "checksum mismatch"),
    ("checksum of the wrong length", {"sha256": "abc"}, (("tensors/000000.bin", PAYLOAD),), "malformed tensor record"),
    ("unknown dtype", {"dtype": "complex64"}, (("tensors/000000.bin", PAYLOAD),), "malformed tensor record"),
    ("negative extent", {"shape": [-4]}, (("tensors/000000.bin", PAYLOAD),), "malformed tensor record"),
    ("extent as float", {"shape": [4.0]}, (("tensors/000000.bin", PAYLOAD),), "malformed tensor record"),
    ("shape not a list", {"shape": 4}, (("tensors/000000.bin", PAYLOAD),), "malformed tensor record"),
    ("nbytes as bool", {"nbytes": True}, (("tensors/000000.bin", PAYLOAD),), "malformed tensor record"),
]


@pytest.mark.parametrize("label,patch,members,message", TENSOR_FAULTS, ids=[f[0] for f in TENSOR_FAULTS])
def test_tensor_record_faults_are_refused_before_the_model_changes(tmp_path, label, patch, members, message):
    record = dict(TENSOR)
    record.update(patch)
    p = write(tmp_path / "t.ckpt", manifest(model=model_section(record)), members)
    m = small_model()
    before = values(m)
    with pytest.raises(RuntimeError, match="^checkpoint: .*" + message):
        ob.load_checkpoint(p, m)
    assert values(m) == before


def test_compressed_payloads_are_refused(tmp_path):
    p = write(tmp_path / "c.ckpt", manifest(model=model_section()), [("tensors/000000.bin", PAYLOAD)], compression=zipfile.ZIP_DEFLATED)
    with pytest.raises(RuntimeError, match="^checkpoint: .*stored uncompressed"):
        ob.load_checkpoint(p)


def test_one_payload_cannot_back_two_tensors(tmp_path):
    section = {"k": "dict", "v": [["a", dict(TENSOR)], ["b", dict(TENSOR)]]}
    p = write(tmp_path / "two.ckpt", manifest(model=section), [("tensors/000000.bin", PAYLOAD)])
    with pytest.raises(RuntimeError, match="^checkpoint: .*more than once"):
        ob.load_checkpoint(p)


VALUE_FAULTS = [
    ("record without a kind", {"v": 1}), ("unknown kind", {"k": "set", "v": []}), ("bool holding an int", {"k": "bool", "v": 1}),
    ("int holding a bool", {"k": "int", "v": True}), ("int holding a float", {"k": "int", "v": 1.5}), ("float holding text", {"k": "float", "v": "big"}),
    ("float holding a bool", {"k": "float", "v": False}), ("str holding a number", {"k": "str", "v": 3}), ("list holding a mapping", {"k": "list", "v": {}}),
    ("dict item that is not a pair", {"k": "dict", "v": [["only-key"]]}), ("dict key that is not text", {"k": "dict", "v": [[1, {"k": "null"}]]}),
    ("dict with a repeated key", {"k": "dict", "v": [["a", {"k": "null"}], ["a", {"k": "null"}]]}), ("bare json value", 5),
]


@pytest.mark.parametrize("label,node", VALUE_FAULTS, ids=[f[0] for f in VALUE_FAULTS])
def test_value_records_outside_the_vocabulary_are_refused(tmp_path, label, node):
    p = write(tmp_path / "v.ckpt", manifest(metadata={"k": "dict", "v": [["x", node]]}))
    with pytest.raises(RuntimeError, match="^checkpoint: "):
        ob.load_checkpoint(p)


def test_metadata_and_model_sections_must_have_the_right_shape(tmp_path):
    with pytest.raises(RuntimeError, match="^checkpoint: .*metadata section is not a mapping"):
        ob.load_checkpoint(write(tmp_path / "a.ckpt", manifest(metadata={"k": "list", "v": []})))
    with pytest.raises(RuntimeError, match="^checkpoint: .*Tensor state mapping"):
        ob.load_checkpoint(write(tmp_path / "b.ckpt", manifest(model={"k": "dict", "v": [["w", {"k": "int", "v": 1}]]})))
    with pytest.raises(RuntimeError, match="^checkpoint: .*no model section"):
        ob.load_checkpoint(write(tmp_path / "c.ckpt", manifest()), small_model())
    m = small_model()
    ob.save_checkpoint(tmp_path / "d.ckpt", m)
    with pytest.raises(RuntimeError, match="^checkpoint: .*no optimizer section"):
        ob.load_checkpoint(tmp_path / "d.ckpt", m, ob.optim.SGD(m.parameters(), lr=0.1))


@pytest.mark.parametrize("value", [None, True, False, 0, -7, 2 ** 70, 1.5, -0.0, float("inf"), float("-inf"), "", "text\né", [], [1, [2, [3]]],
                                   (), (1, "a"), {}, {"k": {"nested": (1, 2)}}, [None, True, 1, 1.0, "1"]])
def test_metadata_values_round_trip_with_their_types(tmp_path, value):
    ob.save_checkpoint(tmp_path / "meta.ckpt", metadata={"value": value})
    got = ob.load_checkpoint(tmp_path / "meta.ckpt")["value"]
    assert got == value and type(got) is type(value)
    if isinstance(value, float):
        assert np.signbit(got) == np.signbit(value)


def test_nan_metadata_round_trips(tmp_path):
    ob.save_checkpoint(tmp_path / "nan.ckpt", metadata={"value": float("nan")})
    assert np.isnan(ob.load_checkpoint(tmp_path / "nan.ckpt")["value"])


@pytest.mark.parametrize("value", [object(), {1: "int key"}, {"set": {1, 2}}, b"bytes", np.float32(1.0), complex(1, 2)])
def test_values_outside_the_vocabulary_cannot_be_saved(tmp_path, value):
    target = tmp_path / "bad.ckpt"
    with pytest.raises(TypeError):
        ob.save_checkpoint(target, metadata={"value": value})
    assert not target.exists() and not [f for f in os.listdir(tmp_path) if f != "bad.ckpt"]


# ------------------------------------------------------------- file properties
def test_archives_are_deterministic_and_self_describing(tmp_path):
    m = small_model()
    ob.save_checkpoint(tmp_path / "a.ckpt", m, metadata={"b": 1, "a": 2})
    ob.save_checkpoint(tmp_path / "b.ckpt", m, metadata={"b": 1, "a": 2})
    assert (tmp_path / "a.ckpt").read_bytes() == (tmp_path / "b.ckpt").read_bytes()
    with zipfile.ZipFile(tmp_path / "a.ckpt") as zf:
        infos = zf.infolist()
        assert [i.filename for i in infos] == ["manifest.json"] + [f"tensors/{i:06d}.bin" for i in range(4)]
        assert all(i.date_time == (1980, 1, 1, 0, 0, 0) for i in infos)
        assert all(i.external_attr == 0o600 << 16 and i.create_system == 0 for i in infos)
        assert infos[0].compress_type == zipfile.ZIP_DEFLATED
        assert all(i.compress_type == zipfile.ZIP_STORED for i in infos[1:])
        text = zf.read("manifest.json").decode()
        assert ": " not in text and ", " not in text                     # compact separators
        doc = json.loads(text)
        names = [item[0] for item in doc["sections"]["model"]["v"]]
        assert names == sorted(names)                                     # sorted in the file
        assert [item[0] for item in doc["sections"]["metadata"]["v"]] == ["b", "a"]   # metadata keeps its order


def test_saving_replaces_the_target_atomically(tmp_path):
    target = tmp_path / "model.ckpt"
    target.write_bytes(b"previous contents")
    m = small_model()

    class Exploding:
        def state_dict(self):
            raise RuntimeError("state_dict failed")

    with pytest.raises(RuntimeError, match="state_dict failed"):
        ob.save_checkpoint(target, Exploding())
    assert target.read_bytes() == b"previous contents"
    ob.save_checkpoint(target, m)
    assert target.read_bytes()[:2] == b"PK"
    assert os.listdir(tmp_path) == ["model.ckpt"]                         # no temporary files left behind


def test_save_and_load_state_dict_helpers(tmp_path):
    m, other = small_model(1), small_model(2)
    ob.save_state_dict(m, tmp_path / "s.ckpt")
    ob.load_state_dict(other, tmp_path / "s.ckpt")
    assert values(other) == values(m)


def test_loading_consumes_no_random_numbers(tmp_path):
    m = small_model()
    ob.save_checkpoint(tmp_path / "r.ckpt", m)
    ob.manual_seed(11)
    first = ob._random.uniform(0.0, 1.0)
    ob.manual_seed(11)
    ob.load_checkpoint(tmp_path / "r.ckpt", m)
    ob.save_checkpoint(tmp_path / "r2.ckpt", m)
    assert ob._random.uniform(0.0, 1.0) == first


# ---------------------------------------------------------- restore transaction
class Recorder:
    """Duck-typed recipient that records what happens to it."""

    def __init__(self, log, name, fail_on_load=False):
        self.log, self.name, self.fail_on_load, self.state = log, name, fail_on_load, {"v": 0}

    def state_dict(self):
        return dict(self.state)

    def load_state_dict(self, state, map_location=None):
        self.log.append((self.name, state.get("v")))
        if self.fail_on_load and state.get("v") != 0:
            raise RuntimeError(f"{self.name} refused")
        self.state = dict(state)


def test_generic_recipients_are_restored_in_order_and_rolled_back_in_reverse(tmp_path):
    log = []
    p = write(tmp_path / "g.ckpt", manifest(model={"k": "dict", "v": []}, optimizer={"k": "dict", "v": [["v", {"k": "int", "v": 5}]]}))
    model, optimizer = Recorder(log, "model"), Recorder(log, "optimizer", fail_on_load=True)
    model.state = {}
    log.clear()
    with pytest.raises(RuntimeError, match="optimizer refused"):
        ob.load_checkpoint(p, model, optimizer)
    assert [entry[0] for entry in log] == ["model", "optimizer", "optimizer", "model"]   # commit, commit (fails), rollback x2
    assert optimizer.state == {"v": 0}


def test_optimizer_failure_rolls_the_model_back(tmp_path):
    m = small_model(1)
    opt = ob.optim.Adam(m.parameters(), lr=0.1)
    ob.cross_entropy(m(ob.ones([2, 2])), [0, 1]).backward()
    opt.step()
    ob.save_checkpoint(tmp_path / "t.ckpt", m, opt)
    target = small_model(2)
    before = values(target)

    class Refusing:
        def state_dict(self):
            return {}

        def load_state_dict(self, state, map_location=None):
            if state:
                raise RuntimeError("optimizer refused")

    with pytest.raises(RuntimeError, match="optimizer refused"):
        ob.load_checkpoint(tmp_path / "t.ckpt", target, Refusing())
    assert values(target) == before


def test_a_transaction_commits_once():
    from orthon_b200._serialization.transaction import RestoreTransaction
    tx = RestoreTransaction.prepare(None, None, None, None)
    tx.commit()
    with pytest.raises(RuntimeError, match="already committed"):
        tx.commit()


@pytest.mark.parametrize("location,error", [("cpu", None), ("cuda:x", ValueError), ("tpu", ValueError), (3, TypeError)])
def test_map_location_is_validated_before_the_archive_is_opened(tmp_path, location, error):
    m = small_model()
    ob.save_checkpoint(tmp_path / "l.ckpt", m)
    if error is None:
        ob.load_checkpoint(tmp_path / "l.ckpt", m, map_location=location)
    else:
        with pytest.raises(error):
            ob.load_checkpoint(tmp_path / "absent.ckpt", m, map_location=location)


def test_model_and_optimizer_restore_together_or_not_at_all(tmp_path):
    m = small_model(1)
    opt = ob.optim.Adam(m.parameters(), lr=0.1)
    for _ in range(2):
        opt.zero_grad()
        ob.cross_entropy(m(ob.ones([2, 2])), [0, 1]).backward()
        opt.step()
    ob.save_checkpoint(tmp_path / "both.ckpt", m, opt, {"step": 2})
    fresh = small_model(9)
    fresh_opt = ob.optim.Adam(fresh.parameters(), lr=5.0)
    assert ob.load_checkpoint(tmp_path / "both.ckpt", fresh, fresh_opt) == {"step": 2}
    assert values(fresh) == values(m) and fresh_opt._t == 2 and fresh_opt.get_lr() == 0.1
    # the restored moments belong to the restored optimizer, not to the file or the saved optimizer
    assert fresh_opt.state_dict()["m"][0]._buffer_id != opt.state_dict()["m"][0]._buffer_id
