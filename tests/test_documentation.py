"""The documents under docs/ are checked against the package: the API manifest lists exactly the
public names, the checkpoint format document states what the reader enforces.
(reference project: tests/python/test_documentation_architecture.py, docs/api.md:216-324)"""
import importlib
import json
import os
import re
import sys
import zipfile

import pytest

import orthon_b200 as ob

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
API = open(os.path.join(ROOT, "docs", "api.md")).read()
FORMAT = open(os.path.join(ROOT, "docs", "checkpoint_format.md")).read()
MODULES = re.findall(r"<!-- api:([\w.]+) -->", API)


def _documented(module):
    block = re.search(rf"<!-- api:{re.escape(module)} -->(.*?)<!-- /api:{re.escape(module)} -->", API, re.S).group(1)
    return sorted(re.findall(r"`([^`]+)`", block))


def _public(module):
    m = importlib.import_module(module)
    names = getattr(m, "__all__", None)
    if names is None:
        names = [n for n in dir(m) if not n.startswith("_") and not isinstance(getattr(m, n), type(sys))]
    return sorted(names)


def test_manifest_covers_every_public_module():
    assert set(MODULES) >= {"orthon_b200", "orthon_b200.nn", "orthon_b200.functional", "orthon_b200.optim", "orthon_b200.amp",
                            "orthon_b200.training", "orthon_b200.checkpoint", "orthon_b200.distributed"}


@pytest.mark.parametrize("module", MODULES)
def test_manifest_lists_exactly_the_public_names(module):
    assert _documented(module) == _public(module)


@pytest.mark.parametrize("module", MODULES)
def test_documented_names_resolve(module):
    m = importlib.import_module(module)
    for name in _documented(module):
        assert getattr(m, name) is not None or name == "grad"


def test_documented_tensor_members_exist():
    section = API.split("## Tensor methods")[1].split("## Environment switches")[0]
    members = {n.split("(")[0] for n in re.findall(r"`([a-z_]+(?:\([^`]*\))?)`", section)}
    members -= {"orthon_b200", "retain_graph", "dim", "keepdim", "other", "alpha", "start", "end"}
    t = ob.zeros([2])
    missing = [n for n in sorted(members) if not hasattr(t, n)]
    assert not missing, missing


def test_documented_switches_are_the_ones_the_sources_read():
    section = API.split("## Environment switches")[1].split("## Additions")[0]
    documented = set(re.findall(r"`(ORTHON_[A-Z0-9_]+)\*?`", section))
    used = set()
    for base in ("orthon_b200", "csrc", "benchmarks", "baseline"):
        for folder, _, files in os.walk(os.path.join(ROOT, base)):
            if "_ref" in folder:
                continue
            for f in files:
                if f.endswith((".py", ".cpp", ".cu", ".h", ".cuh")):
                    used |= set(re.findall(r"ORTHON_[A-Z0-9_]+", open(os.path.join(folder, f), errors="replace").read()))
    used = {u for u in used if not u.startswith(("ORTHON_GEMM_", "ORTHON_REF_", "ORTHON_NOALLOC_")) and not u.endswith("_")}
    documented_plain = {d for d in documented if not d.startswith("ORTHON_GEMM_")}
    assert used <= documented_plain, sorted(used - documented_plain)
    assert "ORTHON_GEMM_" in section


def test_format_document_matches_what_the_writer_produces(tmp_path):
    m = ob.nn.Linear(2, 2)
    ob.save_checkpoint(tmp_path / "c.ckpt", m, ob.optim.SGD(m.parameters(), lr=0.1), {"epoch": 1, "note": (1.5, None)})
    with zipfile.ZipFile(tmp_path / "c.ckpt") as zf:
        doc = json.loads(zf.read("manifest.json"))
        names = zf.namelist()
    assert doc["format"] in FORMAT and f'"format_version": {doc["format_version"]}' in FORMAT
    assert sorted(doc["sections"]) == ["metadata", "model", "optimizer"]
    assert all(re.fullmatch(r"tensors/[0-9]{6}\.bin", n) for n in names[1:])
    kinds = set()

    def walk(node):
        if isinstance(node, dict) and "k" in node:
            kinds.add(node["k"])
            value = node.get("v")
            if node["k"] == "dict":
                for _, child in value:
                    walk(child)
            elif node["k"] in ("list", "tuple"):
                for child in value:
                    walk(child)

    for section in doc["sections"].values():
        walk(section)
    for kind in kinds:
        assert f"`{kind}`" in FORMAT, kind
    for field in ("shape", "dtype", "nbytes", "sha256", "payload"):
        assert f"`{field}`" in FORMAT
    for dtype in ("float32", "float64", "float16", "bfloat16", "int32", "int64", "uint8", "int8", "bool"):
        assert dtype in FORMAT
    assert "`checkpoint: `" in FORMAT and "8 MiB" in FORMAT and "128 levels" in FORMAT
