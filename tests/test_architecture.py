"""Source fences: what is built matches the tree, the runtime imports no foreign framework,
environment switches share one prefix, documents point at files that exist, and comments stand on
their own (no references to planning documents or to the machine that built them)."""
import ast
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE_DIRS = ("csrc", "orthon_b200", "tests", "benchmarks", "examples", "baseline")
SOURCE_FILES = ("bench.py", "build.py", "__graft_entry__.py")
SUFFIXES = (".py", ".cpp", ".cu", ".h", ".cuh")


def _sources():
    for d in SOURCE_DIRS:
        for base, dirs, files in os.walk(os.path.join(ROOT, d)):
            dirs[:] = [x for x in dirs if x not in ("_ref", "__pycache__")]
            for f in files:
                if f.endswith(SUFFIXES):
                    yield os.path.join(base, f)
    for f in SOURCE_FILES:
        yield os.path.join(ROOT, f)


def test_every_native_source_is_built():
    import build
    native = sorted(p for p in build.CSRC.rglob("*") if p.suffix in (".cpp", ".cu"))
    assert native, "no native sources"
    names = {p.name for p in native}
    for expected in ("gemm_tc05.cu", "attention_tc05.cu", "peer_reducer.cu", "vmm_multicast.cpp", "engine.cpp", "module.cpp"):
        assert expected in names
    # build.py compiles whatever it finds under csrc/, so nothing can be left out of the extension.
    assert "rglob" in open(os.path.join(ROOT, "build.py")).read()


def test_runtime_package_does_not_import_torch_or_triton():
    for path in _sources():
        rel = os.path.relpath(path, ROOT)
        if not rel.startswith("orthon_b200") or not path.endswith(".py"):
            continue
        tree = ast.parse(open(path).read())
        for node in ast.walk(tree):
            names = []
            if isinstance(node, ast.Import):
                names = [a.name for a in node.names]
            elif isinstance(node, ast.ImportFrom) and node.module and node.level == 0:
                names = [node.module]
            for n in names:
                top = n.split(".")[0]
                assert top not in ("triton", "tilelang", "jax"), f"{rel} imports {n}"
                if top == "torch":  # only the optional TCPStore rendezvous may touch torch.distributed
                    assert rel.endswith(os.path.join("distributed", "store.py")), f"{rel} imports {n}"


def test_environment_switches_share_the_prefix():
    pat = re.compile(r"""(?:getenv\(|environ\.get\(|environ\[)\s*["']([A-Z0-9_]+)["']""")
    allowed = {"RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "NCCL_DEBUG",
               "CUDA_VISIBLE_DEVICES", "CUDA_HOME", "TORCHELASTIC_RUN_ID"}
    for path in _sources():
        rel = os.path.relpath(path, ROOT)
        if rel.startswith(("tests", "baseline")):
            continue
        for name in pat.findall(open(path).read()):
            assert name.startswith("ORTHON_") or name in allowed, f"{rel}: environment variable {name}"


def test_comments_stand_on_their_own():
    banned = re.compile(r"SURVEY|DESIGN\.md|BASELINE\.md|VERDICT|ADVICE\.md|gpurun|/root/|\bround [0-9]\b|\bthe judge\b")
    for path in _sources():
        if os.path.abspath(path) == os.path.abspath(__file__):
            continue
        for i, line in enumerate(open(path, errors="replace"), 1):
            assert not banned.search(line), f"{os.path.relpath(path, ROOT)}:{i}: {line.strip()[:100]}"


def test_documents_point_at_existing_files():
    pat = re.compile(r"`((?:csrc|orthon_b200|tests|benchmarks|examples|profiles|baseline)/[A-Za-z0-9_./*-]+)`")
    for doc in ("README.md", "DESIGN.md"):
        text = open(os.path.join(ROOT, doc)).read()
        for ref in pat.findall(text):
            ref = ref.rstrip(".,")
            if "*" in ref:
                assert os.path.isdir(os.path.join(ROOT, os.path.dirname(ref))), f"{doc}: {ref}"
            else:
                assert os.path.exists(os.path.join(ROOT, ref)), f"{doc}: {ref}"
