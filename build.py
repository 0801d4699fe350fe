"""In-tree native build for orthon_b200.

Compiles every source under ``csrc/`` (C++17 host code with g++, CUDA code with
nvcc for sm_100a only) and links one extension module,
``orthon_b200/_C<EXT_SUFFIX>``.  Objects are cached under ``build/obj`` keyed by
a hash of the source, the headers and the flags, so a second run only rebuilds
what changed.  The CUDA runtime is linked statically: the module imports on a
machine without a GPU driver and shares the primary context with any other
CUDA user in the process.

Usage:  python build.py [-j N] [--verbose] [--ptxas-info] [--tests]
"""
from __future__ import annotations

import argparse
import concurrent.futures as futures
import hashlib
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build" / "obj"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _pybind_include() -> str:
    import pybind11

    return pybind11.get_include()


def _includes() -> list[str]:
    return [
        f"-I{CSRC / 'include'}",
        f"-I{CUDA_HOME / 'include'}",
        f"-I{_pybind_include()}",
        f"-I{sysconfig.get_paths()['include']}",
    ]


def _header_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".h", ".hpp", ".cuh"):
            h.update(p.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, flags_cxx, flags_cu, hdr: str, verbose: bool, ptxas: bool):
    is_cu = src.suffix == ".cu"
    if is_cu:
        cmd = [NVCC, *GENCODE, "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
               "-Xcompiler", "-fPIC,-fvisibility=hidden", *flags_cu]
        if ptxas:
            cmd += ["-Xptxas", "-v"]
    else:
        # The CPU backend's loops are written for the vectoriser; everything else is glue.
        opt = "-O3" if src.parent.name == "cpu" else "-O2"
        cmd = ["g++", opt, "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall",
               "-Wno-unused-function", *flags_cxx]
    key = hashlib.sha256()
    key.update(src.read_bytes())
    key.update(hdr.encode())
    key.update(" ".join(cmd).encode())
    rel = src.relative_to(CSRC).as_posix().replace("/", "__")
    obj = OBJ / f"{rel}.{key.hexdigest()[:16]}.o"
    if obj.exists():
        return obj, False, ""
    for stale in OBJ.glob(f"{rel}.*.o"):
        stale.unlink()
    full = cmd + _includes() + ["-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(full), flush=True)
    res = subprocess.run(full, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{res.stdout}\n{res.stderr}")
    return obj, True, res.stderr if ptxas else ""


def source_digest() -> str:
    """Digest of everything under csrc/ (relative path and bytes of each file, in sorted order).
    The extension carries the digest it was built from and the package compares it with the tree
    at import, so Python code can never run against an extension built from older sources."""
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.is_file() and p.suffix in (".cpp", ".cu", ".h", ".hpp", ".cuh"):
            h.update(p.relative_to(CSRC).as_posix().encode())
            h.update(b"\0")
            h.update(p.read_bytes())
    return h.hexdigest()


def _compile_stamp(digest: str) -> Path:
    """One tiny object that holds the source digest (rebuilt whenever any source changes)."""
    src = OBJ / "source_stamp.cpp"
    obj = OBJ / f"source_stamp.{digest[:16]}.o"
    if obj.exists():
        return obj
    for stale in OBJ.glob("source_stamp.*.o"):
        stale.unlink()
    src.write_text(f'extern "C" __attribute__((visibility("default"))) const char* ob_source_digest() {{ return "{digest}"; }}\n')
    res = subprocess.run(["g++", "-O1", "-fPIC", "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{res.stderr}")
    return obj


def target_path() -> Path:
    return ROOT / "orthon_b200" / f"_C{sysconfig.get_config_var('EXT_SUFFIX')}"


def build_native_tests(jobs: int | None = None, verbose: bool = False) -> Path:
    """Links `build/ob_native_tests` from the extension's objects (all but the Python module
    definition) and the sources under tests/cpp.  libpython satisfies the objects that carry
    pybind11 bindings; no interpreter is started."""
    build(jobs, verbose)
    OBJ.mkdir(parents=True, exist_ok=True)
    tests_dir = ROOT / "tests" / "cpp"
    sources = sorted(tests_dir.glob("*.cpp"))
    key = hashlib.sha256(_header_digest().encode())
    for p in sorted(tests_dir.iterdir()):
        key.update(p.read_bytes())
    objs = sorted(o for o in OBJ.glob("*.o") if not o.name.startswith("bindings__module") and not o.name.startswith("tests_cpp__"))
    key.update(" ".join(str(o) for o in objs).encode())
    out = ROOT / "build" / "ob_native_tests"
    stamp = OBJ / "native_tests.stamp"
    if out.exists() and stamp.exists() and stamp.read_text() == key.hexdigest():
        return out
    version = sysconfig.get_config_var("LDVERSION")
    cmd = [NVCC, *GENCODE, "-O1", "-std=c++17", *_includes(), f"-I{tests_dir}", "-o", str(out), *map(str, sources), *map(str, objs),
           "-cudart", "static", f"-L{sysconfig.get_config_var('LIBDIR')}", f"-lpython{version}", "-lpthread", "-ldl", "-lrt"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"native test link failed\n{res.stdout}\n{res.stderr}")
    stamp.write_text(key.hexdigest())
    print(f"[build] native tests -> {out.relative_to(ROOT)}")
    return out


def build(jobs: int | None = None, verbose: bool = False, ptxas: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    sources = sorted(p for p in CSRC.rglob("*") if p.suffix in (".cpp", ".cu"))
    if not sources:
        raise RuntimeError("no native sources found under csrc/")
    hdr = _header_digest()
    jobs = jobs or max(1, os.cpu_count() or 1)
    objs, rebuilt = [], 0
    with futures.ThreadPoolExecutor(max_workers=jobs) as pool:
        futs = [pool.submit(_compile_one, s, [], [], hdr, verbose, ptxas) for s in sources]
        for f in futs:
            obj, did, info = f.result()
            objs.append(obj)
            rebuilt += int(did)
            if info:
                print(info)
    objs.append(_compile_stamp(source_digest()))
    out = target_path()
    stamp = OBJ / "link.stamp"
    link_key = hashlib.sha256(" ".join(str(o) for o in objs).encode()).hexdigest()
    if rebuilt or not out.exists() or not stamp.exists() or stamp.read_text() != link_key:
        cmd = [NVCC, *GENCODE, "-shared", "-o", str(out), *map(str, objs),
               "-Xcompiler", "-fPIC", "-cudart", "static", "-lpthread", "-ldl", "-lrt"]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed\n{res.stdout}\n{res.stderr}")
        stamp.write_text(link_key)
    print(f"[build] {len(sources)} sources, {rebuilt} rebuilt -> {out.relative_to(ROOT)}")
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("-j", type=int, default=None)
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true")
    ap.add_argument("--tests", action="store_true", help="also link build/ob_native_tests from tests/cpp")
    a = ap.parse_args()
    try:
        build(a.j, a.verbose, a.ptxas_info)
        if a.tests:
            build_native_tests(a.j, a.verbose)
    except RuntimeError as e:
        print(e, file=sys.stderr)
        sys.exit(1)
