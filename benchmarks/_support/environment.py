"""Provenance block of a benchmark document: what ran, on what, from which source state."""
import datetime
import os
import platform
import subprocess
import sys


def _command(argv, cwd=None):
    try:
        out = subprocess.run(argv, cwd=cwd, capture_output=True, text=True, timeout=10)
    except (OSError, subprocess.SubprocessError):
        return None
    return out.stdout.strip() if out.returncode == 0 else None


def cpu_name():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return platform.processor() or platform.machine()


def provenance():
    import orthon_b200 as ob

    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dirty = _command(["git", "status", "--porcelain"], root)
    try:
        import torch
        torch_version = torch.__version__
    except ImportError:
        torch_version = None
    return {
        "timestamp_utc": datetime.datetime.now(datetime.timezone.utc).isoformat(),
        "git_commit": _command(["git", "rev-parse", "HEAD"], root),
        "git_dirty": None if dirty is None else bool(dirty),
        "package": "orthon_b200", "package_version": getattr(ob, "__version__", None), "extension_path": ob._C.__file__,
        "python": sys.version.split()[0], "platform": platform.platform(), "cpu": cpu_name(), "logical_cpu_count": os.cpu_count(),
        "cuda_enabled": bool(ob.cuda_enabled()), "nccl_enabled": bool(ob.nccl_enabled()),
        "gpu": _command(["nvidia-smi", "--query-gpu=name,driver_version", "--format=csv,noheader"]),
        "torch_version": torch_version,
    }
