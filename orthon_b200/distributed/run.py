"""Single-node launcher:  python -m orthon_b200.distributed.run --nproc_per_node N [--backend B] script.py args...

Starts one process per rank with RANK / WORLD_SIZE / LOCAL_RANK / LOCAL_WORLD_SIZE,
ORTHON_DISTRIBUTED_BACKEND and a fresh ORTHON_STORE_DIR, polls the children every 50 ms and,
when one fails, terminates (then kills) the rest and returns its exit code.
(reference project: python/orthon/distributed/run.py:9-93)"""
import argparse
import os
import subprocess
import sys
import tempfile
import time


def _parse(argv):
    ap = argparse.ArgumentParser(prog="python -m orthon_b200.distributed.run")
    ap.add_argument("--nproc_per_node", "--nproc-per-node", type=int, required=True)
    ap.add_argument("--backend", default=None)
    ap.add_argument("script")
    ap.add_argument("script_args", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    if args.nproc_per_node < 1:
        ap.error("--nproc_per_node must be >= 1")
    return args


def _stop(children):
    for c in children:
        if c.poll() is None:
            c.terminate()
    deadline = time.monotonic() + 5.0
    for c in children:
        try:
            c.wait(timeout=max(0.0, deadline - time.monotonic()))
        except subprocess.TimeoutExpired:
            c.kill()
            c.wait()


def main(argv=None):
    args = _parse(sys.argv[1:] if argv is None else argv)
    n = args.nproc_per_node
    with tempfile.TemporaryDirectory(prefix="orthon-store-") as store_dir:
        children = []
        try:
            for rank in range(n):
                env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(n), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(n),
                           ORTHON_STORE_DIR=store_dir, ORTHON_NCCL_STORE_DIR=store_dir)
                if args.backend:
                    env["ORTHON_DISTRIBUTED_BACKEND"] = args.backend
                children.append(subprocess.Popen([sys.executable, args.script, *args.script_args], env=env))
            while True:
                codes = [c.poll() for c in children]
                failed = [code for code in codes if code not in (None, 0)]
                if failed:
                    _stop(children)
                    return failed[0]
                if all(code == 0 for code in codes):
                    return 0
                time.sleep(0.05)
        except KeyboardInterrupt:
            _stop(children)
            return 130
        finally:
            _stop(children)


if __name__ == "__main__":
    sys.exit(main())
