"""Square matmul sweep (M = N = K) for the tcgen05 GEMM, with a relative-error check against
a float32 torch reference on the smaller sizes.

    python benchmarks/bench_matmul.py --dtype bfloat16 --sizes 512 1024 2048 4096 8192
"""
import argparse
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks._support.timing import time_cuda  # noqa: E402
from orthon_b200 import _C  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--sizes", type=int, nargs="+", default=[512, 1024, 2048, 4096, 8192])
    ap.add_argument("--layouts", nargs="+", default=["nn", "nt", "tn"])
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--torch", action="store_true", help="also time torch.matmul (cuBLAS) on the same shapes")
    args = ap.parse_args()
    rng = np.random.default_rng(0)
    rows = []
    for n in args.sizes:
        a_np = rng.standard_normal((n, n)).astype(np.float32)
        b_np = rng.standard_normal((n, n)).astype(np.float32)
        a = _C.from_numpy(a_np, args.dtype).to("cuda:0")
        b = _C.from_numpy(b_np, args.dtype).to("cuda:0")
        for layout in args.layouts:
            ta, tb = layout[0] == "t", layout[1] == "t"
            stats = time_cuda(lambda: _C._gemm(a, ta, b, tb))
            row = {"n": n, "dtype": args.dtype, "layout": layout, **stats,
                   "tflops": 2.0 * n ** 3 / (stats["median_ms"] * 1e-3) / 1e12}
            if args.check and n <= 2048:
                import torch
                ta_ = torch.tensor(a.numpy().astype(np.float32)).cuda()
                tb_ = torch.tensor(b.numpy().astype(np.float32)).cuda()
                ref = (ta_.t() if ta else ta_).double() @ (tb_.t() if tb else tb_).double()
                out = torch.tensor(_C._gemm(a, ta, b, tb).numpy().astype(np.float32)).cuda().double()
                row["rel_err"] = float((out - ref).norm() / ref.norm())
            if args.torch:
                import torch
                dt = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[args.dtype]
                x = torch.randn(n, n, device="cuda", dtype=dt); y = torch.randn(n, n, device="cuda", dtype=dt)
                for _ in range(5):
                    x @ y
                torch.cuda.synchronize()
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                ts = []
                for _ in range(20):
                    _C._flush_l2(0); _C.cuda_synchronize()
                    ev[0].record(); x @ y; ev[1].record(); torch.cuda.synchronize()
                    ts.append(ev[0].elapsed_time(ev[1]))
                ts.sort()
                row["cublas_tflops"] = 2.0 * n ** 3 / (ts[len(ts) // 2] * 1e-3) / 1e12
            rows.append(row)
            print(json.dumps(row), flush=True)
    return rows


if __name__ == "__main__":
    main()
