"""Reducer sweep: fused peer-memory all-reduce (peer-load and, where available, in-switch multimem
variants; + unscale, inf check, 1/world scaling, FP32-master Adam) against NCCL all-reduce followed by a local fused Adam kernel, for gradient buckets of
4 KB .. 1 GB in float32 and bfloat16.

    python benchmarks/bench_reducer.py --gpus 2 [--max-mb 1024] [--dtypes float32 bfloat16]

Every number is device time (CUDA events on the launching stream, L2 flushed before each timed
launch, median of the samples, then the MAX over ranks).  Bus bandwidth is
2 * S * (world-1)/world / t with S the bucket size in bytes of the gradient dtype; the roofline
for a two-shot exchange is the same expression over the measured 770 GB/s NVLink peer copy rate.
"""
import argparse
import json
import os
import statistics
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_PEER_GBS = 770.0
ESZ = {"float32": 4, "bfloat16": 2, "float16": 2}


def worker(rank, dtypes, max_mb, iters):
    import orthon_b200.distributed as dist
    from orthon_b200 import _C
    from orthon_b200.distributed import group as _group
    group = _group.active()
    be = group.backend
    ws, dev_i = group.world_size, be.device
    dev = f"cuda:{dev_i}"
    max_bytes = max_mb << 20
    rows = []
    from orthon_b200.distributed.nccl_backend import NcclBackend
    nccl_be = NcclBackend(rank, ws, dev_i, be._store)
    for dtype in dtypes:
        esz = ESZ[dtype]
        n_max = max_bytes // esz
        region = be.allocate_symmetric(n_max * esz + n_max * 4 + _C._PEER_FLAG_BYTES, multicast=True)
        mc = getattr(region, "mc", None) or 0
        grads = list(region.ptrs)
        staging = [p + n_max * esz for p in region.ptrs]
        flags = [p + n_max * esz + n_max * 4 for p in region.ptrs]
        grad_t = _C._tensor_from_ptr(region.local, [n_max], dtype, dev_i)
        rng = np.random.default_rng(rank)
        chunk = _C.from_numpy((rng.standard_normal(1 << 20) * 1e-3 * 128).astype(np.float32), dtype).to(dev)
        for off in range(0, n_max, 1 << 20):
            k = min(1 << 20, n_max - off)
            grad_t._copy_flat_range_from(off, chunk, 0, k)
        master = _C._zeros_on([n_max], "float32", dev)
        m, v = _C._zeros_on([n_max], "float32", dev), _C._zeros_on([n_max], "float32", dev)
        model = None if dtype == "float32" else _C._zeros_on([n_max], dtype, dev)
        status, found = be.status_tensors()
        hyper = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, bias_c1=0.1, bias_c2=0.001)
        size = 4096
        while size <= max_bytes:
            n = size // esz
            oneshot = size <= (512 << 10)

            def timed(fn):
                for _ in range(3):
                    fn()
                _C.cuda_synchronize()
                dist.barrier()
                samples = []
                for _ in range(iters):
                    _C._flush_l2(dev_i)
                    a = _C.CudaEvent.record(dev_i)
                    fn()
                    b = _C.CudaEvent.record(dev_i)
                    samples.append(b.elapsed_ms_since(a))
                return statistics.median(samples)

            def fused(mode, mc_ptr=0):
                return lambda: _C._peer_reduce(rank, ws, dev_i, grads, staging, flags, n, dtype, be.next_epoch(),
                                               1.0 / (128.0 * ws), mode, oneshot and not mc_ptr,
                                               master=_C._view_flat(master, 0, [n]), m=_C._view_flat(m, 0, [n]),
                                               v=_C._view_flat(v, 0, [n]),
                                               model=None if model is None else _C._view_flat(model, 0, [n]),
                                               hyper=dict(hyper), status=status, found_inf=found, stream_kind=0, mc_grads=mc_ptr)

            view = _C._view_flat(grad_t, 0, [n])

            def nccl_only():
                nccl_be._group.all_reduce(view)

            def nccl_adam():
                nccl_be._group.all_reduce(view)
                _C._adam_step_(_C._view_flat(master, 0, [n]), _C._view_flat(m, 0, [n]), _C._view_flat(v, 0, [n]), view,
                               None if model is None else _C._view_flat(model, 0, [n]), 1e-3, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001,
                               1.0 / (128.0 * ws))

            t = {"fused_average": timed(fused("average")), "fused_adam": timed(fused("adam")),
                 "nccl_allreduce": timed(nccl_only), "nccl_then_adam": timed(nccl_adam),
                 "nvls_average": timed(fused("average", mc)) if mc else 0.0,
                 "nvls_adam": timed(fused("adam", mc)) if mc else 0.0}
            # max over ranks
            vec = np.zeros([ws, 6], dtype=np.float32)
            vec[rank] = [t["fused_average"], t["fused_adam"], t["nccl_allreduce"], t["nccl_then_adam"], t["nvls_average"],
                         t["nvls_adam"]]
            tt = _C.from_numpy(vec).to(dev)
            dist.all_reduce(tt)
            worst = np.asarray(tt.tolist()).reshape(ws, 6).max(axis=0)
            bus = lambda ms: 2.0 * size * (ws - 1) / ws / (ms * 1e-3) / 1e9  # noqa: E731
            rows.append({"dtype": dtype, "bytes": size, "world": ws, "oneshot": oneshot,
                         "fused_average_ms": float(worst[0]), "fused_adam_ms": float(worst[1]),
                         "nccl_allreduce_ms": float(worst[2]), "nccl_then_adam_ms": float(worst[3]),
                         "fused_average_bus_gbs": bus(worst[0]), "fused_adam_bus_gbs": bus(worst[1]),
                         "nccl_bus_gbs": bus(worst[2]),
                         "nvls_average_ms": float(worst[4]), "nvls_adam_ms": float(worst[5]),
                         "nvls_average_bus_gbs": bus(worst[4]) if worst[4] > 0 else None,
                         "fused_average_frac_of_nvlink_roofline": bus(worst[0]) / NVLINK_PEER_GBS,
                         "fused_average_frac_of_nominal_900": bus(worst[0]) / 900.0,
                         "nvls_average_frac_of_nominal_900": bus(worst[4]) / 900.0 if worst[4] > 0 else None})
            size *= 2
        be.check_status()
    nccl_be.shutdown()
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--dtypes", nargs="+", default=["float32", "bfloat16"])
    a = ap.parse_args()
    import orthon_b200.distributed as dist
    res = dist.spawn(worker, args=(a.dtypes, a.max_mb, a.iters), nprocs=a.gpus, backend="p2p")
    for row in res[0]:
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
