"""Command-line options shared by the benchmark scripts."""
from .timing import TimingConfig


def add_options(parser, *, timing=True):
    parser.add_argument("--device", default="cpu", help="cpu, cuda or cuda:N")
    parser.add_argument("--dtype", default="float32", choices=["float32", "float64", "float16", "bfloat16"])
    parser.add_argument("--output", default="", help="write the result document to this JSON file")
    parser.add_argument("--quick", action="store_true", help="tiny shapes and a short timer (smoke run)")
    parser.add_argument("--seed", type=int, default=0)
    if timing:
        parser.add_argument("--warmup", type=int, default=None)
        parser.add_argument("--samples", type=int, default=None)
        parser.add_argument("--target-ms", type=float, default=None)


def timing_config(args):
    base = TimingConfig.quick() if args.quick else TimingConfig()
    return TimingConfig(warmup=base.warmup if args.warmup is None else args.warmup,
                        samples=base.samples if args.samples is None else args.samples,
                        target_ms=base.target_ms if args.target_ms is None else args.target_ms,
                        cap_ms=max(base.cap_ms, base.target_ms if args.target_ms is None else args.target_ms))


def sync_for(device):
    """Callable that drains the device a case runs on (nothing to do for the CPU)."""
    if not device.startswith("cuda"):
        return lambda: None
    import orthon_b200 as ob
    return ob.cuda_synchronize


def torch_sync_for(device):
    if not device.startswith("cuda"):
        return lambda: None
    import torch
    return torch.cuda.synchronize
