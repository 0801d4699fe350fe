"""Training-step benchmarks through the public API: whole steps (zero_grad, forward, loss,
backward, optimizer step) of three workloads, in float32 and under AMP, plus the cost of a
checkpoint save / load next to a step.

    python benchmarks/benchmark_training.py --workload mlp --device cpu
    python benchmarks/benchmark_training.py --workload tiny_mlp --device cpu --quick
    python benchmarks/benchmark_training.py --workload cnn --device cuda --amp bfloat16
    python benchmarks/benchmark_training.py --workload tiny_lm --device cuda --amp float16
    python benchmarks/benchmark_training.py --workload mlp --device cuda --compare-amp
    python benchmarks/benchmark_training.py --workload mlp --checkpoint-overhead

Workloads: `tiny_mlp` (32-64-10, batch 16: host overhead per step), `mlp` (784-256-128-10,
batch 64), `wide_mlp` (2048 -> 4096 x 4 -> 1024, batch 1024), `cnn` (three 3x3 convolutions,
128 images), `tiny_lm` (4-layer causal transformer, d 256, 4 heads, vocabulary 8192, 8 x 256
tokens).  AMP = parameters cast to the 16-bit dtype, FP32 masters inside
MixedPrecisionOptimizer, GradScaler (enabled for float16, initial scale 128).
(reference project: benchmarks/bench_model_training.py, bench_tiny_mlp_training.py,
bench_amp_vs_fp32.py, bench_checkpoint_overhead.py, benchmark_training.py)
"""
import argparse
import os
import sys
import tempfile

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
from benchmarks._support import cli, results, timing  # noqa: E402
from orthon_b200 import _C, models  # noqa: E402


def build_workload(name, quick):
    """Returns (model, make_batch(rng) -> (x float32 array or int64 ids, y int64 array), examples per step, loss kind)."""
    if name == "tiny_mlp":
        return models.MLP((32, 64, 10)), (lambda rng: (rng.standard_normal((16, 32)).astype(np.float32), rng.integers(0, 10, 16))), 16, "ce"
    if name == "mlp":
        return models.MLP(), (lambda rng: (rng.standard_normal((64, 784)).astype(np.float32), rng.integers(0, 10, 64))), 64, "ce"
    if name == "wide_mlp":
        sizes = (64, 128, 128, 32) if quick else (2048, 4096, 4096, 4096, 4096, 1024)
        batch = 32 if quick else 1024
        return (models.MLP(sizes), (lambda rng: (rng.standard_normal((batch, sizes[0])).astype(np.float32), rng.integers(0, sizes[-1], batch))),
                batch, "ce")
    if name == "cnn":
        batch = 8 if quick else 128
        return models.SmallCNN(), (lambda rng: (rng.standard_normal((batch, 3, 32, 32)).astype(np.float32), rng.integers(0, 10, batch))), batch, "ce"
    if name == "tiny_lm":
        from orthon_b200.models import CausalLM, CausalLMConfig  # noqa: F811
        cfg = CausalLMConfig(vocab_size=512 if quick else 8192, d_model=64 if quick else 256, n_layers=2 if quick else 4,
                             n_heads=4, d_ff=256 if quick else 1024, max_seq=64 if quick else 256)
        b, s = (2, 64) if quick else (8, 256)
        return CausalLM(cfg), (lambda rng: (rng.integers(0, cfg.vocab_size, (b, s)), rng.integers(0, cfg.vocab_size, b * s))), b * s, "lm"
    raise ValueError(name)


def make_step(model, optimizer, scaler, make_batch, device, amp_dtype, kind, seed):
    rng = np.random.default_rng(seed)
    x_np, y_np = make_batch(rng)
    if kind == "lm":
        x = _C.from_numpy(x_np.astype(np.int64)).to(device)
    else:
        x = ob.from_numpy(x_np).to(device)
        if amp_dtype:
            x = ob.cast(x, amp_dtype)
    y = _C.from_numpy(y_np.astype(np.int64)).to(device)

    def step():
        optimizer.zero_grad()
        out = model(x)
        if out.ndim == 3:
            out = out.reshape([out.shape[0] * out.shape[1], out.shape[2]])
        loss = ob.cross_entropy(out, y)
        if scaler is None:
            loss.backward()
            optimizer.step()
        else:
            scaler.scale(loss).backward()
            scaler.step(optimizer)
            scaler.update()
        return loss
    return step


def prepare(name, device, amp_dtype, quick, seed=0):
    ob.manual_seed(seed)
    model, make_batch, examples, kind = build_workload(name, quick)
    if amp_dtype:
        model.cast(amp_dtype)
    model.to(device)
    if amp_dtype:
        optimizer = ob.amp.MixedPrecisionOptimizer(model, ob.optim.Adam, lr=1e-3)
        scaler = ob.amp.GradScaler(init_scale=128.0, enabled=(amp_dtype == "float16"))
    else:
        optimizer, scaler = ob.optim.Adam(model.parameters(), lr=1e-3), None
    return model, optimizer, make_step(model, optimizer, scaler, make_batch, device, amp_dtype, kind, seed), examples


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--workload", default="mlp", choices=["tiny_mlp", "mlp", "wide_mlp", "cnn", "tiny_lm"])
    ap.add_argument("--amp", default="", choices=["", "float16", "bfloat16"])
    ap.add_argument("--compare-amp", action="store_true", help="float32 and both AMP dtypes side by side (CUDA)")
    ap.add_argument("--checkpoint-overhead", action="store_true")
    cli.add_options(ap)
    args = ap.parse_args(argv)
    config = cli.timing_config(args)
    sync = cli.sync_for(args.device)
    variants = ["", "bfloat16", "float16"] if args.compare_amp else [args.amp]
    if any(variants) and not args.device.startswith("cuda"):
        raise SystemExit("AMP needs --device cuda (16-bit compute is CUDA only)")
    cases = []
    baseline = None
    for amp_dtype in variants:
        model, optimizer, step, examples = prepare(args.workload, args.device, amp_dtype, args.quick, args.seed)
        first = float(step().item())
        stats = timing.measure(step, sync, config)
        last = float(step().item())
        per_s = examples / (stats.median / 1e3)
        if baseline is None:
            baseline = stats.median
        cases.append(results.case_result(f"train_step/{args.workload}", stats, shape=examples, implementation="orthon", device=args.device,
                                         dtype=amp_dtype or "float32", mode="amp" if amp_dtype else "fp32", examples_per_s=per_s,
                                         first_loss=first, last_loss=last, speedup_vs_first_variant=baseline / stats.median,
                                         correctness="loss-decreased" if last < first else "loss-not-decreased"))
        if args.checkpoint_overhead:
            with tempfile.TemporaryDirectory() as tmp:
                path = os.path.join(tmp, "bench.ckpt")
                save = timing.measure(lambda: ob.save_checkpoint(path, model, optimizer, {"step": 1}), sync, timing.TimingConfig.quick())
                size = os.path.getsize(path)
                load = timing.measure(lambda: ob.load_checkpoint(path, model, optimizer), sync, timing.TimingConfig.quick())
            for label, st in (("checkpoint_save", save), ("checkpoint_load", load)):
                cases.append(results.case_result(f"{label}/{args.workload}", st, shape=size, implementation="orthon", device=args.device,
                                                 dtype=amp_dtype or "float32", mode=label, file_bytes=size,
                                                 steps_equivalent=st.median / stats.median))
    doc = results.document("training", cases, {"workload": args.workload, "device": args.device, "quick": args.quick, "timer": config.__dict__})
    results.emit(doc, args.output or None)
    for c in cases:
        if "examples_per_s" in c:
            print(f"    {c['name']} {c['dtype']}: {c['examples_per_s']:.1f} examples/s, loss {c['first_loss']:.4f} -> {c['last_loss']:.4f}")
        if "file_bytes" in c:
            print(f"    {c['name']}: {c['file_bytes']} bytes, {c['steps_equivalent']:.2f} training steps")
    return doc


if __name__ == "__main__":
    main()
