"""Reference arm: the same causal-LM training step driven through the UNMODIFIED reference
package (installed under baseline/_ref) and its own public API.

What is stock: every operator, autograd, nn.LayerNorm, nn.Linear.forward,
MixedPrecisionOptimizer, Adam, DistributedDataParallel, the NCCL backend.  What the harness has
to do itself, because the reference cannot do it otherwise:
  * parameters are created with from_numpy + Parameter (the stock module constructors fill
    weights one element at a time from Python, which is infeasible for 1.3 B parameters);
  * the embeddings stay float32 and their output is cast, attention scores are cast to float32
    around the softmax, logits are cast to float32 before log_softmax + nll_loss, because
    those reference kernels are float32-only on CUDA.
Timing is wall-clock between cuda_synchronize() calls (the reference exposes no event API).
"""
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _import_reference():
    if not os.path.isdir(os.path.join(REF, "orthon")):
        raise RuntimeError("baseline/_ref/orthon is missing (reference not installed)")
    sys.path.insert(0, REF)
    import orthon  # noqa: F401
    return orthon


def build_model(ortho, cfg, dtype, device, seed):
    nn = ortho.nn
    rng = np.random.default_rng(seed)

    def lower(t, dt):
        # float16 tensors can only be produced by the reference's CUDA cast kernel.
        if dt == "float16" and device != "cpu":
            return ortho.cast(t.to(device), dt)
        return ortho.cast(t, dt)

    def normal(shape, dt="float32"):
        arr = (rng.standard_normal(shape, dtype=np.float32) * cfg["init_std"]).astype(np.float32)
        if dt == "float32":
            return ortho.from_numpy(arr)
        return ortho.from_numpy(arr, dtype=dt) if dt == "bfloat16" else lower(ortho.from_numpy(arr), dt)

    def const(shape, value):
        t = ortho.full(shape, value)
        return t if dtype == "float32" else lower(t, dtype)

    def linear(i, o):
        lin = nn.Linear.__new__(nn.Linear)  # stock forward; weights filled in bulk
        nn.Module.__init__(lin)
        lin.weight = nn.Parameter(normal((i, o), dtype))
        lin.bias = nn.Parameter(const([o], 0.0))
        return lin

    def layer_norm():
        ln = nn.LayerNorm(cfg["d_model"])
        if dtype != "float32":
            ln.weight = nn.Parameter(const([cfg["d_model"]], 1.0))
            ln.bias = nn.Parameter(const([cfg["d_model"]], 0.0))
        return ln

    E, H, F, V, T = cfg["d_model"], cfg["n_heads"], cfg["d_ff"], cfg["vocab_size"], cfg["max_seq"]
    low = dtype != "float32"

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj, self.k_proj, self.v_proj, self.out_proj = linear(E, E), linear(E, E), linear(E, E), linear(E, E)

        def forward(self, x, mask):
            B, Tn, _ = x.shape
            flat = x.reshape([B * Tn, E])

            def heads(proj):
                y = proj(flat).reshape([B, Tn, H, E // H]).transpose(1, 2).contiguous()
                return y.reshape([B * H, Tn, E // H])

            q, k, v = heads(self.q_proj), heads(self.k_proj), heads(self.v_proj)
            scores = ortho.matmul(q, k.transpose(-2, -1))
            if low:
                scores = ortho.cast(scores, "float32")
            scores = scores * ((E // H) ** -0.5) + mask
            weights = ortho.exp(ortho.log_softmax(scores, dim=-1))
            if low:
                weights = ortho.cast(weights, dtype)
            y = ortho.matmul(weights, v).reshape([B, H, Tn, E // H]).transpose(1, 2).contiguous()
            return self.out_proj(y.reshape([B * Tn, E])).reshape([B, Tn, E])

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.ln2 = layer_norm(), layer_norm()
            self.attn = Attention()
            self.fc1, self.fc2 = linear(E, F), linear(F, E)

        def forward(self, x, mask):
            x = x + self.attn(self.ln1(x), mask)
            B, Tn, _ = x.shape
            h = self.ln2(x).reshape([B * Tn, E])
            h = self.fc2(ortho.gelu(self.fc1(h)))
            return x + h.reshape([B, Tn, E])

    class LM(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok = nn.Parameter(normal((V, E)))
            self.pos = nn.Parameter(normal((T, E)))
            for i in range(cfg["n_layers"]):
                setattr(self, f"block_{i}", Block())
            self.ln_f = layer_norm()
            self.head = linear(E, V)

        def forward(self, idx, pos, mask):
            x = ortho.embedding(idx, self.tok) + ortho.embedding(pos, self.pos)
            if low:
                x = ortho.cast(x, dtype)
            for i in range(cfg["n_layers"]):
                x = getattr(self, f"block_{i}")(x, mask)
            x = self.ln_f(x)
            B, Tn, _ = x.shape
            logits = self.head(x.reshape([B * Tn, E]))
            if low:
                logits = ortho.cast(logits, "float32")
            return ortho.log_softmax(logits, dim=-1)

    model = LM()
    if device != "cpu":
        model.to(device)
    return model


CONFIGS = {
    "1p3b": (dict(vocab_size=32000, d_model=2048, n_layers=24, n_heads=16, d_ff=8192, max_seq=1024, init_std=0.02), 8, 1024,
             "causal-transformer-1.3B (vocab 32000, d2048, L24, H16, ffn 8192)"),
    "tiny": (dict(vocab_size=8192, d_model=512, n_layers=8, n_heads=8, d_ff=2048, max_seq=512, init_std=0.02), 32, 512,
             "tiny-causal-lm (vocab 8192, d512, L8, H8, ffn 2048)"),
}


def _measure(ortho, args, model_key, amp, micro, rank, world, local):
    """W warm-up steps, K timed steps and K end-to-end steps of one configuration.  `micro` > 1
    splits each step's batch into that many equal slices whose gradients accumulate in `.grad`
    (the reference's own accumulate-until-zero_grad contract) before the single optimizer step."""
    import orthon.distributed as ddist
    from orthon.amp import GradScaler, MixedPrecisionOptimizer
    from orthon.optim import Adam

    cfg, batch, seq, name = CONFIGS[model_key]
    fp16 = amp == "fp16"
    dtype = "float16" if fp16 else "bfloat16"
    device = f"cuda:{local}"
    if batch % micro:
        raise ValueError("micro-batch count must divide the batch")
    mb = batch // micro

    # The reference pool never splits blocks, so cached blocks of one size class cannot serve
    # another; on the 1.3 B config the cache alone exhausts 180 GB.  Its own runtime toggle caps
    # the cache so that the configuration fits.
    cap_gb = os.environ.get("ORTHON_REF_POOL_CAP_GB", "16" if model_key == "1p3b" else "")
    if cap_gb:
        ortho._C._memory_pool_set_max_cached_bytes(int(float(cap_gb) * (1 << 30)))

    model = build_model(ortho, cfg, dtype, device, seed=1234)
    wrapped = model
    if world > 1:
        wrapped = ddist.DistributedDataParallel(model, sync_grads=False)
    opt = MixedPrecisionOptimizer(wrapped, Adam, lr=3e-4)
    scaler = GradScaler(init_scale=128.0, enabled=fp16)

    rng = np.random.default_rng(100 + rank)
    mask_np = np.triu(np.full((seq, seq), -1e9, dtype=np.float32), k=1).reshape(1, seq, seq)
    mask = ortho.from_numpy(mask_np).to(device)
    pos = ortho.from_numpy(np.tile(np.arange(seq, dtype=np.int64), (mb, 1))).to(device)

    def make_batch():
        tok = rng.integers(0, cfg["vocab_size"], size=(batch, seq + 1), dtype=np.int64)
        out = []
        for i in range(micro):
            rows = tok[i * mb:(i + 1) * mb]
            x = ortho.from_numpy(np.ascontiguousarray(rows[:, :-1])).to(device)
            y = ortho.from_numpy(np.ascontiguousarray(rows[:, 1:]).reshape(-1)).to(device)
            out.append((x, y))
        return out

    def step(slices):
        opt.zero_grad()
        total = None
        for x, y in slices:
            log_probs = wrapped(x, pos, mask)
            loss = ortho.nll_loss(log_probs, y, reduction="mean")
            if micro > 1:
                loss = loss * (1.0 / micro)
            scaler.scale(loss).backward()
            total = loss if total is None else total + loss
        scaler.step(opt)
        scaler.update()
        return total

    def sync():
        ortho.cuda_synchronize()
        if world > 1:
            ddist.barrier()

    slices = make_batch()
    for _ in range(args.warmup):
        step(slices)
    sync()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(slices)
    sync()
    device_s = time.perf_counter() - t0

    t0 = time.perf_counter()
    last = None
    for _ in range(args.steps):
        slices = make_batch()                 # host -> device copy of this step's inputs
        last = float(step(slices).item())     # device -> host read of the loss
    sync()
    e2e_s = time.perf_counter() - t0

    if world > 1:
        rows = np.zeros((world, 2), dtype=np.float32)  # max over ranks via a sum of one-hot rows
        rows[rank] = [device_s, e2e_s]
        t = ortho.from_numpy(rows).to(device)
        ddist.all_reduce(t)
        vals = np.asarray(t.to("cpu").tolist()).reshape(world, 2)
        device_s, e2e_s = float(vals[:, 0].max()), float(vals[:, 1].max())
    tokens = batch * seq * world * args.steps
    config = {"model": name, "global_batch": batch * world, "seq_len": seq, "parallelism": f"dp{world}",
              "optimizer": "FP32-master Adam (reference MixedPrecisionOptimizer, " + ("GradScaler init 128)" if fp16 else "scaler disabled)"),
              "timing": "wall clock between cuda_synchronize() calls (no event API in the reference)"}
    if micro > 1:
        config["micro_batches"] = micro
        config["note"] = (f"the full batch does not fit in device memory with the reference's kernels; each step runs {micro} "
                          f"slices of {mb} sequences whose gradients accumulate before the one optimizer step")
    return {"value": tokens / device_s, "ms_per_step": device_s / args.steps * 1e3,
            "dtype": "fp16" if fp16 else "bf16", "config": config,
            "e2e": {"value": tokens / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * batch * seq * 8,
                    "d2h_bytes_per_step": 4, "last_loss": last}}


def _worker_main(argv):
    """One attempt in a process of its own (a fresh reference pool and CUDA context): prints one
    JSON line, {"ok": result} or {"oom": note} or {"error": text}."""
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--amp", required=True)
    ap.add_argument("--micro", type=int, required=True)
    ap.add_argument("--steps", type=int, required=True)
    ap.add_argument("--warmup", type=int, required=True)
    a = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    try:
        ortho = _import_reference()
        if not ortho.cuda_enabled():
            print(json.dumps({"error": "reference build has no CUDA support"}), flush=True)
            return
        import orthon.distributed as ddist
        if world > 1:
            store = f"/tmp/orthon_ref_store_{os.environ.get('MASTER_PORT', '0')}_{os.environ.get('ORTHON_REF_ATTEMPT', '0')}"
            os.makedirs(store, exist_ok=True)
            os.environ["ORTHON_NCCL_STORE_DIR"] = store
            ddist.init_process_group("nccl", rank=rank, world_size=world, device=local)
        try:
            out = {"ok": _measure(ortho, a, a.model, a.amp, a.micro, rank, world, local)}
        except RuntimeError as exc:
            if "out of memory" not in str(exc):
                raise
            stats = ortho._C._memory_pool_stats() if hasattr(ortho._C, "_memory_pool_stats") else {}
            out = {"oom": f"{a.micro} slice(s) per step: out of device memory (pool peak {stats.get('peak_bytes')} bytes)"}
        print(json.dumps(out), flush=True)
        if world > 1 and "ok" in out:
            ddist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001
        print(json.dumps({"error": f"{type(exc).__name__}: {exc}"[:300]}), flush=True)


def _attempt(args, model_key, amp, micro, tag):
    import subprocess
    env = dict(os.environ, ORTHON_REF_ATTEMPT=f"{tag}_{model_key}_{micro}_{os.environ.get('TORCHELASTIC_RUN_ID', '')}")
    cmd = [sys.executable, os.path.abspath(__file__), "--worker", "--model", model_key, "--amp", amp, "--micro", str(micro),
           "--steps", str(args.steps), "--warmup", str(args.warmup)]
    try:
        res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=float(os.environ.get("ORTHON_REF_ATTEMPT_TIMEOUT", 1500)))
    except subprocess.TimeoutExpired:
        return {"error": f"attempt with {micro} slice(s) per step did not finish in time"}
    for line in reversed(res.stdout.strip().splitlines()):
        try:
            doc = json.loads(line)
        except ValueError:
            continue
        if isinstance(doc, dict) and ({"ok", "oom", "error"} & set(doc)):
            return doc
    return {"error": f"worker exited with code {res.returncode}: {res.stderr.strip()[-300:]}"}


def _measure_with_fallback(args, model_key, amp, tag):
    """Tries the full batch first; while the reference runs out of device memory, halves the
    slice.  Every attempt runs in a fresh process.  Returns (result or None, notes)."""
    batch = CONFIGS[model_key][1]
    notes, micro = [], 1
    while micro <= batch:
        doc = _attempt(args, model_key, amp, micro, tag)
        if "ok" in doc:
            return doc["ok"], notes
        if "error" in doc:
            notes.append(doc["error"])
            return None, notes
        notes.append(doc["oom"])
        micro *= 2
    return None, notes


ANCHOR = ("tiny", "fp16")


def run_reference_lm(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not os.path.isdir(os.path.join(REF, "orthon")):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/orthon is missing (reference not installed)"}))
        return
    amp = getattr(args, "amp", "bf16")
    main, notes = _measure_with_fallback(args, args.model, amp, "main")
    if main is None:
        line = {"impl": "reference", "unavailable": "the reference cannot run this config: " + "; ".join(notes)[:600]}
    else:
        line = {"metric": "ddp_train_tokens_per_s", "value": main["value"], "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": main["dtype"],
                "data": "synthetic token ids, random-init weights", "impl": "reference", "config": main["config"],
                "e2e": main["e2e"]}
        if notes:
            line["config"]["out_of_memory"] = notes
    if getattr(args, "anchor", True) and (args.model, amp) != ANCHOR:
        a, a_notes = _measure_with_fallback(args, ANCHOR[0], ANCHOR[1], "anchor")
        line["anchor"] = {"unavailable": "; ".join(a_notes)[:600]} if a is None else {
            "config": a["config"], "dtype": a["dtype"], "value": a["value"], "unit": "tokens/s",
            "ms_per_step": a["ms_per_step"], "e2e": a["e2e"]}
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "--worker":
        _worker_main(sys.argv[2:])
