"""Tiny causal language model on arithmetic progressions (token i+1 = token i + d mod V), with
greedy generation at the end.  Runs on the CPU in float32 or on a GPU in bfloat16 / float16
with explicit AMP.

    python examples/tiny_causal_lm.py [--device cuda:0 --dtype bfloat16] [--steps 200]
"""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import orthon_b200 as ob  # noqa: E402
from orthon_b200 import _C  # noqa: E402
from orthon_b200.models import CausalLM, CausalLMConfig  # noqa: E402


def make_batch(rng, batch, block, vocab):
    start = rng.integers(0, vocab, size=(batch, 1))
    step = rng.integers(1, 4, size=(batch, 1))
    seq = (start + step * np.arange(block + 1)[None, :]) % vocab
    return seq[:, :-1].astype(np.int64), seq[:, 1:].astype(np.int64)


def generate(model, prompt, n_new, device):
    ctx = list(prompt)
    with ob.no_grad():
        for _ in range(n_new):
            window = ctx[-model.cfg.max_seq:]
            ids = _C.from_numpy(np.asarray([window], dtype=np.int64))
            if device != "cpu":
                ids = ids.to(device)
            logits = model(ids)
            last = logits.slice(0, len(window) - 1, len(window))
            ctx.append(int(ob.cast(last, "float32").argmax(1).tolist()[0]))
    return ctx


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--steps", type=int, default=150)
    a = ap.parse_args()
    cfg = CausalLMConfig(vocab_size=32, d_model=64, n_layers=2, n_heads=4, d_ff=128, max_seq=16)
    ob.manual_seed(0)
    model = CausalLM(cfg)
    if a.dtype != "float32":
        model.cast(a.dtype)
    if a.device != "cpu":
        model.to(a.device)
    opt = ob.amp.MixedPrecisionOptimizer(model, ob.optim.Adam, lr=3e-3)
    scaler = ob.amp.GradScaler(init_scale=128.0, enabled=a.dtype == "float16")
    rng = np.random.default_rng(0)
    for step in range(a.steps):
        x, y = make_batch(rng, 32, cfg.max_seq, cfg.vocab_size)
        ids, tgt = _C.from_numpy(x), _C.from_numpy(y)
        if a.device != "cpu":
            ids, tgt = ids.to(a.device), tgt.to(a.device)
        opt.zero_grad()
        loss = model.loss(ids, tgt)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        if step % 25 == 0 or step == a.steps - 1:
            print(f"step {step:4d} loss {loss.item():.4f}")
    print("generated:", generate(model, [3, 5, 7], 8, a.device))


if __name__ == "__main__":
    main()
