"""Decoder-only causal language model: token + learned position embeddings, N pre-LayerNorm
blocks (multi-head causal self-attention, GELU MLP), final LayerNorm, linear head.

Each block is six kernel families: LayerNorm, one QKV GEMM (bias in the epilogue), packed-QKV
attention (heads read in place, causal mask applied in the softmax kernel), output projection
with the residual add in the epilogue, LayerNorm, and the MLP as two GEMMs with GELU and the
second residual add in their epilogues.  Weights are N(0, init_std).
(reference project: examples/tiny_causal_lm.py:59-112)"""
import math
from dataclasses import dataclass

import numpy as np

from .. import _C, nn
from .._random import normal_array


@dataclass(frozen=True)
class CausalLMConfig:
    vocab_size: int
    d_model: int
    n_layers: int
    n_heads: int
    d_ff: int
    max_seq: int
    init_std: float = 0.02
    eps: float = 1e-5


TINY_LM = CausalLMConfig(vocab_size=8192, d_model=512, n_layers=8, n_heads=8, d_ff=2048, max_seq=512)
LM_1P3B = CausalLMConfig(vocab_size=32000, d_model=2048, n_layers=24, n_heads=16, d_ff=8192, max_seq=1024)


def _normal(shape, std):
    return nn.Parameter(_C.from_numpy(normal_array(tuple(shape), std)))


class Block(nn.Module):
    def __init__(self, cfg: CausalLMConfig):
        super().__init__()
        E, F = cfg.d_model, cfg.d_ff
        self.n_heads = cfg.n_heads
        self.scale = 1.0 / math.sqrt(E // cfg.n_heads)
        self.ln1 = nn.LayerNorm(E, eps=cfg.eps)
        self.qkv_weight, self.qkv_bias = _normal((E, 3 * E), cfg.init_std), nn.Parameter(_C.zeros([3 * E]))
        self.proj_weight, self.proj_bias = _normal((E, E), cfg.init_std), nn.Parameter(_C.zeros([E]))
        self.ln2 = nn.LayerNorm(E, eps=cfg.eps)
        self.fc1_weight, self.fc1_bias = _normal((E, F), cfg.init_std), nn.Parameter(_C.zeros([F]))
        self.fc2_weight, self.fc2_bias = _normal((F, E), cfg.init_std), nn.Parameter(_C.zeros([E]))

    def forward(self, x):
        h = self.ln1(x)
        qkv = _C.linear(h, self.qkv_weight, self.qkv_bias)
        a = _C._attention_qkv(qkv, self.n_heads, None, True, self.scale)
        x = _C.linear(a, self.proj_weight, self.proj_bias, "none", x)
        h = self.ln2(x)
        return _C._mlp_gelu(h, self.fc1_weight, self.fc1_bias, self.fc2_weight, self.fc2_bias, x)


class CausalLM(nn.Module):
    def __init__(self, cfg: CausalLMConfig):
        super().__init__()
        self.cfg = cfg
        self.tok_emb = _normal((cfg.vocab_size, cfg.d_model), cfg.init_std)
        self.pos_emb = _normal((cfg.max_seq, cfg.d_model), cfg.init_std)
        self.blocks = nn.Sequential(*[Block(cfg) for _ in range(cfg.n_layers)])
        self.ln_f = nn.LayerNorm(cfg.d_model, eps=cfg.eps)
        self.head_weight = _normal((cfg.d_model, cfg.vocab_size), cfg.init_std)
        self.register_buffer("positions", _C.from_numpy(np.arange(cfg.max_seq, dtype=np.int64)), persistent=False)

    def forward(self, ids):
        """ids: int tensor [B, T] -> logits [B*T, vocab]."""
        B, T = ids.shape
        if T > self.cfg.max_seq:
            raise ValueError(f"sequence length {T} exceeds max_seq {self.cfg.max_seq}")
        pos = self.positions if T == self.cfg.max_seq else self.positions.slice(0, 0, T).contiguous()
        x = _C.embedding(ids, self.tok_emb) + _C.embedding(pos, self.pos_emb)
        x = self.blocks(x)
        x = self.ln_f(x)
        return _C.linear(x.reshape([B * T, self.cfg.d_model]), self.head_weight)

    def loss(self, ids, targets):
        """Mean next-token cross-entropy; `targets` is an int tensor [B, T] (or [B*T])."""
        logits = self.forward(ids)
        flat = targets if targets.ndim == 1 else targets.reshape([-1])
        return _C.cross_entropy(logits, flat)

    def parameter_count(self):
        return sum(int(p.numel) for p in self.parameters())
