"""Self-attention modules over [B, T, E] inputs.

Heads are never materialised by transposed copies: the projections are viewed as
[B, H, T, D] through strides and handed to the attention operator, whose GEMMs read them in
place through rank-4 tensor maps.
(reference project: python/orthon/nn/attention.py:13-106)"""
from ..functional import scaled_dot_product_attention
from .linear import Linear
from .module import Module


class SelfAttention(Module):
    def __init__(self, embed_dim, dropout=0.0):
        super().__init__()
        self.embed_dim = int(embed_dim)
        if self.embed_dim <= 0:
            raise ValueError("embed_dim must be positive")
        self.dropout = float(dropout)
        self.q_proj = Linear(self.embed_dim, self.embed_dim)
        self.k_proj = Linear(self.embed_dim, self.embed_dim)
        self.v_proj = Linear(self.embed_dim, self.embed_dim)
        self.out_proj = Linear(self.embed_dim, self.embed_dim)

    def forward(self, x, mask=None, is_causal=False):
        if x.ndim != 3:
            raise ValueError("SelfAttention expects input with shape [B, T, E]")
        if int(x.shape[-1]) != self.embed_dim:
            raise ValueError("SelfAttention input embedding dimension mismatch")
        y = scaled_dot_product_attention(self.q_proj(x), self.k_proj(x), self.v_proj(x), mask=mask,
                                         dropout_p=self.dropout, training=self.training, is_causal=is_causal)
        return self.out_proj(y)


class MultiHeadSelfAttention(Module):
    def __init__(self, embed_dim, num_heads, dropout=0.0):
        super().__init__()
        if embed_dim <= 0:
            raise ValueError("embed_dim must be positive")
        if num_heads <= 0:
            raise ValueError("num_heads must be positive")
        if embed_dim % num_heads != 0:
            raise ValueError("embed_dim must be divisible by num_heads")
        self.embed_dim, self.num_heads = int(embed_dim), int(num_heads)
        self.head_dim = self.embed_dim // self.num_heads
        self.dropout = float(dropout)
        self.q_proj = Linear(embed_dim, embed_dim)
        self.k_proj = Linear(embed_dim, embed_dim)
        self.v_proj = Linear(embed_dim, embed_dim)
        self.out_proj = Linear(embed_dim, embed_dim)

    def forward(self, x, mask=None, is_causal=False):
        if len(x.shape) != 3:
            raise ValueError("MultiHeadSelfAttention expects input shape [B, T, E]")
        B, T, E = x.shape
        if E != self.embed_dim:
            raise ValueError(f"expected embed_dim={self.embed_dim}, got {E}")
        split = [B, T, self.num_heads, self.head_dim]
        q = self.q_proj(x).reshape(split).transpose(1, 2)
        k = self.k_proj(x).reshape(split).transpose(1, 2)
        v = self.v_proj(x).reshape(split).transpose(1, 2)
        y = scaled_dot_product_attention(q, k, v, mask=mask, dropout_p=self.dropout, training=self.training,
                                         is_causal=is_causal)
        y = y.transpose(1, 2).contiguous().reshape([B, T, E])
        return self.out_proj(y)
