"""Fused tcgen05 attention (packed qkv) against a plain PyTorch float32 reference."""
import numpy as np
import pytest
import torch

from orthon_b200 import _C

pytestmark = pytest.mark.gpu


def _reference(qkv, heads, causal, scale):
    B, T, E3 = qkv.shape
    E = E3 // 3
    D = E // heads
    q, k, v = (qkv[:, :, i * E:(i + 1) * E].reshape(B, T, heads, D).transpose(1, 2) for i in range(3))
    s = (q @ k.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), float("-inf"))
    out = torch.softmax(s, dim=-1) @ v
    return out.transpose(1, 2).reshape(B, T, E)


CASES = [
    # B, T, H, D, causal, dtype
    (2, 256, 2, 128, True, "bfloat16"),
    (1, 512, 2, 128, False, "bfloat16"),
    (2, 200, 3, 64, True, "bfloat16"),      # sequence not a multiple of any tile
    (1, 130, 2, 64, False, "float16"),
    (1, 1024, 2, 128, True, "float16"),
    (1, 64, 1, 128, True, "bfloat16"),      # shorter than one tile
]


@pytest.mark.parametrize("B,T,H,D,causal,dtype", CASES)
def test_flash_attention_forward_backward(B, T, H, D, causal, dtype):
    rng = np.random.default_rng(B * 1000 + T + H + D)
    E = H * D
    qkv_np = rng.standard_normal((B, T, 3 * E)).astype(np.float32)
    do_np = rng.standard_normal((B, T, E)).astype(np.float32)
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float16
    qkv_ref = torch.tensor(qkv_np).to(tdt).float().requires_grad_(True)
    do_ref = torch.tensor(do_np).to(tdt).float()
    scale = D ** -0.5
    ref = _reference(qkv_ref, H, causal, scale)
    ref.backward(do_ref)

    qkv = _C.from_numpy(qkv_np, dtype).to("cuda:0")
    qkv.requires_grad_(True)
    assert _C._attention_qkv_fused(qkv, H)
    out = _C._attention_qkv(qkv, H, None, causal, scale)
    assert out._grad_fn_name == "FlashAttentionNode"
    got = torch.tensor(out.numpy().astype(np.float32))
    tol = 2e-2 if dtype == "bfloat16" else 4e-3
    assert (got - ref.detach()).abs().max().item() <= tol * max(1.0, ref.abs().max().item())

    (out * _C.from_numpy(do_np, dtype).to("cuda:0")).sum().backward()
    _C.cuda_synchronize()
    g = torch.tensor(qkv.grad.numpy().astype(np.float32))
    gref = qkv_ref.grad
    gtol = 4e-2 if dtype == "bfloat16" else 8e-3
    for name, lo in (("dq", 0), ("dk", E), ("dv", 2 * E)):
        err = (g[:, :, lo:lo + E] - gref[:, :, lo:lo + E]).abs().max().item()
        bound = gtol * max(1.0, gref[:, :, lo:lo + E].abs().max().item())
        assert err <= bound, f"{name}: max err {err} > {bound}"


def test_flash_matches_composed_path_in_model_shape():
    """Same op through the composed (GEMM + softmax kernel) path: a mask tensor forces it."""
    rng = np.random.default_rng(5)
    B, T, H, D = 2, 256, 4, 64
    E = H * D
    qkv_np = rng.standard_normal((B, T, 3 * E)).astype(np.float32)
    qkv = _C.from_numpy(qkv_np, "bfloat16").to("cuda:0")
    fused = _C._attention_qkv(qkv, H, None, True, D ** -0.5)
    zero_mask = _C.from_numpy(np.zeros((T, T), dtype=np.float32), "bfloat16").to("cuda:0")
    composed = _C._attention_qkv(qkv, H, zero_mask, True, D ** -0.5)
    a = fused.numpy().astype(np.float32)
    b = composed.numpy().astype(np.float32)
    assert np.abs(a - b).max() <= 3e-2 * max(1.0, np.abs(b).max())
