"""End-to-end GPU checks of the flagship model path (packed attention, fused linear epilogues,
AMP optimizer) against a float32 PyTorch model with the same weights."""
import numpy as np
import pytest
import torch

import orthon_b200 as ob
from orthon_b200 import _C
from orthon_b200.models import CausalLM, CausalLMConfig

pytestmark = pytest.mark.gpu


def torch_forward(params, ids, tgt, cfg):
    F = torch.nn.functional
    B, T = ids.shape
    E, H = cfg.d_model, cfg.n_heads
    x = params["tok_emb"][ids] + params["pos_emb"][:T]
    for i in range(cfg.n_layers):
        p = lambda n: params[f"blocks.{i}.{n}"]  # noqa: E731
        h = F.layer_norm(x, (E,), p("ln1.weight"), p("ln1.bias"), cfg.eps)
        qkv = h @ p("qkv_weight") + p("qkv_bias")
        q, k, v = qkv.split(E, dim=-1)
        sp = lambda z: z.reshape(B, T, H, E // H).transpose(1, 2)  # noqa: E731
        a = F.scaled_dot_product_attention(sp(q), sp(k), sp(v), is_causal=True).transpose(1, 2).reshape(B, T, E)
        x = x + a @ p("proj_weight") + p("proj_bias")
        h = F.layer_norm(x, (E,), p("ln2.weight"), p("ln2.bias"), cfg.eps)
        h = F.gelu(h @ p("fc1_weight") + p("fc1_bias"))
        x = x + h @ p("fc2_weight") + p("fc2_bias")
    x = F.layer_norm(x, (E,), params["ln_f.weight"], params["ln_f.bias"], cfg.eps)
    logits = x.reshape(B * T, E) @ params["head_weight"]
    return F.cross_entropy(logits, tgt.reshape(-1))


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-3), ("bfloat16", 6e-2)])
def test_causal_lm_matches_torch(dtype, tol):
    cfg = CausalLMConfig(vocab_size=512, d_model=128, n_layers=2, n_heads=4, d_ff=256, max_seq=64)
    ob.manual_seed(3)
    model = CausalLM(cfg)
    ref = {k: torch.tensor(v.numpy()).double().requires_grad_(True) for k, v in model.state_dict().items()}
    model.cast(dtype).to("cuda:0")
    rng = np.random.default_rng(0)
    tok = rng.integers(0, cfg.vocab_size, size=(4, 65), dtype=np.int64)
    ids, tgt = np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:])
    loss = model.loss(_C.from_numpy(ids).to("cuda:0"), _C.from_numpy(tgt).to("cuda:0"))
    loss.backward()
    tl = torch_forward(ref, torch.tensor(ids), torch.tensor(tgt), cfg)
    tl.backward()
    assert abs(loss.item() - tl.item()) < tol * 5
    for name, p in model.named_parameters():
        g = torch.tensor(p.grad.numpy().astype(np.float32)).double()
        e = ref[name].grad
        denom = e.abs().max().item() + 1e-6
        assert (g - e).abs().max().item() / denom < tol * 4, name
    _C.cuda_synchronize()


def test_smoke_entry():
    import __graft_entry__ as entry
    entry.smoke()
