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


def _example(name):
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(f"example_{name}", os.path.join(root, "examples", f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_examples_train_on_the_gpu_in_float32():
    """The float32 examples on CUDA: MLP on synthetic digits and both CNNs (convolutions through
    the GEMM lowering, max pooling, Adam) learn and agree with the CPU run of the same script."""
    mlp = _example("mnist_mlp")
    gpu = mlp.main(["--synthetic", "--train-limit", "512", "--test-limit", "128", "--epochs", "2", "--device", "cuda"])
    cpu = mlp.main(["--synthetic", "--train-limit", "512", "--test-limit", "128", "--epochs", "2", "--device", "cpu"])
    assert gpu["history"][-1]["test"]["accuracy"] > 0.9
    assert abs(gpu["history"][0]["train"]["loss"] - cpu["history"][0]["train"]["loss"]) < 1e-3
    cnn = _example("cifar10_cnn")
    args = ["--synthetic", "--train-limit", "64", "--test-limit", "32", "--batch-size", "16", "--epochs", "2", "--channels", "8"]
    g = cnn.main(args + ["--device", "cuda"])
    c = cnn.main(args + ["--device", "cpu"])
    assert abs(g["history"][0]["train"]["loss"] - c["history"][0]["train"]["loss"]) < 2e-3
    assert g["history"][1]["train"]["loss"] < g["history"][0]["train"]["loss"]
    vgg = cnn.main(["--synthetic", "--model", "minivgg", "--vgg-base-channels", "8", "--hidden", "32", "--train-limit", "64",
                    "--test-limit", "32", "--batch-size", "32", "--epochs", "2", "--device", "cuda"])
    assert vgg["history"][1]["train"]["loss"] < vgg["history"][0]["train"]["loss"] + 0.05


def test_float32_training_step_is_the_same_under_both_matmul_precisions():
    """`high` precision changes rounding, not results beyond float32 noise: one MLP step."""
    from orthon_b200.models import MLP

    def one_step(level):
        ob.set_float32_matmul_precision(level)
        try:
            ob.manual_seed(3)
            model = MLP((512, 1024, 256, 10))
            model.to("cuda:0")
            opt = ob.optim.SGD(model.parameters(), lr=0.05)
            rng = np.random.default_rng(0)
            x = ob.from_numpy(rng.standard_normal((512, 512)).astype(np.float32)).to("cuda:0")
            y = _C.from_numpy(rng.integers(0, 10, 512).astype(np.int64)).to("cuda:0")
            opt.zero_grad()
            loss = ob.cross_entropy(model(x), y)
            loss.backward()
            opt.step()
            return float(loss.item()), np.asarray(next(iter(model.parameters())).to("cpu").tolist())
        finally:
            ob.set_float32_matmul_precision("highest")

    loss_a, w_a = one_step("highest")
    loss_b, w_b = one_step("high")
    assert abs(loss_a - loss_b) < 1e-4 * max(1.0, abs(loss_a))
    assert np.abs(w_a - w_b).max() < 1e-5
