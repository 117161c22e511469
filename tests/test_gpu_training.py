"""Training with the CUDA kernels follows the loss curve of the reference recipe.

The reference recipe is run from the oracle: `OracleNvfp4Linear` restates
custom/linear/nvfp4.py:25-90 with the restated quantizer and fp32 matmuls on dequantized
operands.  Both models start from the same weights and consume the CUDA generator in the same
order (dropout masks in forward; per layer in backward the dgrad noise, then the wgrad noise),
so the only differences are fp32 accumulation order and bf16 rounding of GEMM outputs.
Tolerance: per-step |loss difference| <= 0.1 and mean <= 0.04 over 20 steps (losses ~2.3;
the two runs drift apart slowly as rounding differences feed back through the optimizer)."""
import os

import pytest
import torch
from torch import nn

from custom import CublasltNvfp4Linear, CustomLinear
from models import TinyViT
from oracle.fp4t_oracle import OracleNvfp4Linear

pytestmark = pytest.mark.gpu


class OracleLinear(CustomLinear):
    def forward(self, input):
        shape = input.shape
        x = input.reshape(-1, shape[-1])
        w, b = self.weight, self.bias
        if torch.is_autocast_enabled():
            x, w, b = x.to(torch.bfloat16), w.to(torch.bfloat16), (None if b is None else b.to(torch.bfloat16))
        with torch.autocast("cuda", enabled=False):
            y = OracleNvfp4Linear.apply(x, w, b)
        return y.reshape(shape[:-1] + (self.out_features,))


def _swap_linears(module, cls):
    for name, child in module.named_children():
        if isinstance(child, CublasltNvfp4Linear):
            setattr(module, name, cls.from_linear(child))
        else:
            _swap_linears(child, cls)


def _run(model, steps, seed, batch=64):
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    torch.manual_seed(seed)
    gen = torch.Generator(device="cuda").manual_seed(seed + 1)
    losses = []
    for _ in range(steps):
        x = torch.rand(batch, 1, 28, 28, device="cuda", generator=gen)
        y = torch.randint(0, 10, (batch,), device="cuda", generator=gen)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = nn.functional.cross_entropy(model(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return losses


def test_loss_curve_tracks_reference_recipe(monkeypatch):
    monkeypatch.setenv("FP4T_PARITY", "1")
    torch.manual_seed(0)
    ours = TinyViT(patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=2, linear_impl="cublaslt_nvfp4").cuda()
    ref = TinyViT(patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=2, linear_impl="cublaslt_nvfp4").cuda()
    ref.load_state_dict(ours.state_dict())
    _swap_linears(ref, OracleLinear)
    assert sum(isinstance(m, OracleLinear) for m in ref.modules()) == 12
    a = _run(ours, 20, 3)
    b = _run(ref, 20, 3)
    diffs = [abs(x - y) for x, y in zip(a, b)]
    assert all(v == v for v in a + b)
    assert max(diffs) <= 0.1, (a, b)
    assert sum(diffs) / len(diffs) <= 0.04, (a, b)
    assert abs(a[0] - b[0]) <= 5e-3          # first step: identical weights and inputs
    from backend import ops
    ops.check_status()


def test_loss_curve_full_configuration(monkeypatch):
    """The TinyViT configuration of the benchmark as specified: depth 6 (36 NVFP4 projections),
    batch 512, AdamW lr 1e-3, 200 steps, seed 0, against the reference recipe on identical seeds.
    Both curves are written as JSON lines (tinyvit_config4_losses.jsonl in the run's output
    folder at the repository root, when that can be created) and the gaps are asserted per window: the two runs differ only in
    fp32 accumulation order and bf16 rounding of GEMM outputs."""
    import json
    monkeypatch.setenv("FP4T_PARITY", "1")
    torch.manual_seed(0)
    kw = dict(patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=6, linear_impl="cublaslt_nvfp4")
    ours = TinyViT(**kw).cuda()
    ref = TinyViT(**kw).cuda()
    ref.load_state_dict(ours.state_dict())
    _swap_linears(ref, OracleLinear)
    assert sum(isinstance(m, OracleLinear) for m in ref.modules()) == 36
    a = _run(ours, 200, 0, batch=512)
    b = _run(ref, 200, 0, batch=512)
    diffs = [abs(x - y) for x, y in zip(a, b)]
    summary = {"max_gap": max(diffs), "mean_gap": sum(diffs) / len(diffs), "final_gap": diffs[-1],
               "first_gap": diffs[0], "ours_final": a[-1], "reference_recipe_final": b[-1]}
    try:
        out_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gpurun_out")
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, "tinyvit_config4_losses.jsonl"), "w") as f:
            for i, (x, y) in enumerate(zip(a, b)):
                f.write(json.dumps({"step": i, "loss": x, "reference_recipe_loss": y}) + "\n")
            f.write(json.dumps(summary) + "\n")
    except OSError:
        pass
    assert all(v == v for v in a + b)
    # Identical weights, data and noise: the first steps agree to rounding, then the two runs
    # separate the way any two rounding-perturbed runs of this recipe do (random labels, lr 1e-3:
    # the loss wanders between 2.3 and 2.7).  Tolerances by window; measured on B200: first step
    # 0.0, steps 0-9 <= 0.018, steps 10-49 <= 0.055, whole run max 0.21 / mean 0.051 / final 0.022.
    assert diffs[0] <= 5e-3, summary
    assert max(diffs[:10]) <= 0.04, (summary, diffs[:10])
    assert max(diffs[10:50]) <= 0.10, (summary, max(diffs[10:50]))
    assert summary["max_gap"] <= 0.35 and summary["mean_gap"] <= 0.09 and summary["final_gap"] <= 0.25, summary
    from backend import ops
    ops.check_status()


def test_training_script_runs_and_learns():
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "fp4-training_b200"))
    from train_tinyvit import train
    out = train("cublaslt_nvfp4", steps=12, warmup=2, batch=64, depth=2, seed=0)
    assert out["world"] == 1 and len(out["losses"]) == 14
    assert all(v == v and v < 10 for v in out["losses"])


def test_loss_curve_with_library_layernorm_tracks_reference_recipe(monkeypatch):
    """fused_norm=True (the library's LayerNorm kernels) against the reference recipe on
    nn.LayerNorm: the normalised rows differ in the last fp32 bit before their bf16 rounding, so
    the curves track each other as closely as with torch's LayerNorm on both sides."""
    monkeypatch.setenv("FP4T_PARITY", "1")
    torch.manual_seed(0)
    kw = dict(patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=2, linear_impl="cublaslt_nvfp4")
    ours = TinyViT(fused_norm=True, **kw).cuda()
    ref = TinyViT(**kw).cuda()
    ref.load_state_dict(ours.state_dict())
    _swap_linears(ref, OracleLinear)
    a = _run(ours, 20, 3)
    b = _run(ref, 20, 3)
    diffs = [abs(x - y) for x, y in zip(a, b)]
    assert all(v == v for v in a + b)
    assert max(diffs) <= 0.1, (a, b)
    assert sum(diffs) / len(diffs) <= 0.04, (a, b)
    assert abs(a[0] - b[0]) <= 5e-3
    from backend import ops
    ops.check_status()


def _run_learnable(model, steps, seed, batch=128):
    """A task with something to learn: the label is the brightest of ten fixed image regions."""
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    torch.manual_seed(seed)
    gen = torch.Generator(device="cuda").manual_seed(seed + 1)
    losses = []
    for _ in range(steps):
        x = torch.rand(batch, 1, 28, 28, device="cuda", generator=gen)
        y = torch.randint(0, 10, (batch,), device="cuda", generator=gen)
        rows = torch.arange(batch, device="cuda")
        for k in range(10):                                  # brighten region k of the images labelled k
            sel = rows[y == k]
            r0, c0 = 2 + 5 * (k // 5) * 2, 2 + 5 * (k % 5)
            x[sel, :, r0:r0 + 5, c0:c0 + 5] += 1.0
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = nn.functional.cross_entropy(model(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return losses


def test_block_options_learn_like_the_reference_module_tree():
    """fused_norm + fuse_qkv (+ sdpa) change kernels, not the recipe: on a learnable task the loss
    falls at least as fast as on the reference's module tree (in-kernel stochastic rounding, so the
    curves agree statistically, not step by step; the loss is still falling steeply at step 60, so
    the bound is one-sided)."""
    kw = dict(patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=2, linear_impl="cublaslt_nvfp4")
    torch.manual_seed(0)
    plain = TinyViT(**kw).cuda()
    state = {k: v.clone() for k, v in plain.state_dict().items()}
    curves = {"plain": _run_learnable(plain, 60, 11)}
    for name, opts in (("fused", dict(fused_norm=True, fuse_qkv=True)),
                       ("fused+sdpa", dict(fused_norm=True, fuse_qkv=True, sdpa=True))):
        m = TinyViT(**kw, **opts).cuda()
        m.load_state_dict(state)
        curves[name] = _run_learnable(m, 60, 11)
    tail = {k: sum(v[-10:]) / 10 for k, v in curves.items()}
    assert tail["plain"] < 1.2, f"the task was not learned: {tail}"          # from ln(10) = 2.30
    for name in ("fused", "fused+sdpa"):      # measured: 0.82 plain, 0.62 and 0.57 with the options
        assert tail[name] < 1.2 and tail[name] <= tail["plain"] + 0.25, tail
    from backend import ops
    ops.check_status()
