"""Projections that share their input computed as one quantization + one GEMM over the stacked
weights (forward_stacked, model option fuse_qkv): forward values equal the separate layers' bit
for bit; weight gradients too where no stochastic rounding is involved (MXFP8); the input
gradient is the one-GEMM sum instead of three bf16-rounded partial sums; NVFP4 gradients differ
by their stochastic-rounding draws only."""
import pytest
import torch

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu


def _layers(cls_name, e, outs, seed=0):
    import custom
    cls = getattr(custom, cls_name)
    torch.manual_seed(seed)
    return [cls(e, o).to(device="cuda", dtype=torch.bfloat16) for o in outs]


def _run(layers, x, grads, stacked):
    xi = x.clone().requires_grad_(True)
    for m in layers:
        m.zero_grad(set_to_none=True)
    outs = type(layers[0]).forward_stacked(layers, xi) if stacked else [m(xi) for m in layers]
    torch.autograd.backward(outs, grads)
    return ([o.detach().clone() for o in outs], xi.grad.clone(), [m.weight.grad.clone() for m in layers],
            [m.bias.grad.clone() for m in layers])


@pytest.mark.parametrize("cls_name", ["CublasltMxfp8Linear", "CublasltNvfp4Linear"])
@pytest.mark.parametrize("shape", [(4, 64, 192, (192, 192, 192)), (2, 160, 256, (256, 64, 64)), (1, 96, 128, (128, 128))])
def test_stacked_equals_separate(cls_name, shape):
    from backend import ops
    b, l, e, outs = shape
    layers = _layers(cls_name, e, outs)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(b, l, e, device="cuda", dtype=torch.bfloat16, generator=g)
    grads = [torch.randn(b, l, o, device="cuda", dtype=torch.bfloat16, generator=g) * 1e-2 for o in outs]
    ya, dxa, dwa, dba = _run(layers, x, grads, stacked=False)
    yb, dxb, dwb, dbb = _run(layers, x, grads, stacked=True)
    for a, c in zip(ya, yb):
        assert torch.equal(a, c), "forward differs"
    # what the gradients should be, from the unquantized operands
    want_dx = sum(gr.float().reshape(-1, o) @ m.weight.float() for gr, o, m in zip(grads, outs, layers)).reshape(b, l, e)
    tol = 0.08 if "Mxfp8" in cls_name else 0.35      # NVFP4: stochastically rounded dY times RNE-rounded W
    assert orc.rel_frobenius(dxb.float().cpu(), want_dx.cpu()) <= tol
    assert orc.rel_frobenius(dxb.float().cpu(), want_dx.cpu()) <= 1.15 * orc.rel_frobenius(dxa.float().cpu(), want_dx.cpu()) + 1e-3
    for wa, wb, ba, bb in zip(dwa, dwb, dba, dbb):
        if "Mxfp8" in cls_name:
            assert torch.equal(wa, wb), "weight gradient differs without stochastic rounding"
        else:
            assert orc.rel_frobenius(wb.float().cpu(), wa.float().cpu()) <= 0.35      # two independent rounding draws
        assert torch.allclose(ba.float(), bb.float(), rtol=2e-2, atol=1e-4)
    ops.check_status()


def test_frozen_projection_and_missing_gradient():
    """One of the stacked layers frozen, and one output unused in the loss."""
    layers = _layers("CublasltNvfp4Linear", 192, (192, 192, 192))
    for p in layers[1].parameters():
        p.requires_grad_(False)
    x = torch.randn(128, 192, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    q, k, v = type(layers[0]).forward_stacked(layers, x)
    (q.float().sum() + k.float().sum()).backward()            # v is unused
    assert layers[1].weight.grad is None and layers[0].weight.grad is not None
    assert float(layers[2].weight.grad.abs().max()) == 0.0      # no gradient flowed into v
    assert x.grad is not None


def test_model_option_gives_the_same_logits():
    from models import TinyViT
    torch.manual_seed(0)
    kw = dict(img_size=28, patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=2, linear_impl="cublaslt_nvfp4")
    a = TinyViT(**kw).cuda().eval()
    b = TinyViT(fuse_qkv=True, **kw).cuda().eval()
    b.load_state_dict(a.state_dict())
    x = torch.rand(64, 1, 28, 28, device="cuda")
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        assert torch.equal(a(x), b(x))


def test_sdpa_option_matches_the_explicit_attention():
    """sdpa=True: same attention arithmetic through torch's fused kernel (eval mode: no dropout).
    Checked on unquantized fp32 linears, where nothing amplifies the last-bit differences of the
    two softmax implementations."""
    from models import TinyViT
    torch.manual_seed(0)
    kw = dict(img_size=28, patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=2, linear_impl="torch")
    a = TinyViT(**kw).cuda().eval()
    b = TinyViT(sdpa=True, **kw).cuda().eval()
    b.load_state_dict(a.state_dict())
    x = torch.rand(64, 1, 28, 28, device="cuda")
    with torch.no_grad():
        la, lb = a(x), b(x)
    assert torch.allclose(la, lb, rtol=1e-3, atol=1e-4)
