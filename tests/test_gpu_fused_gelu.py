"""GELU fused into the quantizer (fp4t_quantize_*_gelu): codes and scales equal the quantizer
applied to torch's own bf16 GELU output, bit for bit; the fused layer call gives the same
output and gradients as GELU followed by the layer; the model option gives the same logits."""
import pytest
import torch
import torch.nn.functional as F

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from backend import ops as _ops
    return _ops


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("rows,cols", [(128, 128), (256, 768), (96, 160), (32, 32), (1024, 3072), (160, 1056)])
def test_fused_gelu_quantizer_equals_quantizer_of_torch_gelu(ops, fmt, rows, cols):
    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=g) * 2.0).to(torch.bfloat16).cuda()
    x[0, :8] = torch.tensor([0.0, -0.0, 1e-3, -1e-3, 8.0, -8.0, 30.0, -30.0], dtype=torch.bfloat16)
    codes, sf, codes_t, sf_t = ops.quantize_gelu(fmt, x, True, True)
    y = F.gelu(x)                                            # torch's bf16 GELU on the GPU
    quant = ops.quantize_nvfp4 if fmt == "nvfp4" else ops.quantize_mxfp8
    c2, s2, ct2, st2 = quant(y, True, True)
    assert torch.equal(codes, c2) and torch.equal(sf, s2), "row-wise operand differs from quantize(gelu(x))"
    assert torch.equal(codes_t, ct2) and torch.equal(sf_t, st2), "transposed operand differs"
    want = (orc.nvfp4_quantize if fmt == "nvfp4" else orc.mxfp8_quantize)(y.cpu(), want_t=True)
    assert torch.equal(codes.cpu(), want["codes"]) and torch.equal(sf_t.cpu(), want["sf_t"])
    ops.check_status()


@pytest.mark.parametrize("cls_name", ["CublasltNvfp4Linear", "CublasltMxfp8Linear"])
def test_fused_layer_equals_gelu_then_layer(cls_name, monkeypatch):
    import custom
    monkeypatch.setenv("FP4T_PARITY", "1")                   # stochastic rounding on torch.rand: same draws both ways
    cls = getattr(custom, cls_name)
    torch.manual_seed(0)
    layer = cls(768, 192).to(device="cuda", dtype=torch.bfloat16)
    pre = torch.randn(4, 64, 768, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(4, 64, 192, device="cuda", dtype=torch.bfloat16) * 1e-2
    a = pre.clone().requires_grad_(True)
    torch.manual_seed(1)
    ya = layer.forward_gelu(a)
    ya.backward(g)
    ga, gwa, gba = a.grad.clone(), layer.weight.grad.clone(), layer.bias.grad.clone()
    layer.zero_grad(set_to_none=True)
    b = pre.clone().requires_grad_(True)
    torch.manual_seed(1)
    yb = layer(F.gelu(b))
    yb.backward(g)
    assert torch.equal(ya, yb), "forward differs"
    assert torch.equal(gwa, layer.weight.grad) and torch.allclose(gba.float(), layer.bias.grad.float(), rtol=1e-2, atol=1e-4)
    assert orc.rel_frobenius(ga.float().cpu(), b.grad.float().cpu()) <= 1e-2      # same dH; gelu_backward in bf16 both ways
    from backend import ops
    ops.check_status()


def test_model_option_gives_the_same_logits():
    from models import TinyViT
    torch.manual_seed(0)
    kw = dict(patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=2, linear_impl="cublaslt_nvfp4")
    plain = TinyViT(**kw).cuda().eval()
    fused = TinyViT(fuse_gelu=True, **kw).cuda().eval()
    fused.load_state_dict(plain.state_dict())
    x = torch.rand(64, 1, 28, 28, device="cuda")
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        a, b = plain(x), fused(x)
    assert torch.equal(a, b)
