"""Drop-in behaviour of the `custom` Linear family, following the reference's
tests/test_custom_linear.py: construction, from_linear aliasing, and forward+backward
against nn.Linear.  The reference's own tolerances were deliberately loose (0.8 / 3.0 /
5.0 absolute); here the quantized layers are held to a relative-Frobenius bound instead,
plus the reference's absolute bound."""
import pytest
import torch
import torch.nn as nn

from custom import (
    AddmmLinear,
    CublasltFwdNvfp4BwdMxfp8Linear,
    CublasltLinear,
    CublasltMxfp8Linear,
    CublasltNvfp4Linear,
    CustomLinear,
    FakeMxfp8Linear,
)

LINEAR_TOLERANCES = [
    # (class, reference atol, relative Frobenius bound on outputs and grads)
    (CustomLinear, 1e-5, 1e-6),
    (AddmmLinear, 1e-5, 1e-6),
    (CublasltLinear, 1e-2, 1e-6),
    (FakeMxfp8Linear, 0.8, 1e-1),
    (CublasltMxfp8Linear, 3.0, 1e-1),
    (CublasltNvfp4Linear, 5.0, 2.5e-1),
    (CublasltFwdNvfp4BwdMxfp8Linear, 5.0, 2.5e-1),
]
LINEAR_TESTLIST = [t[0] for t in LINEAR_TOLERANCES]
dtype_label = {torch.float32: "f32", torch.bfloat16: "bf16"}


def _rel(a, b):
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


@pytest.mark.parametrize("use_bias", [True, False], ids=lambda x: f"bias-{x}")
@pytest.mark.parametrize("oc", [5, 30], ids=lambda x: f"{x}.oc")
@pytest.mark.parametrize("ic", [10, 50], ids=lambda x: f"{x}.ic")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=lambda x: dtype_label.get(x))
@pytest.mark.parametrize("constructor", LINEAR_TESTLIST)
def test_construction_cpu(ic, oc, use_bias, dtype, constructor):
    layer = constructor(ic, oc, bias=use_bias).to(dtype=dtype)
    assert layer.in_features == ic and layer.out_features == oc
    assert layer.weight.shape == (oc, ic) and layer.weight.dtype == dtype
    assert (layer.bias.shape == (oc,) and layer.bias.dtype == dtype) if use_bias else layer.bias is None
    torch_linear = nn.Linear(ic, oc, bias=use_bias).to(dtype=dtype)
    aliased = constructor.from_linear(torch_linear)
    assert aliased.weight is torch_linear.weight
    assert (aliased.bias is torch_linear.bias) if use_bias else aliased.bias is None
    assert aliased.in_features == ic and aliased.out_features == oc
    if hasattr(layer, "quantizers"):
        assert list(aliased.quantizers.keys()) == list(layer.quantizers.keys())


def test_quantizer_tables_match_reference_layout():
    """Keys and row/column choice of the per-GEMM quantizer tables
    (custom/linear/nvfp4.py:108-116, custom/linear/mxfp8.py:103-110)."""
    from custom.quantize import q_mxfp8_colwise, q_mxfp8_rowwise, q_nvfp4_rowwise
    nv = CublasltNvfp4Linear(32, 32).quantizers
    assert list(nv) == ['1A', '1B', '2A', '2B', '3A', '3B']
    assert nv['1A'] is q_nvfp4_rowwise and nv['2B'].keywords == {'sr': True} and nv['3B'].keywords == {'sr': True}
    mx = CublasltMxfp8Linear(32, 32).quantizers
    assert [mx[k] for k in mx] == [q_mxfp8_rowwise, q_mxfp8_rowwise, q_mxfp8_colwise, q_mxfp8_rowwise,
                                   q_mxfp8_colwise, q_mxfp8_colwise]
    hy = CublasltFwdNvfp4BwdMxfp8Linear(32, 32).quantizers
    assert hy['1A'] is q_nvfp4_rowwise and hy['2A'] is q_mxfp8_colwise and hy['2B'] is q_mxfp8_rowwise


def test_cpu_tensors_are_rejected():
    layer = CublasltNvfp4Linear(32, 32)
    with pytest.raises((AssertionError, NotImplementedError, ValueError)):
        layer(torch.randn(4, 32))


@pytest.mark.gpu
@pytest.mark.parametrize("use_bias", [True, False], ids=lambda x: "bias" if x else "xbias")
@pytest.mark.parametrize("oc", [32, 64, 128], ids=lambda x: f"{x}.oc")
@pytest.mark.parametrize("ic", [64, 32, 256], ids=lambda x: f"{x}.ic")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=lambda x: dtype_label.get(x))
@pytest.mark.parametrize("constructor_tol", LINEAR_TOLERANCES, ids=lambda x: x[0].__name__)
def test_fwd_bwd_cuda(ic, oc, use_bias, dtype, constructor_tol):
    constructor, atol, rtol = constructor_tol
    if dtype == torch.bfloat16:
        rtol = max(rtol, 2e-2)
        atol = max(atol, 1e-1)
    torch.manual_seed(ic * 1000 + oc)
    torch_linear = nn.Linear(ic, oc, bias=use_bias).to(device="cuda", dtype=dtype)
    custom_linear = constructor(ic, oc, bias=use_bias).to(device="cuda", dtype=dtype)
    custom_linear.load_state_dict(torch_linear.state_dict())

    B, L = 4, 16
    x = torch.randn(B, ic).to(device="cuda", dtype=dtype)          # 2-D input, forward only
    y, ref_y = custom_linear(x), torch_linear(x)
    assert y.shape == (B, oc) and y.dtype == dtype and y.is_cuda
    assert torch.allclose(y, ref_y, atol=atol)
    assert _rel(y, ref_y) <= rtol

    x = torch.randn(B, L, ic).to(device="cuda", dtype=dtype)       # 3-D input, forward + backward
    ref_x = x.clone()
    x.requires_grad = True
    ref_x.requires_grad = True
    y, ref_y = custom_linear(x), torch_linear(ref_x)
    assert y.shape == (B, L, oc) and y.dtype == dtype
    assert torch.allclose(y, ref_y, atol=atol)
    assert custom_linear.weight.data_ptr() != torch_linear.weight.data_ptr()
    gen = torch.Generator(device="cuda").manual_seed(1)
    go = (torch.randn(y.shape, device="cuda", generator=gen) * 0.1).to(dtype)
    y.backward(go)
    ref_y.backward(go)
    for got, want, name in ((custom_linear.weight.grad, torch_linear.weight.grad, "dW"), (x.grad, ref_x.grad, "dX")):
        assert got.shape == want.shape and got.dtype == want.dtype, name
        assert torch.allclose(got, want, atol=atol), name
        assert _rel(got, want) <= rtol * 1.5, f"{name}: {_rel(got, want)}"
    if use_bias:
        assert torch.allclose(custom_linear.bias.grad, torch_linear.bias.grad, atol=atol)
    from backend import ops
    ops.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("cls", [CublasltNvfp4Linear, CublasltMxfp8Linear, CublasltFwdNvfp4BwdMxfp8Linear])
def test_fused_path_equals_operator_path(cls, monkeypatch):
    """A customised quantizer table makes the layer walk the reference's call sequence
    (separate quantizer calls, bf16 transposes, the xops operators).  With identical
    noise both routes must produce the same numbers."""
    monkeypatch.setenv("FP4T_PARITY", "1")
    torch.manual_seed(0)
    a = cls(128, 64).cuda()
    b = cls(128, 64).cuda()
    b.load_state_dict(a.state_dict())
    first = next(iter(b.quantizers))
    stock = b.quantizers[first]
    b.quantizers[first] = lambda t: stock(t)          # same arithmetic, no longer the stock object
    x = torch.randn(96, 128, device="cuda")
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    go = torch.randn(96, 64, device="cuda") * 1e-3
    with torch.autocast("cuda", dtype=torch.bfloat16):
        ya = a(xa)
        yb = b(xb)
    assert torch.equal(ya, yb)
    torch.manual_seed(5)
    ya.backward(go)
    torch.manual_seed(5)
    yb.backward(go)
    assert torch.equal(xa.grad, xb.grad)
    assert torch.equal(a.weight.grad, b.weight.grad)
    assert torch.equal(a.bias.grad, b.bias.grad)


@pytest.mark.gpu
@pytest.mark.parametrize("n", [48, 16, 80])
def test_nvfp4_batch_multiple_of_16_but_not_32(n):
    """wgrad contracts over the batch, and an FP4 GEMM's K has to be a multiple of 32: a batch of
    48 cannot train the layer.  Forward runs (the reference's own tests call it with a batch of 4);
    backward raises a ValueError naming the batch before it launches anything; with frozen
    parameters the same batch runs forward and backward."""
    torch.manual_seed(n)
    ic, oc = 64, 96
    ref = nn.Linear(ic, oc).to(device="cuda", dtype=torch.bfloat16)
    layer = CublasltNvfp4Linear(ic, oc).to(device="cuda", dtype=torch.bfloat16)
    layer.load_state_dict(ref.state_dict())
    x = torch.randn(n, ic, device="cuda", dtype=torch.bfloat16)
    y = layer(x)
    assert y.shape == (n, oc) and _rel(y, ref(x)) <= 2.5e-1
    with pytest.raises(ValueError, match="multiple of 32"):
        y.backward(torch.randn_like(y))
    layer.requires_grad_(False)
    xg = x.clone().requires_grad_(True)
    xr = x.clone().requires_grad_(True)
    y, yr = layer(xg), ref(xr)
    assert y.shape == (n, oc) and _rel(y, yr) <= 2.5e-1
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    assert _rel(xg.grad, xr.grad) <= 3e-1
