"""LayerNorm kernels (fp4t_layernorm_forward / _backward) against torch's fp32 / fp64 layer_norm:
values within fp32 rounding, the bf16 output equal to the rounded fp32 result, gradients against
autograd in float64, reproducible parameter gradients, and the module as an nn.LayerNorm drop-in."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

SHAPES = [(25600, 192), (1000, 64), (777, 1024), (33, 4), (128, 768), (4096, 260), (1, 512)]


@pytest.fixture(scope="module")
def ops():
    from backend import ops as _ops
    return _ops


def _inputs(rows, cols, seed=0):
    g = torch.Generator().manual_seed(seed + rows + cols)
    x = (torch.randn(rows, cols, generator=g) * 1.7 + 0.3 * torch.randn(rows, 1, generator=g)).cuda()
    gamma = (1.0 + 0.2 * torch.randn(cols, generator=g)).cuda()
    beta = (0.1 * torch.randn(cols, generator=g)).cuda()
    dy = torch.randn(rows, cols, generator=g).cuda()
    return x, gamma, beta, dy


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_forward_matches_torch(ops, rows, cols):
    x, gamma, beta, _ = _inputs(rows, cols)
    want = F.layer_norm(x.double(), (cols,), gamma.double(), beta.double(), 1e-5)
    y, mean, rstd = ops.layernorm_forward(x, gamma, beta, 1e-5, torch.float32)
    assert y.dtype == torch.float32 and y.shape == x.shape
    assert torch.allclose(y.double(), want, rtol=2e-6, atol=4e-6)               # fp32 rounding of a few operations
    assert torch.allclose(mean.double(), x.double().mean(1), rtol=1e-6, atol=1e-6)
    var = x.double().var(1, unbiased=False)
    assert torch.allclose(rstd.double(), (var + 1e-5).rsqrt(), rtol=3e-6)
    # bf16 output = the fp32 result rounded once: never more than one bf16 step from the exact value's rounding
    yb, _, _ = ops.layernorm_forward(x, gamma, beta, 1e-5, torch.bfloat16)
    assert yb.dtype == torch.bfloat16
    assert torch.equal(yb, y.to(torch.bfloat16))
    # bf16 input
    xb = x.to(torch.bfloat16)
    y2, _, _ = ops.layernorm_forward(xb, gamma, beta, 1e-5, torch.float32)
    want2 = F.layer_norm(xb.double(), (cols,), gamma.double(), beta.double(), 1e-5)
    assert torch.allclose(y2.double(), want2, rtol=2e-6, atol=4e-6)


@pytest.mark.parametrize("dy_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", SHAPES)
def test_backward_matches_autograd_in_float64(ops, rows, cols, dy_dtype):
    x, gamma, beta, dy = _inputs(rows, cols, seed=5)
    dy = dy.to(dy_dtype)
    xd = x.double().requires_grad_(True)
    gd = gamma.double().requires_grad_(True)
    bd = beta.double().requires_grad_(True)
    F.layer_norm(xd, (cols,), gd, bd, 1e-5).backward(dy.double())
    _, mean, rstd = ops.layernorm_forward(x, gamma, beta, 1e-5, torch.float32)
    dx, dgamma, dbeta = ops.layernorm_backward(dy, x, mean, rstd, gamma)
    assert dx.dtype == x.dtype and dgamma.dtype == torch.float32

    def rel(a, b):
        return float((a.double() - b).norm() / b.norm().clamp_min(1e-30))
    assert rel(dx, xd.grad) <= 2e-6
    assert rel(dgamma, gd.grad) <= 2e-6 and rel(dbeta, bd.grad) <= 2e-6       # fp32 column sums over `rows` terms
    dx2, dgamma2, dbeta2 = ops.layernorm_backward(dy, x, mean, rstd, gamma)
    assert torch.equal(dx, dx2) and torch.equal(dgamma, dgamma2) and torch.equal(dbeta, dbeta2), "not reproducible"
    ops.check_status()


def test_shape_errors(ops):
    x, gamma, beta, _ = _inputs(16, 64)
    with pytest.raises(ValueError):
        ops.layernorm_forward(x[:, :62], gamma[:62], beta[:62], 1e-5, torch.float32)       # not a multiple of 4
    with pytest.raises(ValueError):
        ops.layernorm_forward(torch.zeros(4, 2048, device="cuda"), torch.ones(2048, device="cuda"),
                              torch.zeros(2048, device="cuda"), 1e-5, torch.float32)
    with pytest.raises(NotImplementedError):
        ops.layernorm_forward(x.cpu(), gamma.cpu(), beta.cpu(), 1e-5, torch.float32)


def test_module_is_a_layernorm_drop_in():
    from custom import FusedLayerNorm
    torch.manual_seed(0)
    ref = torch.nn.LayerNorm(192).cuda()
    with torch.no_grad():
        ref.weight.add_(0.1 * torch.randn(192, device="cuda"))
        ref.bias.add_(0.1 * torch.randn(192, device="cuda"))
    ours = FusedLayerNorm(192).cuda()
    ours.load_state_dict(ref.state_dict())
    x = torch.randn(8, 50, 192, device="cuda")
    g = torch.randn(8, 50, 192, device="cuda")
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya, yb = ref(xa), ours(xb)
    assert yb.dtype == torch.float32 and torch.allclose(ya, yb, rtol=1e-5, atol=1e-5)
    ya.backward(g)
    yb.backward(g)
    assert torch.allclose(xa.grad, xb.grad, rtol=1e-4, atol=1e-5)
    assert torch.allclose(ref.weight.grad, ours.weight.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(ref.bias.grad, ours.bias.grad, rtol=1e-4, atol=1e-4)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        yc = ours(x)
        yr = ref(x)                      # fp32 under autocast; the projection behind it would cast to bf16
    assert yc.dtype == torch.bfloat16
    assert (yc.float() - yr.to(torch.bfloat16).float()).abs().max() <= 2.0 ** -7 * yr.abs().max()


def test_model_with_fused_norm_matches_model_without():
    from models import TinyViT
    torch.manual_seed(0)
    a = TinyViT(img_size=28, patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=2,
                linear_impl="cublaslt_nvfp4").cuda().eval()
    b = TinyViT(img_size=28, patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=2,
                linear_impl="cublaslt_nvfp4", fused_norm=True).cuda().eval()
    b.load_state_dict(a.state_dict())
    x = torch.rand(64, 1, 28, 28, device="cuda")
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        la, lb = a(x), b(x)
    # same computation up to the last fp32 bit of the normalised rows before their bf16 rounding
    assert (la.float() - lb.float()).abs().max() <= 0.05 * la.float().abs().max().clamp_min(1.0)
