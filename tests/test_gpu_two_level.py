"""Two-level NVFP4 (per-tensor scale in front of the block quantization, alpha in the GEMM
epilogue) and the 16-block random Hadamard transform: bit-exact against the CPU restatement,
the identities the options must keep, and the accuracy they exist for."""
import pytest
import torch

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu

SIGNS = 0xA5C3


@pytest.fixture(scope="module")
def ops():
    from backend import ops as _ops
    return _ops


def _same(got, want):
    codes, sf, codes_t, sf_t = got
    assert torch.equal(codes.cpu(), want["codes"]), "row-wise codes"
    assert torch.equal(sf.cpu(), want["sf"]), "row-wise scales"
    if codes_t is not None:
        assert torch.equal(codes_t.cpu(), want["codes_t"]), "transposed codes"
        assert torch.equal(sf_t.cpu(), want["sf_t"]), "transposed scales"


def _input(rows, cols, dtype, mag=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + rows * 7 + cols)
    x = torch.randn(rows, cols, generator=g) * mag
    x[0, :4] = torch.tensor([0.0, -0.0, mag * 1e-3, -mag * 5.0])
    if rows > 40 and cols > 40:
        x[33, 16:32] = 0.0                      # an all-zero block
    return x.to(dtype)


@pytest.mark.parametrize("scale", [2.0 ** 10, 2.0 ** -3, 1.0, 2.0 ** 20])
@pytest.mark.parametrize("rows,cols", [(128, 128), (256, 768), (96, 160), (1024, 1024), (32, 48)])
def test_power_of_two_scale_on_tiled_kernel_bit_exact(ops, scale, rows, cols):
    mag = 1.0 / scale
    x = _input(rows, cols, torch.bfloat16, mag).cuda()
    got = ops.quantize_nvfp4_scaled(x, scale, True, True)
    _same(got, orc.nvfp4_quantize_scaled(x.cpu(), scale, want_t=True))
    # a power-of-two scale on bf16 data is an exact multiplication: same codes and scales as
    # quantizing the pre-multiplied tensor with the one-level entry point
    y = (x.float() * scale).to(torch.bfloat16)
    c1, s1, ct1, st1 = ops.quantize_nvfp4(y, True, True)
    assert torch.equal(got[0], c1) and torch.equal(got[1], s1) and torch.equal(got[2], ct1) and torch.equal(got[3], st1)
    ops.check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("scale", [3.7, 1000.0, 0.3])
def test_general_scale_bit_exact(ops, dtype, scale):
    x = _input(256, 320, dtype, 1.0 / scale).cuda()
    _same(ops.quantize_nvfp4_scaled(x, scale, True, True), orc.nvfp4_quantize_scaled(x.cpu(), scale, want_t=True))
    ops.check_status()


def test_scale_one_is_the_one_level_quantizer(ops):
    x = _input(512, 512, torch.bfloat16).cuda()
    a = ops.quantize_nvfp4_scaled(x, 1.0, True, True)
    b = ops.quantize_nvfp4(x, True, True)
    assert all(torch.equal(p, q) for p, q in zip(a, b))


def test_scaled_stochastic_rounding_matches_unscaled_draws(ops):
    """In-kernel stochastic rounding draws by element position: x * 2^k with scale 2^-k... the
    scaled call on x and the one-level call on x * t see the same values and the same draws."""
    x = _input(256, 256, torch.bfloat16, 2.0 ** -12).cuda()
    t = 2.0 ** 12
    a = ops.quantize_nvfp4_scaled(x, t, True, True, sr=ops.SR_HASH, seed=77)
    b = ops.quantize_nvfp4((x.float() * t).to(torch.bfloat16), True, True, sr=ops.SR_HASH, seed=77)
    assert all(torch.equal(p, q) for p, q in zip(a, b))


def test_bad_scale_is_an_error(ops):
    x = _input(64, 64, torch.bfloat16).cuda()
    for bad in (0.0, -2.0, float("inf"), float("nan")):
        with pytest.raises(ValueError):
            ops.quantize_nvfp4_scaled(x, bad)


def test_tiny_gradients_need_the_second_level(ops):
    """Blocks with amax below 6 * 2^-9 sit under the smallest UE4M3 block scale: one-level
    NVFP4 quantizes them on a grid that is too coarse (or to zero).  Lifted by a tensor scale
    and brought back by alpha, the product is as accurate as for well-ranged data."""
    n, k, m = 256, 512, 384
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(n, k, generator=g) * 2.0 ** -14).to(torch.bfloat16).cuda()
    b = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    ref = a.float() @ b.float().t()
    bc, bsf, _, _ = ops.quantize_nvfp4(b)
    ac, asf, _, _ = ops.quantize_nvfp4(a)
    one = ops.gemm_nvfp4(ac, asf, bc, bsf, None, torch.float32)
    t = 2.0 ** 14
    ac2, asf2, _, _ = ops.quantize_nvfp4_scaled(a, t)
    two = ops.gemm_nvfp4(ac2, asf2, bc, bsf, None, torch.float32, alpha=1.0 / t)
    e1 = orc.rel_frobenius(one.cpu(), ref.cpu())
    e2 = orc.rel_frobenius(two.cpu(), ref.cpu())
    assert e1 > 0.5, f"one-level error {e1}: the test data is not below the block-scale range"
    assert e2 < 0.15, f"two-level error {e2}"
    ops.check_status()


@pytest.mark.parametrize("rows,cols,k", [(256, 384, 512), (64, 96, 4096), (1024, 1024, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_alpha_in_the_gemm_epilogue(ops, rows, cols, k, out_dtype):
    g = torch.Generator().manual_seed(rows + k)
    a = torch.randn(rows, k, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(cols, k, generator=g).to(torch.bfloat16).cuda()
    bias = torch.randn(cols, generator=g).to(torch.bfloat16).cuda()
    ac, asf, _, _ = ops.quantize_nvfp4(a)
    bc, bsf, _, _ = ops.quantize_nvfp4(b)
    plain = ops.gemm_nvfp4(ac, asf, bc, bsf, None, torch.float32, split_k=False)
    # a power-of-two alpha scales the fp32 accumulator exactly; the bias is added after it
    got = ops.gemm_nvfp4(ac, asf, bc, bsf, bias, out_dtype, split_k=False, alpha=0.25)
    want = (plain * 0.25 + bias.float()).to(out_dtype)
    assert torch.equal(got, want)
    # any alpha, and the split-K form where it applies: within rounding of the fp32 product
    got = ops.gemm_nvfp4(ac, asf, bc, bsf, bias, torch.float32, alpha=0.3)
    assert orc.rel_frobenius(got.cpu(), (plain * 0.3 + bias.float()).cpu()) <= 1e-5
    ops.check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(128, 128), (256, 320), (96, 160)])
def test_hadamard_quantizer_bit_exact(ops, dtype, rows, cols):
    x = _input(rows, cols, dtype).cuda()
    got = ops.quantize_nvfp4_scaled(x, 1.0, True, True, rht_signs=SIGNS)
    _same(got, orc.nvfp4_quantize_scaled(x.cpu(), 1.0, want_t=True, rht_signs=SIGNS))
    got = ops.quantize_nvfp4_scaled(x, 8.0, True, False, rht_signs=0x0001)
    _same(got, orc.nvfp4_quantize_scaled(x.cpu(), 8.0, rht_signs=0x0001))
    ops.check_status()


def test_hadamard_keeps_the_product(ops):
    """Both operands transformed with the same signs along K: the GEMM still approximates the
    untransformed product, with an error of the same order as the untransformed operands give.
    (A 16-point transform inside 16-element scale blocks does not lower the Frobenius error --
    on one 40-sigma outlier per block it is 0.15 against 0.12 -- its use is to decorrelate the
    rounding error from the data, as recipes that transform the wgrad operands do.)"""
    n, k, m = 256, 1024, 256
    g = torch.Generator().manual_seed(11)
    a = torch.randn(n, k, generator=g)
    a[:, ::16] *= 40.0                              # one outlier in every 16-block
    a = a.to(torch.bfloat16).cuda()
    b = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    ref = a.float() @ b.float().t()
    ac, asf, _, _ = ops.quantize_nvfp4(a)
    bc, bsf, _, _ = ops.quantize_nvfp4(b)
    plain = ops.gemm_nvfp4(ac, asf, bc, bsf, None, torch.float32)
    ah, ahsf, _, _ = ops.quantize_nvfp4_scaled(a, 1.0, rht_signs=SIGNS)
    bh, bhsf, _, _ = ops.quantize_nvfp4_scaled(b, 1.0, rht_signs=SIGNS)
    rht = ops.gemm_nvfp4(ah, ahsf, bh, bhsf, None, torch.float32)
    e_plain = orc.rel_frobenius(plain.cpu(), ref.cpu())
    e_rht = orc.rel_frobenius(rht.cpu(), ref.cpu())
    assert e_rht < 0.2 and e_plain < 0.2, f"product error: transformed {e_rht}, plain {e_plain}"
    # the GEMM itself is exact on the codes: compare with the dequantized operands
    wa = orc.nvfp4_quantize_scaled(a.cpu(), 1.0, rht_signs=SIGNS)
    wb = orc.nvfp4_quantize_scaled(b.cpu(), 1.0, rht_signs=SIGNS)
    da = orc.nvfp4_dequant(orc.unpack_fp4_pairs(wa["codes"]), wa["sf_logical"])
    db = orc.nvfp4_dequant(orc.unpack_fp4_pairs(wb["codes"]), wb["sf_logical"])
    assert orc.rel_frobenius(rht.cpu(), da @ db.t()) <= 1e-5
    ops.check_status()


def test_layer_with_gradient_tensor_scale():
    """CublasltNvfp4Linear(grad_tensor_scale=t): same forward; for gradients far below the
    block-scale range the input and weight gradients stay accurate where the one-level layer
    loses them."""
    import custom
    from backend import ops
    torch.manual_seed(0)
    base = custom.CublasltNvfp4Linear(512, 256).to(device="cuda", dtype=torch.bfloat16)
    lifted = custom.CublasltNvfp4Linear(512, 256, grad_tensor_scale=2.0 ** 14).to(device="cuda", dtype=torch.bfloat16)
    lifted.load_state_dict(base.state_dict())
    x = torch.randn(128, 512, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16) * 2.0 ** -15
    want_dx = g.float() @ base.weight.float()
    want_dw = g.float().t() @ x.float()
    errs = {}
    for name, layer in (("one", base), ("two", lifted)):
        xi = x.clone().requires_grad_(True)
        y = layer(xi)
        y.backward(g)
        errs[name] = (orc.rel_frobenius(xi.grad.float().cpu(), want_dx.cpu()),
                      orc.rel_frobenius(layer.weight.grad.float().cpu(), want_dw.cpu()),
                      y.detach().clone())
        assert torch.allclose(layer.bias.grad.float(), g.float().sum(0), rtol=2e-2, atol=1e-7)
    assert torch.equal(errs["one"][2], errs["two"][2]), "the option must not change the forward pass"
    assert errs["two"][0] < 0.2 and errs["two"][1] < 0.2, errs["two"][:2]
    assert errs["one"][0] > 2 * errs["two"][0] and errs["one"][1] > 2 * errs["two"][1], (errs["one"][:2], errs["two"][:2])
    ops.check_status()
