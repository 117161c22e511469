"""Block-quantized GEMM outputs (fp4t_gemm_*_qout): the epilogue's codes and scales equal the
oracle's quantizer applied to the SAME kernel's fp32 output (the accumulators are identical:
same tiling, fixed accumulation order), bit for bit; a GEMM fed by such an output matches the
dequantized matmul; and the reference operator with Dout = uint8 returns them."""
import pytest
import torch

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from backend import ops as _ops
    return _ops


def _operands(ops, fmt, m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    b = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    quant = ops.quantize_nvfp4 if fmt == "nvfp4" else ops.quantize_mxfp8
    ac, asf, _, _ = quant(a)
    bc, bsf, _, _ = quant(b)
    return ac, asf, bc, bsf


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("out_fmt", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("m,n,k,bias", [(256, 256, 512, False), (300, 160, 256, True), (96, 64, 128, True),
                                         (1024, 768, 1024, False), (128, 8192, 256, True)])
def test_qout_equals_oracle_quantizer_of_fp32_output(ops, fmt, out_fmt, m, n, k, bias):
    ac, asf, bc, bsf = _operands(ops, fmt, m, n, k, m + n + k)
    b = (torch.randn(n, generator=torch.Generator().manual_seed(1)) * 0.5).to(torch.bfloat16).cuda() if bias else None
    gemm = ops.gemm_nvfp4 if fmt == "nvfp4" else ops.gemm_mxfp8
    d32 = gemm(ac, asf, bc, bsf, b, torch.float32)
    codes, sf = ops.gemm_qout(fmt, ac, asf, bc, bsf, b, out_fmt)
    torch.cuda.synchronize()
    if out_fmt == "mxfp8":
        want_c, want_s = orc.mxfp8_quantize_rowwise(d32.cpu())
    else:
        c, want_s = orc.nvfp4_quantize_rowwise(d32.cpu())
        want_c = orc.pack_fp4_pairs(c)
    assert codes.shape == want_c.shape
    assert torch.equal(codes.cpu(), want_c), f"{int((codes.cpu() != want_c).sum())} code bytes differ"
    assert torch.equal(sf.cpu(), orc.swizzle_rowwise(want_s)), "scale bytes (tile layout, zero padding included) differ"
    ops.check_status()


@pytest.mark.parametrize("out_fmt", ["mxfp8", "nvfp4"])
def test_chained_gemms_without_requantization(ops, out_fmt):
    """H = X W1^T leaves the first GEMM already quantized and feeds the second as its P operand."""
    n, ic, hid, oc = 512, 256, 1024, 384
    g = torch.Generator().manual_seed(7)
    x = torch.randn(n, ic, generator=g).to(torch.bfloat16).cuda()
    w1 = (torch.randn(hid, ic, generator=g) * 0.05).to(torch.bfloat16).cuda()
    w2 = (torch.randn(oc, hid, generator=g) * 0.05).to(torch.bfloat16).cuda()
    quant = ops.quantize_nvfp4 if out_fmt == "nvfp4" else ops.quantize_mxfp8
    gemm = ops.gemm_nvfp4 if out_fmt == "nvfp4" else ops.gemm_mxfp8
    xc, xsf, _, _ = quant(x)
    w1c, w1sf, _, _ = quant(w1)
    w2c, w2sf, _, _ = quant(w2)
    hc, hsf = ops.gemm_qout(out_fmt, xc, xsf, w1c, w1sf, None, out_fmt)
    y = gemm(hc, hsf, w2c, w2sf, None, torch.float32)
    if out_fmt == "nvfp4":
        hd = orc.nvfp4_dequant(orc.unpack_fp4_pairs(hc.cpu()), orc.unswizzle_rowwise(hsf.cpu(), n, hid // 16))
        wd = orc.nvfp4_dequant(orc.unpack_fp4_pairs(w2c.cpu()), orc.unswizzle_rowwise(w2sf.cpu(), oc, hid // 16))
    else:
        hd = orc.mxfp8_dequant(hc.cpu(), orc.unswizzle_rowwise(hsf.cpu(), n, hid // 32))
        wd = orc.mxfp8_dequant(w2c.cpu(), orc.unswizzle_rowwise(w2sf.cpu(), oc, hid // 32))
    assert orc.rel_frobenius(y.cpu(), hd.double() @ wd.double().t()) <= 1e-5
    ops.check_status()


def test_reference_operator_with_uint8_dout(ops):
    """torch.ops.xops.cublaslt_mm_mxfp8(..., DoutType=torch.uint8) -> (E4M3 codes, scaleDout)."""
    import backend.xops  # noqa: F401
    m, n, k = 128, 256, 512          # A [m, k] is the weight-like operand, B [n, k] the batch
    ac, asf, bc, bsf = _operands(ops, "mxfp8", m, n, k, 3)
    dt, sd = torch.ops.xops.cublaslt_mm_mxfp8(0, torch.uint8, ac, asf, bc, bsf, None)
    assert dt.dtype == torch.uint8 and dt.shape == (n, m)
    assert sd.dtype == torch.uint8 and sd.shape == ((m // 32 + 3) // 4 * 4, (n + 127) // 128 * 128)
    d32 = ops.gemm_mxfp8(bc, bsf, ac, asf, None, torch.float32)
    want_c, want_s = orc.mxfp8_quantize_rowwise(d32.cpu())
    assert torch.equal(dt.cpu(), want_c)
    assert torch.equal(sd.cpu().reshape(-1), orc.swizzle_rowwise(want_s).reshape(-1))
    with pytest.raises(RuntimeError):
        torch.ops.xops.cublaslt_mm_mxfp8(0, torch.uint8, ac[:48], asf, bc, bsf, None)     # m not a multiple of 32


def test_qout_argument_errors(ops):
    ac, asf, bc, bsf = _operands(ops, "mxfp8", 64, 48, 128, 5)
    with pytest.raises(ValueError):
        ops.gemm_qout("mxfp8", ac, asf, bc, bsf, None, "mxfp8")          # 48 columns: not a multiple of 32
