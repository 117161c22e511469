"""GPU parity of the tcgen05 block-scaled GEMMs against the dequantized-fp32 matmul oracle.

Tolerance: relative Frobenius error <= 1e-2 for bf16 output (the bf16 rounding of the
output alone is ~2e-3); fp32 output is held to 1e-5 because operands, scales and the
fp32 accumulation are the same numbers on both sides."""
import pytest
import torch

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu

TOL_BF16 = 1e-2
TOL_F32 = 1e-5


@pytest.fixture(scope="module")
def ops():
    from backend import ops as _ops
    return _ops


def _operands(fmt, rows, cols, k, seed):
    g = torch.Generator().manual_seed(seed)
    p = torch.randn(rows, k, generator=g).to(torch.bfloat16)
    q = (torch.randn(cols, k, generator=g) * 0.05).to(torch.bfloat16)
    if fmt == "nvfp4":
        pq, qq = orc.nvfp4_quantize(p), orc.nvfp4_quantize(q)
        pd = orc.nvfp4_dequant(orc.unpack_fp4_pairs(pq["codes"]), pq["sf_logical"])
        qd = orc.nvfp4_dequant(orc.unpack_fp4_pairs(qq["codes"]), qq["sf_logical"])
    else:
        pq, qq = orc.mxfp8_quantize(p), orc.mxfp8_quantize(q)
        pd = orc.mxfp8_dequant(pq["codes"], pq["sf_logical"])
        qd = orc.mxfp8_dequant(qq["codes"], qq["sf_logical"])
    return pq, qq, pd, qd


SHAPES = [
    (128, 128, 256), (128, 256, 256), (128, 256, 512), (256, 512, 1024), (128, 128, 64), (128, 128, 32),
    (128, 128, 96), (64, 96, 64), (200, 320, 160), (4, 32, 64), (64, 128, 32), (384, 192, 768), (130, 264, 2048),
    (1024, 768, 192), (512, 1024, 4096),
]


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("rows,cols,k", SHAPES)
def test_gemm_matches_dequantized_matmul(ops, fmt, rows, cols, k):
    pq, qq, pd, qd = _operands(fmt, rows, cols, k, rows + cols + k)
    g = torch.Generator().manual_seed(1)
    bias = torch.randn(cols, generator=g).to(torch.bfloat16)
    fn = ops.gemm_nvfp4 if fmt == "nvfp4" else ops.gemm_mxfp8
    args = (pq["codes"].cuda(), pq["sf"].cuda(), qq["codes"].cuda(), qq["sf"].cuda())
    ref = orc.gemm_dequant_fp32(pd, qd, None, double=True)
    ref_b = orc.gemm_dequant_fp32(pd, qd, bias, double=True)

    out32 = fn(*args, None, torch.float32)
    ops.check_status()
    assert out32.shape == (rows, cols) and out32.dtype == torch.float32
    assert orc.rel_frobenius(out32.cpu(), ref) <= TOL_F32

    out = fn(*args, bias.cuda(), torch.bfloat16)
    ops.check_status()
    assert out.dtype == torch.bfloat16
    assert orc.rel_frobenius(out.float().cpu(), ref_b) <= TOL_BF16
    assert torch.isfinite(out).all()


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
def test_gemm_many_tiles_per_cta(ops, fmt):
    """More tiles than SMs: exercises the persistent loop, both accumulators and stage wrap."""
    rows, cols, k = 2048, 3072, 512
    g = torch.Generator().manual_seed(3)
    p = torch.randn(rows, k, generator=g).to(torch.bfloat16).cuda()
    q = (torch.randn(cols, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    if fmt == "nvfp4":
        pc, ps, _, _ = ops.quantize_nvfp4(p)
        qc, qs, _, _ = ops.quantize_nvfp4(q)
        pd = orc.nvfp4_dequant(orc.unpack_fp4_pairs(pc.cpu()), orc.unswizzle_rowwise(ps.cpu(), rows, k // 16))
        qd = orc.nvfp4_dequant(orc.unpack_fp4_pairs(qc.cpu()), orc.unswizzle_rowwise(qs.cpu(), cols, k // 16))
        out = ops.gemm_nvfp4(pc, ps, qc, qs, None, torch.float32)
    else:
        pc, ps, _, _ = ops.quantize_mxfp8(p)
        qc, qs, _, _ = ops.quantize_mxfp8(q)
        pd = orc.mxfp8_dequant(pc.cpu(), orc.unswizzle_rowwise(ps.cpu(), rows, k // 32))
        qd = orc.mxfp8_dequant(qc.cpu(), orc.unswizzle_rowwise(qs.cpu(), cols, k // 32))
        out = ops.gemm_mxfp8(pc, ps, qc, qs, None, torch.float32)
    ops.check_status()
    ref = pd @ qd.t()
    assert orc.rel_frobenius(out.cpu(), ref) <= TOL_F32
    # linearity in the scale bytes is the size-independent property: doubling every P scale
    # (exponent +1) doubles the output exactly
    if fmt == "mxfp8":
        out2 = ops.gemm_mxfp8(pc, (ps + (ps > 0).to(torch.uint8)), qc, qs, None, torch.float32)
        live = (ps.cpu() > 0)
        if bool(live.all()):
            assert torch.equal(out2, out * 2)


def test_gemm_argument_errors(ops):
    z = torch.zeros(128, 24, dtype=torch.uint8, device="cuda")
    s = torch.zeros(32, 16, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        ops.gemm_nvfp4(z, s, z, s)          # K = 48 is not a multiple of 32
    with pytest.raises(RuntimeError):
        ops.gemm_nvfp4(z, s, torch.zeros(128, 32, dtype=torch.uint8, device="cuda"), s)
