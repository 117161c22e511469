"""GPU parity of the fused quantizers against the CPU oracle and the golden fixtures.
Bit-exact comparisons: codes, scale bytes and their swizzled placement."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")
NVFP4_FILES = sorted(glob.glob(os.path.join(GOLD, "nvfp4_rowwise_*.npz")))


@pytest.fixture(scope="module")
def ops():
    from backend import ops as _ops
    return _ops


def _bf16(bits):
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)


def _eq(a: torch.Tensor, b: torch.Tensor, what: str):
    a, b = a.cpu(), b.cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    if not torch.equal(a, b):
        bad = (a != b).nonzero()
        raise AssertionError(f"{what}: {bad.shape[0]} of {a.numel()} bytes differ, first at {bad[0].tolist()}: "
                             f"got {a[tuple(bad[0])].item()} want {b[tuple(bad[0])].item()}")


@pytest.mark.parametrize("path", NVFP4_FILES, ids=lambda p: os.path.basename(p)[14:-4])
def test_nvfp4_matches_reference_fixtures(ops, path):
    z = np.load(path)
    x = _bf16(z["x_bits"]).cuda()
    want_t = "codes_t" in z and x.shape[0] % 32 == 0
    codes, sf, codes_t, sf_t = ops.quantize_nvfp4(x, want_row=True, want_t=want_t)
    _eq(codes, orc.pack_fp4_pairs(torch.from_numpy(z["codes"].copy())), "codes")
    _eq(sf, torch.from_numpy(z["scale_swizzled"].copy()), "swizzled scales")
    if want_t:
        _eq(codes_t, orc.pack_fp4_pairs(torch.from_numpy(z["codes_t"].copy())), "transposed codes")
        _eq(sf_t, torch.from_numpy(z["scale_swizzled_t"].copy()), "transposed swizzled scales")
    # stochastic rounding with the reference's own noise tensor
    noise = torch.from_numpy(z["sr_noise"].copy()).cuda()
    sr_codes, sr_sf, _, _ = ops.quantize_nvfp4(x, sr=ops.SR_NOISE, noise=noise)
    _eq(sr_codes, orc.pack_fp4_pairs(torch.from_numpy(z["sr_codes"].copy())), "SR codes")
    _eq(sr_sf, torch.from_numpy(z["scale_swizzled"].copy()), "SR scales")


SHAPES = [(128, 128), (256, 384), (64, 2048), (32, 16), (160, 48), (1024, 192), (96, 4096), (2, 32), (50, 64),
          (384, 1040)]


def _rand(rows, cols, kind, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    if kind == "outlier":
        x = torch.where(torch.rand(rows, cols, generator=g) < 1e-3, x * 50, x)
    elif kind == "grad":
        x = x * 1e-3
    elif kind == "wide":
        x = x * torch.logspace(-6, 4, cols).unsqueeze(0)
    elif kind == "zeros":
        x[:, : cols // 2] = 0
        x[0] = -0.0
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("kind", ["outlier", "grad", "wide", "zeros"])
@pytest.mark.parametrize("rows,cols", SHAPES)
def test_nvfp4_matches_oracle(ops, rows, cols, kind):
    x = _rand(rows, cols, kind, rows * 7 + cols)
    want_t = rows % 32 == 0
    want = orc.nvfp4_quantize(x, want_t=want_t)
    codes, sf, codes_t, sf_t = ops.quantize_nvfp4(x.cuda(), want_row=True, want_t=want_t)
    _eq(codes, want["codes"], "codes")
    _eq(sf, want["sf"], "scales")
    if want_t:
        _eq(codes_t, want["codes_t"], "transposed codes")
        _eq(sf_t, want["sf_t"], "transposed scales")


@pytest.mark.parametrize("rows,cols", [(128, 256), (64, 96), (32, 1024)])
def test_nvfp4_transposed_only_and_fp32_input(ops, rows, cols):
    x = _rand(rows, cols, "outlier", 5)
    want = orc.nvfp4_quantize(x, want_t=True)
    _, _, codes_t, sf_t = ops.quantize_nvfp4(x.cuda(), want_row=False, want_t=True)
    _eq(codes_t, want["codes_t"], "transposed codes")
    _eq(sf_t, want["sf_t"], "transposed scales")
    # fp32 input takes the generic kernel (true division); values are the same numbers
    codes, sf, codes_t, sf_t = ops.quantize_nvfp4(x.float().cuda(), want_row=True, want_t=True)
    _eq(codes, want["codes"], "fp32-in codes")
    _eq(sf, want["sf"], "fp32-in scales")
    _eq(codes_t, want["codes_t"], "fp32-in transposed codes")
    _eq(sf_t, want["sf_t"], "fp32-in transposed scales")


def test_nvfp4_full_fp32_input_matches_oracle(ops):
    g = torch.Generator().manual_seed(11)
    x = torch.randn(96, 160, generator=g) * 3.0       # 24-bit mantissas: exercises the division path
    want = orc.nvfp4_quantize(x)
    codes, sf, _, _ = ops.quantize_nvfp4(x.cuda())
    _eq(codes, want["codes"], "codes")
    _eq(sf, want["sf"], "scales")


@pytest.mark.parametrize("rows,cols", [(128, 256), (64, 64), (256, 48)])
def test_nvfp4_stochastic_noise_mode_both_outputs(ops, rows, cols):
    x = _rand(rows, cols, "grad", 3)
    g = torch.Generator().manual_seed(4)
    u = torch.rand(rows, cols, generator=g)
    ut = torch.rand(cols, rows, generator=g)
    want = orc.nvfp4_quantize(x, noise_row=u, want_t=True, noise_t=ut)
    codes, sf, codes_t, sf_t = ops.quantize_nvfp4(x.cuda(), want_t=True, sr=ops.SR_NOISE, noise=u.cuda(),
                                                  noise_t=ut.cuda())
    _eq(codes, want["codes"], "SR codes")
    _eq(codes_t, want["codes_t"], "SR transposed codes")
    _eq(sf, want["sf"], "scales")
    _eq(sf_t, want["sf_t"], "transposed scales")


def test_nvfp4_hash_sr_is_unbiased_and_on_neighbours(ops):
    """In-kernel noise: every code is one of the two grid neighbours of x/s and the mean
    of the dequantized values tracks the input (no parity claim, statistical check)."""
    g = torch.Generator().manual_seed(8)
    x = (torch.randn(512, 512, generator=g) * 1e-3).to(torch.bfloat16)
    codes, sf, _, _ = ops.quantize_nvfp4(x.cuda(), sr=ops.SR_HASH, seed=1234)
    codes2, _, _, _ = ops.quantize_nvfp4(x.cuda(), sr=ops.SR_HASH, seed=1234)
    codes3, _, _, _ = ops.quantize_nvfp4(x.cuda(), sr=ops.SR_HASH, seed=99)
    assert torch.equal(codes, codes2)
    assert not torch.equal(codes, codes3)
    s32 = orc.nvfp4_block_scales(x).repeat_interleave(16, dim=1)
    q = orc.e2m1_decode(orc.unpack_fp4_pairs(codes.cpu()))
    y = x.float() / s32
    grid = torch.tensor(orc.E2M1_GRID)
    lo = grid[(torch.bucketize(y.abs().clamp(max=6), grid, right=True) - 1).clamp(0, 7)]
    hi = grid[torch.bucketize(y.abs().clamp(max=6), grid, right=False).clamp(0, 7)]
    assert torch.all((q.abs() == lo) | (q.abs() == hi))
    assert abs(float((q * s32 - x.float()).mean())) < 2e-6
    _eq(sf, orc.nvfp4_quantize(x)["sf"], "scales")


@pytest.mark.parametrize("kind", ["outlier", "grad", "wide", "zeros"])
@pytest.mark.parametrize("rows,cols", [(128, 128), (256, 384), (64, 2048), (32, 32), (160, 96), (96, 4096),
                                       (2, 64), (50, 64), (1024, 160)])
def test_mxfp8_matches_oracle(ops, rows, cols, kind):
    x = _rand(rows, cols, kind, rows + cols * 3)
    want_t = rows % 32 == 0
    want = orc.mxfp8_quantize(x, want_t=want_t)
    codes, sf, codes_t, sf_t = ops.quantize_mxfp8(x.cuda(), want_row=True, want_t=want_t)
    _eq(codes, want["codes"], "codes")
    _eq(sf, want["sf"], "scales")
    if want_t:
        _eq(codes_t, want["codes_t"], "transposed codes")
        _eq(sf_t, want["sf_t"], "transposed scales")
    c32, s32_, _, _ = ops.quantize_mxfp8(x.float().cuda(), want_row=True, want_t=False)
    _eq(c32, want["codes"], "fp32-in codes")
    _eq(s32_, want["sf"], "fp32-in scales")


def test_argument_errors(ops):
    x = torch.zeros(4, 24, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.quantize_nvfp4(x)
    with pytest.raises(ValueError):
        ops.quantize_nvfp4(torch.zeros(4, 4, 32, device="cuda"))
    with pytest.raises(ValueError):
        ops.quantize_nvfp4(torch.zeros(48, 32, dtype=torch.bfloat16, device="cuda"), want_t=True)
    with pytest.raises(NotImplementedError):
        ops.quantize_nvfp4(torch.zeros(32, 32, dtype=torch.bfloat16))
    empty = ops.quantize_nvfp4(torch.zeros(0, 32, dtype=torch.bfloat16, device="cuda"))
    assert empty[0].shape == (0, 16)


def test_misc_byte_ops(ops):
    g = torch.Generator().manual_seed(2)
    for (a, b) in [(128, 4), (300, 5), (16, 256), (50, 12), (2, 2), (129, 9)]:
        m = torch.randint(0, 256, (a, b), generator=g).to(torch.uint8)
        _eq(ops.swizzle_rowwise(m.cuda()), orc.swizzle_rowwise(m), f"rowwise {a}x{b}")
        _eq(ops.swizzle_colwise(m.cuda()), orc.swizzle_colwise_reference_layout(m), f"colwise {a}x{b}")
        back = ops.colwise_to_canonical(orc.swizzle_colwise_reference_layout(m).cuda(), a, b)
        _eq(back, orc.swizzle_rowwise(m.t().contiguous()), f"colwise->canonical {a}x{b}")
        _eq(ops.transpose_bytes(m.cuda()), m.t().contiguous(), "transpose")
    vals = torch.tensor(orc.E2M1_GRID + tuple(-v for v in orc.E2M1_GRID))[torch.randint(0, 16, (8, 64), generator=g)]
    packed = ops.pack_e2m1(vals.cuda())
    _eq(packed, orc.pack_fp4_pairs(orc.e2m1_encode_rne_sat(vals)), "pack")
    assert torch.equal(ops.unpack_e2m1(packed).cpu(), vals)
    _eq(ops.pack_e2m1(vals.to(torch.bfloat16).cuda()), packed, "pack bf16")


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("rows,cols", [(256, 384), (64, 96), (1024, 192), (96, 4096), (50, 64), (32, 40)])
def test_fused_bias_gradient(ops, fmt, rows, cols):
    """Column sums taken inside the quantizer pass equal the separate fp32 column sum, and the
    codes are the same as without the fusion."""
    if fmt == "mxfp8" and cols % 32:
        pytest.skip("row-wise MXFP8 needs cols % 32 == 0")
    if fmt == "nvfp4" and cols % 16:
        cols = cols // 16 * 16 + 16
    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=g) * 1e-2).to(torch.bfloat16).cuda()
    want_t = rows % 32 == 0
    q = ops.quantize_nvfp4 if fmt == "nvfp4" else ops.quantize_mxfp8
    plain = q(x, True, want_t)
    for dt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 8e-3)):
        fused = q(x, True, want_t, bias_grad_dtype=dt)
        for a, b in zip(plain, fused[:4]):
            assert (a is None and b is None) or torch.equal(a, b)
        ref = x.float().sum(dim=0)
        assert fused[4].dtype == dt and fused[4].shape == (cols,)
        assert torch.allclose(fused[4].float(), ref, rtol=tol, atol=tol * float(ref.abs().max()) + 1e-7)
    # two calls in a row share the scratch buffer and must not leak into each other
    again = q(x * 2, True, want_t, bias_grad_dtype=torch.float32)
    assert torch.allclose(again[4], (x * 2).float().sum(dim=0), rtol=1e-6, atol=1e-6)
