"""Pins the CPU oracle: against the committed golden fixtures (generated from the
reference's own quantize/swizzle code) and, when a reference checkout is present,
against that code run live on fresh random inputs."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import fp4t_oracle as orc
from tests.golden.make_golden import load_reference, reference_pack

GOLD = os.path.join(os.path.dirname(__file__), "golden")
NVFP4_FILES = sorted(glob.glob(os.path.join(GOLD, "nvfp4_rowwise_*.npz")))


def _bf16(bits):
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)


def test_fixtures_present():
    assert len(NVFP4_FILES) >= 8
    assert os.path.isfile(os.path.join(GOLD, "swizzle_cases.npz"))


@pytest.mark.parametrize("path", NVFP4_FILES, ids=lambda p: os.path.basename(p)[14:-4])
def test_nvfp4_oracle_matches_golden(path):
    z = np.load(path)
    x = _bf16(z["x_bits"])
    codes, sb = orc.nvfp4_quantize_rowwise(x)
    assert np.array_equal(codes.numpy(), z["codes"])
    assert np.array_equal(sb.numpy(), z["scale_bytes"])
    assert np.array_equal(orc.swizzle_rowwise(sb).numpy(), z["scale_swizzled"])
    sr_codes, sb2 = orc.nvfp4_quantize_rowwise(x, torch.from_numpy(z["sr_noise"].copy()))
    assert np.array_equal(sr_codes.numpy(), z["sr_codes"])
    assert np.array_equal(sb2.numpy(), z["scale_bytes"])
    if "codes_t" in z:
        out = orc.nvfp4_quantize(x, want_t=True)
        assert np.array_equal(orc.unpack_fp4_pairs(out["codes_t"]).numpy(), z["codes_t"])
        assert np.array_equal(out["sf_t"].numpy(), z["scale_swizzled_t"])


def test_swizzles_match_golden():
    z = np.load(os.path.join(GOLD, "swizzle_cases.npz"))
    names = [k[3:] for k in z.files if k.startswith("in_")]
    assert names
    for n in names:
        m = torch.from_numpy(z[f"in_{n}"].copy())
        assert np.array_equal(orc.swizzle_rowwise(m).numpy(), z[f"row_{n}"]), n
        assert np.array_equal(orc.swizzle_colwise_reference_layout(m).numpy(), z[f"col_{n}"]), n
        a, b = m.shape
        assert torch.equal(orc.unswizzle_rowwise(orc.swizzle_rowwise(m), a, b), m)


def test_colwise_reference_layout_is_canonical_only_for_one_outer_tile():
    g = torch.Generator().manual_seed(3)
    small = torch.randint(0, 256, (8, 128), generator=g).to(torch.uint8)   # [K-blocks, outer]
    big = torch.randint(0, 256, (8, 256), generator=g).to(torch.uint8)
    assert torch.equal(orc.swizzle_colwise_reference_layout(small).reshape(-1),
                       orc.swizzle_rowwise(small.t().contiguous()).reshape(-1))
    assert not torch.equal(orc.swizzle_colwise_reference_layout(big).reshape(-1),
                           orc.swizzle_rowwise(big.t().contiguous()).reshape(-1))


def test_pack_roundtrip_and_nibble_order():
    codes = torch.arange(16, dtype=torch.uint8).repeat(4, 2)
    packed = orc.pack_fp4_pairs(codes)
    assert packed[0, 0].item() == (0 | (1 << 4)) and packed[0, 1].item() == (2 | (3 << 4))
    assert torch.equal(orc.unpack_fp4_pairs(packed), codes)


def test_e2m1_ties_to_even():
    y = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.0, -0.1, -5.0, 100.0])
    want = torch.tensor([0, 2, 2, 4, 4, 6, 6, 7, 8, 8, 14, 7], dtype=torch.uint8)
    assert torch.equal(orc.e2m1_encode_rne_sat(y), want)


def test_mxfp8_restatement_properties():
    """Unpinned quantizer: check the properties the reference's wrapper relies on
    (custom/quantize.py:29-33,133-136): codes are exact E4M3, scale is a biased
    power of two, reconstruction error is within half an E4M3 step."""
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(64, 256, generator=g) * torch.logspace(-3, 3, 256)).to(torch.bfloat16)
    codes, sb = orc.mxfp8_quantize_rowwise(x)
    deq = orc.mxfp8_dequant(codes, sb)
    x32 = x.float()
    amax = x32.view(64, 8, 32).abs().amax(-1)
    s = orc.e8m0_decode(sb)
    assert torch.all(amax / s < 512) and torch.all(amax / s >= 256)
    err = (deq - x32).abs().view(64, 8, 32)
    # half a step of the top binade (32 * s / 2) plus saturation of (448, 512) to 448
    assert torch.all(err <= 64 * s.unsqueeze(-1))
    zero = torch.zeros(4, 32, dtype=torch.bfloat16)
    c0, s0 = orc.mxfp8_quantize_rowwise(zero)
    assert torch.all(c0 == 0) and torch.all(s0 == 0)
    fq = orc.mxfp8_fake_quant(x, -2)
    assert fq.shape == x.shape and fq.dtype == x.dtype


@pytest.mark.skipif(load_reference() is None, reason="reference checkout not present")
@pytest.mark.parametrize("scale,rows,cols", [(1.0, 64, 256), (1e-3, 128, 64), (30.0, 32, 512), (0.02, 96, 96)])
def test_nvfp4_oracle_matches_live_reference(scale, rows, cols):
    rq, rs = load_reference()
    g = torch.Generator().manual_seed(int(scale * 1000) + rows)
    x = (torch.randn(rows, cols, generator=g) * scale).to(torch.bfloat16)
    q, s = rq.quantize_nvfp4(x, rowwise=True, simulated=False)
    codes, sb = orc.nvfp4_quantize_rowwise(x)
    assert torch.equal(reference_pack(q), codes)
    assert torch.equal(s.view(torch.uint8), sb)
    torch.manual_seed(7)
    q3, _ = rq.quantize_nvfp4(x, rowwise=True, simulated=False, stochastic_rounding=True)
    torch.manual_seed(7)
    u = torch.rand(rows, cols // 16, 16)
    codes3, _ = orc.nvfp4_quantize_rowwise(x, u)
    assert torch.equal(reference_pack(q3), codes3)
    # simulated (dequantized) output equals decode(codes) * unrounded scale only up to the
    # E4M3 rounding of the scale; check the codes decode to the reference's q values instead
    assert torch.equal(orc.e2m1_decode(codes), q.clamp(-6, 6))
    sw_ref = rs.swizzle_rowwise_scale(s.view(torch.uint8))
    assert torch.equal(sw_ref, orc.swizzle_rowwise(sb))
