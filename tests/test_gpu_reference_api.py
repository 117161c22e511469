"""The quantizer and swizzle entry points under the reference's own names
(custom.quantize.*, custom.swizzle.*) against what the reference returned for the same
calls (tests/golden/nvfp4_api_*.npz, swizzle_cases.npz; made by tests/golden/make_golden.py).

Values, dtypes, shapes and scale bytes are compared exactly.  Stochastic rounding is compared
with the reference's own noise: `torch.rand` is patched to hand back the stored draw (row-wise
in the blocked shape [R, C/16, 16]; column-wise in the [R, C] layout in which the reference's
strided `rand_like` consumes the stream).  One documented difference: a value the
reference leaves at 8 (its pack kernel clips it to 6 later) comes back as 6 here; and a
stochastic zero may carry either sign.
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")
API_FILES = sorted(glob.glob(os.path.join(GOLD, "nvfp4_api_*.npz")))


def _bf16(bits):
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a).copy())


def _same(got: torch.Tensor, want: torch.Tensor, what: str):
    got = got.cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert got.dtype == want.dtype, f"{what}: dtype {got.dtype} vs {want.dtype}"
    if not torch.equal(got, want):
        bad = (got != want).nonzero()
        raise AssertionError(f"{what}: {bad.shape[0]} of {got.numel()} entries differ, first at {bad[0].tolist()}: "
                             f"got {got[tuple(bad[0])].item()} want {want[tuple(bad[0])].item()}")


@pytest.fixture(scope="module")
def cq():
    from custom import quantize
    return quantize


def test_fixtures_present():
    assert len(API_FILES) >= 4


@pytest.mark.parametrize("path", API_FILES, ids=lambda p: os.path.basename(p)[10:-4])
@pytest.mark.parametrize("rowwise", [True, False], ids=["rowwise", "colwise"])
def test_quantize_nvfp4_by_reference_name(cq, path, rowwise):
    z = np.load(path)
    tag = "row" if rowwise else "col"
    x = _bf16(z["x_bits"]).cuda()
    # simulated=False: (fp32 E2M1-valued tensor of the input's shape, float8_e4m3fn logical scales)
    q, s = cq.quantize_nvfp4(x, rowwise=rowwise, simulated=False, stochastic_rounding=False)
    _same(q, _t(z[f"q_{tag}"]), f"quantize_nvfp4(rowwise={rowwise}) values")
    assert s.dtype == torch.float8_e4m3fn
    _same(s.contiguous().view(torch.uint8), _t(z[f"s_{tag}"]), f"quantize_nvfp4(rowwise={rowwise}) scales")
    # simulated=True (the default): dequantized fp32 tensor, multiplied by the UNROUNDED fp32 scale
    sim = cq.quantize_nvfp4(x, rowwise=rowwise)
    _same(sim.contiguous(), _t(z[f"sim_{tag}"]), f"quantize_nvfp4(rowwise={rowwise}, simulated=True)")


@pytest.mark.parametrize("path", API_FILES, ids=lambda p: os.path.basename(p)[10:-4])
@pytest.mark.parametrize("rowwise", [True, False], ids=["q_nvfp4_rowwise", "q_nvfp4_colwise"])
def test_q_nvfp4_by_reference_name(cq, path, rowwise, monkeypatch):
    z = np.load(path)
    tag = "row" if rowwise else "col"
    x = _bf16(z["x_bits"]).cuda()
    fn = cq.q_nvfp4_rowwise if rowwise else cq.q_nvfp4_colwise
    q, sw = fn(x)
    assert q.is_contiguous() and sw.dtype == torch.uint8 and sw.ndim == 2
    _same(q, _t(z[f"q_{tag}"]), f"{fn.__name__} values")
    _same(sw.contiguous(), _t(z[f"sw_{tag}"]), f"{fn.__name__} swizzled scales")

    # stochastic rounding on the reference's noise draw
    noise = _t(z[f"sr_noise_{tag}"]).cuda()
    real_rand = torch.rand

    def fake_rand(*shape, **kw):
        shp = tuple(shape[0]) if len(shape) == 1 and not isinstance(shape[0], int) else tuple(shape)
        if shp == tuple(noise.shape):
            return noise.clone()
        return real_rand(*shape, **kw)

    monkeypatch.setattr(torch, "rand", fake_rand)
    qs, sws = fn(x, sr=True)
    monkeypatch.undo()
    want = _t(z[f"sr_q_{tag}"]).clamp(-6.0, 6.0)            # the pack kernel's saturation, applied early here
    got = qs.cpu()
    assert got.shape == want.shape and got.dtype == want.dtype
    assert torch.equal(got.abs(), want.abs()), f"{fn.__name__}(sr=True): magnitudes differ"
    nz = want != 0
    assert torch.equal(torch.signbit(got[nz]), torch.signbit(want[nz])), f"{fn.__name__}(sr=True): signs differ"
    _same(sws.contiguous(), _t(z[f"sw_{tag}"]), f"{fn.__name__}(sr=True) scales")


def test_swizzles_by_reference_name():
    from custom import swizzle
    z = np.load(os.path.join(GOLD, "swizzle_cases.npz"))
    names = sorted(k[3:] for k in z.files if k.startswith("in_"))
    assert names
    for n in names:
        m = _t(z[f"in_{n}"]).cuda()
        _same(swizzle.swizzle_rowwise_scale(m).contiguous(), _t(z[f"row_{n}"]), f"swizzle_rowwise_scale {n}")
        _same(swizzle.swizzle_colwise_scale(m).contiguous(), _t(z[f"col_{n}"]), f"swizzle_colwise_scale {n}")


@pytest.mark.parametrize("rows,cols", [(64, 128), (96, 160), (256, 64), (32, 4096)])
def test_q_mxfp8_by_reference_name(cq, rows, cols):
    """MXFP8 entry points against the oracle's restatement of the OCP-MX conversion (the
    reference's own quantizer library is not available anywhere: parity unpinned)."""
    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=g) * torch.logspace(-3, 2, cols).unsqueeze(0)).to(torch.bfloat16)
    want = orc.mxfp8_quantize(x, want_t=True)
    codes, sw = cq.q_mxfp8_rowwise(x.cuda())
    assert codes.dtype == torch.uint8 and sw.dtype == torch.uint8
    _same(codes, want["codes"], "q_mxfp8_rowwise codes")
    _same(sw, want["sf"], "q_mxfp8_rowwise scales")
    codes_c, sw_c = cq.q_mxfp8_colwise(x.cuda())
    # column-wise codes keep the input's shape; the scales of logical [R/32, C] are in the
    # reference's column-wise layout
    _same(codes_c, want["codes_t"].t().contiguous(), "q_mxfp8_colwise codes")
    logical_t = want["sf_t_logical"]                                         # [C, R/32]
    _same(sw_c.contiguous(), orc.swizzle_colwise_reference_layout(logical_t.t().contiguous()).contiguous(),
          "q_mxfp8_colwise scales")
    # fake quantization = codes x 2^(scale-127), in the input's dtype
    fq = cq.fq_mxfp8_rowwise(x.cuda())
    assert fq.dtype == x.dtype and fq.shape == x.shape
    _same(fq, orc.mxfp8_fake_quant(x, axis=-1), "fq_mxfp8_rowwise")
    fqc = cq.fq_mxfp8_colwise(x.cuda())
    _same(fqc.contiguous(), orc.mxfp8_fake_quant(x, axis=-2).contiguous(), "fq_mxfp8_colwise")


def test_reference_error_behaviour(cq):
    x3 = torch.zeros(2, 16, 16, device="cuda")
    for fn in (cq.q_nvfp4_rowwise, cq.q_nvfp4_colwise, cq.q_mxfp8_rowwise, cq.q_mxfp8_colwise):
        with pytest.raises(ValueError):
            fn(x3)
    with pytest.raises(ValueError):
        cq.quantize_nvfp4(torch.zeros(16, 24, device="cuda"), rowwise=True)
    with pytest.raises(ValueError):
        cq.quantize_nvfp4(torch.zeros(24, 16, device="cuda"), rowwise=False)
    with pytest.raises(NotImplementedError):
        cq.q_nvfp4_rowwise(torch.zeros(32, 32))
