"""CPU checks of the oracle's restatements that have no counterpart in the reference (second
scale level, 16-point Hadamard transform): the identities they must satisfy, so that the GPU
parity tests compare against something that is itself pinned by construction."""
import numpy as np
import torch

from oracle import fp4t_oracle as orc


def _x(rows, cols, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * scale).to(torch.bfloat16)


def test_hadamard_matrix_and_orthogonality():
    h = np.array([[1.0]])
    for _ in range(4):
        h = np.block([[h, h], [h, -h]])                      # Sylvester order
    eye = torch.eye(16)
    assert np.array_equal(orc.hadamard16_blocks(eye, 0).numpy() * 4, h)
    signs = 0xA5C3
    d = np.diag([-1.0 if (signs >> j) & 1 else 1.0 for j in range(16)])
    # row i of the result is H . D . e_i / 4, i.e. column i of H D / 4
    assert np.array_equal(orc.hadamard16_blocks(eye, signs).numpy() * 4, (h @ d).T)
    x = torch.randn(32, 64, dtype=torch.float64).float()
    y = torch.randn(32, 64, dtype=torch.float64).float()
    hx, hy = orc.hadamard16_blocks(x, signs), orc.hadamard16_blocks(y, signs)
    assert torch.allclose((hx * hy).sum(), (x * y).sum(), rtol=1e-5)      # dot products are kept
    assert torch.allclose(hx.reshape(32, 4, 16).pow(2).sum(-1), x.reshape(32, 4, 16).pow(2).sum(-1), rtol=1e-5)
    # an involution up to the signs: H D (H D)^T / 16 = I  ->  applying D H / 4 undoes it
    back = orc.hadamard16_blocks(hx, 0) * torch.tensor(np.diag(d), dtype=torch.float32).repeat(4)
    assert torch.allclose(back, x, atol=1e-5)


def test_power_of_two_tensor_scale_is_a_relabelling():
    x = _x(64, 96, seed=3, scale=2.0 ** -11)
    t = 2.0 ** 11
    a = orc.nvfp4_quantize_scaled(x, t, want_t=True)
    b = orc.nvfp4_quantize((x.float() * t).to(torch.bfloat16), want_t=True)
    for k in ("codes", "sf", "codes_t", "sf_t"):
        assert torch.equal(a[k], b[k]), k
    one = orc.nvfp4_quantize_scaled(x, 1.0, want_t=True)
    ref = orc.nvfp4_quantize(x, want_t=True)
    for k in ("codes", "sf", "codes_t", "sf_t"):
        assert torch.equal(one[k], ref[k]), k


def test_second_level_rescues_blocks_below_the_scale_range():
    """amax < 6 * 2^-9: the one-level block scale clamps and the codes collapse towards zero; the
    same data lifted by a tensor scale dequantizes (codes x block scale / tensor scale) close to x."""
    x = _x(32, 64, seed=5, scale=2.0 ** -14)
    one = orc.nvfp4_quantize(x)
    lifted = orc.nvfp4_quantize_scaled(x, 2.0 ** 14)

    def deq(q, t):
        return orc.nvfp4_dequant(orc.unpack_fp4_pairs(q["codes"]), q["sf_logical"]) / t
    e1 = orc.rel_frobenius(deq(one, 1.0), x.float())
    e2 = orc.rel_frobenius(deq(lifted, 2.0 ** 14), x.float())
    assert e1 > 0.5 and e2 < 0.12, (e1, e2)


def test_hadamard_quantizer_dequantizes_to_the_transformed_tensor():
    x = _x(48, 128, seed=9)
    q = orc.nvfp4_quantize_scaled(x, 1.0, want_t=True, rht_signs=0x1234)
    want = orc.hadamard16_blocks(x.float(), 0x1234)
    got = orc.nvfp4_dequant(orc.unpack_fp4_pairs(q["codes"]), q["sf_logical"])
    assert orc.rel_frobenius(got, want) < 0.12
    want_t = orc.hadamard16_blocks(x.float().t().contiguous(), 0x1234)
    got_t = orc.nvfp4_dequant(orc.unpack_fp4_pairs(q["codes_t"]), q["sf_t_logical"])
    assert orc.rel_frobenius(got_t, want_t) < 0.12
