"""The quantizer kernels divide by the block scale as `q = x * r; rem = fma(-q, s, x);
y = fma(rem, r, q)` with `r = RN(1/s)` (`div_corrected` in fp4-training_b200/csrc/fp4t_common.cuh)
instead of an IEEE division.  The reference divides (`y = x / s32`, custom/quantize.py:78), and a
result that is one ulp off flips an E2M1 code when it sits on a rounding boundary.  This checks
the three-instruction form against the true fp32 quotient for every pair of bf16 mantissas
(x, block abs-max) over 40 octaves of |x| / amax and three octaves of amax -- the arithmetic is
invariant under a common power-of-two factor, so that covers every bf16 input whose block scale is
not clamped -- with the FMAs emulated in 64-bit-mantissa long double (exact for the first FMA)."""
import numpy as np
import pytest

f32, ld = np.float32, np.longdouble


def _fma(a, b, c):
    return (a.astype(ld) * b.astype(ld) + c.astype(ld)).astype(f32)


@pytest.mark.skipif(np.finfo(ld).nmant < 63, reason="needs an 80-bit long double")
def test_corrected_reciprocal_multiply_equals_division():
    mant = (128 + np.arange(128)) / 128.0
    checked = uncorrected_bad = 0
    for ea in (0, 3, -5):
        amax = (mant * 2.0 ** ea).astype(f32)
        s = (amax / f32(6.0)).astype(f32)
        r = (f32(1.0) / s).astype(f32)
        for ex in range(0, -40, -1):
            x = (mant * 2.0 ** (ea + ex)).astype(f32)
            X, S = np.meshgrid(x, s)
            _, R = np.meshgrid(x, r)
            _, A = np.meshgrid(x, amax)
            inside = X <= A                       # |x| never exceeds its block's abs-max
            want = (X / S).astype(f32)
            q0 = (X * R).astype(f32)
            y = _fma(_fma(-q0, S, X), R, q0)
            assert not np.any((y != want) & inside)
            uncorrected_bad += int(np.sum((q0 != want) & inside))
            checked += int(np.sum(inside))
    assert checked > 1_000_000
    assert uncorrected_bad > 0      # the plain reciprocal multiply is NOT enough, hence the correction
