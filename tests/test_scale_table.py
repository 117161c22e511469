"""The quantizer kernels take the NVFP4 block scale from a 128-entry table keyed by the bf16
mantissa of the block's abs-max instead of dividing (`nvfp4_scale_from_table` in
fp4-training_b200/csrc/fp4t_common.cuh).  This restates that integer / min / max arithmetic
with numpy and checks it against the reference formula `clamp(amax / 6, 2^-9, 448)`
(custom/quantize.py:75-76) and its correctly rounded reciprocal for EVERY non-negative bf16
abs-max, zero, subnormals and infinity included."""
import numpy as np


def test_table_scale_equals_true_division_for_every_bf16_amax():
    bits = (np.arange(0, 0x7F81, dtype=np.uint32) << 16).astype(np.uint32)     # +0 ... +inf
    amax = bits.view(np.float32)
    m = np.arange(128, dtype=np.float32)
    tab_s = ((np.float32(1.0) + m / np.float32(128.0)) / np.float32(6.0)).astype(np.float32)
    tab_r = (np.float32(1.0) / tab_s).astype(np.float32)

    b = np.maximum(bits, np.uint32(0x0C800000))
    idx = (b >> 16) & 0x7F
    e = (b & np.uint32(0x7F800000)).astype(np.int64) - 0x3F800000
    sf = ((tab_s[idx].view(np.uint32).astype(np.int64) + e) & 0xFFFFFFFF).astype(np.uint32).view(np.float32)
    rf = ((tab_r[idx].view(np.uint32).astype(np.int64) - e) & 0xFFFFFFFF).astype(np.uint32).view(np.float32)
    with np.errstate(all="ignore"):
        s = np.minimum(np.maximum(sf, np.float32(2.0 ** -9)), np.float32(448.0))
        r = np.minimum(np.fmax(rf, np.float32(1.0) / np.float32(448.0)), np.float32(512.0))
        want_s = np.minimum(np.maximum((amax / np.float32(6.0)).astype(np.float32), np.float32(2.0 ** -9)),
                            np.float32(448.0))
        want_r = (np.float32(1.0) / want_s).astype(np.float32)
    assert np.array_equal(s.view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(r.view(np.uint32), want_r.view(np.uint32))
