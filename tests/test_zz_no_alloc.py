"""The allocation-free bias-gradient quantizer (fp4t_quantize_nvfp4_bgrad_static).

Hosts that own all device memory themselves (a framework that only lends plugins their
input/output tensors, a server that pre-reserved the GPU for its pool) or that cannot afford
the device-wide stall of an allocation have no scratch buffer to pass.  This entry point
keeps its column-sum scratch inside the library instead.  The test calls it directly through
the C ABI with caller-owned inputs and outputs, twice in a row with different data (the
built-in scratch is shared and still holds the first call's sums when the second starts), and
checks every output against fp4t_quantize_nvfp4_bgrad, the entry point that takes caller
scratch: codes and scales bit for bit, the bias gradient to fp32 summation-order tolerance.
It runs last so that a failure here cannot hide the result of any other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_MAX_COLS = 16384


def _run(L, _lib, x, static, seed):
    rows, cols = x.shape
    dev = x.device
    out = {
        "codes": torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev),
        "sf": torch.empty(_lib.sf_shape(rows, cols // 16), dtype=torch.uint8, device=dev),
        "codes_t": torch.empty(cols, rows // 2, dtype=torch.uint8, device=dev),
        "sf_t": torch.empty(_lib.sf_shape(cols, rows // 16), dtype=torch.uint8, device=dev),
        "bgrad": torch.empty(cols, dtype=torch.float32, device=dev),
    }
    stream = _lib.stream_ptr(dev)
    common = (_lib.ptr(x), _lib.DT_BF16, rows, cols, x.stride(0), _lib.ptr(out["codes"]), _lib.ptr(out["sf"]),
              _lib.ptr(out["codes_t"]), _lib.ptr(out["sf_t"]), _lib.SR_HASH, None, None, ctypes.c_uint64(seed))
    if static:
        rc = L.fp4t_quantize_nvfp4_bgrad_static(*common, _lib.ptr(out["bgrad"]), _lib.DT_F32, stream)
    else:
        scratch = torch.full((cols,), 123.0, dtype=torch.float32, device=dev)   # stale contents on purpose
        rc = L.fp4t_quantize_nvfp4_bgrad(*common, _lib.ptr(scratch), _lib.ptr(out["bgrad"]), _lib.DT_F32, stream)
    _lib.check(rc, "bgrad quantizer")
    return out


def test_static_scratch_entry_point_matches_caller_scratch_entry_point():
    from backend import _lib
    L = _lib.lib()
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(2024)
    # second call uses fewer columns and different data than the first: stale sums of the
    # first call sit in the shared scratch when it starts
    shapes = [(512, 1024), (256, 384)]
    for i, (rows, cols) in enumerate(shapes):
        x = (torch.randn(rows, cols, generator=g) * (1e-2 * (i + 1))).to(torch.bfloat16).cuda()
        got = _run(L, _lib, x, static=True, seed=7 + i)
        want = _run(L, _lib, x, static=False, seed=7 + i)
        torch.cuda.synchronize()
        for k in ("codes", "sf", "codes_t", "sf_t"):
            assert torch.equal(got[k], want[k]), f"call {i}: {k} differ"
        ref = x.float().sum(dim=0)
        tol = 1e-5 * float(ref.abs().max()) + 1e-7
        assert torch.allclose(got["bgrad"], want["bgrad"], rtol=1e-5, atol=tol), f"call {i}: bias gradient"
        assert torch.allclose(got["bgrad"], ref, rtol=1e-5, atol=tol), f"call {i}: bias gradient vs column sum"


def test_static_scratch_entry_point_rejects_oversized_cols():
    from backend import _lib
    L = _lib.lib()
    x = torch.zeros(32, 32, dtype=torch.bfloat16, device="cuda")
    rc = L.fp4t_quantize_nvfp4_bgrad_static(_lib.ptr(x), _lib.DT_BF16, 32, STATIC_MAX_COLS + 16, STATIC_MAX_COLS + 16,
                                            None, None, None, None, 0, None, None, ctypes.c_uint64(0),
                                            _lib.ptr(x), _lib.DT_F32, _lib.stream_ptr(x.device))
    assert rc == -1
    msg = L.fp4t_last_error().decode()
    assert "exceeds" in msg and str(STATIC_MAX_COLS) in msg
