"""Failure detection without a GPU fault, and guard bands around kernel outputs.

1. A bounded wait that runs out: the in-switch all-reduce is launched as rank 0 of a
   two-rank job whose second rank does not exist (its flag array is just another local
   buffer that nothing writes).  The very first cross-rank wait -- which comes before any
   multicast access -- gives up after the (shortened) limit, the kernel records status 41 and
   returns, `check_status` raises, and ordinary launches afterwards work.  Nothing faults,
   traps or hangs: the wait simply ends.
2. Guard bands: quantizer and GEMM outputs are carved out of a larger buffer pre-filled with a
   pattern; after the launch every byte outside the outputs still holds the pattern (what a
   memory checker would flag as an out-of-bounds write).
"""
import ctypes

import pytest
import torch

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from backend import ops as _ops
    return _ops


def test_allreduce_wait_runs_out_and_context_survives(ops):
    from backend import _lib
    L = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    status = ops.status_word(dev)
    status.zero_()
    numel = 4096
    buf = torch.ones(numel, dtype=torch.bfloat16, device=dev)          # stands in for the multicast address; never dereferenced
    flags = [torch.zeros(256 * 8, dtype=torch.int32, device=dev) for _ in range(2)]
    ptrs = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    torch.cuda.synchronize()
    _lib.check(L.fp4t_set_wait_timeout_ns(10_000_000), "fp4t_set_wait_timeout_ns")     # 10 ms (peer waits: 5 ms)
    try:
        rc = L.fp4t_allreduce_sum_bf16_multimem(buf.data_ptr(), ptrs, 0, 2, numel, 1, 4, status.data_ptr(),
                                                _lib.stream_ptr(dev))
        _lib.check(rc, "fp4t_allreduce_sum_bf16_multimem")
        torch.cuda.synchronize()
    finally:
        _lib.check(L.fp4t_set_wait_timeout_ns(4_000_000_000), "fp4t_set_wait_timeout_ns")
    assert int(status[0].item()) == 41, "the first cross-rank wait should have given up with code 41"
    assert bool((buf == 1).all()), "the buffer must be untouched: the kernel returned before its first access"
    with pytest.raises(RuntimeError, match="abandoned a wait"):
        ops.check_status(dev)
    assert int(status[0].item()) == 0                                   # check_status cleared it
    # the context is intact: a quantizer and a GEMM launch give oracle-equal results afterwards
    x = torch.randn(256, 512, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    want = orc.nvfp4_quantize(x)
    codes, sf, _, _ = ops.quantize_nvfp4(x.cuda())
    assert torch.equal(codes.cpu(), want["codes"]) and torch.equal(sf.cpu(), want["sf"])
    y = ops.gemm_nvfp4(codes, sf, codes, sf, None, torch.float32)
    d = orc.nvfp4_dequant(orc.unpack_fp4_pairs(want["codes"]), want["sf_logical"])
    assert orc.rel_frobenius(y.cpu(), d @ d.t()) <= 1e-5
    ops.check_status(dev)


def test_set_wait_timeout_rejects_nonsense():
    from backend import _lib
    assert _lib.lib().fp4t_set_wait_timeout_ns(5) == -1


PATTERN = 0xA5
GUARD = 4096          # bytes of guard band on each side of every output


class _Arena:
    """One patterned byte buffer; `take(nbytes)` returns 256-byte aligned views separated by guard bands."""

    def __init__(self, total, device):
        self.buf = torch.full((total,), PATTERN, dtype=torch.uint8, device=device)
        self.off = GUARD
        self.used = []

    def take(self, nbytes):
        start = (self.off + 255) // 256 * 256
        assert start + nbytes + GUARD <= self.buf.numel()
        self.used.append((start, start + nbytes))
        self.off = start + nbytes + GUARD
        return self.buf[start:start + nbytes]

    def check(self, what):
        mask = torch.ones(self.buf.numel(), dtype=torch.bool, device=self.buf.device)
        for a, b in self.used:
            mask[a:b] = False
        outside = self.buf[mask]
        bad = int((outside != PATTERN).sum().item())
        assert bad == 0, f"{what}: {bad} bytes outside the outputs were overwritten"


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("rows,cols", [(160, 48 * 2), (128, 128), (96, 1056), (32, 32), (416, 160)])
def test_quantizer_writes_stay_inside_outputs(ops, fmt, rows, cols):
    from backend import _lib
    L = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    blk = 16 if fmt == "nvfp4" else 32
    if cols % blk:
        pytest.skip("shape not a multiple of the block size")
    x = (torch.randn(rows, cols, generator=torch.Generator().manual_seed(rows + cols)) * 3).to(torch.bfloat16).cuda()
    arena = _Arena(4 << 20, dev)
    cb = rows * cols // 2 if fmt == "nvfp4" else rows * cols
    codes, codes_t = arena.take(cb), arena.take(cb)
    sf = arena.take(L.fp4t_sf_bytes(rows, cols // blk))
    sf_t = arena.take(L.fp4t_sf_bytes(cols, rows // blk))
    bgrad = arena.take(cols * 4)
    scratch = arena.take(cols * 4)
    ops._bind_status(dev)
    if fmt == "nvfp4":
        rc = L.fp4t_quantize_nvfp4_bgrad(x.data_ptr(), 0, rows, cols, x.stride(0), codes.data_ptr(), sf.data_ptr(),
                                         codes_t.data_ptr(), sf_t.data_ptr(), 2, None, None, ctypes.c_uint64(9),
                                         scratch.data_ptr(), bgrad.data_ptr(), 1, _lib.stream_ptr(dev))
    else:
        rc = L.fp4t_quantize_mxfp8_bgrad(x.data_ptr(), 0, rows, cols, x.stride(0), codes.data_ptr(), sf.data_ptr(),
                                         codes_t.data_ptr(), sf_t.data_ptr(), scratch.data_ptr(), bgrad.data_ptr(), 1,
                                         _lib.stream_ptr(dev))
    _lib.check(rc, "quantize")
    torch.cuda.synchronize()
    arena.check(f"{fmt} quantizer {rows}x{cols}")
    # and the outputs themselves are the oracle's (deterministic parts)
    want = (orc.nvfp4_quantize if fmt == "nvfp4" else orc.mxfp8_quantize)(x.cpu(), want_t=True)
    assert torch.equal(sf.cpu().view(want["sf"].shape), want["sf"])
    assert torch.equal(sf_t.cpu().view(want["sf_t"].shape), want["sf_t"])
    if fmt == "mxfp8":
        assert torch.equal(codes.cpu().view(rows, cols), want["codes"])
        assert torch.equal(codes_t.cpu().view(cols, rows), want["codes_t"])
    assert torch.allclose(bgrad.view(torch.float32).cpu(), x.float().sum(0).cpu(), rtol=1e-5, atol=1e-5)
    ops.check_status(dev)


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k", [(96, 72, 64), (64, 100, 64), (256, 256, 256), (300, 136, 512), (128, 520, 96), (640, 264, 1024)])
def test_gemm_writes_stay_inside_output(ops, fmt, dtype, m, n, k):
    dev = torch.device("cuda", torch.cuda.current_device())
    if fmt == "nvfp4" and k % 32:
        pytest.skip("K not a multiple of 32")
    g = torch.Generator().manual_seed(m * 3 + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(n, k, generator=g).to(torch.bfloat16).cuda()
    quant = ops.quantize_nvfp4 if fmt == "nvfp4" else ops.quantize_mxfp8
    gemm = ops.gemm_nvfp4 if fmt == "nvfp4" else ops.gemm_mxfp8
    ac, asf, _, _ = quant(a)
    bc, bsf, _, _ = quant(b)
    esz = 2 if dtype == torch.bfloat16 else 4
    arena = _Arena(8 << 20, dev)
    out = arena.take(m * n * esz).view(dtype).view(m, n)
    gemm(ac, asf, bc, bsf, None, dtype, out=out)
    torch.cuda.synchronize()
    arena.check(f"{fmt} gemm {m}x{n}x{k} {dtype}")
    if fmt == "nvfp4":
        ad = orc.nvfp4_dequant(orc.unpack_fp4_pairs(ac.cpu()), orc.unswizzle_rowwise(asf.cpu(), m, k // 16))
        bd = orc.nvfp4_dequant(orc.unpack_fp4_pairs(bc.cpu()), orc.unswizzle_rowwise(bsf.cpu(), n, k // 16))
    else:
        ad = orc.mxfp8_dequant(ac.cpu(), orc.unswizzle_rowwise(asf.cpu(), m, k // 32))
        bd = orc.mxfp8_dequant(bc.cpu(), orc.unswizzle_rowwise(bsf.cpu(), n, k // 32))
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert orc.rel_frobenius(out.float().cpu(), ad.double() @ bd.double().t()) <= tol
    ops.check_status(dev)
