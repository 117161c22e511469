"""Full-size cases of the benchmark configurations, checked through properties that do not
need a CPU pass over the whole tensor:

  * NVFP4 codes and scale bytes of the benchmark tensors are compared byte for byte with the
    oracle's quantizer evaluated on the same (GPU-resident) tensors,
  * GEMM outputs match an fp32 matmul of the dequantized operands (oracle dequantizers run
    on the GPU tensors), rel-Frobenius <= 1e-2 for bf16 output.
"""
import pytest
import torch

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from backend import ops as _ops
    return _ops


def _inputs(n, ic, oc, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(n, ic, device="cuda", generator=g)
    x = torch.where(torch.rand(n, ic, device="cuda", generator=g) < 1e-3, x * 50, x).to(torch.bfloat16)
    w = (torch.randn(oc, ic, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    gr = (torch.randn(n, oc, device="cuda", generator=g) * 1e-3).to(torch.bfloat16)
    return x, w, gr


def _unswz(sf, outer, inner):
    return orc.unswizzle_rowwise(sf.cpu(), outer, inner).cuda()


def _oracle_codes_and_scales(t, noise=None):
    """The oracle's row-wise quantizer run on the GPU tensors (it is plain torch arithmetic,
    IEEE divisions included): packed codes [R, C/2] and logical scale bytes [R, C/16]."""
    codes, sb = orc.nvfp4_quantize_rowwise(t, noise)
    return orc.pack_fp4_pairs(codes), sb


def _count_diff(a, b):
    return int((a != b).sum().item())


def test_nvfp4_quantizer_config2_bit_exact(ops):
    """Every code and every scale byte of the three tensors of the benchmark configuration
    (X with its x50 outliers, W, dY with stochastic rounding on a given noise tensor), row-wise
    and transposed, against the oracle on the same tensors: 0 differing bytes."""
    n, ic, oc = 8192, 4096, 4096
    x, w, g = _inputs(n, ic, oc, 0)
    for name, t in (("X", x), ("W", w)):
        r, c = t.shape
        codes, sf, codes_t, sf_t = ops.quantize_nvfp4(t, True, True)
        want_c, want_s = _oracle_codes_and_scales(t)
        assert _count_diff(codes, want_c) == 0, f"{name}: row-wise codes"
        assert _count_diff(_unswz(sf, r, c // 16), want_s) == 0, f"{name}: row-wise scales"
        del want_c, want_s
        want_c, want_s = _oracle_codes_and_scales(t.t().contiguous())
        assert _count_diff(codes_t, want_c) == 0, f"{name}: transposed codes"
        assert _count_diff(_unswz(sf_t, c, r // 16), want_s) == 0, f"{name}: transposed scales"
        del want_c, want_s, codes, codes_t
    # dY: stochastic rounding with explicit noise (one tensor per emitted copy, as the reference
    # draws one per quantizer call)
    gen = torch.Generator(device="cuda").manual_seed(77)
    u = torch.rand(n, oc, device="cuda", generator=gen)
    ut = torch.rand(oc, n, device="cuda", generator=gen)
    codes, sf, codes_t, sf_t = ops.quantize_nvfp4(g, True, True, sr=ops.SR_NOISE, noise=u, noise_t=ut)
    want_c, want_s = _oracle_codes_and_scales(g, u)
    assert _count_diff(codes, want_c) == 0, "dY: row-wise SR codes"
    assert _count_diff(_unswz(sf, n, oc // 16), want_s) == 0, "dY: row-wise scales"
    del want_c, want_s
    want_c, want_s = _oracle_codes_and_scales(g.t().contiguous(), ut)
    assert _count_diff(codes_t, want_c) == 0, "dY: transposed SR codes"
    assert _count_diff(_unswz(sf_t, oc, n // 16), want_s) == 0, "dY: transposed scales"
    # padding bytes of the scale buffers are zero (they are read by the GEMM's K tail handling)
    assert int(sf.sum().item()) == int(_unswz(sf, n, oc // 16).sum().item())
    ops.check_status()


def test_nvfp4_linear_config2_against_dequantized_matmul(ops):
    n, ic, oc = 8192, 4096, 4096
    x, w, g = _inputs(n, ic, oc, 1)
    bias = (torch.randn(oc, device="cuda") * 0.1).to(torch.bfloat16)
    xc, xsf, xtc, xtsf = ops.quantize_nvfp4(x, True, True)
    wc, wsf, wtc, wtsf = ops.quantize_nvfp4(w, True, True)
    gc, gsf, gtc, gtsf, db = ops.quantize_nvfp4(g, True, True, sr=ops.SR_HASH, seed=5, bias_grad_dtype=torch.float32)

    def deq(c, s, outer, k):
        return orc.nvfp4_dequant(orc.unpack_fp4_pairs(c), _unswz(s, outer, k // 16))

    y = ops.gemm_nvfp4(xc, xsf, wc, wsf, bias, torch.bfloat16)
    ref = deq(xc, xsf, n, ic) @ deq(wc, wsf, oc, ic).t() + bias.float()
    assert orc.rel_frobenius(y.float(), ref) <= 1e-2
    dx = ops.gemm_nvfp4(gc, gsf, wtc, wtsf, None, torch.bfloat16)
    ref = deq(gc, gsf, n, oc) @ deq(wtc, wtsf, ic, oc).t()
    assert orc.rel_frobenius(dx.float(), ref) <= 1e-2
    dw = ops.gemm_nvfp4(gtc, gtsf, xtc, xtsf, None, torch.float32)
    ref = deq(gtc, gtsf, oc, n) @ deq(xtc, xtsf, ic, n).t()
    assert orc.rel_frobenius(dw, ref) <= 1e-4          # fp32 out: only the accumulation order differs
    assert torch.allclose(db, g.float().sum(0), rtol=1e-4, atol=1e-6)
    # the stochastic codes are unbiased at this size: mean of dequantized dY tracks dY
    assert abs(float((deq(gc, gsf, n, oc) - g.float()).mean())) < 2e-7
    ops.check_status()


def test_mxfp8_mlp_pair_config3_against_dequantized_matmul(ops):
    """Up- and down-projection shapes of the MXFP8 MLP configuration, forward GEMMs at full size."""
    n, ic, hid = 16384, 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(2)
    chan = torch.distributions.StudentT(3.0).sample((ic,)).abs().cuda()
    x = (torch.randn(n, ic, device="cuda", generator=g) * chan).to(torch.bfloat16)
    w_up = (torch.randn(hid, ic, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w_dn = (torch.randn(ic, hid, device="cuda", generator=g) * 0.02).to(torch.bfloat16)

    def deq(c, s, outer, k):
        return orc.mxfp8_dequant(c, _unswz(s, outer, k // 32))

    xc, xsf, xtc, xtsf = ops.quantize_mxfp8(x, True, True)
    c2, s2, _, _ = ops.quantize_mxfp8(x.t().contiguous(), True, False)
    assert torch.equal(xtc, c2) and torch.equal(xtsf, s2)
    uc, usf, _, _ = ops.quantize_mxfp8(w_up, True, False)
    h = ops.gemm_mxfp8(xc, xsf, uc, usf, None, torch.bfloat16)
    ref = deq(xc, xsf, n, ic) @ deq(uc, usf, hid, ic).t()
    assert orc.rel_frobenius(h.float(), ref) <= 1e-2
    del ref
    hc, hsf, _, _ = ops.quantize_mxfp8(h, True, False)
    dc, dsf, _, _ = ops.quantize_mxfp8(w_dn, True, False)
    out = ops.gemm_mxfp8(hc, hsf, dc, dsf, None, torch.bfloat16)
    ref = deq(hc, hsf, n, hid) @ deq(dc, dsf, ic, hid).t()
    assert orc.rel_frobenius(out.float(), ref) <= 1e-2
    ops.check_status()


def test_mxfp8_mlp_pair_config3_backward_gemms(ops):
    """dgrad and wgrad of both projections of the MXFP8 MLP configuration at full size
    (N=16384, 4096 -> 14336 -> 4096), each against the fp32 matmul of its dequantized operands.
    Operand forms follow the reference's backward (custom/linear/mxfp8.py:60-80): dY row-wise
    for dgrad, the column-wise (here: transposed) copies of W, X and dY for the rest."""
    n, ic, hid = 16384, 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(3)
    chan = torch.distributions.StudentT(3.0).sample((ic,)).abs().cuda()
    x = (torch.randn(n, ic, device="cuda", generator=g) * chan).to(torch.bfloat16)
    w_up = (torch.randn(hid, ic, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w_dn = (torch.randn(ic, hid, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    gy = (torch.randn(n, ic, device="cuda", generator=g) * 1e-3).to(torch.bfloat16)

    def deq(c, s, outer, k):
        return orc.mxfp8_dequant(c, _unswz(s, outer, k // 32))

    def check(pc, ps, qc, qs, rows, cols, k, what):
        out = ops.gemm_mxfp8(pc, ps, qc, qs, None, torch.bfloat16)
        ref = deq(pc, ps, rows, k) @ deq(qc, qs, cols, k).t()
        err = orc.rel_frobenius(out.float(), ref)
        assert err <= 1e-2, f"{what}: rel-Frobenius {err:.3e}"
        return out

    # forward intermediates needed by the backward operands
    xc, xsf, xtc, xtsf = ops.quantize_mxfp8(x, True, True)
    uc, usf, utc, utsf = ops.quantize_mxfp8(w_up, True, True)
    h = ops.gemm_mxfp8(xc, xsf, uc, usf, None, torch.bfloat16)
    del xc, xsf, uc, usf
    _, _, htc, htsf = ops.quantize_mxfp8(h, False, True)
    del h
    _, _, dtc, dtsf = ops.quantize_mxfp8(w_dn, False, True)
    # down-projection backward: dH = G W_dn, dW_dn = G^T H
    gc, gsf, gtc, gtsf = ops.quantize_mxfp8(gy, True, True)
    dh = check(gc, gsf, dtc, dtsf, n, hid, ic, "down-projection dgrad")
    check(gtc, gtsf, htc, htsf, ic, hid, n, "down-projection wgrad")
    del gc, gsf, gtc, gtsf, htc, htsf, dtc, dtsf
    # up-projection backward: dX = dH W_up, dW_up = dH^T X
    hc, hsf, hgt, hgtsf = ops.quantize_mxfp8(dh, True, True)
    del dh
    check(hc, hsf, utc, utsf, n, ic, hid, "up-projection dgrad")
    check(hgt, hgtsf, xtc, xtsf, hid, ic, n, "up-projection wgrad")
    ops.check_status()


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("m,n,k", [(16, 8192, 8192), (128, 8192, 8192), (1024, 16384, 2048), (16384, 1024, 4096)])
def test_gemm_sweep_shapes(ops, fmt, m, n, k):
    """Skinny and large members of the GEMM sweep configuration."""
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn(n, k, device="cuda", generator=g).to(torch.bfloat16)
    if fmt == "nvfp4":
        ac, asf, _, _ = ops.quantize_nvfp4(a)
        bc, bsf, _, _ = ops.quantize_nvfp4(b)
        ad = orc.nvfp4_dequant(orc.unpack_fp4_pairs(ac), _unswz(asf, m, k // 16))
        bd = orc.nvfp4_dequant(orc.unpack_fp4_pairs(bc), _unswz(bsf, n, k // 16))
        out = ops.gemm_nvfp4(ac, asf, bc, bsf, None, torch.bfloat16)
    else:
        ac, asf, _, _ = ops.quantize_mxfp8(a)
        bc, bsf, _, _ = ops.quantize_mxfp8(b)
        ad = orc.mxfp8_dequant(ac, _unswz(asf, m, k // 32))
        bd = orc.mxfp8_dequant(bc, _unswz(bsf, n, k // 32))
        out = ops.gemm_mxfp8(ac, asf, bc, bsf, None, torch.bfloat16)
    assert orc.rel_frobenius(out.float(), ad @ bd.t()) <= 1e-2
    ops.check_status()


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("m,n,k,dtype", [(4096, 4096, 8192, torch.float32), (8192, 4096, 4096, torch.bfloat16),
                                         (8192, 4096, 4096, torch.float32), (2048, 1536, 4096, torch.bfloat16)])
def test_gemm_is_deterministic(ops, fmt, m, n, k, dtype):
    """The GEMM has a fixed accumulation order, so repeated launches on the same operands must
    agree bit for bit.  A hand-over between the kernel's roles that is not properly ordered (a
    ring slot refilled while it is still being read, a scale buffer overwritten early) shows up
    here as a few rows that differ by one K slab's contribution, far below the parity tolerance."""
    gen = torch.Generator(device="cuda").manual_seed(m + k)
    a = torch.randn(m, k, device="cuda", generator=gen).to(torch.bfloat16)
    b = torch.randn(n, k, device="cuda", generator=gen).to(torch.bfloat16)
    quant = ops.quantize_nvfp4 if fmt == "nvfp4" else ops.quantize_mxfp8
    gemm = ops.gemm_nvfp4 if fmt == "nvfp4" else ops.gemm_mxfp8
    ac, asf, _, _ = quant(a, True, False)
    bc, bsf, _, _ = quant(b, True, False)
    first = gemm(ac, asf, bc, bsf, None, dtype).clone()
    for _ in range(20):
        again = gemm(ac, asf, bc, bsf, None, dtype)
        assert torch.equal(again, first)
    ops.check_status()


def test_tile_counter_reset_keeps_results(ops):
    """fp4t_reset_tile_counters zeroes the per-stream tile counters (what a host does after a launch
    reported a timed-out wait); launches after it give the same bits as before."""
    from backend import _lib
    gen = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randn(1024, 2048, device="cuda", generator=gen).to(torch.bfloat16)
    b = torch.randn(768, 2048, device="cuda", generator=gen).to(torch.bfloat16)
    ac, asf, _, _ = ops.quantize_nvfp4(a, True, False)
    bc, bsf, _, _ = ops.quantize_nvfp4(b, True, False)
    first = ops.gemm_nvfp4(ac, asf, bc, bsf, None, torch.float32).clone()
    _lib.check(_lib.lib().fp4t_reset_tile_counters(_lib.stream_ptr(a.device)), "fp4t_reset_tile_counters")
    ac2, asf2, _, _ = ops.quantize_nvfp4(a, True, False)
    assert torch.equal(ac, ac2) and torch.equal(asf, asf2)
    assert torch.equal(ops.gemm_nvfp4(ac, asf, bc, bsf, None, torch.float32), first)
    ops.check_status()


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
def test_chained_layer_calls_are_deterministic(ops, fmt):
    """Forward + backward of one layer is six kernels launched back to back, each allowed to set
    itself up under the tail of its predecessor (programmatic dependent launch) and each drawing
    its tiles dynamically.  Repeating the chain on the same inputs must give the same bits: a
    kernel that touched its predecessor's output before that kernel completed would show here."""
    n, ic, oc = 4096, 2048, 3072
    x, w, g = _inputs(n, ic, oc, 3)
    bias = (torch.randn(oc, device="cuda") * 0.1).to(torch.bfloat16)
    ref = None
    for _ in range(8):
        y, ws = ops.linear_forward(fmt, x, w, bias, True, True, torch.bfloat16)
        dx, dw, db = ops.linear_backward(fmt, g, ws, ic, True, True, True, sr=ops.SR_HASH, seed=7)
        cur = (y.clone(), dx.clone(), dw.clone())
        if ref is None:
            ref = cur
        else:
            for a, b in zip(cur, ref):
                assert torch.equal(a, b)
    ops.check_status()


def test_layer_chain_replays_from_a_cuda_graph(ops):
    """Quantizer and GEMM launches captured into a CUDA graph (static tile order inside a capture,
    dependent-launch attribute kept) replay to the same bits as the eager launches."""
    gen = torch.Generator(device="cuda").manual_seed(21)
    a = torch.randn(2048, 1024, device="cuda", generator=gen).to(torch.bfloat16)
    b = torch.randn(1536, 1024, device="cuda", generator=gen).to(torch.bfloat16)
    ac, asf, _, _ = ops.quantize_nvfp4(a, True, False)
    bc, bsf, _, _ = ops.quantize_nvfp4(b, True, False)
    want = ops.gemm_nvfp4(ac, asf, bc, bsf, None, torch.bfloat16).clone()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    out = torch.empty_like(want)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for _ in range(2):      # warm-up on the capture stream
            c2, s2, _, _ = ops.quantize_nvfp4(a, True, False)
            ops.gemm_nvfp4(c2, s2, bc, bsf, None, torch.bfloat16, out=out)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            c2, s2, _, _ = ops.quantize_nvfp4(a, True, False)
            ops.gemm_nvfp4(c2, s2, bc, bsf, None, torch.bfloat16, out=out)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
    ops.check_status()
