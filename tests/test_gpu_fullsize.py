"""Full-size cases of the benchmark configurations, checked through properties that do not
need a CPU pass over the whole tensor:

  * the transposed output of one fused launch is bit-identical to a row-wise launch on the
    materialised transpose (two different code paths of the kernel),
  * scale bytes are the E4M3 / E8M0 encodings of the block amax rule, recomputed with torch
    on the GPU from the oracle's formulas,
  * dequantized codes stay within half a grid step of the input,
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


def test_nvfp4_quantizer_config2_properties(ops):
    x, _, _ = _inputs(8192, 4096, 4096, 0)
    codes, sf, codes_t, sf_t = ops.quantize_nvfp4(x, True, True)
    # transposed output == row-wise quantization of the materialised transpose
    c2, s2, _, _ = ops.quantize_nvfp4(x.t().contiguous(), True, False)
    assert torch.equal(codes_t, c2) and torch.equal(sf_t, s2)
    # scale rule, recomputed with the oracle's formula on the GPU
    want = orc.nvfp4_block_scales(x).to(torch.float8_e4m3fn).view(torch.uint8)
    got = _unswz(sf, 8192, 256)
    assert torch.equal(got, want)
    # codes decode to within half a step of x / s (steps: 0.5 below 2, 1 below 4, 2 above)
    s32 = orc.nvfp4_block_scales(x).repeat_interleave(16, dim=1)
    y = x.float() / s32
    q = orc.e2m1_decode(orc.unpack_fp4_pairs(codes))
    step = torch.where(y.abs() < 2, 0.5, torch.where(y.abs() < 4, 1.0, 2.0))
    assert bool(((q - y).abs() <= step / 2 + 1e-6).all())
    assert bool((q.abs() <= 6).all())


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
