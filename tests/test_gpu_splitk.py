"""Split-K: a small output over a long K (the wgrad of a small layer over a long batch) is
spread over the SMs that would otherwise idle.  Checked against the dequantized matmul, against
the unsplit kernel (same value up to fp32 summation order), for determinism, and through the
layer call that uses it for dW."""
import pytest
import torch

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from backend import ops as _ops
    return _ops


def _deq(fmt, codes, sf, outer, k):
    if fmt == "nvfp4":
        return orc.nvfp4_dequant(orc.unpack_fp4_pairs(codes.cpu()), orc.unswizzle_rowwise(sf.cpu(), outer, k // 16))
    return orc.mxfp8_dequant(codes.cpu(), orc.unswizzle_rowwise(sf.cpu(), outer, k // 32))


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k,bias", [(192, 192, 25600, False), (768, 192, 25600, True), (64, 96, 8192, True),
                                         (200, 72, 4096, False), (256, 512, 16384, True)])
def test_splitk_matches_dequantized_matmul_and_unsplit_kernel(ops, fmt, dtype, m, n, k, bias):
    from backend import _lib
    assert _lib.lib().fp4t_gemm_splitk_workspace_bytes(m, n) > 0
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(n, k, generator=g).to(torch.bfloat16).cuda()
    bv = (torch.randn(n, generator=g) * 3).to(torch.bfloat16).cuda() if bias else None
    quant = ops.quantize_nvfp4 if fmt == "nvfp4" else ops.quantize_mxfp8
    gemm = ops.gemm_nvfp4 if fmt == "nvfp4" else ops.gemm_mxfp8
    ac, asf, _, _ = quant(a)
    bc, bsf, _, _ = quant(b)
    split = gemm(ac, asf, bc, bsf, bv, dtype)
    whole = gemm(ac, asf, bc, bsf, bv, dtype, split_k=False)
    ref = _deq(fmt, ac, asf, m, k).double() @ _deq(fmt, bc, bsf, n, k).double().t()
    if bias:
        ref = ref + bv.double().cpu()
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert orc.rel_frobenius(split.float().cpu(), ref) <= tol
    assert orc.rel_frobenius(whole.float().cpu(), ref) <= tol
    assert orc.rel_frobenius(split.float().cpu(), whole.double().cpu()) <= (8e-3 if dtype == torch.bfloat16 else 1e-5)
    for _ in range(5):                                    # fixed summation order: repeatable bits
        assert torch.equal(gemm(ac, asf, bc, bsf, bv, dtype), split)
    ops.check_status()


def test_large_outputs_do_not_ask_for_a_workspace():
    from backend import _lib
    L = _lib.lib()
    assert L.fp4t_gemm_splitk_workspace_bytes(8192, 4096) == 0
    assert L.fp4t_gemm_splitk_workspace_bytes(0, 128) == 0


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
def test_layer_backward_uses_splitk_for_small_weight_gradients(ops, fmt):
    """TinyViT-sized projection (25600 tokens, 192 -> 768): dW is 768 x 192 over K = 25600."""
    n, ic, oc = 25600, 192, 768
    g = torch.Generator().manual_seed(5)
    x = torch.randn(n, ic, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(oc, ic, generator=g) * 0.05).to(torch.bfloat16).cuda()
    gy = (torch.randn(n, oc, generator=g) * 1e-2).to(torch.bfloat16).cuda()
    y, ws = ops.linear_forward(fmt, x, w, None, True, True, torch.bfloat16)
    dx, dw, _ = ops.linear_backward(fmt, gy, ws, ic, True, True, False)
    quant = ops.quantize_nvfp4 if fmt == "nvfp4" else ops.quantize_mxfp8
    _, _, xtc, xtsf = quant(x, False, True)
    _, _, gtc, gtsf = quant(gy, False, True)
    ref = _deq(fmt, gtc, gtsf, oc, n).double() @ _deq(fmt, xtc, xtsf, ic, n).double().t()
    assert orc.rel_frobenius(dw.float().cpu(), ref) <= 1e-2
    dx2, dw2, _ = ops.linear_backward(fmt, gy, ws, ic, True, True, False)
    assert torch.equal(dw, dw2) and torch.equal(dx, dx2)
    ops.check_status()
