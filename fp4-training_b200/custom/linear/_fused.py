"""Fused operand preparation shared by the quantized Linear autograd functions.

The reference quantizes each GEMM operand separately and materialises bf16 transposes
first (custom/linear/nvfp4.py:59,74-75; custom/linear/mxfp8.py:59-80).  Here each of X, W
and dY is read once by one kernel that emits the row-wise operand and the transposed
operand together, so a linear layer's forward+backward is three quantizer launches and
three GEMM launches.
"""
from __future__ import annotations

import os
from functools import partial

import torch

from backend import ops as _ops

from .. import quantize as Q


def parity_mode() -> bool:
    """FP4T_PARITY=1: stochastic-rounding noise comes from `torch.rand`, drawn with the
    shapes and in the order of the reference (dgrad operand first, then wgrad operand),
    instead of the in-kernel generator."""
    return os.environ.get("FP4T_PARITY", "0") == "1"


def is_stock(quant, expected) -> bool:
    """True when the module's quantizer table still holds the stock entries, i.e. the fused
    kernels compute exactly what the table describes."""
    if quant is None or list(quant.keys()) != list(expected.keys()):
        return False
    for k, want in expected.items():
        got = quant[k]
        if isinstance(want, partial):
            if not (isinstance(got, partial) and got.func is want.func and got.keywords == want.keywords):
                return False
        elif got is not want:
            return False
    return True


def quant_pair(fmt, t, want_row, want_t, sr=False, bias_grad_dtype=None):
    """(codes, sf, codes_t, sf_t) of tensor t in format fmt ('nvfp4' | 'mxfp8'); with
    bias_grad_dtype a fifth element, the column sums of t, computed in the same pass."""
    if fmt == "mxfp8":
        return Q.mxfp8_fused(t, want_row, want_t, bias_grad_dtype)
    if not sr:
        return Q.nvfp4_fused(t, want_row, want_t, bias_grad_dtype=bias_grad_dtype)
    if parity_mode():
        r, c = t.shape
        noise = torch.rand(r, c // 16, 16, device=t.device) if want_row else None
        noise_t = torch.rand(c, r // 16, 16, device=t.device) if want_t else None
        return Q.nvfp4_fused(t, want_row, want_t, sr=True, noise=noise, noise_t=noise_t,
                             bias_grad_dtype=bias_grad_dtype)
    return Q.nvfp4_fused(t, want_row, want_t, sr=True, bias_grad_dtype=bias_grad_dtype)


def grad_quant(fmt, grad_Y, need_dx, need_dw, need_db, sr):
    """Quantize dY for dgrad / wgrad and, if asked, take the bias gradient in the same pass.
    -> (codes, sf, codes_t, sf_t, grad_b or None)."""
    if need_db and need_dw:      # the column sums ride on the transposed pass
        return quant_pair(fmt, grad_Y, need_dx, need_dw, sr=sr, bias_grad_dtype=grad_Y.dtype)
    out = quant_pair(fmt, grad_Y, need_dx, need_dw, sr=sr) if (need_dx or need_dw) else (None,) * 4
    return (*out, grad_Y.sum(dim=0) if need_db else None)


def grad_quant_scaled(grad_Y, tensor_scale, need_dx, need_dw):
    """NVFP4 operands of dY * tensor_scale with in-kernel stochastic rounding -> (codes, sf, codes_t, sf_t)."""
    if not (need_dx or need_dw):
        return (None,) * 4
    return _ops.quantize_nvfp4_scaled(grad_Y, tensor_scale, need_dx, need_dw, sr=_ops.SR_HASH, seed=Q._next_seed())


def gemm(fmt, p, p_sf, q, q_sf, bias, out_dtype, alpha=1.0):
    if fmt == "nvfp4":
        return _ops.gemm_nvfp4(p, p_sf, q, q_sf, bias, out_dtype, alpha=alpha)
    return _ops.gemm_mxfp8(p, p_sf, q, q_sf, bias, out_dtype)


def can_transpose(t) -> bool:
    return t.shape[0] % 32 == 0


def layer_call_ok(fmt, X, W, need_dx, need_dw) -> bool:
    """Shapes the one-call layer entry points take: every GEMM's K a multiple of 32 and the
    transposed operands constructible."""
    n, ic = X.shape
    oc = W.shape[0]
    if X.dtype not in (torch.bfloat16, torch.float32) or W.dtype != X.dtype:
        return False
    if ic % 32 or n == 0:
        return False
    if need_dx and oc % 32:
        return False
    if need_dw and n % 32:
        return False
    return X.stride(1) == 1 and W.stride(1) == 1


def layer_forward(fmt, X, W, b, need_dx, need_dw):
    return _ops.linear_forward(fmt, X, W, b, need_dx, need_dw, X.dtype)


def layer_backward(fmt, grad_Y, ws, ic, need_dx, need_dw, need_db, sr):
    if not (need_dx or need_dw):
        return None, None, (grad_Y.sum(dim=0) if need_db else None)
    if fmt == "nvfp4" and sr:
        if parity_mode():
            n, oc = grad_Y.shape
            noise = torch.rand(n, oc // 16, 16, device=grad_Y.device) if need_dx else None
            noise_t = torch.rand(oc, n // 16, 16, device=grad_Y.device) if need_dw else None
            return _ops.linear_backward(fmt, grad_Y, ws, ic, need_dx, need_dw, need_db, _ops.SR_NOISE, noise, noise_t)
        return _ops.linear_backward(fmt, grad_Y, ws, ic, need_dx, need_dw, need_db, _ops.SR_HASH, seed=Q._next_seed())
    return _ops.linear_backward(fmt, grad_Y, ws, ic, need_dx, need_dw, need_db)


class GeluQuantizedMatmul(torch.autograd.Function):
    """Y = GELU(P) W^T + b with GELU applied inside the quantizer of the activation operand
    (`fp4t_quantize_*_gelu`): the pre-activation P is read once and GELU(P) is never written as
    a bf16 tensor.  Values are those of `linear(F.gelu(P))` with the stock quantizer table, bit
    for bit (the kernel evaluates torch's own GELU formula and rounds to bf16 before quantizing).
    Backward: dY is quantized once, dH = dY W and dW = dY^T GELU(P) come from the saved transposed
    codes, and dP = dH * GELU'(P) is torch's gelu_backward on the saved pre-activation."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, P, W, b, fmt, sr):
        if P.ndim != 2 or W.ndim != 2:
            raise ValueError("Input tensor must be 2D")
        P = P.contiguous()
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        Xc, Xsf, Xtc, Xtsf = _ops.quantize_gelu(fmt, P, True, need_dw)
        Wc, Wsf, Wtc, Wtsf = quant_pair(fmt, W, True, need_dx)
        Y = gemm(fmt, Xc, Xsf, Wc, Wsf, b, P.dtype)
        ctx.fmt, ctx.sr, ctx.has_bias = fmt, sr, b is not None
        ctx.save_for_backward(P, Wtc, Wtsf, Xtc, Xtsf)
        return Y

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_Y):
        P, Wtc, Wtsf, Xtc, Xtsf = ctx.saved_tensors
        grad_Y = grad_Y.contiguous()
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_db = ctx.has_bias and ctx.needs_input_grad[2]
        Gc, Gsf, Gtc, Gtsf, grad_b = grad_quant(ctx.fmt, grad_Y, need_dx, need_dw, need_db, sr=ctx.sr)
        grad_P = grad_W = None
        if need_dx:
            grad_H = gemm(ctx.fmt, Gc, Gsf, Wtc, Wtsf, None, grad_Y.dtype)
            grad_P = torch.ops.aten.gelu_backward(grad_H, P.to(grad_H.dtype))
        if need_dw:
            grad_W = gemm(ctx.fmt, Gtc, Gtsf, Xtc, Xtsf, None, grad_Y.dtype)
        return grad_P, grad_W, grad_b, None, None


def gelu_linear(module, pre, fmt, sr):
    """module(GELU(pre)) through GeluQuantizedMatmul; `pre` may have leading dims."""
    shape = pre.shape
    out = GeluQuantizedMatmul.apply(pre.reshape(-1, shape[-1]), module.weight, module.bias, fmt, sr)
    return out.view(shape[:-1] + (module.out_features,))


class StackedMatmul(torch.autograd.Function):
    """Y_i = X W_i^T + b_i for several projections of the SAME input (the q / k / v projections of
    the reference's attention block, models/transformer_block.py:60-66) as one quantization of X
    and ONE GEMM over the row-stacked weights; backward: the output gradients are laid side by
    side, quantized once, and dX = dY W and dW = dY^T X are one GEMM each.  Values equal the
    separate layers' up to the stochastic-rounding draws (the same distribution, other seeds);
    launches per block and step drop from 24 to 9.

    forward(X, fmt, sr, n, W_1..W_n, b_1..b_n) -> (Y_1, ..., Y_n), column slices of one buffer."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, X, fmt, sr, n, *wb):
        Ws, bs = wb[:n], wb[n:]
        if X.ndim != 2:
            raise ValueError("Input tensor must be 2D")
        X = X.contiguous()
        has_bias = bs[0] is not None
        need_dx = ctx.needs_input_grad[0]
        need_dw = any(ctx.needs_input_grad[4:4 + n])
        W = torch.cat(Ws, dim=0)
        b = torch.cat(bs) if has_bias else None
        Xc, Xsf, Xtc, Xtsf = quant_pair(fmt, X, True, need_dw)
        Wc, Wsf, Wtc, Wtsf = quant_pair(fmt, W, True, need_dx)
        Y = gemm(fmt, Xc, Xsf, Wc, Wsf, b, X.dtype)
        ctx.fmt, ctx.sr, ctx.n, ctx.has_bias = fmt, sr, n, has_bias
        ctx.splits = [w.shape[0] for w in Ws]
        ctx.save_for_backward(Wtc, Wtsf, Xtc, Xtsf)
        return tuple(Y.split(ctx.splits, dim=1))

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, *grads):
        Wtc, Wtsf, Xtc, Xtsf = ctx.saved_tensors
        n = ctx.n
        ref = next(g for g in grads if g is not None)
        parts = [g if g is not None else ref.new_zeros(ref.shape[0], o) for g, o in zip(grads, ctx.splits)]
        grad_Y = torch.cat(parts, dim=1)
        need_dx = ctx.needs_input_grad[0]
        need_dw = any(ctx.needs_input_grad[4:4 + n])
        need_db = ctx.has_bias and any(ctx.needs_input_grad[4 + n:4 + 2 * n])
        Gc, Gsf, Gtc, Gtsf, grad_b = grad_quant(ctx.fmt, grad_Y, need_dx, need_dw, need_db, sr=ctx.sr)
        grad_X = gemm(ctx.fmt, Gc, Gsf, Wtc, Wtsf, None, grad_Y.dtype) if need_dx else None
        grad_Ws = [None] * n
        if need_dw:
            grad_Ws = list(gemm(ctx.fmt, Gtc, Gtsf, Xtc, Xtsf, None, grad_Y.dtype).split(ctx.splits, dim=0))
        grad_bs = list(grad_b.split(ctx.splits)) if need_db else [None] * n
        return (grad_X, None, None, None, *grad_Ws, *grad_bs)


def stacked_linear(modules, x, fmt, sr):
    """[m(x) for m in modules] through StackedMatmul; `x` may have leading dims."""
    shape = x.shape
    ws = [m.weight for m in modules]
    bs = [m.bias for m in modules]
    if any(b is None for b in bs) and not all(b is None for b in bs):
        raise ValueError("stacked projections need a bias on all layers or on none")
    outs = StackedMatmul.apply(x.reshape(-1, shape[-1]), fmt, sr, len(modules), *ws, *bs)
    return [o.view(shape[:-1] + (m.out_features,)) for o, m in zip(outs, modules)]
