"""MXFP8 linear layer: E4M3 codes with UE8M0 scales per 32 elements in all three GEMMs
(reference: custom/linear/mxfp8.py:17-121)."""
from collections import OrderedDict
from enum import Enum

import torch
from torch.amp import custom_bwd, custom_fwd

import backend.xops  # noqa: F401

from ..quantize import q_mxfp8_colwise, q_mxfp8_rowwise
from . import _fused as F
from .cublaslt import TransAB
from .custom import CustomLinear, flatten_apply

op = torch.ops.xops


class DoutType(Enum):
    F32 = torch.float32
    BF16 = torch.bfloat16
    F8 = torch.float8_e4m3fn


STOCK = OrderedDict([
    ('1A', q_mxfp8_rowwise), ('1B', q_mxfp8_rowwise),
    ('2A', q_mxfp8_colwise), ('2B', q_mxfp8_rowwise),
    ('3A', q_mxfp8_colwise), ('3B', q_mxfp8_colwise),
])


def mxfp8_backward(ctx, grad_Y, W, X, Wt, Xt):
    """dgrad / wgrad / bias grad in MXFP8.  Wt / Xt are (codes_t, sf_t) pairs or None.
    -> (grad_X, grad_W, grad_b)."""
    need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    grad_X = grad_W = None
    if need_dx and Wt is None:
        Wt = F.quant_pair("mxfp8", W.to(grad_Y.dtype), False, True)[2:]
    if need_dw and Xt is None:
        Xt = F.quant_pair("mxfp8", X.to(grad_Y.dtype), False, True)[2:]
    need_db = ctx.has_bias and ctx.needs_input_grad[2]
    Gc, Gsf, Gtc, Gtsf, grad_b = F.grad_quant("mxfp8", grad_Y, need_dx, need_dw, need_db, sr=False)
    if need_dx:
        grad_X = F.gemm("mxfp8", Gc, Gsf, Wt[0], Wt[1], None, grad_Y.dtype)
    if need_dw:
        grad_W = F.gemm("mxfp8", Gtc, Gtsf, Xt[0], Xt[1], None, grad_Y.dtype)
    return grad_X, grad_W, grad_b


def mxfp8_backward_unfused(ctx, grad_Y, X, W):
    """The reference's call sequence (custom/linear/mxfp8.py:57-80) through the operator API."""
    grad_X = grad_W = None
    if ctx.needs_input_grad[0]:
        Wq, sW = ctx.quant['2A'](W.to(grad_Y.dtype))
        Gq, sG = ctx.quant['2B'](grad_Y)
        grad_X, _ = op.cublaslt_mm_mxfp8(TransAB.NN.value, grad_Y.dtype, Wq, sW, Gq, sG, None)
    if ctx.needs_input_grad[1]:
        Xq, sX = ctx.quant['3A'](X.to(grad_Y.dtype))
        Gq, sG = ctx.quant['3B'](grad_Y)
        grad_W, _ = op.cublaslt_mm_mxfp8(TransAB.NT.value, grad_Y.dtype, Xq, sX, Gq, sG, None)
    return grad_X, grad_W


class Mxfp8MatMul(torch.autograd.Function):
    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, X, W, b, quant: OrderedDict):
        ctx.quant = quant
        ctx.has_bias = b is not None
        ctx.fused = F.is_stock(quant, STOCK)
        if not ctx.fused:
            Wq, sW = quant['1A'](W)
            Xq, sX = quant['1B'](X)
            Y, _ = op.cublaslt_mm_mxfp8(TransAB.TN.value, X.dtype, Wq, sW, Xq, sX, b)
            ctx.save_for_backward(X, W)
            return Y
        if X.ndim != 2 or W.ndim != 2:
            raise ValueError("Input tensor must be 2D for mxfp8 quantization")
        X = X.contiguous()
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        ctx.layer_call = F.layer_call_ok("mxfp8", X, W, need_dx, need_dw)
        if ctx.layer_call:
            Y, ws = F.layer_forward("mxfp8", X, W, b, need_dx, need_dw)
            ctx.ic = X.shape[1]
            ctx.save_for_backward(ws)
            return Y
        Wc, Wsf, Wtc, Wtsf = F.quant_pair("mxfp8", W, True, need_dx and F.can_transpose(W))
        Xc, Xsf, Xtc, Xtsf = F.quant_pair("mxfp8", X, True, need_dw and F.can_transpose(X))
        Y = F.gemm("mxfp8", Xc, Xsf, Wc, Wsf, b, X.dtype)
        ctx.save_for_backward(Wtc, Wtsf, Xtc, Xtsf,
                              W if (need_dx and Wtc is None) else None,
                              X if (need_dw and Xtc is None) else None)
        return Y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_Y):
        grad_Y = grad_Y.contiguous()
        if not ctx.fused:
            X, W = ctx.saved_tensors
            grad_X, grad_W = mxfp8_backward_unfused(ctx, grad_Y, X, W)
            grad_b = grad_Y.sum(dim=0) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        elif ctx.layer_call:
            (ws,) = ctx.saved_tensors
            need_db = ctx.has_bias and ctx.needs_input_grad[2]
            grad_X, grad_W, grad_b = F.layer_backward("mxfp8", grad_Y, ws, ctx.ic, ctx.needs_input_grad[0],
                                                      ctx.needs_input_grad[1], need_db, sr=False)
        else:
            Wtc, Wtsf, Xtc, Xtsf, W, X = ctx.saved_tensors
            grad_X, grad_W, grad_b = mxfp8_backward(ctx, grad_Y, W, X,
                                                    None if Wtc is None else (Wtc, Wtsf),
                                                    None if Xtc is None else (Xtc, Xtsf))
        return grad_X, grad_W, grad_b, None


class CublasltMxfp8Linear(CustomLinear):
    """`nn.Linear` drop-in whose three GEMMs run in MXFP8 on tcgen05."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._init_quantizers()

    @classmethod
    def from_linear(cls, linear_layer):
        linear = super().from_linear(linear_layer)
        linear._init_quantizers()
        return linear

    def _init_quantizers(self):
        self.quantizers = OrderedDict(STOCK)

    def forward(self, input):
        return flatten_apply(self, Mxfp8MatMul.apply, input, self.quantizers)

    def forward_gelu(self, pre_activation):
        """self(GELU(pre_activation)) with the activation fused into the quantizer of the input
        operand (no bf16 GELU output in HBM).  Needs the stock quantizer table."""
        if not F.is_stock(self.quantizers, STOCK):
            return self.forward(torch.nn.functional.gelu(pre_activation))
        return F.gelu_linear(self, pre_activation, "mxfp8", False)

    @staticmethod
    def forward_stacked(modules, input):
        """[m(input) for m in modules] for layers of this class that share their input (q / k / v):
        one quantization of the input and one GEMM over the stacked weights.  Falls back to the
        separate calls where a layer's quantizer table is customised."""
        ok = all(F.is_stock(m.quantizers, STOCK) for m in modules)
        if not ok or input.shape[-1] % 32 or sum(m.out_features for m in modules) % 32:
            return [m(input) for m in modules]
        return F.stacked_linear(modules, input, "mxfp8", False)
