"""NVFP4 linear layer: E2M1 codes with UE4M3 scales per 16 elements in all three GEMMs,
stochastic rounding on the gradient operand (reference: custom/linear/nvfp4.py:17-127)."""
from collections import OrderedDict
from functools import partial

import torch
from torch.amp import custom_bwd, custom_fwd

import backend.xops  # noqa: F401

from ..quantize import q_nvfp4_rowwise
from . import _fused as F
from .cublaslt import TransAB
from .custom import CustomLinear, flatten_apply

op = torch.ops.xops

STOCK = OrderedDict([
    ('1A', q_nvfp4_rowwise), ('1B', q_nvfp4_rowwise),
    ('2A', q_nvfp4_rowwise), ('2B', partial(q_nvfp4_rowwise, sr=True)),
    ('3A', q_nvfp4_rowwise), ('3B', partial(q_nvfp4_rowwise, sr=True)),
])


class Nvfp4Matmul(torch.autograd.Function):
    """Y = X W^T + b, dX = dY W, dW = dY^T X with every operand in NVFP4.

    With the stock quantizer table the fused path runs: X, W (forward) and dY (backward)
    are each quantized once into both operand forms.  A customised table falls back to the
    reference's own sequence of calls (custom/linear/nvfp4.py:25-90): bf16 transposes, one
    quantizer call per operand and the packing `xops.cublaslt_mm_nvfp4` operator."""

    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, X, W, b, quant: OrderedDict, grad_scale: float = 1.0):
        ctx.quant = quant
        ctx.grad_scale = float(grad_scale)
        ctx.has_bias = b is not None
        ctx.fused = F.is_stock(quant, STOCK)
        if ctx.grad_scale != 1.0 and not ctx.fused:
            raise ValueError("grad_tensor_scale needs the stock quantizer table")
        if not ctx.fused:
            Wq, sW = quant['1A'](W)
            Xq, sX = quant['1B'](X)
            Y, _ = op.cublaslt_mm_nvfp4(TransAB.TN.value, X.dtype, Wq, sW, Xq, sX, b)
            ctx.save_for_backward(X, W)
            return Y
        if X.ndim != 2 or W.ndim != 2:
            raise ValueError("Input tensor must be 2D for nvfp4 quantization")
        X = X.contiguous()
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        # wgrad contracts over the batch and dgrad over out_features: an FP4 GEMM's K must be a
        # multiple of 32 (rows of 16-byte multiples).  The forward pass is defined for such shapes
        # (inference under grad mode, the reference's own forward-only checks); the backward pass is
        # not, and says so as soon as it is entered, naming the dimension.
        ctx.shape_error = None
        if need_dw and X.shape[0] % 32:
            ctx.shape_error = f"nvfp4 weight gradients need the flattened batch ({X.shape[0]}) to be a multiple of 32"
        elif need_dx and W.shape[0] % 32:
            ctx.shape_error = f"nvfp4 input gradients need out_features ({W.shape[0]}) to be a multiple of 32"
        if ctx.shape_error is not None:
            Wc, Wsf, _, _ = F.quant_pair("nvfp4", W, True, False)
            Xc, Xsf, _, _ = F.quant_pair("nvfp4", X, True, False)
            ctx.layer_call = False
            return F.gemm("nvfp4", Xc, Xsf, Wc, Wsf, b, X.dtype)
        ctx.layer_call = F.layer_call_ok("nvfp4", X, W, need_dx, need_dw) and ctx.grad_scale == 1.0
        if ctx.layer_call:      # one C call for the layer; the workspace holds the backward operands
            Y, ws = F.layer_forward("nvfp4", X, W, b, need_dx, need_dw)
            ctx.ic = X.shape[1]
            ctx.save_for_backward(ws)
            return Y
        Wc, Wsf, Wtc, Wtsf = F.quant_pair("nvfp4", W, True, need_dx and F.can_transpose(W))
        Xc, Xsf, Xtc, Xtsf = F.quant_pair("nvfp4", X, True, need_dw and F.can_transpose(X))
        Y = F.gemm("nvfp4", Xc, Xsf, Wc, Wsf, b, X.dtype)
        # operands of the backward GEMMs; the bf16 tensor is kept only where the transposed
        # form could not be built (the backward pass then reports the shape error)
        ctx.save_for_backward(Wtc, Wtsf, Xtc, Xtsf,
                              W if (need_dx and Wtc is None) else None,
                              X if (need_dw and Xtc is None) else None)
        return Y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_Y):
        if getattr(ctx, "shape_error", None) is not None:
            raise ValueError(ctx.shape_error)
        grad_Y = grad_Y.contiguous()
        grad_X = grad_W = grad_b = None
        if not ctx.fused:
            X, W = ctx.saved_tensors
            if ctx.needs_input_grad[0]:
                Wtq, sWt = ctx.quant['2A'](W.to(grad_Y.dtype).T.contiguous())
                Gq, sG = ctx.quant['2B'](grad_Y)
                grad_X, _ = op.cublaslt_mm_nvfp4(TransAB.TN.value, grad_Y.dtype, Wtq, sWt, Gq, sG, None)
            if ctx.needs_input_grad[1]:
                Xtq, sXt = ctx.quant['3A'](X.to(grad_Y.dtype).T.contiguous())
                Gtq, sGt = ctx.quant['3B'](grad_Y.T.contiguous())
                grad_W, _ = op.cublaslt_mm_nvfp4(TransAB.TN.value, grad_Y.dtype, Xtq, sXt, Gtq, sGt, None)
        elif ctx.layer_call:
            (ws,) = ctx.saved_tensors
            need_db = ctx.has_bias and ctx.needs_input_grad[2]
            grad_X, grad_W, grad_b = F.layer_backward("nvfp4", grad_Y, ws, ctx.ic, ctx.needs_input_grad[0],
                                                      ctx.needs_input_grad[1], need_db, sr=True)
            return grad_X, grad_W, grad_b, None, None
        else:
            Wtc, Wtsf, Xtc, Xtsf, W, X = ctx.saved_tensors
            need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
            if need_dx and Wtc is None:
                _, _, Wtc, Wtsf = F.quant_pair("nvfp4", W, False, True)
            if need_dw and Xtc is None:
                _, _, Xtc, Xtsf = F.quant_pair("nvfp4", X, False, True)
            need_db = ctx.has_bias and ctx.needs_input_grad[2]
            t = ctx.grad_scale
            if t != 1.0:     # second scale level on dY: quantize dY * t, give 1/t back in the GEMM epilogue
                Gc, Gsf, Gtc, Gtsf = F.grad_quant_scaled(grad_Y, t, need_dx, need_dw)
                grad_b = grad_Y.sum(dim=0) if need_db else None
            else:
                Gc, Gsf, Gtc, Gtsf, grad_b = F.grad_quant("nvfp4", grad_Y, need_dx, need_dw, need_db, sr=True)
            if need_dx:
                grad_X = F.gemm("nvfp4", Gc, Gsf, Wtc, Wtsf, None, grad_Y.dtype, alpha=1.0 / t)
            if need_dw:
                grad_W = F.gemm("nvfp4", Gtc, Gtsf, Xtc, Xtsf, None, grad_Y.dtype, alpha=1.0 / t)
            return grad_X, grad_W, grad_b, None, None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_b = grad_Y.sum(dim=0)
        return grad_X, grad_W, grad_b, None, None


class CublasltNvfp4Linear(CustomLinear):
    """`nn.Linear` drop-in whose three GEMMs run in NVFP4 on tcgen05.

    `grad_tensor_scale` (default 1, i.e. the reference's one-level recipe) is a per-tensor scale
    on the gradient operand: dY * grad_tensor_scale is what gets block-quantized, and the dgrad
    and wgrad GEMMs multiply their accumulators by its reciprocal.  A power of two keeps the
    quantizer on its tiled kernel.  It lifts gradients whose blocks sit below the smallest
    UE4M3 block scale (amax < 6 * 2^-9) back into the range the block scale can express."""

    grad_tensor_scale = 1.0

    def __init__(self, *args, grad_tensor_scale: float = 1.0, **kwargs):
        super().__init__(*args, **kwargs)
        self.grad_tensor_scale = float(grad_tensor_scale)
        self._init_quantizers()

    @classmethod
    def from_linear(cls, linear_layer):
        linear = super().from_linear(linear_layer)
        linear._init_quantizers()
        return linear

    def _init_quantizers(self):
        self.quantizers = OrderedDict(STOCK)   # all row-wise: every GEMM is K-major on both sides

    def forward(self, input):
        return flatten_apply(self, Nvfp4Matmul.apply, input, self.quantizers, self.grad_tensor_scale)

    def forward_gelu(self, pre_activation):
        """self(GELU(pre_activation)) with the activation fused into the quantizer of the input
        operand (no bf16 GELU output in HBM).  Needs the stock quantizer table."""
        if not F.is_stock(self.quantizers, STOCK):
            return self.forward(torch.nn.functional.gelu(pre_activation))
        return F.gelu_linear(self, pre_activation, "nvfp4", True)

    @staticmethod
    def forward_stacked(modules, input):
        """[m(input) for m in modules] for layers of this class that share their input (q / k / v):
        one quantization of the input and one GEMM over the stacked weights.  Falls back to the
        separate calls where a layer's quantizer table is customised, a gradient tensor scale is
        set, or the bit-exact stochastic-rounding mode is on (its draws follow the separate
        layers' order)."""
        ok = all(F.is_stock(m.quantizers, STOCK) and m.grad_tensor_scale == 1.0 for m in modules) and not F.parity_mode()
        if not ok or input.shape[-1] % 32 or sum(m.out_features for m in modules) % 32:
            return [m(input) for m in modules]
        return F.stacked_linear(modules, input, "nvfp4", True)
