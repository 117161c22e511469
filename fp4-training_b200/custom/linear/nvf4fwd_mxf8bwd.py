"""Hybrid recipe: NVFP4 forward GEMM, MXFP8 backward GEMMs
(reference: custom/linear/nvf4fwd_mxf8bwd.py:17-117)."""
from collections import OrderedDict

import torch
from torch.amp import custom_bwd, custom_fwd

import backend.xops  # noqa: F401

from ..quantize import q_mxfp8_colwise, q_mxfp8_rowwise, q_nvfp4_rowwise
from . import _fused as F
from .cublaslt import TransAB
from .custom import CustomLinear, flatten_apply
from .mxfp8 import mxfp8_backward, mxfp8_backward_unfused

op = torch.ops.xops

STOCK = OrderedDict([
    ('1A', q_nvfp4_rowwise), ('1B', q_nvfp4_rowwise),
    ('2A', q_mxfp8_colwise), ('2B', q_mxfp8_rowwise),
    ('3A', q_mxfp8_colwise), ('3B', q_mxfp8_colwise),
])


class FwdNvfp4BwdMxfp8Matmul(torch.autograd.Function):
    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, X, W, b, quant: OrderedDict):
        ctx.quant = quant
        ctx.has_bias = b is not None
        ctx.fused = F.is_stock(quant, STOCK)
        if not ctx.fused:
            Wq, sW = quant['1A'](W)
            Xq, sX = quant['1B'](X)
            Y, _ = op.cublaslt_mm_nvfp4(TransAB.TN.value, X.dtype, Wq, sW, Xq, sX, b)
        else:
            if X.ndim != 2 or W.ndim != 2:
                raise ValueError("Input tensor must be 2D for nvfp4 quantization")
            X = X.contiguous()
            Wc, Wsf, _, _ = F.quant_pair("nvfp4", W, True, False)
            Xc, Xsf, _, _ = F.quant_pair("nvfp4", X, True, False)
            Y = F.gemm("nvfp4", Xc, Xsf, Wc, Wsf, b, X.dtype)
        ctx.save_for_backward(X, W)
        return Y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_Y):
        X, W = ctx.saved_tensors
        grad_Y = grad_Y.contiguous()
        if not ctx.fused:
            grad_X, grad_W = mxfp8_backward_unfused(ctx, grad_Y, X, W)
            grad_b = grad_Y.sum(dim=0) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        else:
            grad_X, grad_W, grad_b = mxfp8_backward(ctx, grad_Y, W, X, None, None)
        return grad_X, grad_W, grad_b, None


class CublasltFwdNvfp4BwdMxfp8Linear(CustomLinear):
    """`nn.Linear` drop-in: NVFP4 fprop, MXFP8 dgrad and wgrad."""

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
        return flatten_apply(self, FwdNvfp4BwdMxfp8Matmul.apply, input, self.quantizers)
