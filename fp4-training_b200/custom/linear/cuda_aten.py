"""Unquantized layer through `xops.addmm_cuda` (reference: custom/linear/cuda_aten.py:11-65)."""
import torch
from torch.amp import custom_bwd, custom_fwd

import backend.xops  # noqa: F401

from .custom import CustomLinear, flatten_apply

op = torch.ops.xops


class CudaAtenAddmm(torch.autograd.Function):
    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, X, W, b=None):
        Y = op.addmm_cuda(X, W.T, b)
        ctx.save_for_backward(X, W)
        ctx.has_bias = b is not None
        return Y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_Y):
        X, W = ctx.saved_tensors
        grad_X = grad_W = grad_b = None
        if ctx.needs_input_grad[0]:
            grad_X = op.addmm_cuda(grad_Y, W)
        if ctx.needs_input_grad[1]:
            grad_W = op.addmm_cuda(grad_Y.T, X)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_b = grad_Y.sum(dim=0)
        return grad_X, grad_W, grad_b


class AddmmLinear(CustomLinear):
    def forward(self, input):
        return flatten_apply(self, CudaAtenAddmm.apply, input)
