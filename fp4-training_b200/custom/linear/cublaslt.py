"""Unquantized bf16/fp32 layer through `xops.cublaslt_mm_fp32_or_bf16` and the `TransAB`
layout enum the quantized layers share (reference: custom/linear/cublaslt.py:14-73)."""
from enum import IntEnum

import torch
from torch.amp import custom_bwd, custom_fwd

import backend.xops  # noqa: F401

from .custom import CustomLinear, flatten_apply

op = torch.ops.xops


class TransAB(IntEnum):
    TN = 0
    NN = 1
    NT = 2


class CublasltMMFunc(torch.autograd.Function):
    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, X, W, b=None):
        Y = op.cublaslt_mm_fp32_or_bf16(TransAB.TN, W, X, b)
        ctx.save_for_backward(X, W)
        ctx.has_bias = b is not None
        return Y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_Y):
        X, W = ctx.saved_tensors
        grad_Y = grad_Y.contiguous()
        grad_X = grad_W = grad_b = None
        if ctx.needs_input_grad[0]:
            grad_X = op.cublaslt_mm_fp32_or_bf16(TransAB.NN, W, grad_Y, None)
        if ctx.needs_input_grad[1]:
            grad_W = op.cublaslt_mm_fp32_or_bf16(TransAB.NT, X, grad_Y, None)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_b = grad_Y.sum(dim=0)
        return grad_X, grad_W, grad_b


class CublasltLinear(CustomLinear):
    def forward(self, input):
        return flatten_apply(self, CublasltMMFunc.apply, input)
