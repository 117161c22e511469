"""LayerNorm for the blocks whose projections are quantized: `nn.LayerNorm` with the same
parameters and state dict, computed by the library's kernels.

In the reference the `preln` modules are `nn.LayerNorm` (models/transformer_block.py:45-52,
89-93); under bf16 autocast they return fp32, and each projection that follows casts that to
bf16 again.  Here the forward kernel reads the (fp32) residual stream once and writes the
normalised rows directly in the dtype the projections consume, and the backward kernel produces
the input gradient and the weight / bias gradients in one pass over the rows."""
from __future__ import annotations

import torch
from torch import nn

from backend import ops as _ops


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_dtype):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        y, mean, rstd = _ops.layernorm_forward(x2, weight, bias, eps, out_dtype)
        ctx.save_for_backward(x2, mean, rstd, weight)
        ctx.shape = shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, mean, rstd, weight = ctx.saved_tensors
        dx, dgamma, dbeta = _ops.layernorm_backward(dy.reshape(x2.shape), x2, mean, rstd, weight)
        return dx.view(ctx.shape), dgamma.to(weight.dtype), dbeta.to(weight.dtype), None, None


class FusedLayerNorm(nn.LayerNorm):
    """`nn.LayerNorm(normalized_shape=E)` drop-in (elementwise affine with bias, last dimension
    only, E a multiple of 4 up to 1024).  Under autocast the output has the autocast dtype --
    what the projection behind it would cast to anyway -- otherwise the input's dtype."""

    def __init__(self, normalized_shape, eps: float = 1e-5, **kwargs):
        super().__init__(normalized_shape, eps=eps, elementwise_affine=True, bias=True, **kwargs)
        if len(self.normalized_shape) != 1:
            raise ValueError("FusedLayerNorm normalizes the last dimension only")

    def forward(self, x):
        if x.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("FusedLayerNorm takes float32 or bfloat16 input")
        out_dtype = x.dtype
        if x.is_cuda and torch.is_autocast_enabled("cuda"):
            ac = torch.get_autocast_dtype("cuda")
            if ac in (torch.float32, torch.bfloat16):
                out_dtype = ac
        return _LayerNormFn.apply(x, self.weight, self.bias, self.eps, out_dtype)
