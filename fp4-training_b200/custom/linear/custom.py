"""`CustomLinear`: the `nn.Linear` subclass every quantized layer derives from, and the
plain three-GEMM autograd function (reference: custom/linear/custom.py:12-109)."""
import math

import torch
from torch.amp import custom_bwd, custom_fwd

import backend.xops  # noqa: F401  (registers torch.ops.xops)

op = torch.ops.xops


class CustomMatMul(torch.autograd.Function):
    """fprop Y = X W^T (+b), dgrad dX = dY W, wgrad dW = dY^T X, written with torch matmuls
    (custom/linear/custom.py:12-59)."""

    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, X, W, b=None):
        if X.ndim != 2 or W.ndim != 2:
            raise ValueError("Expected 2D inputs")
        Y = torch.addmm(b, X, W.T) if b is not None else torch.mm(X, W.T)
        ctx.save_for_backward(X, W)
        ctx.has_bias = b is not None
        return Y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_Y):
        X, W = ctx.saved_tensors
        grad_X = grad_W = grad_b = None
        if ctx.needs_input_grad[0]:
            grad_X = torch.mm(grad_Y, W)
        if ctx.needs_input_grad[1]:
            grad_W = torch.mm(grad_Y.T, X)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_b = grad_Y.sum(dim=0)
        return grad_X, grad_W, grad_b


def flatten_apply(module, fn, input, *extra):
    """N-D input -> 2-D [-1, in_features] view, apply, restore the leading dims
    (custom/linear/custom.py:96-105)."""
    shapes = None
    if input.ndim > 2:
        shapes = input.shape
        input = input.view(-1, shapes[-1])
    out = fn(input, module.weight, module.bias, *extra)
    if shapes is not None:
        out = out.view(shapes[:-1] + (module.out_features,))
    return out


class CustomLinear(torch.nn.Linear):
    """Same constructor and parameters as `nn.Linear`; weights start as N(0, 0.023)
    (custom/linear/custom.py:62-109)."""

    def reset_parameters(self):
        torch.nn.init.normal_(self.weight, mean=0.0, std=0.023)
        if self.bias is not None:
            fan_in, _ = torch.nn.init._calculate_fan_in_and_fan_out(self.weight)
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            torch.nn.init.uniform_(self.bias, -bound, bound)

    @classmethod
    def from_linear(cls, linear_layer):
        """Wrap an existing `nn.Linear`, sharing (not copying) its parameters."""
        obj = cls.__new__(cls)
        torch.nn.Module.__init__(obj)
        obj.in_features = linear_layer.in_features
        obj.out_features = linear_layer.out_features
        obj.register_parameter('weight', linear_layer.weight)
        obj.register_parameter('bias', linear_layer.bias)
        return obj

    def forward(self, input):
        return flatten_apply(self, CustomMatMul.apply, input)

    def extra_repr(self) -> str:
        return f"IC={self.in_features}, OC={self.out_features}, b={'True' if self.bias is not None else 'False'}"
