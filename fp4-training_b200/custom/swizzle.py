"""Scale-factor swizzles with the reference's names (custom/swizzle.py:6-77), on the GPU.

swizzle_rowwise_scale: logical [outer, kblocks] -> the 128x4 tile layout, zero padded,
returned as a 2-D [ceil(outer/128)*32, ceil(kblocks/4)*16] tensor.
swizzle_colwise_scale: logical [kblocks, outer] -> the reference's column-wise layout
(custom/swizzle.py:43-60), returned as [ceil(kblocks/4)*32, ceil(outer/128)*16]; it equals
the tile layout only while outer <= 128, exactly as in the reference.
"""
import torch

from backend import ops as _ops


def _as_bytes(scale_mat: torch.Tensor):
    if scale_mat.ndim != 2:
        raise ValueError("scale matrix must be 2D")
    if scale_mat.element_size() != 1:
        raise ValueError("scale matrix must have a one-byte dtype (uint8, float8_e4m3fn, float8_e8m0fnu)")
    return scale_mat.contiguous().view(torch.uint8), scale_mat.dtype


def swizzle_rowwise_scale(scale_mat: torch.Tensor) -> torch.Tensor:
    b, dt = _as_bytes(scale_mat)
    return _ops.swizzle_rowwise(b).view(dt)


def swizzle_colwise_scale(scale_mat: torch.Tensor) -> torch.Tensor:
    b, dt = _as_bytes(scale_mat)
    return _ops.swizzle_colwise(b).view(dt)
