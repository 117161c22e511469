"""Quantizer entry points with the reference's names and return conventions
(custom/quantize.py:8-122), served by the fused CUDA quantizers.

  q_nvfp4_rowwise(t, sr=False) -> (fp32 E2M1-valued [R, C], swizzled UE4M3 scales uint8)
  q_nvfp4_colwise(t, sr=False) -> (fp32 E2M1-valued [R, C], scales in the reference's column-wise layout)
  q_mxfp8_rowwise(t)           -> (E4M3 codes uint8 [R, C], swizzled UE8M0 scales uint8)
  q_mxfp8_colwise(t)           -> (E4M3 codes uint8 [R, C], scales in the reference's column-wise layout)
  quantize_nvfp4(t, rowwise, simulated, stochastic_rounding), fq_mxfp8_rowwise/colwise

The `*_fused` functions return the packed / transposed operand forms the Linear modules
feed straight to the GEMMs.  Stochastic rounding draws `torch.rand` with the blocked shape
the reference uses (custom/quantize.py:88), so a seeded run consumes the generator in the
same order; the quantized values are bit-identical given the same noise, except that a
value the reference leaves at 8 (to be clipped to 6 by its pack kernel) is returned as 6.
"""
from __future__ import annotations

import torch

from backend import ops as _ops

mxfp8_spec = {
    'scale_bits': 8,
    'block_size': 32,
    'shared_exp_method': 'max',
    'round': 'nearest',
    'mx_flush_fp32_subnorms': False,
    'custom_cuda': True,   # the quantizer is a CUDA kernel of this package
}

E2_MAX = 2
E2_MIN = 0
E2M1_NORM_MAX = 6.0
E4M3_NORM_MAX = 448.0
E4M3_SUBNORM_MIN = 2 ** -9


_seed_state = {"base": None, "count": 0}


def _next_seed() -> int:
    """Seed of the next in-kernel noise stream: torch's initial seed mixed with a call counter
    (splitmix64), so `torch.manual_seed` makes runs repeatable without a device round trip."""
    base = torch.initial_seed()
    if _seed_state["base"] != base:
        _seed_state["base"], _seed_state["count"] = base, 0
    _seed_state["count"] += 1
    z = (base + 0x9E3779B97F4A7C15 * _seed_state["count"]) & (2 ** 64 - 1)
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & (2 ** 64 - 1)
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & (2 ** 64 - 1)
    return z ^ (z >> 31)


def _check_2d(tensor, what):
    if tensor.ndim != 2:
        raise ValueError(f"Input tensor must be 2D for {what} quantization")


# ------------------------------------------------------------------ NVFP4
def nvfp4_fused(tensor, want_row=True, want_t=False, sr=False, seed=None, noise=None, noise_t=None,
                bias_grad_dtype=None):
    """-> (codes [R, C/2], sf, codes_t [C, R/2], sf_t) as uint8 tensors (None where not requested).

    sr=True with explicit noise tensors is the bit-exact parity mode; without them the
    kernel generates its own uniform noise from `seed`.  bias_grad_dtype adds a fifth result:
    the column sums of `tensor` (the bias gradient when `tensor` is dY), taken in the same pass."""
    _check_2d(tensor, "nvfp4")
    if not sr:
        mode = _ops.SR_NONE
    elif noise is not None or noise_t is not None:
        mode = _ops.SR_NOISE
    else:
        mode = _ops.SR_HASH
        if seed is None:
            seed = _next_seed()
    return _ops.quantize_nvfp4(tensor, want_row, want_t, mode, noise, noise_t, seed or 0, bias_grad_dtype)


def quantize_nvfp4(tensor, rowwise=True, simulated=True, stochastic_rounding=False):
    """custom/quantize.py:57-106.  simulated=True returns the dequantized tensor (fp32);
    otherwise (E2M1-valued fp32 tensor, float8_e4m3fn logical scales)."""
    tensor = tensor.to(torch.float32)
    _check_2d(tensor, "nvfp4")
    r, c = tensor.shape
    if rowwise is True and c % 16 != 0:
        raise ValueError("For nvfp4 row-wise quantization, the number of columns must be a multiple of 16")
    if rowwise is False and r % 16 != 0:
        raise ValueError("For nvfp4 column-wise quantization, the number of rows must be a multiple of 16")
    src = tensor if rowwise else tensor.T.contiguous()
    noise = _sr_noise(r, c, rowwise, tensor.device) if stochastic_rounding else None
    codes, sf, _, _ = nvfp4_fused(src, True, False, sr=stochastic_rounding, noise=noise)
    q = _ops.unpack_e2m1(codes)
    scales = unswizzle_rowwise(sf, src.shape[0], src.shape[1] // 16).view(torch.float8_e4m3fn)
    if simulated:
        # the reference multiplies by the fp32 scale BEFORE its rounding to E4M3
        # (custom/quantize.py:75-76,96-97): recompute it from the block maxima
        amax = src.reshape(src.shape[0], -1, 16).abs().amax(dim=-1)
        # a tensor divisor: on CUDA, division by a Python scalar becomes a multiply by 1/6
        s32 = (amax / torch.full_like(amax, E2M1_NORM_MAX)).clamp(E4M3_SUBNORM_MIN, E4M3_NORM_MAX)
        out = q * s32.repeat_interleave(16, dim=1)
        return out if rowwise else out.T
    scales = scales.squeeze()
    if rowwise:
        return q, scales
    return q.T, scales.T


def _sr_noise(r: int, c: int, rowwise: bool, device) -> torch.Tensor:
    """Uniform noise for a [r, c] input in the order the reference consumes its generator
    (custom/quantize.py:88): row-wise one draw per element of the blocked [r, c/16, 16] tensor;
    column-wise the reference's blocked tensor is a strided view of the transposed input and
    `rand_like` fills it in memory order, i.e. in the layout of the original [r, c] tensor.
    Returned in the logical layout of the tensor that is quantized row-wise."""
    if rowwise:
        return torch.rand(r, c // 16, 16, device=device)
    return torch.rand(r, c, device=device).T.contiguous()


def unswizzle_rowwise(sf: torch.Tensor, outer: int, inner: int) -> torch.Tensor:
    """Tile layout -> logical [outer, inner] bytes (a gather; used by the value-returning API only)."""
    ntx = (inner + 3) // 4
    o = torch.arange(outer, device=sf.device).view(-1, 1)
    i = torch.arange(inner, device=sf.device).view(1, -1)
    off = ((o // 128) * ntx + i // 4) * 512 + (o % 32) * 16 + ((o % 128) // 32) * 4 + i % 4
    return sf.reshape(-1)[off]


def q_nvfp4_rowwise(tensor, sr=False):
    """custom/quantize.py:108-114."""
    _check_2d(tensor, "nvfp4")
    if tensor.shape[1] % 16 != 0:
        raise ValueError("For nvfp4 row-wise quantization, the number of columns must be a multiple of 16")
    noise = _sr_noise(tensor.shape[0], tensor.shape[1], True, tensor.device) if sr else None
    codes, sf, _, _ = nvfp4_fused(tensor, True, False, sr=sr, noise=noise)
    return _ops.unpack_e2m1(codes), sf


def q_nvfp4_colwise(tensor, sr=False):
    """custom/quantize.py:116-122: blocks of 16 along dim 0; values keep the input's shape."""
    _check_2d(tensor, "nvfp4")
    r, c = tensor.shape
    if r % 16 != 0:
        raise ValueError("For nvfp4 column-wise quantization, the number of rows must be a multiple of 16")
    t = tensor.T.contiguous()
    noise = _sr_noise(r, c, False, tensor.device) if sr else None
    codes, sf, _, _ = nvfp4_fused(t, True, False, sr=sr, noise=noise)
    from .swizzle import swizzle_colwise_scale
    logical = unswizzle_rowwise(sf, c, r // 16)            # [C, R/16]
    return _ops.unpack_e2m1(codes).T.contiguous(), swizzle_colwise_scale(logical.T.contiguous())


# ------------------------------------------------------------------ MXFP8
def mxfp8_fused(tensor, want_row=True, want_t=False, bias_grad_dtype=None):
    """-> (codes [R, C], sf, codes_t [C, R], sf_t) as uint8 tensors (None where not requested);
    with bias_grad_dtype also the column sums of `tensor`."""
    _check_2d(tensor, "mxfp8")
    return _ops.quantize_mxfp8(tensor, want_row, want_t, bias_grad_dtype)


def q_mxfp8_rowwise(tensor):
    """custom/quantize.py:23-35."""
    _check_2d(tensor, "mxfp8")
    codes, sf, _, _ = mxfp8_fused(tensor, True, False)
    return codes, sf


def q_mxfp8_colwise(tensor):
    """custom/quantize.py:37-49: blocks of 32 along dim 0; codes keep the input's shape and the
    scales come in the reference's column-wise layout."""
    _check_2d(tensor, "mxfp8")
    r, c = tensor.shape
    if r % 32:
        raise ValueError("column-wise mxfp8 quantization needs rows to be a multiple of 32")
    _, _, codes_t, sf_t = mxfp8_fused(tensor, False, True)
    from .swizzle import swizzle_colwise_scale
    logical = unswizzle_rowwise(sf_t, c, r // 32)           # [C, R/32]
    return _ops.transpose_bytes(codes_t), swizzle_colwise_scale(logical.T.contiguous())


def _fq_mxfp8(tensor, axis):
    if tensor.ndim != 2:
        tensor2 = tensor.reshape(-1, tensor.shape[-1])
    else:
        tensor2 = tensor
    src = tensor2 if axis == -1 else tensor2.T.contiguous()
    codes, sf, _, _ = mxfp8_fused(src, True, False)
    scale = torch.pow(2.0, unswizzle_rowwise(sf, src.shape[0], src.shape[1] // 32).to(torch.float32) - 127.0)
    deq = codes.view(torch.float8_e4m3fn).to(torch.float32) * scale.repeat_interleave(32, dim=1)
    deq = deq if axis == -1 else deq.T
    return deq.to(tensor.dtype).reshape(tensor.shape)


def fq_mxfp8_rowwise(tensor):
    """Fake quantization along the last dim (custom/quantize.py:17)."""
    return _fq_mxfp8(tensor, -1)


def fq_mxfp8_colwise(tensor):
    """Fake quantization along dim -2 (custom/quantize.py:18)."""
    return _fq_mxfp8(tensor, -2)
