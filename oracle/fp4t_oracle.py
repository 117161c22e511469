"""CPU oracle for the quantized-linear training path (TEST INFRASTRUCTURE ONLY).

This module restates, on the CPU and in plain torch/numpy arithmetic, what the
reference project computes on the path  quantize(X, W, G) -> fprop / dgrad /
wgrad block-scaled GEMMs.  It exists to check the CUDA kernels; nothing in the
shipped package imports it.  Only tests, the smoke check and the CPU-baseline
leg of the benchmark may call it.

Parity status
-------------
* NVFP4 quantizer, FP4 pack rule and both scale swizzles: PINNED.  The
  reference's own Python (custom/quantize.py, custom/swizzle.py) runs on CPU
  and the fixtures under tests/golden/ were generated from it; see
  tests/golden/make_golden.py and tests/test_oracle_pins.py.
* MXFP8 quantizer: PARITY UNPINNED.  The arithmetic lives in the third-party
  package `microxcaling` (fork vuiseng9/microxcaling, branch return_quantized,
  referenced from .gitmodules:1-4; commit unknown, directory empty).  What is
  restated here is the published OCP Microscaling v1.0 MXFP8 conversion as the
  microxcaling emulation library implements it, driven by the parameters the
  reference passes at custom/quantize.py:8-21.  The details that cannot be
  checked against source are named constants below.

Every function cites the reference file:line it follows.
"""
from __future__ import annotations

import math

import numpy as np
import torch

# ----------------------------------------------------------------------------
# Format tables
# ----------------------------------------------------------------------------

# E2M1 magnitudes by 3-bit code (custom/quantize.py:52-56 names the extremes;
# the grid is the OCP FP4 grid the pack intrinsic targets,
# custom/backend/csrc/cublaslt_mm_nvfp4.cu:113-124).
E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)

E2M1_NORM_MAX = 6.0          # custom/quantize.py:54
E4M3_NORM_MAX = 448.0        # custom/quantize.py:55
E4M3_SUBNORM_MIN = 2.0 ** -9  # custom/quantize.py:56
NVFP4_BLOCK = 16
MXFP8_BLOCK = 32             # custom/quantize.py:10

# MXFP8 details that the missing microxcaling source would settle.
MX_E4M3_EMAX = 8             # largest unbiased exponent of an E4M3 normal (448 = 1.75 * 2^8)
MX_E4M3_MIN_EXP = -6         # smallest normal exponent; below it the grid is 2^-9 (denormals kept)
MX_E4M3_MBITS = 3            # explicit mantissa bits
MX_SCALE_EMAX = 127          # 2^(scale_bits-1) - 1 with scale_bits = 8 (custom/quantize.py:9)
MX_ROUND_HALF_AWAY = True    # 'round': 'nearest' (custom/quantize.py:12): sign(x)*floor(|x|+0.5)
MX_ZERO_BLOCK_AMAX = 2.0 ** -126  # all-zero block: exponent of the smallest fp32 normal, then clamped


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    """4-bit codes (uint8, 0..15) -> fp32 values; bit 3 is the sign."""
    grid = torch.tensor(E2M1_GRID, dtype=torch.float32, device=codes.device)
    mag = grid[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -mag, mag)


def e2m1_encode_rne_sat(y: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit code, round-to-nearest-even onto the E2M1 grid, saturating at 6.

    Semantics of `cvt.rn.satfinite.e2m1x2.f32`, the instruction behind the pack
    kernel at custom/backend/csrc/cublaslt_mm_nvfp4.cu:113-124.  Ties go to the
    even code: .25->0, .75->1, 1.25->1, 1.75->2, 2.5->2, 3.5->4, 5->4.
    The sign bit is the sign bit of the input (so -0.0 -> 0x8).
    """
    a = y.abs()
    mag = ((a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8)
           + (a > 1.25).to(torch.uint8) + (a >= 1.75).to(torch.uint8)
           + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8)
           + (a > 5.0).to(torch.uint8))
    sign = torch.signbit(y).to(torch.uint8) << 3
    return (mag | sign).to(torch.uint8)


def pack_fp4_pairs(codes: torch.Tensor) -> torch.Tensor:
    """[R, C] 4-bit codes -> [R, C/2] bytes; even column in the low nibble.

    custom/backend/csrc/cublaslt_mm_nvfp4.cu:145-166 (pair (c0, c0+1) -> one byte).
    """
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()


def unpack_fp4_pairs(packed: torch.Tensor) -> torch.Tensor:
    out = torch.empty(packed.shape[0], packed.shape[1] * 2, dtype=torch.uint8, device=packed.device)
    out[:, 0::2] = packed & 0xF
    out[:, 1::2] = packed >> 4
    return out


def e4m3_decode(b: torch.Tensor) -> torch.Tensor:
    return b.contiguous().view(torch.float8_e4m3fn).to(torch.float32)


def e8m0_decode(b: torch.Tensor) -> torch.Tensor:
    """Biased-by-127 power-of-two scale byte -> fp32 (custom/quantize.py:32-33)."""
    return torch.pow(2.0, b.to(torch.float32) - 127.0)


# ----------------------------------------------------------------------------
# Scale swizzles
# ----------------------------------------------------------------------------

def swizzled_shape(outer: int, inner: int) -> tuple[int, int]:
    """2-D shape of the swizzled buffer for a logical [outer, inner] scale matrix."""
    return (math.ceil(outer / 128) * 32, math.ceil(inner / 4) * 16)


def swizzle_rowwise(scale: torch.Tensor) -> torch.Tensor:
    """Logical [outer, inner] bytes -> 128x4-tile layout, zero padded.

    custom/swizzle.py:6-23.  Element (o, i) goes to byte
      ((o//128) * ceil(inner/4) + i//4) * 512 + (o%32)*16 + ((o%128)//32)*4 + i%4
    which is the offset rule the reference documents at custom/swizzle.py:103-104.
    Written here as an index scatter so that it does not share code shape with
    the view/transpose formulation it is checked against.
    """
    outer, inner = scale.shape
    nty, ntx = math.ceil(outer / 128), math.ceil(inner / 4)
    flat = torch.zeros(nty * ntx * 512, dtype=scale.dtype)
    o = torch.arange(outer).view(-1, 1).expand(outer, inner)
    i = torch.arange(inner).view(1, -1).expand(outer, inner)
    off = ((o // 128) * ntx + i // 4) * 512 + (o % 32) * 16 + ((o % 128) // 32) * 4 + i % 4
    flat[off.reshape(-1)] = scale.reshape(-1)
    return flat.view(nty * 32, ntx * 16)


def unswizzle_rowwise(sw: torch.Tensor, outer: int, inner: int) -> torch.Tensor:
    ntx = math.ceil(inner / 4)
    o = torch.arange(outer).view(-1, 1).expand(outer, inner)
    i = torch.arange(inner).view(1, -1).expand(outer, inner)
    off = ((o // 128) * ntx + i // 4) * 512 + (o % 32) * 16 + ((o % 128) // 32) * 4 + i % 4
    return sw.reshape(-1)[off.reshape(-1)].view(outer, inner)


def swizzle_colwise_reference_layout(scale: torch.Tensor) -> torch.Tensor:
    """Logical [inner(K-blocks), outer] bytes -> the layout of custom/swizzle.py:43-60.

    Element (ki, o) goes to byte ((ki//4)*32 + o%32) * (ntx*16) + (o//128)*16
    + ((o%128)//32)*4 + ki%4, with ntx = ceil(outer/128).  This equals the
    canonical tile order only while ntx == 1 (outer <= 128).
    """
    inner, outer = scale.shape
    nty, ntx = math.ceil(inner / 4), math.ceil(outer / 128)
    flat = torch.zeros(nty * 32 * ntx * 16, dtype=scale.dtype)
    ki = torch.arange(inner).view(-1, 1).expand(inner, outer)
    o = torch.arange(outer).view(1, -1).expand(inner, outer)
    off = ((ki // 4) * 32 + o % 32) * (ntx * 16) + (o // 128) * 16 + ((o % 128) // 32) * 4 + ki % 4
    flat[off.reshape(-1)] = scale.reshape(-1)
    return flat.view(nty * 32, ntx * 16)


# ----------------------------------------------------------------------------
# NVFP4 quantizer
# ----------------------------------------------------------------------------

def nvfp4_block_scales(x: torch.Tensor) -> torch.Tensor:
    """[R, C] -> fp32 [R, C/16] unrounded block scales (custom/quantize.py:72-76)."""
    r, c = x.shape
    blk = x.to(torch.float32).reshape(r, c // NVFP4_BLOCK, NVFP4_BLOCK)
    amax = blk.abs().amax(dim=-1)
    # a tensor divisor keeps this an IEEE division on every device (CUDA turns division by a
    # Python scalar into a multiply by the reciprocal, which changes the last bit of some scales)
    return (amax / torch.full_like(amax, E2M1_NORM_MAX)).clamp(E4M3_SUBNORM_MIN, E4M3_NORM_MAX)


def nvfp4_quantize_rowwise(x: torch.Tensor, noise: torch.Tensor | None = None):
    """Row-wise NVFP4 (1x16 blocks along the last dim).

    Returns (codes uint8 [R, C] in 0..15, scale bytes uint8 [R, C/16] (E4M3)).

    Deterministic path (noise is None), custom/quantize.py:78-93 followed by the
    pack conversion: code = RNE-saturate-E2M1(x / s32), where the division uses
    the unrounded fp32 scale; sign(0) is 0 in the reference, so an input of
    -0.0 encodes as +0 while a negative value that rounds to zero keeps its
    sign bit.

    Stochastic path (custom/quantize.py:84-89,93): noise holds u ~ U[0,1) with
    the blocked shape [R, C/16, 16] (or anything that reshapes to it);
      e = clamp(floor(log2|y|), 0, 2); m = |y| / 2^e;
      r = rint(2m + (u - 0.5)); q = sign(y) * 2^e * (r / 2)
    then the pack conversion saturates q to +-6.
    The stored scale is float8_e4m3fn(s32) (custom/quantize.py:103).
    """
    r, c = x.shape
    if c % NVFP4_BLOCK:
        raise ValueError("columns must be a multiple of 16")
    x32 = x.to(torch.float32)
    s32 = nvfp4_block_scales(x32).unsqueeze(-1)
    y = x32.reshape(r, c // NVFP4_BLOCK, NVFP4_BLOCK) / s32
    if noise is None:
        y = torch.where(y == 0, torch.zeros_like(y), y)       # sign(+-0) = 0
        codes = e2m1_encode_rne_sat(y)
    else:
        u = noise.to(torch.float32).reshape(y.shape)
        sgn = torch.sign(y)
        a = y.abs()
        # floor(log2(a)) clamped to [0, 2] depends only on a >= 2 and a >= 4.
        e = (a >= 2.0).to(torch.float32) + (a >= 4.0).to(torch.float32)
        p2 = torch.pow(2.0, e)
        m = a / p2
        rr = torch.round(m * 2 + (u - 0.5)) / 2
        q = sgn * p2 * rr
        codes = e2m1_encode_rne_sat(q)
    sbytes = s32.squeeze(-1).to(torch.float8_e4m3fn).view(torch.uint8)
    return codes.reshape(r, c), sbytes


def nvfp4_quantize(x: torch.Tensor, noise_row=None, want_t: bool = False, noise_t=None):
    """What the fused CUDA quantizer emits for one tensor.

    Row-wise: packed codes [R, C/2] + swizzled scales of logical [R, C/16].
    Transposed (want_t): the same for x.T, i.e. packed [C, R/2] + swizzled
    scales of logical [C, R/16] -- the operand the reference builds with
    `.T.contiguous()` before quantizing (custom/linear/nvfp4.py:59,74-75).
    """
    codes, sb = nvfp4_quantize_rowwise(x, noise_row)
    out = {"codes": pack_fp4_pairs(codes), "sf": swizzle_rowwise(sb), "sf_logical": sb}
    if want_t:
        ct, sbt = nvfp4_quantize_rowwise(x.t().contiguous(), noise_t)
        out.update({"codes_t": pack_fp4_pairs(ct), "sf_t": swizzle_rowwise(sbt), "sf_t_logical": sbt})
    return out


def hadamard16_blocks(x: torch.Tensor, sign_mask: int) -> torch.Tensor:
    """Random Hadamard transform of every 16-element block along the last dim: element j of a
    block is negated when bit j of sign_mask is set, then the Sylvester-ordered 16-point
    Walsh-Hadamard butterflies run with strides 1, 2, 4, 8 (pairs (j, j+h) -> (a+b, a-b), fp32),
    then the block is multiplied by 1/4 (H16 / 4 is orthogonal).  This recipe step is not in
    the reference (its README lists it under features to add); the definition is this
    framework's own and the CUDA quantizer follows it operation for operation."""
    r, c = x.shape
    v = x.to(torch.float32).reshape(r, c // 16, 16).clone()
    signs = torch.tensor([-1.0 if (sign_mask >> j) & 1 else 1.0 for j in range(16)], dtype=torch.float32,
                         device=x.device)
    v = v * signs
    for h in (1, 2, 4, 8):
        w = v.reshape(r, c // 16, 16 // (2 * h), 2, h)
        a, b = w[..., 0, :], w[..., 1, :]
        v = torch.stack((a + b, a - b), dim=-2).reshape(r, c // 16, 16)
    return (v * 0.25).reshape(r, c)


def nvfp4_quantize_scaled(x: torch.Tensor, tensor_scale: float, want_t: bool = False, rht_signs=None):
    """Two-level NVFP4: the block quantization of fp32(x) * tensor_scale (round-to-nearest),
    optionally with the 16-block Hadamard transform in front of it.  Same outputs as
    nvfp4_quantize.  Not in the reference (one scale level, custom/quantize.py:72-76)."""
    def prep(t):
        t = t.to(torch.float32) * torch.full((), tensor_scale, dtype=torch.float32, device=t.device)
        return hadamard16_blocks(t, rht_signs) if rht_signs is not None else t
    codes, sb = nvfp4_quantize_rowwise(prep(x))
    out = {"codes": pack_fp4_pairs(codes), "sf": swizzle_rowwise(sb), "sf_logical": sb}
    if want_t:
        ct, sbt = nvfp4_quantize_rowwise(prep(x.t().contiguous()))
        out.update({"codes_t": pack_fp4_pairs(ct), "sf_t": swizzle_rowwise(sbt), "sf_t_logical": sbt})
    return out


def nvfp4_dequant(codes: torch.Tensor, sbytes: torch.Tensor) -> torch.Tensor:
    """Unpacked codes [R, C] + logical E4M3 scale bytes [R, C/16] -> fp32 [R, C]."""
    v = e2m1_decode(codes)
    s = e4m3_decode(sbytes).repeat_interleave(NVFP4_BLOCK, dim=1)
    return v * s


# ----------------------------------------------------------------------------
# MXFP8 quantizer (parity unpinned, see module docstring)
# ----------------------------------------------------------------------------

def _floor_log2(a: torch.Tensor) -> torch.Tensor:
    """Exact floor(log2(a)) for positive finite fp32 via frexp (no libm rounding)."""
    _, e = torch.frexp(a)
    return (e - 1).to(torch.float32)


def mxfp8_quantize_rowwise(x: torch.Tensor):
    """1x32 blocks along the last dim -> (E4M3 bytes [R, C], E8M0 bytes [R, C/32]).

    Follows the call at custom/quantize.py:20,28-33 into microxcaling's
    quantize_mx_op with the spec at custom/quantize.py:8-15:
      shared_exp = floor(log2(block amax)) - emax(E4M3), clamped to +-127;
      elements are divided by 2^shared_exp, rounded to 3 mantissa bits
      (half away from zero), denormals kept down to 2^-9, clamped to +-448;
      scale byte = shared_exp + 127.
    """
    r, c = x.shape
    if c % MXFP8_BLOCK:
        raise ValueError("columns must be a multiple of 32")
    x32 = x.to(torch.float32).reshape(r, c // MXFP8_BLOCK, MXFP8_BLOCK)
    amax = x32.abs().amax(dim=-1, keepdim=True)
    amax = torch.where(amax == 0, torch.full_like(amax, MX_ZERO_BLOCK_AMAX), amax)
    sexp = _floor_log2(amax) - MX_E4M3_EMAX
    sexp = sexp.clamp(min=-MX_SCALE_EMAX, max=MX_SCALE_EMAX)
    y = x32 / torch.pow(2.0, sexp)
    a = y.abs()
    pe = _floor_log2(torch.where(a == 0, torch.ones_like(a), a)).clamp(min=MX_E4M3_MIN_EXP)
    t = a / torch.pow(2.0, pe) * (2.0 ** MX_E4M3_MBITS)
    if MX_ROUND_HALF_AWAY:
        t = torch.floor(t + 0.5)
    else:
        t = torch.round(t)
    q = (t / (2.0 ** MX_E4M3_MBITS) * torch.pow(2.0, pe)).clamp(max=E4M3_NORM_MAX)
    q = torch.where(y < 0, -q, q)                 # sign(0) = 0, so -0.0 encodes as +0
    codes = q.reshape(r, c).to(torch.float8_e4m3fn).view(torch.uint8)
    sbytes = (sexp.squeeze(-1) + 127.0).to(torch.uint8)
    return codes, sbytes


def mxfp8_quantize(x: torch.Tensor, want_t: bool = False):
    codes, sb = mxfp8_quantize_rowwise(x)
    out = {"codes": codes, "sf": swizzle_rowwise(sb), "sf_logical": sb}
    if want_t:
        ct, sbt = mxfp8_quantize_rowwise(x.t().contiguous())
        out.update({"codes_t": ct, "sf_t": swizzle_rowwise(sbt), "sf_t_logical": sbt})
    return out


def mxfp8_dequant(codes: torch.Tensor, sbytes: torch.Tensor) -> torch.Tensor:
    v = e4m3_decode(codes)
    return v * e8m0_decode(sbytes).repeat_interleave(MXFP8_BLOCK, dim=1)


def mxfp8_fake_quant(x: torch.Tensor, axis: int = -1) -> torch.Tensor:
    """quantize -> dequantize in the input dtype (custom/quantize.py:17-18)."""
    if axis in (-2, 0):
        return mxfp8_fake_quant(x.t().contiguous(), -1).t()
    codes, sb = mxfp8_quantize_rowwise(x)
    return mxfp8_dequant(codes, sb).to(x.dtype)


# ----------------------------------------------------------------------------
# GEMM oracle
# ----------------------------------------------------------------------------

def gemm_dequant_fp32(p_deq: torch.Tensor, q_deq: torch.Tensor, bias: torch.Tensor | None = None,
                      double: bool = False) -> torch.Tensor:
    """D[rows, cols] = P[rows, K] @ Q[cols, K]^T (+ bias[cols]) on dequantized operands.

    The contraction of custom/backend/csrc/cublaslt_mm_nvfp4.cu:426-436 (and the
    MXFP8 twin at cublaslt_mm_mxfp8.cu:298-308) with P = the reference's B
    argument and Q = its A argument; the bias is rounded to bf16 first as the
    binding does at cublaslt_mm_nvfp4.cu:260-262.
    """
    dt = torch.float64 if double else torch.float32
    d = p_deq.to(dt) @ q_deq.to(dt).t()
    if bias is not None:
        d = d + bias.to(torch.bfloat16).to(dt)
    return d


def rel_frobenius(a: torch.Tensor, ref: torch.Tensor) -> float:
    a = a.detach().double()
    ref = ref.detach().double()
    return float((a - ref).norm() / ref.norm().clamp_min(1e-300))


# ----------------------------------------------------------------------------
# CPU baselines (timed by the benchmark's cpu_baseline / reference arm)
# ----------------------------------------------------------------------------

def fake_mxfp8_linear_fwd_bwd(x: torch.Tensor, w: torch.Tensor, g: torch.Tensor, b=None):
    """MXFP8 fake-quantized linear, forward + backward, on whatever device x is on.

    custom/linear/fake_mxfp8.py:16-59: Y = fq_row(W) fq_row(X)^T (transposed back)
    + b; dX = fq_row(G) fq_col(W); dW = fq_col(G)^T fq_col(X); db = G.sum(0).
    """
    fqx = mxfp8_fake_quant(x, -1)
    fqw = mxfp8_fake_quant(w, -1)
    y = torch.matmul(fqw, fqx.t()).t()
    if b is not None:
        y = y + b
    dx = torch.matmul(mxfp8_fake_quant(g, -1), mxfp8_fake_quant(w, -2))
    dw = torch.matmul(mxfp8_fake_quant(g, -2).t(), mxfp8_fake_quant(x, -2))
    db = g.sum(dim=0) if b is not None else None
    return y, dx, dw, db


def nvfp4_linear_fwd_bwd(x, w, g, b=None, noise_g=None, noise_gt=None):
    """NVFP4 linear fwd+bwd on dequantized operands (custom/linear/nvfp4.py:25-90)."""
    def deq(t, noise=None):
        c, s = nvfp4_quantize_rowwise(t, noise)
        return nvfp4_dequant(c, s)
    y = gemm_dequant_fp32(deq(x), deq(w), b)
    dx = gemm_dequant_fp32(deq(g, noise_g), deq(w.t().contiguous()))
    dw = gemm_dequant_fp32(deq(g.t().contiguous(), noise_gt), deq(x.t().contiguous()))
    db = g.float().sum(dim=0) if b is not None else None
    return y, dx, dw, db


class OracleNvfp4Linear(torch.autograd.Function):
    """The reference recipe of custom/linear/nvfp4.py:25-90 as plain torch arithmetic on
    dequantized operands, on whatever device the tensors live: every operand goes through the
    restated quantizer, stochastic rounding (dgrad operand first, then wgrad operand, as the
    reference draws them) uses torch.rand on that device, GEMMs are fp32 matmuls whose result
    is rounded to the input dtype.  Used by tests to check that training with the CUDA
    kernels follows the same loss curve."""

    @staticmethod
    def forward(ctx, x, w, b):
        dt = x.dtype
        xq = x.to(torch.bfloat16) if dt != torch.float32 else x
        ctx.save_for_backward(x, w)
        ctx.has_bias = b is not None

        def deq(t, noise=None):
            c, s = nvfp4_quantize_rowwise(t, noise)
            return nvfp4_dequant(c, s)
        y = deq(xq) @ deq(w.to(xq.dtype)).t()
        if b is not None:
            y = y + b.to(torch.bfloat16).float()
        return y.to(dt)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        g = g.contiguous()

        def deq(t, noise=None):
            c, s = nvfp4_quantize_rowwise(t, noise)
            return nvfp4_dequant(c, s)
        n, oc = g.shape
        u = torch.rand(n, oc // 16, 16, device=g.device)
        ut = torch.rand(oc, n // 16, 16, device=g.device)
        dx = deq(g, u) @ deq(w.to(g.dtype).t().contiguous()).t()
        dw = deq(g.t().contiguous(), ut) @ deq(x.to(g.dtype).t().contiguous()).t()
        db = g.sum(dim=0) if ctx.has_bias else None
        return dx.to(g.dtype), dw.to(g.dtype), db


# ----------------------------------------------------------------------------
# Synthetic workloads (shapes and distributions of the benchmark configurations)
# ----------------------------------------------------------------------------

def make_linear_inputs(n: int, ic: int, oc: int, seed: int = 0, outliers: bool = True,
                       device: str = "cpu"):
    """X ~ N(0,1) with 0.1 % of entries x50, W ~ N(0, 0.02), G ~ N(0, 1e-3), all bf16."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(n, ic, generator=gen)
    if outliers:
        mask = torch.rand(n, ic, generator=gen) < 1e-3
        x = torch.where(mask, x * 50.0, x)
    w = torch.randn(oc, ic, generator=gen) * 0.02
    g = torch.randn(n, oc, generator=gen) * 1e-3
    return (x.to(torch.bfloat16).to(device), w.to(torch.bfloat16).to(device),
            g.to(torch.bfloat16).to(device))


def as_numpy_u8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).cpu().numpy()
