"""`torch.ops.xops`: the operator schema of the reference extension, served by fp4t.

Importing this module defines the four operators of the reference's
custom/backend/csrc/xops.cpp:15-20 with identical schema strings and registers CUDA
implementations only, so CPU tensors raise NotImplementedError from the dispatcher as
they do in the reference.

  cublaslt_mm_nvfp4 / cublaslt_mm_mxfp8   -> hand-written tcgen05 block-scaled GEMMs
  addmm_cuda / cublaslt_mm_fp32_or_bf16   -> unquantized teaching steps; thin ATen calls
"""
from __future__ import annotations

import torch

from . import ops

TN, NN, NT = 0, 1, 2

_lib_def = torch.library.Library("xops", "DEF")
_lib_def.define("addmm_cuda(Tensor a, Tensor b, Tensor? c=None) -> Tensor")
_lib_def.define("cublaslt_mm_fp32_or_bf16(int gemm_id, Tensor A, Tensor B, Tensor? b=None) -> Tensor")
_lib_def.define("cublaslt_mm_mxfp8(int gemm_id, ScalarType DoutType, Tensor A, Tensor scaleA, Tensor B, "
                "Tensor scaleB, Tensor? b=None) -> (Tensor Dt, Tensor scaleDout)")
_lib_def.define("cublaslt_mm_nvfp4(int gemm_id, ScalarType DoutType, Tensor A, Tensor scaleA, Tensor B, "
                "Tensor scaleB, Tensor? b=None) -> (Tensor Dt, Tensor scaleDout)")
_lib_impl = torch.library.Library("xops", "IMPL", "CUDA")


def _check_mode(mode: int):
    if mode not in (TN, NN, NT):
        raise IndexError("invalid mode (expected 0,1,2)")


def _check_common(A, scaleA, B, scaleB):
    for t, n in ((A, "A"), (B, "B"), (scaleA, "scaleA"), (scaleB, "scaleB")):
        if t.ndim != 2:
            raise RuntimeError(f"{n} must be 2D")
        if not t.is_contiguous():
            raise RuntimeError(f"{n} must be contiguous")
    if not (A.device == B.device == scaleA.device == scaleB.device):
        raise RuntimeError("A, B, scaleA and scaleB must be on the same CUDA device")
    if scaleA.dtype != torch.uint8 or scaleB.dtype != torch.uint8:
        raise RuntimeError("Only supports torch.uint8 for scaleA / scaleB")


def _check_dout(dt):
    if dt not in (torch.float32, torch.bfloat16, torch.uint8):
        raise RuntimeError("Only torch.float32, torch.bfloat16 and torch.uint8 (block-quantized output) are "
                           f"supported for Dout; but found {dt}")


def _qout(fmt, out_fmt, p, p_sf, q, q_sf, bias, m, n):
    """Dout = uint8: the output leaves as block-quantized codes with its own scales
    (custom/backend/csrc/cublaslt_mm_mxfp8.cu:155-161,247-253; the NVFP4 counterpart is a TODO at
    cublaslt_mm_nvfp4.cu:241-247).  scaleDout holds the tile-layout bytes; it is returned with the
    2-D shape the reference allocates, [roundoff(m / block, 4), roundoff(n, 128)]."""
    blk = 32 if out_fmt == "mxfp8" else 16
    if m % 32:
        raise RuntimeError("When Dout is FP8/FP4 (stored as uint8), batch size m must be a multiple of 32; "
                           f"got m={m}.")
    codes, sf = ops.gemm_qout(fmt, p, p_sf, q, q_sf, bias, out_fmt)
    return codes, sf.reshape((m // blk + 3) // 4 * 4, (n + 127) // 128 * 128)


def _addmm_cuda(a, b, c=None):
    """custom/backend/csrc/aten_mm.cpp:12-46."""
    if a.dtype not in (torch.float32, torch.bfloat16) or b.dtype != a.dtype:
        raise RuntimeError("a and b must share the same dtype (float32 or bfloat16)")
    if a.ndim != 2 or b.ndim != 2 or a.shape[1] != b.shape[0]:
        raise RuntimeError("matmul inner dims must match")
    if c is not None:
        if c.ndim != 1 or c.shape[0] != b.shape[1] or c.dtype != a.dtype:
            raise RuntimeError(f"c must be 1D of length {b.shape[1]} with the dtype of a/b")
        return torch.addmm(c, a.contiguous(), b.contiguous())
    return torch.mm(a.contiguous(), b.contiguous())


def _mm_fp32_or_bf16(mode, A, B, bias=None):
    """custom/backend/csrc/cublaslt_mm_fp32bf16.cu:99-240: Dt[n, m] for the three layouts."""
    _check_mode(mode)
    if A.dtype not in (torch.float32, torch.bfloat16) or A.dtype != B.dtype:
        raise RuntimeError("This op only supports float32 or bfloat16 with A and B of the same dtype")
    a = A if mode == TN else A.t()          # [m, k]
    b = B.t() if mode == NT else B          # [n, k]
    if a.shape[1] != b.shape[1]:
        raise RuntimeError(f"Mismatch matmul inner: A's k = {a.shape[1]}, B's k = {b.shape[1]}")
    if bias is not None:
        if bias.dtype != A.dtype or bias.ndim != 1 or bias.shape[0] != a.shape[0]:
            raise RuntimeError(f"bias is expected to be 1D of length {a.shape[0]} with the dtype of A")
        return torch.addmm(bias, b, a.t())
    return torch.mm(b, a.t())


def _mm_nvfp4(mode, DoutType, A, scaleA, B, scaleB, bias=None):
    """custom/backend/csrc/cublaslt_mm_nvfp4.cu:184-448: A [m, k], B [n, k] hold E2M1-valued
    fp32/bf16 numbers; they are packed to FP4 here, then Dt[n, m] = B A^T (+ bias[m])."""
    if mode != TN:
        raise RuntimeError("NVFP4 limitation: Only TN layout is supported")
    _check_common(A, scaleA, B, scaleB)
    if A.dtype not in (torch.float32, torch.bfloat16) or A.dtype != B.dtype:
        raise RuntimeError("Only supports torch.float32/bfloat16 E2M1-valued A and B of the same dtype")
    _check_dout(DoutType)
    if A.shape[1] != B.shape[1]:
        raise RuntimeError(f"Mismatch matmul inner: A's k = {A.shape[1]}, B's k = {B.shape[1]}")
    if A.shape[1] % 2:
        raise RuntimeError("k must be even (pad horizontally if needed).")
    if bias is not None and (bias.ndim != 1 or bias.shape[0] != A.shape[0]):
        raise RuntimeError(f"bias is expected to be 1D of length {A.shape[0]}, but got shape {tuple(bias.shape)}")
    qa, qb = ops.pack_e2m1(A), ops.pack_e2m1(B)
    if DoutType == torch.uint8:
        return _qout("nvfp4", "nvfp4", qb, scaleB, qa, scaleA, bias, A.shape[0], B.shape[0])
    out = ops.gemm_nvfp4(qb, scaleB, qa, scaleA, bias, DoutType)
    return out, out.new_empty(0)


def _mm_mxfp8(mode, DoutType, A, scaleA, B, scaleB, bias=None):
    """custom/backend/csrc/cublaslt_mm_mxfp8.cu:103-320.  TN takes row-wise quantized A [m, k],
    B [n, k].  NN takes A [k, m] quantized along k with scales in the layout of
    custom/swizzle.py:43-60; NT takes both operands that way.  Those forms are brought to the
    K-major layout of the kernel by a byte transpose and a scale re-layout."""
    _check_mode(mode)
    _check_common(A, scaleA, B, scaleB)
    if A.dtype not in (torch.uint8, torch.float8_e4m3fn) or B.dtype != A.dtype:
        raise RuntimeError("A and B must be E4M3 codes (torch.uint8 or torch.float8_e4m3fn) of the same dtype")
    _check_dout(DoutType)
    A8, B8 = A.view(torch.uint8), B.view(torch.uint8)
    if mode == TN:
        q, q_sf = A8, scaleA
    else:
        k, m = A8.shape
        q, q_sf = ops.transpose_bytes(A8), ops.colwise_to_canonical(scaleA, (k + 31) // 32, m)
    if mode == NT:
        k, n = B8.shape
        p, p_sf = ops.transpose_bytes(B8), ops.colwise_to_canonical(scaleB, (k + 31) // 32, n)
    else:
        p, p_sf = B8, scaleB
    if p.shape[1] != q.shape[1]:
        raise RuntimeError(f"Mismatch matmul inner: A's k = {q.shape[1]}, B's k = {p.shape[1]}")
    if bias is not None and (bias.ndim != 1 or bias.shape[0] != q.shape[0]):
        raise RuntimeError(f"bias is expected to be 1D of length {q.shape[0]}, but got shape {tuple(bias.shape)}")
    if DoutType == torch.uint8:
        return _qout("mxfp8", "mxfp8", p, p_sf, q, q_sf, bias, q.shape[0], p.shape[0])
    out = ops.gemm_mxfp8(p, p_sf, q, q_sf, bias, DoutType)
    return out, out.new_empty(0)


_lib_impl.impl("addmm_cuda", _addmm_cuda)
_lib_impl.impl("cublaslt_mm_fp32_or_bf16", _mm_fp32_or_bf16)
_lib_impl.impl("cublaslt_mm_nvfp4", _mm_nvfp4)
_lib_impl.impl("cublaslt_mm_mxfp8", _mm_mxfp8)
