"""Tensor-level wrappers over the fp4t C ABI.

Outputs are allocated with torch (caching allocator, current device), the kernels run on
torch's current stream, and nothing here synchronises.  CPU tensors are rejected: there
is no host implementation.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import SR_HASH, SR_NOISE, SR_NONE  # noqa: F401  (re-exported)

NVFP4_BLOCK = 16
MXFP8_BLOCK = 32

import contextlib
import threading

_status = {}
_tls = threading.local()
LAUNCHES = {"quantize": 0, "gemm": 0, "misc": 0, "allreduce": 0, "norm": 0}   # kernels enqueued by this process


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NotImplementedError("fp4t operators run on CUDA tensors only (no CPU implementation)")


def status_word(device) -> torch.Tensor:
    """Device int32[4] the GEMM kernels write to if one of their bounded waits runs out."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
    return _status[key]


def _on_device(dev):
    """Context that makes `dev` current; free when it already is (the common case)."""
    if dev.index is None or dev.index == torch.cuda.current_device():
        return contextlib.nullcontext()
    return torch.cuda.device(dev)


def _bind_status(dev):
    """Point this host thread's status reporting at the device's status word (once per thread/device)."""
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if getattr(_tls, "status_dev", None) != key:
        _lib.lib().fp4t_set_status_word(_lib.ptr(status_word(dev)))
        _tls.status_dev = key


def check_status(device="cuda") -> None:
    """Synchronising check of the status word; raises if a kernel gave up on a wait."""
    s = status_word(device)
    code = int(s[0].item())
    if code != 0:
        s.zero_()
        # a kernel that gave up may have left its tile counters nonzero
        with torch.cuda.device(s.device):
            _lib.check(_lib.lib().fp4t_reset_tile_counters(_lib.stream_ptr(s.device)), "fp4t_reset_tile_counters")
        raise RuntimeError(f"fp4t kernel abandoned a wait (role code {code})")


def _alloc_q(outer, inner, blk, packed, device):
    codes = torch.empty((outer, inner // 2 if packed else inner), dtype=torch.uint8, device=device)
    sf = torch.empty(_lib.sf_shape(outer, inner // blk), dtype=torch.uint8, device=device)
    return codes, sf


_colsum_scratch = {}


def _scratch(dev, cols):
    """fp32 scratch of at least `cols` values on `dev` for the fused bias-gradient sums
    (grown on demand, reused by the calls of one stream, which are ordered)."""
    # one buffer per (device, stream): calls on one stream are ordered, calls on different streams
    # may overlap on the GPU and must not share the accumulator
    key = (dev.type, dev.index, _lib.stream_ptr(dev))
    buf = _colsum_scratch.get(key)
    if buf is None or buf.numel() < cols:
        buf = torch.empty(max(cols, 4096), dtype=torch.float32, device=dev)
        _colsum_scratch[key] = buf
    return buf


def _quantize(fmt, x, want_row, want_t, sr, noise, noise_t, seed, bias_grad_dtype=None):
    if x.ndim != 2:
        raise ValueError("Input tensor must be 2D for block quantization")
    _need_cuda(x, noise, noise_t)
    blk = NVFP4_BLOCK if fmt == "nvfp4" else MXFP8_BLOCK
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.to(torch.float32)
    if x.stride(1) != 1:
        x = x.contiguous()
    rows, cols = x.shape
    if want_row and cols % blk:
        raise ValueError(f"row-wise {fmt} quantization needs columns to be a multiple of {blk}")
    if want_t and rows % 32:
        raise ValueError(f"transposed {fmt} quantization needs rows to be a multiple of 32")
    dev = x.device
    codes = sf = codes_t = sf_t = bgrad = None
    with _on_device(dev):
        if bias_grad_dtype is not None:
            bgrad = torch.empty(cols, dtype=bias_grad_dtype, device=dev)
        if want_row:
            codes, sf = _alloc_q(rows, cols, blk, fmt == "nvfp4", dev)
        if want_t:
            codes_t, sf_t = _alloc_q(cols, rows, blk, fmt == "nvfp4", dev)
        if rows == 0 or cols == 0:
            if bgrad is not None:
                bgrad.zero_()
                return codes, sf, codes_t, sf_t, bgrad
            return codes, sf, codes_t, sf_t
        L = _lib.lib()
        _bind_status(dev)
        if fmt == "nvfp4":
            if noise is not None:
                noise = noise.to(torch.float32).reshape(rows, cols).contiguous()
            if noise_t is not None:
                noise_t = noise_t.to(torch.float32).reshape(cols, rows).contiguous()
            if bgrad is None:
                rc = L.fp4t_quantize_nvfp4(_lib.ptr(x), _lib.dtype_code(x.dtype), rows, cols, x.stride(0),
                                           _lib.ptr(codes), _lib.ptr(sf), _lib.ptr(codes_t), _lib.ptr(sf_t),
                                           int(sr), _lib.ptr(noise), _lib.ptr(noise_t),
                                           ctypes.c_uint64(seed & (2 ** 64 - 1)), _lib.stream_ptr(dev))
            else:
                rc = L.fp4t_quantize_nvfp4_bgrad(_lib.ptr(x), _lib.dtype_code(x.dtype), rows, cols, x.stride(0),
                                                 _lib.ptr(codes), _lib.ptr(sf), _lib.ptr(codes_t), _lib.ptr(sf_t),
                                                 int(sr), _lib.ptr(noise), _lib.ptr(noise_t),
                                                 ctypes.c_uint64(seed & (2 ** 64 - 1)), _lib.ptr(_scratch(dev, cols)),
                                                 _lib.ptr(bgrad), _lib.dtype_code(bgrad.dtype), _lib.stream_ptr(dev))
            _lib.check(rc, "fp4t_quantize_nvfp4")
        else:
            if bgrad is None:
                rc = L.fp4t_quantize_mxfp8(_lib.ptr(x), _lib.dtype_code(x.dtype), rows, cols, x.stride(0),
                                           _lib.ptr(codes), _lib.ptr(sf), _lib.ptr(codes_t), _lib.ptr(sf_t),
                                           _lib.stream_ptr(dev))
            else:
                rc = L.fp4t_quantize_mxfp8_bgrad(_lib.ptr(x), _lib.dtype_code(x.dtype), rows, cols, x.stride(0),
                                                 _lib.ptr(codes), _lib.ptr(sf), _lib.ptr(codes_t), _lib.ptr(sf_t),
                                                 _lib.ptr(_scratch(dev, cols)), _lib.ptr(bgrad),
                                                 _lib.dtype_code(bgrad.dtype), _lib.stream_ptr(dev))
            _lib.check(rc, "fp4t_quantize_mxfp8")
        LAUNCHES["quantize"] += 1 if bgrad is None else 2
    if bgrad is not None:
        return codes, sf, codes_t, sf_t, bgrad
    return codes, sf, codes_t, sf_t


def quantize_nvfp4(x, want_row=True, want_t=False, sr=SR_NONE, noise=None, noise_t=None, seed=0,
                   bias_grad_dtype=None):
    """-> (codes [R, C/2], sf, codes_t [C, R/2], sf_t); entries not requested are None.
    With bias_grad_dtype a fifth element is returned: the column sums of x in that dtype."""
    return _quantize("nvfp4", x, want_row, want_t, sr, noise, noise_t, seed, bias_grad_dtype)


def quantize_mxfp8(x, want_row=True, want_t=False, bias_grad_dtype=None):
    """-> (codes [R, C], sf, codes_t [C, R], sf_t) (+ column sums of x when bias_grad_dtype is given)."""
    return _quantize("mxfp8", x, want_row, want_t, SR_NONE, None, None, 0, bias_grad_dtype)


def quantize_nvfp4_scaled(x, tensor_scale, want_row=True, want_t=False, sr=SR_NONE, seed=0, rht_signs=None):
    """NVFP4 block quantization of x * tensor_scale (the second, per-tensor scale level), with
    an optional random Hadamard transform of each 16-block (rht_signs: 16-bit sign mask).
    -> (codes, sf, codes_t, sf_t); the operands describe x * tensor_scale, so a GEMM of two of
    them takes alpha = 1 / (t_p * t_q) (gemm_nvfp4(..., alpha=...))."""
    if x.ndim != 2:
        raise ValueError("Input tensor must be 2D for block quantization")
    _need_cuda(x)
    if not (tensor_scale > 0.0 and tensor_scale < 3.0e38):
        raise ValueError("tensor_scale must be positive and finite")
    if rht_signs is not None and sr != SR_NONE:
        raise ValueError("the Hadamard-transformed quantizer rounds to nearest")
    if sr not in (SR_NONE, SR_HASH):
        raise ValueError("the scaled quantizer takes round-to-nearest or in-kernel stochastic rounding")
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.to(torch.float32)
    if x.stride(1) != 1:
        x = x.contiguous()
    rows, cols = x.shape
    if want_row and cols % NVFP4_BLOCK:
        raise ValueError("row-wise nvfp4 quantization needs columns to be a multiple of 16")
    if want_t and rows % 32:
        raise ValueError("transposed nvfp4 quantization needs rows to be a multiple of 32")
    dev = x.device
    codes = sf = codes_t = sf_t = None
    with _on_device(dev):
        if want_row:
            codes, sf = _alloc_q(rows, cols, NVFP4_BLOCK, True, dev)
        if want_t:
            codes_t, sf_t = _alloc_q(cols, rows, NVFP4_BLOCK, True, dev)
        if rows == 0 or cols == 0:
            return codes, sf, codes_t, sf_t
        _bind_status(dev)
        L = _lib.lib()
        if rht_signs is None:
            rc = L.fp4t_quantize_nvfp4_scaled(_lib.ptr(x), _lib.dtype_code(x.dtype), rows, cols, x.stride(0),
                                              _lib.ptr(codes), _lib.ptr(sf), _lib.ptr(codes_t), _lib.ptr(sf_t), int(sr),
                                              ctypes.c_uint64(seed & (2 ** 64 - 1)), float(tensor_scale),
                                              _lib.stream_ptr(dev))
            _lib.check(rc, "fp4t_quantize_nvfp4_scaled")
        else:
            rc = L.fp4t_quantize_nvfp4_rht(_lib.ptr(x), _lib.dtype_code(x.dtype), rows, cols, x.stride(0),
                                           _lib.ptr(codes), _lib.ptr(sf), _lib.ptr(codes_t), _lib.ptr(sf_t),
                                           int(rht_signs) & 0xFFFF, float(tensor_scale), _lib.stream_ptr(dev))
            _lib.check(rc, "fp4t_quantize_nvfp4_rht")
        LAUNCHES["quantize"] += 1
    return codes, sf, codes_t, sf_t


def quantize_gelu(fmt, x, want_row=True, want_t=False):
    """Quantization of GELU(x) for a bf16 pre-activation x, the activation applied inside the
    quantizer (its bf16 result is never materialised).  -> (codes, sf, codes_t, sf_t)."""
    if x.ndim != 2:
        raise ValueError("Input tensor must be 2D for block quantization")
    _need_cuda(x)
    if x.dtype != torch.bfloat16:
        raise ValueError("the fused GELU quantizer takes a bfloat16 pre-activation")
    blk = NVFP4_BLOCK if fmt == "nvfp4" else MXFP8_BLOCK
    if x.stride(1) != 1:
        x = x.contiguous()
    rows, cols = x.shape
    if want_row and cols % blk:
        raise ValueError(f"row-wise {fmt} quantization needs columns to be a multiple of {blk}")
    if want_t and rows % 32:
        raise ValueError(f"transposed {fmt} quantization needs rows to be a multiple of 32")
    dev = x.device
    codes = sf = codes_t = sf_t = None
    with _on_device(dev):
        if want_row:
            codes, sf = _alloc_q(rows, cols, blk, fmt == "nvfp4", dev)
        if want_t:
            codes_t, sf_t = _alloc_q(cols, rows, blk, fmt == "nvfp4", dev)
        if rows == 0 or cols == 0:
            return codes, sf, codes_t, sf_t
        _bind_status(dev)
        fn = _lib.lib().fp4t_quantize_nvfp4_gelu if fmt == "nvfp4" else _lib.lib().fp4t_quantize_mxfp8_gelu
        rc = fn(_lib.ptr(x), rows, cols, x.stride(0), _lib.ptr(codes), _lib.ptr(sf), _lib.ptr(codes_t), _lib.ptr(sf_t),
                _lib.stream_ptr(dev))
        if rc == -3:
            raise NotImplementedError(_lib.lib().fp4t_last_error().decode("utf-8", "replace"))
        _lib.check(rc, f"fp4t_quantize_{fmt}_gelu")
        LAUNCHES["quantize"] += 1
    return codes, sf, codes_t, sf_t


def _gemm(fmt, p_codes, p_sf, q_codes, q_sf, bias, out_dtype, out=None, split_k=True, alpha=1.0):
    _need_cuda(p_codes, p_sf, q_codes, q_sf, bias)
    rows, cols = p_codes.shape[0], q_codes.shape[0]
    kbytes = p_codes.shape[1]
    if q_codes.shape[1] != kbytes:
        raise RuntimeError(f"Mismatch matmul inner: P has {kbytes} code bytes per row, Q has {q_codes.shape[1]}")
    k = kbytes * 2 if fmt == "nvfp4" else kbytes
    dev = p_codes.device
    if bias is not None:
        if bias.ndim != 1 or bias.shape[0] != cols:
            raise RuntimeError(f"bias is expected to be 1D of length {cols}, but got shape {tuple(bias.shape)}")
        bias = bias.to(torch.bfloat16).contiguous()
    with _on_device(dev):
        if out is None:
            out = torch.empty((rows, cols), dtype=out_dtype, device=dev)
        if rows == 0 or cols == 0:
            return out
        L = _lib.lib()
        ws_bytes = L.fp4t_gemm_splitk_workspace_bytes(rows, cols) if (split_k and k >= 2048) else 0
        if alpha != 1.0:
            if fmt != "nvfp4":
                raise ValueError("alpha (per-tensor operand scales) is an NVFP4 option")
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes > 0 else None
            rc = L.fp4t_gemm_nvfp4_scaled(_lib.ptr(p_codes), _lib.ptr(p_sf), _lib.ptr(q_codes), _lib.ptr(q_sf),
                                          _lib.ptr(bias), _lib.ptr(out), _lib.dtype_code(out.dtype), out.stride(0),
                                          rows, cols, k, float(alpha), _lib.ptr(ws), max(ws_bytes, 0),
                                          _lib.ptr(status_word(dev)), _lib.stream_ptr(dev))
        elif ws_bytes > 0:      # a small output over a long K: let the idle SMs share the K loop
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            fn = L.fp4t_gemm_nvfp4_splitk if fmt == "nvfp4" else L.fp4t_gemm_mxfp8_splitk
            rc = fn(_lib.ptr(p_codes), _lib.ptr(p_sf), _lib.ptr(q_codes), _lib.ptr(q_sf), _lib.ptr(bias),
                    _lib.ptr(out), _lib.dtype_code(out.dtype), out.stride(0), rows, cols, k, _lib.ptr(ws), ws_bytes,
                    _lib.ptr(status_word(dev)), _lib.stream_ptr(dev))
        else:
            fn = L.fp4t_gemm_nvfp4 if fmt == "nvfp4" else L.fp4t_gemm_mxfp8
            rc = fn(_lib.ptr(p_codes), _lib.ptr(p_sf), _lib.ptr(q_codes), _lib.ptr(q_sf), _lib.ptr(bias),
                    _lib.ptr(out), _lib.dtype_code(out.dtype), out.stride(0), rows, cols, k,
                    _lib.ptr(status_word(dev)), _lib.stream_ptr(dev))
        _lib.check(rc, f"fp4t_gemm_{fmt}")
        LAUNCHES["gemm"] += 1
    return out


def gemm_nvfp4(p_codes, p_sf, q_codes, q_sf, bias=None, out_dtype=torch.bfloat16, out=None, split_k=True, alpha=1.0):
    """D[rows, cols] = alpha * P . Q^T (+bias); P/Q packed E2M1 codes [outer, K/2].  split_k=False
    keeps a small-output / long-K product on the unsplit kernel (one fixed accumulation order);
    alpha undoes per-tensor operand scales (quantize_nvfp4_scaled)."""
    return _gemm("nvfp4", p_codes, p_sf, q_codes, q_sf, bias, out_dtype, out, split_k, alpha)


def gemm_mxfp8(p_codes, p_sf, q_codes, q_sf, bias=None, out_dtype=torch.bfloat16, out=None, split_k=True):
    """D[rows, cols] = P . Q^T (+bias); P/Q E4M3 codes [outer, K]."""
    return _gemm("mxfp8", p_codes, p_sf, q_codes, q_sf, bias, out_dtype, out, split_k)


def gemm_qout(fmt, p_codes, p_sf, q_codes, q_sf, bias=None, out_fmt="mxfp8"):
    """D = P . Q^T (+bias) written as a block-quantized row-wise operand: -> (codes, sf) with
    codes [rows, cols] E4M3 bytes (out_fmt 'mxfp8') or [rows, cols/2] packed E2M1 ('nvfp4') and the
    scales of logical [rows, cols/32] or [rows, cols/16] in the tile layout."""
    _need_cuda(p_codes, p_sf, q_codes, q_sf, bias)
    rows, cols = p_codes.shape[0], q_codes.shape[0]
    kbytes = p_codes.shape[1]
    if q_codes.shape[1] != kbytes:
        raise RuntimeError(f"Mismatch matmul inner: P has {kbytes} code bytes per row, Q has {q_codes.shape[1]}")
    if cols % 32:
        raise ValueError("a quantized GEMM output needs a multiple of 32 columns")
    k = kbytes * 2 if fmt == "nvfp4" else kbytes
    dev = p_codes.device
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    blk = 16 if out_fmt == "nvfp4" else 32
    with _on_device(dev):
        codes = torch.empty((rows, cols // 2 if out_fmt == "nvfp4" else cols), dtype=torch.uint8, device=dev)
        sf = torch.empty(_lib.sf_shape(rows, cols // blk), dtype=torch.uint8, device=dev)
        if rows == 0 or cols == 0:
            return codes, sf
        fn = _lib.lib().fp4t_gemm_nvfp4_qout if fmt == "nvfp4" else _lib.lib().fp4t_gemm_mxfp8_qout
        rc = fn(_lib.ptr(p_codes), _lib.ptr(p_sf), _lib.ptr(q_codes), _lib.ptr(q_sf), _lib.ptr(bias), _lib.ptr(codes),
                _lib.ptr(sf), _lib.QOUT_NVFP4 if out_fmt == "nvfp4" else _lib.QOUT_MXFP8, codes.stride(0), rows, cols, k,
                _lib.ptr(status_word(dev)), _lib.stream_ptr(dev))
        _lib.check(rc, f"fp4t_gemm_{fmt}_qout")
        LAUNCHES["gemm"] += 1
    return codes, sf


def pack_e2m1(values: torch.Tensor) -> torch.Tensor:
    """fp32/bf16 values on the E2M1 grid [R, C] -> packed codes [R, C/2]."""
    _need_cuda(values)
    values = values.contiguous()
    rows, cols = values.shape
    out = torch.empty((rows, cols // 2), dtype=torch.uint8, device=values.device)
    with torch.cuda.device(values.device):
        rc = _lib.lib().fp4t_pack_e2m1(_lib.ptr(values), _lib.dtype_code(values.dtype), _lib.ptr(out), rows, cols,
                                       _lib.stream_ptr(values.device))
        _lib.check(rc, "fp4t_pack_e2m1")
        LAUNCHES["misc"] += 1
    return out


def unpack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """packed codes [R, C/2] -> fp32 values [R, C]."""
    _need_cuda(codes)
    codes = codes.contiguous()
    rows, half = codes.shape
    out = torch.empty((rows, half * 2), dtype=torch.float32, device=codes.device)
    with torch.cuda.device(codes.device):
        rc = _lib.lib().fp4t_unpack_e2m1(_lib.ptr(codes), _lib.ptr(out), rows, half * 2,
                                         _lib.stream_ptr(codes.device))
        _lib.check(rc, "fp4t_unpack_e2m1")
        LAUNCHES["misc"] += 1
    return out


def _relayout(fn_name, src, outer, inner):
    _need_cuda(src)
    src = src.contiguous()
    shape = _lib.sf_shape(outer, inner)
    if fn_name == "fp4t_swizzle_colwise":   # the reference returns [ceil(inner/4)*32, ceil(outer/128)*16]
        shape = ((inner + 3) // 4 * 32, (outer + 127) // 128 * 16)
    out = torch.empty(shape, dtype=torch.uint8, device=src.device)
    with torch.cuda.device(src.device):
        fn = getattr(_lib.lib(), fn_name)
        if fn_name == "fp4t_swizzle_rowwise":
            rc = fn(_lib.ptr(src), _lib.ptr(out), outer, inner, _lib.stream_ptr(src.device))
        else:
            rc = fn(_lib.ptr(src), _lib.ptr(out), inner, outer, _lib.stream_ptr(src.device))
        _lib.check(rc, fn_name)
        LAUNCHES["misc"] += 1
    return out


def swizzle_rowwise(scale: torch.Tensor) -> torch.Tensor:
    """logical [outer, inner] bytes -> canonical 128x4 tile layout."""
    return _relayout("fp4t_swizzle_rowwise", scale, scale.shape[0], scale.shape[1])


def swizzle_colwise(scale: torch.Tensor) -> torch.Tensor:
    """logical [inner, outer] bytes -> the reference's column-wise layout."""
    return _relayout("fp4t_swizzle_colwise", scale, scale.shape[1], scale.shape[0])


def colwise_to_canonical(sw: torch.Tensor, inner: int, outer: int) -> torch.Tensor:
    """Reference column-wise layout of a logical [inner, outer] matrix -> canonical tiles of its transpose."""
    return _relayout("fp4t_unswizzle_colwise_to_rowwise", sw, outer, inner)


def transpose_bytes(src: torch.Tensor) -> torch.Tensor:
    _need_cuda(src)
    src = src.contiguous()
    rows, cols = src.shape
    out = torch.empty((cols, rows), dtype=torch.uint8, device=src.device)
    with torch.cuda.device(src.device):
        rc = _lib.lib().fp4t_transpose_bytes(_lib.ptr(src), _lib.ptr(out), rows, cols, _lib.stream_ptr(src.device))
        _lib.check(rc, "fp4t_transpose_bytes")
        LAUNCHES["misc"] += 1
    return out


_FMT = {"nvfp4": 0, "mxfp8": 1}


def linear_forward(fmt, x, w, bias, keep_wt, keep_xt, out_dtype):
    """One C call: quantize W and X (plus the transposed operands asked for) and compute
    Y = X W^T + bias.  -> (Y, workspace); the workspace feeds linear_backward."""
    _need_cuda(x, w, bias)
    n, ic = x.shape
    oc = w.shape[0]
    dev = x.device
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    with _on_device(dev):
        L = _lib.lib()
        _bind_status(dev)
        ws = torch.empty(L.fp4t_linear_workspace_bytes(_FMT[fmt], n, ic, oc), dtype=torch.uint8, device=dev)
        y = torch.empty((n, oc), dtype=out_dtype, device=dev)
        rc = L.fp4t_linear_forward(_FMT[fmt], x.data_ptr(), _lib.dtype_code(x.dtype), n, ic, x.stride(0),
                                   w.data_ptr(), _lib.dtype_code(w.dtype), oc, w.stride(0), _lib.ptr(bias),
                                   y.data_ptr(), _lib.dtype_code(out_dtype), oc, ws.data_ptr(),
                                   (1 if keep_wt else 0) | (2 if keep_xt else 0), status_word(dev).data_ptr(),
                                   _lib.stream_ptr(dev))
        _lib.check(rc, "fp4t_linear_forward")
        LAUNCHES["quantize"] += 2
        LAUNCHES["gemm"] += 1
    return y, ws


def linear_backward(fmt, g, ws, ic, need_dx, need_dw, need_db, sr=SR_NONE, noise=None, noise_t=None, seed=0,
                    out_dw=None, out_db=None):
    """One C call: quantize dY once and compute dX, dW and the bias gradient (those asked for).
    out_dw [oc, ic] / out_db [oc] (dtype of g, contiguous) receive the results in place, e.g.
    views of one flat gradient buffer that is all-reduced with a single collective."""
    _need_cuda(g, ws)
    n, oc = g.shape
    dev = g.device
    with _on_device(dev):
        L = _lib.lib()
        _bind_status(dev)
        bws = torch.empty(L.fp4t_linear_backward_workspace_bytes(_FMT[fmt], n, oc, ic), dtype=torch.uint8, device=dev)
        dx = torch.empty((n, ic), dtype=g.dtype, device=dev) if need_dx else None
        dw = (out_dw if out_dw is not None else torch.empty((oc, ic), dtype=g.dtype, device=dev)) if need_dw else None
        db = (out_db if out_db is not None else torch.empty((oc,), dtype=g.dtype, device=dev)) if need_db else None
        if noise is not None:
            noise = noise.to(torch.float32).reshape(n, oc).contiguous()
        if noise_t is not None:
            noise_t = noise_t.to(torch.float32).reshape(oc, n).contiguous()
        rc = L.fp4t_linear_backward(_FMT[fmt], g.data_ptr(), _lib.dtype_code(g.dtype), n, oc, g.stride(0), ic,
                                    ws.data_ptr(), bws.data_ptr(), _lib.ptr(dx), ic, _lib.ptr(dw), ic, _lib.ptr(db),
                                    _lib.dtype_code(g.dtype), int(sr), _lib.ptr(noise), _lib.ptr(noise_t),
                                    ctypes.c_uint64(seed & (2 ** 64 - 1)), status_word(dev).data_ptr(),
                                    _lib.stream_ptr(dev))
        _lib.check(rc, "fp4t_linear_backward")
        LAUNCHES["quantize"] += 2 if need_db else 1
        LAUNCHES["gemm"] += int(need_dx) + int(need_dw)
    return dx, dw, db


# ------------------------------------------------------------------ LayerNorm
def layernorm_forward(x, gamma, beta, eps, out_dtype):
    """x [rows, cols] (fp32 or bf16, unit column stride) -> (y [rows, cols] in out_dtype, mean, rstd);
    statistics in fp32.  gamma / beta: fp32 [cols]."""
    _need_cuda(x, gamma, beta)
    if x.ndim != 2:
        raise ValueError("layernorm_forward takes a 2-D tensor")
    if x.dtype not in (torch.float32, torch.bfloat16) or out_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("layernorm runs on float32 / bfloat16 tensors")
    rows, cols = x.shape
    if cols % 4 or cols > 1024:
        raise ValueError("layernorm needs a normalized width that is a multiple of 4, at most 1024")
    if x.stride(1) != 1 or x.stride(0) % 4 or x.data_ptr() % 16:
        x = x.contiguous()
    dev = x.device
    gamma = gamma.detach().to(torch.float32).contiguous()
    beta = beta.detach().to(torch.float32).contiguous()
    with _on_device(dev):
        y = torch.empty((rows, cols), dtype=out_dtype, device=dev)
        mean = torch.empty(rows, dtype=torch.float32, device=dev)
        rstd = torch.empty(rows, dtype=torch.float32, device=dev)
        rc = _lib.lib().fp4t_layernorm_forward(_lib.ptr(x), _lib.dtype_code(x.dtype), rows, cols, x.stride(0),
                                               _lib.ptr(gamma), _lib.ptr(beta), float(eps), _lib.ptr(y),
                                               _lib.dtype_code(out_dtype), cols, _lib.ptr(mean), _lib.ptr(rstd),
                                               _lib.stream_ptr(dev))
        _lib.check(rc, "fp4t_layernorm_forward")
        LAUNCHES["norm"] += 1
    return y, mean, rstd


def layernorm_backward(dy, x, mean, rstd, gamma):
    """-> (dx like x, dgamma fp32 [cols], dbeta fp32 [cols]) for the forward above."""
    _need_cuda(dy, x, mean, rstd, gamma)
    rows, cols = x.shape
    if dy.shape != x.shape:
        raise ValueError("dy must have the shape of x")
    if dy.dtype not in (torch.float32, torch.bfloat16):
        dy = dy.to(torch.float32)
    if dy.stride(1) != 1 or dy.stride(0) % 4 or dy.data_ptr() % 16:
        dy = dy.contiguous()
    if x.stride(1) != 1 or x.stride(0) % 4 or x.data_ptr() % 16:
        x = x.contiguous()
    dev = x.device
    gamma = gamma.detach().to(torch.float32).contiguous()
    with _on_device(dev):
        L = _lib.lib()
        dx = torch.empty((rows, cols), dtype=x.dtype, device=dev)
        dgamma = torch.empty(cols, dtype=torch.float32, device=dev)
        dbeta = torch.empty(cols, dtype=torch.float32, device=dev)
        ws_bytes = L.fp4t_layernorm_backward_workspace_bytes(rows, cols)
        if ws_bytes < 0:
            raise RuntimeError("fp4t_layernorm_backward_workspace_bytes: unsupported shape or device")
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        rc = L.fp4t_layernorm_backward(_lib.ptr(dy), _lib.dtype_code(dy.dtype), dy.stride(0), _lib.ptr(x),
                                       _lib.dtype_code(x.dtype), x.stride(0), _lib.ptr(mean), _lib.ptr(rstd),
                                       _lib.ptr(gamma), rows, cols, _lib.ptr(dx), cols, _lib.ptr(dgamma), _lib.ptr(dbeta),
                                       _lib.ptr(ws), _lib.stream_ptr(dev))
        _lib.check(rc, "fp4t_layernorm_backward")
        LAUNCHES["norm"] += 2
    return dx, dgamma, dbeta
