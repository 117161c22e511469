"""ctypes binding of the fp4t C-ABI library (include/fp4t.h).

The library is built in-tree by csrc/build.sh into lib/libfp4t.so.  There is no
fallback: if the library is missing, loading raises and every operator of the
package is unusable.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "..", "lib", "libfp4t.so")

DT_BF16, DT_F32 = 0, 1
SR_NONE, SR_NOISE, SR_HASH = 0, 1, 2
QOUT_MXFP8, QOUT_NVFP4 = 1, 2

_c_i64 = ctypes.c_int64
_c_vp = ctypes.c_void_p

_SIGNATURES = {
    "fp4t_last_error": (ctypes.c_char_p, []),
    "fp4t_version": (ctypes.c_int, []),
    "fp4t_sf_bytes": (_c_i64, [_c_i64, _c_i64]),
    "fp4t_set_status_word": (ctypes.c_int, [_c_vp]),
    "fp4t_set_sm_limit": (ctypes.c_int, [ctypes.c_int]),
    "fp4t_set_seed_offset_word": (ctypes.c_int, [_c_vp]),
    "fp4t_set_wait_timeout_ns": (ctypes.c_int, [ctypes.c_uint64]),
    "fp4t_set_layer_concurrency": (ctypes.c_int, [ctypes.c_int]),
    "fp4t_reset_tile_counters": (ctypes.c_int, [ctypes.c_void_p]),
    "fp4t_allreduce_sum_bf16_multimem": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                                       ctypes.c_int, ctypes.c_int64, ctypes.c_uint32, ctypes.c_int,
                                                       ctypes.c_void_p, ctypes.c_void_p]),
    "fp4t_layernorm_forward": (ctypes.c_int, [_c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp, ctypes.c_float,
                                               _c_vp, ctypes.c_int, _c_i64, _c_vp, _c_vp, _c_vp]),
    "fp4t_layernorm_backward_workspace_bytes": (_c_i64, [_c_i64, _c_i64]),
    "fp4t_layernorm_backward": (ctypes.c_int, [_c_vp, ctypes.c_int, _c_i64, _c_vp, ctypes.c_int, _c_i64, _c_vp, _c_vp, _c_vp,
                                                _c_i64, _c_i64, _c_vp, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp]),
    "fp4t_rank_meet": (ctypes.c_int, [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_void_p, ctypes.c_void_p]),
    "fp4t_reduce_shard_bf16_multimem": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                                       ctypes.c_void_p]),
    "fp4t_sum_bf16_shards": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int64,
                                            ctypes.c_int, ctypes.c_void_p]),
    "fp4t_quantize_nvfp4": (ctypes.c_int, [_c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp,
                                            ctypes.c_int, _c_vp, _c_vp, ctypes.c_uint64, _c_vp]),
    "fp4t_quantize_mxfp8": (ctypes.c_int, [_c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp,
                                            _c_vp]),
    "fp4t_quantize_nvfp4_scaled": (ctypes.c_int, [_c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp,
                                                   ctypes.c_int, ctypes.c_uint64, ctypes.c_float, _c_vp]),
    "fp4t_quantize_nvfp4_rht": (ctypes.c_int, [_c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp,
                                                ctypes.c_uint32, ctypes.c_float, _c_vp]),
    "fp4t_quantize_nvfp4_gelu": (ctypes.c_int, [_c_vp, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp]),
    "fp4t_quantize_mxfp8_gelu": (ctypes.c_int, [_c_vp, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp]),
    "fp4t_quantize_nvfp4_bgrad": (ctypes.c_int, [_c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp,
                                                  ctypes.c_int, _c_vp, _c_vp, ctypes.c_uint64, _c_vp, _c_vp, ctypes.c_int,
                                                  _c_vp]),
    "fp4t_quantize_nvfp4_bgrad_static": (ctypes.c_int, [_c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp, _c_vp,
                                                         _c_vp, ctypes.c_int, _c_vp, _c_vp, ctypes.c_uint64, _c_vp,
                                                         ctypes.c_int, _c_vp]),
    "fp4t_quantize_mxfp8_bgrad": (ctypes.c_int, [_c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp,
                                                  _c_vp, _c_vp, ctypes.c_int, _c_vp]),
    "fp4t_gemm_nvfp4": (ctypes.c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64,
                                        _c_i64, _c_vp, _c_vp]),
    "fp4t_gemm_mxfp8": (ctypes.c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64,
                                        _c_i64, _c_vp, _c_vp]),
    "fp4t_gemm_nvfp4_qout": (ctypes.c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, ctypes.c_int, _c_i64, _c_i64,
                                             _c_i64, _c_i64, _c_vp, _c_vp]),
    "fp4t_gemm_mxfp8_qout": (ctypes.c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, ctypes.c_int, _c_i64, _c_i64,
                                             _c_i64, _c_i64, _c_vp, _c_vp]),
    "fp4t_linear_workspace_bytes": (_c_i64, [ctypes.c_int, _c_i64, _c_i64, _c_i64]),
    "fp4t_linear_backward_workspace_bytes": (_c_i64, [ctypes.c_int, _c_i64, _c_i64, _c_i64]),
    "fp4t_gemm_splitk_workspace_bytes": (_c_i64, [_c_i64, _c_i64]),
    "fp4t_gemm_nvfp4_splitk": (ctypes.c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64,
                                               _c_i64, _c_vp, _c_i64, _c_vp, _c_vp]),
    "fp4t_gemm_nvfp4_scaled": (ctypes.c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64,
                                               _c_i64, ctypes.c_float, _c_vp, _c_i64, _c_vp, _c_vp]),
    "fp4t_gemm_mxfp8_splitk": (ctypes.c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64,
                                               _c_i64, _c_vp, _c_i64, _c_vp, _c_vp]),
    "fp4t_linear_forward": (ctypes.c_int, [ctypes.c_int, _c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64, _c_vp, ctypes.c_int,
                                            _c_i64, _c_i64, _c_vp, _c_vp, ctypes.c_int, _c_i64, _c_vp, ctypes.c_int, _c_vp,
                                            _c_vp]),
    "fp4t_linear_backward": (ctypes.c_int, [ctypes.c_int, _c_vp, ctypes.c_int, _c_i64, _c_i64, _c_i64, _c_i64, _c_vp, _c_vp,
                                             _c_vp, _c_i64, _c_vp, _c_i64, _c_vp, ctypes.c_int, ctypes.c_int, _c_vp, _c_vp,
                                             ctypes.c_uint64, _c_vp, _c_vp]),
    "fp4t_pack_e2m1": (ctypes.c_int, [_c_vp, ctypes.c_int, _c_vp, _c_i64, _c_i64, _c_vp]),
    "fp4t_unpack_e2m1": (ctypes.c_int, [_c_vp, _c_vp, _c_i64, _c_i64, _c_vp]),
    "fp4t_swizzle_rowwise": (ctypes.c_int, [_c_vp, _c_vp, _c_i64, _c_i64, _c_vp]),
    "fp4t_swizzle_colwise": (ctypes.c_int, [_c_vp, _c_vp, _c_i64, _c_i64, _c_vp]),
    "fp4t_unswizzle_colwise_to_rowwise": (ctypes.c_int, [_c_vp, _c_vp, _c_i64, _c_i64, _c_vp]),
    "fp4t_transpose_bytes": (ctypes.c_int, [_c_vp, _c_vp, _c_i64, _c_i64, _c_vp]),
}

_lib = None


def exported_symbols():
    """Names every build of the library must export (kept in step with include/fp4t.h)."""
    return sorted(_SIGNATURES)


def lib():
    global _lib
    if _lib is None:
        path = os.path.abspath(LIB_PATH)
        if not os.path.isfile(path):
            raise RuntimeError(
                f"fp4t native library not found at {path}; build it with fp4-training_b200/csrc/build.sh "
                "(there is no non-CUDA fallback)")
        handle = ctypes.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int, what: str):
    if rc != 0:
        msg = lib().fp4t_last_error().decode("utf-8", "replace")
        if rc == -1:
            raise ValueError(f"{what}: {msg}")
        raise RuntimeError(f"{what} failed ({rc}): {msg}")


def ptr(t):
    """Device address of a tensor as a plain int (ctypes converts it for c_void_p parameters)."""
    return None if t is None else t.data_ptr()


def stream_ptr(device):
    """Raw handle of torch's current stream on `device`."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(idx)


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return DT_BF16
    if dt == torch.float32:
        return DT_F32
    raise ValueError(f"only torch.bfloat16 and torch.float32 are supported, got {dt}")


def sf_shape(outer: int, kblocks: int):
    """2-D shape of the swizzled scale buffer for a logical [outer, kblocks] matrix."""
    return ((outer + 127) // 128 * 32, (kblocks + 3) // 4 * 16)
