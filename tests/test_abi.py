"""The C-ABI library loads without a GPU and exports every symbol include/fp4t.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fp4t.h")


def _declared():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"FP4T_API[^;(]*?\b(fp4t_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    from backend import _lib
    assert _declared() == _lib.exported_symbols()


def test_library_exports_every_declared_symbol():
    from backend import _lib
    if not os.path.isfile(_lib.LIB_PATH):
        pytest.fail(f"{_lib.LIB_PATH} is not built; run fp4-training_b200/csrc/build.sh")
    handle = ctypes.CDLL(os.path.abspath(_lib.LIB_PATH))
    for name in _declared():
        assert hasattr(handle, name), name
    L = _lib.lib()
    assert L.fp4t_version() >= 100
    assert L.fp4t_sf_bytes(8192, 256) == 64 * 64 * 512
    assert L.fp4t_sf_bytes(129, 5) == 2 * 2 * 512
    assert L.fp4t_sf_bytes(0, 5) == 0


def test_argument_errors_need_no_gpu():
    """Argument validation happens before any CUDA call."""
    from backend import _lib
    L = _lib.lib()
    rc = L.fp4t_quantize_nvfp4(None, 0, 4, 32, 32, None, None, None, None, 0, None, None, 0, None)
    assert rc == -1 and b"x is null" in L.fp4t_last_error()
    rc = L.fp4t_gemm_nvfp4(None, None, None, None, None, None, 0, 0, 1, 1, 32, None, None)
    assert rc == -1 and b"null pointer" in L.fp4t_last_error()
    with pytest.raises(ValueError):
        _lib.check(rc, "fp4t_gemm_nvfp4")


def test_allreduce_argument_errors_need_no_gpu():
    """The in-switch all-reduce rejects bad world sizes, ranks, lengths and epochs before it
    touches the device."""
    from backend import _lib
    L = _lib.lib()
    buf = ctypes.c_void_p(0x1000)
    flags = (ctypes.c_void_p * 8)(*[0x2000 + 0x100 * i for i in range(8)])

    def call(world=2, rank=0, numel=64, epoch=1, ctas=16, ptr=buf, fl=flags):
        return L.fp4t_allreduce_sum_bf16_multimem(ptr, fl, rank, world, numel, epoch, ctas, None, None)

    assert call(world=9) == -1 and b"world size" in L.fp4t_last_error()
    assert call(rank=2) == -1 and b"rank" in L.fp4t_last_error()
    assert call(numel=12) == -1 and b"multiple of 8" in L.fp4t_last_error()
    assert call(epoch=0) == -1 and b"epoch" in L.fp4t_last_error()
    assert call(ctas=0) == -1 and b"ctas" in L.fp4t_last_error()
    assert call(ptr=None) == -1 and b"null pointer" in L.fp4t_last_error()
    assert call(ptr=ctypes.c_void_p(0x1008)) == -1 and b"aligned" in L.fp4t_last_error()
    assert call(numel=0) == 0          # nothing to do, nothing launched
