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
