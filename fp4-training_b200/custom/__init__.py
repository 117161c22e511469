"""Drop-in `custom` package: quantized `nn.Linear` modules, quantizer entry points and the
scale swizzles, with the names and signatures of the reference's custom/__init__.py:1-18.
Everything numeric runs in the fp4t CUDA library (sm_100a); there is no CPU path."""
from .linear.custom import CustomLinear
from .linear.cublaslt import CublasltLinear
from .linear.mxfp8 import CublasltMxfp8Linear
from .linear.nvfp4 import CublasltNvfp4Linear
from .linear.nvf4fwd_mxf8bwd import CublasltFwdNvfp4BwdMxfp8Linear

from .linear.cuda_aten import AddmmLinear
from .linear.fake_mxfp8 import FakeMxfp8Linear
from .norm import FusedLayerNorm

__all__ = [
    "CustomLinear",
    "CublasltLinear",
    "CublasltMxfp8Linear",
    "CublasltNvfp4Linear",
    "CublasltFwdNvfp4BwdMxfp8Linear",
    "FakeMxfp8Linear",
    "AddmmLinear",
    "FusedLayerNorm",
]
