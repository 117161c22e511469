"""Generate the golden fixtures in this directory from the reference's own Python.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py --reference /path/to/fp4-training
    (or FP4T_REFERENCE=/path/to/fp4-training python tests/golden/make_golden.py)

It imports the reference's custom/swizzle.py and custom/quantize.py by file
path (the NVFP4 quantizer and both swizzles are pure PyTorch and run on CPU),
with the absent `microxcaling` package stubbed so the import succeeds; nothing
of the MXFP8 path is executed.  The outputs are small .npz files:

  nvfp4_rowwise_*.npz   inputs (bf16 bits), E2M1 codes after the pack rule of
                        custom/backend/csrc/cublaslt_mm_nvfp4.cu:113-166, E4M3
                        scale bytes (logical and swizzled), for the
                        deterministic and the stochastic path (noise stored)
  swizzle_*.npz         scale matrices and both reference swizzles
  nvfp4_api_*.npz       what the reference's public entry points return, call by call:
                        quantize_nvfp4(rowwise in {True, False}, simulated in {True, False}),
                        q_nvfp4_rowwise / q_nvfp4_colwise with and without stochastic
                        rounding (the noise the reference drew is stored)

The GPU box has no reference checkout; tests read only these fixtures there.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_REFERENCE = os.environ.get("FP4T_REFERENCE", "")


def load_reference(ref_root: str = DEFAULT_REFERENCE):
    """Return (quantize_module, swizzle_module) of the reference checkout at `ref_root`
    (argument, or the FP4T_REFERENCE environment variable), or None if there is none."""
    if not ref_root:
        return None
    qpath = os.path.join(ref_root, "custom", "quantize.py")
    spath = os.path.join(ref_root, "custom", "swizzle.py")
    if not (os.path.isfile(qpath) and os.path.isfile(spath)):
        return None

    def _raise(*a, **k):
        raise RuntimeError("microxcaling is not available")

    for name in ("microxcaling", "microxcaling.mx", "microxcaling.mx.mx_ops", "microxcaling.mx.specs"):
        if name not in sys.modules:
            sys.modules[name] = types.ModuleType(name)
    sys.modules["microxcaling.mx.mx_ops"].quantize_mx_op = _raise
    sys.modules["microxcaling.mx.specs"].MxSpecs = type("MxSpecs", (dict,), {})

    pkg = types.ModuleType("_fp4t_refpkg")
    pkg.__path__ = [os.path.join(ref_root, "custom")]
    sys.modules["_fp4t_refpkg"] = pkg
    mods = []
    for short, path in (("swizzle", spath), ("quantize", qpath)):
        spec = importlib.util.spec_from_file_location(f"_fp4t_refpkg.{short}", path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"_fp4t_refpkg.{short}"] = mod
        spec.loader.exec_module(mod)
        mods.append(mod)
    return mods[1], mods[0]


def reference_pack(values_f32: torch.Tensor) -> torch.Tensor:
    """The pack kernel's conversion restated for the fixture: RNE, saturate to +-6."""
    sys.path.insert(0, os.path.join(HERE, "..", ".."))
    from oracle.fp4t_oracle import e2m1_encode_rne_sat
    return e2m1_encode_rne_sat(values_f32)


def _inputs(kind: str, rows: int, cols: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    if kind == "normal":
        x = torch.randn(rows, cols, generator=g)
    elif kind == "outlier":
        x = torch.randn(rows, cols, generator=g)
        x = torch.where(torch.rand(rows, cols, generator=g) < 1e-2, x * 50, x)
    elif kind == "grad":
        x = torch.randn(rows, cols, generator=g) * 1e-3
    elif kind == "weight":
        x = torch.randn(rows, cols, generator=g) * 0.02
    elif kind == "ties":
        # values that land exactly on rounding ties and grid points after scaling by amax=6
        grid = torch.tensor([0, .25, .5, .75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 6, -0.0,
                             -.25, -.75, -1.25, -1.75, -2.5, -3.5, -5, -6, 1e-3, -1e-3, 0.24, 0.26,
                             4.99, 5.01, 3.49, 3.51])
        idx = torch.randint(0, grid.numel(), (rows, cols), generator=g)
        x = grid[idx]
        x[:, ::16] = 6.0
    elif kind == "tiny":
        x = torch.randn(rows, cols, generator=g) * 1e-5
        x[0, :16] = 0.0
        x[1, :16] = -0.0
    elif kind == "huge":
        x = torch.randn(rows, cols, generator=g) * 1000.0
    else:
        raise ValueError(kind)
    return x.to(torch.bfloat16)


CASES = [
    ("normal", 128, 256, 1), ("outlier", 64, 512, 2), ("grad", 256, 64, 3), ("weight", 192, 192, 4),
    ("ties", 32, 64, 5), ("tiny", 16, 32, 6), ("huge", 48, 96, 7), ("normal", 2, 32, 8),
    ("grad", 50 * 2, 48, 9),
]

# cases for the public entry points (rows and cols multiples of 16, at least two blocks each way)
API_CASES = [("normal", 64, 128, 11), ("outlier", 32, 512, 12), ("grad", 48, 80, 13), ("weight", 96, 192, 14)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    args = ap.parse_args()
    loaded = load_reference(args.reference)
    if loaded is None:
        raise SystemExit(f"no reference checkout at {args.reference}")
    rq, rs = loaded

    for kind, rows, cols, seed in CASES:
        x = _inputs(kind, rows, cols, seed)
        out = {"x_bits": x.view(torch.int16).numpy()}
        q, s = rq.quantize_nvfp4(x, rowwise=True, simulated=False, stochastic_rounding=False)
        out["codes"] = reference_pack(q).numpy()
        out["scale_bytes"] = s.view(torch.uint8).numpy()
        q2, s2 = rq.q_nvfp4_rowwise(x)
        assert torch.equal(q2, q)
        out["scale_swizzled"] = s2.numpy()
        # stochastic path: the reference draws torch.rand_like on the blocked tensor
        torch.manual_seed(1000 + seed)
        q3, s3 = rq.quantize_nvfp4(x, rowwise=True, simulated=False, stochastic_rounding=True)
        torch.manual_seed(1000 + seed)
        u = torch.rand(rows, cols // 16, 16)
        out["sr_noise"] = u.reshape(rows, cols).numpy()
        out["sr_codes"] = reference_pack(q3).numpy()
        assert torch.equal(s3.view(torch.uint8), s.view(torch.uint8))
        # the transposed operand the reference builds with .T.contiguous()
        if rows % 16 == 0 and rows >= 32:
            xt = x.t().contiguous()
            qt, st = rq.q_nvfp4_rowwise(xt)
            out["codes_t"] = reference_pack(qt).numpy()
            out["scale_swizzled_t"] = st.numpy()
        np.savez_compressed(os.path.join(HERE, f"nvfp4_rowwise_{kind}_{rows}x{cols}.npz"), **out)

    for kind, rows, cols, seed in API_CASES:
        x = _inputs(kind, rows, cols, seed)
        out = {"x_bits": x.view(torch.int16).numpy()}
        for rowwise in (True, False):
            tag = "row" if rowwise else "col"
            out[f"sim_{tag}"] = rq.quantize_nvfp4(x, rowwise=rowwise, simulated=True).contiguous().numpy()
            q, s = rq.quantize_nvfp4(x, rowwise=rowwise, simulated=False)
            out[f"q_{tag}"] = q.contiguous().numpy()
            out[f"s_{tag}"] = s.contiguous().view(torch.uint8).numpy()
            fn = rq.q_nvfp4_rowwise if rowwise else rq.q_nvfp4_colwise
            qv, sw_ = fn(x)
            assert torch.equal(qv, q.contiguous())
            out[f"sw_{tag}"] = sw_.contiguous().numpy()
            # stochastic rounding: the reference draws rand_like on the blocked tensor.  Row-wise
            # that tensor is contiguous [R, C/16, 16].  Column-wise it is a VIEW of the transposed
            # input (strides (1, 16 C, C)), rand_like keeps those strides and fills memory order,
            # so the stream is consumed in the layout of the original [R, C] tensor: the noise
            # of element (r, c) is draw number r*C + c.
            torch.manual_seed(2000 + seed)
            qs, ss = fn(x, sr=True)
            torch.manual_seed(2000 + seed)
            u = torch.rand(rows, cols // 16, 16) if rowwise else torch.rand(rows, cols)
            out[f"sr_noise_{tag}"] = u.numpy()
            out[f"sr_q_{tag}"] = qs.numpy()
            assert torch.equal(ss, sw_)
        np.savez_compressed(os.path.join(HERE, f"nvfp4_api_{kind}_{rows}x{cols}.npz"), **out)

    g = torch.Generator().manual_seed(99)
    sw = {}
    for (a, b) in [(128, 4), (4, 128), (8192 // 64, 16), (50, 12), (300, 5), (129, 9), (16, 256), (2, 2)]:
        m = torch.randint(0, 256, (a, b), generator=g, dtype=torch.int32).to(torch.uint8)
        sw[f"in_{a}x{b}"] = m.numpy()
        sw[f"row_{a}x{b}"] = rs.swizzle_rowwise_scale(m).numpy()
        sw[f"col_{a}x{b}"] = rs.swizzle_colwise_scale(m).contiguous().numpy()
    np.savez_compressed(os.path.join(HERE, "swizzle_cases.npz"), **sw)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
