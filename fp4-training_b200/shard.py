"""Column-sharded block-scaled GEMM for the GEMM-sweep configuration on several GPUs.

`D[M, N] = X[M, K] . W[N, K]^T` with the `[N, K]` operand sharded on N: rank r quantizes and keeps
rows `[r N/g, (r+1) N/g)` of W once, X is replicated, every rank computes its column block
`D[:, r N/g : (r+1) N/g]` with the library's GEMM, and one all-gather assembles D on every rank.
The blocks are independent (no reduction), so the result is bit-identical to the unsharded GEMM:
each output element accumulates over K in the same order whichever rank computes it.

The gathered buffer is `[g, M, N/g]` (contiguous per rank, which is what NCCL's all-gather
writes); `__call__` returns it as the logical `[M, N]` matrix through a strided view
`[M, g, N/g]`, or as a contiguous `[M, N]` copy with `contiguous=True`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _default_ops(fmt):
    from backend import ops
    if fmt == "nvfp4":
        return (lambda t: ops.quantize_nvfp4(t, True, False)[:2]), ops.gemm_nvfp4
    if fmt == "mxfp8":
        return (lambda t: ops.quantize_mxfp8(t, True, False)[:2]), ops.gemm_mxfp8
    raise ValueError(f"unknown format {fmt!r}")


class ColumnShardedGemm:
    def __init__(self, w: torch.Tensor, fmt: str = "nvfp4", process_group=None, quantize=None, gemm=None):
        """w: the full `[N, K]` operand (every rank passes the same tensor; only this rank's rows
        are quantized and kept).  `quantize(t) -> (codes, scales)` and
        `gemm(pc, psf, qc, qsf, bias, out_dtype) -> [rows(p), rows(q)]` default to the library's
        kernels for `fmt`; they exist as parameters so the host logic can be exercised on CPU."""
        if w.dim() != 2:
            raise ValueError("w must be 2-D [N, K]")
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        n = w.shape[0]
        if n % self.world:
            raise ValueError(f"N={n} is not divisible by the number of ranks ({self.world})")
        self.n, self.k = n, w.shape[1]
        self.cols = n // self.world
        self.lo = self.rank * self.cols
        if quantize is None or gemm is None:
            q, g = _default_ops(fmt)
            quantize, gemm = quantize or q, gemm or g
        self._quantize, self._gemm = quantize, gemm
        self.wc, self.wsf = quantize(w[self.lo:self.lo + self.cols].contiguous())

    def local_block(self, x: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
        """This rank's column block `[M, N/g]` (no communication)."""
        if x.dim() != 2 or x.shape[1] != self.k:
            raise ValueError(f"x must be [M, {self.k}]")
        xc, xsf = self._quantize(x)
        return self._gemm(xc, xsf, self.wc, self.wsf, None, out_dtype)

    def __call__(self, x: torch.Tensor, out_dtype=torch.bfloat16, contiguous: bool = False) -> torch.Tensor:
        local = self.local_block(x, out_dtype)
        if self.world == 1:
            return local
        m = local.shape[0]
        gathered = torch.empty((self.world, m, self.cols), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(gathered.view(-1), local.contiguous().view(-1), group=self.group)
        view = gathered.permute(1, 0, 2)          # [M, g, N/g]: column r*cols + j lives at [., r, j]
        return view.reshape(m, self.n) if contiguous else view
