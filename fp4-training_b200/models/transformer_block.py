"""Pre-LN transformer block whose six projections come from the `linear_impl` recipe
switch (reference: models/transformer_block.py:16-106)."""
import torch.nn.functional as F
from torch import nn

from custom import (
    AddmmLinear,
    CublasltFwdNvfp4BwdMxfp8Linear,
    CublasltLinear,
    CublasltMxfp8Linear,
    CublasltNvfp4Linear,
    CustomLinear,
    FusedLayerNorm,
)

LINEAR_IMPL = {
    "torch": nn.Linear,
    "custom_py": CustomLinear,
    "custom_aten": AddmmLinear,
    "cublaslt": CublasltLinear,
    "cublaslt_mxfp8": CublasltMxfp8Linear,
    "cublaslt_nvfp4": CublasltNvfp4Linear,
    "cublaslt_nvf4_fw_mxf8_bw": CublasltFwdNvfp4BwdMxfp8Linear,
}

REF_IMPL = ["torch", "custom_py", "custom_aten", "cublaslt", "cublaslt_mxfp8", "cublaslt_nvfp4",
            "cublaslt_nvf4_fw_mxf8_bw"]


class AttentionBlock(nn.Module):
    """x + o_proj(softmax(q k^T * attn_scale) v).  As in the reference
    (models/transformer_block.py:74,95) attn_scale is 1 / dh**-0.5, i.e. the scores are
    MULTIPLIED by sqrt(dh); loss-curve parity depends on keeping that."""

    def __init__(self, E, H, dropout=0.1, impl="torch", fused_norm=False, fuse_qkv=False, sdpa=False):
        super().__init__()
        self.fuse_qkv = fuse_qkv        # an addition: q / k / v as one quantization + one GEMM over stacked weights
        # an addition: the attention core through torch's scaled_dot_product_attention (a library
        # kernel, the same for every recipe) instead of the reference's matmul / softmax / dropout
        # sequence with its layout copies; same arithmetic, the dropout mask comes from another generator
        self.sdpa = sdpa
        assert E % H == 0, "head size is not multiple of embedding size"
        self.E, self.H, self.dh = E, H, E // H
        self.attn_scale = 1 / (self.dh ** -0.5)
        self.preln = FusedLayerNorm(E) if fused_norm else nn.LayerNorm(E)
        linear = LINEAR_IMPL[impl]
        self.q_proj = linear(E, E)
        self.k_proj = linear(E, E)
        self.v_proj = linear(E, E)
        self.o_proj = linear(E, E)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x):
        B, L, E = x.shape
        residual = x
        x = self.preln(x)
        if self.fuse_qkv and hasattr(self.q_proj, "forward_stacked"):
            q, k, v = self.q_proj.forward_stacked([self.q_proj, self.k_proj, self.v_proj], x)
        else:
            q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        q = q.view(B, L, self.H, self.dh).transpose(1, 2)
        if self.sdpa:
            k = k.view(B, L, self.H, self.dh).transpose(1, 2)
            v = v.view(B, L, self.H, self.dh).transpose(1, 2)
            attn = F.scaled_dot_product_attention(q, k, v, dropout_p=self.dropout.p if self.training else 0.0,
                                                  scale=self.attn_scale)
            return residual + self.o_proj(attn.transpose(1, 2).reshape(B, L, E))
        k_t = k.view(B, L, self.H, self.dh).transpose(1, 2).transpose(-2, -1)
        v = v.view(B, L, self.H, self.dh).transpose(1, 2)
        prob = self.dropout(F.softmax((q @ k_t) * self.attn_scale, dim=-1))
        attn = (prob @ v).transpose(1, 2).contiguous().view(B, L, E)
        return residual + self.o_proj(attn)


class TransformerBlock(nn.Module):
    def __init__(self, E, F, H, dropout=0.1, impl="torch", fuse_gelu=False, fused_norm=False, fuse_qkv=False, sdpa=False):
        super().__init__()
        self.E, self.F, self.H, self.impl = E, F, H, impl
        self.fuse_gelu = fuse_gelu      # an addition: see forward()
        # fused_norm (an addition): the two `preln` modules run on the library's LayerNorm kernels
        # (same parameters and state dict as nn.LayerNorm)
        self.attn = AttentionBlock(E, H, dropout, impl=impl, fused_norm=fused_norm, fuse_qkv=fuse_qkv, sdpa=sdpa)
        linear = LINEAR_IMPL[impl]
        self.ffn = nn.ModuleDict({
            "preln": FusedLayerNorm(E) if fused_norm else nn.LayerNorm(E),
            "up_proj": linear(E, F),
            "act": nn.GELU(),
            "act_dropout": nn.Dropout(dropout),
            "down_proj": linear(F, E),
            "dropout": nn.Dropout(dropout),
        })

    def forward(self, x):
        hidden = self.attn(x)
        residual = hidden           # the FFN residual is the attention output
        ffn = self.ffn
        act_dropout_off = (not self.training) or ffn["act_dropout"].p == 0.0
        if self.fuse_gelu and act_dropout_off and hasattr(ffn["down_proj"], "forward_gelu"):
            # GELU goes into the quantizer of down_proj's input operand: same values, one
            # kernel and one HBM round trip less (only where no dropout sits between them)
            hidden = ffn["dropout"](ffn["down_proj"].forward_gelu(ffn["up_proj"](ffn["preln"](hidden))))
            return residual + hidden
        for layer in ffn.values():
            hidden = layer(hidden)
        return residual + hidden
