"""TinyViT classifier (reference: models/vit.py:12-87) with two additions: `depth`, the
number of transformer blocks (the reference builds exactly one; depth=1 reproduces its
module tree, parameter names included), `fuse_gelu`, which lets the MLP's GELU run inside
the quantizer of the down-projection's input where no dropout sits between them, and
`fused_norm`, which runs the blocks' LayerNorms on the library's kernels, and `fuse_qkv`, which
computes the q / k / v projections with one quantization of their input and one GEMM; `sdpa`
routes the attention core through torch's scaled_dot_product_attention."""
import torch
from torch import nn

from .transformer_block import TransformerBlock


class TinyViT(nn.Module):
    def __init__(self, img_size=28, patch_size=7, in_chans=1, num_classes=10, embed_dim=64, num_heads=4,
                 mlp_ratio=2.0, linear_impl="torch", depth=1, fuse_gelu=False, fused_norm=False, fuse_qkv=False, sdpa=False):
        super().__init__()
        self.linear_impl = linear_impl
        assert img_size % patch_size == 0, "patch_size must divide img_size exactly"
        self.num_patches = (img_size // patch_size) ** 2
        self.patch_embed = nn.Conv2d(in_chans, embed_dim, kernel_size=patch_size, stride=patch_size)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, embed_dim))
        self.pos_embed = nn.Parameter(torch.zeros(1, 1 + self.num_patches, embed_dim))
        nn.init.trunc_normal_(self.pos_embed, std=0.02)
        nn.init.trunc_normal_(self.cls_token, std=0.02)

        def block():
            return TransformerBlock(E=embed_dim, F=int(embed_dim * mlp_ratio), H=num_heads, impl=linear_impl,
                                    fuse_gelu=fuse_gelu, fused_norm=fused_norm, fuse_qkv=fuse_qkv, sdpa=sdpa)

        self.depth = depth
        self.encoder = block() if depth == 1 else nn.Sequential(*[block() for _ in range(depth)])
        self.mlp_head = nn.Linear(embed_dim, num_classes)   # the head is always nn.Linear

    def forward(self, x):
        B = x.size(0)
        x = self.patch_embed(x).flatten(2).transpose(1, 2)
        x = torch.cat((self.cls_token.expand(B, -1, -1), x), dim=1) + self.pos_embed
        x = self.encoder(x)
        return self.mlp_head(x[:, 0])
