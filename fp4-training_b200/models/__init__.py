from .transformer_block import TransformerBlock, LINEAR_IMPL, REF_IMPL
from .vit import TinyViT

__all__ = ["TransformerBlock", "TinyViT", "LINEAR_IMPL", "REF_IMPL"]
