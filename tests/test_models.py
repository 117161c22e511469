"""Model wiring, following the reference's tests/test_models.py."""
import pytest
import torch
import torch.nn as nn

from custom import CustomLinear
from models import LINEAR_IMPL, REF_IMPL, TinyViT, TransformerBlock

IMPL_TESTLIST = list(LINEAR_IMPL.keys())
NO_CPU_IMPL = ["custom_aten", "cublaslt", "cublaslt_mxfp8", "cublaslt_nvfp4", "cublaslt_nvf4_fw_mxf8_bw"]


def test_recipe_strings():
    assert REF_IMPL == ["torch", "custom_py", "custom_aten", "cublaslt", "cublaslt_mxfp8", "cublaslt_nvfp4",
                        "cublaslt_nvf4_fw_mxf8_bw"]
    assert set(REF_IMPL) <= set(LINEAR_IMPL)


@pytest.mark.parametrize("linear_impl", IMPL_TESTLIST)
def test_block_construction(linear_impl):
    blk = TransformerBlock(E=64, F=128, H=4, impl=linear_impl)
    assert isinstance(blk.attn.k_proj, LINEAR_IMPL[linear_impl])
    assert isinstance(blk.ffn.down_proj, LINEAR_IMPL[linear_impl])
    assert blk.attn.attn_scale == pytest.approx(4.0)     # scores are multiplied by sqrt(dh)


@pytest.mark.parametrize("linear_impl", IMPL_TESTLIST)
def test_block_forward_cpu(linear_impl):
    blk = TransformerBlock(E=64, F=128, H=4, impl=linear_impl)
    x = torch.randn(32, 10, 64)
    if linear_impl in NO_CPU_IMPL:
        with pytest.raises((AssertionError, NotImplementedError, ValueError)):
            blk(x)
    else:
        assert blk(x).shape == x.shape


@pytest.mark.parametrize("linear_impl", IMPL_TESTLIST)
def test_vit_construction(linear_impl):
    vit = TinyViT(linear_impl=linear_impl)
    names = [n for n, _ in vit.named_modules()]
    assert "encoder.attn.q_proj" in names and "encoder.ffn.up_proj" in names and "mlp_head" in names
    for n, m in vit.named_modules():
        if isinstance(m, nn.Linear) and "_proj" in n:
            assert isinstance(m, LINEAR_IMPL[linear_impl]), n
    assert type(vit.mlp_head) is nn.Linear
    deep = TinyViT(linear_impl=linear_impl, patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=6)
    assert sum(isinstance(m, LINEAR_IMPL[linear_impl]) and "_proj" in n for n, m in deep.named_modules()) == 36
    if linear_impl == "custom_py":
        assert isinstance(vit.encoder.attn.q_proj, CustomLinear)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=lambda x: str(x).split(".")[-1])
@pytest.mark.parametrize("linear_impl", IMPL_TESTLIST)
def test_block_forward_cuda(linear_impl, dtype):
    blk = TransformerBlock(E=64, F=128, H=4, impl=linear_impl).to(device="cuda", dtype=dtype)
    x = torch.randn(32, 10, 64, device="cuda", dtype=dtype)
    y = blk(x)
    assert y.shape == x.shape and torch.isfinite(y).all()


@pytest.mark.gpu
@pytest.mark.parametrize("linear_impl", ["cublaslt_nvfp4", "cublaslt_mxfp8", "cublaslt_nvf4_fw_mxf8_bw"])
def test_vit_train_step_cuda(linear_impl):
    torch.manual_seed(0)
    vit = TinyViT(linear_impl=linear_impl, patch_size=4, embed_dim=192, num_heads=3, mlp_ratio=4.0, depth=2).cuda()
    opt = torch.optim.AdamW(vit.parameters(), lr=1e-3)
    x = torch.rand(64, 1, 28, 28, device="cuda")
    y = torch.randint(0, 10, (64,), device="cuda")
    losses = []
    for _ in range(8):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = nn.functional.cross_entropy(vit(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert all(l == l for l in losses)
    assert losses[-1] < losses[0]            # memorising one batch must reduce the loss
    from backend import ops
    ops.check_status()


def test_block_options_keep_the_module_tree():
    """fused_norm / fuse_qkv / sdpa / fuse_gelu change kernels, not parameters: the state dict of a
    model built with them loads into the reference's module tree and back."""
    from custom import FusedLayerNorm
    plain = TinyViT(embed_dim=64, num_heads=4, depth=2, linear_impl="cublaslt_nvfp4")
    opts = TinyViT(embed_dim=64, num_heads=4, depth=2, linear_impl="cublaslt_nvfp4", fused_norm=True, fuse_qkv=True,
                   sdpa=True, fuse_gelu=True)
    assert list(plain.state_dict().keys()) == list(opts.state_dict().keys())
    opts.load_state_dict(plain.state_dict())
    plain.load_state_dict(opts.state_dict())
    blk = opts.encoder[0]
    assert isinstance(blk.attn.preln, FusedLayerNorm) and isinstance(blk.ffn["preln"], FusedLayerNorm)
    assert isinstance(blk.attn.preln, nn.LayerNorm)                  # a subclass: isinstance checks of callers keep working
    assert blk.attn.fuse_qkv and blk.attn.sdpa and blk.fuse_gelu


def test_library_layernorm_has_no_cpu_path():
    from custom import FusedLayerNorm
    ln = FusedLayerNorm(64)
    with pytest.raises(NotImplementedError):
        ln(torch.randn(4, 64))
    with pytest.raises(ValueError):
        FusedLayerNorm((8, 64))                                      # last dimension only


def test_options_with_torch_linears_run_on_cpu_where_they_can():
    """fuse_qkv needs a quantized layer class and is ignored for nn.Linear; sdpa is plain torch."""
    blk = TransformerBlock(E=64, F=128, H=4, impl="torch", fuse_qkv=True, sdpa=True).eval()
    ref = TransformerBlock(E=64, F=128, H=4, impl="torch").eval()
    ref.load_state_dict(blk.state_dict())
    x = torch.randn(4, 10, 64)
    with torch.no_grad():
        assert torch.allclose(blk(x), ref(x), rtol=1e-4, atol=1e-5)
