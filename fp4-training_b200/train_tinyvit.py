#!/usr/bin/env python
"""TinyViT-style classifier trained with quantized linears on synthetic data, optionally data
parallel (one process per GPU under torchrun).

    python train_tinyvit.py --impl cublaslt_nvfp4 --steps 200
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 train_tinyvit.py ...

Model: 28x28x1 images, patch 4 (49 tokens + CLS), hidden 192, depth 6, 3 heads, MLP 768 -- the
reference's TinyViT (models/vit.py) with `depth` blocks.  Data: images ~ U(0,1), labels uniform
over 10 classes, 512 per GPU per step, seeded per rank (MNIST itself needs a download).
Optimizer AdamW lr 1e-3, bf16 autocast as in the reference's training loop
(main_train_tinyvit_mnist.py:35-38,62-76).  Prints one JSON line with steps/s and the loss
curve; --log writes per-step losses as JSON lines; --graph replays the step from CUDA graphs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
from torch import nn  # noqa: E402

from dp import GradAllReducer, broadcast_parameters  # noqa: E402
from models import REF_IMPL, TinyViT  # noqa: E402


def build_model(impl, depth, device, fused_norm=False, fuse_qkv=False, sdpa=False):
    return TinyViT(img_size=28, patch_size=4, in_chans=1, num_classes=10, embed_dim=192, num_heads=3,
                   mlp_ratio=4.0, linear_impl=impl, depth=depth, fused_norm=fused_norm, fuse_qkv=fuse_qkv, sdpa=sdpa).to(device)


def _sync(device, world):
    if device.type == "cuda":
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()


def train(impl="cublaslt_nvfp4", steps=200, warmup=5, batch=512, depth=6, seed=0, lr=1e-3, device=None, log=None,
          fp32=False, graph=False, fused_norm=False, fuse_qkv=False, sdpa=False):
    """graph=True (CUDA only): forward + backward and the optimizer step are captured once into
    two CUDA graphs and replayed per step, with the gradient all-reduce (one NCCL call on a flat
    buffer that all `.grad` tensors are views of) between them.  The step is launch-bound at
    this model size (a few hundred small kernels), so replaying removes most of its cost; the
    in-kernel stochastic-rounding noise is refreshed each replay through a device counter
    (fp4t_set_seed_offset_word)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device(device or (f"cuda:{local}" if torch.cuda.is_available() else "cpu"))
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo")
    torch.manual_seed(seed)
    model = build_model(impl, depth, device, fused_norm, fuse_qkv, sdpa)
    broadcast_parameters(model)
    crit = nn.CrossEntropyLoss()
    torch.manual_seed(seed + 1000 * (rank + 1))        # data, dropout and rounding noise differ per rank
    gen = torch.Generator(device=device).manual_seed(seed + 77 * (rank + 1))

    def batch_of():
        x = torch.rand(batch, 1, 28, 28, device=device, generator=gen)
        y = torch.randint(0, 10, (batch,), device=device, generator=gen)
        return x, y

    losses = []
    t0 = None
    if graph:
        if device.type != "cuda":
            raise ValueError("graph=True needs a CUDA device")
        from backend import _lib
        params = [p for p in model.parameters() if p.requires_grad]
        flat = torch.zeros(sum(p.numel() for p in params), dtype=params[0].dtype, device=device)
        off = 0
        for p in params:                                  # every .grad is a view of one flat buffer
            p.grad = flat[off:off + p.numel()].view_as(p)
            off += p.numel()
        opt = torch.optim.AdamW(params, lr=lr, capturable=True)
        counter = torch.zeros(1, dtype=torch.int64, device=device)
        _lib.check(_lib.lib().fp4t_set_seed_offset_word(counter.data_ptr()), "fp4t_set_seed_offset_word")
        sx, sy = batch_of()

        def fwd_bwd():
            flat.zero_()
            counter.add_(1)
            with torch.autocast(device.type, dtype=torch.bfloat16, enabled=not fp32):
                loss = crit(model(sx), sy)
            loss.backward()
            return loss.detach()

        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):                            # eager passes: lazy initialisation, allocator warm-up
                fwd_bwd()
                if world > 1:
                    dist.all_reduce(flat)
                    flat.div_(world)
                opt.step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g_step, g_opt = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_step):
            static_loss = fwd_bwd()
        with torch.cuda.graph(g_opt):
            opt.step()
        try:
            for step in range(warmup + steps):
                if step == warmup:
                    _sync(device, world)
                    t0 = time.perf_counter()
                x, y = batch_of()
                sx.copy_(x)
                sy.copy_(y)
                g_step.replay()
                if world > 1:
                    dist.all_reduce(flat)
                    flat.div_(world)
                g_opt.replay()
                losses.append(static_loss.clone())
            _sync(device, world)
        finally:
            _lib.lib().fp4t_set_seed_offset_word(None)
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=lr)
        reducer = GradAllReducer(model.parameters())
        for step in range(warmup + steps):
            if step == warmup:
                _sync(device, world)
                t0 = time.perf_counter()
            x, y = batch_of()
            with torch.autocast(device.type, dtype=torch.bfloat16, enabled=not fp32):
                loss = crit(model(x), y)
            opt.zero_grad(set_to_none=True)
            loss.backward()
            reducer.finish()
            opt.step()
            losses.append(loss.detach())
        _sync(device, world)
    dt = time.perf_counter() - t0
    losses = [float(v) for v in losses]
    if log and rank == 0:
        with open(log, "w") as f:
            for i, v in enumerate(losses):
                f.write(json.dumps({"step": i, "loss": v}) + "\n")
    return {"impl": impl, "steps": steps, "world": world, "batch_per_gpu": batch, "depth": depth, "graph": bool(graph),
            "fused_norm": bool(fused_norm), "fuse_qkv": bool(fuse_qkv), "sdpa": bool(sdpa),
            "steps_per_s": steps / dt, "images_per_s": steps * batch * world / dt, "first_loss": losses[0],
            "last_loss": losses[-1], "losses": losses}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="cublaslt_nvfp4", choices=REF_IMPL)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("-b", "--batch-size", type=int, default=512)
    ap.add_argument("--depth", type=int, default=6)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("-lr", type=float, default=1e-3)
    ap.add_argument("--fp32", action="store_true")
    ap.add_argument("--log", default=None)
    ap.add_argument("--graph", action="store_true", help="replay the step from CUDA graphs")
    ap.add_argument("--fused-norm", action="store_true", help="LayerNorms on the library's kernels")
    ap.add_argument("--fuse-qkv", action="store_true", help="q / k / v as one quantization and one GEMM")
    ap.add_argument("--sdpa", action="store_true", help="attention core through torch's scaled_dot_product_attention")
    a = ap.parse_args()
    out = train(a.impl, a.steps, a.warmup, a.batch_size, a.depth, a.seed, a.lr, None, a.log, a.fp32, a.graph, a.fused_norm, a.fuse_qkv, a.sdpa)
    if int(os.environ.get("RANK", "0")) == 0:
        out["losses"] = out["losses"][:: max(1, len(out["losses"]) // 20)]
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
