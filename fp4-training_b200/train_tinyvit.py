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
curve; --log writes per-step losses as JSON lines.
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


def build_model(impl, depth, device):
    return TinyViT(img_size=28, patch_size=4, in_chans=1, num_classes=10, embed_dim=192, num_heads=3,
                   mlp_ratio=4.0, linear_impl=impl, depth=depth).to(device)


def train(impl="cublaslt_nvfp4", steps=200, warmup=5, batch=512, depth=6, seed=0, lr=1e-3, device=None, log=None,
          fp32=False):
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
    model = build_model(impl, depth, device)
    broadcast_parameters(model)
    opt = torch.optim.AdamW(model.parameters(), lr=lr)
    reducer = GradAllReducer(model.parameters())
    crit = nn.CrossEntropyLoss()
    torch.manual_seed(seed + 1000 * (rank + 1))        # data, dropout and rounding noise differ per rank
    gen = torch.Generator(device=device).manual_seed(seed + 77 * (rank + 1))
    losses = []
    t0 = None
    for step in range(warmup + steps):
        if step == warmup:
            if device.type == "cuda":
                torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
        x = torch.rand(batch, 1, 28, 28, device=device, generator=gen)
        y = torch.randint(0, 10, (batch,), device=device, generator=gen)
        with torch.autocast(device.type, dtype=torch.bfloat16, enabled=not fp32):
            loss = crit(model(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        reducer.finish()
        opt.step()
        losses.append(loss.detach())
    if device.type == "cuda":
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    dt = time.perf_counter() - t0
    losses = [float(v) for v in losses]
    if log and rank == 0:
        with open(log, "w") as f:
            for i, v in enumerate(losses):
                f.write(json.dumps({"step": i, "loss": v}) + "\n")
    return {"impl": impl, "steps": steps, "world": world, "batch_per_gpu": batch, "depth": depth,
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
    a = ap.parse_args()
    out = train(a.impl, a.steps, a.warmup, a.batch_size, a.depth, a.seed, a.lr, None, a.log, a.fp32)
    if int(os.environ.get("RANK", "0")) == 0:
        out["losses"] = out["losses"][:: max(1, len(out["losses"]) // 20)]
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
