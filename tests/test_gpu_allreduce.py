"""In-switch gradient all-reduce (fp4t_allreduce_sum_bf16_multimem) against an fp32 sum.

Needs two GPUs on one NVSwitch with NVLink multicast; skipped otherwise.  Each rank fills the
symmetric buffer with its own bf16 values; after the call every rank must hold the sum, equal to
the fp32 sum of the inputs up to one bf16 rounding (the switch accumulates in fp32 and rounds
once), and identical on all ranks."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, numel, result):
    import sys
    import torch.distributed as dist
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "fp4-training_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    os.environ["NCCL_NVLS_ENABLE"] = "0"      # NCCL is only the checker here
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    try:
        from backend import ops
        from dp import SwitchAllReducer
        try:
            red = SwitchAllReducer(numel, dev)
        except RuntimeError as e:      # no multicast on this box
            result[rank] = f"skip: {e}"
            return
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        for trial in range(3):
            src = torch.randn(red.numel, device=dev, generator=gen).to(torch.bfloat16)
            red.flat.copy_(src)
            want = src.float()
            dist.all_reduce(want)
            torch.cuda.synchronize()
            dist.barrier()
            red.all_reduce(ops.status_word(dev))
            torch.cuda.synchronize()
            ops.check_status(dev)
            got = red.flat.float()
            ulp = torch.clamp(want.abs(), min=2.0 ** -126) * 2.0 ** -7      # one bf16 step at that magnitude
            assert bool(((got - want).abs() <= ulp).all()), "sum differs from the fp32 sum by more than one bf16 step"
            mine = red.flat.clone()
            other = mine.clone()
            dist.broadcast(other, src=0)
            assert torch.equal(mine, other), "ranks hold different sums"
        result[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("numel", [4096 * 4096 + 4096, 8 * 1000 + 8])
def test_switch_allreduce_matches_fp32_sum(numel):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, numel, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("all-reduce worker did not finish")
        assert p.exitcode == 0
    if any(str(v).startswith("skip") for v in result.values()):
        pytest.skip(str(list(result.values())[0]))
    assert dict(result) == {0: "ok", 1: "ok"}


def _copy_worker(rank, world, port, numel, reduce, graph, result):
    import sys
    import torch.distributed as dist
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "fp4-training_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    os.environ["NCCL_NVLS_ENABLE"] = "0"      # NCCL is only the checker here
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    try:
        from backend import ops
        from dp import CopyEngineAllReducer
        try:
            red = CopyEngineAllReducer(numel, dev, reduce=reduce, graph=graph)
        except RuntimeError as e:      # no symmetric memory / multicast on this box
            result[rank] = f"skip: {e}"
            return
        assert red.padded >= numel and red.padded % (8 * world) == 0
        gen = torch.Generator(device=dev).manual_seed(99 + rank)
        for trial in range(4):          # calls 2.. replay the captured sequence and reuse every buffer
            src = torch.randn(numel, device=dev, generator=gen).to(torch.bfloat16)
            red.flat[:numel].copy_(src)
            want = src.float()
            dist.all_reduce(want)
            torch.cuda.synchronize()
            red.all_reduce()
            torch.cuda.synchronize()
            ops.check_status(dev)
            got = red.flat[:numel].float()
            ulp = torch.clamp(want.abs(), min=2.0 ** -126) * 2.0 ** -7
            assert bool(((got - want).abs() <= ulp).all()), "sum differs from the fp32 sum by more than one bf16 step"
            other = red.flat[:numel].clone()
            dist.broadcast(other, src=0)
            assert torch.equal(red.flat[:numel], other), "ranks hold different sums"
        result[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("reduce,graph", [("switch", True), ("sum", True), ("sum", False)])
@pytest.mark.parametrize("numel", [4096 * 4096 + 4096, 8 * 1000 + 24])
def test_copy_engine_allreduce_matches_fp32_sum(numel, reduce, graph):
    """dp.CopyEngineAllReducer (rendezvous + shard reduction kernels, peer copies for the bulk):
    the sum equals the fp32 sum within one bf16 rounding and is identical on both ranks, with the
    in-switch and the plain shard reduction, eagerly and replayed from the captured graph, for a
    length that is not a multiple of world x 8 (padded tail)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_copy_worker, args=(r, 2, port, numel, reduce, graph, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    for p in procs:
        if p.is_alive():
            p.kill()
    vals = [result.get(r) for r in range(2)]
    if any(isinstance(v, str) and v.startswith("skip") for v in vals):
        pytest.skip(str(vals))
    assert vals == ["ok", "ok"], vals
