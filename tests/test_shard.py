"""Column-sharded GEMM (GEMM-sweep configuration on several GPUs).

CPU part (gloo, two ranks): the host logic -- shard bounds, gather layout, strided view -- with a
plain matmul standing in for the kernel.  GPU part (two GPUs, skipped otherwise): the sharded
product is bit-identical to the unsharded library GEMM."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _paths():
    for p in (ROOT, os.path.join(ROOT, "fp4-training_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)


def _cpu_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    _paths()
    from shard import ColumnShardedGemm
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(3)
    w = torch.randn(24, 16, generator=g)
    x = torch.randn(10, 16, generator=g)
    sg = ColumnShardedGemm(w, quantize=lambda t: (t, None),
                           gemm=lambda pc, ps, qc, qs, b, dt: (pc @ qc.t()).to(dt))
    assert (sg.lo, sg.cols) == (rank * 12, 12)
    view = sg(x, out_dtype=torch.float32)
    full = sg(x, out_dtype=torch.float32, contiguous=True)
    want = x @ w.t()
    ok = view.shape == (10, 2, 12) and torch.equal(view.reshape(10, 24), want) and torch.equal(full, want) \
        and full.is_contiguous() and torch.equal(sg.local_block(x, torch.float32), want[:, sg.lo:sg.lo + 12])
    q.put((rank, bool(ok)))
    dist.destroy_process_group()


def test_two_rank_sharding_and_gather_layout_cpu():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_cpu_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, True), (1, True)]


def test_indivisible_n_is_rejected():
    _paths()
    from shard import ColumnShardedGemm
    sg = ColumnShardedGemm(torch.randn(6, 4), quantize=lambda t: (t, None),
                           gemm=lambda pc, ps, qc, qs, b, dt: (pc @ qc.t()).to(dt))
    assert sg.world == 1 and torch.equal(sg(torch.ones(2, 4), torch.float32), torch.ones(2, 4) @ sg.wc.t())
    with pytest.raises(ValueError):
        ColumnShardedGemm(torch.randn(4), quantize=lambda t: (t, None), gemm=None)


def _gpu_worker(rank, world, port, fmt, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    _paths()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    try:
        from backend import ops
        from shard import ColumnShardedGemm
        g = torch.Generator(device=dev).manual_seed(9)          # the same operands on every rank
        w = torch.randn(2048, 4096, device=dev, generator=g).to(torch.bfloat16)
        x = torch.randn(1024, 4096, device=dev, generator=g).to(torch.bfloat16)
        sg = ColumnShardedGemm(w, fmt=fmt)
        got = sg(x, contiguous=True)
        quant = ops.quantize_nvfp4 if fmt == "nvfp4" else ops.quantize_mxfp8
        gemm = ops.gemm_nvfp4 if fmt == "nvfp4" else ops.gemm_mxfp8
        wc, wsf, _, _ = quant(w, True, False)
        xc, xsf, _, _ = quant(x, True, False)
        want = gemm(xc, xsf, wc, wsf, None, torch.bfloat16)
        torch.cuda.synchronize()
        ops.check_status(dev)
        result[rank] = "ok" if torch.equal(got, want) else "sharded product differs from the unsharded GEMM"
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
def test_sharded_gemm_equals_unsharded_two_gpus(fmt):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_worker, args=(r, 2, port, fmt, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("worker did not finish")
        assert p.exitcode == 0
    assert dict(result) == {0: "ok", 1: "ok"}
