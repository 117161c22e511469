"""Data-parallel gradient exchange on CPU ranks (gloo, world size 2): the averaged gradients
equal the gradients of the same model over the concatenated batch, and a rank that never joins
makes the others fail with an error instead of hanging."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "fp4-training_b200"))
    from dp import GradAllReducer, broadcast_parameters
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(100 + rank)                      # different initial weights per rank ...
    model = nn.Sequential(nn.Linear(16, 32), nn.GELU(), nn.Linear(32, 8))
    broadcast_parameters(model)                        # ... made equal to rank 0's here
    reducer = GradAllReducer(model.parameters(), bucket_bytes=1024)   # several buckets
    assert len(reducer.buckets) > 1
    g = torch.Generator().manual_seed(5)
    x_all, y_all = torch.randn(8, 16, generator=g), torch.randn(8, 8, generator=g)
    xs, ys = x_all[rank * 4:(rank + 1) * 4], y_all[rank * 4:(rank + 1) * 4]
    out = []
    for _ in range(2):                                  # two steps: buckets are reusable
        model.zero_grad(set_to_none=True)
        nn.functional.mse_loss(model(xs), ys).backward()
        reducer.finish()
        out.append([p.grad.clone() for p in model.parameters()])
    # numpy arrays travel by value; tensors would be handed over through the sender's descriptor
    # server, which is gone if this process exits before the parent has read the queue
    q.put((rank, [p.detach().numpy().copy() for p in model.parameters()], [t.numpy().copy() for t in out[-1]]))
    dist.destroy_process_group()


def test_two_rank_gradient_average_matches_full_batch():
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted([q.get(timeout=120) for _ in procs], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, w0, g0), (_, w1, g1) = [(r, [torch.from_numpy(a) for a in w], [torch.from_numpy(a) for a in g])
                                for r, w, g in results]
    for a, b in zip(w0, w1):
        assert torch.equal(a, b)
    for a, b in zip(g0, g1):
        assert torch.allclose(a, b, atol=1e-7)
    # reference: one process, full batch (mean over 8 samples = average of the two 4-sample means)
    model = nn.Sequential(nn.Linear(16, 32), nn.GELU(), nn.Linear(32, 8))
    with torch.no_grad():
        for p, w in zip(model.parameters(), w0):
            p.copy_(w)
    g = torch.Generator().manual_seed(5)
    x_all, y_all = torch.randn(8, 16, generator=g), torch.randn(8, 8, generator=g)
    nn.functional.mse_loss(model(x_all), y_all).backward()
    for p, got in zip(model.parameters(), g0):
        assert torch.allclose(p.grad, got, atol=1e-6)


def _accum_worker(rank, world, port, q):
    """Gradient accumulation (two backwards per step, with and without no_sync) and a parameter
    that takes no part in the loss while its .grad tensor persists between steps."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "fp4-training_b200"))
    from dp import GradAllReducer, broadcast_parameters
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(7)
    model = nn.Sequential(nn.Linear(16, 32), nn.GELU(), nn.Linear(32, 8))
    unused = nn.Linear(8, 8)
    broadcast_parameters(model)
    params = list(model.parameters()) + list(unused.parameters())
    reducer = GradAllReducer(params, bucket_bytes=1024)
    g = torch.Generator().manual_seed(5)
    x_all, y_all = torch.randn(16, 16, generator=g), torch.randn(16, 8, generator=g)
    # rank r owns micro-batches 2r and 2r+1 (4 samples each)
    mb = [(x_all[i * 4:(i + 1) * 4], y_all[i * 4:(i + 1) * 4]) for i in range(4)]
    mine = mb[2 * rank:2 * rank + 2]
    res = {}
    for mode in ("no_sync", "plain"):
        for step in range(2):
            for p in params:
                if p.grad is not None:
                    p.grad.zero_()                      # set_to_none=False style: stale tensors stay
            if step == 0:
                # give the unused layer a stale nonzero gradient that must NOT be averaged back in
                for p in unused.parameters():
                    p.grad = torch.full_like(p, 3.0)
                    p.grad.zero_()
            if mode == "no_sync":
                with reducer.no_sync():
                    nn.functional.mse_loss(model(mine[0][0]), mine[0][1]).backward()
                nn.functional.mse_loss(model(mine[1][0]), mine[1][1]).backward()
            else:
                nn.functional.mse_loss(model(mine[0][0]), mine[0][1]).backward()
                nn.functional.mse_loss(model(mine[1][0]), mine[1][1]).backward()
            reducer.finish()
        res[mode] = [p.grad.clone().numpy().copy() for p in params]
    q.put((rank, res))
    dist.destroy_process_group()


def test_accumulation_and_unused_parameters():
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_accum_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # reference: sum over the four micro-batch mean losses, divided by the 2 ranks
    torch.manual_seed(7)
    model = nn.Sequential(nn.Linear(16, 32), nn.GELU(), nn.Linear(32, 8))
    g = torch.Generator().manual_seed(5)
    x_all, y_all = torch.randn(16, 16, generator=g), torch.randn(16, 8, generator=g)
    for i in range(4):
        nn.functional.mse_loss(model(x_all[i * 4:(i + 1) * 4]), y_all[i * 4:(i + 1) * 4]).backward()
    want = [p.grad / 2 for p in model.parameters()]
    for mode in ("no_sync", "plain"):
        for rank in (0, 1):
            got = [torch.from_numpy(a) for a in results[rank][mode]]
            for w, gt in zip(want, got[:len(want)]):
                assert torch.allclose(w, gt, atol=1e-6), f"{mode}: rank {rank} gradient differs from the full-batch one"
            for gt in got[len(want):]:
                assert float(gt.abs().max()) == 0.0, f"{mode}: an unused parameter received a gradient"


def _lonely_worker(port, q):
    """Rank 0 of a 2-rank job whose rank 1 never starts."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK="0", WORLD_SIZE="2")
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        q.put("joined")
    except Exception as e:  # noqa: BLE001
        q.put("error: " + type(e).__name__)


def test_missing_rank_is_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely_worker, args=(_free_port(), q))
    p.start()
    msg = q.get(timeout=90)
    p.join(timeout=30)
    assert msg.startswith("error")


def test_single_process_is_a_no_op():
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "fp4-training_b200"))
    from dp import GradAllReducer
    m = nn.Linear(4, 4)
    r = GradAllReducer(m.parameters())
    m(torch.randn(2, 4)).sum().backward()
    g = m.weight.grad.clone()
    r.finish()
    assert torch.equal(g, m.weight.grad)
    r.remove()


def test_shard_plan_covers_the_buffer_in_16_byte_shards():
    """Host arithmetic of the copy-engine exchange: every rank's shard is a whole number of
    16-byte items and the shards cover the buffer."""
    from dp import shard_plan
    for world in range(1, 9):
        for numel in (1, 7, 8, 9, 8024, 4096 * 4096 + 4096, 192 * 192 * 31 + 5):
            shard, padded = shard_plan(numel, world)
            assert shard % 8 == 0 and padded == shard * world and padded >= numel
            assert padded - numel < world * 8 + world, (numel, world, shard, padded)
