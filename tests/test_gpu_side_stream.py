"""With fp4t_set_layer_concurrency(1) large layers run part of a layer call on the library's helper
stream (X's quantizer beside W's, dgrad beside wgrad) and join: results are those of the
sequential call bit for bit, the call composes with other work on the caller's stream without
extra synchronisation, and it can be captured into a CUDA graph and replayed."""
import pytest
import torch

from oracle import fp4t_oracle as orc

pytestmark = pytest.mark.gpu

N, IC, OC = 8192, 2048, 2048          # above both size gates of fp4t_linear.cu


@pytest.fixture(autouse=True)
def _concurrent_layers():
    from backend import _lib
    _lib.lib().fp4t_set_layer_concurrency(1)
    yield
    _lib.lib().fp4t_set_layer_concurrency(0)


def _inputs():
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(N, IC, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(OC, IC, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    b = (torch.randn(OC, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    dy = (torch.randn(N, OC, device="cuda", generator=g) * 1e-2).to(torch.bfloat16)
    return x, w, b, dy


def _step(ops, x, w, b, dy):
    y, ws = ops.linear_forward("nvfp4", x, w, b, True, True, torch.bfloat16)
    dx, dw, db = ops.linear_backward("nvfp4", dy, ws, IC, True, True, True, sr=ops.SR_HASH, seed=5)
    return y, dx, dw, db


def test_large_layer_matches_unquantized_and_is_ordered_on_the_callers_stream():
    from backend import ops
    x, w, b, dy = _inputs()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):                       # a non-default caller stream
        x2 = x * 1.0                                    # producer on the caller's stream right before the call
        y, dx, dw, db = _step(ops, x2, w, b, dy)
        s = y.float().sum() + dx.float().sum() + dw.float().sum()     # consumers right after it, no sync in between
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    ops.check_status()
    assert bool(torch.isfinite(s))
    assert orc.rel_frobenius(y.float().cpu(), (x.float() @ w.float().t() + b.float()).cpu()) <= 0.2
    assert orc.rel_frobenius(dx.float().cpu(), (dy.float() @ w.float()).cpu()) <= 0.35     # SR-rounded dY x RNE-rounded W
    assert orc.rel_frobenius(dw.float().cpu(), (dy.float().t() @ x.float()).cpu()) <= 0.35
    assert torch.allclose(db.float(), dy.float().sum(0), rtol=2e-2, atol=1e-3)
    # the sequential call gives the same bytes (fixed seed): nothing races between the two streams
    from backend import _lib
    _lib.lib().fp4t_set_layer_concurrency(0)
    y2, dx2, dw2, db2 = _step(ops, x, w, b, dy)
    torch.cuda.synchronize()
    assert torch.equal(y, y2) and torch.equal(dx, dx2) and torch.equal(dw, dw2) and torch.equal(db, db2)


def test_large_layer_call_is_graph_capturable():
    from backend import ops
    x, w, b, dy = _inputs()
    want = _step(ops, x, w, b, dy)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        _step(ops, x, w, b, dy)                         # warm-up on the capture stream (lazy set-up, allocator)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        got = _step(ops, x, w, b, dy)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ops.check_status()
    for a, c, name in zip(got, want, ("y", "dx", "dw", "db")):
        assert torch.equal(a, c), f"{name} differs between the replayed graph and the eager call"
