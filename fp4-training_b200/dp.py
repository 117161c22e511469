"""Data-parallel gradient exchange for the quantized-linear training step.

The reference trains on one GPU (`main_train_tinyvit_mnist.py:31`); running its step data
parallel adds exactly one exchange: the all-reduce (average) of the parameter gradients the
wgrad GEMMs produce.  `GradAllReducer` does that exchange with `torch.distributed` (NCCL over
NVLink on GPUs, gloo on CPU for tests): parameters are grouped into buckets in reverse
registration order (the order backward produces their gradients), a bucket's all-reduce is
launched asynchronously as soon as its last gradient has been accumulated, so the reduction of
late layers overlaps the backward pass of earlier ones, and `finish()` waits for all buckets
and writes the averaged gradients back.

`SwitchAllReducer` is the exchange for one flat bf16 gradient buffer on GPUs that share an
NVSwitch: the buffer lives in symmetric memory bound to an NVLink multicast object and is summed
in place by `fp4t_allreduce_sum_bf16_multimem` (reduction inside the switch, a kernel small
enough to be resident beside the persistent quantizers and GEMMs it overlaps with).

`CopyEngineAllReducer` is the exchange that leaves the SMs to the step it overlaps: a
reduce-scatter + all-gather whose bulk bytes travel as peer-to-peer copies on the copy engines,
with a one-warp rendezvous between the ranks and a reduction of this rank's shard only (inside
the switch where the GPUs offer multicast) as its only kernels.
"""
from __future__ import annotations

import contextlib
import ctypes

import torch
import torch.distributed as dist


class _Bucket:
    def __init__(self, params):
        self.params = params
        p0 = params[0]
        self.flat = torch.zeros(sum(p.numel() for p in params), dtype=p0.dtype, device=p0.device)
        self.views = []
        off = 0
        for p in params:
            self.views.append(self.flat[off:off + p.numel()].view_as(p))
            off += p.numel()
        self.fired = [False] * len(params)
        self.work = None


class GradAllReducer:
    """Bucketed, overlapped all-reduce (average) of parameter gradients.

    One `finish()` per optimizer step.  With gradient accumulation, run all but the last
    backward of a step inside `no_sync()`: hooks then leave the buckets alone and the last
    backward's hooks reduce the accumulated `.grad`.  A backward outside `no_sync()` after a
    bucket's collective has already started (a second backward without `finish()` in between)
    is handled too: the running collective is waited for and the bucket is reduced again from
    the up-to-date `.grad` in `finish()`.
    """

    def __init__(self, params, process_group=None, bucket_bytes: int = 4 << 20):
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        params = [p for p in params if p.requires_grad]
        self.buckets = []
        cur, cur_bytes, key = [], 0, None
        for p in reversed(params):
            k = (p.dtype, p.device)
            if cur and (k != key or cur_bytes + p.numel() * p.element_size() > bucket_bytes):
                self.buckets.append(_Bucket(cur))
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += p.numel() * p.element_size()
            key = k
        if cur:
            self.buckets.append(_Bucket(cur))
        self._index = {}
        self._handles = []
        self._sync = True
        for b in self.buckets:
            for i, p in enumerate(b.params):
                self._index[p] = (b, i)
                self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside this context only accumulate into `.grad`."""
        old, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = old

    def _on_grad(self, p):
        if self.world == 1 or not self._sync:
            return
        b, i = self._index[p]
        if b.work is not None:
            # this bucket's collective is already in flight and its gradient changed again:
            # let it finish before the buffer is touched, and reduce afresh in finish()
            b.work.wait()
            b.work = None
            b.fired = [False] * len(b.params)
            return
        b.views[i].copy_(p.grad)
        b.fired[i] = True
        if all(b.fired):
            b.work = dist.all_reduce(b.flat, group=self.group, async_op=True)

    def finish(self):
        """Wait for every bucket and store the averaged gradients in `.grad`."""
        if self.world == 1:
            return
        for b in self.buckets:
            if b.work is None:
                # not every hook fired (unused parameter, accumulation, a repeated backward):
                # take each gradient as it stands now, zeros where there is none
                for i, p in enumerate(b.params):
                    if p.grad is None:
                        b.views[i].zero_()
                    else:
                        b.views[i].copy_(p.grad)
                b.work = dist.all_reduce(b.flat, group=self.group, async_op=True)
            b.work.wait()
            b.flat.div_(self.world)
            for v, p in zip(b.views, b.params):
                if p.grad is None:
                    p.grad = v.clone()
                else:
                    p.grad.copy_(v)
            b.fired = [False] * len(b.params)
            b.work = None

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []


def broadcast_parameters(module: torch.nn.Module, src: int = 0, process_group=None):
    """Make every rank start from rank `src`'s parameters and buffers."""
    if not dist.is_initialized() or dist.get_world_size(process_group) == 1:
        return
    for t in list(module.parameters()) + list(module.buffers()):
        dist.broadcast(t.data, src=src, group=process_group)


class SwitchAllReducer:
    """In-place sum all-reduce of `self.flat` (bf16, `numel` rounded up to a multiple of 8) over
    the ranks of `process_group`, all on one NVSwitch domain.  Every rank constructs it with the
    same arguments and calls `all_reduce()` the same number of times; the call is asynchronous on
    the current stream.  Raises at construction if the GPUs offer no NVLink multicast."""

    def __init__(self, numel: int, device, process_group=None, ctas: int = 148):
        import torch.distributed._symmetric_memory as symm_mem
        from backend import _lib
        self._lib = _lib
        group = process_group if process_group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("SwitchAllReducer handles at most 8 ranks")
        self.device = torch.device(device)
        self.numel = (numel + 7) // 8 * 8
        self.ctas = ctas
        self.flat = symm_mem.empty(self.numel, dtype=torch.bfloat16, device=self.device)
        self.flat.zero_()
        self._handle = symm_mem.rendezvous(self.flat, group.group_name)
        if not getattr(self._handle, "multicast_ptr", 0):
            raise RuntimeError("symmetric memory has no multicast address on these GPUs")
        flag_words = 256 * 8          # FP4T_ALLREDUCE_FLAG_WORDS
        self._flags = symm_mem.empty(flag_words, dtype=torch.int32, device=self.device)
        self._flags.zero_()
        self._flag_handle = symm_mem.rendezvous(self._flags, group.group_name)
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self._flag_handle.buffer_ptrs])
        torch.cuda.synchronize(self.device)
        dist.barrier(group)           # every rank's flags are zero before anyone's first call
        self._epoch = 0

    def all_reduce(self, status=None):
        """Sum `self.flat` over the ranks, in place, on the current stream of `self.device`."""
        self._epoch += 1
        L = self._lib
        with torch.cuda.device(self.device):
            L.check(L.lib().fp4t_allreduce_sum_bf16_multimem(
                int(self._handle.multicast_ptr), self._flag_ptrs, self.rank, self.world, self.numel,
                self._epoch, self.ctas, L.ptr(status) if status is not None else None,
                L.stream_ptr(self.device)), "fp4t_allreduce_sum_bf16_multimem")


def shard_plan(numel: int, world: int) -> tuple[int, int]:
    """(shard, padded): elements per rank, a multiple of 8 (16 bytes of bf16), and the buffer
    length `world * shard` >= numel that the exchange works on."""
    shard = (numel + world - 1) // world
    shard = (shard + 7) // 8 * 8
    return shard, shard * world


class CopyEngineAllReducer:
    """In-place sum all-reduce of `self.flat[:numel]` (bf16) whose bulk bytes move on the GPUs'
    copy engines, so that the exchange takes no SM from the persistent quantizer / GEMM kernels
    of the step it overlaps.

    Reduce-scatter + all-gather over peer-mapped symmetric memory: after a rendezvous every rank
    pulls its own shard of each peer's buffer with peer-to-peer copies, sums the `world` partial
    shards in rank order with fp32 accumulation (`fp4t_sum_bf16_shards`, the only SM work: a few
    MB), and after a second rendezvous pulls the other ranks' reduced shards.  Each shard is
    reduced exactly once, by its owner, so all ranks end with identical bytes.  The sequence is
    captured once in a CUDA graph (`graph=True`): a call is then one graph launch.

    Where the GPUs offer NVLink multicast (`reduce="switch"`, what "auto" picks there) the pulls
    of the first half and the sum are replaced by `fp4t_reduce_shard_bf16_multimem`: the switch
    adds the `world` copies of this rank's shard, so 1/world of the buffer passes through SMs
    and nothing else; `reduce="sum"` is the form without multicast.

    Every rank constructs it with the same arguments and makes the same calls; a call is
    asynchronous on the current stream."""

    def __init__(self, numel: int, device, process_group=None, reduce_ctas: int = 0, graph: bool = True,
                 reduce: str = "auto"):
        import torch.distributed._symmetric_memory as symm_mem
        from backend import _lib
        from backend import ops as _ops
        self._lib, self._ops = _lib, _ops
        group = process_group if process_group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("CopyEngineAllReducer handles at most 8 ranks")
        self.device = torch.device(device)
        self.numel = numel
        self.shard, self.padded = shard_plan(numel, self.world)
        w, r, sh = self.world, self.rank, self.shard
        self.flat = symm_mem.empty(self.padded, dtype=torch.bfloat16, device=self.device)
        self.flat.zero_()
        self._h_flat = symm_mem.rendezvous(self.flat, group.group_name)
        self._reduced = symm_mem.empty(sh, dtype=torch.bfloat16, device=self.device)
        self._h_red = symm_mem.rendezvous(self._reduced, group.group_name)
        self._flags = symm_mem.empty(256 * 8, dtype=torch.int32, device=self.device)   # FP4T_ALLREDUCE_FLAG_WORDS
        self._flags.zero_()
        self._h_flags = symm_mem.rendezvous(self._flags, group.group_name)
        self._flag_ptrs = (ctypes.c_void_p * w)(*[int(p) for p in self._h_flags.buffer_ptrs])
        self._stage = torch.empty((max(w - 1, 1), sh), dtype=torch.bfloat16, device=self.device)
        self._peers = [p for p in range(w) if p != r]
        # peer views: my shard inside every peer's gradient buffer, and every peer's reduced shard
        self._peer_part = {p: self._h_flat.get_buffer(p, (sh,), torch.bfloat16, r * sh) for p in self._peers}
        self._peer_red = {p: self._h_red.get_buffer(p, (sh,), torch.bfloat16, 0) for p in self._peers}
        srcs, j = [], 0
        for p in range(w):                      # rank order, own shard in its place
            if p == r:
                srcs.append(self.flat[r * sh:(r + 1) * sh].data_ptr())
            else:
                srcs.append(self._stage[j].data_ptr())
                j += 1
        self._srcs = (ctypes.c_void_p * w)(*srcs)
        self._status = _ops.status_word(self.device)
        mc = int(getattr(self._h_flat, "multicast_ptr", 0) or 0)
        if reduce == "auto":
            reduce = "switch" if mc else "sum"
        if reduce not in ("switch", "sum"):
            raise ValueError("reduce must be 'auto', 'switch' or 'sum'")
        if reduce == "switch" and not mc:
            raise RuntimeError("symmetric memory has no multicast address on these GPUs")
        self.reduce = reduce
        self._mc_shard = mc + r * sh * 2 if mc else 0
        # CTAs of the reduction: enough loads in flight for its bytes, few enough to stay a guest
        if reduce_ctas <= 0:
            bytes_through_sms = sh * 2 * (1 if reduce == "switch" else w)
            reduce_ctas = max(16, min(148, bytes_through_sms // (256 << 10)))
        self.reduce_ctas = int(reduce_ctas)
        torch.cuda.synchronize(self.device)
        dist.barrier(group)                     # every rank's flags are zero before anyone's first call
        self._graph = None
        if graph and w > 1:
            self._capture()

    def _meet(self, slot: int):
        L = self._lib
        L.check(L.lib().fp4t_rank_meet(self._flag_ptrs, self.rank, self.world, slot, L.ptr(self._status),
                                       L.stream_ptr(self.device)), "fp4t_rank_meet")

    def _sequence(self):
        L = self._lib
        r, sh = self.rank, self.shard
        if self.world == 1:
            return
        self._meet(0)                           # every rank's gradients are complete
        if self.reduce == "switch":
            L.check(L.lib().fp4t_reduce_shard_bf16_multimem(self._mc_shard, self._reduced.data_ptr(), sh,
                                                            self.reduce_ctas, L.stream_ptr(self.device)),
                    "fp4t_reduce_shard_bf16_multimem")
        else:
            for j, p in enumerate(self._peers):
                self._stage[j].copy_(self._peer_part[p])
            L.check(L.lib().fp4t_sum_bf16_shards(self._reduced.data_ptr(), self._srcs, self.world, sh,
                                                 self.reduce_ctas, L.stream_ptr(self.device)), "fp4t_sum_bf16_shards")
        self._meet(1)                           # every reduced shard is complete (and every pull above is done)
        self.flat[r * sh:(r + 1) * sh].copy_(self._reduced)
        for p in self._peers:
            self.flat[p * sh:(p + 1) * sh].copy_(self._peer_red[p])
        # a peer overwrites its reduced shard only after the first rendezvous of its next call,
        # which this rank joins after the pulls above (stream order)

    def _capture(self):
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        g = torch.cuda.CUDAGraph()
        with torch.cuda.device(self.device), torch.cuda.graph(g, stream=side):
            self._sequence()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self._graph = g

    def all_reduce(self):
        """Sum `self.flat` over the ranks, in place, on the current stream of `self.device`."""
        with torch.cuda.device(self.device):
            if self._graph is not None:
                self._graph.replay()
            else:
                self._sequence()
