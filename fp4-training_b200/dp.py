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
