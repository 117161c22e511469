#!/usr/bin/env python
"""Benchmark of the NVFP4 quantized-linear training path on B200.

A "step" is one pass of the hot path over one synthetic batch:
    quantize X, W (row-wise + transposed operand forms)  -> fprop  Y  = X W^T + b
    quantize dY with stochastic rounding (both forms)    -> dgrad  dX = dY W
                                                         -> wgrad  dW = dY^T X,  db = sum(dY)
at N=8192, IC=OC=4096, bf16 in / bf16 out  (6*N*IC*OC = 824.6 GFLOP per step).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  `value` is whole-job TFLOP/s with inputs resident in HBM;
`e2e` is the same metric through the public module API (custom.CublasltNvfp4Linear) with
pinned host buffers copied in every step and the loss read back.  With --gpus N > 1 (under
torchrun) every rank runs its own batch against replicated weights and the weight gradient
is all-reduced with NCCL (data parallel, weak scaling).

--impl reference times the CPU restatement of the reference's path (the oracle) on the
host cores, on a bounded row sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "fp4-training_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

N, IC, OC = 8192, 4096, 4096
FLOP_PER_STEP = 6.0 * N * IC * OC
# algorithmic HBM bytes of the three quantizer launches: bf16 in once, two code copies
# (0.5 B each) and two scale copies (1/16 B each) out, per element
QUANT_BYTES = (2.0 + 2 * 0.5 + 2.0 / 16) * (N * IC + OC * IC + N * OC)
FP4_NOMINAL_TFLOPS = 9000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu captures summarised
# under profiles/ (fprop GEMM; quantizer of X).  Both working sets fit the 126 MB L2, so part
# of the written data had not reached DRAM when the kernel ended.
GEMM_DRAM_TRAFFIC = {"bytes": 47.3e6, "launch": "fprop 8192x4096x4096", "algorithmic_bytes": 94.4e6 / 3 + 67.1e6}
QUANT_DRAM_TRAFFIC = {"bytes": 71.2e6, "launch": "X 8192x4096 row+transposed", "algorithmic_bytes": 3.125 * N * IC}
METRIC = "nvfp4_linear_fwd_bwd_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "nvfp4_linear_fwd_bwd N=8192 IC=OC=4096 bf16 (quantize x3 + fprop/dgrad/wgrad)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16": float(d["bf16_tflops_sustained"]),
                    "bf16_burst": float(d["bf16_tflops"]), "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16": 1400.0, "bf16_burst": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def synth_inputs(n, ic, oc, seed, device="cpu"):
    """X ~ N(0,1) with 0.1 % of entries x50, W ~ N(0, 0.02), G ~ N(0, 1e-3), bf16, seeded."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(n, ic, generator=gen)
    x = torch.where(torch.rand(n, ic, generator=gen) < 1e-3, x * 50.0, x)
    w = torch.randn(oc, ic, generator=gen) * 0.02
    g = torch.randn(n, oc, generator=gen) * 1e-3
    b = torch.zeros(oc)
    return [t.to(torch.bfloat16).to(device) for t in (x, w, g, b)]


# --------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle on the host cores, bounded row sample
# --------------------------------------------------------------------------------------
def cpu_path_seconds(rows: int, steps: int, warmup: int):
    from oracle import fp4t_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    x, w, g, b = synth_inputs(rows, IC, OC, 0)
    times = []
    for i in range(warmup + steps):
        gen = torch.Generator().manual_seed(i)
        u = torch.rand(rows, OC, generator=gen)
        ut = torch.rand(OC, rows, generator=gen)
        t0 = time.perf_counter()
        orc.nvfp4_linear_fwd_bwd(x, w, g, b, noise_g=u, noise_gt=ut)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    return times


def run_reference(args, rank: int):
    if rank != 0:
        return
    rows = 256
    times = cpu_path_seconds(rows, args.steps, min(args.warmup, 1))
    ms = 1e3 * sum(times) / len(times)
    val = 6.0 * rows * IC * OC / (ms * 1e-3) / 1e12
    cores = torch.get_num_threads()
    sample = f"{rows} of {N} rows of X and dY against the full 4096x4096 W, per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample, "device": "host CPU"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------
def run_ours(args, rank: int, world: int, local_rank: int):
    import torch.distributed as dist

    from backend import ops

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    reserve = int(os.environ.get("FP4T_RESERVE_SMS", "0")) if world > 1 else 0
    if reserve:
        # optional experiment knob: cap the persistent grids so that some SMs stay free for the
        # NCCL all-reduce that overlaps the next step's kernels (measured: no gain, default off)
        from backend import _lib as _l
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        _l.lib().fp4t_set_sm_limit(sms - reserve)
    peaks = measured_peaks()
    nsets = 2   # rotate input sets; one set alone (160 MB bf16) already exceeds the 126 MB L2
    sets = [synth_inputs(N, IC, OC, 100 * rank + s, dev) for s in range(nsets)]
    for s in sets[1:]:
        s[1] = sets[0][1]          # weights are shared state, only the batch changes
    bias = sets[0][3]
    ev = torch.cuda.Event
    # weight and bias gradients land in one flat buffer (two of them, rotating) so that a single
    # NCCL all-reduce per step, on a side stream, can overlap the kernels of step i+1, as it
    # does under the backward pass of the previous layer in data-parallel training
    reducers = None
    if world > 1 and os.environ.get("FP4T_ALLREDUCE", "nccl") == "switch":
        # the library's own in-switch all-reduce (opt-in: inside the step it measured a few per
        # cent behind NCCL -- 0.335 against 0.300 ms on 2 GPUs, 0.350 against 0.341 ms on 8);
        # NCCL if these GPUs offer no NVLink multicast
        try:
            from dp import SwitchAllReducer
            reducers = [SwitchAllReducer(OC * IC + OC, dev, ctas=int(os.environ.get("FP4T_ALLREDUCE_CTAS", "148")))
                        for _ in range(2)]
        except Exception as e:   # noqa: BLE001
            if rank == 0:
                print(f"bench: in-switch all-reduce unavailable ({e!r}); using NCCL", file=sys.stderr)
            reducers = None
    if reducers is not None:
        grad_bufs = [r.flat for r in reducers]
    else:
        grad_bufs = [torch.empty(OC * IC + OC, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    comm_stream = torch.cuda.Stream(device=dev) if world > 1 else None
    comm_done = [None, None]

    def hot_step(i):
        x, w, g, _ = sets[i % nsets]
        y, ws = ops.linear_forward("nvfp4", x, w, bias, True, True, torch.bfloat16)
        slot = i % 2
        if comm_done[slot] is not None:
            torch.cuda.current_stream().wait_event(comm_done[slot])   # buffer free again
        flat = grad_bufs[slot]
        dx, dw, db = ops.linear_backward("nvfp4", g, ws, IC, True, True, True, sr=ops.SR_HASH, seed=i,
                                         out_dw=flat[:OC * IC].view(OC, IC), out_db=flat[OC * IC:])
        if world > 1:
            ready = ev()
            ready.record()
            with torch.cuda.stream(comm_stream):
                comm_stream.wait_event(ready)
                if reducers is not None:
                    reducers[slot].all_reduce(ops.status_word(dev))
                    ops.LAUNCHES["allreduce"] += 1
                else:
                    dist.all_reduce(flat)
                comm_done[slot] = ev()
                comm_done[slot].record()
        return y, dx, dw, db

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        hot_step(i)
    barrier()
    launches0 = dict(ops.LAUNCHES)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_start, t_end = ev(enable_timing=True), ev(enable_timing=True)
    barrier()
    t_start.record()
    host_t0 = time.perf_counter()
    for i in range(args.steps):
        hot_step(i)
    host_enqueue_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps   # CPU time to enqueue one step
    t_end.record()
    barrier()
    ms_total = t_start.elapsed_time(t_end)
    launches = sum(ops.LAUNCHES.values()) - sum(launches0.values())
    ops.check_status(dev)

    # per-kernel durations: each kernel of the step launched back to back between two CUDA
    # events (events between the kernels of a live step would time launch gaps instead)
    kern_ms = time_kernels(ops, sets[0], bias, max(10, min(args.steps, 50)))

    # end-to-end through the module API with host buffers
    e2e_ms, h2d, d2h = run_e2e(args, dev, rank, world)
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms_total, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = float(t[0]), float(t[1])
    if rank != 0:
        return
    ms_step = ms_total / args.steps
    value = world * FLOP_PER_STEP / (ms_step * 1e-3) / 1e12
    gemm_ms = kern_ms["fprop"] + kern_ms["dgrad"] + kern_ms["wgrad"]
    gemm_tflops = FLOP_PER_STEP / (gemm_ms * 1e-3) / 1e12
    quant_ms = kern_ms["quant_w"] + kern_ms["quant_x"] + kern_ms["quant_g"]
    quant_gbs = QUANT_BYTES / (quant_ms * 1e-3) / 1e9
    fp4_peak = 4.0 * peaks["bf16"]

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        rows = 256
        times = cpu_path_seconds(rows, 3, 1)
        sec = sum(times) / len(times)
        cpu = {"value": 6.0 * rows * IC * OC / sec / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
               "kind": "port",
               "sample": f"{rows} of {N} rows of X and dY against the full 4096x4096 W, 3 timed passes"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate, bf16 out)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "inputs larger than L2 (160 MB bf16 per step, two sets rotated)",
                   "parallelism": f"dp{world}" if world > 1 else "single",
                   "allreduce": ("none" if world == 1 else
                                 "fp4t in-switch multimem kernel on a side stream, one call per step" if reducers is not None
                                 else "NCCL on a side stream, one call per step"),
                   "bias_grad": "fused into the dY quantizer (fp32 atomics + finishing kernel)",
                   "frac_of_nominal_fp4_peak": value / world / FP4_NOMINAL_TFLOPS},
        "roofline": {"bound": "tensor", "kernel": "gemm2_blockscaled_kernel<nvfp4, 256> two-CTA (fprop+dgrad+wgrad)",
                     "achieved": gemm_tflops, "peak": fp4_peak, "unit": UNIT, "frac": gemm_tflops / fp4_peak,
                     "peak_basis": f"4 x {peaks['source']} sustained bf16 cuBLAS TFLOP/s (FP4:BF16 dense ratio); "
                                   f"nominal dense FP4 is {FP4_NOMINAL_TFLOPS:.0f}",
                     "frac_of_nominal": gemm_tflops / FP4_NOMINAL_TFLOPS, "traffic": GEMM_DRAM_TRAFFIC,
                     "ms_per_launch": gemm_ms / 3},
        "roofline_quantize": {"bound": "hbm", "kernel": "quantize_tma_kernel<nvfp4> (X, W, dY)",
                              "achieved": quant_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                              "frac": quant_gbs / peaks["hbm_gbs"], "peak_basis": f"{peaks['source']} copy bandwidth",
                              "traffic": QUANT_DRAM_TRAFFIC, "ms_per_launch": quant_ms / 3},
        "kernel_ms": kern_ms,
        "e2e": {"value": world * FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "api": "custom.CublasltNvfp4Linear forward+backward under bf16 autocast"},
        "gpu_launches": launches,
        "host_enqueue_ms_per_step": host_enqueue_ms,
        "clocks": clocks,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)


def kernel_closures(ops, inputs, bias):
    """The seven launches of one step as standalone closures over prepared operands."""
    x, w, g, _ = inputs
    wc, wsf, wtc, wtsf = ops.quantize_nvfp4(w, True, True)
    xc, xsf, xtc, xtsf = ops.quantize_nvfp4(x, True, True)
    gc, gsf, gtc, gtsf = ops.quantize_nvfp4(g, True, True, sr=ops.SR_HASH, seed=1)
    y = torch.empty(N, OC, dtype=torch.bfloat16, device=x.device)
    dx = torch.empty(N, IC, dtype=torch.bfloat16, device=x.device)
    dw = torch.empty(OC, IC, dtype=torch.bfloat16, device=x.device)
    return {
        "quant_w": lambda: ops.quantize_nvfp4(w, True, True),
        "quant_x": lambda: ops.quantize_nvfp4(x, True, True),
        "quant_g": lambda: ops.quantize_nvfp4(g, True, True, sr=ops.SR_HASH, seed=1, bias_grad_dtype=torch.bfloat16),
        "fprop": lambda: ops.gemm_nvfp4(xc, xsf, wc, wsf, bias, torch.bfloat16, out=y),
        "dgrad": lambda: ops.gemm_nvfp4(gc, gsf, wtc, wtsf, None, torch.bfloat16, out=dx),
        "wgrad": lambda: ops.gemm_nvfp4(gtc, gtsf, xtc, xtsf, None, torch.bfloat16, out=dw),
    }


def time_kernels(ops, inputs, bias, reps, only=None):
    out = {}
    for name, fn in kernel_closures(ops, inputs, bias).items():
        if only is not None and name != only:
            continue
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        out[name] = a.elapsed_time(b) / reps
    return out


def run_single_kernel(args):
    """--kernel NAME: launch one kernel of the step --steps times (after --warmup launches).
    This is the small command the ncu captures under profiles/ were taken with."""
    from backend import ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    inputs = synth_inputs(N, IC, OC, 0, dev)
    fn = kernel_closures(ops, inputs, inputs[3])[args.kernel]
    for _ in range(args.warmup):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(args.steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    ops.check_status(dev)
    print(json.dumps({"kernel": args.kernel, "launches": args.steps, "ms_per_launch": a.elapsed_time(b) / args.steps}))


def run_e2e(args, dev, rank, world):
    """Same metric through the module API.  Every step copies its own X, W and dY from pinned
    host memory, runs the layer's forward+backward under autocast and reads the scalar sum of
    Y back.  The copies of step i+1 are issued on a copy stream into the second of two device
    buffer sets before the host waits for step i's result, so they overlap step i's kernels the
    way a prefetching input pipeline does; the timed region (wall clock between device
    synchronisations) contains all copies, all kernels and all read-backs."""
    import torch.distributed as dist

    from custom import CublasltNvfp4Linear

    x, w, g, b = synth_inputs(N, IC, OC, 7 + rank)
    hx, hw, hg = x.pin_memory(), w.pin_memory(), g.pin_memory()
    layer = CublasltNvfp4Linear(IC, OC, device=dev, dtype=torch.bfloat16)
    bufs = [(torch.empty(N, IC, dtype=torch.bfloat16, device=dev), torch.empty(OC, IC, dtype=torch.bfloat16, device=dev),
             torch.empty(N, OC, dtype=torch.bfloat16, device=dev)) for _ in range(2)]
    h2d = hx.numel() * 2 + hw.numel() * 2 + hg.numel() * 2
    steps = max(3, min(args.steps, 20))
    copy_stream = torch.cuda.Stream(device=dev)
    copied = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    host_out = torch.empty(1, dtype=torch.float32).pin_memory()

    def start_copy(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])          # the step that last used this set is done with it
            dx, dw_, dg = bufs[slot]
            dx.copy_(hx, non_blocking=True)
            dw_.copy_(hw, non_blocking=True)
            dg.copy_(hg, non_blocking=True)
            copied[slot].record()

    def compute(slot):
        cur = torch.cuda.current_stream()
        cur.wait_event(copied[slot])
        dx, dw_, dg = bufs[slot]
        with torch.no_grad():
            layer.weight.copy_(dw_)
        xin = dx.detach().requires_grad_(True)
        layer.weight.grad = None
        layer.bias.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = layer(xin)
        y.backward(dg)
        if world > 1:
            dist.all_reduce(layer.weight.grad)
            dist.all_reduce(layer.bias.grad)
        host_out.copy_(y.detach().float().sum().reshape(1), non_blocking=True)     # 4-byte read-back of the step's result
        consumed[slot].record()

    def run(nsteps):
        consumed[0].record()
        consumed[1].record()
        start_copy(0)
        total = 0.0
        for i in range(nsteps):
            compute(i % 2)
            if i + 1 < nsteps:
                start_copy((i + 1) % 2)
            torch.cuda.current_stream().synchronize()       # the host has this step's result
            total += float(host_out[0])
        return total

    run(2)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    run(steps)
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) * 1e3 / steps, h2d, 4


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel", default=None,
                    choices=["quant_w", "quant_x", "quant_g", "fprop", "dgrad", "wgrad"],
                    help="run only this kernel of the step (profiling aid); no benchmark line")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    if args.kernel is not None:
        run_single_kernel(args)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
