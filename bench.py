#!/usr/bin/env python
"""Benchmark of the quantized-linear training path on B200.

Default workload (--config linear_nvfp4): one NVFP4 linear layer, forward + backward.  A "step"
is one pass of the hot path over one synthetic batch:
    quantize X, W (row-wise + transposed operand forms)  -> fprop  Y  = X W^T + b
    quantize dY with stochastic rounding (both forms)    -> dgrad  dX = dY W
                                                         -> wgrad  dW = dY^T X,  db = sum(dY)
at N=8192, IC=OC=4096, bf16 in / bf16 out  (6*N*IC*OC = 824.6 GFLOP per step).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config linear_nvfp4|mlp_mxfp8|gemm_sweep|tinyvit]

Prints ONE JSON line (rank 0).  `value` is whole-job TFLOP/s with inputs resident in HBM over
exactly K timed steps; `sustained` repeats the K-step block until at least --min-seconds of
device time have passed (clocks sampled inside that region); `e2e` is the same metric through
the public module API (custom.CublasltNvfp4Linear) with pinned host buffers copied in every
step and the loss read back.  `roofline` is the dominant kernel (the block-scaled GEMM) timed
alone, against 4 x the measured burst bf16 rate, with the same kernel timed in a seconds-long
loop against 4 x the sustained rate beside it; `comparator` times the library kernel
(cuBLASLt NVFP4 through torch._scaled_mm) on the same codes and scales.  With --gpus N > 1
(under torchrun) every rank runs its own batch against replicated weights and the weight
gradient is all-reduced (data parallel, weak scaling); before the timed region the library's
own multi-GPU code is checked (`multi_gpu_check`).

The other configurations print the same line shape for their own metric:
  mlp_mxfp8   MXFP8 MLP pair (16384 x 4096 -> 14336 -> 4096), forward + backward, 11.54 TFLOP
  gemm_sweep  NVFP4 and MXFP8 GEMMs over M, N, K in {1024..16384} plus skinny M in {16, 128}
  tinyvit     TinyViT-style classifier, all linears NVFP4, steps/s (data parallel with --gpus N)

--impl reference times the CPU restatement of the reference's path (the oracle) on the host
cores, on the same full-size workload.
"""
from __future__ import annotations

import argparse
import json
import math
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
FP8_NOMINAL_TFLOPS = 4500.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu captures summarised
# under profiles/ (fprop GEMM; quantizer of X).  Both working sets fit the 126 MB L2, so part
# of the written data had not reached DRAM when the kernel ended.
GEMM_DRAM_TRAFFIC = {"bytes": 48.6e6, "launch": "fprop 8192x4096x4096", "algorithmic_bytes": 94.4e6 / 3 + 67.1e6}
QUANT_DRAM_TRAFFIC = {"bytes": 71.6e6, "launch": "X 8192x4096 row+transposed", "algorithmic_bytes": 3.125 * N * IC}
METRIC = "nvfp4_linear_fwd_bwd_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "nvfp4_linear_fwd_bwd N=8192 IC=OC=4096 bf16 (quantize x3 + fprop/dgrad/wgrad)"
L2_NOTE = "inputs larger than L2 (160 MB bf16 per step, two sets rotated)"


def base_config(world: int):
    """The `config` object both arms print for the default workload."""
    return {"workload": WORKLOAD, "l2": L2_NOTE, "parallelism": f"dp{world}" if world > 1 else "single"}


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
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

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
            return self
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def mark(self):
        """Host time stamp to select the samples of a sub-region later."""
        return time.perf_counter()

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()

    def summary(self, t0=None, t1=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, ln in list(self.lines):
            if (t0 is not None and ts < t0) or (t1 is not None and ts > t1):
                continue
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
            if len(parts) > 6:
                try:
                    pw.append(float(parts[6]))
                except ValueError:
                    pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons)}


def synth_inputs(n, ic, oc, seed, device="cpu"):
    """X ~ N(0,1) with 0.1 % of entries x50, W ~ N(0, 0.02), G ~ N(0, 1e-3), bf16, seeded."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(n, ic, generator=gen)
    x = torch.where(torch.rand(n, ic, generator=gen) < 1e-3, x * 50.0, x)
    w = torch.randn(oc, ic, generator=gen) * 0.02
    g = torch.randn(n, oc, generator=gen) * 1e-3
    b = torch.zeros(oc)
    return [t.to(torch.bfloat16).to(device) for t in (x, w, g, b)]


def event_pair():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def time_loop(fn, reps, warm=3):
    """Mean milliseconds per call of fn over `reps` back-to-back calls (CUDA events on the
    current stream, synchronised on both sides)."""
    for _ in range(warm):
        fn()
    a, b = event_pair()
    torch.cuda.synchronize()
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def time_graph(fn, reps):
    """Mean milliseconds per call of fn with the `reps` calls captured into one CUDA graph and
    replayed: no host work between the launches, so kernels shorter than the host's enqueue
    cost (tens of microseconds through Python) are timed on the device's terms.  Inside a
    capture the persistent kernels take their tiles in the static order."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    graph.replay()
    a, b = event_pair()
    torch.cuda.synchronize()
    a.record()
    graph.replay()
    b.record()
    torch.cuda.synchronize()
    del graph
    return a.elapsed_time(b) / reps


def time_kernel(fn, reps, warm=3, host_bound_ms=0.045):
    """Back-to-back launches; re-timed from a CUDA graph when the launches are short enough
    for the host's enqueue cost to show.  -> (ms, how)"""
    ms = time_loop(fn, reps, warm)
    if ms < host_bound_ms:
        return min(ms, time_graph(fn, reps)), "graph"
    return ms, "stream"


def time_for_seconds(fn, seconds, probe_reps=10):
    """Mean milliseconds per call of fn in a loop sized to last at least `seconds` on the device."""
    ms = time_loop(fn, probe_reps)
    reps = max(probe_reps, int(math.ceil(seconds * 1e3 / max(ms, 1e-6))))
    return time_loop(fn, reps, warm=0), reps


# --------------------------------------------------------------------------------------
# reference arm / CPU baselines: the oracle on the host cores
# --------------------------------------------------------------------------------------
def cpu_path_seconds(rows: int, steps: int, warmup: int):
    """Seconds per NVFP4 linear forward+backward of the CPU oracle on `rows` rows of X and dY
    against the full W (rows == N is the whole workload)."""
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


def cpu_config1_baseline(reps: int = 25):
    """BASELINE config 1: one MXFP8 fake-quantized linear, forward + backward, on the host cores
    (X 512x768 ~N(0,1), W 768x768 ~N(0,0.02), G 512x768 ~N(0,1e-3), seed 0), median of `reps`."""
    from oracle import fp4t_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(512, 768, generator=gen).to(torch.bfloat16)
    w = (torch.randn(768, 768, generator=gen) * 0.02).to(torch.bfloat16)
    g = (torch.randn(512, 768, generator=gen) * 1e-3).to(torch.bfloat16)
    for _ in range(5):
        orc.fake_mxfp8_linear_fwd_bwd(x, w, g)
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        orc.fake_mxfp8_linear_fwd_bwd(x, w, g)
        ts.append(time.perf_counter() - t0)
    med = statistics.median(ts)
    flop = 6.0 * 512 * 768 * 768
    return {"workload": "mxfp8 fake-quantized linear fwd+bwd N=512 IC=OC=768 (6 fake-quants + 3 matmuls)",
            "median_ms": med * 1e3, "min_ms": min(ts) * 1e3, "value": flop / med / 1e12, "unit": UNIT,
            "cores": torch.get_num_threads(), "runs": reps,
            "kind": "port (CPU restatement of the microxcaling emulation; MXFP8 parity unpinned)"}


def run_reference(args, rank: int):
    """The reference's CPU implementation of the path (oracle port), full-size workload, all
    host threads.  Under torchrun only rank 0 works."""
    if rank != 0:
        return
    if args.config != "linear_nvfp4":
        print(json.dumps({"impl": "reference", "unavailable":
                          f"the CPU reference arm covers the default workload only (asked for {args.config})"}), flush=True)
        return
    rows = N if args.sample_rows <= 0 else min(N, args.sample_rows)
    times = cpu_path_seconds(rows, args.steps, args.warmup)
    ms = 1e3 * sum(times) / len(times)
    val = 6.0 * rows * IC * OC / (ms * 1e-3) / 1e12
    cores = torch.get_num_threads()
    sample = ("the whole workload (all 8192 rows), one pass per step" if rows == N else
              f"{rows} of {N} rows of X and dY against the full 4096x4096 W, per step")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": base_config(args.gpus),
        "device": "host CPU (oracle port of the reference path)",
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# library comparator: cuBLASLt NVFP4 through torch._scaled_mm on the same operands
# --------------------------------------------------------------------------------------
def library_gemm_nvfp4(pc, ps, qc, qs):
    return torch._scaled_mm(pc.view(torch.float4_e2m1fn_x2), qc.view(torch.float4_e2m1fn_x2).t(),
                            ps.view(torch.float8_e4m3fn).flatten(), qs.view(torch.float8_e4m3fn).flatten(),
                            out_dtype=torch.bfloat16)


def run_comparator(ops, operands, ours_ms, reps):
    """cuBLASLt's NVFP4 GEMM on the very codes and swizzled scales our kernel consumes, for the
    three GEMMs of the step (comparator leg only; never on the product path)."""
    out = {"library": "cuBLASLt NVFP4 via torch._scaled_mm (bf16 out, no bias)", "reps": reps}
    try:
        tot = 0.0
        for name, (pc, ps, qc, qs) in operands.items():
            y_lib = library_gemm_nvfp4(pc, ps, qc, qs)
            y = ops.gemm_nvfp4(pc, ps, qc, qs, None, torch.bfloat16)
            diff = float((y.float() - y_lib.float()).norm() / y_lib.float().norm().clamp_min(1e-30))
            ms = time_loop(lambda: library_gemm_nvfp4(pc, ps, qc, qs), reps)
            out[name] = {"library_ms": ms, "ours_ms": ours_ms[name], "ratio": ms / ours_ms[name],
                         "rel_diff_of_outputs": diff}
            tot += ms
            del y_lib, y
        ours = sum(ours_ms[n] for n in operands)
        out["library_ms_3gemm"] = tot
        out["ours_ms_3gemm"] = ours
        out["ratio"] = tot / ours       # > 1: ours is faster
    except Exception as e:   # noqa: BLE001  (an older torch without NVFP4 _scaled_mm)
        out["unavailable"] = f"{type(e).__name__}: {e}"[:200]
    return out


# --------------------------------------------------------------------------------------
# multi-GPU correctness, checked under the benchmark's own launch (N > 1)
# --------------------------------------------------------------------------------------
def multi_gpu_check(ops, dev, rank, world):
    """Runs before the timed region: the library's in-switch all-reduce against NCCL's sum, and
    the column-sharded GEMM (+ all-gather) against the unsharded GEMM.  Returns a dict for the
    JSON line; never raises (a failed check is reported, not hidden)."""
    import torch.distributed as dist
    res = {}
    try:
        from dp import SwitchAllReducer
        numel = 1 << 20
        red = SwitchAllReducer(numel, dev, ctas=64)
        gen = torch.Generator(device=dev).manual_seed(4321 + rank)
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
        ulp = torch.clamp(want.abs(), min=2.0 ** -126) * 2.0 ** -7
        ok = bool(((got - want).abs() <= ulp).all())
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        res["switch_allreduce_vs_nccl_sum"] = {"ok": bool(flag.item()), "numel": red.numel,
                                               "tolerance": "one bf16 step of the fp32 sum"}
        del red
    except Exception as e:   # noqa: BLE001
        res["switch_allreduce_vs_nccl_sum"] = {"ok": False, "error": f"{type(e).__name__}: {e}"[:200]}
    try:
        from dp import CopyEngineAllReducer
        numel = (1 << 20) + 40                      # not a multiple of world * 8: the padded tail is exercised
        red = CopyEngineAllReducer(numel, dev)
        gen = torch.Generator(device=dev).manual_seed(8765 + rank)
        ok = True
        for _ in range(3):                          # replays of the captured sequence
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
            ok = ok and bool(((got - want).abs() <= ulp).all())
            same = red.flat[:numel].clone()
            dist.broadcast(same, src=0)
            ok = ok and torch.equal(same, red.flat[:numel])
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        res["copy_engine_allreduce_vs_nccl_sum"] = {"ok": bool(flag.item()), "numel": numel, "calls": 3,
                                                    "tolerance": "one bf16 step of the fp32 sum, identical on all ranks"}
        del red
    except Exception as e:   # noqa: BLE001
        res["copy_engine_allreduce_vs_nccl_sum"] = {"ok": False, "error": f"{type(e).__name__}: {e}"[:300]}
    try:
        from shard import ColumnShardedGemm
        gen = torch.Generator(device=dev).manual_seed(99)           # the same operands on every rank
        m, n, k = 1024, 2048 * world if 2048 * world <= 16384 else 16384, 2048
        xs = torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16)
        ws = torch.randn(n, k, device=dev, generator=gen).to(torch.bfloat16)
        for fmt in ("nvfp4", "mxfp8"):
            sharded = ColumnShardedGemm(ws, fmt)(xs, contiguous=True)
            quant = ops.quantize_nvfp4 if fmt == "nvfp4" else ops.quantize_mxfp8
            gemm = ops.gemm_nvfp4 if fmt == "nvfp4" else ops.gemm_mxfp8
            xc, xsf, _, _ = quant(xs, True, False)
            wc, wsf, _, _ = quant(ws, True, False)
            full = gemm(xc, xsf, wc, wsf, None, torch.bfloat16)
            ok = torch.equal(sharded, full)
            flag = torch.tensor([1 if ok else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            res[f"column_sharded_gemm_{fmt}_bit_identical"] = {"ok": bool(flag.item()), "shape": [m, n, k]}
        ops.check_status(dev)
    except Exception as e:   # noqa: BLE001
        res["column_sharded_gemm"] = {"ok": False, "error": f"{type(e).__name__}: {e}"[:200]}
    res["all_ok"] = all(v.get("ok", False) for v in res.values() if isinstance(v, dict))
    return res


# --------------------------------------------------------------------------------------
# our arm, default workload
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
    # One GPU, nothing else on it: let large layers run the independent halves of a layer call on
    # two streams.  Off with a gradient exchange in flight (its rendezvous kernels wait for other
    # GPUs, and work queued behind them on a shared hardware queue would wait too).
    from backend import _lib as _l0
    _l0.lib().fp4t_set_layer_concurrency(1 if world == 1 else 0)
    peaks = measured_peaks()
    mg_check = multi_gpu_check(ops, dev, rank, world) if world > 1 else None

    nsets = 2   # rotate input sets; one set alone (160 MB bf16) already exceeds the 126 MB L2
    sets = [synth_inputs(N, IC, OC, 100 * rank + s, dev) for s in range(nsets)]
    for s in sets[1:]:
        s[1] = sets[0][1]          # weights are shared state, only the batch changes
    bias = sets[0][3]
    ev = torch.cuda.Event
    # weight and bias gradients land in one flat buffer (two of them, rotating) so that a single
    # all-reduce per step, on a side stream, can overlap the kernels of step i+1, as it does
    # under the backward pass of the previous layer in data-parallel training
    reducers = None
    # default: the library's copy-engine exchange (measured inside the step at 4 GPUs: 0.267-0.284 ms
    # against 0.29-0.30 with NCCL and 0.254 with no exchange at all); FP4T_ALLREDUCE=nccl|switch|off
    exchange = os.environ.get("FP4T_ALLREDUCE", "copy") if world > 1 else "none"
    exchange_note = None
    if exchange == "copy" and mg_check is not None and not mg_check.get("copy_engine_allreduce_vs_nccl_sum", {}).get("ok", False):
        exchange, exchange_note = "nccl", "the copy-engine exchange failed its check before the timed region; NCCL used"
    if exchange == "copy":
        # reduce-scatter + all-gather on the copy engines (no SM taken from the step's kernels
        # beyond a few-MB sum); NCCL if symmetric memory cannot be set up on these GPUs
        try:
            from dp import CopyEngineAllReducer
            reducers = [CopyEngineAllReducer(OC * IC + OC, dev, reduce_ctas=int(os.environ.get("FP4T_ALLREDUCE_CTAS", "0")),
                                             reduce=os.environ.get("FP4T_ALLREDUCE_REDUCE", "auto"))
                        for _ in range(2)]
        except Exception as e:   # noqa: BLE001
            if rank == 0:
                print(f"bench: copy-engine all-reduce unavailable ({e!r}); using NCCL", file=sys.stderr)
            reducers, exchange = None, "nccl"
    if exchange == "switch":
        # the library's own in-switch all-reduce (opt-in: inside the step it measured a few per
        # cent behind NCCL); NCCL if these GPUs offer no NVLink multicast
        try:
            from dp import SwitchAllReducer
            reducers = [SwitchAllReducer(OC * IC + OC, dev, ctas=int(os.environ.get("FP4T_ALLREDUCE_CTAS", "148")))
                        for _ in range(2)]
        except Exception as e:   # noqa: BLE001
            if rank == 0:
                print(f"bench: in-switch all-reduce unavailable ({e!r}); using NCCL", file=sys.stderr)
            reducers, exchange = None, "nccl"
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
                                         out_dw=flat[:OC * IC].view(OC, IC), out_db=flat[OC * IC:OC * IC + OC])
        if world > 1:
            ready = ev()
            ready.record()
            with torch.cuda.stream(comm_stream):
                comm_stream.wait_event(ready)
                if exchange == "switch":
                    reducers[slot].all_reduce(ops.status_word(dev))
                    ops.LAUNCHES["allreduce"] += 1
                elif exchange == "copy":
                    reducers[slot].all_reduce()
                    ops.LAUNCHES["allreduce"] += 3      # two rendezvous launches and the shard sum
                elif exchange == "nccl":
                    dist.all_reduce(flat)
                comm_done[slot] = ev()
                comm_done[slot].record()
        return y, dx, dw, db

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()          # nvidia-smi needs a moment before its first sample: start it ahead of the warm-up
    for i in range(warm):
        hot_step(i)
    barrier()
    if exchange in ("copy", "switch"):
        # a wait of the library's exchange that ran out (a peer that never arrived) shows in the
        # status word: finish the measurement on NCCL rather than not at all, and say so
        bad = torch.tensor([int(ops.status_word(dev)[0].item())], device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()) != 0:
            exchange_note = f"the {exchange} exchange reported status {int(bad.item())} during warm-up; NCCL used"
            if rank == 0:
                print(f"bench: {exchange_note}", file=sys.stderr)
            ops.status_word(dev).zero_()
            exchange, comm_done[0], comm_done[1] = "nccl", None, None
            for i in range(warm):
                hot_step(i)
            barrier()
    launches0 = dict(ops.LAUNCHES)

    # ---- exactly K timed steps ----
    t_start, t_end = event_pair()
    barrier()
    mark0 = sampler.mark()
    t_start.record()
    host_t0 = time.perf_counter()
    for i in range(args.steps):
        hot_step(i)
    host_enqueue_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps   # CPU time to enqueue one step
    t_end.record()
    barrier()
    mark1 = sampler.mark()
    ms_total = t_start.elapsed_time(t_end)
    launches = sum(ops.LAUNCHES.values()) - sum(launches0.values())
    ops.check_status(dev)
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t[0])
    ms_step = ms_total / args.steps

    # ---- the same K-step block repeated until >= min_seconds of device time ----
    blocks = max(1, int(math.ceil(args.min_seconds * 1e3 / max(ms_total, 1e-6))))
    s_start, s_end = event_pair()
    barrier()
    smark0 = sampler.mark()
    s_start.record()
    for b in range(blocks):
        for i in range(args.steps):
            hot_step(b * args.steps + i)
    s_end.record()
    barrier()
    smark1 = sampler.mark()
    ops.check_status(dev)
    t = torch.tensor([s_start.elapsed_time(s_end)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sus_ms_total = float(t[0])
    sus_ms_step = sus_ms_total / (blocks * args.steps)

    # per-kernel durations: each kernel of the step launched back to back between two CUDA
    # events (events between the kernels of a live step would time launch gaps instead)
    reps = max(10, min(args.steps, 50))
    closures, operands = kernel_closures(ops, sets[0], bias)
    timed = {name: time_kernel(fn, reps) for name, fn in closures.items()}
    kern_ms = {name: t[0] for name, t in timed.items()}
    kern_how = {name: t[1] for name, t in timed.items()}
    gemm_names = ("fprop", "dgrad", "wgrad")

    def three_gemms():
        for n in gemm_names:
            closures[n]()

    def three_quants():
        for n in ("quant_w", "quant_x", "quant_g"):
            closures[n]()

    kmark0 = sampler.mark()
    gemm_sus_ms, gemm_sus_reps = time_for_seconds(three_gemms, args.kernel_seconds)
    kmark1 = sampler.mark()
    quant_sus_ms, _ = time_for_seconds(three_quants, min(args.kernel_seconds, 0.5))
    comparator = run_comparator(ops, operands, kern_ms, reps) if rank == 0 or world == 1 else None
    del closures, operands

    # end-to-end through the module API with host buffers
    e2e_ms, h2d, d2h, h2d_gbs = run_e2e(args, dev, rank, world)
    sampler.stop()

    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t[0])
    if rank != 0:
        return
    value = world * FLOP_PER_STEP / (ms_step * 1e-3) / 1e12
    gemm_ms = sum(kern_ms[n] for n in gemm_names)
    gemm_tflops = FLOP_PER_STEP / (gemm_ms * 1e-3) / 1e12
    gemm_sus_tflops = FLOP_PER_STEP / (gemm_sus_ms * 1e-3) / 1e12
    quant_ms = kern_ms["quant_w"] + kern_ms["quant_x"] + kern_ms["quant_g"]
    quant_gbs = QUANT_BYTES / (quant_ms * 1e-3) / 1e9
    quant_sus_gbs = QUANT_BYTES / (quant_sus_ms * 1e-3) / 1e9
    peak_burst, peak_sus = 4.0 * peaks["bf16_burst"], 4.0 * peaks["bf16"]
    clocks = sampler.summary(mark0, mark1)
    if not clocks.get("samples"):
        clocks = sampler.summary(mark0, smark1)     # K steps can be shorter than one sampling period
    sus_clocks = sampler.summary(smark0, smark1)
    gemm_clocks = sampler.summary(kmark0, kmark1)

    cpu = cpu1 = None
    if world == 1 and not args.no_cpu_baseline:
        times = cpu_path_seconds(N, 1, 0)
        cpu = {"value": FLOP_PER_STEP / times[0] / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
               "kind": "port", "seconds": times[0],
               "sample": "one pass over the whole workload (all 8192 rows), no warm-up pass"}
        cpu1 = cpu_config1_baseline()

    config = base_config(world)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate, bf16 out)", "data": "synthetic",
        "config": config,
        "details": {"allreduce": {"none": "none",
                                  "off": "EXPERIMENT: no exchange (not a data-parallel step)",
                                  "switch": "fp4t in-switch multimem kernel on a side stream, one call per step",
                                  "copy": "fp4t reduce-scatter + all-gather on the copy engines (peer copies, one-warp "
                                          "rendezvous, shard sum), one graph launch per step on a side stream",
                                  "nccl": "NCCL on a side stream, one call per step"}.get(exchange, exchange),
                    **({"allreduce_note": exchange_note} if exchange_note else {}),
                    "bias_grad": "fused into the dY quantizer (fp32 atomics + finishing kernel)",
                    "layer_concurrency": ("on: X's quantizer beside W's, dgrad beside wgrad (two streams, joined)"
                                          if world == 1 else "off (a gradient exchange is in flight)"),
                    "frac_of_nominal_fp4_peak": value / world / FP4_NOMINAL_TFLOPS},
        "sustained": {"value": world * FLOP_PER_STEP / (sus_ms_step * 1e-3) / 1e12, "unit": UNIT,
                      "ms_per_step": sus_ms_step, "steps": blocks * args.steps, "seconds": sus_ms_total * 1e-3,
                      "clocks": sus_clocks,
                      "ms_x_sm_mhz": (sus_ms_step * sus_clocks["sm_mhz"]) if sus_clocks.get("sm_mhz") else None,
                      "frac_of_nominal_fp4_peak": FLOP_PER_STEP / (sus_ms_step * 1e-3) / 1e12 / FP4_NOMINAL_TFLOPS},
        "roofline": {"bound": "tensor", "kernel": "gemm_blockscaled_kernel<nvfp4, 256, 2> CTA pairs (fprop+dgrad+wgrad)",
                     "achieved": gemm_tflops, "peak": peak_burst, "unit": UNIT, "frac": gemm_tflops / peak_burst,
                     "peak_basis": f"4 x {peaks['source']} burst bf16 cuBLAS TFLOP/s (FP4:BF16 dense ratio) for the "
                                   f"kernel timed alone over {reps} launches; nominal dense FP4 is {FP4_NOMINAL_TFLOPS:.0f}",
                     "frac_of_nominal": gemm_tflops / FP4_NOMINAL_TFLOPS, "traffic": GEMM_DRAM_TRAFFIC,
                     "ms_per_launch": gemm_ms / 3,
                     "sustained": {"achieved": gemm_sus_tflops, "peak": peak_sus, "frac": gemm_sus_tflops / peak_sus,
                                   "frac_of_nominal": gemm_sus_tflops / FP4_NOMINAL_TFLOPS,
                                   "peak_basis": f"4 x {peaks['source']} sustained bf16 cuBLAS TFLOP/s",
                                   "ms_per_launch": gemm_sus_ms / 3, "launches": 3 * gemm_sus_reps,
                                   "clocks": gemm_clocks}},
        "roofline_quantize": {"bound": "hbm", "kernel": "quantize_tma_kernel<nvfp4> (X, W, dY)",
                              "achieved": quant_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                              "frac": quant_gbs / peaks["hbm_gbs"], "peak_basis": f"{peaks['source']} copy bandwidth",
                              "traffic": QUANT_DRAM_TRAFFIC, "ms_per_launch": quant_ms / 3,
                              "sustained": {"achieved": quant_sus_gbs, "frac": quant_sus_gbs / peaks["hbm_gbs"]}},
        "kernel_ms": kern_ms,
        "kernel_timing": kern_how,
        "comparator": comparator,
        "e2e": {"value": world * FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "h2d_gbs_per_rank_alone": h2d_gbs,      # the same pinned buffers copied with nothing else running, slowest rank
                "api": "custom.CublasltNvfp4Linear forward+backward under bf16 autocast"},
        "gpu_launches": launches,
        "host_enqueue_ms_per_step": host_enqueue_ms,
        "clocks": clocks,
    }
    if mg_check is not None:
        line["multi_gpu_check"] = mg_check
    if cpu is not None:
        line["cpu_baseline"] = cpu
        line["cpu_baseline_config1"] = cpu1
    print(json.dumps(line), flush=True)


def kernel_closures(ops, inputs, bias):
    """The launches of one step as standalone closures over prepared operands, and the GEMM
    operands by name (for the library comparator)."""
    x, w, g, _ = inputs
    wc, wsf, wtc, wtsf = ops.quantize_nvfp4(w, True, True)
    xc, xsf, xtc, xtsf = ops.quantize_nvfp4(x, True, True)
    gc, gsf, gtc, gtsf = ops.quantize_nvfp4(g, True, True, sr=ops.SR_HASH, seed=1)
    y = torch.empty(N, OC, dtype=torch.bfloat16, device=x.device)
    dx = torch.empty(N, IC, dtype=torch.bfloat16, device=x.device)
    dw = torch.empty(OC, IC, dtype=torch.bfloat16, device=x.device)
    closures = {
        "quant_w": lambda: ops.quantize_nvfp4(w, True, True),
        "quant_x": lambda: ops.quantize_nvfp4(x, True, True),
        "quant_g": lambda: ops.quantize_nvfp4(g, True, True, sr=ops.SR_HASH, seed=1, bias_grad_dtype=torch.bfloat16),
        "fprop": lambda: ops.gemm_nvfp4(xc, xsf, wc, wsf, bias, torch.bfloat16, out=y),
        "dgrad": lambda: ops.gemm_nvfp4(gc, gsf, wtc, wtsf, None, torch.bfloat16, out=dx),
        "wgrad": lambda: ops.gemm_nvfp4(gtc, gtsf, xtc, xtsf, None, torch.bfloat16, out=dw),
    }
    operands = {"fprop": (xc, xsf, wc, wsf), "dgrad": (gc, gsf, wtc, wtsf), "wgrad": (gtc, gtsf, xtc, xtsf)}
    return closures, operands


def run_single_kernel(args):
    """--kernel NAME: launch one kernel of the step --steps times (after --warmup launches).
    This is the small command the ncu captures under profiles/ were taken with."""
    from backend import ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.kernel in ("layernorm_fwd", "layernorm_bwd"):
        # the LayerNorm of the small model: 512 x 50 tokens of width 192, fp32 residual stream in,
        # bf16 out / bf16 gradient in (29.5 and 49 MB of traffic per launch)
        g = torch.Generator(device=dev).manual_seed(0)
        x = torch.randn(25600, 192, device=dev, generator=g)
        gamma = torch.ones(192, device=dev)
        beta = torch.zeros(192, device=dev)
        dy = torch.randn(25600, 192, device=dev, generator=g).to(torch.bfloat16)
        _, mean, rstd = ops.layernorm_forward(x, gamma, beta, 1e-5, torch.bfloat16)
        if args.kernel == "layernorm_fwd":
            fn = lambda: ops.layernorm_forward(x, gamma, beta, 1e-5, torch.bfloat16)      # noqa: E731
        else:
            fn = lambda: ops.layernorm_backward(dy, x, mean, rstd, gamma)                  # noqa: E731
        ms = time_loop(fn, args.steps, warm=args.warmup)
        print(json.dumps({"kernel": args.kernel, "launches": args.steps, "ms_per_launch": ms}))
        return
    if args.kernel == "gemm_short_k":
        # an output-bound product of the small model: 25600 x 768 x 192 (one K stage per tile, 39 MB
        # of bf16 output), the shape the eight-warp epilogue form exists for
        g = torch.Generator(device=dev).manual_seed(0)
        a = torch.randn(25600, 192, device=dev, generator=g).to(torch.bfloat16)
        b = (torch.randn(768, 192, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        ac, asf, _, _ = ops.quantize_nvfp4(a)
        bc, bsf, _, _ = ops.quantize_nvfp4(b)
        out = torch.empty(25600, 768, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.gemm_nvfp4(ac, asf, bc, bsf, None, torch.bfloat16, out=out)      # noqa: E731
        ms = time_loop(fn, args.steps, warm=args.warmup)
        ops.check_status(dev)
        print(json.dumps({"kernel": args.kernel, "launches": args.steps, "ms_per_launch": ms}))
        return
    inputs = synth_inputs(N, IC, OC, 0, dev)
    fn = kernel_closures(ops, inputs, inputs[3])[0][args.kernel]
    ms = time_loop(fn, args.steps, warm=args.warmup)
    ops.check_status(dev)
    print(json.dumps({"kernel": args.kernel, "launches": args.steps, "ms_per_launch": ms}))


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
    # what the host side can feed: the same pinned buffers copied with nothing else running, all
    # ranks at once (the end-to-end number is bound by this copy, so it is printed beside it)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    c0 = time.perf_counter()
    for _ in range(3):
        start_copy(0)
        consumed[0].record()
    copy_stream.synchronize()
    h2d_gbs = 3 * h2d / (time.perf_counter() - c0) / 1e9
    if world > 1:
        tmin = torch.tensor([h2d_gbs], device=dev, dtype=torch.float64)
        dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
        h2d_gbs = float(tmin[0])
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    run(steps)
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) * 1e3 / steps, h2d, 4, h2d_gbs


# --------------------------------------------------------------------------------------
# --config mlp_mxfp8: MXFP8 transformer-MLP linear pair, forward + backward
# --------------------------------------------------------------------------------------
def run_mlp_mxfp8(args, rank, world, local_rank):
    import torch.distributed as dist

    from backend import ops
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    n, ic, hid = 16384, 4096, 14336
    flop = 2 * 3 * 2.0 * n * ic * hid            # two linears x three GEMMs
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    torch.manual_seed(0)
    chan = torch.distributions.StudentT(3.0).sample((ic,)).abs().to(dev)      # heavy-tailed channels
    x = (torch.randn(n, ic, device=dev, generator=gen) * chan).to(torch.bfloat16)
    w_up = (torch.randn(hid, ic, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    w_dn = (torch.randn(ic, hid, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    gy = (torch.randn(n, ic, device=dev, generator=gen) * 1e-3).to(torch.bfloat16)
    grads = torch.empty(2 * hid * ic, dtype=torch.bfloat16, device=dev)

    def step(i):
        h, ws_up = ops.linear_forward("mxfp8", x, w_up, None, True, True, torch.bfloat16)
        y, ws_dn = ops.linear_forward("mxfp8", h, w_dn, None, True, True, torch.bfloat16)
        dh, _, _ = ops.linear_backward("mxfp8", gy, ws_dn, hid, True, True, False,
                                       out_dw=grads[:hid * ic].view(ic, hid))
        dx, _, _ = ops.linear_backward("mxfp8", dh, ws_up, ic, True, True, False,
                                       out_dw=grads[hid * ic:].view(hid, ic))
        if world > 1:
            dist.all_reduce(grads)
        return y, dx

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for i in range(warm):
        step(i)
    barrier()
    l0 = sum(ops.LAUNCHES.values())
    a, b = event_pair()
    m0 = sampler.mark()
    a.record()
    for i in range(args.steps):
        step(i)
    b.record()
    barrier()
    m1 = sampler.mark()
    sampler.stop()
    launches = sum(ops.LAUNCHES.values()) - l0
    ops.check_status(dev)
    t = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t[0]) / args.steps
    # the dominant kernel alone: the up-projection forward GEMM
    xc, xsf, _, _ = ops.quantize_mxfp8(x, True, False)
    uc, usf, _, _ = ops.quantize_mxfp8(w_up, True, False)
    h = torch.empty(n, hid, dtype=torch.bfloat16, device=dev)
    gemm_ms = time_loop(lambda: ops.gemm_mxfp8(xc, xsf, uc, usf, None, torch.bfloat16, out=h), 10)
    quant_ms = time_loop(lambda: ops.quantize_mxfp8(x, True, True), 10)
    if rank != 0:
        return
    gemm_tf = 2.0 * n * ic * hid / (gemm_ms * 1e-3) / 1e12
    peak = 2.0 * peaks["bf16_burst"]
    value = world * flop / (ms_step * 1e-3) / 1e12
    qbytes = (2.0 + 2 * 1.0 + 2.0 / 32) * n * ic
    line = {"metric": "mxfp8_mlp_pair_fwd_bwd_tflops", "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "mxfp8 (e4m3 x ue8m0, fp32 accumulate, bf16 out)", "data": "synthetic",
            "config": {"workload": "mxfp8 MLP pair fwd+bwd N=16384 4096->14336->4096 (8 quantizer + 6 GEMM launches)",
                       "l2": "inputs larger than L2 (X 134 MB, H 470 MB)",
                       "parallelism": f"dp{world}" if world > 1 else "single"},
            "roofline": {"bound": "tensor", "kernel": "gemm_blockscaled_kernel<mxfp8, 256, 2> (up-projection fprop 16384x14336x4096)",
                         "achieved": gemm_tf, "peak": peak, "unit": UNIT, "frac": gemm_tf / peak,
                         "peak_basis": f"2 x {peaks['source']} burst bf16 cuBLAS TFLOP/s (FP8:BF16 dense ratio); nominal dense FP8 is 4500",
                         "frac_of_nominal": gemm_tf / FP8_NOMINAL_TFLOPS, "traffic": None, "ms_per_launch": gemm_ms},
            "roofline_quantize": {"bound": "hbm", "kernel": "quantize_tma_kernel<mxfp8> (X 16384x4096 row+transposed)",
                                  "achieved": qbytes / (quant_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                  "frac": qbytes / (quant_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "ms_per_launch": quant_ms},
            "frac_of_nominal_fp8_peak": value / world / FP8_NOMINAL_TFLOPS,
            "gpu_launches": launches, "clocks": sampler.summary(m0, m1),
            "parity_note": "MXFP8 quantizer parity is unpinned (the reference's microxcaling source is absent)"}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# --config gemm_sweep
# --------------------------------------------------------------------------------------
def run_gemm_sweep(args, rank, world, local_rank):
    import torch.distributed as dist

    from backend import ops
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    sizes = [1024, 2048, 4096, 8192, 16384]
    shapes = [(m, n, k) for m in sizes for n in sizes for k in sizes] + [(16, 8192, 8192), (128, 8192, 8192)]
    if args.sweep_max:
        shapes = [s for s in shapes if max(s) <= args.sweep_max or s[0] < 1024]
    gen = torch.Generator(device=dev).manual_seed(0)
    rows = []
    tot_flop = {"nvfp4": 0.0, "mxfp8": 0.0}
    tot_ms = {"nvfp4": 0.0, "mxfp8": 0.0}
    launches = 0
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    cache = {}

    def operand(fmt, outer, k):
        key = (fmt, outer, k)
        if key not in cache:
            if len(cache) > 12:
                cache.clear()
            t = torch.randn(outer, k, device=dev, generator=gen).to(torch.bfloat16)
            q = ops.quantize_nvfp4 if fmt == "nvfp4" else ops.quantize_mxfp8
            cache[key] = q(t, True, False)[:2]
        return cache[key]

    reps = max(3, min(args.steps, 10))
    for fmt in ("nvfp4", "mxfp8"):
        gemm = ops.gemm_nvfp4 if fmt == "nvfp4" else ops.gemm_mxfp8
        for (m, n, k) in sorted(shapes, key=lambda s: (s[2], s[0], s[1])):
            n_local = n // world if world > 1 and n % (128 * world) == 0 else n
            ac, asf = operand(fmt, m, k)
            bc, bsf = operand(fmt, n, k)
            if n_local != n:
                bc = bc[rank * n_local:(rank + 1) * n_local]
                nt = (k // (16 if fmt == "nvfp4" else 32) + 3) // 4
                bsf = bsf.view(-1)[rank * (n_local // 128) * nt * 512:(rank + 1) * (n_local // 128) * nt * 512]
            out = torch.empty(m, n_local, dtype=torch.bfloat16, device=dev)
            gathered = torch.empty(world, m, n_local, dtype=torch.bfloat16, device=dev) if n_local != n else None

            def call():
                gemm(ac, asf, bc, bsf, None, torch.bfloat16, out=out)
                if gathered is not None:
                    dist.all_gather_into_tensor(gathered.view(-1), out.view(-1))

            if world == 1:
                ms, _how = time_kernel(call, reps, warm=max(1, min(args.warmup, 3)))
            else:
                ms = time_loop(call, reps, warm=max(1, min(args.warmup, 3)))
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t[0])
            launches += reps
            flop = 2.0 * m * n * k
            eb = 0.5 + 1.0 / 16 if fmt == "nvfp4" else 1.0 + 1.0 / 32
            byts = (m + n) * k * eb + 2.0 * m * n
            tot_flop[fmt] += flop
            tot_ms[fmt] += ms
            nominal = FP4_NOMINAL_TFLOPS if fmt == "nvfp4" else FP8_NOMINAL_TFLOPS
            tf = flop / (ms * 1e-3) / 1e12
            rows.append({"fmt": fmt, "m": m, "n": n, "k": k, "ms": round(ms, 5), "tflops": round(tf, 1),
                         "frac_of_nominal": round(tf / world / nominal, 4),
                         "gbs": round(byts / (ms * 1e-3) / 1e9, 1),
                         "bound": "hbm" if m < 1024 else "tensor",
                         "sharded_all_gather": n_local != n})
    sampler.stop()
    ops.check_status(dev)
    if rank != 0:
        return
    value = (tot_flop["nvfp4"] + tot_flop["mxfp8"]) / ((tot_ms["nvfp4"] + tot_ms["mxfp8"]) * 1e-3) / 1e12
    skinny = [r for r in rows if r["m"] < 1024]
    best = {fmt: max((r for r in rows if r["fmt"] == fmt), key=lambda r: r["tflops"]) for fmt in ("nvfp4", "mxfp8")}
    line = {"metric": "blockscaled_gemm_sweep_tflops", "value": value, "unit": UNIT, "n_gpus": world,
            "steps": reps, "warmup": max(1, min(args.warmup, 3)), "ms_per_step": tot_ms["nvfp4"] + tot_ms["mxfp8"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "nvfp4 and mxfp8 block-scaled, fp32 accumulate, bf16 out", "data": "synthetic",
            "config": {"workload": f"GEMM sweep, {len(shapes)} shapes x 2 formats, operands quantized once (not timed)",
                       "l2": "each GEMM repeated back to back on the same operands; operand sets above 126 MB exceed L2",
                       "parallelism": ("single" if world == 1 else
                                       f"N (the [N,K] operand) sharded over {world} ranks + NCCL all-gather of Y")},
            "per_format_tflops": {f: tot_flop[f] / (tot_ms[f] * 1e-3) / 1e12 for f in tot_flop},
            "roofline": {"bound": "tensor", "kernel": "gemm_blockscaled_kernel (best shape per format)",
                         "achieved": best["nvfp4"]["tflops"], "peak": 4.0 * peaks["bf16_burst"], "unit": UNIT,
                         "frac": best["nvfp4"]["tflops"] / world / (4.0 * peaks["bf16_burst"]),
                         "best": best, "traffic": None},
            "roofline_skinny": {"bound": "hbm", "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "rows": [{**r, "frac": round(r["gbs"] / peaks["hbm_gbs"], 4)} for r in skinny]},
            "shapes": rows, "gpu_launches": launches, "clocks": sampler.summary()}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# --config tinyvit
# --------------------------------------------------------------------------------------
def run_tinyvit(args, rank, world, local_rank):
    """steps/s of the TinyViT-style training step with all 36 projections in NVFP4.  The headline
    replays the step from CUDA graphs (the step is launch-bound at this size); the same model
    run eagerly, and a plain bf16 torch model both ways, are reported beside it."""
    from backend import ops
    from train_tinyvit import train
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    steps = args.steps if args.steps_given else 200
    warm = max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    l0 = sum(ops.LAUNCHES.values())
    m0 = sampler.mark()
    # headline: the model with the library's block-level options (LayerNorm kernels, q / k / v as one
    # quantization + one GEMM); the same recipe on the reference's module tree, and plain bf16
    # torch with and without the LayerNorm kernels, are measured beside it
    res = train("cublaslt_nvfp4", steps=steps, warmup=warm, batch=512, depth=6, seed=0, graph=True,
                fused_norm=True, fuse_qkv=True)
    m1 = sampler.mark()
    launches_captured = sum(ops.LAUNCHES.values()) - l0
    plain = train("cublaslt_nvfp4", steps=steps, warmup=warm, batch=512, depth=6, seed=0, graph=True)
    eager = train("cublaslt_nvfp4", steps=min(steps, 50), warmup=warm, batch=512, depth=6, seed=0,
                  fused_norm=True, fuse_qkv=True)
    base = train("torch", steps=min(steps, 50), warmup=warm, batch=512, depth=6, seed=0)
    base_graph = train("torch", steps=steps, warmup=warm, batch=512, depth=6, seed=0, graph=True)
    base_norm_graph = train("torch", steps=steps, warmup=warm, batch=512, depth=6, seed=0, graph=True, fused_norm=True)
    # the attention core through torch's scaled_dot_product_attention (a library kernel, not this
    # library's): reported beside the headline for both recipes, not as the headline
    sdpa = train("cublaslt_nvfp4", steps=steps, warmup=warm, batch=512, depth=6, seed=0, graph=True,
                 fused_norm=True, fuse_qkv=True, sdpa=True)
    base_sdpa = train("torch", steps=steps, warmup=warm, batch=512, depth=6, seed=0, graph=True, fused_norm=True, sdpa=True)
    sampler.stop()
    ops.check_status(dev)
    if rank != 0:
        return
    # per block: q/k/v stacked + o + up + down = 4 projection groups of 3 launches forward (W, X, GEMM) and
    # 5-6 backward (zero, dY, finish, dgrad, wgrad + split-K sum), 2 LayerNorms of 1 + 2 launches
    per_step = 6 * (4 * 8 + 2 * 3)
    line = {"metric": "tinyvit_nvfp4_steps_per_s", "value": res["steps_per_s"], "unit": "steps/s", "n_gpus": world,
            "steps": steps, "warmup": warm, "ms_per_step": 1e3 / res["steps_per_s"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "nvfp4 linears (36 projections; q/k/v stacked), bf16 autocast elsewhere", "data": "synthetic",
            "config": {"workload": "TinyViT-style classifier: 28x28x1, patch 4, hidden 192, depth 6, 3 heads, MLP 768, "
                                   "batch 512 per GPU, AdamW lr 1e-3, seed 0",
                       "l2": "model and activations fit L2; each step draws a fresh batch on the device",
                       "parallelism": f"dp{world}" if world > 1 else "single",
                       "execution": "forward+backward and optimizer step replayed from two CUDA graphs, "
                                    "one all-reduce of the flat gradient buffer between them"},
            "images_per_s": res["images_per_s"], "first_loss": res["first_loss"], "last_loss": res["last_loss"],
            "loss_curve": [round(v, 4) for v in res["losses"][:: max(1, len(res["losses"]) // 25)]],
            "model_options": {"fused_norm": True, "fuse_qkv": True},
            "eager_steps_per_s": eager["steps_per_s"],
            "nvfp4_reference_module_tree_graph_steps_per_s": plain["steps_per_s"],
            "bf16_torch_steps_per_s": base["steps_per_s"], "bf16_torch_graph_steps_per_s": base_graph["steps_per_s"],
            "bf16_torch_graph_with_fused_norm_steps_per_s": base_norm_graph["steps_per_s"],
            "speedup_over_bf16_torch": res["steps_per_s"] / base["steps_per_s"],
            "speedup_over_bf16_torch_graph": res["steps_per_s"] / base_graph["steps_per_s"],
            "speedup_over_bf16_torch_graph_with_fused_norm": res["steps_per_s"] / base_norm_graph["steps_per_s"],
            "speedup_reference_module_tree_over_bf16_torch_graph": plain["steps_per_s"] / base_graph["steps_per_s"],
            "with_torch_sdpa": {"nvfp4_steps_per_s": sdpa["steps_per_s"],
                                "bf16_torch_with_fused_norm_steps_per_s": base_sdpa["steps_per_s"],
                                "speedup": sdpa["steps_per_s"] / base_sdpa["steps_per_s"],
                                "note": "attention core = torch scaled_dot_product_attention in both arms"},
            "gpu_launches": per_step * steps, "gpu_launches_note":
                f"{per_step} kernels of this library per replayed step ({launches_captured} enqueued by the host for warm-up and capture)",
            "clocks": sampler.summary(m0, m1)}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="linear_nvfp4", choices=["linear_nvfp4", "mlp_mxfp8", "gemm_sweep", "tinyvit"])
    ap.add_argument("--min-seconds", type=float, default=2.0, help="length of the sustained region (device time)")
    ap.add_argument("--kernel-seconds", type=float, default=1.0, help="length of the GEMM-only sustained loop")
    ap.add_argument("--sample-rows", type=int, default=0,
                    help="reference arm: rows of X and dY per step (0 = the whole workload)")
    ap.add_argument("--sweep-max", type=int, default=0, help="gemm_sweep: largest dimension to include (0 = all)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel", default=None,
                    choices=["quant_w", "quant_x", "quant_g", "fprop", "dgrad", "wgrad", "layernorm_fwd", "layernorm_bwd",
                             "gemm_short_k"],
                    help="run only this kernel of the step (profiling aid); no benchmark line")
    args = ap.parse_args()
    args.steps_given = args.steps is not None
    if args.steps is None:
        args.steps = 200 if args.impl == "ours" else 3

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
        runner = {"linear_nvfp4": run_ours, "mlp_mxfp8": run_mlp_mxfp8, "gemm_sweep": run_gemm_sweep,
                  "tinyvit": run_tinyvit}[args.config]
        runner(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
