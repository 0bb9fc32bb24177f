#!/usr/bin/env python
"""Benchmark of the W4A4 linear hot path (quantizer + GEMM) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c1] [--impl ours|reference]

One JSON line on stdout (rank 0).  A step = one pass of the hot path over one
batch: quantize_w4a4_act_fuse_lora followed by gemm_w4a4 on a 4352-row slab.
With N > 1 (torchrun, one rank per GPU) every rank owns its own slab of rows
and a replica of the weights; there is no data-path collective, so the job is
weak-scaled and `value` is the sum over ranks divided by the slowest rank's
time.

How the device-resident numbers are timed.  One step is two kernels of 10-100 us,
far shorter than a Python launch, so exactly K steps are captured into ONE CUDA
graph (rotating over NSETS input/output sets, more than 3x the L2) and nothing is
launched eagerly inside a timed region.  The graph is replayed once untimed and
then R times, each replay bracketed by CUDA events, until the replays add up to
at least --min-time seconds; `ms_per_step` is the MEDIAN replay divided by K.
The quantizer-only and GEMM-only graphs (K launches each) are timed the same way.

`value`  : TFLOP/s of 2*M*N*K (LoRA FLOPs excluded, the reference's convention)
           with inputs resident in HBM.
`e2e`    : the same metric through the host-buffer C-ABI call: pinned host x in,
           pinned host y out, both copies inside the timed region.
`roofline`: the GEMM kernel alone; `roofline_quantizer`: the quantizer alone.
`config.other_configs`: the other benchmark configurations (c2..c4), per kernel.
`config.tp` (N > 1): the column-sharded (tensor-parallel) form on the c4 shape.
`--impl reference` times the CPU oracle (the reference's PyTorch path restated
in numpy; the reference itself is Python and is not shipped to the GPU box).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NSETS = 6  # rotating input/output sets: 6 x ~70 MB is > 3 x the 126 MB L2

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch, from one ncu capture per kernel and
# configuration (the capture command is in the kernel's profile summary).  Output lines are still in
# L2 when a captured launch ends, so the write-back of y / act shows up in later launches, not here.
# Configurations without a capture report null.
NCU_DRAM_BYTES = {
    "c1": {"gemm_w4a4_kernel": 17_990_400 + 27_904, "quantize_fused_kernel": 34_496_256 + 7_168},
    "c2": {"gemm_w4a4_kernel": 47_763_456 + 84_982_272},
}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


NVFP4_NOMINAL_TFLOPS = 10000.0     # dense NVFP4 peak the targets are stated against
HBM_NOMINAL_GBS = 8000.0


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) every 20 ms.

    Started before the warm-up so that its start-up does not fall into a timed region; only the
    samples taken between mark_begin() and mark_end() count as "under load"."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.period = period_s
        self.samples, self.reasons, self.max_mhz, self.h, self.nv = [], set(), None, None, None
        self._stop_evt = threading.Event()
        self._lock = threading.Lock()
        self._windows, self._open = [], None
        try:
            import pynvml as nv
            nv.nvmlInit()
            # NVML enumerates physical devices; honour CUDA_VISIBLE_DEVICES when it is a plain index list
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis and all(v.strip().isdigit() for v in vis.split(",")):
                index = int(vis.split(",")[index])
            self.h = nv.nvmlDeviceGetHandleByIndex(index)
            self.nv = nv
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
            self.names = {
                nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            }
        except Exception as e:  # NVML missing: report it instead of clocks
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def sample(self):
        if self.nv is None:
            return
        try:
            mhz = self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)
            r = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            with self._lock:
                self.samples.append((time.perf_counter(), mhz, r))
        except Exception as e:
            self.reasons.add(f"nvml_error:{type(e).__name__}")

    def run(self):
        while not self._stop_evt.is_set():
            self.sample()
            self._stop_evt.wait(self.period)

    def mark_begin(self):
        self.sample()
        self._open = time.perf_counter()

    def mark_end(self):
        self.sample()
        if self._open is not None:
            self._windows.append((self._open, time.perf_counter()))
            self._open = None

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        with self._lock:
            inside = [(m, r) for (t, m, r) in self.samples if any(a - 0.03 <= t <= b + 0.03 for a, b in self._windows)]
        mhz = sorted(m for m, _ in inside)
        for _, r in inside:
            for bit, name in getattr(self, "names", {}).items():
                if r & bit:
                    self.reasons.add(name)
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_min_mhz": mhz[0] if mhz else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(mhz)}


def _np_bits(t):
    import numpy as np
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _host_threads():
    ncpu = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = str(ncpu)
    return ncpu


def _blas_threads():
    try:
        from threadpoolctl import threadpool_info
        return max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        return os.cpu_count()


def _oracle_step(shape, rows):
    """(callable running one quantizer + GEMM pass of the CPU oracle over `rows` rows, dtype name)."""
    import torch
    from oracle import nvfp4_oracle as O
    from svdquant_kernels_b200.workloads import make_inputs
    inp = make_inputs(shape, m_rows=rows)
    name = "fp16" if shape.dtype == torch.float16 else "bf16"
    wgt, wsc = O.quantize_nvfp4_rows(inp.w.numpy(), 1)
    xb, ldb, smb = _np_bits(inp.x), _np_bits(inp.lora_down), _np_bits(inp.smooth)
    lub, wcb, bb = _np_bits(inp.lora_up), _np_bits(inp.wcscales), _np_bits(inp.bias)

    def step():
        act, asc, la = O.quantize_w4a4_act_fuse_lora(xb, ldb, smb, name)
        y_bits, y_f32 = O.gemm_w4a4(act, wgt, asc, wsc, la, lub, wcb, bb, name)[:2]
        step.last = (act, asc, la, y_bits, y_f32)
        return y_bits

    step.inputs = inp
    return step, name


def run_reference(args):
    """CPU arm: the oracle (numpy restatement of the reference's PyTorch path) on all rows of the
    same workload, every host core it can use."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ncpu = _host_threads()          # also under torchrun, which exports OMP_NUM_THREADS=1 to every rank
    import torch
    torch.set_num_threads(ncpu)
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=ncpu)
    except Exception:
        pass
    from svdquant_kernels_b200.workloads import CONFIGS, SMALL_M
    shape = CONFIGS.get(args.config) or SMALL_M[args.config]
    rows = shape.M if args.cpu_rows <= 0 else min(shape.M, args.cpu_rows)
    step, name = _oracle_step(shape, rows)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    m_pad = -(-rows // 256) * 256
    tflops = 2.0 * m_pad * shape.N * shape.K / dt / 1e12
    cores = _blas_threads()
    sample = (f"all {rows} rows per step" if rows == shape.M else f"first {rows} of {shape.M} rows per step") + \
        " (quantizer + GEMM oracle, numpy/BLAS)"
    line = {
        "impl": "reference", "metric": "w4a4_linear_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"{shape.name}: W4A4 linear M={shape.M} K={shape.K} N={shape.N} R={shape.R} {name}, rows sharded over ranks, weights replicated",
                   "per_rank_rows": shape.M, "rows_per_step": rows},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


class GraphTimer:
    """Times CUDA graphs by replaying them: one untimed replay, then timed replays (each between two
    CUDA events on the current stream) until they add up to `min_time_s`; reports the median."""

    def __init__(self, torch, min_time_s, min_repeats=5, max_repeats=4000):
        self.torch, self.min_time_s, self.min_repeats, self.max_repeats = torch, min_time_s, min_repeats, max_repeats

    def time(self, graph):
        torch = self.torch
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        first = e0.elapsed_time(e1)
        reps = int(min(self.max_repeats, max(self.min_repeats, math.ceil(self.min_time_s * 1e3 / max(first, 1e-3)))))
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        torch.cuda.synchronize()
        ev[0].record()
        for i in range(reps):
            graph.replay()
            ev[i + 1].record()
        torch.cuda.synchronize()
        ms = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(reps))
        return {"median_ms": ms[len(ms) // 2], "min_ms": ms[0], "p90_ms": ms[min(len(ms) - 1, int(0.9 * len(ms)))],
                "repeats": reps, "total_s": sum(ms) * 1e-3}


class DeviceLinear:
    """One configuration resident on the device: weights, NSETS rotating activation / output sets
    (allocated once; the operators write into them through `out=`), and the graphs over them."""

    def __init__(self, torch, ops, shape, dev, rank=0, nsets=NSETS):
        from svdquant_kernels_b200.workloads import make_inputs
        self.torch, self.ops, self.shape, self.nsets = torch, ops, shape, nsets
        inp = make_inputs(shape, row_offset=rank)          # every rank: its own rows, the same weights
        self.inp = inp
        self.wgt, self.wsc = ops.quantize_nvfp4_rows(inp.w.to(dev), pad_size=1)
        ops.swizzle_scales(self.wsc)
        self.ld, self.lu = inp.lora_down.to(dev), inp.lora_up.to(dev)
        self.sm, self.wc, self.bias = inp.smooth.to(dev), inp.wcscales.to(dev), inp.bias.to(dev)
        self.xs = [inp.x.to(dev)]
        for i in range(1, nsets):
            self.xs.append(self.xs[0].roll(i, dims=0).contiguous())
        # first pass allocates every set's outputs (and their layout twins); later passes reuse them
        self.q = [ops.quantize_w4a4_act_fuse_lora(x, self.ld, self.sm) for x in self.xs]
        self.y = [ops.gemm_w4a4(q[0], self.wgt, q[1], self.wsc, q[2], self.lu, self.wc, self.bias, shape.dtype) for q in self.q]
        torch.cuda.synchronize()

    def quant(self, i):
        i %= self.nsets
        return self.ops.quantize_w4a4_act_fuse_lora(self.xs[i], self.ld, self.sm, out=self.q[i])

    def gemm(self, i):
        i %= self.nsets
        act, asc, la = self.q[i]
        return self.ops.gemm_w4a4(act, self.wgt, asc, self.wsc, la, self.lu, self.wc, self.bias, self.shape.dtype, out=self.y[i])

    def step(self, i):
        self.quant(i)
        return self.gemm(i)

    def gemm_next(self, i):
        """The GEMM that also quantises its result for a following linear (smooth_next -> qout, oscales)."""
        i %= self.nsets
        if not hasattr(self, "sn"):
            torch = self.torch
            g = torch.Generator().manual_seed(99)
            self.sn = (torch.rand(self.shape.N, generator=g) * 1.5 + 0.25).to(self.shape.dtype).to(self.wgt.device)
        act, asc, la = self.q[i]
        return self.ops.gemm_w4a4(act, self.wgt, asc, self.wsc, la, self.lu, self.wc, self.bias, self.shape.dtype,
                                  smooth_next=self.sn)

    def capture(self, fn, n):
        g = self.torch.cuda.CUDAGraph()
        with self.torch.cuda.graph(g):
            for i in range(n):
                fn(i)
        return g


def _kernel_figures(shape, q_us, g_us, peaks):
    from svdquant_kernels_b200.workloads import gemm_flops, quantizer_bytes
    M_pad = -(-shape.M // 256) * 256
    g_tflops = gemm_flops(M_pad, shape.N, shape.K) / (g_us * 1e-6) / 1e12
    q_gbs = quantizer_bytes(shape.M, shape.K, shape.R) / (q_us * 1e-6) / 1e9
    return {"quantizer_us": q_us, "gemm_us": g_us, "gemm_tflops": g_tflops, "pct_of_10pf_nominal": 100.0 * g_tflops / NVFP4_NOMINAL_TFLOPS,
            "quantizer_gbs": q_gbs, "quantizer_frac_hbm": q_gbs / peaks["hbm_gbs"],
            "quantizer_pct_of_8tbs_nominal": 100.0 * q_gbs / HBM_NOMINAL_GBS}


def _tp_block(torch, dist, ops, dev, rank, world, timer_iters=60):
    """Column-sharded (tensor-parallel) form on the c4 shape: x replicated, weight rows sharded.
    fused = svdq_gemm_w4a4_columns (all-gather folded into the GEMM epilogue as TMA stores into the peers'
    copies, a rank barrier on either side); nccl = local slab GEMM + NCCL all-gather + strided copy."""
    from svdquant_kernels_b200 import sharding
    from svdquant_kernels_b200.workloads import CONFIGS, make_inputs
    shape = CONFIGS["c4"]
    inp = make_inputs(shape)                       # same rows and weights on every rank
    M, K, N, R, dt = shape.M, shape.K, shape.N, shape.R, shape.dtype
    col0, n = sharding.column_slab(N, world, rank)
    wgt, wsc = ops.quantize_nvfp4_rows(inp.w.to(dev), pad_size=1)
    lu, wc, bias = inp.lora_up.to(dev), inp.wcscales.to(dev), inp.bias.to(dev)
    act, asc, la = ops.quantize_w4a4_act_fuse_lora(inp.x.to(dev), inp.lora_down.to(dev), inp.smooth.to(dev))
    y_one = ops.gemm_w4a4(act, wgt, asc, wsc, la, lu, wc, bias, dt)            # the single-GPU result
    wgt_s, wsc_s = wgt[col0:col0 + n].contiguous(), wsc[:, col0:col0 + n].contiguous()
    lu_s, wc_s, b_s = lu[col0:col0 + n].contiguous(), wc[col0:col0 + n].contiguous(), bias[col0:col0 + n].contiguous()
    ops.swizzle_scales(wsc_s)
    M_pad = act.shape[0]
    lin = sharding.ColumnShardedLinear(M_pad, N, dt, wgt=wgt_s, wscales=wsc_s, lora_up=lu_s, wcscales=wc_s, bias=b_s)
    y_slab = torch.empty((M_pad, n), dtype=dt, device=dev)

    def local():
        return ops.gemm_w4a4(act, wgt_s, asc, wsc_s, la, lu_s, wc_s, b_s, dt, out=y_slab)

    def fused():
        return lin.forward(act, asc, la)

    def nccl():
        return sharding.linear_columns(None, lambda _x: local(), N)

    def bars():
        lin.handle.barrier(channel=0)
        lin.handle.barrier(channel=1)

    def timed(fn, iters=timer_iters):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
        ev[0].record()
        for i in range(iters):
            fn()
            ev[i + 1].record()
        torch.cuda.synchronize()
        ms = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(iters))
        return ms[len(ms) // 2] * 1e3

    def graphed(fn, calls=10):
        """Device time per call: `calls` calls captured in one CUDA graph, median of 20 replays.  Eager
        calls of these few-kernel sequences are bound by the Python launch path, not by the GPU."""
        try:
            fn()
            torch.cuda.synchronize()
            dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(calls):
                    fn()
            return timed(g.replay, 20) / calls
        except Exception:                              # capture refused: the eager figure stands alone
            torch.cuda.synchronize()
            return float("nan")

    y_f = fused()
    torch.cuda.synchronize()
    same_fused = bool(torch.equal(y_f, y_one))
    same_nccl = bool(torch.equal(nccl(), y_one))
    eager = [timed(local), timed(fused), timed(nccl)]
    graph = [graphed(local), graphed(fused), graphed(bars), graphed(nccl)]
    same_fused = same_fused and bool(torch.equal(fused(), y_one))
    t = torch.tensor(eager + graph + [0.0 if same_fused else 1.0, 0.0 if same_nccl else 1.0], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    local_eager, fused_eager, nccl_eager, local_us, fused_us, bars_us, nccl_us, bad_f, bad_n = t.tolist()
    if fused_us != fused_us or local_us != local_us:   # no graph figure on some rank
        local_us, fused_us, bars_us = local_eager, fused_eager, None
    if nccl_us != nccl_us:
        nccl_us = nccl_eager
    pushed = M_pad * n * 2 * (world - 1)
    return {
        "workload": f"c4 shape M={M} K={K} N={N} R={R} fp16, x replicated, N sharded {world} ways ({n} columns per rank)",
        "timing": "device time per call: 10 calls in one CUDA graph, median of 20 replays, max over ranks; "
                  f"*_eager_us: Python calls, CUDA events per call, median of {timer_iters} (bound by the launch path)",
        "local_gemm_us": local_us, "fused_us": fused_us, "rank_barriers_us": bars_us, "nccl_allgather_us": nccl_us,
        "local_gemm_eager_us": local_eager, "fused_eager_us": fused_eager, "nccl_allgather_eager_us": nccl_eager,
        "bytes_pushed_per_rank": pushed, "fused_push_gbs": pushed / (fused_us * 1e-6) / 1e9,
        "nvlink_measured_gbs_per_direction": 770.0,
        "limiter": "NVLink" if pushed / 770e9 * 1e6 > local_us else "local GEMM + the two rank barriers",
        "nvlink_floor_us": pushed / 770e9 * 1e6,
        "bit_identical_to_1gpu": bad_f == 0.0, "nccl_form_bit_identical_to_1gpu": bad_n == 0.0,
    }


def run_ours(args):
    import torch
    import torch.distributed as dist
    from svdquant_kernels_b200 import _lib, ops
    from svdquant_kernels_b200.workloads import CONFIGS, SMALL_M, gemm_flops, quantizer_bytes

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the product kernels")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    sampler = ClockSampler(local)
    sampler.start()

    shape = CONFIGS.get(args.config) or SMALL_M[args.config]
    name = "fp16" if shape.dtype == torch.float16 else "bf16"
    M, K, N, R = shape.M, shape.K, shape.N, shape.R
    M_pad = -(-M // 256) * 256
    lin = DeviceLinear(torch, ops, shape, dev, rank)
    warm = max(args.warmup, 3)
    for i in range(warm):
        lin.step(i)
    torch.cuda.synchronize()
    rc, words = _lib.device_status()
    if rc != 0:
        raise SystemExit(f"device status after warm-up: {words}")
    if args.eager_only > 0:
        # for profilers: a few more plain launches and nothing else (no graphs, no JSON line)
        for i in range(args.eager_only):
            lin.step(i)
            if args.next_layer:
                lin.gemm_next(i)
        torch.cuda.synchronize()
        sampler.stop()
        print(f"eager-only: {warm + args.eager_only} steps done, status {_lib.device_status()}", file=sys.stderr)
        if world > 1:
            dist.destroy_process_group()
        return

    # eager API-level wall: what a caller that launches step after step from Python sees
    # (host glue + launches; no graphs), on the same rotating sets
    n_eager = 200
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(n_eager):
        lin.step(i)
    torch.cuda.synchronize()
    eager_api_us = (time.perf_counter() - t0) / n_eager * 1e6
    t0 = time.perf_counter()
    for i in range(n_eager):
        lin.step(i)
    host_issue_us = (time.perf_counter() - t0) / n_eager * 1e6       # host time to queue a step (no wait)
    torch.cuda.synchronize()

    steps = args.steps
    g_all = lin.capture(lin.step, steps)
    g_q = lin.capture(lin.quant, steps)
    g_g = lin.capture(lin.gemm, steps)
    timer = GraphTimer(torch, args.min_time)

    # ---- timed region: replays of the K-step graph, inputs resident in HBM ----
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.mark_begin()
    r_all = timer.time(g_all)
    r_q = timer.time(g_q)
    r_g = timer.time(g_g)
    torch.cuda.synchronize()
    sampler.mark_end()
    if world > 1:
        dist.barrier()
    rc, words = _lib.device_status()
    if rc != 0:
        raise SystemExit(f"device status after the timed region: {words}")
    # The long timed region above runs at the board's power cap (the SM clock settles below its maximum).
    # For comparison with figures measured in short runs: the same per-kernel graphs replayed twice after
    # the GPU has idled for half a second, i.e. at the clock a single call or a short burst sees.
    burst = {}
    for key, g_ in (("quantizer_us", g_q), ("gemm_us", g_g), ("step_us", g_all)):
        time.sleep(0.5)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = None
        for _ in range(2):
            e0.record()
            g_.replay()
            e1.record()
            torch.cuda.synchronize()
            t_ = e0.elapsed_time(e1) / steps * 1e3
            best = t_ if best is None else min(best, t_)
        burst[key] = best
    ms_per_step = r_all["median_ms"] / steps
    q_us = r_q["median_ms"] / steps * 1e3
    g_us = r_g["median_ms"] / steps * 1e3
    # the GEMM with the next layer's quantisation fused into its epilogue (a graph of its own; its outputs
    # are allocated inside the capture, from the graph's pool)
    next_us = None
    if rank == 0 and world == 1 and not args.no_other_configs:
        lin.gemm_next(0)
        torch.cuda.synchronize()
        g_n = lin.capture(lin.gemm_next, steps)
        next_us = timer.time(g_n)["median_ms"] / steps * 1e3
        del g_n

    # ---- end to end: host buffers through the C-ABI plan ----
    inp = lin.inp
    wgt_h, wsc_h = lin.wgt.cpu(), lin.wsc.view(torch.uint8).cpu()
    plan = ops.LinearPlan(M, K, N, R, shape.dtype, wgt=wgt_h, wscales=wsc_h, lora_down=inp.lora_down,
                          lora_up=inp.lora_up, smooth=inp.smooth, wcscales=inp.wcscales, bias=inp.bias, device=local)
    xh = [inp.x.pin_memory(), inp.x.roll(1, dims=0).contiguous().pin_memory()]
    yh = [torch.empty((M, N), dtype=shape.dtype).pin_memory() for _ in range(2)]
    e2e_steps = max(10, min(steps, 50))
    for i in range(2):
        plan.forward_host(xh[i % 2], yh[i % 2])
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    # one call at a time: every step's copies and kernels run back to back
    def batches(run_batch, min_s=0.15, at_least=3, at_most=40):
        """median wall time per step over batches of e2e_steps steps (a single 20-step batch lasts
        15 ms: one hiccup of a shared host moved it by a third)"""
        per_step, total = [], 0.0
        while len(per_step) < at_least or (total < min_s and len(per_step) < at_most):
            t0 = time.perf_counter()
            run_batch()
            dt = time.perf_counter() - t0
            per_step.append(dt * 1e3 / e2e_steps)
            total += dt
        per_step.sort()
        return per_step[len(per_step) // 2], len(per_step)

    def sync_batch():
        for i in range(e2e_steps):
            plan.forward_host(xh[i % 2], yh[i % 2])  # returns after y is on the host

    e2e_sync_ms, _ = batches(sync_batch)
    # pipelined calls (two in flight): a step's copies overlap its neighbours' kernels and copies;
    # every step still moves its own x in and its own y out inside the timed region
    if world > 1:
        dist.barrier()
    def pipelined_batch():
        for i in range(e2e_steps):
            plan.submit(xh[i % 2], yh[i % 2])
        plan.wait()

    e2e_ms, e2e_batches = batches(pipelined_batch)
    plan.close()
    # sanity: both paths computed the same thing
    y_dev = lin.step(0)
    torch.cuda.synchronize()
    same = torch.equal(y_dev[:M].cpu(), yh[0])

    t = torch.tensor([ms_per_step, q_us, g_us, e2e_ms, e2e_sync_ms, eager_api_us], dtype=torch.float64, device=dev)
    if world > 1:
        per_rank = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(per_rank, t)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        per_rank = [[round(v, 3) for v in r.tolist()[:3]] for r in per_rank]
    else:
        per_rank = None
    ms_per_step, q_us, g_us, e2e_ms, e2e_sync_ms, eager_api_us = t.tolist()

    # ---- the other benchmark configurations, per kernel (1 GPU) ----
    other = None
    if world == 1 and args.config == "c1" and not args.no_other_configs:
        other = {}
        peaks0 = _peaks()
        lin = g_all = g_q = g_g = None
        for cname in ("c2", "c3", "c4"):
            lin2 = gq = gg = None
            torch.cuda.empty_cache()
            lin2 = DeviceLinear(torch, ops, CONFIGS[cname], dev, 0, nsets=4)
            n_l = 16
            for i in range(3):
                lin2.step(i)
            gq, gg = lin2.capture(lin2.quant, n_l), lin2.capture(lin2.gemm, n_l)
            short = GraphTimer(torch, min(args.min_time, 0.25))
            sampler.mark_begin()
            rq, rg = short.time(gq), short.time(gg)
            sampler.mark_end()
            fig = _kernel_figures(CONFIGS[cname], rq["median_ms"] / n_l * 1e3, rg["median_ms"] / n_l * 1e3, peaks0)
            fig["launches_per_replay"] = n_l
            fig["repeats"] = [rq["repeats"], rg["repeats"]]
            other[cname] = fig
        lin2 = gq = gg = None
        rc, words = _lib.device_status()
        if rc != 0:
            raise SystemExit(f"device status after the other configurations: {words}")

    # ---- tensor-parallel option (N > 1) ----
    tp = None
    if world > 1 and not args.no_tp:
        try:
            tp = _tp_block(torch, dist, ops, dev, rank, world)
        except Exception as e:  # symmetric memory / peer access unavailable: say so, keep the line
            tp = {"error": f"{type(e).__name__}: {e}"[:300]}
    clocks = sampler.stop()

    peaks = _peaks()
    flops = gemm_flops(M_pad, N, K)
    qbytes = quantizer_bytes(M, K, R)
    value = world * flops / (ms_per_step * 1e-3) / 1e12
    e2e_value = world * flops / (e2e_ms * 1e-3) / 1e12
    fig = _kernel_figures(shape, q_us, g_us, peaks)
    g_tflops, q_gbs = fig["gemm_tflops"], fig["quantizer_gbs"]
    h2d, d2h = M * K * 2, M * N * 2
    config = {
        "workload": f"{shape.name}: W4A4 linear M={M} K={K} N={N} R={R} {name}, rows sharded over ranks, weights replicated",
        "per_rank_rows": M,
        "launch": f"one CUDA graph of exactly {steps} steps (quantizer + GEMM each), replayed; median replay / steps",
        "repeats": r_all["repeats"], "timed_region_s": r_all["total_s"],
        "replay_ms": {"median": r_all["median_ms"], "min": r_all["min_ms"], "p90": r_all["p90_ms"]},
        "l2": f"rotating {NSETS} activation/output sets (> 3x L2) between steps",
        "quantizer_us": q_us, "gemm_us": g_us, "kernel_sum_us": q_us + g_us,
        "pct_of_10pf_nominal": fig["pct_of_10pf_nominal"],
        "quantizer_pct_of_8tbs_nominal": fig["quantizer_pct_of_8tbs_nominal"],
        "burst_after_idle": dict(burst, note="the same graphs replayed twice after 0.5 s of idle (min): the clock of a short run, "
                                             "before the power cap lowers it; the headline figures are the sustained ones"),
        "eager_api_us": eager_api_us, "eager_host_issue_us": host_issue_us,
        "eager_api_note": "wall per step of back-to-back Python calls of the two operators (no graphs), outputs reused through out=",
        "ms_per_step_x_sm_mhz": ms_per_step * (clocks.get("sm_mhz") or 0),
    }
    if next_us is not None:
        config["gemm_with_next_layer_quantisation_us"] = next_us
    if per_rank is not None:
        config["per_rank_ms_q_us_g_us"] = per_rank
    if other is not None:
        config["other_configs"] = other
    if tp is not None:
        config["tp"] = tp
    line = {
        "metric": "w4a4_linear_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": config,
        "roofline": {"bound": "tensor", "achieved": g_tflops, "peak": NVFP4_NOMINAL_TFLOPS, "unit": "TFLOP/s",
                     "frac": g_tflops / NVFP4_NOMINAL_TFLOPS,
                     "traffic": NCU_DRAM_BYTES.get(shape.name, {}).get("gemm_w4a4_kernel"),
                     "algorithmic_bytes": M_pad * K // 2 + N * K // 2 + (M_pad + N) * K // 16 + M_pad * N * 2 + (M_pad + N) * R * 2,
                     "kernel": "gemm_w4a4_kernel",
                     "frac_of_4x_measured_bf16_burst": g_tflops / (4.0 * peaks["bf16_tflops"]),
                     "frac_of_measured_bf16_burst": g_tflops / peaks["bf16_tflops"],
                     "peak_note": "nominal dense NVFP4 peak (10 PFLOP/s): no NVFP4 figure is measured on this pool; the "
                                  f"{peaks['source']} bf16 cuBLAS burst is {peaks['bf16_tflops']} TFLOP/s, fractions of it and of "
                                  "4 x it (the nominal nvfp4:bf16 ratio) are given beside"},
        "roofline_quantizer": {"bound": "hbm", "achieved": q_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                               "frac": q_gbs / peaks["hbm_gbs"],
                               "traffic": NCU_DRAM_BYTES.get(shape.name, {}).get("quantize_fused_kernel"),
                               "algorithmic_bytes": qbytes, "kernel": "quantize_fused_kernel",
                               "peak_note": f"{peaks['source']} copy bandwidth"},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": world * h2d,
                "d2h_bytes_per_step": world * d2h, "ms_per_step": e2e_ms, "steps": e2e_steps, "batches": e2e_batches,
                "timing": "wall clock around batches of `steps` pipelined calls, median batch / steps",
                "api": "LinearPlan.submit / wait (svdq_linear_plan_submit, two batches in flight, pinned host buffers)",
                "bound": "host copy (PCIe)", "h2d_gbs_per_gpu": h2d / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_gpu": d2h / (e2e_ms * 1e-3) / 1e9,
                "kernel_share": (q_us + g_us) * 1e-3 / e2e_ms,
                "one_call_at_a_time": {"value": world * flops / (e2e_sync_ms * 1e-3) / 1e12, "ms_per_step": e2e_sync_ms,
                                       "api": "LinearPlan.forward_host"},
                "matches_device_path": bool(same)},
        "gpu_launches": 2 * steps * r_all["repeats"], "launches_per_step": 2,
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(shape, args)
        line["parity"] = line["cpu_baseline"].pop("parity")
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _parity(step, name):
    """The product's two operators on the inputs the CPU oracle has just been timed on, against the
    oracle's outputs of its last pass: codes and scales bit for bit, lora_act and y by relative L2 norm
    (the tolerance of both is 1e-3)."""
    import numpy as np
    import torch
    from oracle import nvfp4_oracle as O
    from svdquant_kernels_b200 import ops
    inp = step.inputs
    o_act, o_asc, o_la, o_ybits, o_y = step.last
    dev = torch.device("cuda", torch.cuda.current_device())
    act, asc, la = ops.quantize_w4a4_act_fuse_lora(inp.x.to(dev), inp.lora_down.to(dev), inp.smooth.to(dev))
    wgt, wsc = ops.quantize_nvfp4_rows(inp.w.to(dev), pad_size=1)
    y = ops.gemm_w4a4(act, wgt, asc, wsc, la, inp.lora_up.to(dev), inp.wcscales.to(dev), inp.bias.to(dev), inp.x.dtype)
    torch.cuda.synchronize()
    y_f32 = y.float().cpu().numpy()
    return {
        "against": "the CPU oracle's outputs on the same inputs (all rows of the cpu_baseline sample)",
        "codes_bit_exact": bool((act.cpu().numpy() == o_act).all()),
        "scales_bit_exact": bool((asc.view(torch.uint8).cpu().numpy() == o_asc).all()),
        "lora_act_rel_l2": O.rel_l2(la.cpu().numpy(), o_la),
        "y_rel_l2": O.rel_l2(y_f32, O.bits_to_f32(o_ybits, name)),
        "y_rel_l2_vs_uncast_fp32": O.rel_l2(y_f32, o_y),
        "tolerance_rel_l2": 1e-3,
    }


def cpu_baseline(shape, args):
    """The oracle on this box's host cores, all rows of the same workload, for about ten seconds; then
    the parity of the product's outputs with the oracle's on those inputs."""
    rows = shape.M if args.cpu_rows <= 0 else min(shape.M, args.cpu_rows)
    step, name = _oracle_step(shape, rows)
    step()
    t0 = time.perf_counter()
    reps = 0
    while reps < 2 or (time.perf_counter() - t0 < 10.0 and reps < 50):
        step()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    m_pad = -(-rows // 256) * 256
    what = f"all {rows} rows" if rows == shape.M else f"the first {rows} of {shape.M} rows"
    out = {"value": 2.0 * m_pad * shape.N * shape.K / dt / 1e12, "unit": "TFLOP/s", "cores": _blas_threads(), "kind": "port",
           "sample": f"{reps} passes over {what} (quantizer + GEMM oracle, numpy/BLAS), {dt:.2f} s each"}
    out["parity"] = _parity(step, name)
    return out


def _claim_stdout():
    """Keep the real stdout for the one JSON line and send everything else that writes to file
    descriptor 1 (library banners such as NCCL's version line, stray prints) to stderr."""
    real = os.fdopen(os.dup(1), "w")
    sys.stdout.flush()
    os.dup2(2, 1)
    sys.stdout = real
    return real


def main():
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c1", help="c1..c4 (benchmark configurations) or s0..s2 (a few hundred rows)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--min-time", type=float, default=0.4, help="seconds of timed graph replays per figure")
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows per pass of the CPU oracle (0 = all rows of the workload)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the per-kernel figures of c2..c4")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel block (N > 1)")
    ap.add_argument("--next-layer", action="store_true", help="with --eager-only: each step also runs the GEMM with the next layer's quantisation in its epilogue")
    ap.add_argument("--eager-only", type=int, default=0, help="after warm-up run this many plain launches of each kernel and exit (for profilers)")
    args = ap.parse_args()
    if args.steps < 1:
        raise SystemExit("--steps must be at least 1")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
