#!/usr/bin/env python
"""Benchmark of the W4A4 linear hot path (quantizer + GEMM) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c1] [--impl ours|reference]

One JSON line on stdout (rank 0).  A step = one pass of the hot path over one
batch: quantize_w4a4_act_fuse_lora followed by gemm_w4a4 on a 4352-row slab.
With N > 1 (torchrun, one rank per GPU) every rank owns its own slab of rows
and a replica of the weights; there is no data-path collective, so the job is
weak-scaled and `value` is the sum over ranks divided by the slowest rank's
time.

`value`  : TFLOP/s of 2*M*N*K (LoRA FLOPs excluded, the reference's convention)
           with inputs resident in HBM.
`e2e`    : the same metric through the host-buffer C-ABI call: pinned host x in,
           pinned host y out, both copies inside the timed region.
`roofline`: the GEMM kernel alone (CUDA events around its launches inside the
           timed loop); `roofline_quantizer`: the quantizer alone, HBM-bound.
`--impl reference` times the CPU oracle (the reference's PyTorch path restated
in numpy; the reference itself is Python and is not shipped to the GPU box).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NSETS = 6  # rotating input/output sets: 6 x ~70 MB is > 3 x the 126 MB L2

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures summarised
# under profiles/ (one launch each, c1).  Output lines are still in L2 when a captured launch ends, so
# the write-back of y / act shows up in later launches, not here.
NCU_DRAM_BYTES = {
    "c1": {"gemm_w4a4_kernel": 18_053_888, "quantize_fused_kernel": 34_494_208},
}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "sustained_mhz": (p.get("clocks_under_load") or {}).get("sm_mhz_median"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "sustained_mhz": 1300.0, "source": "fallback"}


def _tensor_peak(peaks, clocks):
    """bf16 peak to compare against, and a note.  The burst figure belongs to the maximum SM clock, the
    sustained one to the clock the seconds-long loop settled at under the power cap.  A run that the
    power cap held at a clock in between gets the figure interpolated at its own median clock, so that
    a few per cent of clock never swing the denominator by the whole burst-sustained gap."""
    burst, sus = peaks["bf16_tflops"], peaks.get("bf16_tflops_sustained")
    f, fmax, fsus = clocks.get("sm_mhz"), clocks.get("sm_max_mhz"), peaks.get("sustained_mhz")
    capped = "sw_power_cap" in (clocks.get("reasons") or [])
    if not (capped and sus and f and fmax and fsus and fsus < fmax and f < 0.97 * fmax):
        return burst, "burst"
    t = min(1.0, max(0.0, (f - fsus) / (fmax - fsus)))
    peak = sus + (burst - sus) * t
    return peak, f"between sustained ({sus} at {fsus:.0f} MHz) and burst ({burst} at {fmax:.0f} MHz), at this run's {f:.0f} MHz under the power cap"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs.

    NVML is initialised in the constructor (before the timed region); one sample is taken at
    start() and one at stop() so that even a millisecond-long region has samples inside it."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.max_mhz, self.h, self.nv = [], set(), None, None, None
        self._stop_evt = threading.Event()
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
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            r = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            for bit, name in self.names.items():
                if r & bit:
                    self.reasons.add(name)
        except Exception as e:
            self.reasons.add(f"nvml_error:{type(e).__name__}")

    def run(self):
        while not self._stop_evt.is_set():
            self.sample()
            time.sleep(0.002)

    def stop(self):
        self.sample()
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def _np_bits(t):
    import numpy as np
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def run_reference(args):
    """CPU arm: the oracle (numpy restatement of the reference's PyTorch path) on a bounded row sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # all host cores, also under torchrun (which exports OMP_NUM_THREADS=1 to every rank)
    ncpu = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = str(ncpu)
    import numpy as np
    import torch
    torch.set_num_threads(ncpu)
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=ncpu)
    except Exception:
        pass
    from oracle import nvfp4_oracle as O
    from svdquant_kernels_b200.workloads import CONFIGS, SMALL_M, make_inputs
    shape = CONFIGS.get(args.config) or SMALL_M[args.config]
    rows = min(shape.M, args.cpu_rows)
    inp = make_inputs(shape, m_rows=rows)
    name = "fp16" if shape.dtype == torch.float16 else "bf16"
    wgt, wsc = O.quantize_nvfp4_rows(inp.w.numpy(), 1)
    xb, ldb, smb = _np_bits(inp.x), _np_bits(inp.lora_down), _np_bits(inp.smooth)
    lub, wcb, bb = _np_bits(inp.lora_up), _np_bits(inp.wcscales), _np_bits(inp.bias)

    def step():
        act, asc, la = O.quantize_w4a4_act_fuse_lora(xb, ldb, smb, name)
        return O.gemm_w4a4(act, wgt, asc, wsc, la, lub, wcb, bb, name)[0]

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    m_pad = -(-rows // 256) * 256
    tflops = 2.0 * m_pad * shape.N * shape.K / dt / 1e12
    try:
        from threadpoolctl import threadpool_info
        cores = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        cores = os.cpu_count()
    line = {
        "impl": "reference", "metric": "w4a4_linear_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"{shape.name}: W4A4 linear M={shape.M} K={shape.K} N={shape.N} R={shape.R} {name}",
                   "rows_per_step": rows},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"first {rows} of {shape.M} rows per step (quantizer + GEMM oracle, numpy/BLAS)"},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from svdquant_kernels_b200 import _lib, ops
    from svdquant_kernels_b200.workloads import CONFIGS, SMALL_M, gemm_flops, make_inputs, quantizer_bytes

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

    shape = CONFIGS.get(args.config) or SMALL_M[args.config]
    name = "fp16" if shape.dtype == torch.float16 else "bf16"
    # every rank: its own rows, the same weights
    inp = make_inputs(shape, row_offset=rank)
    M, K, N, R = shape.M, shape.K, shape.N, shape.R
    M_pad = -(-M // 256) * 256
    wgt, wsc = ops.quantize_nvfp4_rows(inp.w.to(dev), pad_size=1)
    ops.swizzle_scales(wsc)
    ld, lu = inp.lora_down.to(dev), inp.lora_up.to(dev)
    sm, wc, bias = inp.smooth.to(dev), inp.wcscales.to(dev), inp.bias.to(dev)
    xs = [inp.x.to(dev)]
    for i in range(1, NSETS):
        xs.append(xs[0].roll(i, dims=0).contiguous())

    def quant(i):
        return ops.quantize_w4a4_act_fuse_lora(xs[i % NSETS], ld, sm)

    def gemm(q):
        act, asc, la = q
        return ops.gemm_w4a4(act, wgt, asc, wsc, la, lu, wc, bias, shape.dtype)

    def step(i):
        return gemm(quant(i))

    ys = [None] * NSETS
    for i in range(max(args.warmup, 3)):
        ys[i % NSETS] = step(i)
    torch.cuda.synchronize()
    rc, words = _lib.device_status()
    if rc != 0:
        raise SystemExit(f"device status after warm-up: {words}")

    # Each step is two kernels of ~10-100 us, far shorter than a Python launch, so the launches are
    # captured in CUDA graphs and the timed loops only replay them.  Three graphs over the NSETS
    # rotating buffer sets: all steps in order (quantizer, GEMM, quantizer, GEMM, ...) for the
    # headline, and the NSETS quantizer launches / the NSETS GEMM launches on their own for the
    # per-kernel durations the rooflines use.
    use_graphs = not args.no_graphs
    graph_note = "eager launches"
    if use_graphs:
        try:
            qs = [quant(s_) for s_ in range(NSETS)]          # static inputs of the GEMM-only graph
            torch.cuda.synchronize()
            g_all, g_q, g_g = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            keep = []
            with torch.cuda.graph(g_all):
                for s_ in range(NSETS):
                    keep.append(step(s_))
            with torch.cuda.graph(g_q):
                for s_ in range(NSETS):
                    keep.append(quant(s_))
            with torch.cuda.graph(g_g):
                for s_ in range(NSETS):
                    keep.append(gemm(qs[s_]))
            for g_ in (g_all, g_q, g_g):
                g_.replay()
            torch.cuda.synchronize()
            graph_note = f"CUDA-graph replays ({NSETS} steps per graph)"
        except Exception as e:  # capture refused: fall back to eager launches and say so
            use_graphs = False
            graph_note = f"graph capture failed ({type(e).__name__}: {e}); eager launches"

    last_q = qs if use_graphs else [quant(s_) for s_ in range(NSETS)]
    eager = {"all": step, "q": quant, "g": lambda j: gemm(last_q[j % NSETS])}

    def run_steps(n, which="all"):
        """Queue exactly n steps (which="all") or n launches of one kernel ("q" / "g")."""
        full, rest = divmod(n, NSETS) if use_graphs else (0, n)
        g_ = {"all": g_all, "q": g_q, "g": g_g}[which] if use_graphs else None
        for _ in range(full):
            g_.replay()
        for i in range(rest):          # remainder of a graph (or everything without graphs): eager
            eager[which](i)

    def timed(n, which):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        run_steps(n, which)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    # ---- timed region: K steps, inputs resident in HBM ----
    sampler = ClockSampler(local)
    sampler.start()
    if world > 1:
        dist.barrier()
    total_ms = timed(args.steps, "all")
    sampler.sample()
    q_us = timed(args.steps, "q") / args.steps * 1e3
    g_us = timed(args.steps, "g") / args.steps * 1e3
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    rc, words = _lib.device_status()
    if rc != 0:
        raise SystemExit(f"device status after the timed region: {words}")

    # ---- end to end: host buffers through the C-ABI plan ----
    wgt_h, wsc_h = wgt.cpu(), wsc.view(torch.uint8).cpu()
    plan = ops.LinearPlan(M, K, N, R, shape.dtype, wgt=wgt_h, wscales=wsc_h, lora_down=inp.lora_down,
                          lora_up=inp.lora_up, smooth=inp.smooth, wcscales=inp.wcscales, bias=inp.bias, device=local)
    xh = [inp.x.pin_memory(), inp.x.roll(1, dims=0).contiguous().pin_memory()]
    yh = [torch.empty((M, N), dtype=shape.dtype).pin_memory() for _ in range(2)]
    e2e_steps = max(3, min(args.steps, 50))
    for i in range(2):
        plan.forward_host(xh[i % 2], yh[i % 2])
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    # one call at a time: every step's copies and kernels run back to back
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        plan.forward_host(xh[i % 2], yh[i % 2])      # returns after y is on the host
    e2e_sync_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    # pipelined calls (two in flight): a step's copies overlap its neighbours' kernels and copies;
    # every step still moves its own x in and its own y out inside the timed region
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        plan.submit(xh[i % 2], yh[i % 2])
    plan.wait()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    plan.close()
    # sanity: both paths computed the same thing
    y_dev = step(0)
    torch.cuda.synchronize()
    same = torch.equal(y_dev[:M].cpu(), yh[0])

    t = torch.tensor([total_ms, q_us, g_us, e2e_ms, e2e_sync_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, q_us, g_us, e2e_ms, e2e_sync_ms = t.tolist()

    peaks = _peaks()
    flops = gemm_flops(M_pad, N, K)
    qbytes = quantizer_bytes(M, K, R)
    ms_per_step = total_ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12
    e2e_value = world * flops / (e2e_ms * 1e-3) / 1e12
    g_tflops = flops / (g_us * 1e-6) / 1e12
    q_gbs = qbytes / (q_us * 1e-6) / 1e9
    # tensor peak: the cuBLAS bf16 burst figure, lowered towards the sustained one only as far as the
    # power cap lowered this run's own median SM clock
    bf16_peak, peak_kind = _tensor_peak(peaks, clocks)
    nvfp4_peak = 4.0 * bf16_peak
    line = {
        "metric": "w4a4_linear_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {
            "workload": f"{shape.name}: W4A4 linear M={M} K={K} N={N} R={R} {name}, rows sharded over ranks, weights replicated",
            "per_rank_rows": M, "launch": graph_note, "l2": f"rotating {NSETS} activation/output sets (> 3x L2) between steps",
            "quantizer_us": q_us, "gemm_us": g_us, "pct_of_10pf_nominal": 100.0 * g_tflops / 10000.0,
            "quantizer_pct_of_8tbs_nominal": 100.0 * q_gbs / 8000.0,
        },
        "roofline": {"bound": "tensor", "achieved": g_tflops, "peak": nvfp4_peak, "unit": "TFLOP/s",
                     "frac": g_tflops / nvfp4_peak, "traffic": NCU_DRAM_BYTES.get(shape.name, {}).get("gemm_w4a4_kernel"),
                     "algorithmic_bytes": M_pad * K // 2 + N * K // 2 + (M_pad + N) * K // 16 + M_pad * N * 2 + (M_pad + N) * R * 2,
                     "kernel": "gemm_w4a4_kernel",
                     "peak_note": f"4 x {peaks['source']} bf16 cuBLAS {peak_kind} "
                                  f"({bf16_peak:.1f} TF/s): no NVFP4 figure is measured on this pool; 4 is the nominal nvfp4:bf16 rate ratio"},
        "roofline_quantizer": {"bound": "hbm", "achieved": q_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                               "frac": q_gbs / peaks["hbm_gbs"], "traffic": NCU_DRAM_BYTES.get(shape.name, {}).get("quantize_fused_kernel"),
                               "algorithmic_bytes": qbytes, "kernel": "quantize_fused_kernel",
                               "peak_note": f"{peaks['source']} copy bandwidth"},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": world * M * K * 2,
                "d2h_bytes_per_step": world * M * N * 2, "ms_per_step": e2e_ms, "steps": e2e_steps,
                "api": "LinearPlan.submit / wait (svdq_linear_plan_submit, two batches in flight, pinned host buffers)",
                "one_call_at_a_time": {"value": world * flops / (e2e_sync_ms * 1e-3) / 1e12, "ms_per_step": e2e_sync_ms,
                                       "api": "LinearPlan.forward_host"},
                "matches_device_path": bool(same)},
        "gpu_launches": 2 * args.steps, "kernel_timing_launches": 2 * args.steps,
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(shape, args)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(shape, args):
    """The oracle on this box's host cores, on a bounded sample of the same workload."""
    import torch
    from oracle import nvfp4_oracle as O
    from svdquant_kernels_b200.workloads import make_inputs
    rows = min(shape.M, args.cpu_rows)
    inp = make_inputs(shape, m_rows=rows)
    name = "fp16" if shape.dtype == torch.float16 else "bf16"
    wgt, wsc = O.quantize_nvfp4_rows(inp.w.numpy(), 1)
    t0 = time.perf_counter()
    reps = 0
    while reps < 2 or (time.perf_counter() - t0 < 10.0 and reps < 50):
        act, asc, la = O.quantize_w4a4_act_fuse_lora(_np_bits(inp.x), _np_bits(inp.lora_down), _np_bits(inp.smooth), name)
        O.gemm_w4a4(act, wgt, asc, wsc, la, _np_bits(inp.lora_up), _np_bits(inp.wcscales), _np_bits(inp.bias), name)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    m_pad = -(-rows // 256) * 256
    try:
        from threadpoolctl import threadpool_info
        cores = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        cores = os.cpu_count()
    return {"value": 2.0 * m_pad * shape.N * shape.K / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{reps} passes over the first {rows} of {shape.M} rows (quantizer + GEMM oracle, numpy/BLAS), {dt:.2f} s each"}


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
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c1", help="c1..c4 (benchmark configurations) or s0..s2 (a few hundred rows)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=1024, help="rows per pass of the CPU oracle sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graphs", action="store_true", help="launch eagerly instead of replaying CUDA graphs")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
