#!/usr/bin/env python
"""Times the reference's own GPU kernels on this box, next to this repository's, on the benchmark
configurations: the Triton quantizer (triton_kernels/quantize_w4a4_act_fuse_lora/kernel.py:289-400)
and the CuTe-DSL GEMM launch_v2 with use_2cta=False (cute_kernels/gemm_w4a4/kernel_v2_fa4.py:113-225;
the 2-CTA form shares one scale tile between the CTAs of a cluster with a broadcast load, a kind of
copy this pool keeps off its GPUs, so it is left alone: its published numbers are quoted instead).  Single GPU only.  Needs baseline/_ref (see
install_reference.sh); without it, or if a kernel fails to compile or run, that is what the line says.

Per configuration and side: kernel-only time (CUDA-graph replays where capture works, else CUDA
events around eager launches) and the eager API-level wall per call (20 warm-up + 500 timed calls
between two events, the reference's own recipe, docs/gpu.md:337-349).

    python baseline/run_reference_kernels.py [--configs c1,c2,c3,c4] > comparators.jsonl
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.path.join(HERE, "_ref")


def eager_wall_us(torch, fn, warm=20, iters=500):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def graph_kernel_us(torch, fns, replays=20):
    """fns: one callable per rotating buffer set; all are captured into one graph."""
    g = torch.cuda.CUDAGraph()
    keep = []
    with torch.cuda.graph(g):
        for f in fns:
            keep.append(f())
    g.replay()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
    ev[0].record()
    for i in range(replays):
        g.replay()
        ev[i + 1].record()
    torch.cuda.synchronize()
    ms = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(replays))
    return ms[len(ms) // 2] / len(fns) * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="c1,c2,c3,c4")
    ap.add_argument("--sets", type=int, default=4)
    args = ap.parse_args()
    sys.path.insert(0, ROOT)
    import torch
    from svdquant_kernels_b200 import ops
    from svdquant_kernels_b200.workloads import CONFIGS, gemm_flops, make_inputs, quantizer_bytes

    have_ref = os.path.isdir(os.path.join(REF, "cute_kernels"))
    if have_ref:
        sys.path.insert(0, REF)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    for cname in args.configs.split(","):
        s = CONFIGS[cname]
        inp = make_inputs(s)
        M_pad = -(-s.M // 256) * 256
        xs = [inp.x.to(dev)] + [inp.x.to(dev).roll(i, 0).contiguous() for i in range(1, args.sets)]
        ld, sm, lu = inp.lora_down.to(dev), inp.smooth.to(dev), inp.lora_up.to(dev)
        wc, bias = inp.wcscales.to(dev), inp.bias.to(dev)
        wgt, wsc = ops.quantize_nvfp4_rows(inp.w.to(dev), pad_size=1)
        qs = [ops.quantize_w4a4_act_fuse_lora(x, ld, sm) for x in xs]
        ys = [ops.gemm_w4a4(q[0], wgt, q[1], wsc, q[2], lu, wc, bias, s.dtype) for q in qs]
        torch.cuda.synchronize()
        rec = {"config": cname, "shape": [s.M, s.K, s.N, s.R], "dtype": str(s.dtype).split(".")[-1],
               "gemm_gflop": gemm_flops(M_pad, s.N, s.K) / 1e9, "quantizer_mbytes": quantizer_bytes(s.M, s.K, s.R) / 1e6}

        # ---- this repository ----
        ours_q = [lambda i=i: ops.quantize_w4a4_act_fuse_lora(xs[i], ld, sm, out=qs[i]) for i in range(args.sets)]
        ours_g = [lambda i=i: ops.gemm_w4a4(qs[i][0], wgt, qs[i][1], wsc, qs[i][2], lu, wc, bias, s.dtype, out=ys[i])
                  for i in range(args.sets)]
        k = [0]

        def rot(fns):
            def f():
                k[0] += 1
                return fns[k[0] % len(fns)]()
            return f
        rec["ours"] = {"quantizer_kernel_us": graph_kernel_us(torch, ours_q), "gemm_kernel_us": graph_kernel_us(torch, ours_g),
                       "quantizer_eager_wall_us": eager_wall_us(torch, rot(ours_q)), "gemm_eager_wall_us": eager_wall_us(torch, rot(ours_g))}

        # ---- the reference ----
        ref = {}
        if not have_ref:
            ref["unavailable"] = "baseline/_ref is missing (run baseline/install_reference.sh where the reference is mounted)"
        else:
            try:
                from triton_kernels.quantize_w4a4_act_fuse_lora.kernel import quantize_w4a4_act_fuse_lora as ref_quant
                rq = [lambda i=i: ref_quant(xs[i], ld, sm, fp4=True) for i in range(args.sets)]
                out = rq[0]()
                torch.cuda.synchronize()
                ref["quantizer_codes_equal_ours"] = bool(torch.equal(out[0], qs[0][0]))
                ref["quantizer_eager_wall_us"] = eager_wall_us(torch, rot(rq))
                try:
                    ref["quantizer_kernel_us"] = graph_kernel_us(torch, rq)
                    ref["quantizer_kernel_note"] = "graph replays of the whole call (its zero-fill of lora_act included)"
                except Exception as e:
                    ref["quantizer_kernel_us"] = None
                    ref["quantizer_kernel_note"] = f"graph capture failed: {type(e).__name__}: {e}"[:200]
            except Exception as e:
                ref["quantizer_error"] = f"{type(e).__name__}: {e}"[:400]
                traceback.print_exc(file=sys.stderr)
            try:
                from cute_kernels.gemm_w4a4.kernel_v2_fa4 import launch_v2
                act, asc, la = qs[0]
                t0 = time.perf_counter()
                tiler = None
                try:
                    y_ref = launch_v2(act, wgt, asc, wsc, la, lu, wc, bias, out_dtype=s.dtype, use_2cta=False)
                except AssertionError as e:
                    # its default 128 x 256 tile does not fit shared memory at this rank: take its small tile
                    ref["gemm_default_tile_error"] = f"{e}"[:200]
                    tiler = (128, 128)
                    y_ref = launch_v2(act, wgt, asc, wsc, la, lu, wc, bias, out_dtype=s.dtype, use_2cta=False, tiler_mn=tiler)
                torch.cuda.synchronize()
                ref["gemm_compile_s"] = time.perf_counter() - t0
                d = (y_ref.float() - ys[0].float())
                ref["gemm_rel_l2_vs_ours"] = float(d.norm() / ys[0].float().norm())
                rg = [lambda i=i: launch_v2(qs[i][0], wgt, qs[i][1], wsc, qs[i][2], lu, wc, bias, out_dtype=s.dtype, use_2cta=False,
                                            tiler_mn=tiler) for i in range(args.sets)]
                ref["gemm_eager_wall_us"] = eager_wall_us(torch, rot(rg))
                ref["gemm_form"] = "launch_v2(use_2cta=False" + (f", tiler_mn={tiler})" if tiler else ")")
                try:
                    ref["gemm_call_graph_us"] = graph_kernel_us(torch, rg)
                    ref["gemm_call_graph_note"] = "graph replays of the whole call: GEMM kernel + its scale repack and cast kernels"
                except Exception as e:
                    ref["gemm_call_graph_us"] = None
                    ref["gemm_call_graph_note"] = f"graph capture failed: {type(e).__name__}: {e}"[:200]
            except Exception as e:
                ref["gemm_error"] = f"{type(e).__name__}: {e}"[:400]
                traceback.print_exc(file=sys.stderr)
        rec["reference"] = ref
        print(json.dumps(rec), flush=True)
        del xs, qs, ys, wgt, wsc
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
