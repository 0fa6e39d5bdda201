#!/usr/bin/env python
"""MoE-FFN benchmark.  python bench.py --gpus N --steps K --warmup W [--impl reference]

A step = one pass of one quantised MoE FFN layer (router top-k -> gather -> gate/up/down expert matmuls ->
SwiGLU -> weighted combine) over one batch of synthetic tokens.  Default workload: the NVFP4 batched-decode
configuration (hidden 2048, 128 experts, top-8, intermediate 768) at 64 tokens.  Successive steps rotate over
several distinct weight sets so no step finds its weights in L2.  N > 1: every rank runs the same layer shape on
its own batch (data-parallel replicas, no data-path collective), value = all ranks' tokens / max-over-ranks time.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "moe_ffn_tokens_per_s"
UNIT = "tokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2_nvfp4", choices=["c2_nvfp4", "c5_latent"])
    ap.add_argument("--tokens", type=int, default=0, help="batch size per step (default: 64 for c2, 256 for c5)")
    ap.add_argument("--weight-sets", type=int, default=3, help="distinct weight copies rotated over (L2 defeat)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--overlap", action="store_true", help="programmatic dependent launches between the kernels of a step (library default: off)")
    ap.add_argument("--expert-path", type=int, default=0, help="0 library default, 1 integer (bit-exact) kernels, 2 tcgen05 GEMM, 3 integer gate/up + tcgen05 down, 4 tcgen05 GEMM + exact re-quantisation fix-up")
    ap.add_argument("--no-graph", action="store_true", help="launch every step's kernels from the host instead of replaying CUDA graphs")
    return ap.parse_args()


def workload_config(args):
    from edge0_b200 import workloads as W
    cfg = W.CONFIGS[args.workload]
    T = args.tokens or (64 if args.workload == "c2_nvfp4" else 256)
    return cfg, T


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (reads only)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_reference_run(cfg, T, steps, warmup, budget_s=25.0):
    """Times the reference's own CPU implementation of the layer (oracle/_ref when it is present, else the plain-C
    restatement) on this host's cores.  Returns (tokens/s, info dict)."""
    from edge0_b200 import workloads as W
    from oracle import oracle as O
    have_ref = O.have_reference()
    chk = O.reference() if have_ref else O.restatement()
    cores = (os.cpu_count() or 1) if have_ref else 1
    T_s = T if have_ref else min(T, 4)
    layer = W.make_layer(cfg)
    x = W.make_tokens(cfg, T_s, bf16=True)
    kw = layer.checker_kwargs()
    t0 = time.time()
    r = chk.moe_layer(x=x, n_threads=cores, repeats=max(1, warmup), **kw)   # first evaluation + warm-up repeats
    per = max(r.ms_median, 1e-3)
    reps = int(max(3, min(steps, budget_s * 1e3 / per)))
    r = chk.moe_layer(x=x, n_threads=cores, repeats=reps, **kw)
    tps = T_s / (r.ms_median * 1e-3)
    info = {"value": tps, "unit": UNIT, "cores": cores, "kind": chk.kind,
            "sample": f"{reps} passes of the same layer at {T_s} tokens (median {r.ms_median:.3f} ms, best {r.ms_best:.3f} ms), "
                      f"{'ggml CPU backend built for AVX2+FMA' if have_ref else 'scalar restatement'}; set-up {time.time() - t0:.1f}s"}
    return tps, info, reps, r.ms_median


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg, T = workload_config(args)
    tps, info, reps, ms = cpu_reference_run(cfg, T, args.steps, args.warmup, budget_s=60.0)
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": reps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xfp4 (fp32 accumulate)",
            "data": "synthetic", "config": {"workload": f"{cfg.name} T={T}", "where": "host CPU cores"},
            "cpu_baseline": info, "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def roll_layer(host, shift):
    """A distinct weight set from the same draws: experts rotated by `shift` (different bytes at every address)."""
    import copy
    h = copy.copy(host)
    for name in ("router_w", "gate", "up", "down", "router_bias", "gate_scale", "up_scale", "down_scale"):
        a = getattr(host, name)
        if a is not None:
            setattr(h, name, np.roll(a, shift, axis=0))
    return h


def run_b200_arm(args):
    import torch
    import torch.distributed as dist

    from edge0_b200 import moe
    from edge0_b200 import workloads as W
    from edge0_b200.capi import TYPE_NVFP4

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg, T = workload_config(args)
    ctx = moe.Context(local)
    ctx.set_expert_path(args.expert_path)
    ctx.set_launch_overlap(args.overlap)
    dev = torch.device("cuda", local)

    host = W.make_layer(cfg)
    layers = [roll_layer(host, 17 * i).to_device(ctx) if i else host.to_device(ctx) for i in range(max(1, args.weight_sets))]
    n_sets = len(layers)
    xs_np = [W.make_tokens(cfg, T, bf16=True, seed_offset=1000 * rank + i) for i in range(n_sets)]
    xs = [torch.from_numpy(a).to(dev).to(torch.bfloat16) for a in xs_np]
    xs_pinned = [torch.from_numpy(a).to(torch.bfloat16).pin_memory() for a in xs_np]
    out = torch.empty((T, cfg.n_embd), dtype=torch.float32, device=dev)
    out_pinned = torch.empty((T, cfg.n_embd), dtype=torch.float32).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def make_stepper(x_list, out_t):
        """Returns (step, eager_step).  step replays one CUDA graph per weight set (the step's kernel launches captured
        once, so the host's launch cost is off the critical path) unless --no-graph; the library's calls are plain
        stream work and capture as they are."""
        def eager(i):
            layers[i % n_sets].forward(x_list[i % n_sets], out=out_t)
        if args.no_graph:
            return eager, eager
        for i in range(n_sets):
            eager(i)                        # sizes scratch and sets kernel attributes outside of capture
        ctx.synchronize()
        gs = []
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(n_sets):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    eager(i)
                gs.append(g)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        return (lambda i: gs[i % n_sets].replay()), eager

    step, eager_step = make_stepper(xs, out)
    graphs = not args.no_graph

    # ---- device-resident timing: K steps between two events, barrier + synchronize on both sides
    for i in range(args.warmup):
        step(i)
    ctx.synchronize()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = ctx.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    launches = ctx.launches() - l0
    if graphs:   # replays do not pass through the library's counter: count one eager step and multiply
        c0 = ctx.launches()
        eager_step(0)
        ctx.synchronize()
        launches = (ctx.launches() - c0) * args.steps
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    ctx.synchronize()
    clocks_main = sampler.stop()
    ms_per_step = total_ms / args.steps
    value = world * T * args.steps / (total_ms * 1e-3)

    # ---- end to end through the host entry point: pinned host input, H2D + compute + D2H + wait every step
    for i in range(min(args.warmup, 5)):
        layers[i % n_sets].forward_host(xs_pinned[i % n_sets], out=out_pinned)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(args.steps):
        layers[i % n_sets].forward_host(xs_pinned[i % n_sets], out=out_pinned)
    f1.record()
    barrier()
    e2e_ms = max_over_ranks(f0.elapsed_time(f1))
    e2e = {"value": world * T * args.steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * cfg.n_embd * 2,
           "d2h_bytes_per_step": T * cfg.n_embd * 4, "ms_per_step": e2e_ms / args.steps}

    # ---- per-kernel times of the same steps (CUDA events on the launching stream around each expert-matmul launch)
    ctx.enable_kernel_timing(True)
    ctx.kernel_times()
    for i in range(args.steps):
        eager_step(i)
    ctx.synchronize()
    (n_gu, ms_gu), (n_dn, ms_dn) = ctx.kernel_times()
    ctx.enable_kernel_timing(False)

    # experts actually touched (distinct ids), averaged over the rotated batches
    touched = []
    for i in range(n_sets):
        ids, _ = layers[i].route(xs[i])
        touched.append(int(torch.unique(ids).numel()))
    ctx.synchronize()
    U = float(np.mean(touched))
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured copy bandwidth (MEASURED_PEAKS.json)" if peaks else "fallback 6650 GB/s"
    gu_bytes = U * 2 * cfg.n_ff * moe.row_size(cfg.wtype, cfg.n_in)
    dn_bytes = U * cfg.n_in * moe.row_size(cfg.wtype, cfg.n_ff)
    gu_us = ms_gu / max(n_gu, 1) * 1e3
    dn_us = ms_dn / max(n_dn, 1) * 1e3
    achieved = gu_bytes / (gu_us * 1e-6) / 1e9 if n_gu else 0.0
    # which engine the library's policy picked for gate/up (documented at b200moe_set_expert_path)
    rows = T * cfg.top_k
    can_tc = cfg.wtype == TYPE_NVFP4 and cfg.n_ff % 128 == 0 and cfg.n_in % 128 == 0
    gu_tensor = can_tc and (args.expert_path in (2, 4, 5) or (args.expert_path == 0 and rows >= 2 * cfg.n_expert))
    gu_kernel = ("expert_gemm_nvfp4_kernel<DUAL> (tcgen05 grouped GEMM: gate+up+SwiGLU)" if gu_tensor
                 else "expert_gemv_kernel<DUAL> (integer GEMV: gate+up+SwiGLU)")
    # DRAM traffic of one gate/up launch: dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture of this workload
    # (summary committed under profiles/: 227.29 MB + 5.22 MB with 126 experts touched), scaled by the experts touched here
    traffic, traffic_src = None, None
    if cfg.name == "c2_nvfp4" and T == 64 and gu_tensor:
        traffic = (227.294208e6 + 5.220608e6) * U / 126.0
        traffic_src = "ncu capture of the same workload (summary committed under profiles/), scaled by experts touched"
    roofline = {"bound": "hbm", "kernel": gu_kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_src, "peak_source": peak_kind,
                "algorithmic_bytes_per_launch": gu_bytes,
                "avg_launch_us": gu_us,
                "down_kernel": {"achieved": dn_bytes / (dn_us * 1e-6) / 1e9 if n_dn else 0.0, "avg_launch_us": dn_us,
                                "algorithmic_bytes_per_launch": dn_bytes},
                "whole_step": {"algorithmic_bytes": W.algorithmic_bytes(cfg, T, int(round(U)), 2),
                               "achieved": W.algorithmic_bytes(cfg, T, int(round(U)), 2) / (ms_per_step * 1e-3) / 1e9,
                               "frac": W.algorithmic_bytes(cfg, T, int(round(U)), 2) / (ms_per_step * 1e-3) / 1e9 / peak}}

    extras = {}
    if not args.no_extras and world == 1 and args.workload == "c2_nvfp4":
        for Tx in (1, 8, 32):
            xe = [torch.from_numpy(W.make_tokens(cfg, Tx, bf16=True, seed_offset=50 + i)).to(dev).to(torch.bfloat16) for i in range(n_sets)]
            oe = torch.empty((Tx, cfg.n_embd), dtype=torch.float32, device=dev)
            stepx, _ = make_stepper(xe, oe)
            for i in range(5):
                stepx(i)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(args.steps):
                stepx(i)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / args.steps
            Ux = float(np.mean([torch.unique(layers[i].route(xe[i])[0]).numel() for i in range(n_sets)]))
            by = W.algorithmic_bytes(cfg, Tx, int(round(Ux)), 2)
            extras[f"T={Tx}"] = {"tokens_per_s": Tx / (ms * 1e-3), "ms_per_step": ms, "experts_touched": Ux,
                                 "hbm_gbs": by / (ms * 1e-3) / 1e9, "frac_of_peak": by / (ms * 1e-3) / 1e9 / peak}
        ctx.synchronize()
        # the Q3_K one-token decode configuration (hidden 2048, 128 experts, top-8, intermediate 768), same rotation scheme
        cfg1 = W.CONFIGS["c1_q3k"]
        host1 = W.make_layer(cfg1)
        layers_saved, layers[:] = list(layers), [roll_layer(host1, 17 * i).to_device(ctx) if i else host1.to_device(ctx) for i in range(n_sets)]
        x1 = [torch.from_numpy(W.make_tokens(cfg1, 1, seed_offset=70 + i)).to(dev) for i in range(n_sets)]
        o1 = torch.empty((1, cfg1.n_embd), dtype=torch.float32, device=dev)
        step1, _ = make_stepper(x1, o1)
        for i in range(5):
            step1(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.steps):
            step1(i)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        by = W.algorithmic_bytes(cfg1, 1, cfg1.top_k, 4)
        extras["c1_q3k T=1"] = {"tokens_per_s": 1 / (ms * 1e-3), "ms_per_step": ms, "experts_touched": cfg1.top_k, "algorithmic_bytes": by,
                                "hbm_gbs": by / (ms * 1e-3) / 1e9, "frac_of_peak": by / (ms * 1e-3) / 1e9 / peak}
        layers[:] = layers_saved
        ctx.synchronize()
        # configuration 3: 4096-token prefill with a per-expert logit bias (skewed loads), eager launches, one weight set (340 MB > L2)
        try:
            cfg3 = W.CONFIGS["c3_nvfp4_prefill"]
            l3 = W.make_layer(cfg3).to_device(ctx)
            x3 = torch.from_numpy(W.make_tokens(cfg3, 4096, bf16=True)).to(dev).to(torch.bfloat16)
            o3 = torch.empty((4096, cfg3.n_embd), dtype=torch.float32, device=dev)
            for _ in range(2):
                l3.forward(x3, out=o3)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n3 = 5
            a.record()
            for _ in range(n3):
                l3.forward(x3, out=o3)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / n3
            flop = 2.0 * 4096 * cfg3.top_k * 3 * cfg3.n_embd * cfg3.n_ff
            extras["c3_nvfp4_prefill T=4096"] = {"tokens_per_s": 4096 / (ms * 1e-3), "ms_per_step": ms, "useful_tflops": flop / (ms * 1e-3) / 1e12,
                                                 "engine": "tcgen05 kind::f16 gate/up + exact re-quantisation fix-up, tcgen05 down (library default)"}
            del l3
        except Exception as ex:  # an extra, never a reason to lose the headline number
            extras["c3_nvfp4_prefill T=4096"] = {"error": repr(ex)}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            _, cpu, _, _ = cpu_reference_run(cfg, T, 50, 1, budget_s=20.0)
        except Exception as ex:  # the baseline is a report, never a reason to lose the GPU number
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "unavailable", "sample": repr(ex)[:200]}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": ("fp16 (int8-grid activations as hi+lo, NVFP4 weights exact) on tcgen05, fp32 accumulate" if gu_tensor
                          else "int8 x fp4 integer dots, fp32 accumulate"), "data": "synthetic",
                "config": {"workload": f"{cfg.name} T={T} per GPU", "n_embd": cfg.n_embd, "n_expert": cfg.n_expert, "top_k": cfg.top_k,
                           "n_ff": cfg.n_ff, "n_latent": cfg.n_latent, "weights": "NVFP4 (ggml block_nvfp4) + fp32 per-expert scale",
                           "activations": "bf16 in, int8 grid of the reference (Q8_0) inside, fp32 out",
                           "l2": f"{n_sets} distinct weight sets rotated ({n_sets * layers[0].weight_bytes() / 1e6:.0f} MB > 126 MB L2)",
                           "experts_touched_per_step": U, "expert_path": args.expert_path, "launch": "eager" if args.no_graph else "CUDA graph replay (one graph per weight set)", "parallelism": f"replicas x{world}" if world > 1 else "single GPU"},
                "e2e": e2e, "gpu_launches": launches, "clocks": clocks_main, "roofline": roofline, "cpu_baseline": cpu,
                "other_batch_sizes": extras}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_c5_arm(args):
    """Expert-parallel latent layer (hidden 4096 -> latent 1024, 512 experts, top-10, intermediate 1024), 256 tokens in
    total whatever N is: experts are sharded 512/N per GPU, tokens T/N per GPU, token dispatch and combine are NCCL
    all-to-alls.  Strong scaling: value = 256 tokens / max-over-ranks step time."""
    import torch
    import torch.distributed as dist

    from edge0_b200 import moe
    from edge0_b200 import workloads as W
    from edge0_b200.expert_parallel import CudaBackend, ExpertParallelLayer, token_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg, T = workload_config(args)
    ctx = moe.Context(local)
    per = cfg.n_expert // world
    n_sets = max(1, args.weight_sets)
    eps, xs = [], []
    lo, hi = token_range(T, world, rank)
    for i in range(n_sets):
        host = W.make_layer(cfg, seed_offset=i, expert_range=(rank * per, (rank + 1) * per))
        eps.append(ExpertParallelLayer(CudaBackend(ctx, host, rank, world), cfg.n_expert, cfg.top_k, rank, world))
        x = W.make_tokens(cfg, T, bf16=True, seed_offset=i)[lo:hi]
        xs.append(torch.from_numpy(np.ascontiguousarray(x)).to(dev))
        del host

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(i):
        return eps[i % n_sets].forward(xs[i % n_sets])

    for i in range(args.warmup):
        step(i)
    ctx.synchronize()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = ctx.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    launches = ctx.launches() - l0
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ctx.synchronize()
    clocks = sampler.stop()
    # end to end: this rank's tokens start in pinned host memory and the result returns to the host every step
    xh = [x.cpu().pin_memory() for x in xs]
    oh = torch.empty((hi - lo, cfg.n_embd), dtype=torch.float32).pin_memory()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(args.steps):
        xd = xh[i % n_sets].to(dev, non_blocking=True)
        oh.copy_(eps[i % n_sets].forward(xd), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    if world > 1:
        t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    # per-phase device times of a few more steps (rank 0's view; not part of the timed region)
    phases = {}
    n_ph = min(8, max(1, args.steps))
    for i in range(n_ph):
        eps[i % n_sets].enable_phase_timing(True)
        step(i)
        for k, v in eps[i % n_sets].phase_times_ms().items():
            phases[k] = phases.get(k, 0.0) + v / n_ph
        eps[i % n_sets].enable_phase_timing(False)
    barrier()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    ids, _ = eps[0].b.route(xs[0])
    touched = torch.zeros(cfg.n_expert, device=dev)
    touched[ids.reshape(-1).long()] = 1
    if world > 1:
        dist.all_reduce(touched)
    U = int((touched > 0).sum().item())
    alg = W.algorithmic_bytes(cfg, T, U, 4)
    step_ms = ms / args.steps
    if rank == 0:
        line = {"metric": METRIC, "value": T * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int8-grid activations x NVFP4 weights (integer dots or fp16 hi+lo on tcgen05 by the library's policy), fp32 accumulate", "data": "synthetic",
                "config": {"workload": f"{cfg.name} T={T} total", "n_embd": cfg.n_embd, "n_latent": cfg.n_latent, "n_expert": cfg.n_expert,
                           "top_k": cfg.top_k, "n_ff": cfg.n_ff, "parallelism": f"ep{world} (experts {per}/GPU, tokens {T // world}/GPU, NCCL all-to-all dispatch+combine)",
                           "l2": f"{n_sets} distinct weight sets rotated", "experts_touched_per_step": U, "expert_path": args.expert_path, "launch": "eager"},
                "e2e": {"value": T * args.steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * cfg.n_embd * 4,
                        "d2h_bytes_per_step": T * cfg.n_embd * 4, "ms_per_step": e2e_ms / args.steps},
                "phases_ms": {k: round(v, 4) for k, v in phases.items()},
                "gpu_launches": launches, "clocks": clocks,
                "roofline": {"bound": "hbm", "kernel": "whole step (all ranks)", "achieved": alg / (step_ms * 1e-3) / 1e9, "peak": peak * world, "unit": "GB/s",
                             "frac": alg / (step_ms * 1e-3) / 1e9 / (peak * world), "traffic": None, "algorithmic_bytes_per_step": alg,
                             "peak_source": "measured copy bandwidth x N"},
                "cpu_baseline": None}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "c5_latent":
        run_c5_arm(args)
    else:
        run_b200_arm(args)


if __name__ == "__main__":
    main()
