#!/usr/bin/env python
"""MoE-FFN benchmark.  python bench.py --gpus N --steps K --warmup W [--impl reference]

A step = one pass of one quantised MoE FFN layer (router top-k -> gather -> gate/up/down expert matmuls -> SwiGLU -> weighted
combine) over one batch of synthetic tokens.

Default workload, at every N: the expert-parallel latent layer (hidden 4096 -> latent 1024, 512 NVFP4 experts, top-10,
intermediate 1024) at 256 tokens IN TOTAL.  Experts are sharded 512/N per GPU, tokens 256/N per GPU; token dispatch and combine
are two equal-split all-to-alls over NCCL (edge0_b200/expert_parallel.py).  Strong scaling: value = 256 tokens / max-over-ranks
step time.  Successive steps rotate over several distinct weight sets so no step finds its weights in L2; a step is replayed
from a CUDA graph (one per weight set) unless --no-graph.

At N = 1 the same line carries, as extras with a roofline object each, the single-GPU configurations: NVFP4 batched decode at
64 / 32 / 8 / 1 tokens, Q3_K one-token decode and the 4096-token NVFP4 prefill.  `--workload c2_nvfp4` makes the 64-token NVFP4
layer the headline instead (N > 1 then runs independent replicas: a throughput figure, not a scaling result).

`--impl reference` times the reference's own ggml CPU backend (oracle/_ref) on the host cores on the same layer and batch.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
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
FP4_VENDOR_TFLOPS = 9000.0      # NVIDIA's dense FP4 figure per GPU (the published 2:4-sparse figure halved)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c5_latent", choices=["c5_latent", "c2_nvfp4"])
    ap.add_argument("--tokens", type=int, default=0, help="batch size per step (default: 256 in total for c5, 64 per GPU for c2)")
    ap.add_argument("--weight-sets", type=int, default=3, help="distinct weight copies rotated over (L2 defeat)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--expert-path", type=int, default=-1, help="expert kernel path of b200moe_set_expert_path (default: the library's / the expert owners' own choice)")
    ap.add_argument("--no-graph", action="store_true", help="launch every step's kernels from the host instead of replaying CUDA graphs")
    return ap.parse_args()


def workload_config(args):
    from edge0_b200 import workloads as W
    cfg = W.CONFIGS[args.workload]
    T = args.tokens or (64 if args.workload == "c2_nvfp4" else 256)
    return cfg, T


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        return {}


def physical_cores() -> int:
    """Physical cores of this host (distinct (package, core) pairs), falling back to the logical count."""
    try:
        pairs, phys, core = set(), None, None
        for line in open("/proc/cpuinfo"):
            if line.startswith("physical id"):
                phys = line.split(":")[1].strip()
            elif line.startswith("core id"):
                core = line.split(":")[1].strip()
            elif not line.strip():
                if phys is not None and core is not None:
                    pairs.add((phys, core))
                phys = core = None
        if pairs:
            return len(pairs)
    except OSError:
        pass
    return os.cpu_count() or 1


# DRAM bytes per algorithmic byte of the gate/up expert kernel, from the ncu capture summarised in profiles/ (627.26 MB / 598.08 MB)
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0488


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (reads only).  One sampler per job
    (rank 0, its own GPU): eight nvidia-smi pollers on one box were measured to slow every rank's kernel launches threefold
    (the queries serialise in the driver), so the other ranks start none."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, enabled: bool = True):
        self.index, self.rows, self.proc, self.enabled = index, [], None, enabled

    def start(self):
        if not self.enabled:
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.enabled:
            return {}
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


# ------------------------------------------------------------------------------------------------ the reference on the host cores

def cpu_reference_run(cfg, T, threads, budget_s, max_passes=50, layer=None):
    """Times the reference's own CPU implementation of the layer (oracle/_ref when it is present, else the plain-C restatement
    on a few tokens) on this host's cores.  Returns a dict with tokens/s from the median pass and the best pass."""
    from edge0_b200 import workloads as W
    from oracle import oracle as O
    have_ref = O.have_reference()
    chk = O.reference() if have_ref else O.restatement()
    threads = threads if have_ref else 1
    T_s = T if have_ref else min(T, 4)
    layer = layer or W.make_layer(cfg)
    x = W.make_tokens(cfg, T_s, bf16=True)
    kw = layer.checker_kwargs()
    t0 = time.time()
    r = chk.moe_layer(x=x, n_threads=threads, repeats=1, **kw)          # first evaluation + one warm-up pass
    per = max(r.ms_median, 1e-3)
    reps = int(max(5, min(max_passes, budget_s * 1e3 / per)))
    r = chk.moe_layer(x=x, n_threads=threads, repeats=reps, **kw)
    return {"value": T_s / (r.ms_median * 1e-3), "value_best_pass": T_s / (r.ms_best * 1e-3), "unit": UNIT, "cores": threads, "kind": chk.kind,
            "ms_median": r.ms_median, "ms_best": r.ms_best, "passes": reps,
            "sample": f"{reps} passes of the same layer at {T_s} tokens on {threads} threads (median {r.ms_median:.2f} ms, best {r.ms_best:.2f} ms), "
                      f"{'ggml CPU backend built for AVX2+FMA' if have_ref else 'scalar restatement'}; set-up {time.time() - t0:.1f}s"}, layer


def run_reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cfg, T = workload_config(args)
    phys = physical_cores()
    main, layer = cpu_reference_run(cfg, T, phys, budget_s=75.0, max_passes=max(50, args.steps if args.steps < 200 else 50))
    dflt, _ = cpu_reference_run(cfg, T, 4, budget_s=30.0, max_passes=50, layer=layer)     # the reference's own default: 4 decode / 4 prefill threads
    main["at_reference_default_threads"] = {k: dflt[k] for k in ("value", "value_best_pass", "cores", "ms_median", "ms_best", "passes")}
    main["host"] = {"logical_cpus": os.cpu_count(), "physical_cores": phys}
    line = {"impl": "reference", "metric": METRIC, "value": main["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": main["passes"], "warmup": 1,
            "ms_per_step": main["ms_median"], "higher_is_better": True, "scaling": "strong" if args.workload == "c5_latent" else "weak",
            "vs_baseline": None, "dtype": "int8 x fp4 integer dots, fp32 accumulate", "data": "synthetic",
            "config": {"workload": workload_name(args, cfg, T), "where": "host CPU cores", "threads": phys},
            "cpu_baseline": main, "e2e": {"value": main["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_name(args, cfg, T):
    return f"{cfg.name} T={T} total" if args.workload == "c5_latent" else f"{cfg.name} T={T} per GPU"


# ------------------------------------------------------------------------------------------------ helpers of the GPU arms

def roll_layer(host, shift):
    """A distinct weight set from the same draws: experts rotated by `shift` (different bytes at every address)."""
    import copy
    h = copy.copy(host)
    for name in ("router_w", "gate", "up", "down", "router_bias", "gate_scale", "up_scale", "down_scale"):
        a = getattr(host, name)
        if a is not None:
            setattr(h, name, np.roll(a, shift, axis=0))
    return h


def finish(world, barrier):
    """End of a multi-rank run: every rank has finished its device work, the line is out.  The process then exits without tearing
    the communicator down: destroying a process group while captured graphs still hold its collectives was seen to block for
    good (the measurement had long been printed)."""
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        barrier()
        os._exit(0)


def make_graph_stepper(eager, n_sets, ctx, use_graphs):
    """eager(i) launches step i.  Returns step(i) that replays one CUDA graph per weight set (the step's launches captured once,
    so the host's launch cost is off the critical path), or eager itself.  The library's calls are plain stream work and capture
    as they are; scratch is sized and kernel attributes are set by the eager passes before."""
    import torch
    if not use_graphs:
        return eager, "eager"
    for i in range(n_sets):
        eager(i)
    ctx.synchronize()
    try:
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
        return (lambda i: gs[i % n_sets].replay()), "CUDA graph replay (one graph per weight set)"
    except Exception as ex:   # capture is an optimisation of the launch path, never a reason to lose the number
        torch.cuda.synchronize()
        return eager, f"eager (graph capture failed: {type(ex).__name__})"


def timed_steps(step, steps, warmup, barrier):
    import torch
    for i in range(warmup):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    barrier()
    return e0.elapsed_time(e1)


def kernel_split(ctx, eager, steps):
    """Per-launch device times of the expert kernels over `steps` eager steps (CUDA events on the launching stream)."""
    ctx.enable_kernel_timing(True)
    ctx.kernel_times()
    for i in range(steps):
        eager(i)
    ctx.synchronize()
    kt = ctx.kernel_times()
    ctx.enable_kernel_timing(False)
    return [(n, ms / max(n, 1) * 1e3) for n, ms in kt]     # (launches, us per launch) for gate/up, down, dense


def fp4_peak(device):
    """Dense FP4 rate of the tensor cores measured with the library's probe (best of two instruction shapes)."""
    from edge0_b200 import capi
    lib = capi.load()
    best, how = 0.0, None
    for n_mma, n_acc in ((256, 1), (232, 2)):
        tf = ctypes.c_double(0.0)
        if lib.b200moe_probe_fp4_rate(device, n_mma, n_acc, 20000, ctypes.byref(tf)) == 0 and tf.value > best:
            best, how = tf.value, f"tcgen05.mma kind::mxf4nvf4 M=128 N={n_mma} K=64, {n_acc} accumulator(s), operands resident in shared memory, every SM"
    return best, how


def single_layer_extras(ctx, dev, args, peak, peaks):
    """The single-GPU configurations with a roofline object each (N = 1 only)."""
    import torch
    from edge0_b200 import moe
    from edge0_b200 import workloads as W
    out = {}
    n_sets = max(1, args.weight_sets)

    def measure(cfg, host, T, steps, bf16, sets):
        layers = [roll_layer(host, 17 * i).to_device(ctx) if i else host.to_device(ctx) for i in range(sets)]
        xs = [torch.from_numpy(W.make_tokens(cfg, T, bf16=bf16, seed_offset=50 + i)).to(dev) for i in range(sets)]
        if bf16:
            xs = [x.to(torch.bfloat16) for x in xs]
        o = torch.empty((T, cfg.n_embd), dtype=torch.float32, device=dev)
        eager = lambda i: layers[i % sets].forward(xs[i % sets], out=o)
        step, how = make_graph_stepper(eager, sets, ctx, not args.no_graph)
        ms = timed_steps(step, steps, 5, torch.cuda.synchronize) / steps
        U = float(np.mean([torch.unique(layers[i].route(xs[i])[0]).numel() for i in range(sets)]))
        ks = kernel_split(ctx, eager, min(steps, 20))
        by = W.algorithmic_bytes(cfg, T, int(round(U)), 2 if bf16 else 4)
        gu_b = U * 2 * cfg.n_ff * moe.row_size(cfg.wtype, cfg.n_in)
        dn_b = U * cfg.n_in * moe.row_size(cfg.wtype, cfg.n_ff)
        r = {"tokens_per_s": T / (ms * 1e-3), "ms_per_step": ms, "experts_touched": U, "launch": how,
             "roofline": {"bound": "hbm", "kernel": "whole step", "algorithmic_bytes": by, "achieved": by / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                          "frac": by / (ms * 1e-3) / 1e9 / peak, "frac_of_8TBs": by / (ms * 1e-3) / 1e9 / 8000.0,
                          "gate_up_kernel": {"avg_launch_us": ks[0][1], "algorithmic_bytes": gu_b, "achieved": gu_b / (ks[0][1] * 1e-6) / 1e9 if ks[0][0] else None,
                                             "frac": gu_b / (ks[0][1] * 1e-6) / 1e9 / peak if ks[0][0] else None},
                          "down_kernel": {"avg_launch_us": ks[1][1], "algorithmic_bytes": dn_b, "achieved": dn_b / (ks[1][1] * 1e-6) / 1e9 if ks[1][0] else None,
                                          "frac": dn_b / (ks[1][1] * 1e-6) / 1e9 / peak if ks[1][0] else None}}}
        del layers
        return r

    try:
        cfg2 = W.CONFIGS["c2_nvfp4"]
        host2 = W.make_layer(cfg2)
        for Tx in (64, 32, 8, 1):
            out[f"c2_nvfp4 T={Tx}"] = measure(cfg2, host2, Tx, args.steps, True, n_sets)
        del host2
    except Exception as ex:
        out["c2_nvfp4"] = {"error": repr(ex)[:300]}
    try:
        cfg1 = W.CONFIGS["c1_q3k"]
        out["c1_q3k T=1"] = measure(cfg1, W.make_layer(cfg1), 1, args.steps, False, n_sets)
    except Exception as ex:
        out["c1_q3k T=1"] = {"error": repr(ex)[:300]}
    try:
        cfg3 = W.CONFIGS["c3_nvfp4_prefill"]
        r = measure(cfg3, W.make_layer(cfg3), 4096, 5, True, 1)
        flop = 2.0 * 4096 * cfg3.top_k * 3 * cfg3.n_embd * cfg3.n_ff
        tf = flop / (r["ms_per_step"] * 1e-3) / 1e12
        bf16_peak = float(peaks.get("bf16_tflops", 1590.0))
        f4, f4_how = fp4_peak(ctx.device)
        r["roofline_tensor"] = {"bound": "tensor", "useful_flop": flop, "achieved": tf, "unit": "TFLOP/s",
                                "peak_bf16_measured": bf16_peak, "frac_of_bf16_measured": tf / bf16_peak,
                                "peak_fp4_measured": f4, "peak_fp4_measured_how": f4_how, "frac_of_fp4_measured": tf / f4 if f4 else None,
                                "peak_fp4_vendor_dense": FP4_VENDOR_TFLOPS, "frac_of_fp4_vendor": tf / FP4_VENDOR_TFLOPS,
                                "engine": "tcgen05 kind::f16 (activations as fp16 hi + lo: 2 x the useful flop issued) + exact re-quantisation fix-up"}
        out["c3_nvfp4_prefill T=4096"] = r
    except Exception as ex:
        out["c3_nvfp4_prefill T=4096"] = {"error": repr(ex)[:300]}
    return out


# ------------------------------------------------------------------------------------------------ default arm: expert-parallel latent layer

def run_c5_arm(args):
    import torch
    import torch.distributed as dist

    from edge0_b200 import moe
    from edge0_b200 import workloads as W
    from edge0_b200.expert_parallel import CudaBackend, ExpertParallelLayer, slot_capacity, token_range

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
    lo, hi = token_range(T, world, rank)
    cap = slot_capacity(T, world, cfg.top_k)
    host = W.make_layer(cfg, expert_range=(rank * per, (rank + 1) * per))
    eps, xs = [], []
    for i in range(n_sets):
        h = roll_layer(host, 17 * i) if i else host           # experts rotated inside the shard, router rotated alike on every rank
        h.expert_lo = host.expert_lo
        b = CudaBackend(ctx, h, rank, world)
        if args.expert_path >= 0:
            ctx.set_expert_path(args.expert_path)
        eps.append(ExpertParallelLayer(b, cfg.n_expert, cfg.top_k, rank, world, capacity=cap))
        x = W.make_tokens(cfg, T, bf16=True, seed_offset=i)[lo:hi]
        xs.append(torch.from_numpy(np.ascontiguousarray(x)).to(dev).to(torch.bfloat16))
    owner_path = 8 if args.expert_path < 0 else args.expert_path
    outs = [None] * n_sets

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

    def eager(i):
        outs[i % n_sets] = eps[i % n_sets].forward(xs[i % n_sets])

    step, how = make_graph_stepper(eager, n_sets, ctx, not args.no_graph)
    sampler = ClockSampler(local, enabled=(rank == 0))
    for i in range(args.warmup):
        step(i)
    ctx.synchronize()
    barrier()
    sampler.start()
    ms_total = max_over_ranks(timed_steps(step, args.steps, 0, barrier))
    ctx.synchronize()
    clocks = sampler.stop()
    step_ms = ms_total / args.steps
    all_ctx = [ctx] + [e.b.ctx_router for e in eps]          # the router runs in a context (and on a stream) of its own
    c0 = sum(c.launches() for c in all_ctx)
    eager(0)
    torch.cuda.synchronize()
    launches = (sum(c.launches() for c in all_ctx) - c0) * args.steps

    # end to end: this rank's tokens start in pinned host memory and the result returns to the host every step
    xh = [x.cpu().pin_memory() for x in xs]
    xd = [torch.empty_like(x) for x in xs]
    oh = torch.empty((hi - lo, cfg.n_embd), dtype=torch.float32).pin_memory()

    def e2e_eager(i):
        j = i % n_sets
        outs[j] = eps[j].forward(xd[j])

    e2e_step, _ = make_graph_stepper(e2e_eager, n_sets, ctx, not args.no_graph)

    def e2e_one(i):
        j = i % n_sets
        xd[j].copy_(xh[j], non_blocking=True)
        e2e_step(i)
        oh.copy_(outs[j], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_ms = max_over_ranks(timed_steps(e2e_one, args.steps, min(args.warmup, 5), barrier))

    # per-phase device times of a few eager steps (rank 0's view; not part of the timed region)
    phases = {}
    n_ph = min(8, max(1, args.steps))
    for i in range(n_ph):
        eps[i % n_sets].enable_phase_timing(True)
        eager(i)
        for k, v in eps[i % n_sets].phase_times_ms().items():
            phases[k] = phases.get(k, 0.0) + v / n_ph
        eps[i % n_sets].enable_phase_timing(False)
    barrier()
    ks = kernel_split(ctx, eager, min(args.steps, 20))
    barrier()

    peaks = measured_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured copy bandwidth (MEASURED_PEAKS.json)" if peaks else "fallback 6650 GB/s"
    ids, _ = eps[0].b.route(xs[0])
    touched = torch.zeros(cfg.n_expert, device=dev)
    touched[ids.reshape(-1).long()] = 1
    if world > 1:
        dist.all_reduce(touched)
    U = int((touched > 0).sum().item())
    U_local = int((touched[rank * per:(rank + 1) * per] > 0).sum().item())
    alg = W.algorithmic_bytes(cfg, T, U, 2)
    gu_b = U_local * 2 * cfg.n_ff * moe.row_size(cfg.wtype, cfg.n_in)
    dn_b = U_local * cfg.n_in * moe.row_size(cfg.wtype, cfg.n_ff)
    gu_us, dn_us = ks[0][1], ks[1][1]

    extras, lib_call = {}, None
    if world == 1 and not args.no_extras:
        # the same layer as ONE library call (no exchange): what a single-GPU caller of b200moe_layer_forward gets
        try:
            if args.expert_path < 0:
                ctx.set_expert_path(0)
            full = [h2.to_device(ctx) for h2 in ([host] + [roll_layer(host, 17 * i) for i in range(1, n_sets)])]
            o = torch.empty((T, cfg.n_embd), dtype=torch.float32, device=dev)
            lib_eager = lambda i: full[i % n_sets].forward(xs[i % n_sets], out=o)
            lstep, lhow = make_graph_stepper(lib_eager, n_sets, ctx, not args.no_graph)
            lms = timed_steps(lstep, args.steps, 5, torch.cuda.synchronize) / args.steps
            lib_call = {"ms_per_step": lms, "tokens_per_s": T / (lms * 1e-3), "launch": lhow,
                        "frac_of_hbm_peak": alg / (lms * 1e-3) / 1e9 / peak}
            del full
        except Exception as ex:
            lib_call = {"error": repr(ex)[:300]}
        torch.cuda.empty_cache()
        extras = single_layer_extras(ctx, dev, args, peak, peaks)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            full_host = host if per == cfg.n_expert else W.make_layer(cfg)
            cpu, _ = cpu_reference_run(cfg, T, physical_cores(), budget_s=20.0, max_passes=30, layer=full_host)
        except Exception as ex:  # the baseline is a report, never a reason to lose the GPU number
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "unavailable", "sample": repr(ex)[:200]}

    if rank == 0:
        line = {"metric": METRIC, "value": T * args.steps / (ms_total * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "fp4 x fp4 block-scaled tensor-core MMA on exact digit planes of the reference's int8 activation grid, fp32 accumulate", "data": "synthetic",
                "config": {"workload": workload_name(args, cfg, T), "n_embd": cfg.n_embd, "n_latent": cfg.n_latent, "n_expert": cfg.n_expert,
                           "top_k": cfg.top_k, "n_ff": cfg.n_ff, "weights": "NVFP4 (ggml block_nvfp4) + fp32 per-expert scale",
                           "activations": "bf16 in, int8 grid of the reference (Q8_0) inside, fp32 out",
                           "parallelism": f"ep{world} (experts {per}/GPU, tokens {T // world}/GPU, two equal-split NCCL all-to-alls of {cap} slots per peer)",
                           "l2": f"{n_sets} distinct weight sets rotated ({n_sets * 906 // world} MB per GPU > 126 MB L2)",
                           "experts_touched_per_step": U, "expert_path": owner_path, "launch": how},
                "e2e": {"value": T * args.steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * cfg.n_embd * 2,
                        "d2h_bytes_per_step": T * cfg.n_embd * 4, "ms_per_step": e2e_ms / args.steps},
                "phases_ms": {k: round(v, 4) for k, v in phases.items()},
                "gpu_launches": launches, "clocks": clocks,
                "roofline": {"bound": "hbm", "kernel": "expert_gemm_fp4_kernel<1024, DUAL> (gate+up+SwiGLU of this rank's experts, tcgen05 kind::mxf4nvf4)",
                             "achieved": gu_b / (gu_us * 1e-6) / 1e9 if gu_us else 0.0, "peak": peak, "unit": "GB/s",
                             "frac": gu_b / (gu_us * 1e-6) / 1e9 / peak if gu_us else 0.0, "traffic": gu_b * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE,
                             "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of this kernel in the ncu capture of the one-GPU step "
                                               "(profiles/expert_gemm_fp4_c5_latent_T256.md: 627.26 MB for 598.08 MB algorithmic), scaled by the "
                                               "experts this rank holds", "peak_source": peak_kind,
                             "algorithmic_bytes_per_launch": gu_b, "avg_launch_us": gu_us, "experts_touched_on_rank0": U_local,
                             "down_kernel": {"achieved": dn_b / (dn_us * 1e-6) / 1e9 if dn_us else 0.0, "avg_launch_us": dn_us,
                                             "algorithmic_bytes_per_launch": dn_b, "frac": dn_b / (dn_us * 1e-6) / 1e9 / peak if dn_us else 0.0},
                             "dense_projections": {"launches_per_step": ks[2][0] / max(1, min(args.steps, 20)), "avg_launch_us": ks[2][1]},
                             "whole_step": {"algorithmic_bytes": alg, "achieved": alg / (step_ms * 1e-3) / 1e9,
                                            "frac_of_aggregate_peak": alg / (step_ms * 1e-3) / 1e9 / (peak * world)}},
                "cpu_baseline": cpu, "library_call_one_gpu": lib_call, "other_configurations": extras}
        print(json.dumps(line))
    finish(world, barrier)


# ------------------------------------------------------------------------------------------------ --workload c2_nvfp4

def run_c2_arm(args):
    """The 64-token NVFP4 batched-decode layer as the headline (one library call per step).  N > 1: independent replicas."""
    import torch
    import torch.distributed as dist

    from edge0_b200 import moe
    from edge0_b200 import workloads as W

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
    if args.expert_path >= 0:
        ctx.set_expert_path(args.expert_path)
    host = W.make_layer(cfg)
    n_sets = max(1, args.weight_sets)
    layers = [roll_layer(host, 17 * i).to_device(ctx) if i else host.to_device(ctx) for i in range(n_sets)]
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

    eager = lambda i: layers[i % n_sets].forward(xs[i % n_sets], out=out)
    step, how = make_graph_stepper(eager, n_sets, ctx, not args.no_graph)
    sampler = ClockSampler(local, enabled=(rank == 0))
    for i in range(args.warmup):
        step(i)
    barrier()
    sampler.start()
    total_ms = max_over_ranks(timed_steps(step, args.steps, 0, barrier))
    clocks = sampler.stop()
    ms_per_step = total_ms / args.steps
    c0 = ctx.launches()
    eager(0)
    ctx.synchronize()
    launches = (ctx.launches() - c0) * args.steps
    host_step = lambda i: layers[i % n_sets].forward_host(xs_pinned[i % n_sets], out=out_pinned)
    e2e_ms = max_over_ranks(timed_steps(host_step, args.steps, min(args.warmup, 5), barrier))
    ks = kernel_split(ctx, eager, min(args.steps, 20))
    U = float(np.mean([torch.unique(layers[i].route(xs[i])[0]).numel() for i in range(n_sets)]))
    ctx.synchronize()
    peaks = measured_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    gu_b = U * 2 * cfg.n_ff * moe.row_size(cfg.wtype, cfg.n_in)
    dn_b = U * cfg.n_in * moe.row_size(cfg.wtype, cfg.n_ff)
    alg = W.algorithmic_bytes(cfg, T, int(round(U)), 2)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cpu, _ = cpu_reference_run(cfg, T, physical_cores(), budget_s=20.0, layer=host)
        except Exception as ex:
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "unavailable", "sample": repr(ex)[:200]}
    if rank == 0:
        line = {"metric": METRIC, "value": world * T * args.steps / (total_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "fp4 x fp4 block-scaled tensor-core MMA on exact digit planes of the reference's int8 activation grid, fp32 accumulate", "data": "synthetic",
                "config": {"workload": workload_name(args, cfg, T), "n_embd": cfg.n_embd, "n_expert": cfg.n_expert, "top_k": cfg.top_k, "n_ff": cfg.n_ff,
                           "weights": "NVFP4 (ggml block_nvfp4) + fp32 per-expert scale", "l2": f"{n_sets} distinct weight sets rotated",
                           "experts_touched_per_step": U, "expert_path": args.expert_path, "launch": how,
                           "parallelism": f"replicas x{world} (independent copies, no collective: not a scaling result)" if world > 1 else "single GPU"},
                "e2e": {"value": world * T * args.steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * cfg.n_embd * 2,
                        "d2h_bytes_per_step": T * cfg.n_embd * 4, "ms_per_step": e2e_ms / args.steps},
                "gpu_launches": launches, "clocks": clocks,
                "roofline": {"bound": "hbm", "kernel": "gate+up+SwiGLU expert kernel of the library's default path", "achieved": gu_b / (ks[0][1] * 1e-6) / 1e9 if ks[0][0] else 0.0,
                             "peak": peak, "unit": "GB/s", "frac": gu_b / (ks[0][1] * 1e-6) / 1e9 / peak if ks[0][0] else 0.0, "traffic": None,
                             "algorithmic_bytes_per_launch": gu_b, "avg_launch_us": ks[0][1],
                             "down_kernel": {"achieved": dn_b / (ks[1][1] * 1e-6) / 1e9 if ks[1][0] else 0.0, "avg_launch_us": ks[1][1], "algorithmic_bytes_per_launch": dn_b},
                             "whole_step": {"algorithmic_bytes": alg, "achieved": alg / (ms_per_step * 1e-3) / 1e9, "frac": alg / (ms_per_step * 1e-3) / 1e9 / peak}},
                "cpu_baseline": cpu}
        print(json.dumps(line))
    finish(world, barrier)


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "c5_latent":
        run_c5_arm(args)
    else:
        run_c2_arm(args)


if __name__ == "__main__":
    main()
