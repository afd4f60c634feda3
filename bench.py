#!/usr/bin/env python
"""Benchmark of the causal-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one forward + backward pass of causal attention over one batch of the
GPT-2-124M-shape workload (bf16 Q/K/V/dO [B=16,H=12,T=1024,D=64] per GPU, dropout off), through
the C ABI of libdadattn.so. Under torchrun every rank (one per GPU) runs the same amount of work
on its own (batch x head) units with no data-path collective (weak scaling); rank 0 prints ONE
JSON line. Extra measurements ride on the same line: the KV-cache decode workload (HBM GB/s),
forward-only and dropout-on figures, the roofline of the dominant kernel, and the CPU baseline.

--impl reference times the reference's own CPU implementation of the path (its host ops driven
in the reference's call order, oracle/_ref; the C restatement if that library is absent) on the
host cores, same metric and workload, each step a bounded sample of (batch x head) units.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "causal_attn_fwd_bwd_tflops"
UNIT = "TFLOP/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# capture summarised in profiles/flash_bf16_fwd_bwd_gpt2_T1024_D64.md.
NCU_TRAFFIC_BYTES = {"flash_bwd_fused_kernel": 210.9e6}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


class ClockSampler:
    """Polls nvidia-smi for SM clocks and throttle reasons while a timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True,
                                     text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7
                          for n, v in zip(names, r[3:7]) if v.lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.rows)}


# ---------------------------------------------------------------------------------------------
# CPU arm
# ---------------------------------------------------------------------------------------------
def cpu_pass(units: int, threads: int):
    """fwd+bwd of `units` (batch x head) units of the GPT-2 shape on the host; returns
    (seconds, kind)."""
    from dadgpt_b200 import workloads as W
    from oracle.oracle import Oracle, RefHost
    shape = W.gpt2(1024)
    rng = np.random.default_rng(shape.seed)
    q, k, v, do = (W.bf16_to_f32(W.bf16_round(
        rng.standard_normal((units, shape.S, shape.D), dtype=np.float32) * np.float32(0.5)))
        for _ in range(4))
    if RefHost.available():
        ref, kind = RefHost(), "reference"
        t0 = time.perf_counter()
        ref.backward(do, q, k, v, shape.scale, threads=threads)  # runs the forward inside
    else:
        ora, kind = Oracle(), "port"
        t0 = time.perf_counter()
        ora.backward(do, q, k, v, shape.scale, threads=threads)
    return time.perf_counter() - t0, kind


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from dadgpt_b200 import workloads as W
    shape = W.gpt2(1024)
    cores = os.cpu_count() or 1
    units = min(shape.BH, cores)  # one unit per core per step keeps a step near one second
    for _ in range(min(args.warmup, 1)):
        cpu_pass(units, cores)
    total, kind = 0.0, "port"
    for _ in range(args.steps):
        dt, kind = cpu_pass(units, cores)
        total += dt
    f, b = W.attn_flops(units, shape.S, shape.D)
    value = (f + b) * args.steps / total / 1e12
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": shape.name, "phase": "fwd+bwd", "dropout": 0.0,
                   "sample": f"{units} of {shape.BH} (batch x head) units per step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"{units} of {shape.BH} units x {args.steps} steps, fwd+bwd"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    import dadgpt_b200 as dad
    from dadgpt_b200 import _lib
    from dadgpt_b200 import workloads as W
    from dadgpt_b200.attention import device_status, flash_backward_bf16_workspace_bytes

    lib = _lib.load()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path for --impl ours")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.decode_only or args.decode_full:
        d = bench_decode(dad, W, dev, world, barrier, max_over_ranks, torch,
                         steps=None if args.decode_full else args.steps,
                         graph=args.decode_full)
        if rank == 0:
            print(json.dumps(d), flush=True)
        return

    if args.large_only:
        def timed_simple(fn, steps, warm):
            for s in range(warm):
                fn(s)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for s in range(steps):
                fn(s)
            e1.record()
            barrier()
            return max_over_ranks(e0.elapsed_time(e1)) / steps
        d = bench_large(dad, W, dev, rank, world, timed_simple, torch,
                        flash_backward_bf16_workspace_bytes, units=args.large_units,
                        steps=args.steps, warm=args.warmup)
        if rank == 0:
            print(json.dumps(d), flush=True)
        return

    shape = W.gpt2(1024)
    BH, S, D, scale = shape.BH, shape.S, shape.D, shape.scale
    unit0 = rank * BH  # weak scaling: every rank owns BH units of a world*BH-unit batch
    n_sets = 4  # rotated so the ~200 MB working set of a step is never L2-resident (126 MB L2)
    K, Wm = args.steps, args.warmup

    # Set 0 is the configured workload (seeds 1 and 2); the other sets have the same shape and
    # distribution from other seeds. Host copies are pinned for the end-to-end leg.
    host, devs = [], []
    for i in range(n_sets):
        if i == 0 and rank == 0:
            arrs = W.qkv(shape) + [W.dout(shape)]
            hs = [torch.from_numpy(a).to(torch.bfloat16) for a in arrs]
        else:
            g = torch.Generator().manual_seed(1000 * rank + i)
            hs = [(torch.randn(BH, S, D, generator=g) * (0.5 if j < 3 else 1.0)).to(torch.bfloat16)
                  for j in range(4)]
        hs = [h.pin_memory() for h in hs]
        host.append(hs)
        devs.append([h.to(dev) for h in hs])
    outs = [dict(out=torch.empty(BH, S, D, dtype=torch.bfloat16, device=dev),
                 lse=torch.empty(BH, S, device=dev),
                 dq=torch.empty(BH, S, D, dtype=torch.bfloat16, device=dev),
                 dk=torch.empty(BH, S, D, dtype=torch.bfloat16, device=dev),
                 dv=torch.empty(BH, S, D, dtype=torch.bfloat16, device=dev)) for _ in range(n_sets)]
    ws = torch.empty(flash_backward_bf16_workspace_bytes(BH, S, D), dtype=torch.uint8, device=dev)
    host_out = {k: torch.empty_like(v, device="cpu").pin_memory() for k, v in outs[0].items()}

    def fwd(i, rate=0.0):
        q, k, v, _ = devs[i]
        o = outs[i]
        dad.gpu_flash_attention_forward_bf16(o["out"], o["lse"], q, k, v, BH, S, D, scale,
                                             rate=rate, seed=42, offset=0, unit0=unit0)

    def bwd(i, rate=0.0):
        q, k, v, do = devs[i]
        o = outs[i]
        dad.gpu_flash_attention_backward_bf16(o["dq"], o["dk"], o["dv"], ws, do, o["out"], o["lse"],
                                              q, k, v, BH, S, D, scale, rate=rate, seed=42, offset=0,
                                              unit0=unit0)

    def timed(fn, steps, warm):
        for s in range(warm):
            fn(s)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(steps):
            fn(s)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / steps  # ms per step, max over ranks

    f_flops, b_flops = W.attn_flops(BH, S, D)
    f_bytes, b_bytes = W.attn_bytes(BH, S, D)

    # ---- headline: fwd + bwd, inputs resident in HBM, with per-kernel stage events ----
    import ctypes
    stage_ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(K)]

    def step_resident(s, record=None):
        i = s % n_sets
        if record is not None:
            record[0].record()
        fwd(i)
        if record is not None:
            arr = (ctypes.c_void_p * 4)(*[e.cuda_event for e in record[1:]])
            lib.dadattn_set_stage_events(arr, 4)
        bwd(i)
        if record is not None:
            lib.dadattn_set_stage_events(None, 0)

    class NoSampler:
        def __enter__(self): return self
        def __exit__(self, *a): pass
        def summary(self): return None

    def measure():
        # only rank 0 polls nvidia-smi (its clocks go into the line); eight pollers on one host
        # would queue on the driver for nothing
        with (ClockSampler(local) if rank == 0 else NoSampler()) as clk:
            for e in (ev for evs in stage_ev for ev in evs):  # create the underlying CUDA events
                e.record()
            torch.cuda.synchronize()
            ctr = {"s": 0}

            def fn(s):
                rec = stage_ev[ctr["s"]] if ctr["armed"] else None
                step_resident(s, rec)
                if ctr["armed"]:
                    ctr["s"] += 1

            # Headline region: exactly K steps, no events between the kernels (an event record in
            # between would serialise the programmatic launch overlap of consecutive kernels).
            ctr["armed"] = False
            for s in range(Wm):
                fn(s)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for s in range(K):
                fn(s)
            e1.record()
            barrier()
            ms = max_over_ranks(e0.elapsed_time(e1)) / K
            # Per-kernel durations: the same K steps once more, with events between the launches.
            ctr["armed"] = True
            for s in range(K):
                fn(s)
            barrier()
            # a longer burst of the same steps only for the clock sampler to see the load
            t_end = time.time() + (0.0 if args.quick else 1.0)
            while time.time() < t_end:
                for s in range(20):
                    step_resident(s)
                torch.cuda.synchronize()
        return ms, clk.summary()

    # A kernel whose bounded device-side wait ran out leaves a status behind and its results are
    # void: such a measurement is thrown away and taken again (all ranks together), at most twice.
    retries, problems = 0, []
    while True:
        ms_step, clocks = measure()
        status = device_status()
        if max_over_ranks(float(status != 0)) == 0.0:
            break
        mine = (f"rank {rank}: " + _lib.load().dadattn_last_error().decode(errors="replace")) if status != 0 else None
        if world > 1:
            everyone = [None] * world
            dist.all_gather_object(everyone, mine)
        else:
            everyone = [mine]
        problems.extend(x for x in everyone if x)
        if retries == 2:
            raise RuntimeError(f"device status {status} after the timed region: {problems}")
        retries += 1
    value = (f_flops + b_flops) * world / (ms_step * 1e-3) / 1e12

    # events: before fwd | before delta + workspace clear | before the fused gradient kernel |
    # before the fp32 -> bf16 pass over dQ | after it
    st = np.array([[evs[j].elapsed_time(evs[j + 1]) for j in range(4)] for evs in stage_ev])
    ms_fwd, ms_prep, ms_fused, ms_conv = (float(x) for x in st.mean(axis=0))
    # The rounding pass is launched programmatically behind the gradient kernel and overlaps its
    # tail, so the event between them does not separate the two cleanly: count them together.
    ms_fused, ms_conv = ms_fused + ms_conv, 0.0
    ms_bwd = ms_prep + ms_fused

    if args.quick:  # profiling aid: only the headline region above, nothing else is launched
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "quick": True,
                              "ms_per_step": ms_step, "steps": K, "warmup": Wm,
                              "kernels_ms": {"fwd": ms_fwd, "bwd_prepare": ms_prep,
                                             "bwd_fused_and_convert": ms_fused}}),
                  flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end: host buffers in, host buffers out, through the same calls ----
    # Every step copies its q, k, v, dO from pinned host memory and reads out, lse, dQ, dK, dV
    # back. The copies run on their own streams, ordered against the compute stream by events,
    # so the upload of step s+1 and the download of step s-1 overlap the kernels of step s (the
    # rotated buffer sets make that legal); all of it lies inside the timed region.
    s_in, s_cmp, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
    ev_in = [torch.cuda.Event() for _ in range(n_sets)]
    ev_done = [torch.cuda.Event() for _ in range(n_sets)]
    ev_out = [torch.cuda.Event() for _ in range(n_sets)]
    used = [False] * n_sets

    def step_e2e(s):
        i = s % n_sets
        with torch.cuda.stream(s_in):
            if used[i]:
                s_in.wait_event(ev_done[i])      # the kernels that read this set have finished
            for d, h in zip(devs[i], host[i]):
                d.copy_(h, non_blocking=True)
            ev_in[i].record(s_in)
        with torch.cuda.stream(s_cmp):
            s_cmp.wait_event(ev_in[i])
            if used[i]:
                s_cmp.wait_event(ev_out[i])      # this set's previous results have been read out
            fwd(i)
            bwd(i)
            ev_done[i].record(s_cmp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[i])
            for k_, v_ in outs[i].items():
                host_out[k_].copy_(v_, non_blocking=True)
            ev_out[i].record(s_out)
        used[i] = True

    def timed_e2e(steps, warm):
        for s in range(warm):
            step_e2e(s)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cur = torch.cuda.current_stream()
        e0.record(cur)
        for st_ in (s_in, s_cmp, s_out):
            st_.wait_event(e0)
        for s in range(steps):
            step_e2e(warm + s)
        for st_ in (s_in, s_cmp, s_out):
            cur.wait_stream(st_)
        e1.record(cur)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / steps

    ms_e2e = timed_e2e(K, Wm)
    h2d = sum(h.numel() * h.element_size() for h in host[0])
    d2h = sum(v.numel() * v.element_size() for v in host_out.values())
    e2e_value = (f_flops + b_flops) * world / (ms_e2e * 1e-3) / 1e12

    # ---- side measurements (not part of `value`) ----
    ms_fwd_only = timed(lambda s: fwd(s % n_sets), K, Wm)
    ms_drop = timed(lambda s: (fwd(s % n_sets, 0.1), bwd(s % n_sets, 0.1)), max(2, K // 4), 1)
    shorter = {}
    for T in (512, 128):
        qs = [[torch.randn(BH, T, D, device=dev).mul_(0.5).to(torch.bfloat16) for _ in range(3)]
              for _ in range(n_sets * (1024 // T))]
        o_ = torch.empty(BH, T, D, dtype=torch.bfloat16, device=dev)
        l_ = torch.empty(BH, T, device=dev)

        def f_(s, qs=qs, T=T):
            q, k, v = qs[s % len(qs)]
            dad.gpu_flash_attention_forward_bf16(o_, l_, q, k, v, BH, T, D, scale)
        ms = timed(f_, K, Wm)
        shorter[f"T{T}"] = {"ms": ms, "tflops": W.attn_flops(BH, T, D)[0] * world / ms / 1e9,
                            "hbm_gbs": W.attn_bytes(BH, T, D)[0] * world / ms / 1e6, "bound": "hbm"}
        del qs

    devs.clear(); outs.clear(); del ws
    torch.cuda.empty_cache()
    large = bench_large(dad, W, dev, rank, world, timed, torch, flash_backward_bf16_workspace_bytes)

    decode = bench_decode(dad, W, dev, world, barrier, max_over_ranks, torch)
    # The headline region was checked (and repeated if need be) above; a device status raised by
    # one of the side measurements voids those only, and is reported instead of ending the run.
    status = device_status()
    side_status = None
    if status != 0:
        side_status = {"code": status, "reason": _lib.load().dadattn_last_error().decode(errors="replace"),
                       "voids": "e2e, fwd_only, dropout_0p1, large_shape, decode of this rank"}

    peaks = load_peaks()
    peak_tf = float(peaks["bf16_tflops"])
    fused_flops = 5.0 * BH * S * S * D  # S, dP, dV, dK, dQ over the causal half, 2 flops per MAC
    roofline = {
        "kernel": "flash_bwd_fused_kernel", "bound": "tensor",
        "achieved": fused_flops / (ms_fused * 1e-3) / 1e12, "peak": peak_tf, "unit": "TFLOP/s",
        "frac": fused_flops / (ms_fused * 1e-3) / 1e12 / peak_tf,
        "peak_source": f"{peaks['_source']} bf16_tflops (burst: the timed region lasts milliseconds)",
        "traffic": NCU_TRAFFIC_BYTES["flash_bwd_fused_kernel"],
        "ms_per_launch": ms_fused,
        "ms_per_launch_includes": "fused_convert_kernel (dQ fp32 -> bf16), which overlaps its tail",
        "other_kernels_ms": {"flash_fwd_bf16_kernel": ms_fwd, "fused_prepare_kernel": ms_prep},
    }

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        units = min(BH, 4 * cores)
        dt, passes, kind = 0.0, 0, "port"
        while dt < 10.0 and passes < 64:  # about 10-20 s of host work
            t, kind = cpu_pass(units, cores)
            dt += t
            passes += 1
        fu, bu = W.attn_flops(units, S, D)
        cpu_baseline = {"value": (fu + bu) * passes / dt / 1e12, "unit": UNIT, "cores": cores,
                        "kind": kind,
                        "sample": f"{passes} passes over {units} of {BH} (batch x head) units, "
                                  f"fwd+bwd, {dt:.1f} s"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": Wm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": shape.name, "phase": "fwd+bwd", "dropout": 0.0,
                       "units_per_gpu": BH, "l2": f"{n_sets} rotated input/output sets (~200 MB each step) > 126 MB L2",
                       "sharding": "independent (batch x head) units per rank, no collective"},
            "clocks": clocks,
            "retries": retries, "retry_reasons": problems, "side_status": side_status,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": 4 * K * world,
            "roofline": roofline,
            "cpu_baseline": cpu_baseline,
            "fwd_only": {"ms": ms_fwd_only, "tflops": f_flops * world / ms_fwd_only / 1e9,
                         "hbm_gbs": f_bytes * world / ms_fwd_only / 1e6, **shorter},
            "bwd_only": {"ms": ms_bwd, "tflops": b_flops / ms_bwd / 1e9},
            "dropout_0p1": {"ms_per_step": ms_drop,
                            "tflops": (f_flops + b_flops) * world / ms_drop / 1e9,
                            "note": "bit-exact Philox mask regenerated in every kernel"},
            "large_shape": large,
            "decode": decode,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def bench_large(dad, W, dev, rank, world, timed, torch, ws_bytes, units=None, steps=5, warm=2):
    """The large configuration (BH=192, T=8192, D=128), the one shape of the set that is firmly
    tensor-bound: forward and backward timed separately, a few steps each (13 ms per step).
    `units` < 192 cuts the (batch x head) axis, for profiler captures."""
    Lg = W.LARGE
    BH = units or Lg.BH
    gen = torch.Generator(device=dev).manual_seed(Lg.seed + rank)
    lq, lk, lv, ldo = ((torch.randn(BH, Lg.S, Lg.D, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
                       for _ in range(4))
    lo, ll = torch.empty_like(lq), torch.empty(BH, Lg.S, device=dev)
    lg = [torch.empty_like(lq) for _ in range(3)]
    lws = torch.empty(ws_bytes(BH, Lg.S, Lg.D), dtype=torch.uint8, device=dev)
    ms_lf = timed(lambda s: dad.gpu_flash_attention_forward_bf16(lo, ll, lq, lk, lv, BH, Lg.S, Lg.D,
                                                                 Lg.scale), steps, warm)
    ms_lb = timed(lambda s: dad.gpu_flash_attention_backward_bf16(*lg, lws, ldo, lo, ll, lq, lk, lv,
                                                                  BH, Lg.S, Lg.D, Lg.scale), steps, warm)
    lf, lb = W.attn_flops(BH, Lg.S, Lg.D)
    peaks = load_peaks()
    sustained = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    large = {"workload": Lg.name, "units_per_gpu": BH, "fwd_ms": ms_lf, "bwd_ms": ms_lb,
             "fwd_tflops": lf * world / ms_lf / 1e9, "bwd_tflops": lb * world / ms_lb / 1e9,
             "fwd_bwd_tflops": (lf + lb) * world / (ms_lf + ms_lb) / 1e9,
             "frac_of_sustained_bf16_peak": (lf + lb) / (ms_lf + ms_lb) / 1e9 / sustained,
             "frac_of_burst_bf16_peak": (lf + lb) / (ms_lf + ms_lb) / 1e9 / float(peaks["bf16_tflops"]),
             "peak_source": peaks["_source"],
             "note": "inputs (1.6 GB at 192 units) far larger than L2; the timed loops last tens of "
                     "milliseconds, hence the sustained peak beside the burst one"}
    del lq, lk, lv, ldo, lo, ll, lg, lws
    torch.cuda.empty_cache()
    return large


def bench_decode(dad, W, dev, world, barrier, max_over_ranks, torch, steps=None, graph=True):
    """KV-cache decode workload: 64 sequences per GPU, 12 layer caches, 256 steps with append;
    one CUDA graph per 12-layer step. Returns achieved HBM GB/s against the algorithmic bytes."""
    cfg = W.DecodeShape()
    if steps is not None:
        cfg = W.DecodeShape(steps=min(steps, cfg.steps))
    lens0 = W.decode_lengths(cfg)
    caches = [dad.KVCacheBF16(cfg.B, cfg.H, cfg.max_len, cfg.D, device=dev) for _ in range(cfg.layers)]
    for c in caches:
        c.k.normal_()
        c.v.normal_()
    gen = torch.Generator(device=dev).manual_seed(cfg.seed)
    q, kn, vn = (torch.randn(cfg.layers, cfg.B, cfg.H, cfg.D, device=dev, generator=gen).to(torch.bfloat16)
                 for _ in range(3))
    out = torch.empty(cfg.layers, cfg.B, cfg.H, cfg.D, dtype=torch.bfloat16, device=dev)
    lens_dev = torch.from_numpy(lens0).to(dev)

    def reset():
        for c in caches:
            c.lengths.copy_(lens_dev)

    def step():
        for l, c in enumerate(caches):
            dad.decode_attention_bf16(out[l], q[l], kn[l], vn[l], c, cfg.scale)

    reset()
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                step()
        torch.cuda.current_stream().wait_stream(side)
        replay = g.replay
    else:
        replay = step
    for _ in range(3):
        replay()
    reset()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(cfg.steps):
        replay()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    total = sum(W.decode_bytes_per_layer_call(lens0 + s + 1, cfg.H, cfg.D)
                for s in range(cfg.steps)) * cfg.layers
    ok = bool((caches[0].lengths.cpu().numpy() == lens0 + cfg.steps).all())
    peaks = load_peaks()
    gbs = total * world / ms / 1e6
    return {"metric": "kv_decode_hbm_gbs", "value": gbs, "unit": "GB/s", "ms_total": ms,
            "steps": cfg.steps, "layers": cfg.layers, "sequences_per_gpu": cfg.B,
            "algorithmic_gb": total / 1e9, "frac_of_hbm_peak": gbs / world / float(peaks["hbm_gbs"]),
            "peak_source": peaks["_source"], "gpu_launches": cfg.layers * cfg.steps,
            "lengths_advanced": ok, "workload": cfg.name}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true",
                    help="only the fwd+bwd timed region (for ncu captures of a small run)")
    ap.add_argument("--decode-only", action="store_true",
                    help="only the KV-cache decode workload (for ncu captures)")
    ap.add_argument("--large-only", action="store_true",
                    help="only the large configuration (T=8192, D=128); --large-units cuts its batch")
    ap.add_argument("--large-units", type=int, default=None)
    ap.add_argument("--decode-full", action="store_true",
                    help="only the KV-cache decode workload, all 256 steps, one CUDA graph per step")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
