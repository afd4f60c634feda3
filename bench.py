#!/usr/bin/env python
"""Benchmark of the causal-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one forward + backward pass of causal attention over one batch of the
GPT-2-124M-shape workload (bf16 Q/K/V/dO [B=16,H=12,T=1024,D=64] per GPU, dropout off), through
the C ABI of libdadattn.so. Under torchrun every rank (one per GPU) runs the same amount of work
on its own (batch x head) units with no data-path collective (weak scaling); rank 0 prints ONE
JSON line. Extra measurements ride on the same line: the KV-cache decode workload (HBM GB/s),
forward-only and dropout-on figures, the roofline of the dominant kernel, the CPU baseline, and
for N > 1 a `strong` object: the large configuration and the decode workload SHARDED over the
ranks (fixed total work), with the results all-gathered over NCCL after the timed region and
checked on rank 0. After its timed regions (never inside them) the run checks what it timed
against the CPU oracle and reports that as `verify`.

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
NCU_TRAFFIC_BYTES = {"flash_bwd_fused_kernel": 206.1e6}


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
# Verification helpers (run after the timed regions; the oracle is only ever the checker)
# ---------------------------------------------------------------------------------------------
def _rel_l2(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    if np.abs(got - want).max() < 1e-6:
        return 0.0
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


TOL = {"out_max_abs": 2e-2, "lse_max_abs": 1e-2, "grad_rel_l2": 3e-2}  # BASELINE.json's bars


def check_units_against_oracle(q, k, v, do, got, scale, rate=0.0, unit0=0):
    """q, k, v, do: fp32 host arrays [n,S,D] (the bf16 values upcast); got: dict of host arrays
    out, lse, dq, dk, dv computed by the CUDA kernels. The C oracle recomputes all of it."""
    from oracle.oracle import Oracle
    ora = Oracle()
    o_ref, lse_ref = ora.forward(q, k, v, scale, rate=rate, seed=42, offset=0, unit0=unit0)
    g_ref = ora.backward(do, q, k, v, scale, rate=rate, seed=42, offset=0, unit0=unit0)
    r = {"out_max_abs": float(np.abs(got["out"] - o_ref).max()),
         "lse_max_abs": float(np.abs(got["lse"] - lse_ref).max()),
         "grad_rel_l2": max(_rel_l2(got[n], w) for n, w in zip(("dq", "dk", "dv"), g_ref))}
    r["ok"] = all(r[k_] <= TOL[k_] for k_ in TOL)
    return r


def check_unit_against_numpy(q, k, v, do, got, scale):
    """One whole unit of the large shape against oracle/rowcheck.py (blockwise float64)."""
    from oracle.rowcheck import attention_unit
    o, lse, dq, dk, dv = attention_unit(q, k, v, do, scale)
    r = {"out_max_abs": float(np.abs(got["out"] - o).max()),
         "lse_max_abs": float(np.abs(got["lse"] - lse).max()),
         "grad_rel_l2": max(_rel_l2(got[n], w) for n, w in (("dq", dq), ("dk", dk), ("dv", dv)))}
    r["ok"] = all(r[k_] <= TOL[k_] for k_ in TOL)
    return r


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
class Ctx:
    """What every leg of the GPU arm needs: device, rank layout, barrier and max-over-ranks."""

    def __init__(self, torch, dist, dev, rank, world):
        self.torch, self.dist, self.dev, self.rank, self.world = torch, dist, dev, rank, world

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_ok(self, ok: bool) -> bool:
        return self.max_over_ranks(0.0 if ok else 1.0) == 0.0

    def timed(self, fn, steps, warm):
        """ms per step: `warm` untimed steps, then `steps` steps between CUDA events on the
        launching stream, barrier + synchronize on both sides, max over ranks."""
        torch = self.torch
        for s in range(warm):
            fn(s)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(steps):
            fn(s)
        e1.record()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1)) / steps


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
    cx = Ctx(torch, dist, dev, rank, world)
    barrier, max_over_ranks, timed = cx.barrier, cx.max_over_ranks, cx.timed

    if args.decode_only or args.decode_full:
        d = bench_decode(cx, dad, W, steps=None if args.decode_full else args.steps,
                         graph=args.decode_full, verify=False)
        if rank == 0:
            print(json.dumps(d), flush=True)
        return

    if args.large_only:
        d = bench_large(cx, dad, W, flash_backward_bf16_workspace_bytes, units=args.large_units,
                        steps=args.steps, warm=args.warmup, verify=False)
        if rank == 0:
            print(json.dumps(d), flush=True)
        return

    shape = W.gpt2(1024)
    BH, S, D, scale = shape.BH, shape.S, shape.D, shape.scale
    unit0 = rank * BH  # weak scaling: every rank owns BH units of a world*BH-unit batch
    n_sets = 4  # rotated so the ~200 MB working set of a step is never L2-resident (126 MB L2)
    K, Wm = args.steps, args.warmup

    # Set 0 is the configured workload (seeds 1 and 2) on rank 0; the other sets have the same
    # shape and distribution from other seeds. Host copies are pinned for the end-to-end leg.
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

    f_flops, b_flops = W.attn_flops(BH, S, D)
    f_bytes, b_bytes = W.attn_bytes(BH, S, D)

    # ---- headline: fwd + bwd, inputs resident in HBM, with per-kernel stage events ----
    import ctypes
    n_stage = BWD_LAUNCHES + 2  # one event before each kernel of the step and one after the last
    stage_ev = [[torch.cuda.Event(enable_timing=True) for _ in range(n_stage)] for _ in range(K)]

    def step_resident(s, record=None):
        i = s % n_sets
        if record is not None:
            record[0].record()
        fwd(i)
        if record is not None:
            arr = (ctypes.c_void_p * (n_stage - 1))(*[e.cuda_event for e in record[1:]])
            lib.dadattn_set_stage_events(arr, n_stage - 1)
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
            # Headline region: exactly K steps between two events, no events between the kernels
            # (an event record in between would serialise the programmatic launch overlap of
            # consecutive kernels). The region is taken `repeats` times; the median is reported.
            for s in range(Wm):
                step_resident(s)
            regions = []
            for _ in range(max(1, args.repeats)):
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for s in range(K):
                    step_resident(s)
                e1.record()
                barrier()
                regions.append(max_over_ranks(e0.elapsed_time(e1)) / K)
            # Per-kernel durations: the same K steps once more, with events between the launches.
            for s in range(K):
                step_resident(s, stage_ev[s])
            barrier()
            # a longer burst of the same steps only for the clock sampler to see the load
            t_end = time.time() + (0.0 if args.quick else 1.0)
            while time.time() < t_end:
                for s in range(20):
                    step_resident(s)
                torch.cuda.synchronize()
        return regions, clk.summary()

    # A kernel whose bounded device-side wait ran out leaves a status behind and its results are
    # void: such a measurement is thrown away and taken again (all ranks together), at most twice.
    retries, problems = 0, []
    while True:
        regions, clocks = measure()
        status = device_status()
        if max_over_ranks(float(status != 0)) == 0.0:
            break
        mine = (f"rank {rank}: " + lib.dadattn_last_error().decode(errors="replace")) if status != 0 else None
        if world > 1:
            everyone = [None] * world
            dist.all_gather_object(everyone, mine)
        else:
            everyone = [mine]
        problems.extend(x for x in everyone if x)
        if retries == 2:
            raise RuntimeError(f"device status {status} after the timed region: {problems}")
        retries += 1
    ms_step = float(np.median(regions))
    value = (f_flops + b_flops) * world / (ms_step * 1e-3) / 1e12

    # events: before fwd | before each kernel of the backward | after the last one
    st = np.array([[evs[j].elapsed_time(evs[j + 1]) for j in range(n_stage - 1)] for evs in stage_ev])
    stage_ms = [float(x) for x in st.mean(axis=0)]
    ms_fwd, ms_prep = stage_ms[0], stage_ms[1]
    # Kernels launched programmatically behind the gradient kernel overlap its tail, so the
    # event between them does not separate them cleanly: they are counted together.
    ms_fused = float(sum(stage_ms[2:]))
    ms_bwd = ms_prep + ms_fused

    if args.quick:  # profiling aid: only the headline region above, nothing else is launched
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "quick": True,
                              "ms_per_step": ms_step, "steps": K, "warmup": Wm,
                              "kernels_ms": {"fwd": ms_fwd, "bwd_prepare": ms_prep,
                                             "bwd_fused": ms_fused}}),
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

    # ---- side measurements (not part of `value`; every figure below is PER GPU) ----
    ms_fwd_only = timed(lambda s: fwd(s % n_sets), K, Wm)
    # Dropout p = 0.1 (Philox seed 42, offset 0): a step draws the bit-packed mask ONCE
    # (dadattn_dropout_mask_bits), then forward and backward read it. The mask kernel is inside
    # the timed step; its own duration is measured separately as well. For comparison, the same
    # step with every kernel drawing the mask itself (dadattn_flash_*_bf16 with rate > 0).
    drop_steps = max(4, K // 2)
    bits = dad.dropout_mask_bits(BH, S, 0.1, 42, 0, unit0)

    def drop_step(s):
        i = s % n_sets
        q, k, v, do = devs[i]
        o = outs[i]
        dad.dropout_mask_bits(BH, S, 0.1, 42, 0, unit0, out=bits)
        dad.gpu_flash_attention_forward_bf16(o["out"], o["lse"], q, k, v, BH, S, D, scale, rate=0.1,
                                             mask_bits=bits)
        dad.gpu_flash_attention_backward_bf16(o["dq"], o["dk"], o["dv"], ws, do, o["out"], o["lse"], q, k, v,
                                              BH, S, D, scale, rate=0.1, mask_bits=bits)
    ms_drop = timed(drop_step, drop_steps, 2)

    ms_mask = timed(lambda s: dad.dropout_mask_bits(BH, S, 0.1, 42, 0, unit0, out=bits), drop_steps, 2)
    ms_drop_inkernel = timed(lambda s: (fwd(s % n_sets, 0.1), bwd(s % n_sets, 0.1)), max(2, K // 4), 1)
    mask_bytes = int(bits.numel() * 4)
    shorter = {}
    for T in (512, 128):
        qs = [[torch.randn(BH, T, D, device=dev).mul_(0.5).to(torch.bfloat16) for _ in range(3)]
              for _ in range(n_sets * (1024 // T))]
        o_ = torch.empty(BH, T, D, dtype=torch.bfloat16, device=dev)
        l_ = torch.empty(BH, T, device=dev)

        def f_(s, qs=qs, T=T):
            q, k, v = qs[s % len(qs)]
            dad.gpu_flash_attention_forward_bf16(o_, l_, q, k, v, BH, T, D, scale)
        ms_direct = timed(f_, K, Wm)
        # These launches are short enough for the host's launch path (Python, ctypes, three tensor
        # map encodes) to show in a loop of direct calls, so the figure is taken from a CUDA graph
        # of one launch per input set, as a caller with a launch-bound shape would run it; the
        # direct-call figure is kept beside it.
        side_ = torch.cuda.Stream()
        side_.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side_):
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_, stream=side_):
                for s_ in range(len(qs)):
                    f_(s_)
        torch.cuda.current_stream().wait_stream(side_)
        ms = timed(lambda s: g_.replay(), max(4, K // 2), 2) / len(qs)
        peaks_ = load_peaks()
        shorter[f"T{T}"] = {"ms": ms, "ms_direct_calls": ms_direct, "timed_as": f"graph of {len(qs)} launches",
                            "tflops": W.attn_flops(BH, T, D)[0] / ms / 1e9,
                            "hbm_gbs": W.attn_bytes(BH, T, D)[0] / ms / 1e6, "bound": "hbm",
                            "frac_of_hbm_peak": W.attn_bytes(BH, T, D)[0] / ms / 1e6 / float(peaks_["hbm_gbs"])}
        del g_, qs

    # The same step on the activations as the projections leave them, [B*S, H*D] (no head split /
    # merge copies), next to what those eight copies per layer cost when done separately
    # (3 splits + 1 merge around the forward, 1 split + 3 merges around the backward).
    Bb, Hh = 16, BH // 16
    il = [t.view(Bb, Hh, S, D).permute(0, 2, 1, 3).reshape(Bb * S, Hh * D).contiguous() for t in devs[0]]
    il_out = {n: torch.empty_like(il[0]) for n in ("out", "dq", "dk", "dv")}
    il_lse = torch.empty(BH, S, device=dev)

    def il_step(s):
        dad.gpu_flash_attention_forward_bf16_interleaved(il_out["out"], il_lse, il[0], il[1], il[2], Bb, Hh, S, D, scale)
        dad.gpu_flash_attention_backward_bf16_interleaved(il_out["dq"], il_out["dk"], il_out["dv"], ws, il[3],
                                                          il_out["out"], il_lse, il[0], il[1], il[2], Bb, Hh, S, D, scale)
    ms_il = timed(il_step, K, Wm)
    tmp = torch.empty(BH, S, D, dtype=torch.bfloat16, device=dev)

    def copies(s):
        for _ in range(4):   # splits: [B*S, H*D] -> [B*H, S, D]
            tmp.view(Bb, Hh, S, D).copy_(il[0].view(Bb, S, Hh, D).permute(0, 2, 1, 3))
        for _ in range(4):   # merges: back
            il_out["out"].view(Bb, S, Hh, D).copy_(tmp.view(Bb, Hh, S, D).permute(0, 2, 1, 3))
    ms_copies = timed(copies, K, Wm)
    interleaved = {"ms_per_step": ms_il, "tflops": (f_flops + b_flops) / ms_il / 1e9,
                   "split_merge_copies_ms": ms_copies,
                   "note": "q, k, v, dO, out, dQ, dK, dV all [B*S, H*D]; the 8 head split / merge copies per "
                           "layer of the reference (timed here as torch strided copies) are not needed"}
    del il, il_out, tmp

    # ---- verification of what was timed (rank 0 holds the configured seeds in set 0) ----
    verify = None
    pick = [0, BH // 2 - 1, BH - 1]

    def gather_set0(rate):
        fwd(0, rate)
        bwd(0, rate)
        torch.cuda.synchronize()
        got = {n: outs[0][n][pick].float().cpu().numpy() for n in ("out", "lse", "dq", "dk", "dv")}
        ins = [h[pick].float().numpy() for h in host[0]]
        return ins, got

    if not args.no_verify:
        if rank == 0:
            ins, got = gather_set0(0.0)
            verify = {"gpt2_fwd_bwd": check_units_against_oracle(*ins, got, scale)}
            # dropout on: unit 0 of this rank (global unit index unit0 + 0), seed 42, offset 0
            drop_step(0)
            torch.cuda.synchronize()
            got = {n: outs[0][n][:1].float().cpu().numpy() for n in ("out", "lse", "dq", "dk", "dv")}
            ins = [h[:1].float().numpy() for h in host[0]]
            verify["gpt2_dropout_0p1"] = check_units_against_oracle(*ins, got, scale, rate=0.1,
                                                                    unit0=unit0)
            verify["units_checked"] = pick
            verify["tolerances"] = TOL
        barrier()

    devs.clear(); outs.clear(); del ws, bits
    torch.cuda.empty_cache()
    large = bench_large(cx, dad, W, flash_backward_bf16_workspace_bytes, verify=not args.no_verify)
    decode = bench_decode(cx, dad, W, verify=not args.no_verify)
    strong = None
    if world > 1:
        strong = bench_strong(cx, dad, W, flash_backward_bf16_workspace_bytes, large, decode,
                              verify=not args.no_verify)
    if verify is not None:
        verify["large_shape"] = large.pop("verify", None)
        verify["decode"] = decode.pop("verify", None)
        if strong is not None:
            verify["strong"] = strong["ok"]
        verify["ok"] = all(v["ok"] for v in verify.values() if isinstance(v, dict) and "ok" in v) \
            and verify.get("strong", True)
    # The headline region was checked (and repeated if need be) above; a device status raised by
    # one of the side measurements voids those only, and is reported instead of ending the run.
    status = device_status()
    side_status = None
    if status != 0:
        side_status = {"code": status, "reason": lib.dadattn_last_error().decode(errors="replace"),
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
        "ms_per_launch_includes": BWD_TAIL_NOTE,
        "other_kernels_ms": {"flash_fwd64_kernel": ms_fwd, "fused_prepare_kernel": ms_prep},
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
        mhz = (clocks or {}).get("sm_mhz")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": Wm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": shape.name, "phase": "fwd+bwd", "dropout": 0.0,
                       "units_per_gpu": BH, "l2": f"{n_sets} rotated input/output sets (~200 MB each step) > 126 MB L2",
                       "sharding": "independent (batch x head) units per rank, no collective"},
            "timed_regions": {"n": len(regions), "steps_each": K, "ms_per_step_median": ms_step,
                              "ms_per_step_min": float(min(regions)), "ms_per_step_max": float(max(regions)),
                              "ms_x_sm_mhz": ms_step * mhz if mhz else None},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": (1 + BWD_LAUNCHES) * K * world,
            "roofline": roofline,
            "cpu_baseline": cpu_baseline,
            "side_figures": "per GPU (value, e2e and strong are whole-job)",
            "fwd_only": {"ms": ms_fwd_only, "tflops": f_flops / ms_fwd_only / 1e9,
                         "frac_of_burst_bf16_peak": f_flops / ms_fwd_only / 1e9 / peak_tf,
                         "hbm_gbs": f_bytes / ms_fwd_only / 1e6, **shorter},
            "bwd_only": {"ms": ms_bwd, "tflops": b_flops / ms_bwd / 1e9,
                         "frac_of_burst_bf16_peak": b_flops / ms_bwd / 1e9 / peak_tf},
            "dropout_0p1": {"ms_per_step": ms_drop, "vs_dropout_off": ms_drop / ms_step,
                            "tflops": (f_flops + b_flops) / ms_drop / 1e9,
                            "mask_kernel_ms": ms_mask, "mask_bytes": mask_bytes,
                            "ms_per_step_mask_drawn_in_every_kernel": ms_drop_inkernel,
                            "note": DROPOUT_NOTE},
            "interleaved_layout": interleaved,
            "large_shape": large,
            "decode": decode,
            "strong": strong,
            "verify": verify,
            "retries": retries, "retry_reasons": problems, "side_status": side_status,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# How many kernels one dadattn_flash_bwd_bf16 call launches at head size 64 (delta + workspace
# clear, the fused gradient kernel, dQ fp32 -> bf16), what the roofline duration includes, and
# how the dropout figure is produced.
BWD_LAUNCHES = 3
BWD_TAIL_NOTE = "fused_convert_kernel (dQ fp32 -> bf16), which overlaps its tail"
DROPOUT_NOTE = ("bit-exact Philox mask drawn once per step into a bit-packed lower-triangle buffer "
                "(inside the timed step), read by forward and backward")


def large_inputs(torch, dev, Lg, unit_ids):
    """q, k, v, dO of the large configuration for the given global unit indices, bf16 on the
    device. Unit u is drawn from its own generator (seed 1000003 * seed + u), 0.5 N(0,1), so a
    unit's data does not depend on how many ranks share the batch."""
    q, k, v, do = (torch.empty(len(unit_ids), Lg.S, Lg.D, dtype=torch.bfloat16, device=dev)
                   for _ in range(4))
    gen = torch.Generator(device=dev)
    for i, u in enumerate(unit_ids):
        gen.manual_seed(1000003 * Lg.seed + int(u))
        x = torch.randn(4, Lg.S, Lg.D, device=dev, generator=gen) * 0.5
        q[i], k[i], v[i], do[i] = x[0], x[1], x[2], x[3]
    return q, k, v, do


def bench_large(cx, dad, W, ws_bytes, units=None, steps=5, warm=3, verify=True, unit_ids=None):
    """The large configuration (BH=192, T=8192, D=128), the one shape of the set that is firmly
    tensor-bound: forward and backward timed separately, a few steps each (13 ms per step).
    `units` < 192 cuts the (batch x head) axis, for profiler captures; `unit_ids` selects a
    shard of it. Figures are per GPU."""
    torch, dev = cx.torch, cx.dev
    Lg = W.LARGE
    ids = list(unit_ids) if unit_ids is not None else list(range(units or Lg.BH))
    BH = len(ids)
    lq, lk, lv, ldo = large_inputs(torch, dev, Lg, ids)
    lo, ll = torch.empty_like(lq), torch.empty(BH, Lg.S, device=dev)
    lg = [torch.empty_like(lq) for _ in range(3)]
    lws = torch.empty(ws_bytes(BH, Lg.S, Lg.D), dtype=torch.uint8, device=dev)
    ms_lf = cx.timed(lambda s: dad.gpu_flash_attention_forward_bf16(lo, ll, lq, lk, lv, BH, Lg.S, Lg.D,
                                                                    Lg.scale), steps, warm)
    ms_lb = cx.timed(lambda s: dad.gpu_flash_attention_backward_bf16(*lg, lws, ldo, lo, ll, lq, lk, lv,
                                                                     BH, Lg.S, Lg.D, Lg.scale), steps, warm)
    lf, lb = W.attn_flops(BH, Lg.S, Lg.D)
    peaks = load_peaks()
    sustained = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    burst = float(peaks["bf16_tflops"])
    large = {"workload": Lg.name, "units_per_gpu": BH, "fwd_ms": ms_lf, "bwd_ms": ms_lb,
             "fwd_tflops": lf / ms_lf / 1e9, "bwd_tflops": lb / ms_lb / 1e9,
             "fwd_bwd_tflops": (lf + lb) / (ms_lf + ms_lb) / 1e9,
             "frac_of_burst_bf16_peak": (lf + lb) / (ms_lf + ms_lb) / 1e9 / burst,
             "frac_of_sustained_bf16_peak": (lf + lb) / (ms_lf + ms_lb) / 1e9 / sustained,
             "peak_source": peaks["_source"],
             "note": "inputs (1.6 GB at 192 units) far larger than L2; per-unit seeded inputs"}
    if verify and cx.rank == 0:
        # one whole unit (the last of this rank's) against the float64 numpy restatement
        u = BH - 1
        got = {"out": lo[u], "lse": ll[u], "dq": lg[0][u], "dk": lg[1][u], "dv": lg[2][u]}
        got = {n: t.float().cpu().numpy() for n, t in got.items()}
        ins = [t[u].float().cpu().numpy() for t in (lq, lk, lv, ldo)]
        large["verify"] = {"unit": ids[u], **check_unit_against_numpy(*ins, got, Lg.scale)}
    results = {"out": lo, "lse": ll, "dq": lg[0], "dk": lg[1], "dv": lg[2]} if unit_ids is not None else None
    del lq, lk, lv, ldo, lws
    if results is None:
        del lo, ll, lg
        torch.cuda.empty_cache()
        return large
    return large, results


def bench_decode(cx, dad, W, steps=None, graph=True, verify=True, seq_ids=None):
    """KV-cache decode workload: 12 layer caches, 256 steps with append, one CUDA graph per
    12-layer step. By default all 64 sequences on this GPU; `seq_ids` selects a shard of them.
    Returns achieved HBM GB/s (per GPU) against the algorithmic bytes."""
    torch, dev = cx.torch, cx.dev
    cfg = W.DecodeShape()
    if steps is not None:
        cfg = W.DecodeShape(steps=min(steps, cfg.steps))
    ids = np.arange(cfg.B) if seq_ids is None else np.asarray(list(seq_ids))
    B = len(ids)
    lens0 = W.decode_lengths(cfg)[ids]
    caches = [dad.KVCacheBF16(B, cfg.H, cfg.max_len, cfg.D, device=dev) for _ in range(cfg.layers)]
    # every sequence's cache rows and token vectors come from that sequence's own generator, so a
    # shard of the sequences sees the same data as the whole batch
    gen = torch.Generator(device=dev)
    q, kn, vn = (torch.empty(cfg.layers, B, cfg.H, cfg.D, dtype=torch.bfloat16, device=dev) for _ in range(3))
    for i, b in enumerate(ids):
        gen.manual_seed(1000003 * cfg.seed + int(b))
        for c in caches:
            c.k[i].copy_(torch.randn(cfg.H, cfg.max_len, cfg.D, device=dev, generator=gen))
            c.v[i].copy_(torch.randn(cfg.H, cfg.max_len, cfg.D, device=dev, generator=gen))
        x = torch.randn(3, cfg.layers, cfg.H, cfg.D, device=dev, generator=gen)
        q[:, i], kn[:, i], vn[:, i] = x[0], x[1], x[2]
    out = torch.empty(cfg.layers, B, cfg.H, cfg.D, dtype=torch.bfloat16, device=dev)
    lens_dev = torch.from_numpy(lens0.astype(np.int32)).to(dev)

    def reset():
        for c in caches:
            c.lengths.copy_(lens_dev)

    def step():
        for l, c in enumerate(caches):
            dad.decode_attention_bf16(out[l], q[l], kn[l], vn[l], c, cfg.scale)

    # Twelve layer caches, each with its own lengths and workspace: the kernel ahead of a call never
    # writes that call's cache, so the calls may start early (dadattn_set_decode_early_start).
    dad.set_decode_early_start(cfg.layers >= 2)
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
    cx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(cfg.steps):
        replay()
    e1.record()
    cx.barrier()
    ms = cx.max_over_ranks(e0.elapsed_time(e1))
    dad.set_decode_early_start(False)
    total = sum(W.decode_bytes_per_layer_call(lens0 + s + 1, cfg.H, cfg.D)
                for s in range(cfg.steps)) * cfg.layers
    ok = bool((caches[0].lengths.cpu().numpy() == lens0 + cfg.steps).all())
    peaks = load_peaks()
    gbs = total / ms / 1e6
    res = {"metric": "kv_decode_hbm_gbs", "value": gbs, "unit": "GB/s", "ms_total": ms,
           "steps": cfg.steps, "layers": cfg.layers, "sequences_per_gpu": B,
           "algorithmic_gb": total / 1e9, "frac_of_hbm_peak": gbs / float(peaks["hbm_gbs"]),
           "peak_source": peaks["_source"], "gpu_launches": cfg.layers * cfg.steps,
           "lengths_advanced": ok, "workload": cfg.name}
    if verify:
        # The first step once more, from the initial lengths, replayed from the same graph;
        # layers 0 and 11 of it are checked on the host against the oracle (output, appended
        # rows, lengths). Every rank checks its own sequences.
        from oracle.oracle import Oracle
        ora = Oracle()
        reset()
        out.fill_(float("nan"))
        replay()
        torch.cuda.synchronize()
        now = (lens0 + 1).astype(np.int32)
        good, worst = ok, 0.0
        rows = torch.from_numpy(lens0.astype(np.int64)).to(dev)
        ar = torch.arange(B, device=dev)
        for l in (0, cfg.layers - 1):
            c = caches[l]
            good &= bool((c.lengths.cpu().numpy() == now).all())
            good &= bool(torch.equal(c.k[ar, :, rows], kn[l])) and bool(torch.equal(c.v[ar, :, rows], vn[l]))
            want = ora.decode(q[l].float().cpu().numpy(), c.k.float().cpu().numpy(),
                              c.v.float().cpu().numpy(), now, cfg.scale)
            worst = max(worst, float(np.abs(out[l].float().cpu().numpy() - want).max()))
        good &= worst <= 2e-2
        good = cx.all_ok(bool(good))
        res["verify"] = {"ok": good, "out_max_abs": cx.max_over_ranks(worst), "tolerance": 2e-2,
                         "layers_checked": [0, cfg.layers - 1],
                         "what": "one replayed step from the initial lengths: out, appended rows, lengths"}
    return res


def bench_strong(cx, dad, W, ws_bytes, large_1gpu, decode_1gpu, verify=True):
    """Fixed total work sharded over the ranks (the partition the path offers: independent
    (batch x head) units, independent sequences). Rank g owns the contiguous range
    shard_units(total, N, g); no collective inside the timed region. Afterwards every rank's
    out, lse, dQ, dK, dV are all-gathered over NCCL and rank 0 checks whole units that other
    ranks computed. Speed-ups are against the same run's one-GPU figures (`large_shape`,
    `decode`: the full problem on one GPU, measured while the other ranks do the same)."""
    from dadgpt_b200.sharding import all_gather_units, shard_units
    torch, world, rank = cx.torch, cx.world, cx.rank
    Lg = W.LARGE
    sh = shard_units(Lg.BH, world, rank)
    ids = range(sh.unit0, sh.unit0 + sh.count)
    part, res = bench_large(cx, dad, W, ws_bytes, verify=False, unit_ids=ids)
    ms = part["fwd_ms"] + part["bwd_ms"]
    t1 = large_1gpu["fwd_ms"] + large_1gpu["bwd_ms"]
    lf, lb = W.attn_flops(Lg.BH, Lg.S, Lg.D)
    strong = {"large_shape": {"workload": Lg.name, "total_units": Lg.BH, "units_per_gpu": sh.count,
                              "fwd_ms": part["fwd_ms"], "bwd_ms": part["bwd_ms"], "ms": ms,
                              "one_gpu_ms": t1, "speedup": t1 / ms,
                              "tflops_total": (lf + lb) / ms / 1e9}}
    if verify:
        # all-gather over NCCL (NVLink / NVSwitch), outside every timed region
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cx.barrier()
        e0.record()
        full = {n: all_gather_units(t, Lg.BH) for n, t in res.items()}
        e1.record()
        cx.barrier()
        gather_ms = cx.max_over_ranks(e0.elapsed_time(e1))
        nbytes = sum(t.numel() * t.element_size() for t in full.values())
        v = {"ok": True}
        if rank == 0:
            checks = []
            for u in sorted({0, Lg.BH // 2, Lg.BH - 1}):  # units of the first, a middle and the last rank
                q, k, v_, do = (t[0].float().cpu().numpy() for t in large_inputs(torch, cx.dev, Lg, [u]))
                got = {n: t[u].float().cpu().numpy() for n, t in full.items()}
                owner = next(g for g in range(world)
                             if shard_units(Lg.BH, world, g).unit0 <= u
                             < shard_units(Lg.BH, world, g).unit0 + shard_units(Lg.BH, world, g).count)
                checks.append({"unit": u, "computed_by_rank": owner,
                               **check_unit_against_numpy(q, k, v_, do, got, Lg.scale)})
            v = {"ok": all(c["ok"] for c in checks), "units": checks}
        v["ok"] = cx.all_ok(bool(v["ok"]))
        v["all_gather"] = {"bytes_gathered_per_rank": nbytes, "ms": gather_ms,
                           "gbs_per_rank": nbytes * (world - 1) / world / gather_ms / 1e6}
        strong["large_shape"]["verify"] = v
        del full
    del res
    torch.cuda.empty_cache()

    cfg = W.DecodeShape()
    shd = shard_units(cfg.B, world, rank)
    d = bench_decode(cx, dad, W, verify=verify, seq_ids=range(shd.unit0, shd.unit0 + shd.count))
    # whole-job bytes over the max-over-ranks time: every rank reports its own bytes, sum them
    tot = torch.tensor([d["algorithmic_gb"]], device=cx.dev, dtype=torch.float64)
    if world > 1:
        cx.dist.all_reduce(tot)
    strong["decode"] = {"workload": cfg.name, "total_sequences": cfg.B, "sequences_per_gpu": shd.count,
                        "ms_total": d["ms_total"], "one_gpu_ms": decode_1gpu["ms_total"],
                        "speedup": decode_1gpu["ms_total"] / d["ms_total"],
                        "gbs_total": float(tot.item()) / (d["ms_total"] * 1e-3),
                        "verify": d.get("verify"),
                        "note": "few (sequence, head) pairs per GPU: the cache rows of a pair are "
                                "split across CTAs and merged through tickets (split-K branch)"}
    strong["ok"] = bool((not verify) or (strong["large_shape"]["verify"]["ok"] and d["verify"]["ok"]))
    return strong


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=5,
                    help="how many times the K-step headline region is taken (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-verify", action="store_true",
                    help="skip the after-the-timing checks against the oracle")
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
