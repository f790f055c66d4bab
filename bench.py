#!/usr/bin/env python
"""Benchmark of the SparseDrop hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload: one SparseDrop linear at M = N = K = 4096, fp16 inputs, fp32
accumulation, 128 x 128 blocks, p = 0.5, inputs N(0, K^-1/2).  One "step" is the whole hot path for one
batch: the Philox block-plan kernel (mask + kept-block lists), the DSD forward, the SDD dX and the DSD dW.
The metric is useful TFLOP/s: 3 * 2 * 128^2 * N * (kept blocks of that step's mask) / time.

* `value`  — inputs resident in HBM, kernels launched through the C ABI, CUDA-event time over K steps.
             Four rotating input/output sets (768 MB) are used so no step finds its operands in L2.
* `e2e`    — same metric through the public operator API (flash_dropout.functional + autograd) from
             pinned HOST buffers: H2D of x, W, dy and D2H of y, dx, dW inside the timed region.
* roofline — the GEMM kernel (3 launches per step), timed per launch with CUDA events inside the same
             timed region, against the measured dense bf16 peak in MEASURED_PEAKS.json.
* cpu_baseline / --impl reference — the reference's CPU path (oracle/cpu_path.py) on the host cores.
* N > 1    — one process per GPU (torchrun), data parallel: every rank runs the step on its own batch
             shard and the weight gradient is all-reduced over NCCL; weak scaling.
* sub-records, appended last on the same JSON line and measured in the same process: `sustained` (>= 0.5 s of
  back-to-back steps with the clocks seen), `p_sweep` (p = 0 .. 0.9), `conv` (the 256x64x32x32 3x3 conv layer,
  forward + backward), `mlp` / `gpt` (training-step samples/s at this run's N, SparseDrop and vanilla dropout),
  `model_sweep` (whole-MLP step time against p), `c1_cpu` (the reference's 1024^3 fp32 forward on the host).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(REPO, "sparse-dropout_b200"), REPO):
    if _p not in sys.path:
        sys.path.insert(0, _p)

M = N = K = 4096
BLOCK = 128
P_DROP = 0.5
SEED = 0
N_SETS = 4
METRIC = "DSD/SDD useful TFLOP/s (DSD fwd + SDD dX + DSD dW on kept 128x128 blocks) at 4096^3 fp16, p=0.5"
WORKLOAD = ("SparseDrop linear fwd+bwd, M=N=K=4096, fp16 in / fp32 acc, 128x128 blocks, "
            "p=0.5, x,W,dy~N(0,K^-1/2), per-step Philox mask (seed 0, offset=step)")
# DRAM bytes (read + written) per GEMM launch of this workload as an ncu capture counts them: the mean of the
# step's three launches, 60.3 / 92.2 / 63.1 MB.  A profiler figure cannot be taken inside a timed run, so it is
# carried here as a constant and reported as `roofline.traffic`.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 71.9e6


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured burst bf16 (MEASURED_PEAKS.json)"
    except (OSError, KeyError, ValueError):
        return 1590.0, "fallback 1.59 PFLOP/s (MEASURED_PEAKS.json absent)"


def measured_peak(key: str, fallback: float) -> tuple[float, str]:
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)[key]), "measured"
    except (OSError, KeyError, ValueError):
        return fallback, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period, self.samples, self._stop = index, period_s, [], threading.Event()
        self._thread = None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self, t0: float, t1: float) -> dict:
        if not self.nv:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self._stop.set()
        self._thread.join()
        nv = self.nv
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples[-3:]
        mhz = sorted(s[1] for s in inside)
        bits = 0
        for s in inside:
            bits |= s[2]
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": self.max_mhz,
                "reasons": [k for k, v in names.items() if bits & v], "samples": len(inside)}


def useful_flops(kept_tiles: int) -> float:
    return 3 * 2.0 * BLOCK * BLOCK * N * kept_tiles


# ------------------------------------------------------------------------------------------ reference arm
def run_reference(args) -> None:
    """The reference's own CPU implementation of the path (oracle/_ref when present, else the oracle port) on all
    host threads; rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_path
    info = cpu_path.host_info()
    budget = 20.0
    r = cpu_path.time_linear_fwd_bwd(M, N, K, BLOCK, P_DROP, seed=SEED, budget_s=budget,
                                     max_passes=max(1, min(args.steps, 5)))
    tflops = useful_flops(r["kept_tiles"]) / r["seconds_per_pass"] / 1e12
    sample = (f"{r['passes']} full passes of the 4096^3 fwd+dX+dW masked-dense path in fp32 "
              f"(dense work: dropped blocks are not skipped on the CPU), median; {info['cpu_model']}")
    c1 = cpu_path.time_forward_1024(seed=SEED, p=P_DROP)
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": r["passes"], "warmup": 1, "ms_per_step": r["seconds_per_pass"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "host": info["cpu_model"]},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": r["threads"], "kind": r["kind"], "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "c1_cpu": {"workload": "fp32 forward y=(mask o x).W^T/(1-p), 1024^3, 128x128 blocks, p=0.5, seed 0",
                   "ms": c1["ms"], "cores": c1["threads"], "kind": c1["kind"],
                   "dense_equivalent_gflops": c1["dense_equivalent_gflops"]},
    }
    print(json.dumps(line))



# ------------------------------------------------------------------------------------------ our arm
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import flash_dropout.functional as F
    from flash_dropout import _lib
    from flash_dropout import random as sd_random
    from flash_dropout.cuda.binding_gemm import BlockPlan, dsd, sdd

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SparseDrop kernels have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()

    steps, warmup = args.steps, max(args.warmup, 3)
    scale = 1.0 / (1.0 - P_DROP)
    g = torch.Generator().manual_seed(SEED + 1000 * rank)
    sets = []
    # With several ranks the weight-gradient buffers come from a memory pool registered with NCCL as user buffers, so the
    # all-reduce can work on them in place (through the switch where the fabric offers it) with few of its own thread
    # blocks competing with the GEMMs for SMs.
    grad_pool, registered = None, False
    if world > 1 and os.environ.get("SD_BENCH_REGISTER", "1") == "1":
        try:
            backend = dist.group.WORLD._get_backend(dev)
            grad_pool = torch.cuda.MemPool(backend.mem_allocator)
        except Exception:                                   # noqa: BLE001 - not offered by this torch / NCCL build
            grad_pool = None
    for _ in range(N_SETS):
        x = (torch.randn(M, K, generator=g) * K ** -0.25).half().to(dev)
        w = (torch.randn(N, K, generator=g) * K ** -0.25).half().to(dev)
        dy = (torch.randn(M, N, generator=g) * N ** -0.25).half().to(dev)
        if grad_pool is not None:
            with torch.cuda.use_mem_pool(grad_pool):
                dw_buf = torch.empty(N, K, device=dev, dtype=torch.float16)
        else:
            dw_buf = torch.empty(N, K, device=dev, dtype=torch.float16)
        sets.append((x, w, dy, torch.empty(M, N, device=dev, dtype=torch.float16),
                     torch.empty(M, K, device=dev, dtype=torch.float16), dw_buf))
    if grad_pool is not None:
        try:
            backend.register_mem_pool(grad_pool)
            registered = True
        except Exception:                                   # noqa: BLE001
            registered = False
    plans = [BlockPlan(M // BLOCK, K // BLOCK, dev) for _ in range(N_SETS)]
    L = _lib.lib()
    stream = torch.cuda.current_stream(dev)

    # Gradient exchange: the all-reduce of a step's dW is issued from a stream of its own, behind an event that the
    # dW product records, and the compute stream waits for it only when the operand set comes round again.  Events on
    # that stream bracket each all-reduce (its wait for NCCL's stream included), which gives the exchange's own time.
    comm = torch.cuda.Stream(dev) if world > 1 else None
    # The products' persistent grids leave SD_BENCH_SM_MARGIN SMs (default 32: NCCL runs 24 to 32 channels on this
    # fabric) to the all-reduce that runs beside them; without that each all-reduce crawls behind the products for
    # lack of SMs and, where it does get some, stretches the launch whose CTAs wait for them.
    sm_margin = int(os.environ.get("SD_BENCH_SM_MARGIN", "32")) if world > 1 else 0
    import flash_dropout
    prev_margin = flash_dropout.set_sm_margin(sm_margin)
    dw_done = [torch.cuda.Event() for _ in range(N_SETS)]
    reduced = [torch.cuda.Event() for _ in range(N_SETS)]
    pending = [None] * N_SETS

    def drain():
        for j, ev in enumerate(pending):
            if ev is not None:
                stream.wait_event(ev)
                pending[j] = None

    # The mask of step i + 1 does not depend on step i, so its plan kernel (one CTA, a few microseconds) is launched on
    # a second stream while step i's products run, as a training loop that draws the next layer's mask early would;
    # the products of step i + 1 wait for it through an event.  Every step's plan launch is inside the timed region.
    plan_stream = torch.cuda.Stream(dev)
    plan_ready = [torch.cuda.Event() for _ in range(N_SETS)]
    set_free = [torch.cuda.Event() for _ in range(N_SETS)]
    planned = set()

    def launch_plan(i: int):
        plan = plans[i % N_SETS]
        with torch.cuda.stream(plan_stream):
            plan_stream.wait_event(set_free[i % N_SETS])          # the step that last read this plan buffer is done
            # mask + kept-block lists for step i: one launch, offset = step index, rank = Philox subsequence
            _lib.check(L.sd_plan_from_seed(plan.buf.data_ptr(), plan.R, plan.C, 1, 1, SEED, (rank << 40) + i,
                                           P_DROP, None, plan_stream.cuda_stream))
            plan_ready[i % N_SETS].record(plan_stream)
        planned.add(i)

    def step(i: int, events=None, exchange: bool = True):
        x, w, dy, y, dx, dw = sets[i % N_SETS]
        plan = plans[i % N_SETS]
        if pending[i % N_SETS] is not None:
            stream.wait_event(pending[i % N_SETS])
            pending[i % N_SETS] = None
        if i not in planned:
            launch_plan(i)
        planned.discard(i)
        stream.wait_event(plan_ready[i % N_SETS])
        if events is not None:
            events[0].record()
        dsd(x, w, plan, _lib.SD_PLAN_ROWS, scale, out=y)
        if events is not None:
            events[1].record()
        launch_plan(i + 1)                                         # overlaps this step's remaining products
        sdd(dy, w.T, plan, scale, out=dx)
        if events is not None:
            events[2].record()
        dsd(x.T, dy.T, plan, _lib.SD_PLAN_COLS, scale, out=dw.T)
        if events is not None:
            events[3].record()
        set_free[i % N_SETS].record(stream)
        if world > 1 and exchange:
            # the gradient exchange runs while the next steps compute; it is waited for before this operand set is
            # used again (and at the end of the timed region)
            k = i % N_SETS
            dw_done[k].record(stream)
            with torch.cuda.stream(comm):
                comm.wait_event(dw_done[k])
                if events is not None:
                    events[4].record(comm)
                dist.all_reduce(dw)
                if events is not None:
                    events[5].record(comm)
                reduced[k].record(comm)
            pending[k] = reduced[k]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(warmup):
        step(i)
    drain()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        step(warmup + i, evs[i])
    drain()
    e1.record()
    barrier()
    t1 = time.perf_counter()
    clocks = sampler.stop(t0, t1)
    ms_total = e0.elapsed_time(e1)
    # kept blocks of every timed step's mask, recomputed after the timed region (same seed / offsets)
    kept_dev = torch.zeros(1, dtype=torch.int64, device=dev)
    for i in range(steps):
        _lib.check(L.sd_plan_from_seed(plans[0].buf.data_ptr(), plans[0].R, plans[0].C, 1, 1, SEED,
                                       (rank << 40) + warmup + i, P_DROP, None, stream.cuda_stream))
        kept_dev += plans[0].header[0]
    kept = kept_dev.item()
    flash_dropout.set_sm_margin(prev_margin)        # the other measurements below use every SM
    gemm_ms = sum(ev[0].elapsed_time(ev[3]) for ev in evs)
    per_kernel_ms = [sum(ev[j].elapsed_time(ev[j + 1]) for ev in evs) / steps for j in range(3)]
    exchange_ms = sum(ev[4].elapsed_time(ev[5]) for ev in evs) / steps if world > 1 else None

    # ---- end to end through the operator API from pinned host memory.  Three streams, two buffer sets: the
    # H2D copy of step i+1 and the D2H copy of step i-1 run while step i computes (PCIe is full duplex).
    e2e_steps = max(3, min(steps, 20))
    hx, hw, hdy = (torch.empty(M, K, dtype=torch.float16).pin_memory() for _ in range(3))
    hx.copy_(sets[0][0].cpu()); hw.copy_(sets[0][1].cpu()); hdy.copy_(sets[0][2].cpu())
    host_out = [[torch.empty(M, K, dtype=torch.float16).pin_memory() for _ in range(3)] for _ in range(2)]
    dev_in = [[torch.empty(M, K, device=dev, dtype=torch.float16) for _ in range(3)] for _ in range(2)]
    s_in, s_comp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    live = [None, None]           # results of the step that last used a buffer set, kept until its D2H is done
    sd_random.manual_seed(SEED, subsequence=rank)
    e2e_plans = []

    def e2e_step(i: int):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_comp[b])                      # the step that used these inputs has finished
            for d, h in zip(dev_in[b], (hx, hw, hdy)):
                d.copy_(h, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(ev_in[b])
            xa, wa = dev_in[b][0].detach().requires_grad_(), dev_in[b][1].detach().requires_grad_()
            seed, off = sd_random.next_seed_offset()
            plan = BlockPlan.from_seed(M, K, BLOCK, P_DROP, seed, off, dev)
            y = F.cuda_blockwise_dropout_matmul(xa, wa, BLOCK, P_DROP, plan)
            y.backward(dev_in[b][2])
            if world > 1:
                dist.all_reduce(wa.grad)
            ev_comp[b].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])
            s_out.wait_event(ev_out[b])
            for h, d in zip(host_out[b], (y.detach(), xa.grad, wa.grad)):
                h.copy_(d, non_blocking=True)
            ev_out[b].record(s_out)
        live[b] = (y, xa, wa)
        return plan

    for i in range(4):
        e2e_step(i)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for st in (s_in, s_comp, s_out):
        st.wait_event(f0)
    for i in range(e2e_steps):
        e2e_plans.append(e2e_step(i))
    for st in (s_in, s_comp, s_out):
        stream.wait_stream(st)
    f1.record(stream)
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    e2e_kept = sum(int(pl.header[0].item()) for pl in e2e_plans)
    live = [None, None]

    # ---- aggregate over ranks: max time, summed work
    stats = torch.tensor([ms_total, e2e_ms, gemm_ms], device=dev, dtype=torch.float64)
    work = torch.tensor([float(kept), float(e2e_kept)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    ms_total, e2e_ms, gemm_ms_max = stats.tolist()
    kept_all, e2e_kept_all = work.tolist()
    # the end of a timed region is where the host synchronises anyway: did any kernel give up on a wait?
    flash_dropout.check_status(dev)

    # ---- training-step workloads at this run's N (every rank takes part), SparseDrop and vanilla dropout
    train = {}
    if not args.no_extras:
        tsteps = max(10, min(steps, 50))
        for wl in ("mlp", "gpt"):
            rec = {}
            for variant in ("blockwise[cuda]", "vanilla"):
                r = measure_train(wl, variant, dev, world, rank, tsteps, 5, graph=True, e2e=False)
                rec[variant] = {"samples_per_s": r["samples_per_s"], "ms_per_step": r["ms_per_step"]}
                step_desc, wl_name = r["step"], r["workload"]
            rec["speedup_vs_vanilla"] = rec["blockwise[cuda]"]["samples_per_s"] / rec["vanilla"]["samples_per_s"]
            rec.update({"n_gpus": world, "steps": tsteps, "workload": wl_name, "step": step_desc})
            train[wl] = rec
        flash_dropout.check_status(dev)

    # ---- rank 0 only: the same kernels over p (speed-up vs p = 0), a sustained run, the conv layer, CPU legs
    extra = {}
    if rank == 0 and not args.no_extras:
        def time_three(plan, sc, reps=10):
            x, w, dy, y, dx, dw = sets[0]
            out = []
            for fn in (lambda: dsd(x, w, plan, _lib.SD_PLAN_ROWS, sc, out=y), lambda: sdd(dy, w.T, plan, sc, out=dx),
                       lambda: dsd(x.T, dy.T, plan, _lib.SD_PLAN_COLS, sc, out=dw.T)):
                ts = []
                for r in range(reps + 2):
                    for s in sets[1:]:
                        s[3].zero_()     # push set 0 out of L2 between timed launches
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(); fn(); b.record(); torch.cuda.synchronize()
                    if r >= 2:
                        ts.append(a.elapsed_time(b))
                ts.sort()
                out.append(ts[len(ts) // 2])
            return out

        def time_stream(plan, sc, n=40, warm=5):
            """The three launches back to back over the rotating operand sets, as in the timed region above."""
            evs3 = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n)]
            for i in range(warm + n):
                x, w, dy, y, dx, dw = sets[i % N_SETS]
                ev = evs3[i - warm] if i >= warm else None
                if ev: ev[0].record()
                dsd(x, w, plan, _lib.SD_PLAN_ROWS, sc, out=y)
                if ev: ev[1].record()
                sdd(dy, w.T, plan, sc, out=dx)
                if ev: ev[2].record()
                dsd(x.T, dy.T, plan, _lib.SD_PLAN_COLS, sc, out=dw.T)
                if ev: ev[3].record()
            torch.cuda.synchronize()
            return [sum(ev[j].elapsed_time(ev[j + 1]) for ev in evs3) / n for j in range(3)]

        # p = 0, 0.1, ..., 0.9: one mask per p from (seed, offset = index of p); fwd + dX + dW
        ps = [round(0.1 * i, 1) for i in range(10)]
        stream_ms, cold_ms, kept_p = {}, {}, {}
        for idx, p in enumerate(ps):
            plan = BlockPlan.from_seed(M, K, BLOCK, p, SEED, 0 if p in (0.0, 0.5) else idx, dev)
            stream_ms[p] = time_stream(plan, 1.0 / (1.0 - p), n=40 if p in (0.0, 0.5) else 20)
            cold_ms[p] = time_three(plan, 1.0 / (1.0 - p), reps=10 if p in (0.0, 0.5) else 5)
            kept_p[p] = int(plan.header[0].item())
        t0s, t5s = stream_ms[0.0], stream_ms[0.5]
        c0s, c5s = cold_ms[0.0], cold_ms[0.5]
        extra["speedup_vs_p0"] = {"fwd_dsd": t0s[0] / t5s[0], "dx_sdd": t0s[1] / t5s[1], "dw_dsd": t0s[2] / t5s[2],
                                  "fwd_bwd": sum(t0s) / sum(t5s), "ms_p0": t0s, "ms_p0.5": t5s,
                                  "kept_p0.5": kept_p[0.5],
                                  "method": "mean of 40 back-to-back fwd/dX/dW triples over the rotating operand sets "
                                            "(the timed region's loop), same fixed mask for every triple",
                                  "cold_single_launch": {"fwd_bwd": sum(c0s) / sum(c5s), "ms_p0": c0s, "ms_p0.5": c5s,
                                                         "method": "median of 10 single launches, L2 flushed and the "
                                                                   "stream drained between launches"}}
        r3 = lambda v: round(v, 4)
        extra["p_sweep"] = {
            "p": ps, "kept_blocks": [kept_p[p] for p in ps],
            "fwd_bwd_ms": [r3(sum(stream_ms[p])) for p in ps],
            "speedup_vs_p0": [r3(sum(t0s) / sum(stream_ms[p])) for p in ps],
            "useful_tflops": [r3(useful_flops(kept_p[p]) / (sum(stream_ms[p]) * 1e-3) / 1e12) for p in ps],
            "cold_fwd_bwd_ms": [r3(sum(cold_ms[p])) for p in ps],
            "cold_speedup_vs_p0": [r3(sum(c0s) / sum(cold_ms[p])) for p in ps],
            "method": "fwd+dX+dW at 4096^3 fp16, one Philox mask per p; back-to-back triples over rotating operand "
                      "sets (mean), and single launches with L2 flushed and the stream drained (median)"}

        # sustained: the whole step back to back for at least half a second, with the clocks seen meanwhile
        n_sus = max(3000, int(0.6 / max(1e-6, ms_total / steps * 1e-3)))
        torch.cuda.synchronize()
        sampler2 = ClockSampler(local, period_s=0.01)
        sampler2.start()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter()
        s0.record()
        for i in range(n_sus):
            step(10_000 + i, exchange=False)
        s1.record()
        torch.cuda.synchronize()
        w1 = time.perf_counter()
        clocks2 = sampler2.stop(w0, w1)
        sus_ms = s0.elapsed_time(s1)
        kept_dev.zero_()
        for i in range(n_sus):
            _lib.check(L.sd_plan_from_seed(plans[0].buf.data_ptr(), plans[0].R, plans[0].C, 1, 1, SEED,
                                           (rank << 40) + 10_000 + i, P_DROP, None, stream.cuda_stream))
            kept_dev += plans[0].header[0]
        sus_tflops = useful_flops(kept_dev.item()) / (sus_ms * 1e-3) / 1e12
        sus_peak, sus_src = measured_peak("bf16_tflops_sustained", 1400.0)
        extra["sustained"] = {"seconds": sus_ms * 1e-3, "steps": n_sus, "ms_per_step": sus_ms / n_sus,
                              "useful_tflops": sus_tflops, "peak": sus_peak,
                              "peak_source": f"{sus_src} sustained bf16", "frac": sus_tflops / sus_peak,
                              "clocks": clocks2, "power_capped": "sw_power_cap" in (clocks2.get("reasons") or [])}
        flash_dropout.check_status(dev)
        sets.clear()
        plans.clear()
        torch.cuda.empty_cache()
        extra["conv"] = measure_conv(dev, max(10, min(steps, 30)), 3, extras=False)
        if world == 1:      # a single-GPU record (its training steps would issue collectives on this rank alone)
            extra["model_sweep"] = measure_model_sweep(dev)
        flash_dropout.check_status(dev)

    if rank == 0:
        value = useful_flops(kept_all) / (ms_total * 1e-3) / 1e12
        e2e_value = useful_flops(e2e_kept_all) / (e2e_ms * 1e-3) / 1e12
        peak, peak_src = measured_peaks()
        achieved = useful_flops(kept) / (gemm_ms * 1e-3) / 1e12      # this rank's GEMM launches only
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_total / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "parallelism": f"dp{world}" if world > 1 else "single GPU",
                       "l2": f"{N_SETS} rotating operand/result sets (768 MB > 126 MB L2), no flush kernel",
                       "step": "plan kernel (drawn one step ahead on a second stream) + DSD fwd + SDD dX + DSD dW"
                               + ((" + NCCL allreduce(dW)" + (" on registered user buffers" if registered else ""))
                                  if world > 1 else "")},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                         "kernel": "sparsedrop_gemm_kernel (3 launches per step: DSD fwd, SDD dX, DSD dW)",
                         "peak_source": peak_src, "frac_of_nominal_2250": achieved / 2250.0,
                         "avg_launch_ms": {"dsd_fwd": per_kernel_ms[0], "sdd_dx": per_kernel_ms[1], "dsd_dw": per_kernel_ms[2]},
                         "flops_per_launch": useful_flops(kept) / 3 / steps},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": 3 * M * K * 2,
                    "d2h_bytes_per_step": 3 * M * K * 2, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                    "api": "flash_dropout.functional.cuda_blockwise_dropout_matmul + backward, pinned host buffers; "
                           "H2D / compute / D2H of consecutive steps overlap on three streams"},
            "gpu_launches": 4 * steps, "clocks": clocks,
        }
        if exchange_ms is not None:
            line["exchange"] = {"allreduce_ms": exchange_ms, "bytes": N * K * 2, "sm_margin": sm_margin,
                                "method": "CUDA events on the exchange's stream around each all-reduce of dW (rank 0), "
                                          "queueing behind the previous one included"}
        if world == 1 and not args.no_extras:
            from oracle import cpu_path
            info = cpu_path.host_info()
            r = cpu_path.time_linear_fwd_bwd(M, N, K, BLOCK, P_DROP, seed=SEED, budget_s=12.0, max_passes=4)
            line["cpu_baseline"] = {
                "value": useful_flops(r["kept_tiles"]) / r["seconds_per_pass"] / 1e12, "unit": "TFLOP/s",
                "cores": r["threads"], "kind": r["kind"],
                "sample": f"{r['passes']} full 4096^3 fwd+dX+dW passes, fp32 masked-dense (no block skipping), "
                          f"median {r['seconds_per_pass']:.3f} s; {info['cpu_model']}"}
        # sub-records last: a reader that keeps only the end of the line still sees them
        for key in ("speedup_vs_p0", "sustained", "p_sweep", "conv", "model_sweep"):
            if key in extra:
                line[key] = extra[key]
        line.update(train)
        if not args.no_extras:
            from oracle import cpu_path
            c1 = cpu_path.time_forward_1024(seed=SEED, p=P_DROP)
            line["c1_cpu"] = {"workload": "fp32 forward y=(mask o x).W^T/(1-p), 1024^3, 128x128 blocks, p=0.5, seed 0",
                              "ms": c1["ms"], "cores": c1["threads"], "kind": c1["kind"],
                              "dense_equivalent_gflops": c1["dense_equivalent_gflops"]}
        print(json.dumps(line))
    # the registered pool hands its memory back through the communicator: release it while that still exists
    sets.clear()
    dw_buf = None
    if grad_pool is not None:
        torch.cuda.synchronize()
        if registered:
            try:
                backend.deregister_mem_pool(grad_pool)
            except Exception:                               # noqa: BLE001
                pass
        del grad_pool
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------ conv layer
CONV_SHAPE = dict(Nb=256, C=64, H=32, W=32, Ko=128)


def conv_algorithmic_bytes() -> float:
    """Bytes a fused forward + backward of the conv layer has to move: forward reads x and writes y; backward reads
    dy twice (dW and dX), reads x once more (dW) and writes dx; the weights are negligible."""
    c = CONV_SHAPE
    x = c["Nb"] * c["C"] * c["H"] * c["W"] * 2
    y = c["Nb"] * c["Ko"] * c["H"] * c["W"] * 2
    return float(x + y + 2 * y + x + x)


def measure_conv(dev, steps: int, warmup: int, extras: bool) -> dict:
    """Conv2d 64->128, 3x3, pad 1 on 256x64x32x32 fp16 with blockwise dropout p=0.5 on the im2col matrix
    (262144 x 576, 128x128 blocks): forward + backward, replayed from a CUDA graph, L2 flushed between steps."""
    import torch

    import flash_dropout.functional as F
    from flash_dropout import random as sd_random
    from flash_dropout.cuda.binding_gemm import BlockPlan

    c = CONV_SHAPE
    Nb, C, H, W, Ko, p = c["Nb"], c["C"], c["H"], c["W"], c["Ko"], P_DROP
    g = torch.Generator().manual_seed(SEED)
    x = torch.randn(Nb, C, H, W, generator=g).half().to(dev).requires_grad_()
    k = (torch.randn(Ko, C, 3, 3, generator=g) / 24).half().to(dev).requires_grad_()
    dy = torch.randn(Nb, Ko, H, W, generator=g).half().to(dev).contiguous(memory_format=torch.channels_last)
    M, K = Nb * H * W, C * 9
    sd_random.manual_seed(SEED, subsequence=0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def sparse_step():
        x.grad = k.grad = None
        y = F.cuda_blockwise_dropout_conv2d(x, k, BLOCK, p, padding=(1, 1))
        y.backward(dy)

    def dense_step():
        x.grad = k.grad = None
        y = torch.nn.functional.conv2d(x, k, padding=1)
        y.backward(dy)

    def unfold_step():
        x.grad = k.grad = None
        a = torch.nn.functional.unfold(x, (3, 3), padding=1).transpose(1, 2).reshape(M, K)
        y = F.cuda_blockwise_dropout_matmul(a, k.reshape(Ko, K), BLOCK, p)
        y.backward(dy.permute(0, 2, 3, 1).reshape(M, Ko))

    def timeit(fn, n):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(n):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]

    def graphed(fn):
        """fn captured in a CUDA graph (after warm-up on a side stream); masks stay fresh through the device counter."""
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            fn()
        return graph.replay

    # The step is a handful of launches behind ~0.3 ms of Python: timed eagerly it is bound by the host, so the
    # headline is the replay of a captured step (both arms), with the eager times beside it when extras are on.
    out_ms = {}
    if extras:
        out_ms["sparsedrop_eager"] = timeit(sparse_step, steps)
        out_ms["cudnn_dense_eager"] = timeit(dense_step, steps)
        out_ms["torch_unfold+sparsedrop_linear_eager"] = timeit(unfold_step, max(3, steps // 4))
    had_counter = sd_random.device_counter(dev) is not None
    if not had_counter:
        sd_random.enable_device_counter(dev)
    t_sparse, t_dense = timeit(graphed(sparse_step), steps), timeit(graphed(dense_step), steps)
    if not had_counter:
        sd_random.disable_device_counter()
    plan = BlockPlan.from_seed(M, 640, BLOCK, p, SEED, 0, dev)
    mask = plan.tile_mask.cpu()
    widths = torch.tensor([128, 128, 128, 128, 64])            # last K block is 64 wide (576 = 4.5 blocks)
    kept_cols = ((mask == 0).float() * widths).sum().item()    # kept (row block, k) columns
    flops = 3 * 2.0 * 128 * Ko * kept_cols                     # fwd + dW + dX on kept blocks
    hbm, hbm_src = measured_peak("hbm_gbs", 6650.0)
    tens, _ = measured_peak("bf16_tflops", 1590.0)
    bytes_alg = conv_algorithmic_bytes()
    t_roof_ms = max(bytes_alg / (hbm * 1e9), flops / (tens * 1e12)) * 1e3
    out_ms["sparsedrop_graph"] = t_sparse
    out_ms["cudnn_dense_graph"] = t_dense
    return {"workload": "Conv2d 64->128 3x3 pad 1, input 256x64x32x32 fp16, 128x128 blocks on the im2col matrix "
                        "(262144 x 576), p=0.5, fwd+bwd; CUDA graph replay, 256 MB L2 flush between steps",
            "ms_per_step": t_sparse, "useful_tflops": flops / (t_sparse * 1e-3) / 1e12,
            "speedup_vs_cudnn_dense": t_dense / t_sparse, "compare_ms": out_ms,
            "roofline": {"bound": "hbm", "algorithmic_bytes": bytes_alg, "useful_flops": flops,
                         "floor_ms": t_roof_ms, "frac": t_roof_ms / t_sparse,
                         "peak": f"{hbm_src} {hbm:.0f} GB/s copy, {tens:.0f} TFLOP/s"}}


def run_conv(args) -> None:
    import torch
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    steps, warmup = args.steps, max(args.warmup, 3)
    r = measure_conv(dev, steps, warmup, extras=not args.no_extras)
    print(json.dumps({
        "metric": "SparseDrop conv fwd+bwd useful TFLOP/s", "value": r["useful_tflops"], "unit": "TFLOP/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": r["workload"]}, "compare_ms": r["compare_ms"], "roofline": r["roofline"],
        "gpu_launches": 4 * steps}))


# ------------------------------------------------------------------------------------------ training steps
def measure_train(workload: str, variant: str, dev, world: int, rank: int, steps: int, warmup: int,
                  graph: bool = True, e2e: bool = True) -> dict:
    """One optimizer step per "step" of the MLP (784-1024-1024-1024-10, batch 512/GPU, p=0.5, AdamW lr 1e-3) or the
    char-GPT (6 layers, d=384, 6 heads, ctx 256, vocab 65, batch 64/GPU, p=0.2, AdamW), bf16 autocast, batch sharded
    over the ranks.  The process group, if any, is already initialised."""
    import torch
    import torch.distributed as dist

    from flash_dropout import random as sd_random
    from flash_dropout.train import GPT, BasicNet, FlatGradDataParallel, train_step

    torch.manual_seed(SEED)
    if workload == "mlp":
        per_gpu, p = 512, 0.5
        model = BasicNet(784, 2, 1024, 10, dict(p=p, variant=variant, block_size=(128, 128))).to(dev)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, fused=True)
        g = torch.Generator().manual_seed(SEED + 1 + rank)
        host_x = torch.rand(per_gpu, 28, 28, generator=g).pin_memory()
        host_y = torch.randint(0, 10, (per_gpu,), generator=g).pin_memory()
        name = "MLP 784-1024-1024-1024-10, bf16 autocast, batch 512/GPU, p=0.5, AdamW lr 1e-3"
        loss_of = lambda m, x, y: torch.nn.functional.cross_entropy(m(x).float(), y)
    else:
        per_gpu, p = 64, 0.2
        model = GPT(65, 256, 6, 6, 384, dict(p=p, variant=variant, block_size=(128, 128))).to(dev)
        opt = model.configure_optimizers(weight_decay=0.1, lr=3e-4)
        g = torch.Generator().manual_seed(SEED + 1 + rank)
        host_x = torch.randint(0, 65, (per_gpu, 256), generator=g).pin_memory()
        host_y = host_x
        name = "char-GPT 6 layers d=384 6 heads ctx 256 vocab 65, bf16 autocast, batch 64/GPU, p=0.2, AdamW"
        loss_of = lambda m, x, y: m(x)[1]
    dp = FlatGradDataParallel(model, bucket_bytes=int(os.environ.get("SD_DP_BUCKET_MB", "16")) << 20, fuse_wgrad=True)
    sd_random.manual_seed(SEED, subsequence=rank)
    x_dev, y_dev = host_x.to(dev), host_y.to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    graphed = None
    if graph:
        from flash_dropout.train import GraphedTrainStep
        graphed = GraphedTrainStep(model, dp, opt, loss_of, (x_dev, y_dev), autocast_dtype=torch.bfloat16)

    def one(resident: bool):
        if graphed is not None:
            if not resident:                       # the step's batch arrives from pinned host memory
                x_dev.copy_(host_x, non_blocking=True)
                if host_y is not host_x:
                    y_dev.copy_(host_y, non_blocking=True)
            loss = graphed()
            return loss if resident else loss.item()
        if resident:
            x, y = x_dev, y_dev
        else:
            x, y = host_x.to(dev, non_blocking=True), host_y.to(dev, non_blocking=True)
        loss = train_step(model, dp, opt, lambda m: loss_of(m, x, y), autocast_dtype=torch.bfloat16)
        return loss if resident else loss.item()

    results, clocks, last = {}, None, 0.0
    for label, resident in (("value", True), ("e2e", False)):
        if label == "e2e" and not e2e:
            continue
        for _ in range(warmup):
            one(resident)
        barrier()
        sampler = ClockSampler(dev.index) if label == "value" else None
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            last = one(resident)
        e1.record()
        barrier()
        t1 = time.perf_counter()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        results[label] = ms.item()
        if sampler:
            clocks = sampler.stop(t0, t1)
    n_mm = sum(1 for m in model.modules() if m.__class__.__name__ == "DropoutMM")
    out = {"workload": name, "variant": variant, "per_gpu": per_gpu, "n_gpus": world,
           "samples_per_s": per_gpu * world * steps / (results["value"] * 1e-3),
           "ms_per_step": results["value"] / steps, "clocks": clocks, "final_loss": float(last),
           "step": graphed.describe() if graphed is not None and hasattr(graphed, "describe") else
                   ("CUDA graph replay" if graphed is not None else
                    "zero_grad + fwd + bwd (bucketed NCCL all-reduce overlapped) + optimizer"),
           "gpu_launches": (4 * n_mm * steps) if "blockwise[cuda]" in variant else 0,
           "h2d_bytes_per_step": host_x.numel() * host_x.element_size()
                                 + (0 if host_y is host_x else host_y.numel() * 8)}
    if "e2e" in results:
        out["e2e_samples_per_s"] = per_gpu * world * steps / (results["e2e"] * 1e-3)
        out["e2e_ms_per_step"] = results["e2e"] / steps
    # free the step's graph and model before the next measurement
    del graphed, dp, opt, model
    torch.cuda.synchronize()
    return out


def measure_model_sweep(dev, steps: int = 30) -> dict:
    """Whole-model step time against the dropout rate, SparseDrop and vanilla dropout: the reference's model benchmark
    (benchmark/model.py:36-60: MLP 1024-1024-1024-1024-10 on a 1024 x 1x32x32 batch, forward + backward) with the
    optimizer step included, bf16 autocast, replayed from a CUDA graph."""
    import torch

    from flash_dropout import random as sd_random
    from flash_dropout.train import BasicNet, FlatGradDataParallel, GraphedTrainStep

    ps = [0.1, 0.3, 0.5, 0.7, 0.9]
    x = torch.rand(1024, 1, 32, 32, device=dev)
    y = torch.randint(0, 10, (1024,), device=dev)
    out = {"p": ps, "workload": "MLP 1024-1024-1024-1024-10, batch 1024, bf16 autocast, zero_grad + fwd + bwd + AdamW, "
                                "CUDA graph replay"}
    for variant in ("blockwise[cuda]", "vanilla"):
        ms = []
        for p in ps:
            torch.manual_seed(SEED)
            sd_random.manual_seed(SEED, subsequence=0)
            model = BasicNet(1024, 2, 1024, 10, dict(p=p, variant=variant, block_size=(128, 128))).to(dev)
            opt = torch.optim.AdamW(model.parameters(), lr=1e-3, fused=True)
            dp = FlatGradDataParallel(model, fuse_wgrad=True)
            step = GraphedTrainStep(model, dp, opt, lambda m, a, b: torch.nn.functional.cross_entropy(m(a).float(), b),
                                    (x, y), autocast_dtype=torch.bfloat16)
            for _ in range(5):
                step()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                step()
            e1.record()
            torch.cuda.synchronize()
            ms.append(round(e0.elapsed_time(e1) / steps, 4))
            del step, dp, opt, model
        out[variant + "_ms"] = ms
    out["speedup_vs_vanilla"] = [round(v / b, 3) for v, b in zip(out["vanilla_ms"], out["blockwise[cuda]_ms"])]
    return out


def run_train(args) -> None:
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SparseDrop kernels have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    steps, warmup = args.steps, max(args.warmup, 3)
    r = measure_train(args.workload, args.variant, dev, world, rank, steps, warmup, graph=not args.no_graph)
    if rank == 0:
        print(json.dumps({
            "metric": "train-step samples/s", "value": r["samples_per_s"], "unit": "samples/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 autocast (fp32 accumulate, fp32 master weights)",
            "data": "synthetic",
            "config": {"workload": r["workload"], "variant": r["variant"], "parallelism": f"dp{world}", "step": r["step"]},
            "e2e": {"value": r.get("e2e_samples_per_s"), "unit": "samples/s", "h2d_bytes_per_step": r["h2d_bytes_per_step"],
                    "d2h_bytes_per_step": 4, "ms_per_step": r.get("e2e_ms_per_step")},
            "gpu_launches": r["gpu_launches"], "clocks": r["clocks"], "final_loss": r["final_loss"]}))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=("gemm", "mlp", "gpt", "conv"), default="gemm",
                    help="gemm: the headline 4096^3 SparseDrop linear (default); mlp / gpt: one training step")
    ap.add_argument("--variant", default="blockwise[cuda]", help="DropoutMM variant for the training workloads")
    ap.add_argument("--no-graph", action="store_true",
                    help="training workloads: launch every kernel eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the sub-records, the p=0 comparison and the CPU baseline (short runs under a profiler)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1:
        # convenience: relaunch under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__),
               "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup)]
        cmd += ["--workload", args.workload, "--variant", args.variant]
        if args.no_graph:
            cmd.append("--no-graph")
        if args.no_extras:
            cmd.append("--no-extras")
        raise SystemExit(subprocess.call(cmd))
    if args.workload == "conv":
        run_conv(args)
        return
    if args.workload != "gemm":
        run_train(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
