#!/usr/bin/env python
"""Benchmark of the contrastive-loss hot path (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

N = 1   CLIP fwd+bwd, B=32768, D=1152, bf16, pre-normalised inputs, T=0.07 (the configuration the
        headline metric is quoted on).  One step = one forward + backward over the whole batch.
N > 1   ring-distributed CLIP fwd+bwd, global B=262144, D=1024, bf16, T=0.03, text = normalize(image +
        0.5 noise), normalise inside (launched by torch.distributed.run, one rank per GPU); the global
        batch is fixed, so scaling is "strong".  --config ring_clip_b131072_d768_bf16 selects the
        other ring configuration.

--config also takes clip_b4096_d512_f32 (the smallest configuration) and lit_b32768_d1152_bf16 (LiT: the metric
counts 6*B^2*D, the one-pass route executes 4*B^2*(D+8), see config.note in the line).

The metric is TFLOP/s with the 8*B^2*D convention (forward 2, recompute 2, two gradient
contractions 2+2).  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TAGS = ["sum_exp", "coef_panel", "dx_contraction", "dy_contraction", "loss_finalize", "normalize_fwd", "normalize_bwd",
        "transpose", "accumulate_f32"]
N_TENSOR_TAGS = 4          # the first four are tensor-bound; the rest are HBM-bound passes whose "flops" are bytes


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p["bf16_tflops_sustained"],
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [v.strip() for v in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------
# CPU baseline: the dense PyTorch formulation on the host cores (checker code, timed here only)
# --------------------------------------------------------------------------------------------
def cpu_dense_step_tflops(b: int, d: int, temperature: float, repeats: int):
    from oracle import dense
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    x = torch.nn.functional.normalize(torch.randn(b, d, generator=g), dim=1)
    y = torch.nn.functional.normalize(torch.randn(b, d, generator=g), dim=1)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        dense.clip_dense(x, y, temperature, True, dtype=torch.float32)
        best = min(best, time.perf_counter() - t0)
    return 8.0 * b * b * d / best / 1e12, best, cores


def run_reference_arm(args):
    """The reference's loss path has no CPU implementation of its own (it is Triton-only and asserts
    CUDA tensors); the dense PyTorch formulation it restates is timed on the host cores instead."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    b, d = 8192, 1152
    times = []
    cores = os.cpu_count() or 1
    for _ in range(args.warmup):
        cpu_dense_step_tflops(b, d, 0.07, 1)
    t_all0 = time.perf_counter()
    for _ in range(args.steps):
        _, sec, cores = cpu_dense_step_tflops(b, d, 0.07, 1)
        times.append(sec)
    wall = time.perf_counter() - t_all0
    ms = 1e3 * sum(times) / len(times)
    val = 8.0 * b * b * d / (ms / 1e3) / 1e12
    sample = f"dense fp32 PyTorch CLIP fwd+bwd on host CPU at B={b}, D={d} (1/16 of the B=32768 tile pairs per step)"
    line = {
        "impl": "reference", "metric": "clip_fwd_bwd_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "clip_b32768_d1152_bf16", "sample_batch": b, "feature_dim": d, "temperature": 0.07,
                   "flop_convention": "8*B^2*D"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": wall,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def profile_tags(lib):
    n = len(TAGS)
    ms = (ctypes.c_double * n)()
    cnt = (ctypes.c_longlong * n)()
    fl = (ctypes.c_double * n)()
    lib.meclip_profile_end(ms, cnt, fl, n)
    out = []
    for i in range(n):
        t = {"kernel": TAGS[i], "launches": int(cnt[i]), "ms": float(ms[i])}
        t["flops" if i < N_TENSOR_TAGS else "bytes"] = float(fl[i])
        out.append(t)
    return out


def run_ours(args):
    import torch.distributed as dist
    from memoryefficientclip_b200 import _lib, synth
    from memoryefficientclip_b200.clip_loss import MemoryEfficientCLIPLoss
    from memoryefficientclip_b200.lit_loss import MemoryEfficientLiTLoss
    from memoryefficientclip_b200.ring import RingMemoryEfficientCLIPLoss, RingMemoryEfficientLiTLoss

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with python -m torch.distributed.run --nproc-per-node N")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()

    if world == 1:
        name = args.config or "clip_b32768_d1152_bf16"
    else:
        name = args.config or "ring_clip_b262144_d1024_bf16"
    kind, b_global, d, dtype, temperature, normalized_inputs, _gen = synth.CONFIGS[name]
    if args.batch:
        b_global = args.batch
    lit = kind == "lit"        # LiT: forward(text, image), the image side is frozen, 6 B^2 D FLOPs
    b_local = b_global // world
    first, second = synth.make(name, b_global, row_start=rank * b_local, rows=b_local)
    host_a = first.pin_memory()
    host_b = second.pin_memory()
    n_probe = min(4096, b_local)
    diag_cos = float(torch.nn.functional.cosine_similarity(first[:n_probe].float(), second[:n_probe].float(), dim=1).mean())
    if world == 1:
        module = (MemoryEfficientLiTLoss if lit else MemoryEfficientCLIPLoss)(temperature, normalized_inputs)
    else:
        module = (RingMemoryEfficientLiTLoss if lit else RingMemoryEfficientCLIPLoss)(temperature, normalized_inputs)
    flops = (6.0 if lit else 8.0) * b_global * b_global * d

    def sync_all():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    def timed(run_step, steps, warmup, sample_clocks=False):
        for _ in range(warmup):
            run_step()
        sync_all()
        sampler = ClockSampler(local_rank) if sample_clocks and rank == 0 else None
        if sampler:
            sampler.start()
        launches0 = lib.meclip_launch_count()
        # one event before the first step and one after every step: the first and the last bracket exactly the
        # K steps (the reported time), the ones between give the per-step spread
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        marks[0].record()
        for i in range(steps):
            run_step()
            marks[i + 1].record()
        sync_all()
        launches = lib.meclip_launch_count() - launches0
        clocks = sampler.stop() if sampler else None
        per_step = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
        ms = torch.tensor([marks[0].elapsed_time(marks[steps])] + per_step, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        ms = ms.tolist()
        spread = {"median": statistics.median(ms[1:]), "min": min(ms[1:]), "max": max(ms[1:])}
        return ms[0] / steps, launches, clocks, spread

    # ---- device-resident inputs (value) ---------------------------------------------------
    a_dev = host_a.to(dev).requires_grad_(True)
    t_dev = host_b.to(dev).requires_grad_(not lit)

    def step_resident():
        a_dev.grad = None
        t_dev.grad = None
        loss = module(a_dev, t_dev)
        loss.backward()

    ms_value, launches, clocks, spread = timed(step_resident, args.steps, args.warmup, sample_clocks=True)

    # ---- end to end: pinned host -> device, module, loss back to the host (e2e) ------------
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    # Every step copies its own inputs from pinned host memory.  As a training loop would, the copy of the
    # NEXT step's batch runs on a copy stream into the other of two device buffers while this step computes.
    copy_stream = torch.cuda.Stream(device=dev)
    dev_bufs = [(torch.empty_like(a_dev), torch.empty_like(t_dev)) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    free = [torch.cuda.Event() for _ in range(2)]
    state = {"i": 0}

    def start_copy(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(free[slot])             # the step that last used this buffer is done
            dev_bufs[slot][0].copy_(host_a, non_blocking=True)
            dev_bufs[slot][1].copy_(host_b, non_blocking=True)
            ready[slot].record(copy_stream)

    for ev in free:
        ev.record(torch.cuda.current_stream(dev))
    start_copy(0)

    def step_e2e():
        cur = state["i"] % 2
        state["i"] += 1
        start_copy(1 - cur)                                 # one host -> device copy of a full batch per step
        torch.cuda.current_stream(dev).wait_event(ready[cur])
        a = dev_bufs[cur][0].detach().requires_grad_(True)
        t = dev_bufs[cur][1].detach().requires_grad_(not lit)
        loss = module(a, t)
        loss.backward()
        free[cur].record(torch.cuda.current_stream(dev))
        loss_host.copy_(loss.detach(), non_blocking=True)

    ms_e2e, _, _, _ = timed(step_e2e, max(2, args.steps // 2), 1)

    # ---- per-kernel durations with CUDA events on the launch stream -----------------------
    # (the library runs its kernels one after the other while this timing is on; one untimed step first)
    sync_all()
    lib.meclip_profile_begin()
    step_resident()
    torch.cuda.synchronize()
    profile_tags(lib)
    lib.meclip_profile_begin()
    prof_steps = 5 if world == 1 else 2
    for _ in range(prof_steps):
        step_resident()
    torch.cuda.synchronize()
    tags = profile_tags(lib)

    if rank != 0:
        if world > 1:
            dist.barrier(device_ids=[local_rank])
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    tflops = flops / (ms_value / 1e3) / 1e12
    dominant = max(tags[:N_TENSOR_TAGS], key=lambda t: t["ms"])
    dom_ms = dominant["ms"] / max(1, dominant["launches"])
    dom_flops = dominant["flops"] / max(1, dominant["launches"])
    achieved = dom_flops / (dom_ms / 1e3) / 1e12 if dom_ms > 0 else 0.0
    roofline = {
        "bound": "tensor", "kernel": "umma_gemm_pair_kernel/" + dominant["kernel"], "achieved": achieved,
        # the kernels are timed inside back-to-back steps under the power cap: the sustained cuBLAS figure is the
        # matching denominator; the fraction of the burst figure is given beside it
        "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"],
        "peak_source": peaks["source"] + " bf16 sustained", "frac_of_burst": achieved / peaks["bf16_tflops"],
        # DRAM read + write bytes per launch of a contraction kernel, from an ncu capture of this kernel at
        # B=16384, D=1152 (0.83 GB per 537 MB coefficient panel), scaled by the launch's work
        "traffic": (0.827e9 * (dom_flops / 6.18e11) if dominant["kernel"] in ("dx_contraction", "dy_contraction")
                    else None),
        "step_frac_of_burst": tflops * (1 if world == 1 else 1.0 / world) / peaks["bf16_tflops"],
        "step_frac_of_sustained": tflops * (1 if world == 1 else 1.0 / world) / peaks["bf16_tflops_sustained"],
        "per_kernel": [dict(t, ms_per_step=t["ms"] / prof_steps,
                            tflops=(t["flops"] / (t["ms"] / 1e3) / 1e12 if t["ms"] > 0 else 0.0))
                       for t in tags[:N_TENSOR_TAGS]],
        # the HBM-bound passes (normalise, transposes, accumulation): algorithmic bytes / CUDA-event time against
        # the measured copy bandwidth
        "hbm_passes": [dict(t, ms_per_step=t["ms"] / prof_steps, gbs=t["bytes"] / (t["ms"] / 1e3) / 1e9,
                            frac_of_hbm_peak=t["bytes"] / (t["ms"] / 1e3) / 1e9 / peaks["hbm_gbs"])
                       for t in tags[N_TENSOR_TAGS:] if t["launches"] > 0 and t["ms"] > 0 and t["bytes"] > 0],
        "hbm_peak_gbs": peaks["hbm_gbs"],
    }

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cb, cd = 8192, d
        val, sec, cores = cpu_dense_step_tflops(cb, cd, temperature, 2)
        cpu = {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "seconds": sec,
               "sample": f"dense fp32 PyTorch CLIP fwd+bwd on host CPU at B={cb}, D={cd} (1/16 of the tile pairs), best of 2"}
        # the smallest benchmark configuration (B = 4096, D = 512) fits the host as a whole: timed as well
        v1, s1, _ = cpu_dense_step_tflops(4096, 512, 0.07, 2)
        cpu["b4096_d512"] = {"value": v1, "unit": "TFLOP/s", "seconds": s1}

    line = {
        "metric": "lit_fwd_bwd_tflops" if lit else "clip_fwd_bwd_tflops", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_value, "ms_per_step_spread": spread, "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, "global_batch": b_global, "feature_dim": d, "temperature": temperature,
                   "normalized_inputs": normalized_inputs, "flop_convention": "6*B^2*D" if lit else "8*B^2*D",
                   "parallelism": "single" if world == 1 else f"ring{world}",
                   "l2": "inputs and workspace larger than L2 (no flush needed)",
                   "samples_per_s": b_global / (ms_value / 1e3),
                   # mean cosine of the positive pairs of rank 0's rows: shows how the synthetic pairs were drawn
                   "mean_diagonal_cosine": diag_cos,
                   **({"executed_flops_per_step": 4.0 * b_global * b_global * (d + 8),
                       "note": "LiT runs in one tile pass (forward contracts E with [Y | 1], backward is a row kernel): "
                               "4*B^2*(D+8) FLOPs are executed for the 6*B^2*D of the two-pass formulation that the "
                               "metric counts"} if lit and world == 1 else {})},
        "roofline": roofline,
        "cpu_baseline": cpu,
        "e2e": {"value": flops / (ms_e2e / 1e3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(host_a.numel() * host_a.element_size() + host_b.numel() * host_b.element_size()) * world,
                "d2h_bytes_per_step": 4 * world},
        "gpu_launches": int(launches) * world,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier(device_ids=[local_rank])
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=None)
    ap.add_argument("--batch", type=int, default=None, help="override the global batch (debugging)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.steps is None:      # long enough for several clock samples, short enough for a default run
        args.steps = 3 if args.impl == "reference" else (100 if args.gpus == 1 else 10)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
