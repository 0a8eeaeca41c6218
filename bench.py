#!/usr/bin/env python
"""Benchmark of the contrastive-loss hot path (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME] [--check-oracle]

N = 1   CLIP fwd+bwd, B=32768, D=1152, bf16, pre-normalised inputs, T=0.07 (the configuration the
        headline metric is quoted on).  One step = one forward + backward over the whole batch.
N > 1   ring-distributed CLIP fwd+bwd, global B=262144, D=1024, bf16, T=0.03, text = normalize(image +
        0.5 noise), normalise inside (launched by torch.distributed.run, one rank per GPU); the global
        batch is fixed, so scaling is "strong".  --config ring_clip_b131072_d768_bf16 selects the
        other ring configuration.

--config also takes clip_b4096_d512_f32 (the smallest configuration) and lit_b32768_d1152_bf16 (LiT: the metric
counts 6*B^2*D, the one-pass route executes 4*B^2*(D+8), see config.note in the line).

The metric is TFLOP/s with the 8*B^2*D convention (forward 2, recompute 2, two gradient
contractions 2+2).  Prints ONE JSON line on rank 0.  Besides the timed legs the line carries
  parity         results of the timed configuration against a checker, outside every timed region:
                 N = 1: sampled gradient rows and the loss against the row-blocked CPU oracle;
                 N > 1: every rank's slice of loss / dX / dY from the ring against the single-GPU
                 kernels run on the all-gathered global batch (max over ranks);
  status_ok      no kernel of any leg gave up a bounded wait (the module path's status word, read
                 after each leg);
  other_configs  ring_clip_b131072_d768_bf16 at this N (at N = 1 the single-GPU module on the
                 whole batch), so that one workload has a point at every N;
  ring_breakdown (N > 1) CUDA-event times of the phases of one ring step;
  reference_gpu  (N = 1) the reference's own Triton modules timed on this GPU in fp32, when its
                 sources were staged under baseline/_ref (baseline/stage_ref.py).
--check-oracle additionally compares with the row-blocked CPU oracle at the configuration's full size
(minutes of host time for the ring configurations).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
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
PARITY_ROWS = [0, 1, 127, 128, 4095, 8191, 8192, 16383, 20000, 32767]
C4 = "ring_clip_b131072_d768_bf16"


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
# CPU arm: the reference's algorithm restated for the host cores (checker code, timed here only)
# --------------------------------------------------------------------------------------------
def cpu_inputs(name: str, batch=None):
    """The configuration's seeded inputs as the loss sees them: fp32, row-normalised."""
    from memoryefficientclip_b200 import synth
    kind, b, d, _dtype, temperature, _normed, _gen = synth.CONFIGS[name]
    b = batch or b
    first, second = synth.make(name, b)
    xn = torch.nn.functional.normalize(first.float(), dim=1)
    yn = torch.nn.functional.normalize(second.float(), dim=1)
    return kind, b, d, temperature, xn, yn


def cpu_sample_rows(b: int, d: int, flop_limit: float) -> int:
    """Rows of the first matrix one timed CPU step works on: all of them when the whole step fits the
    limit, else a multiple of 512 rows against ALL columns (the work per row is the full problem's)."""
    if 8.0 * b * b * d <= flop_limit:
        return b
    return max(512, int(flop_limit / (8.0 * b * d)) // 512 * 512)


def cpu_blocked_step_seconds(xn, yn, temperature, rows):
    from oracle import dense
    t0 = time.perf_counter()
    dense.clip_blocked_step(xn, yn, temperature, row_block=min(4096, rows), rows=rows)
    return time.perf_counter() - t0


def run_reference_arm(args):
    """The reference's loss path is Triton-only and asserts CUDA tensors, so it has no CPU build of its
    own; this arm times the same two-pass algorithm (sums, then recompute + two contractions), restated
    in row blocks with fp32 PyTorch matmuls, on all host cores.  One step = the whole batch when that fits
    a few seconds of host time, otherwise a row sample of it against all columns (stated in `sample`)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    name = args.config or ("clip_b32768_d1152_bf16" if max(world, args.gpus) == 1 else "ring_clip_b262144_d1024_bf16")
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    kind, b, d, temperature, xn, yn = cpu_inputs(name, args.batch)
    rows = cpu_sample_rows(b, d, 1.2e13)
    for _ in range(args.warmup):
        cpu_blocked_step_seconds(xn, yn, temperature, min(rows, 2048))      # warm the thread pool and the pages
    times = []
    t_all0 = time.perf_counter()
    for _ in range(args.steps):
        times.append(cpu_blocked_step_seconds(xn, yn, temperature, rows))
    wall = time.perf_counter() - t_all0
    sec = sum(times) / len(times)
    flops = 8.0 * rows * b * d
    val = flops / sec / 1e12
    whole = rows == b
    sample = (f"row-blocked fp32 CLIP fwd+bwd (the reference's two-pass algorithm) on {cores} host threads, "
              + (f"the whole batch B={b}, D={d} per step" if whole else
                 f"{rows} of the {b} rows against all {b} columns per step ({rows / b:.4f} of the step's work), D={d}"))
    line = {
        "impl": "reference", "metric": "clip_fwd_bwd_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        # time of a WHOLE step of the configuration at the measured rate (the sample scaled up when there is one)
        "ms_per_step": 1e3 * sec * (b / rows), "ms_per_timed_sample": 1e3 * sec,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "global_batch": b, "feature_dim": d, "temperature": temperature,
                   "flop_convention": "8*B^2*D", "device": "host CPU", "rows_per_step": rows},
        "same_config": whole,
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": wall,
        "host": {"cores": cores, "ram_gb": round(os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES") / 2**30, 1)},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# our arm: helpers
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


def status_clear(dev) -> bool:
    """Synchronous read of the module path's status word: True when no kernel gave up a bounded wait."""
    from memoryefficientclip_b200 import _lib, ops
    try:
        ops.check_status(dev)
        return True
    except _lib.MeclipError:
        return False


def errors_vs(got: torch.Tensor, ref: torch.Tensor):
    """(max|got - ref| / max|ref|, cosine) computed on the device in fp32 / fp64 accumulators."""
    g = got.detach().float().flatten()
    r = ref.detach().float().flatten()
    max_rel = float((g - r).abs().max() / r.abs().max().clamp_min(1e-30))
    cos = float(torch.dot(g.double(), r.double()) / (g.double().norm() * r.double().norm()).clamp_min(1e-300))
    return max_rel, cos


def parity_against_oracle(name, loss, gx, gy, b, temperature, normalized_inputs, first, second, rows, lit=False):
    """Loss and sampled gradient rows against the row-blocked CPU oracle (fp32 matmuls, fp64 sums).  `first`,
    `second` are the host copies of the inputs exactly as the GPU saw them (bf16 values upcast)."""
    from oracle import dense
    t0 = time.perf_counter()
    xf, yf = first.float(), second.float()
    if normalized_inputs:
        xn, yn = xf, yf
    else:
        xn, yn = torch.nn.functional.normalize(xf, dim=1), torch.nn.functional.normalize(yf, dim=1)
    rows = sorted({r for r in rows if r < b})
    ref = dense.clip_streaming(xn, yn, temperature, rows, lit=lit)
    want_x, want_y = ref["dx_rows"], ref.get("dy_rows")
    if not normalized_inputs:        # chain the normalise Jacobian onto the oracle's rows
        inv_x = 1.0 / xf.norm(dim=1).clamp_min(1e-12)
        inv_y = 1.0 / yf.norm(dim=1).clamp_min(1e-12)
        want_x = torch.from_numpy(dense.normalize_jacobian_np(xn[rows].double().numpy(), inv_x[rows].double().numpy(),
                                                              want_x.numpy()))
        if want_y is not None:
            want_y = torch.from_numpy(dense.normalize_jacobian_np(yn[rows].double().numpy(),
                                                                  inv_y[rows].double().numpy(), want_y.numpy()))
    dx_rel, dx_cos = dense.grad_errors(gx[rows].float().cpu(), want_x)
    # LiT: the second argument is frozen, there is no second gradient to compare
    dy_rel, dy_cos = dense.grad_errors(gy[rows].float().cpu(), want_y) if want_y is not None else (0.0, 1.0)
    out = {"against": "row_blocked_cpu_oracle", "workload": name, "rows_sampled": len(rows),
           "loss_rel": dense.loss_rel_err(loss, ref["loss"]), "dx_max_rel": dx_rel, "dx_cos": dx_cos,
           "dy_max_rel": dy_rel, "dy_cos": dy_cos, "oracle_seconds": round(time.perf_counter() - t0, 1)}
    out["ok"] = bool(out["loss_rel"] <= dense.LOSS_RTOL and max(dx_rel, dy_rel) <= dense.GRAD_MAX_REL
                     and min(dx_cos, dy_cos) >= dense.GRAD_COS_MIN)
    return out


def reference_on_gpu(b: int, d: int, steps: int = 3):
    """The reference's Triton modules on this GPU, in a child process (see baseline/ref_gpu_step.py)."""
    script = os.path.join(ROOT, "baseline", "ref_gpu_step.py")
    if not os.path.isfile(os.path.join(ROOT, "baseline", "_ref", "clip_loss.py")):
        return {"unavailable": "baseline/_ref/clip_loss.py is not staged (python baseline/stage_ref.py <checkout>)"}
    try:
        proc = subprocess.run([sys.executable, script, str(b), str(d), str(steps)], capture_output=True, text=True,
                              timeout=600, cwd=os.path.join(ROOT, "baseline"))
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference's step did not finish within 600 s"}
    if proc.returncode != 0:
        tail = (proc.stderr or proc.stdout).strip().splitlines()[-1:] or ["no output"]
        return {"unavailable": f"the reference's modules failed here (exit {proc.returncode}): {tail[0][:200]}"}
    for line in reversed(proc.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    return {"unavailable": "no result line from the reference's step"}


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist
    from memoryefficientclip_b200 import _lib, ring, synth
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

    def sync_all():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    def build(name, batch=None):
        """(module, device inputs, pinned host inputs, config tuple) of a configuration at this world size."""
        kind, b_global, d, _dtype, temperature, normalized_inputs, _gen = synth.CONFIGS[name]
        b_global = batch or b_global
        lit = kind == "lit"
        b_local = b_global // world
        first, second = synth.make(name, b_global, row_start=rank * b_local, rows=b_local)
        host_a, host_b = first.pin_memory(), second.pin_memory()
        if world == 1:
            module = (MemoryEfficientLiTLoss if lit else MemoryEfficientCLIPLoss)(temperature, normalized_inputs)
        else:
            module = (RingMemoryEfficientLiTLoss if lit else RingMemoryEfficientCLIPLoss)(temperature, normalized_inputs)
        a_dev = host_a.to(dev).requires_grad_(True)
        t_dev = host_b.to(dev).requires_grad_(not lit)
        return module, a_dev, t_dev, host_a, host_b, (lit, b_global, b_local, d, temperature, normalized_inputs)

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

    name = args.config or ("clip_b32768_d1152_bf16" if world == 1 else "ring_clip_b262144_d1024_bf16")
    module, a_dev, t_dev, host_a, host_b, cfg = build(name, args.batch)
    lit, b_global, b_local, d, temperature, normalized_inputs = cfg
    flops = (6.0 if lit else 8.0) * b_global * b_global * d
    n_probe = min(4096, b_local)
    diag_cos = float(torch.nn.functional.cosine_similarity(host_a[:n_probe].float(), host_b[:n_probe].float(), dim=1).mean())
    status_ok = True

    # ---- leg 1: device-resident inputs (value) ---------------------------------------------------
    last = {}

    def step_resident():
        a_dev.grad = None
        t_dev.grad = None
        loss = module(a_dev, t_dev)
        loss.backward()
        last["loss"] = loss

    ms_value, launches, clocks, spread = timed(step_resident, args.steps, args.warmup, sample_clocks=True)
    status_ok &= status_clear(dev)

    # ---- leg 2: end to end, pinned host -> device, module, loss back to the host (e2e) ------------
    # Timed directly after leg 1 with the same K and W, so both legs see the same clocks and power state.
    # As a training loop would, the copy of the NEXT step's batch runs on a copy stream into the other of two
    # device buffers while this step computes; every step copies a full batch and reads its loss back.
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()
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

    ms_e2e, _, _, spread_e2e = timed(step_e2e, args.steps, args.warmup)
    status_ok &= status_clear(dev)

    # ---- leg 3: the same without any overlap: copy in, step, loss back, wait (e2e_serial) ----------
    def step_serial():
        a = host_a.to(dev, non_blocking=True).requires_grad_(True)
        t = host_b.to(dev, non_blocking=True).requires_grad_(not lit)
        loss = module(a, t)
        loss.backward()
        loss_host.copy_(loss.detach(), non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()

    ms_serial, _, _, _ = timed(step_serial, max(3, args.steps // 4), 1)
    status_ok &= status_clear(dev)
    del dev_bufs

    # ---- per-kernel durations with CUDA events on the launch stream -----------------------
    # The library runs its kernels one after the other while this timing is on.  The pass lasts at least a
    # second of back-to-back steps, i.e. it runs under the power cap like a training loop does, which is the
    # condition the measured SUSTAINED cuBLAS figure stands for; the fraction of the burst figure is given too.
    sync_all()
    lib.meclip_profile_begin()
    step_resident()
    torch.cuda.synchronize()
    profile_tags(lib)
    prof_steps = max(3 if world > 1 else 5, min(200, math.ceil(1000.0 / ms_value)))
    t_prof0 = time.perf_counter()
    lib.meclip_profile_begin()
    for _ in range(prof_steps):
        step_resident()
    torch.cuda.synchronize()
    prof_seconds = time.perf_counter() - t_prof0
    tags = profile_tags(lib)
    if tags[3]["launches"] == 0 and tags[2]["launches"] > 0:
        # both contractions of a block run as ONE launch (booked under the dX tag by the library)
        tags[2]["kernel"] = "contractions_dx_dy_one_launch"
    status_ok &= status_clear(dev)

    # ---- parity of what was timed, outside every timed region --------------------------------
    parity = None
    if not args.no_parity and (world == 1 or not lit):
        loss_val = float(last["loss"].detach())
        if world == 1:
            if rank == 0:
                rows = PARITY_ROWS + ([b_global // 2, b_global - 1] if b_global > 32768 else [])
                parity = parity_against_oracle(name, loss_val, a_dev.grad, t_dev.grad, b_global, temperature,
                                               normalized_inputs, host_a, host_b, rows, lit=lit)
        else:
            # every rank runs the single-GPU kernels on the all-gathered global batch and compares its own slice
            ga = torch.empty(b_global, d, dtype=a_dev.dtype, device=dev)
            gt = torch.empty(b_global, d, dtype=t_dev.dtype, device=dev)
            dist.all_gather_into_tensor(ga, a_dev.detach())
            dist.all_gather_into_tensor(gt, t_dev.detach())
            ga.requires_grad_(True)
            gt.requires_grad_(True)
            single = MemoryEfficientCLIPLoss(temperature, normalized_inputs)
            ref_loss = single(ga, gt)
            ref_loss.backward()
            sl = slice(rank * b_local, (rank + 1) * b_local)
            dx_rel, dx_cos = errors_vs(a_dev.grad, ga.grad[sl])
            dy_rel, dy_cos = errors_vs(t_dev.grad, gt.grad[sl])
            ref_val = float(ref_loss.detach())
            loss_rel = abs(loss_val - ref_val) / max(abs(ref_val), 1e-30)
            worst = torch.tensor([loss_rel, dx_rel, dy_rel, -dx_cos, -dy_cos], dtype=torch.float64, device=dev)
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            w = worst.tolist()
            parity = {"against": "single_gpu_kernels", "workload": name, "ranks": world,
                      "loss_rel": w[0], "dx_max_rel": w[1], "dx_cos": -w[3], "dy_max_rel": w[2], "dy_cos": -w[4],
                      "note": "max over ranks; each rank compares its slice of the ring's loss and gradients with "
                              "the single-GPU kernels on the all-gathered global batch"}
            parity["ok"] = bool(w[0] <= 1e-3 and max(w[1], w[2]) <= 1e-2 and min(-w[3], -w[4]) >= 0.9999)
            if args.check_oracle and rank == 0:
                # the full-size CPU oracle on rank 0's slice (sampled rows): minutes of host time
                rows = [r for r in PARITY_ROWS if r < b_local]
                parity["oracle"] = parity_against_oracle(name, loss_val, a_dev.grad, t_dev.grad, b_global,
                                                         temperature, normalized_inputs, ga.detach().cpu(),
                                                         gt.detach().cpu(), rows)
            del ga, gt, single, ref_loss
            status_ok &= status_clear(dev)
            sync_all()
        if args.check_oracle and world == 1 and rank == 0 and parity is not None:
            parity["note"] = "full-size check: exact loss and sampled gradient rows of both inputs"

    # ---- where one ring step spends its time (N > 1) -------------------------------------------
    ring_breakdown = None
    if world > 1 and not lit:
        sync_all()
        ring.TRACE = []
        ev0 = torch.cuda.Event(enable_timing=True)
        ev0.record()
        step_resident()
        ev1 = torch.cuda.Event(enable_timing=True)
        ev1.record()
        torch.cuda.synchronize()
        trace, ring.TRACE = ring.TRACE, None
        phases = ring.trace_durations(trace)
        ring_breakdown = {"step_ms": ev0.elapsed_time(ev1), "phases_ms": {k: round(v, 4) for k, v in phases.items()},
                          "phases_sum_ms": sum(phases.values()),
                          "note": "rank 0, one step after the timed region; each phase is the time the compute stream "
                                  "spent between two consecutive marks (kernels of a ring step, waiting for the shard "
                                  "or partial-gradient transfer that ran under them, collectives, fp32 accumulation)"}

    # ---- the other ring configuration at this N (one workload with a point at every N) --------
    other = {}
    if not args.no_extras and name != C4 and args.batch is None:
        del module
        torch.cuda.empty_cache()
        m4, a4, t4, _ha, _hb, cfg4 = build(C4)

        def step_c4():
            a4.grad = None
            t4.grad = None
            m4(a4, t4).backward()

        ms4, _, _, spread4 = timed(step_c4, 5, 3)
        status_ok &= status_clear(dev)
        f4 = 8.0 * cfg4[1] * cfg4[1] * cfg4[3]
        other[C4] = {"ms_per_step": ms4, "median_ms": spread4["median"], "value": f4 / (ms4 / 1e3) / 1e12,
                     "unit": "TFLOP/s", "steps": 5, "warmup": 3, "n_gpus": world,
                     "path": "single-GPU module on the whole batch" if world == 1 else f"ring{world}"}
        del m4, a4, t4
        torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.barrier(device_ids=[local_rank])
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    tflops = flops / (ms_value / 1e3) / 1e12
    per_gpu = 1.0 if world == 1 else 1.0 / world
    dominant = max(tags[:N_TENSOR_TAGS], key=lambda t: t["ms"])
    dom_ms = dominant["ms"] / max(1, dominant["launches"])
    dom_flops = dominant["flops"] / max(1, dominant["launches"])
    achieved = dom_flops / (dom_ms / 1e3) / 1e12 if dom_ms > 0 else 0.0
    # DRAM read + write bytes of one contraction launch per FLOP, from the ncu capture summarised under profiles/
    traffic_per_flop = TRAFFIC_BYTES_PER_FLOP.get(dominant["kernel"])
    median_tflops = flops / (spread["median"] / 1e3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": "umma_gemm_pair_kernel/" + dominant["kernel"], "achieved": achieved,
        "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"],
        "peak_source": f"{peaks['source']} bf16 sustained: the per-kernel pass ran {prof_steps} back-to-back steps "
                       f"({prof_seconds:.2f} s, kernels serialised) under the power cap",
        "frac_of_burst": achieved / peaks["bf16_tflops"], "peak_burst": peaks["bf16_tflops"],
        "launch_ms": dom_ms, "launch_flops": dom_flops,
        "traffic": traffic_per_flop * dom_flops if traffic_per_flop else None,
        "traffic_source": TRAFFIC_SOURCE if traffic_per_flop else None,
        # the step as a whole, from the MEDIAN step of the timed region (what a training loop sees)
        "step_frac_of_burst": median_tflops * per_gpu / peaks["bf16_tflops"],
        "step_frac_of_sustained": median_tflops * per_gpu / peaks["bf16_tflops_sustained"],
        "per_kernel": [dict(t, ms_per_step=t["ms"] / prof_steps,
                            tflops=(t["flops"] / (t["ms"] / 1e3) / 1e12 if t["ms"] > 0 else 0.0))
                       for t in tags[:N_TENSOR_TAGS] if t["launches"] > 0],
        # the HBM-bound passes (normalise, transposes, accumulation): algorithmic bytes / CUDA-event time against
        # the measured copy bandwidth
        "hbm_passes": [dict(t, ms_per_step=t["ms"] / prof_steps, gbs=t["bytes"] / (t["ms"] / 1e3) / 1e9,
                            frac_of_hbm_peak=t["bytes"] / (t["ms"] / 1e3) / 1e9 / peaks["hbm_gbs"])
                       for t in tags[N_TENSOR_TAGS:] if t["launches"] > 0 and t["ms"] > 0 and t["bytes"] > 0],
        "hbm_peak_gbs": peaks["hbm_gbs"],
    }

    cpu = None
    ref_gpu = None
    if world == 1 and not args.no_cpu_baseline and not lit:
        # the same row-blocked two-pass step the reference arm times, once, on all host cores
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        _k, cb, cd, ct, xn, yn = cpu_inputs(name, args.batch)
        rows = cpu_sample_rows(cb, cd, 1.2e13)
        cpu_blocked_step_seconds(xn, yn, ct, min(rows, 1024))
        sec = cpu_blocked_step_seconds(xn, yn, ct, rows)
        cpu = {"value": 8.0 * rows * cb * cd / sec / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
               "seconds": sec,
               "sample": (f"row-blocked fp32 two-pass CLIP step on the host CPU, "
                          + ("the whole batch" if rows == cb else f"{rows} of {cb} rows against all columns")
                          + f" (B={cb}, D={cd}), timed once after a short warm-up")}
        del xn, yn
    if world == 1 and not args.no_extras and not lit:
        ref_gpu = reference_on_gpu(b_global, d)

    line = {
        "metric": "lit_fwd_bwd_tflops" if lit else "clip_fwd_bwd_tflops", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_value, "value_median_ms": spread["median"],
        "ms_per_step_spread": spread, "higher_is_better": True,
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
                "median_ms": spread_e2e["median"], "steps": args.steps, "warmup": args.warmup,
                "h2d_bytes_per_step": int(host_a.numel() * host_a.element_size() + host_b.numel() * host_b.element_size()) * world,
                "d2h_bytes_per_step": 4 * world,
                "note": "timed directly after the resident leg; the next batch's copy runs under the current step"},
        "e2e_serial": {"value": flops / (ms_serial / 1e3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_serial,
                       "note": "copy in, step, loss back, host wait: nothing overlaps"},
        "gpu_launches": int(launches) * world,
        "status_ok": bool(status_ok),
        "parity": parity,
        "clocks": clocks,
    }
    if ring_breakdown is not None:
        line["ring_breakdown"] = ring_breakdown
    if other:
        line["other_configs"] = other
    if ref_gpu is not None:
        line["reference_gpu"] = ref_gpu
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier(device_ids=[local_rank])
        dist.destroy_process_group()


# DRAM bytes (read + written) per FLOP of one contraction launch, from the ncu capture under profiles/
TRAFFIC_BYTES_PER_FLOP = {"dx_contraction": 817.4e6 / 6.18475e11, "dy_contraction": 817.9e6 / 6.18475e11,
                          "contractions_dx_dy_one_launch": 1641.0e6 / 1.23695e12}
TRAFFIC_SOURCE = ("ncu capture of the contractions at the step's own block shape (16384 x 16384 block, D=1152: 1641 MB "
                  "for dX and dY in one launch, 818 MB for either alone; "
                  "profiles/umma_gemm_pair_kernel_contractions_block16384_d1152_ncu_full.md); other shapes: scaled by FLOPs")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=None)
    ap.add_argument("--batch", type=int, default=None, help="override the global batch (debugging)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the parity block")
    ap.add_argument("--no-extras", action="store_true", help="skip other_configs and reference_gpu (quick A/B runs)")
    ap.add_argument("--check-oracle", action="store_true",
                    help="N > 1: also compare rank 0's slice with the full-size CPU oracle (minutes of host time)")
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
