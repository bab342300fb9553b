#!/usr/bin/env python
"""Benchmark of the HAT GEMM(+ReLU) hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

Workload (the configuration the headline metric is quoted on): bf16 GEMM + fused
ReLU, M=65536, N=8192, K=8192, A ~ N(0,1) row-major split by M-row blocks over
the GPUs, B ~ N(0, 1/sqrt(K)) column-major replicated, fp32 accumulate, bf16 C
reassembled on every GPU with an NCCL all-gather.  One step = one pass over the
whole problem.  `value` is whole-job TFLOP/s (2*M*N*K / step time) with inputs
resident in HBM; `e2e` is the same metric through the C ABI with HOST buffers
(host->device copies of A, B, C and the device->host copy of C inside the timed
region).  Under torchrun (N > 1) every rank runs this file; rank 0 prints the line.

`--impl reference` times the CPU oracle (the restatement of the reference's
HOST-target loop nest, all host threads) on a bounded slice of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, N, K = 65536, 8192, 8192
FLOPS = 2.0 * M * N * K
METRIC = "gemm_bf16_relu_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "sharded bf16 GEMM+ReLU M=65536 N=8192 K=8192 (A row-major by M-row blocks, B col-major replicated, bf16 C all-gathered)"


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel on one GPU's shard of this
# workload, from ncu captures of `python -m accera_b200.profile_cases gemm_bf16 --m <rows per GPU>` (one capture per
# shard size; a bench run cannot measure it itself, ncu has to replay the launch).  Keyed by (compute, GPUs).
NCU_TRAFFIC_BYTES = {("tensor_2sm", 1): 12.75e9, ("tensor_2sm", 2): 6.42e9, ("tensor_2sm", 4): 3.14e9, ("tensor_2sm", 8): 1.52e9}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def wait_ready(self, timeout: float = 5.0) -> bool:
        """Blocks until nvidia-smi has delivered its first sample (it needs a few hundred ms to start, longer than
        a short timed region lasts)."""
        t_end = time.time() + timeout
        while self.proc is not None and not self.lines and time.time() < t_end and self.proc.poll() is None:
            time.sleep(0.01)
        return bool(self.lines)

    def mark(self):
        return time.time()

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        for ts, line in self.lines:
            if t0 is not None and not (t0 - 0.02 <= ts <= t1 + 0.03):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"], "samples": 0}
        busy = [c for c, p in zip(sm, power) if p > 250.0] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


# ---------------------------------------------------------------------------
# the reference arm / CPU baseline: the oracle on the host cores
# ---------------------------------------------------------------------------

def host_threads() -> int:
    """Threads for the CPU arm: every core this process may run on.  (Not OMP_NUM_THREADS: torchrun sets that to 1
    for its children, which would time the baseline on a single core.)"""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_gemm_sample(rows: int, threads: int, seed: int = 1005):
    """Times the oracle (fast-math build, `threads` threads) on `rows` rows of the workload; returns seconds."""
    import numpy as np
    import oracle
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((rows, K), dtype=np.float32)
    bt = rng.standard_normal((N, K), dtype=np.float32)
    bt *= np.float32(1.0 / np.sqrt(K))
    a16 = oracle.f32_to_bf16_bits(a)
    b16 = oracle.f32_to_bf16_bits(bt).T                 # [K, N] column-major view
    c16 = np.zeros((rows, N), dtype=np.uint16)
    af, bf = oracle.bf16_bits_to_f32(a16), oracle.bf16_bits_to_f32(b16)   # widening is not part of the timed GEMM
    t0 = time.perf_counter()
    oracle.gemm(af, bf, c16, out_kind="bfloat16", beta=1.0, relu=True, fast=True, threads=threads)
    return time.perf_counter() - t0


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    import oracle
    oracle.build()
    threads = host_threads()
    rows = 64
    t = cpu_gemm_sample(rows, threads)                   # calibration, untimed
    target = 3.0                                         # seconds per step
    rows = int(max(16, min(8192, rows * target / max(t, 1e-3))))
    rows -= rows % 16
    for _ in range(args.warmup if args.warmup < 2 else 1):
        cpu_gemm_sample(rows, threads)
    times = [cpu_gemm_sample(rows, threads) for _ in range(args.steps)]
    per_step = statistics.mean(times)
    tflops = 2.0 * rows * N * K / per_step / 1e12
    sample = f"{rows} of {M} rows per step (same N, K), oracle -O3 -ffast-math, {threads} threads (nproc {os.cpu_count()})"
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3 * (M / rows), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------

def build_workload_package(rows: int, out_dir: str, name: str):
    """The benchmarked function as a HAT package: `C += A @ B` over (rows, N, K) in bf16 with a fused ReLU, B
    column-major, tensorized plan for the B200 target - built with accera_b200.Package and loaded with
    accera_b200.hat.load, the call a user of the reference makes (Package.build + hatlib.load)."""
    import accera_b200 as acc
    from accera_b200 import hat
    A = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.bfloat16, shape=(rows, K))
    B = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.bfloat16, shape=(K, N), layout=acc.Array.Layout.LAST_MAJOR)
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=acc.ScalarType.bfloat16, shape=(rows, N))
    nest = acc.Nest((rows, N, K))
    i, j, k = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[i, j] += A[i, k] * B[k, j]
    plan = nest.create_schedule().create_plan(acc.Target(acc.Target.Model.NVIDIA_B200))
    plan.tensorize(indices=(i, j, k), mma_shape=acc.MMAShape.M16xN16xK16_B1, epilogue_op=acc.MMAFragmentOp.ReLU)
    pkg = acc.Package()
    fn = pkg.add(plan, args=(A, B, C), base_name="matmul_relu_bf16")
    files = pkg.build(name, format=acc.Package.Format.HAT_DYNAMIC, output_dir=out_dir)
    _, fns = hat.load(files[0])
    return fns[fn.name]


def verify_rows_against_oracle(a_rows_dev, b_dev, c_rows_dev, what: str):
    """Checks rows of the result (computed from C = 0: relu(A @ B) rounded to bf16) against the CPU oracle on the
    same bytes, at the tolerance stated for the tensor-core GEMM (2e-2 of max(|want|, |A| @ |B|)).  Outside any timed
    region."""
    import numpy as np
    import torch
    import oracle
    oracle.build()
    a = a_rows_dev.cpu().view(torch.int16).numpy().view(np.uint16)
    b = b_dev.t().contiguous().cpu().view(torch.int16).numpy().view(np.uint16).T        # [K, N] column-major view
    got = oracle.bf16_bits_to_f32(c_rows_dev.cpu().view(torch.int16).numpy().view(np.uint16)).astype(np.float64)
    want_bits = oracle.gemm(a, b, np.zeros((a.shape[0], N), np.uint16), in_kind="bfloat16", out_kind="bfloat16", beta=0.0,
                            relu=True, threads=host_threads())
    want = oracle.bf16_bits_to_f32(want_bits).astype(np.float64)
    scale = np.abs(oracle.bf16_bits_to_f32(a).astype(np.float64)) @ np.abs(oracle.bf16_bits_to_f32(b).astype(np.float64))
    err = np.abs(got - want)
    ok = bool((err <= 2e-2 * np.maximum(np.abs(want), scale)).all())
    if not ok:
        raise SystemExit(f"{what}: result differs from the oracle (max err {err.max():.4g})")
    return {"rows_checked": int(a.shape[0]), "max_abs_err": float(err.max()), "tolerance": "2e-2 * max(|want|, |A|@|B|)",
            "against": "CPU oracle (oracle/hat_oracle.c) on the same bytes"}


def sustained_loop(fn, seconds, device, dist_on, sampler_index, per_step_flops, sample=True):
    """Repeats `fn` for at least `seconds` (the burst figure above comes from a region of tens of milliseconds, in
    which the GPU has not reached its power-capped clock yet) and samples the clocks over that window."""
    import torch
    import torch.distributed as dist
    sampler = ClockSampler(sampler_index) if sample else None
    if sampler is not None:
        sampler.start()
        sampler.wait_ready()
    torch.cuda.synchronize(device)
    if dist_on:
        dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # calibrate with 3 steps, then run the number of steps that fills the window (the same on every rank)
    c0 = time.perf_counter()
    for _ in range(3):
        fn()
    torch.cuda.synchronize(device)
    per = max((time.perf_counter() - c0) / 3, 1e-5)
    steps = int(min(20000, max(10, seconds / per)))
    if dist_on:
        t = torch.tensor([steps], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        steps = int(t.item())
        dist.barrier()
    torch.cuda.synchronize(device)
    w0 = time.time()
    s.record()
    for _ in range(steps):
        fn()
    e.record()
    torch.cuda.synchronize(device)
    w1 = time.time()
    ms = s.elapsed_time(e) / steps
    if dist_on:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop(w0 + 0.3, w1) if sampler is not None else {}      # leave out the ramp at the start of the window
    out = {"seconds": w1 - w0, "steps": steps, "ms_per_step": ms, "value": per_step_flops / (ms * 1e-3) / 1e12, "unit": UNIT,
           "clocks": clocks}
    if clocks.get("sm_mhz"):
        out["ms_times_sm_mhz"] = ms * clocks["sm_mhz"]
    return out


def make_inputs(plan, rank, device):
    """Seeded inputs generated on the host with numpy (the bytes the oracle would see), then moved to HBM."""
    import numpy as np
    import torch
    rng = np.random.default_rng(1005)
    bt = rng.standard_normal((N, K), dtype=np.float32)
    bt *= np.float32(1.0 / np.sqrt(K))
    b_dev = torch.from_numpy(bt).to(device).to(torch.bfloat16).t()          # [K, N] column-major view
    del bt
    # A: each rank generates only its own rows, block by block, from per-block seeds
    parts = []
    for j in range(plan.chunks):
        blk = plan.block_of(rank, j)
        r = np.random.default_rng(2000 + blk)
        rows_left = plan.block_rows
        while rows_left > 0:
            step = min(rows_left, 4096)
            parts.append(torch.from_numpy(r.standard_normal((step, K), dtype=np.float32)).to(device).to(torch.bfloat16))
            rows_left -= step
    a_dev = torch.cat(parts, dim=0)
    del parts
    return a_dev, b_dev


def timed_steps(fn, steps, warmup, device, dist_on):
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    from accera_b200 import runtime as _rt
    wall0 = time.time()
    n0 = _rt.launch_count()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    launches = _rt.launch_count() - n0
    torch.cuda.synchronize(device)
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize(device)
    wall1 = time.time()
    ms = start.elapsed_time(end)
    if dist_on:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps, wall0, wall1, launches


def extras_single_gpu(device, peaks, local_rank=0):
    """The other configurations (N = 1 only), reported beside the headline: device-timed with the inputs in HBM
    (rotating buffer sets larger than L2, at least half a second per configuration so that the clock sampler sees
    the kernel), end to end through the C ABI on host arrays, and the CPU port of the reference's nest on the host cores."""
    import numpy as np
    import torch
    import oracle
    from accera_b200 import runtime as rt
    oracle.build()
    threads = host_threads()
    out = {}

    def timeit(fns, min_seconds=0.5, batch=20, warm=4):
        """Mean launch duration: batches of `batch` back-to-back launches between CUDA-event pairs on the launching
        stream until `min_seconds` have passed.  `fns` rotates over distinct buffer sets that together exceed L2, so
        every launch starts with its inputs out of cache.  Also returns the clocks sampled over the window."""
        for i in range(warm):
            fns[i % len(fns)]()
        torch.cuda.synchronize(device)
        sampler = ClockSampler(local_rank)
        sampler.start()
        sampler.wait_ready()
        pairs = []
        k = 0
        w0 = time.time()
        t_end = time.perf_counter() + min_seconds
        while time.perf_counter() < t_end or len(pairs) < 3:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(batch):
                fns[k % len(fns)]()
                k += 1
            e.record()
            pairs.append((s, e))
            if len(pairs) % 8 == 0:
                torch.cuda.synchronize(device)
        torch.cuda.synchronize(device)
        w1 = time.time()
        rt.synchronize()
        means = [s.elapsed_time(e) * 1e-3 / batch for s, e in pairs]
        clocks = sampler.stop(w0 + 0.1, w1)
        return statistics.mean(means), min(means), clocks

    def host_time(fn, reps=3):
        fn()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        return (time.perf_counter() - t0) / reps

    # ---- reduce_mean over the last axis of X[8192, 4096] ------------------------------------------------------
    x_host = oracle.inputs_reduce_mean(8192, 4096)
    xs = [torch.from_numpy(x_host).to(device).reshape(1, 8192, 4096)] + [torch.randn(1, 8192, 4096, device=device) for _ in range(3)]
    y = torch.empty(8192, device=device)
    t, tmin, clocks = timeit([(lambda x=x: rt.reduce_mean_rank3(x, y, [2])) for x in xs])
    b = 8192 * 4096 * 4 + 8192 * 4
    y_host = np.empty(8192, np.float32)
    x3 = x_host.reshape(1, 8192, 4096)
    t_e2e = host_time(lambda: rt.reduce_mean_rank3(x3, y_host, [2]))
    t_cpu = host_time(lambda: oracle.reduce_mean_last_axis(x_host, fast=True, threads=threads), reps=2)
    out["reduce_mean_f32_8192x4096"] = {
        "us": t * 1e6, "us_min_of_means": tmin * 1e6, "GB/s": b / t / 1e9, "frac_hbm": b / t / 1e9 / peaks["hbm_gbs"],
        "algorithmic_bytes": b, "clocks": clocks, "e2e_us_host_arrays": t_e2e * 1e6,
        "cpu_port": {"us": t_cpu * 1e6, "GB/s": b / t_cpu / 1e9, "cores": threads, "sample": "full size"}}
    del xs, y
    # ---- gather of 16384 rows of T[32000, 4096] -------------------------------------------------------------
    T_host, idx_host = oracle.inputs_gather(32000, 4096, 16384)
    T = torch.from_numpy(T_host).to(device)                                       # 500 MiB table, 256 MiB out
    idxs = [torch.from_numpy(idx_host).to(device), torch.randint(0, 32000, (16384, 1), device=device)]
    outs = [torch.empty(16384, 1, 4096, device=device) for _ in range(2)]
    t, tmin, clocks = timeit([(lambda i=i, o=o: rt.gather_rank2(T, i, o, 0)) for i, o in zip(idxs, outs)])
    b = 2 * 16384 * 4096 * 4 + 16384 * 8
    unique_rows = int(torch.unique(idxs[0]).numel())
    b_dram = (unique_rows + 16384) * 4096 * 4 + 16384 * 8        # every distinct table row once + indices + the output
    o_host = np.empty((16384, 1, 4096), np.float32)
    t_e2e = host_time(lambda: rt.gather_rank2(T_host, idx_host, o_host, 0), reps=2)
    t_cpu = host_time(lambda: oracle.gather_rank2(T_host, idx_host, 0, fast=True, threads=threads), reps=2)
    out["gather_f32_32000x4096_idx16384"] = {
        "us": t * 1e6, "us_min_of_means": tmin * 1e6, "GB/s": b / t / 1e9, "frac_hbm": b / t / 1e9 / peaks["hbm_gbs"],
        "algorithmic_bytes": b, "GB/s_dram_moved": b_dram / t / 1e9, "frac_hbm_dram_moved": b_dram / t / 1e9 / peaks["hbm_gbs"],
        "dram_moved_bytes": b_dram, "distinct_rows": unique_rows,
        "note": "algorithmic bytes count a table row once per index that names it; duplicates are served by L2, so DRAM moves fewer",
        "clocks": clocks, "e2e_us_host_arrays": t_e2e * 1e6,
        "cpu_port": {"us": t_cpu * 1e6, "GB/s": b / t_cpu / 1e9, "cores": threads, "sample": "full size"}}
    del T, idxs, outs, T_host, o_host
    # ---- range ---------------------------------------------------------------------------------------------
    n_range = 1 << 27                                                            # 512 MiB written per launch
    rbuf = torch.empty(n_range, device=device)
    t, tmin, clocks = timeit([lambda: rt.range_f32(rbuf, 0.0, 0.001)])
    out["range_f32_2^27"] = {"us": t * 1e6, "GB/s": n_range * 4 / t / 1e9, "frac_hbm": n_range * 4 / t / 1e9 / peaks["hbm_gbs"],
                             "clocks": clocks}
    del rbuf
    # ---- quickstart fp32 matmul + ReLU, 512^3 ------------------------------------------------------------------
    a1, b1, c1 = oracle.inputs_matmul_relu_f32()
    A1, B1, C1 = (torch.from_numpy(v).to(device) for v in (a1, b1, c1))
    t, tmin, clocks = timeit([lambda: rt.gemm(A1, B1, C1, relu=True, compute="simt")], batch=50)   # 3 MiB: L2 resident by nature
    c1_host = c1.copy()
    t_e2e = host_time(lambda: rt.gemm(a1, b1, c1_host, relu=True, compute="simt"))
    t_cpu = host_time(lambda: oracle.gemm(a1, b1, c1.copy(), relu=True, fast=True, threads=threads))
    t_cpu1 = host_time(lambda: oracle.gemm(a1, b1, c1.copy(), relu=True, fast=True, threads=1))
    out["matmul_relu_f32_simt_512"] = {
        "us": t * 1e6, "us_min_of_means": tmin * 1e6, "TFLOP/s": 2 * 512 ** 3 / t / 1e12, "clocks": clocks,
        "e2e_us_host_arrays": t_e2e * 1e6,
        "cpu_port": {"us": t_cpu * 1e6, "TFLOP/s": 2 * 512 ** 3 / t_cpu / 1e12, "cores": threads, "us_single_thread": t_cpu1 * 1e6,
                     "sample": "full size"}}
    # ---- fp16 -> fp32 4096^3 + ReLU ----------------------------------------------------------------------------
    A = (torch.rand(4096, 4096, device=device) * 2 - 1).half(); B = (torch.rand(4096, 4096, device=device) * 2 - 1).half().t()
    C = torch.zeros(4096, 4096, device=device)
    t, tmin, clocks = timeit([lambda: rt.gemm(A, B, C, relu=True, compute="tensor_2sm")], batch=10)
    a3, b3, c3 = oracle.inputs_gemm_f16(64, 4096, 4096)
    t_cpu = host_time(lambda: oracle.gemm(a3, b3, c3.copy(), relu=True, fast=True, threads=threads), reps=2)
    out["gemm_f16_f32acc_relu_4096"] = {
        "us": t * 1e6, "us_min_of_means": tmin * 1e6, "TFLOP/s": 2 * 4096 ** 3 / t / 1e12,
        "frac_bf16_peak": 2 * 4096 ** 3 / t / 1e12 / peaks["bf16_tflops"], "clocks": clocks,
        "cpu_port": {"TFLOP/s": 2 * 64 * 4096 * 4096 / t_cpu / 1e12, "cores": threads, "sample": "64 of 4096 rows, extrapolates linearly"}}
    # ---- int8 -> int32 8192^3 ----------------------------------------------------------------------------------
    A = torch.randint(-128, 128, (8192, 8192), device=device, dtype=torch.int8)
    B = torch.randint(-128, 128, (8192, 8192), device=device, dtype=torch.int8).t()
    C = torch.zeros(8192, 8192, device=device, dtype=torch.int32)
    t, tmin, clocks = timeit([lambda: rt.gemm(A, B, C, compute="tensor_2sm")], batch=10)
    entry = {"us": t * 1e6, "us_min_of_means": tmin * 1e6, "TOP/s": 2 * 8192 ** 3 / t / 1e12, "clocks": clocks,
             "frac_nominal_int8_peak(2x measured bf16)": 2 * 8192 ** 3 / t / 1e12 / (2 * peaks["bf16_tflops"])}
    try:
        # the library int8 GEMM on the same operands, as a measured ceiling for this box (comparator only)
        tl, tlmin, _ = timeit([lambda: torch._int_mm(A, B)], batch=10, min_seconds=0.3)
        entry["library_int8_TOP/s(torch._int_mm)"] = 2 * 8192 ** 3 / tl / 1e12
        entry["frac_of_library_int8"] = tl / t
    except Exception as exc:
        entry["library_int8"] = f"not measured: {exc!r}"
    a4, b4, c4 = oracle.inputs_gemm_s8(32, 8192, 8192)
    t_cpu = host_time(lambda: oracle.gemm(a4, b4, c4.copy(), fast=True, threads=threads), reps=2)
    entry["cpu_port"] = {"TOP/s": 2 * 32 * 8192 * 8192 / t_cpu / 1e12, "cores": threads, "sample": "32 of 8192 rows, extrapolates linearly"}
    out["gemm_s8_s32_8192"] = entry
    try:
        # the 512^3 launches replayed from a CUDA graph: at ~10 us per launch the Python / driver launch path
        # above is slower than the kernel, the graph shows the device time
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            rt.gemm(A1, B1, C1, relu=True, compute="simt")          # first call on this stream: allocates its split-K workspace
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(20):
                    rt.gemm(A1, B1, C1, relu=True, compute="simt")
            graph.replay()
            torch.cuda.synchronize(device)
            s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_ev.record(side)
            for _ in range(5):
                graph.replay()
            e_ev.record(side)
            torch.cuda.synchronize(device)
            tg = s_ev.elapsed_time(e_ev) * 1e-3 / 100
        out["matmul_relu_f32_simt_512"].update({"us_cuda_graph": tg * 1e6, "TFLOP/s_cuda_graph": 2 * 512 ** 3 / tg / 1e12})
    except Exception as exc:                                   # reported beside the number, never fatal
        out["matmul_relu_f32_simt_512"]["cuda_graph"] = f"not measured: {exc!r}"
    return out


def run_ours(args, rank: int, world: int, local_rank: int):
    import numpy as np
    import torch
    import torch.distributed as dist
    from accera_b200 import runtime as rt
    from accera_b200.sharded import RowBlockPlan, ShardedGemm

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback (use --impl reference for the CPU arm)")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist_on = world > 1
    if dist_on:
        dist.init_process_group("nccl", device_id=device)
    peaks = load_peaks()
    plan = RowBlockPlan.choose(M, world, max_chunks=(1 if args.gather == "fused" and args.chunks_default else args.chunks))
    a_dev, b_dev = make_inputs(plan, rank, device)
    gather = args.gather if dist_on else "nccl"
    c_full = ShardedGemm.allocate_c(M, N, torch.bfloat16, device, gather=gather)
    compute = args.compute

    # with several GPUs, leave a few SMs to the all-gather kernels of the previous chunk (they cannot share an
    # SM with a GEMM CTA, which holds almost all of its shared memory)
    max_ctas = 0
    if dist_on and gather == "nccl" and args.comm_sms > 0:
        max_ctas = max(2, torch.cuda.get_device_properties(device).multi_processor_count - args.comm_sms)

    # beta = 1: the HAT function is "C += A @ B, then ReLU" with C INPUT_OUTPUT
    gemm_kwargs = dict(beta=1.0, relu=True, compute=compute, max_ctas=max_ctas)

    def gemm_fn(a, b, c):
        rt.gemm(a, b, c, **gemm_kwargs)

    sg = ShardedGemm(plan, rank, gemm_fn=gemm_fn, gather=gather, gemm_kwargs=gemm_kwargs)

    def step():
        # C starts as zeros and is INPUT_OUTPUT: every step reads it, adds A @ B, applies the ReLU and writes
        # it back (then all-gathers it).  It is not re-zeroed between steps: that is input preparation, not
        # the hot path, and the work per step does not depend on C's values.
        sg.run(a_dev, b_dev, c_full)

    # one untimed step from C = 0, then rows of the result against the CPU oracle: at one GPU rows of the benchmarked
    # launch itself (first tile row, one deep in the paced part of the launch, the last rows); with several GPUs rows
    # of a block that ANOTHER rank computed and that reached this GPU through the gather
    step()
    torch.cuda.synchronize(device)
    verified = None
    if dist_on:
        other = (rank + 1) % world
        j = plan.chunks - 1
        g0, g1 = plan.global_row_range(other, j)
        r = np.random.default_rng(2000 + plan.block_of(other, j))
        rows = 16
        a_blk = torch.from_numpy(r.standard_normal((rows, K), dtype=np.float32)).to(device).to(torch.bfloat16)
        check = verify_rows_against_oracle(a_blk, b_dev, c_full[g0:g0 + rows], f"rank {rank}: gathered block of rank {other}")
        ok = torch.tensor([1.0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        verified = bool(ok.item() == 1.0)
        del a_blk
    else:
        idx = torch.cat([torch.arange(0, 8), torch.arange(137 * 256 + 40, 137 * 256 + 48), torch.arange(M - 8, M)]).to(device)
        check = verify_rows_against_oracle(a_dev[idx], b_dev, c_full[idx], "benchmarked launch")
    c_full.zero_()
    torch.cuda.synchronize(device)
    if dist_on:
        dist.barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.wait_ready()
    if dist_on:
        dist.barrier()
    ms_per_step, wall0, wall1, gpu_launches = timed_steps(step, args.steps, args.warmup, device, dist_on)
    rt.synchronize()
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    value = FLOPS / (ms_per_step * 1e-3) / 1e12
    sustained = None
    if args.sustained_s > 0:
        sustained = sustained_loop(step, args.sustained_s, device, dist_on, local_rank, FLOPS, sample=(rank == 0))
        rt.synchronize()

    # kernel-only time of the dominant kernel (this rank's GEMM launches), CUDA events on the launching stream
    def gemm_only():
        for j in range(plan.chunks):
            l0, l1 = plan.local_row_range(j)
            g0, g1 = plan.global_row_range(rank, j)
            gemm_fn(a_dev[l0:l1], b_dev, c_full[g0:g1])
    if dist_on:
        kernel_ms, _, _, _ = timed_steps(gemm_only, args.steps, 1, device, dist_on)
    else:
        # one GPU: a step IS one launch of the kernel (no gather), so the timed region above - CUDA events on the
        # launching stream around exactly `steps` launches - is the kernel's average launch duration; a second
        # loop would only sample a different point of the GPU's power / clock state
        kernel_ms = ms_per_step
    kernel_tflops = (FLOPS / world) / (kernel_ms * 1e-3) / 1e12

    # end to end through the C ABI with host buffers (pinned): H2D of A, B, C; GEMM; D2H of C
    rows_local = plan.rows_per_rank
    a_host = torch.empty(rows_local, K, dtype=torch.bfloat16).pin_memory()
    a_host.copy_(a_dev)
    b_host = torch.empty(N, K, dtype=torch.bfloat16).pin_memory()
    b_host.copy_(b_dev.t())
    c_host = torch.zeros(rows_local, N, dtype=torch.bfloat16).pin_memory()
    a_np = a_host.view(torch.int16).numpy().view(np.uint16)
    b_np = b_host.view(torch.int16).numpy().view(np.uint16).T          # [K, N] column-major view
    c_np = c_host.view(torch.int16).numpy().view(np.uint16)
    del c_full
    torch.cuda.empty_cache()

    import tempfile
    pkg_dir = tempfile.mkdtemp(prefix=f"accb_bench_r{rank}_")
    hat_fn = build_workload_package(rows_local, pkg_dir, f"bench_pkg_r{rank}")

    def e2e_step():
        # the plugin call: the function of the built HAT package, host arrays in, host array out; the library stages
        # them through the GPU named by device_id (copies in both directions inside the call)
        hat_fn(a_np, b_np, c_np, device_id=local_rank)

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    if dist_on:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize(device)
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if dist_on:
        t = torch.tensor([e2e_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = FLOPS / e2e_s / 1e12
    h2d = world * (rows_local * K * 2 + N * K * 2 + rows_local * N * 2)
    d2h = world * rows_local * N * 2
    rt.release_workspace()
    import shutil
    shutil.rmtree(pkg_dir, ignore_errors=True)

    extras = None
    cpu_baseline = None
    if rank == 0 and world == 1:
        if not args.no_extras:
            del a_dev
            torch.cuda.empty_cache()
            extras = extras_single_gpu(device, peaks, local_rank)
        try:
            import oracle
            oracle.build()
            threads = host_threads()
            rows = 64
            t = cpu_gemm_sample(rows, threads)
            rows = int(max(16, min(4096, rows * 10.0 / max(t, 1e-3))))
            rows -= rows % 16
            t = cpu_gemm_sample(rows, threads)
            cpu_baseline = {"value": 2.0 * rows * N * K / t / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
                            "sample": f"{rows} of {M} rows (same N, K), oracle -O3 -ffast-math, {threads} threads, {t:.1f} s"}
        except Exception as exc:       # the baseline is reported, never required for the GPU numbers
            cpu_baseline = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"failed: {exc!r}"}

    if rank == 0:
        peak = peaks["bf16_tflops"]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "m": M, "n": N, "k": K, "compute": compute,
                       "row_blocks": f"{plan.world * plan.chunks} blocks of {plan.block_rows} rows, block-cyclic",
                       "chunks": plan.chunks, "gather": gather if dist_on else "none", "gemm_ctas": (max_ctas or "all SMs"), "l2": "inputs larger than L2 (A shard >= 128 MiB, B 128 MiB, C 1 GiB)",
                       "beta": 1.0, "peaks": peaks["source"]},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                    "through": "accera_b200.Package.build -> hat.load(...)[name](A, B, C) on pinned host arrays"},
            "verified": check,
            "gpu_launches": gpu_launches,
            "roofline": {"bound": "tensor", "achieved": kernel_tflops,
                         "peak": peak, "unit": "TFLOP/s", "frac": kernel_tflops / peak,
                         "frac_of_sustained_peak": (kernel_tflops / peaks["bf16_tflops_sustained"]) if peaks.get("bf16_tflops_sustained") else None,
                         "traffic": NCU_TRAFFIC_BYTES.get((compute, world)),
                         "traffic_note": "ncu, one launch of this GPU's shard without replicas (DRAM bytes read + written)",
                         "nvlink_bytes_out_per_gpu_per_step": (world - 1) * plan.rows_per_rank * N * 2 if dist_on else 0,
                         "kernel": "gemm_umma_kernel<bf16,cta_group::2>" if compute == "tensor_2sm" else "gemm_umma_kernel<bf16>",
                         "per": "GPU", "peak_source": peaks["source"] + " burst bf16 (cuBLAS)"},
            "cpu_baseline": cpu_baseline,
        }
        if verified is not None:
            line["gather_verified"] = verified
        if sustained is not None:
            sp = peaks.get("bf16_tflops_sustained")
            sustained["frac_of_sustained_peak_per_gpu"] = (sustained["value"] / world / sp) if sp else None
            line["sustained"] = sustained
        if extras is not None:
            line["other_configs"] = extras
        print(json.dumps(line), flush=True)
    if dist_on:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--compute", default="tensor_2sm", choices=["tensor", "tensor_2sm"])
    ap.add_argument("--chunks", type=int, default=4, help="row-block rounds per rank for GEMM / all-gather overlap (N > 1)")
    ap.add_argument("--gather", default="fused", choices=["nccl", "copy_engine", "fused"],
                    help="how C is reassembled for N > 1: NCCL all-gather, DMA pushes into symmetric memory, or "
                         "stores to every GPU's C from the GEMM epilogue itself")
    ap.add_argument("--comm-sms", type=int, default=16, help="SMs the GEMM leaves to the concurrent all-gather (N > 1)")
    ap.add_argument("--no-extras", action="store_true", help="skip the device-timed numbers of the other configurations")
    ap.add_argument("--sustained-s", type=float, default=2.0,
                    help="after the timed steps, repeat the step for this many seconds and report the sustained figure "
                         "with the clocks over that window (0 = skip)")
    args = ap.parse_args()
    args.chunks_default = "--chunks" not in " ".join(sys.argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1 and args.impl == "ours":
        # convenience: `python bench.py --gpus N` re-launches itself under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29541"), __file__] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3                                   # timing rule: at least 3 warm-up steps
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.gpus = world
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
