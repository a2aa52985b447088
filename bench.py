#!/usr/bin/env python
"""Benchmark of the B200 decode hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Workload `q4_matvec` (BASELINE config 0): one fused Q4 dequantize-matvec, weight 17408x5120 in
the packed Q4_B64 format (codes uniform, f16 block scales log-normal mu=-4 sigma=0.5), f32
activation ~N(0,1), fp32 accumulate. A step is one matvec; `value` is algorithmic bytes per
second (packed weights + activation + output, 47 439 872 B per matvec). Eight distinct weight
replicas (379 MB > 2x the 126 MB L2) are rotated so that every step streams from HBM.

`--impl reference` times the reference's CPU path (the C restatement of backend/cpu.rs in
oracle/, AVX2 arm, rows split over all host threads) on the same configuration.
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

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

Q4_ROWS, Q4_COLS = 17408, 5120
ALGO_BYTES = Q4_ROWS * (Q4_COLS // 64) * 34 + Q4_COLS * 4 + Q4_ROWS * 4  # 47 439 872
REPLICAS = 8


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([p.strip() for p in line.split(",")])

    def stop(self):
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
        for s in self.samples:
            if len(s) < 6:
                continue
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_baseline(threads: int, avx2: bool, repeats: int):
    """Times the oracle port of CpuBackend::fused_matvec on the whole config-0 Q4 matvec."""
    import oracle
    from ctox_llm_b200 import synthetic
    w = synthetic.packed_weights(oracle.Q4B64, Q4_ROWS, Q4_COLS, 0)
    x = synthetic.activations(Q4_COLS, 0)
    op = oracle.FusedMatVec(oracle.Q4B64, w, Q4_ROWS, Q4_COLS, x)
    oracle.fused_matvec(op, threads=threads, avx2=avx2)  # warm-up
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.fused_matvec(op, threads=threads, avx2=avx2)
        times.append(time.perf_counter() - t0)
    return ALGO_BYTES / statistics.median(times) / 1e9, statistics.median(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    # each step is one full matvec on the host; warm-up inside cpu_baseline
    times = []
    import oracle
    from ctox_llm_b200 import synthetic
    w = synthetic.packed_weights(oracle.Q4B64, Q4_ROWS, Q4_COLS, 0)
    x = synthetic.activations(Q4_COLS, 0)
    op = oracle.FusedMatVec(oracle.Q4B64, w, Q4_ROWS, Q4_COLS, x)
    for _ in range(max(args.warmup, 1)):
        oracle.fused_matvec(op, threads=cores, avx2=True)
    steps = min(args.steps, 200)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.fused_matvec(op, threads=cores, avx2=True)
    dt = time.perf_counter() - t0
    value = ALGO_BYTES * steps / dt / 1e9
    line = {
        "impl": "reference", "metric": "q4_matvec_hbm_gbs", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": max(args.warmup, 1),
        "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "q4_matvec 17408x5120 Q4_B64, f32 activations (BASELINE config 0)"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "whole 17408x5120 matvec per step, AVX2 arm of backend/cpu.rs "
                                   "restated in C, rows split over all host threads"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_b200(args):
    import torch
    import torch.distributed as dist
    import ctox_llm_b200 as ctox
    from ctox_llm_b200 import synthetic

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    stream = torch.cuda.Stream(device=local)
    be = ctox.B200Backend(local, stream=stream.cuda_stream)

    x_host = synthetic.activations(Q4_COLS, 0)
    replicas = []
    for r in range(REPLICAS):
        w = synthetic.packed_weights(ctox.Q4B64, Q4_ROWS, Q4_COLS, seed=r)
        replicas.append(be.prepare_fused_matvec(
            ctox.FusedMatVec(ctox.Q4B64, w, Q4_ROWS, Q4_COLS, None)))
    x_dev = torch.from_numpy(x_host).cuda(local)
    y_dev = torch.empty(Q4_ROWS, dtype=torch.float32, device=f"cuda:{local}")
    torch.cuda.synchronize()

    def step(i):
        replicas[i % REPLICAS].dispatch_device(x_dev.data_ptr(), ctox.F32, 1, Q4_COLS,
                                               y_dev.data_ptr(), Q4_ROWS)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # keep the device busy long enough for nvidia-smi to see clocks under load
    t_end = time.time() + 0.5
    i = 0
    while time.time() < t_end:
        step(i)
        i += 1
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        ev0.record(stream)
        for i in range(args.steps):
            step(i)
        ev1.record(stream)
    barrier()
    ms = ev0.elapsed_time(ev1)
    # dominant kernel alone (event pair around each streaming-kernel launch)
    be.kernel_timing(True)
    for i in range(args.steps):
        step(i)
    kernel_ms, launches = be.kernel_timing_read()
    be.kernel_timing(False)
    # end to end through the host API: pinned H2D of x, both kernels, D2H of y, every step
    for i in range(3):
        replicas[i % REPLICAS].dispatch_host(x_host)
    barrier()
    e2e_steps = min(args.steps, 200)
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        replicas[i % REPLICAS].dispatch_host(x_host)
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms, e2e_s], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_s = float(t[0]), float(t[1])

    if rank == 0:
        peak, peak_kind = load_peaks()
        value = ALGO_BYTES * args.steps * world / (ms * 1e-3) / 1e9
        achieved = ALGO_BYTES / (kernel_ms / max(launches, 1) * 1e-3) / 1e9
        cpu_val, cpu_s = cpu_baseline(threads=1, avx2=False, repeats=5)
        line = {
            "metric": "q4_matvec_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "q4_matvec 17408x5120 Q4_B64, f32 activations (BASELINE config 0)",
                       "l2": f"{REPLICAS} weight replicas rotated ({REPLICAS * 47.3:.0f} MB > 2x L2)",
                       "parallelism": "replicas" if world > 1 else "single"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "frac_of_8000_nominal": achieved / 8000.0,
                         "peak_kind": f"of {peak_kind}", "kernel": "k_matvec_stream<Q4>",
                         "kernel_us": kernel_ms / max(launches, 1) * 1e3, "traffic": None},
            "cpu_baseline": {"value": cpu_val, "unit": "GB/s", "cores": 1, "kind": "port",
                             "sample": f"whole 17408x5120 matvec, scalar-verifier arm, median of 5 "
                                       f"({cpu_s * 1e3:.1f} ms each)"},
            "e2e": {"value": ALGO_BYTES * e2e_steps * world / e2e_s / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": Q4_COLS * 4, "d2h_bytes_per_step": Q4_ROWS * 4 + 4,
                    "us_per_step": e2e_s / e2e_steps * 1e6},
            "gpu_launches": 2 * args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    for r in replicas:
        r.destroy()
    be.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
