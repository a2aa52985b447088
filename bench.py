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


# dram__bytes_read.sum + dram__bytes_write.sum of one k_matvec_stream launch over its algorithmic
# bytes: read from the committed ncu summary of the kernel (the line "dram bytes per algorithmic byte").
TRAFFIC_PROFILE = "profiles/k_matvec_stream_q4_17408x5120.md"


def load_traffic_ratio():
    import re
    try:
        with open(os.path.join(ROOT, TRAFFIC_PROFILE)) as f:
            m = re.search(r"dram bytes per algorithmic byte:\s*([0-9.]+)", f.read())
        return float(m.group(1)) if m else None
    except OSError:
        return None


def roofline_report(phase, elapsed_s, accepted_tokens, bytes_read, bytes_written, flops, bandwidth,
                    theoretical_bandwidth=None, compute=1383.2e12, dispatch_floor_s=0.0):
    """The reference's roofline gate record for this run (src/roofline.rs:82-142)."""
    from ctox_llm_b200.roofline import RooflineMeasurement
    return RooflineMeasurement(
        hardware_profile="cuda-sm100a-b200", phase=phase, traffic_source="exact_tensor_schedule",
        elapsed_seconds=elapsed_s, accepted_tokens=accepted_tokens, bytes_read=int(bytes_read),
        bytes_written=int(bytes_written), floating_point_operations=flops,
        sustainable_bandwidth_bytes_per_second=bandwidth, sustainable_compute_flops_per_second=compute,
        dispatch_floor_seconds=dispatch_floor_s, theoretical_bandwidth_bytes_per_second=theoretical_bandwidth,
        theoretical_compute_flops_per_second=2250e12 if theoretical_bandwidth else None).evaluate()


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



BLOCK_BYTES = {"q4": 34, "q2": 18}


def matvec_algo_bytes(dtype, rows, cols, positions=1):
    """Packed weights once + activations in + outputs out (f32), as BASELINE.md section 3 counts them."""
    return rows * (cols // 64) * BLOCK_BYTES[dtype] + positions * (cols + rows) * 4


def measure_matvec(be, stream, local, dtype, rows, cols, positions, steps, warmup=20, static=False, replicas=0):
    """Device-resident timing of one prepared matvec shape: `steps` dispatches over enough weight
    replicas to exceed twice the L2, CUDA events around the whole loop (launches overlap through
    programmatic dependent launch, as in a decode pass) and an event pair around every launch of the
    streaming kernel (serialised: the figure the roofline fraction uses)."""
    import torch
    import ctox_llm_b200 as ctox
    from ctox_llm_b200 import synthetic
    dt = ctox.Q4B64 if dtype == "q4" else ctox.Q2B64
    wbytes = rows * (cols // 64) * BLOCK_BYTES[dtype]
    n_rep = replicas if replicas > 0 else max(8, min(16, -(-300_000_000 // wbytes)))
    reps = [be.prepare_fused_matvec(ctox.FusedMatVec(dt, synthetic.packed_weights(dt, rows, cols, seed=100 + r),
                                                     rows, cols, None)) for r in range(n_rep)]
    x = torch.from_numpy(synthetic.activations(cols, 0, positions=positions).reshape(positions, cols)).cuda(local)
    y = torch.empty(positions, rows, dtype=torch.float32, device=f"cuda:{local}")
    torch.cuda.synchronize()

    def step(i):
        if static:
            reps[i % n_rep].dispatch_static(x.data_ptr(), ctox.F32, positions, cols, y.data_ptr(), rows)
        else:
            reps[i % n_rep].dispatch_device(x.data_ptr(), ctox.F32, positions, cols, y.data_ptr(), rows)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for i in range(steps):
        step(i)
    ev1.record(stream)
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    be.kernel_timing(True)
    for i in range(steps):
        step(i)
    kernel_ms, launches = be.kernel_timing_read()
    be.kernel_timing(False)
    for r in reps:
        r.destroy()
    peak, peak_kind = load_peaks()
    algo = matvec_algo_bytes(dtype, rows, cols, positions)
    kernel_us = kernel_ms / max(launches, 1) * 1e3 * (launches / steps)  # all passes of one dispatch
    return {"shape": f"{dtype} {rows}x{cols} x{positions}", "algo_bytes": algo, "replicas": n_rep,
            "us_per_dispatch": ms / steps * 1e3, "gbs": algo / (ms / steps * 1e-3) / 1e9,
            "kernel_us": kernel_us, "kernel_gbs": algo / (kernel_us * 1e-6) / 1e9,
            "frac": algo / (kernel_us * 1e-6) / 1e9 / peak, "frac_pipelined": algo / (ms / steps * 1e-3) / 1e9 / peak,
            "peak_kind": f"of {peak_kind}"}


def decode_workload_name(context, layers, drafts):
    depth = "" if layers == 64 else ", reduced depth: profiling case"
    return (f"qwen3.8-27b-shaped decode, {layers} layers, batch 1, context {context}, MTP k={drafts} "
            f"(k + 1 verify positions; BASELINE config 4{depth})")


def run_reference(args):
    """The reference's CPU path (C restatement of backend/cpu.rs, AVX2 arm, rows split over all host
    threads). Each step is one bounded sample: a 17408x5120 Q4 fused matvec. For the decode workload
    the sample's bandwidth is scaled to the bytes of one target pass of the same configuration."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
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
    gbs = ALGO_BYTES * steps / dt / 1e9
    if args.workload == "decode":
        import ctox_llm_b200 as ctox
        cfg = ctox.qwen38_27b_config(max_context_tokens=args.context + 4096)
        weights, kv, state = decode_config_bytes(cfg, args.context)
        value = 1.0 / ((weights + kv + state) / (gbs * 1e9))
        metric, unit = "decode_tokens_per_s_mtp", "tokens/s"
        workload = decode_workload_name(args.context, args.layers or 64, args.drafts)
        sample = (f"one 17408x5120 Q4 fused matvec per step at {gbs:.2f} GB/s, scaled to the "
                  f"{(weights + kv + state) / 1e9:.1f} GB of one target pass (one token per pass)")
    else:
        value, metric, unit = gbs, "q4_matvec_hbm_gbs", "GB/s"
        workload = "q4_matvec 17408x5120 Q4_B64, f32 activations (BASELINE config 0)"
        sample = "whole 17408x5120 matvec per step"
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit,
        "n_gpus": args.gpus, "steps": steps, "warmup": max(args.warmup, 1),
        "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.workload == "decode" else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload},
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port",
                         "sample": sample + "; AVX2 arm of backend/cpu.rs restated in C, rows split over "
                                            "all host threads"},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def decode_config_bytes(cfg, positions):
    """Algorithmic bytes of one target pass (weights once, bf16 KV of the context, state r/w)."""
    H, F, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    qw, kvw = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    vw = cfg.linear_num_value_heads * 128
    ch = 2 * cfg.linear_num_key_heads * 128 + vw
    q4 = lambda r, c: r * (c // 64) * 34
    q2 = lambda r, c: r * (c // 64) * 18
    n_full = cfg.num_hidden_layers // cfg.full_attention_interval
    n_lin = cfg.num_hidden_layers - n_full
    mlp = q2(2 * F, H) + q2(H, F)
    full = q4(2 * qw + 2 * kvw, H) + q4(H, qw) + mlp
    lin = q4(ch + vw + 2 * cfg.linear_num_value_heads, H) + q4(H, vw) + mlp
    weights = n_full * full + n_lin * lin + q4(V, H)
    kv = n_full * positions * kvw * 2 * 2
    state = n_lin * cfg.linear_num_value_heads * 128 * 128 * 4 * 2
    return weights, kv, state


def tp_parity_check(be, local, rank, world, drafts):
    """Outside the timed region: a 4-layer model of the full widths, sharded over the group, against
    the same model unsharded on rank 0 (synthetic tensors are functions of the global index, so the
    shards are slices of the one-GPU model). Real prefill of a short prompt, then speculative blocks:
    every rank must resolve the same blocks as the unsharded run, and its vocabulary shard of the
    logits must lie within rel-L2 1e-3 of the unsharded logits. Raises on mismatch."""
    import torch
    import torch.distributed as dist
    import ctox_llm_b200 as ctox
    cfg = ctox.qwen38_27b_config(max_context_tokens=512, num_hidden_layers=4, max_draft_tokens=drafts)
    prompt = [int(t) for t in np.random.default_rng(5).integers(0, cfg.vocab_size, 21)]
    n_blocks = 5

    def run(backend):
        ex = ctox.B200Executor(backend, cfg)
        ex.fill_synthetic(seed=7)
        ex.warmup()
        ex.keep_logits(True)
        ex.prefill(prompt)
        tok, blocks, logits = prompt[-1], [], []
        for _ in range(n_blocks):
            blk = ex.decode(tok, mtp_enabled=True)
            blocks.append((tuple(blk.draft_tokens), tuple(blk.accepted_draft_tokens), blk.token_id))
            logits.append(ex.last_logits(0).copy())
            tok = blk.token_id
        ex.unload()
        return blocks, logits

    blocks, logits = run(be)
    ref = [None, None]
    if rank == 0:
        solo = ctox.B200Backend(local)
        ref = list(run(solo))
        solo.close()
    dist.broadcast_object_list(ref, src=0)
    ref_blocks, ref_logits = ref
    n = cfg.vocab_size // world
    # Logits are comparable while both runs have consumed the same tokens. Sharding changes the order of
    # the sums (1e-5 relative), so a greedy token may differ where the top two logits are that close; from
    # there on the two runs decode different sequences, which is not an error: compare up to that block.
    same_history = 0
    for got_b, want_b in zip(blocks, ref_blocks):
        same_history += 1
        if got_b != want_b:
            break
    worst = 0.0
    for got, want in list(zip(logits, ref_logits))[:same_history]:
        w = want[rank * n:(rank + 1) * n]
        worst = max(worst, float(np.linalg.norm(got - w) / max(np.linalg.norm(w), 1e-30)))
    everyone = [None] * world
    dist.all_gather_object(everyone, (blocks, worst))
    ranks_agree = all(e[0] == everyone[0][0] for e in everyone)
    worst_all = max(e[1] for e in everyone)
    if not ranks_agree or worst_all > 1e-3:
        raise SystemExit(f"tensor-parallel parity check failed: ranks agree on the blocks: {ranks_agree}; largest "
                         f"logits rel-L2 against the unsharded run: {worst_all:.3e}; rank {rank} blocks {blocks}; "
                         f"unsharded {ref_blocks}")
    return {"tp_check": "green", "tp_check_blocks": n_blocks, "tp_check_blocks_equal_to_unsharded": sum(
                g == w for g, w in zip(blocks, ref_blocks)), "tp_check_logits_rel_l2_max": worst_all}



def run_decode(args):
    """BASELINE config 4: random-init Qwen3.8-27B-shaped hybrid decode, Q4 attention/embedding and
    Q2 FFN weights, bf16 paged KV (16-token pages) prefilled to 32768 tokens with random K/V,
    batch 1, MTP speculation (restricted 40000-row draft head). Chained drafts per block: 3 by
    default, i.e. k + 1 = 4 verify positions as BASELINE config 2 states them; `--drafts 4` gives
    the 5-row verify pass of the reference's CUDA candidate (backend/cuda_graph.rs:4565)."""
    import torch
    import torch.distributed as dist
    import ctox_llm_b200 as ctox

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    stream = torch.cuda.Stream(device=local)
    be = ctox.B200Backend(local, stream=stream.cuda_stream)
    tp_report = {}
    if world > 1:  # tensor parallel: every rank holds 1/world of the heads, FFN width and vocabulary
        be.tp_init_from_torch()
        tp_report = tp_parity_check(be, local, rank, world, args.drafts)
    context = args.context
    cfg = ctox.qwen38_27b_config(max_context_tokens=context + 4096)
    cfg.max_draft_tokens = args.drafts
    if args.layers:  # a shallower model of the same layer shapes: small cases for profiler captures
        cfg.num_hidden_layers = args.layers
    ex = ctox.B200Executor(be, cfg)
    ex.fill_synthetic(seed=0)
    ex.warmup()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    host_enqueue_ms = [0.0]
    counted_launches = [0]

    def run_blocks(n_blocks, mtp, force, timed):
        """Returns (device ms, wall s, tokens emitted, drafts accepted) for n_blocks decode calls."""
        ex.prefill_synthetic(context, seed=1)
        tok = 1
        for _ in range(args.warmup):
            tok = ex.decode(tok, mtp_enabled=mtp, force_accept=force).token_id
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        emitted = accepted = 0
        enqueue_us = 0.0
        ev0.record(stream)
        t0 = time.perf_counter()
        launches0 = be.kernel_launches()
        for _ in range(n_blocks):
            # decode + commit_speculative: the two calls of the executor interface per block
            blk = ex.decode(tok, mtp_enabled=mtp, force_accept=force)
            tok = blk.token_id
            emitted += len(blk.emitted)
            accepted += len(blk.accepted_draft_tokens)
            enqueue_us += ex.last_enqueue_us()
        host_enqueue_ms[0] = enqueue_us / n_blocks * 1e-3
        counted_launches[0] = be.kernel_launches() - launches0  # the library's own count of its launches
        wall = time.perf_counter() - t0
        ev1.record(stream)
        barrier()
        return ev0.elapsed_time(ev1), wall, emitted, accepted

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms, wall, emitted, accepted = run_blocks(args.steps, True, -1, True)
    enqueue_ms, timed_launches = host_enqueue_ms[0], counted_launches[0]
    clocks = sampler.stop() if rank == 0 else None
    buckets, plain = {}, None
    if not args.quick:
        for force in range(cfg.max_draft_tokens + 1):  # every acceptance bucket (docs/ROOFLINE_GATES.md:50)
            bms, _, bem, _ = run_blocks(max(args.steps // 8, 8), True, force, False)
            buckets[f"accept_{force}"] = bem / (bms * 1e-3)
        pms, _, pem, _ = run_blocks(max(args.steps // 8, 8), False, -1, False)
        plain = pem / (pms * 1e-3)
    # device time per phase of a block (events at the phase boundaries; outside the timed region)
    phases = None
    if not args.quick:
        ex.phase_timing(True)
        acc = {}
        ex.prefill_synthetic(context, seed=1)
        tok = 1
        for i in range(8):
            tok = ex.decode(tok, mtp_enabled=True, force_accept=-1).token_id
            if i >= 3:
                for name, v in ex.last_phase_ms().items():
                    acc[name] = acc.get(name, 0.0) + v / 5
        ex.phase_timing(False)
        phases = acc
    # dominant kernel (the streaming matvec) alone, event pairs around every launch
    timing_blocks = 1 if args.quick else 4
    be.kernel_timing(True)
    _, _, _, _ = run_blocks(timing_blocks, True, -1, False)
    kernel_ms, launches = be.kernel_timing_read()
    be.kernel_timing(False)
    blocks_timed = timing_blocks + args.warmup

    t = torch.tensor([ms, wall], dtype=torch.float64, device=f"cuda:{local}")
    cnt = torch.tensor([emitted, accepted], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:  # every rank resolves the same blocks: counts are rank 0's, times the slowest rank's
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, wall = float(t[0]), float(t[1])
    emitted, accepted = float(cnt[0]), float(cnt[1])
    collective = be.tp_collective()
    sub = {}
    if rank == 0 and world == 1 and not args.quick:
        # the other half of the headline metric in the same record: BASELINE config 0 (a) and (b)
        bytes_before_unload = be.allocated_bytes()
        ex.unload()
        ex = None
        # the reference's loop bench checks bytes freed after drop == bytes before prepare
        # (src/bin/cuda_target_mtp4_graph_bench.rs:156-161)
        sub["device_bytes"] = {"model_and_session": bytes_before_unload, "after_unload": be.allocated_bytes()}
        sub["q4_matvec"] = measure_matvec(be, stream, local, "q4", Q4_ROWS, Q4_COLS, 1, 400)
        sub["q2_matvec"] = measure_matvec(be, stream, local, "q2", 5120, 17408, 1, 400)
    traffic_ratio = load_traffic_ratio()
    if rank == 0:
        peak, peak_kind = load_peaks()
        weights, kv, state = decode_config_bytes(cfg, context)
        # bytes streamed by the matvec kernel per block: target pass + k MTP passes + draft heads
        mtp_layer = (weights - (cfg.vocab_size * (cfg.hidden_size // 64) * 34)) // cfg.num_hidden_layers
        fc_bytes = cfg.hidden_size * (2 * cfg.hidden_size // 64) * 34  # replicated on every rank
        stream_bytes = weights // world + cfg.max_draft_tokens * (
            mtp_layer // world + fc_bytes + cfg.draft_vocab * (cfg.hidden_size // 64) * 34 // world)
        achieved = stream_bytes * blocks_timed / (kernel_ms * 1e-3) / 1e9
        cpu_val, cpu_s = cpu_baseline(threads=1, avx2=False, repeats=3)
        cpu_tok_s = 1.0 / ((weights + kv + state) / (cpu_val * 1e9))
        line = {
            "metric": "decode_tokens_per_s_mtp", "value": emitted / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": decode_workload_name(context, cfg.num_hidden_layers, cfg.max_draft_tokens),
                       "weights": "Q4_B64 attention/embedding, Q2_B64 FFN, random init",
                       "kv": "bf16, 16-token pages", "l2": "11.8 GB streamed per pass (>> 126 MB L2)",
                       "parallelism": f"tp{world} (one sequence; heads, FFN width and vocabulary split; partial "
                                      f"results of every column-split projection summed by: {collective})"
                                      if world > 1 else "single",
                       "collective": collective,
                       "acceptance": "as measured on random-init weights"},
            "speculative_blocks_per_s": args.steps / (ms * 1e-3),
            "mean_accepted_drafts_per_block": accepted / args.steps,
            "tokens_per_s_without_mtp": plain,
            "tokens_per_s_forced_acceptance": buckets,
            "phase_ms_per_block": phases,
            "host_reads_per_block": 1,
            "host_enqueue_ms_per_block": enqueue_ms,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "frac_of_8000_nominal": achieved / 8000.0,
                         "peak_kind": f"of {peak_kind}", "kernel": "k_matvec_stream (all launches of a block, per GPU)",
                         "bytes_per_block": stream_bytes, "launches_per_block": launches / blocks_timed,
                         "timing_note": "event pair around every launch: serialised, without the overlap of "
                                        "dependent launches that the headline number has",
                         "traffic": stream_bytes * traffic_ratio if traffic_ratio else None,
                         "traffic_note": "per block; dram bytes per algorithmic byte of the ncu capture in "
                                         f"{TRAFFIC_PROFILE} scaled by the bytes streamed"},
            "roofline_gate": roofline_report(
                "speculative_verify", elapsed_s=ms * 1e-3 / args.steps, accepted_tokens=emitted / args.steps,
                bytes_read=(weights + kv + state // 2) // world + (stream_bytes - weights // world),
                bytes_written=state // 2 // world, flops=0.0, bandwidth=peak * 1e9,
                theoretical_bandwidth=8000e9),
            "pass_bytes": {"weights": weights, "kv": kv, "state": state},
            "cpu_baseline": {"value": cpu_tok_s, "unit": "tokens/s", "cores": 1, "kind": "port",
                             "sample": f"scalar-verifier matvec on one 17408x5120 Q4 matrix ({cpu_val:.3f} GB/s, "
                                       f"{cpu_s * 1e3:.0f} ms), scaled to the {(weights + kv + state) / 1e9:.1f} GB "
                                       "of one target pass"},
            "e2e": {"value": emitted / wall, "unit": "tokens/s",
                    # uploads per block: the token (4 B) and the tokens of the MTP catch-up pairs
                    # (4 B per position committed by the previous block); read back: record + error word
                    "h2d_bytes_per_step": 4 + 4 * (emitted / args.steps), "d2h_bytes_per_step": 292 + 4,
                    "note": "decode() + commit_speculative() take a host token and return a host record; "
                            "same calls, wall clock"},
            "gpu_launches": timed_launches,
            "clocks": clocks,
        }
        line.update(tp_report)
        line.update(sub)
        print(json.dumps(line), flush=True)
    if ex is not None:
        ex.unload()
    be.close()
    if world > 1:
        dist.destroy_process_group()


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
        launches0 = be.kernel_launches()
        for i in range(args.steps):
            step(i)
        timed_launches = be.kernel_launches() - launches0
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
                         "kernel_us": kernel_ms / max(launches, 1) * 1e3,
                         "traffic": ALGO_BYTES * load_traffic_ratio() if load_traffic_ratio() else None},
            "cpu_baseline": {"value": cpu_val, "unit": "GB/s", "cores": 1, "kind": "port",
                             "sample": f"whole 17408x5120 matvec, scalar-verifier arm, median of 5 "
                                       f"({cpu_s * 1e3:.1f} ms each)"},
            "e2e": {"value": ALGO_BYTES * e2e_steps * world / e2e_s / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": Q4_COLS * 4, "d2h_bytes_per_step": Q4_ROWS * 4 + 4,
                    "us_per_step": e2e_s / e2e_steps * 1e6},
            "gpu_launches": timed_launches,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    for r in replicas:
        r.destroy()
    be.close()
    if world > 1:
        dist.destroy_process_group()



CONFIG1_LAYER = [  # BASELINE config 1 (q_proj with the interleaved gate rows, as the reference holds it)
    ("q_proj", "q4", 12288, 5120), ("k_proj", "q4", 1024, 5120), ("v_proj", "q4", 1024, 5120),
    ("o_proj", "q4", 5120, 6144), ("gate_proj", "q2", 17408, 5120), ("up_proj", "q2", 17408, 5120),
    ("down_proj", "q2", 5120, 17408)]


def run_micro(args):
    """Single-kernel workloads on one GPU: `matvec` (any shape), `q2_matvec` (BASELINE config 0b),
    `verify_layer` (config 1: the seven projections of one layer at M = 1, 2, 4, 8, 16 positions) and
    `gated_delta` (config 2: 48 layers, T = 4 then T = 1), `kv_pack` (K/V rows of one layer at 32768
    tokens to Q4 blocks, the Q4 -> Q2 demotion and the decode). Inputs are resident in HBM; weights or
    states are rotated over more than twice the L2."""
    import torch
    import ctox_llm_b200 as ctox
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if int(os.environ.get("RANK", "0")) != 0:
        return
    torch.cuda.set_device(local)
    stream = torch.cuda.Stream(device=local)
    be = ctox.B200Backend(local, stream=stream.cuda_stream)
    peak, peak_kind = load_peaks()
    sampler = ClockSampler(local)
    sampler.start()
    line = {"n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic"}
    launches0 = be.kernel_launches()
    with torch.cuda.stream(stream):
        if args.workload in ("matvec", "q2_matvec"):
            dtype, rows, cols, pos = (("q2", 5120, 17408, 1) if args.workload == "q2_matvec"
                                      else (args.dtype, args.rows, args.cols, args.positions))
            r = measure_matvec(be, stream, local, dtype, rows, cols, pos, args.steps, args.warmup, args.static,
                               args.replicas)
            line.update(metric=f"{dtype}_matvec_hbm_gbs", value=r["gbs"], unit="GB/s",
                        ms_per_step=r["us_per_dispatch"] * 1e-3,
                        config={"workload": f"matvec {r['shape']} positions, f32 activations",
                                "l2": f"{r['replicas']} weight replicas rotated"},
                        roofline={"bound": "hbm", "achieved": r["kernel_gbs"], "peak": peak, "unit": "GB/s",
                                  "frac": r["frac"], "peak_kind": r["peak_kind"], "kernel": "k_matvec_stream",
                                  "kernel_us": r["kernel_us"], "frac_pipelined": r["frac_pipelined"],
                                  "traffic": None},
                        )
        elif args.workload == "verify_layer":
            sweep = {}
            for m in (1, 2, 4, 8, 16):
                us = kus = 0.0
                for name, dtype, rows, cols in CONFIG1_LAYER:
                    r = measure_matvec(be, stream, local, dtype, rows, cols, m, max(args.steps // 10, 40), 10)
                    us += r["us_per_dispatch"]
                    kus += r["kernel_us"]
                wbytes = sum(rows * (cols // 64) * BLOCK_BYTES[d] for _, d, rows, cols in CONFIG1_LAYER)
                sweep[f"M{m}"] = {"us_per_layer": us, "gbs": wbytes / (us * 1e-6) / 1e9,
                                  "kernel_us_per_layer": kus, "kernel_frac": wbytes / (kus * 1e-6) / 1e9 / peak,
                                  "gflop": 2 * m * sum(r * c for _, _, r, c in CONFIG1_LAYER) / 1e9}
            ref = sweep["M4"]
            line.update(metric="verify_layer_hbm_gbs", value=ref["gbs"], unit="GB/s",
                        ms_per_step=ref["us_per_layer"] * 1e-3,
                        config={"workload": "BASELINE config 1: q/k/v/o (Q4) and gate/up/down (Q2) of one layer, "
                                            "M verify positions, weights 130 908 160 B read once per M <= 16"},
                        sweep=sweep,
                        roofline={"bound": "hbm", "achieved": 130908160 / (ref["kernel_us_per_layer"] * 1e-6) / 1e9,
                                  "peak": peak, "unit": "GB/s", "frac": ref["kernel_frac"],
                                  "peak_kind": f"of {peak_kind}", "kernel": "k_matvec_stream (M = 4)", "traffic": None})
        elif args.workload == "kv_pack":
            # K and V of one full-attention layer at 32768 tokens: 4 + 4 heads x 256 = 32 blocks per token
            n_blocks = 32768 * 32
            dev = f"cuda:{local}"
            g = torch.Generator(device=dev).manual_seed(3)
            vals = torch.randn(n_blocks * 64, device=dev, generator=g)
            q4 = torch.empty(n_blocks * 34, dtype=torch.uint8, device=dev)
            q2 = torch.empty(n_blocks * 18, dtype=torch.uint8, device=dev)
            back = torch.empty(n_blocks * 64, device=dev)
            ops = {"pack_q4": (lambda: be.kv_pack_q4(vals.data_ptr(), n_blocks, q4.data_ptr()), n_blocks * (256 + 34)),
                   "demote_q4_to_q2": (lambda: be.kv_demote_q4_to_q2(q4.data_ptr(), n_blocks, q2.data_ptr()),
                                       n_blocks * (34 + 18)),
                   "unpack_q2": (lambda: be.kv_unpack(ctox.native.Q2B64, q2.data_ptr(), n_blocks, back.data_ptr()),
                                 n_blocks * (18 + 256))}
            res = {}
            for name, (fn, nbytes) in ops.items():
                for _ in range(args.warmup):
                    fn()
                torch.cuda.synchronize()
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record(stream)
                for _ in range(args.steps):
                    fn()
                ev1.record(stream)
                torch.cuda.synchronize()
                ms = ev0.elapsed_time(ev1) / args.steps
                res[name] = {"us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9,
                             "frac": nbytes / (ms * 1e-3) / 1e9 / peak}
            line.update(metric="kv_pack_hbm_gbs", value=res["pack_q4"]["gbs"], unit="GB/s",
                        ms_per_step=res["pack_q4"]["us"] * 1e-3,
                        config={"workload": "K/V rows of one full-attention layer at 32768 tokens (1 048 576 blocks "
                                            "of 64 values): f32 -> Q4_B64, Q4_B64 -> Q2_B64, Q2_B64 -> f32",
                                "l2": "268 MB of values per launch > 2x L2"},
                        sweep=res,
                        roofline={"bound": "hbm", "achieved": res["pack_q4"]["gbs"], "peak": peak, "unit": "GB/s",
                                  "frac": res["pack_q4"]["frac"], "peak_kind": f"of {peak_kind}",
                                  "kernel": "k_kv_pack_q4", "traffic": None})
        else:  # gated_delta
            heads, qk, layers = 48, 16, 48
            dev = f"cuda:{local}"
            g = torch.Generator(device=dev).manual_seed(2)
            state = [torch.randn(layers, heads, 128, 128, device=dev, generator=g) * 0.02 for _ in range(2)]
            T = 4
            q = torch.nn.functional.normalize(torch.randn(T, qk, 128, device=dev, generator=g), dim=-1)
            k = torch.nn.functional.normalize(torch.randn(T, qk, 128, device=dev, generator=g), dim=-1)
            v = torch.randn(T, heads, 128, device=dev, generator=g)
            gate = torch.log(torch.sigmoid(torch.randn(T, heads, device=dev, generator=g) + 2.0))
            beta = torch.sigmoid(torch.randn(T, heads, device=dev, generator=g))
            out = torch.empty(T, heads, 128, device=dev)
            torch.cuda.synchronize()

            def step(tokens, a, b):
                for l in range(layers):
                    be.gated_delta_scan(q.data_ptr(), k.data_ptr(), v.data_ptr(), gate.data_ptr(), beta.data_ptr(),
                                        state[a][l].data_ptr(), state[b][l].data_ptr(), out.data_ptr(), tokens,
                                        heads, qk)

            res = {}
            for tokens in (4, 1):
                for i in range(args.warmup):
                    step(tokens, i & 1, (i & 1) ^ 1)
                torch.cuda.synchronize()
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record(stream)
                for i in range(args.steps):
                    step(tokens, i & 1, (i & 1) ^ 1)
                ev1.record(stream)
                torch.cuda.synchronize()
                ms = ev0.elapsed_time(ev1) / args.steps
                nbytes = layers * (2 * heads * 128 * 128 * 4 + tokens * ((2 * qk + heads) * 128 + 2 * heads) * 4
                                   + tokens * heads * 128 * 4)
                res[f"T{tokens}"] = {"ms_per_48_layers": ms, "us_per_layer": ms * 1e3 / layers, "bytes": nbytes,
                                     "gbs": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peak}
            # the same 48 scans as ONE launch (the form of the executor's prefix re-scan at commit, where
            # the layers are independent; inside a decode pass they are not)
            ql, kl, vl = (x[None].expand(layers, *x.shape).contiguous() for x in (q, k, v))
            gl, bl = (x[None].expand(layers, *x.shape).contiguous() for x in (gate, beta))
            for tokens in (4, 1):
                def one(a, b):
                    be.gated_delta_scan_layers(ql.data_ptr(), kl.data_ptr(), vl.data_ptr(), gl.data_ptr(), bl.data_ptr(),
                                               state[a].data_ptr(), state[b].data_ptr(), 0, layers, tokens, heads, qk)
                for i in range(args.warmup):
                    one(i & 1, (i & 1) ^ 1)
                torch.cuda.synchronize()
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record(stream)
                for i in range(args.steps):
                    one(i & 1, (i & 1) ^ 1)
                ev1.record(stream)
                torch.cuda.synchronize()
                ms = ev0.elapsed_time(ev1) / args.steps
                nbytes = layers * (2 * heads * 128 * 128 * 4 + tokens * ((2 * qk + heads) * 128 + 2 * heads) * 4)
                res[f"T{tokens}_one_launch"] = {"ms_per_48_layers": ms, "bytes": nbytes,
                                                "gbs": nbytes / (ms * 1e-3) / 1e9,
                                                "frac": nbytes / (ms * 1e-3) / 1e9 / peak}
            line.update(metric="gated_delta_hbm_gbs", value=res["T4"]["gbs"], unit="GB/s",
                        ms_per_step=res["T4"]["ms_per_48_layers"],
                        config={"workload": "BASELINE config 2: gated-delta recurrence, 16 key / 48 value heads, "
                                            "dim 128, fp32 state, 48 layers back to back, T = 4 then T = 1",
                                "l2": "302 MB of state (two buffers of 48 layers) > 2x L2"},
                        sweep=res,
                        roofline={"bound": "hbm", "achieved": res["T4"]["gbs"], "peak": peak, "unit": "GB/s",
                                  "frac": res["T4"]["frac"], "peak_kind": f"of {peak_kind}",
                                  "kernel": "k_gated_delta_scan128 (48 launches per step)", "traffic": None})
    # the library's own count: every launch of this run, warm-up and set-up (weight repacking) included
    line["gpu_launches"] = be.kernel_launches() - launches0
    line["clocks"] = sampler.stop()
    line["e2e"] = None
    line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    be.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode",
                    choices=["decode", "q4_matvec", "q2_matvec", "matvec", "verify_layer", "gated_delta", "kv_pack"])
    ap.add_argument("--dtype", default="q4", choices=["q4", "q2"], help="matvec: code format")
    ap.add_argument("--rows", type=int, default=17408)
    ap.add_argument("--cols", type=int, default=5120)
    ap.add_argument("--positions", type=int, default=1)
    ap.add_argument("--static", action="store_true", help="matvec: use the allocation-free dispatch")
    ap.add_argument("--replicas", type=int, default=0,
                    help="matvec: weight replicas to rotate (default: enough to exceed twice the L2; 1 = weights "
                         "stay in L2, a diagnostic that separates the instruction cost from the HBM stream)")
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--drafts", type=int, default=3,
                    help="decode: chained MTP drafts per block (3 = 4 verify positions, BASELINE config 2; "
                         "4 = the reference candidate's 5-row verify pass)")
    ap.add_argument("--layers", type=int, default=0,
                    help="decode: number of layers (default: the model's 64); fewer = a small profiling case")
    ap.add_argument("--quick", action="store_true",
                    help="decode: only the timed region and one kernel-timing block (for launch lists)")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = {"decode": 256, "verify_layer": 400, "gated_delta": 50, "kv_pack": 50}.get(args.workload, 2000)
    if args.warmup is None:
        args.warmup = {"decode": 4, "gated_delta": 5, "kv_pack": 5}.get(args.workload, 50)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "decode":
        run_decode(args)
    elif args.workload == "q4_matvec":
        run_b200(args)
    else:
        run_micro(args)


if __name__ == "__main__":
    main()
