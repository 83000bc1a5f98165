#!/usr/bin/env python
"""Benchmark of the Q4 dequantize-fused decode GEMVs (metric: HBM GB/s of the quantized GEMV path).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--fmt q4|q8] [--impl reference]

Workload: every quantized GEMV of one Qwen3-8B-shaped decode token (36 layers x {q|k|v, o, gate|up,
down} + lm_head, 145 launches, 4.73 GB of packed Q4 weights), column-sharded over N GPUs with
an all-gather after each exchange point.  A step is one token; `value` is the algorithmic bytes
all ranks move per step divided by the step time (max over ranks, CUDA events, barrier and
synchronize on both sides).  Weights are resident; per-step weight bytes exceed L2 by 4-37x, so
every launch streams from HBM without an explicit flush.

`e2e` is the same step through host buffers: pinned host activations are copied in and the
logits are copied out inside the timed region.  `--impl reference` times the CPU restatement of
meganeura's own kernel math (oracle/) on the host cores; the reference itself needs a Rust
toolchain and a Vulkan device, neither of which exists here.
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

METRIC = "q4_gemv_hbm_gbs"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, val in zip(names, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------- CPU reference

def cpu_layer_buffers(shape, fmt, layers, seed=0):
    """Host packed weights + activations for `layers` layers of the workload (distinct bytes per GEMV)."""
    import numpy as np
    from meganeura_b200 import decode_chain as dc, synth
    rng = np.random.Generator(np.random.PCG64(seed))
    xs = {"h": rng.standard_normal((1, shape.hidden)).astype(np.float32),
          "f": rng.standard_normal((1, shape.ffn)).astype(np.float32)}
    items = []
    for layer in range(layers):
        for sp in dc.layer_specs(shape):
            base, n0, reps = synth.synth_weights_tiled(fmt, sp.k, sp.n, seed=layer * 16 + len(items) % 16, base_cols=256)
            items.append((sp, synth.tile_columns(fmt, base, sp.k, n0, reps)))
    return xs, items


def cpu_pass(coracle, fmt, xs, items, threads):
    """One pass of the oracle's f32 matmul over the buffers; returns (seconds, algorithmic bytes)."""
    from meganeura_b200 import decode_chain as dc
    t0 = time.perf_counter()
    nbytes = 0
    for sp, w in items:
        coracle.matmul(fmt, xs[sp.src], w, sp.k, sp.n, wide=False, variant=0, nthreads=threads)
        nbytes += dc.gemv_bytes(fmt, 1, sp.k, sp.n, sp.residual)
    return time.perf_counter() - t0, nbytes


def build_fast_oracle():
    """The oracle compiled for this host's ISA (falls back to the portable build)."""
    from oracle import oracle as O
    try:
        so = os.path.join(ROOT, "oracle", "liborc_native.so")
        subprocess.run(["gcc", "-O3", "-march=native", "-fPIC", "-ffp-contract=off", "-shared", "-o", so,
                        os.path.join(ROOT, "oracle", "mgq_oracle.c"), "-lm", "-lpthread"], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        return O.COracle(so)
    except (OSError, subprocess.CalledProcessError):
        return O.COracle()


def cpu_baseline(shape, fmt, budget_s=12.0):
    coracle = build_fast_oracle()
    threads = os.cpu_count() or 1
    xs, items = cpu_layer_buffers(shape, fmt, 1)
    cpu_pass(coracle, fmt, xs, items, threads)                   # warm-up (page faults, thread start)
    sec1, bytes1 = cpu_pass(coracle, fmt, xs, items, threads)
    layers = max(1, min(shape.layers, int(budget_s / max(sec1, 1e-3))))
    if layers > 1:
        xs, items = cpu_layer_buffers(shape, fmt, layers)
        cpu_pass(coracle, fmt, xs, items[: len(items) // layers], threads)
    sec, nbytes = cpu_pass(coracle, fmt, xs, items, threads)
    return {"value": round(nbytes / sec / 1e9, 3), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{layers} of {shape.layers} layers of the workload ({nbytes / 1e6:.0f} MB of GEMV bytes), "
                      f"one pass, {sec:.2f} s, C restatement of the reference kernel math, f32"}


def run_reference(args, shape, fmt):
    """The reference's CPU path: the oracle port (the reference itself cannot be built here)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    coracle = build_fast_oracle()
    threads = os.cpu_count() or 1
    xs, probe = cpu_layer_buffers(shape, fmt, 1)
    cpu_pass(coracle, fmt, xs, probe, threads)
    sec1, _ = cpu_pass(coracle, fmt, xs, probe, threads)
    total_steps = args.steps + args.warmup
    layers = max(1, min(shape.layers, int(90.0 / max(sec1 * total_steps, 1e-3))))
    xs, items = cpu_layer_buffers(shape, fmt, layers) if layers > 1 else (xs, probe)
    for _ in range(args.warmup):
        cpu_pass(coracle, fmt, xs, items, threads)
    t0 = time.perf_counter()
    nbytes = 0
    for _ in range(args.steps):
        _, b = cpu_pass(coracle, fmt, xs, items, threads)
        nbytes += b
    sec = time.perf_counter() - t0
    value = nbytes / sec / 1e9
    sample = (f"each step = {layers} of {shape.layers} layers ({nbytes / args.steps / 1e6:.0f} MB of GEMV bytes) on "
              f"{threads} host threads; C restatement of meganeura's quantized matmul math "
              "(the Rust/WGSL reference needs cargo and Vulkan: unavailable on this box)")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(shape, fmt, args.batch, args.gpus),
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------- GPU arm

def decode_tokens_per_s(model: str, steps: int = 128, context: int = 2048):
    """Whole-model greedy decode through Graph / build_inference_session / Session: every operator
    of the step (embedding, norms, RoPE, cache writes, attention, SwiGLU, the quantized GEMVs and
    the greedy pick) runs on the GPU from one captured CUDA graph per token; the host only launches.
    KV caches are pre-filled to `context` positions; weights are the synthetic packed weights."""
    from meganeura_b200 import decode_model as M
    cfg = M.QWEN3_8B if model == "qwen3-8b" else M.SMOLLM2_135M
    if cfg is M.SMOLLM2_135M:
        context = 128
    max_seq = context + steps + 8
    t0 = time.perf_counter()
    dec = M.DecodeSession(cfg, max_seq, seed=3, greedy_history=max_seq)
    dec.fill_caches(context)
    build_s = time.perf_counter() - t0
    s = dec.session
    dec.set_position(1, context)
    s.step()                                     # warm-up outside the graph
    s.wait()
    s.capture()
    dec.set_position(1, context)
    for _ in range(3):
        s.step()
    s.wait()
    dec.set_position(1, context)
    t0 = time.perf_counter()
    for _ in range(steps):
        s.step()
    s.wait()
    tokens = s.read_tokens(context, steps)
    dt = time.perf_counter() - t0
    plan = s.plan().dispatches
    kv_bytes = 2 * cfg.num_hidden_layers * cfg.kv_dim * 4 * (context + steps // 2)
    return {"model": f"{cfg.name}-shaped, random packed weights", "tokens_per_s": round(steps / dt, 1),
            "ms_per_token": round(dt / steps * 1e3, 4), "steps": steps, "kv_context": context, "batch": 1,
            "launches_per_token": len(plan) + 1, "greedy_pick": "device", "timing": "host wall clock around launch + final token read",
            "weight_plus_kv_gbs": round((M.packed_weight_bytes(cfg) + kv_bytes) / (dt / steps) / 1e9, 1),
            "distinct_tokens": int(len(set(int(t) for t in tokens))), "build_s": round(build_s, 1)}


def workload_config(shape, fmt, batch, gpus, exchange="peer"):
    return {
        "workload": f"{shape.name}-shaped decode token, all {'Q4' if fmt == 2 else 'Q8'} GEMVs "
                    f"({shape.layers} layers x q|k|v,o,gate|up,down + lm_head), batch {batch}",
        "weights": "packed codes uniform, f16 block scales log-uniform [1e-3,1e-1], offset 8 (Q4); seeded",
        "activations": "f32 N(0,1), seeded",
        "parallelism": (f"columns sharded x{gpus}, exchange at 4 points per layer + logits: " +
                        ("slices pushed into every peer's buffer by the GEMV kernel (NVLink stores + arrival counters)"
                         if exchange == "peer" else "NCCL all-gather")) if gpus > 1 else "single GPU",
        "l2": "no flush needed: each step streams its weights once, 4-37x the 126 MB L2",
        "launch": "one CUDA graph per token",
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--fmt", choices=["q4", "q8"], default="q4")
    ap.add_argument("--model", choices=["qwen3-8b", "smollm2-135m"], default="qwen3-8b")
    ap.add_argument("--impl", choices=["mgq", "reference"], default="mgq")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-model decode tokens/s measurement")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="multi-GPU exchange: slices pushed over NVLink by the GEMV kernels (default) or NCCL all-gather")
    ap.add_argument("--plan-kernel", action="store_true", help="run the token as one persistent plan kernel instead of one kernel per GEMV")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "mgq" else args.warmup

    from meganeura_b200 import decode_chain as dc
    from meganeura_b200._lib import FMT_Q4, FMT_Q8
    shape = dc.QWEN3_8B if args.model == "qwen3-8b" else dc.SMOLLM2_135M
    fmt = FMT_Q4 if args.fmt == "q4" else FMT_Q8

    if args.impl == "reference":
        run_reference(args, shape, fmt)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path (use --impl reference for the CPU arm)")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    chain = dc.DecodeGemvChain(shape, fmt, batch=args.batch, rank=rank, world=world, seed=0,
                               use_plan=args.plan_kernel, exchange=args.exchange)
    captured = chain.capture()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms_dev = timed(chain.step, args.steps, args.warmup)
    ms_e2e = timed(chain.step_host, args.steps, args.warmup)
    # nvidia-smi delivers a sample every 100 ms and the timed regions last tens of milliseconds: keep
    # replaying the same step for ~0.6 s more (same count on every rank) so that the clock record
    # holds several samples under this load
    for _ in range(max(1, min(2000, int(0.6 / max(1e-6, ms_dev / args.steps * 1e-3))))):
        chain.step()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    if chain.peer is not None and chain.peer.error():
        raise SystemExit("a bounded wait of the peer exchange ran out (MGQ_ERR_TIMEOUT): results are invalid")

    bytes_rank = chain.bytes_per_step()
    total_bytes = bytes_rank * world
    ms_step = ms_dev / args.steps
    value = total_bytes / (ms_step * 1e-3) / 1e9
    e2e_value = total_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    launches = chain.launches_per_step * (args.steps + args.warmup) * 2

    if rank == 0:
        peak, which = measured_peaks()
        per_launch_bytes = bytes_rank / chain.launches_per_step
        per_launch_us = ms_step * 1e3 / chain.launches_per_step
        achieved = bytes_rank / (ms_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(shape, fmt, args.batch, world, args.exchange),
            "tokens_per_s": round(args.batch / (ms_step * 1e-3), 1),
            "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": chain.h2d_bytes(),
                    "d2h_bytes_per_step": chain.d2h_bytes(), "ms_per_step": round(ms_e2e / args.steps, 4),
                    "tokens_per_s": round(args.batch / (ms_e2e / args.steps * 1e-3), 1)},
            "gpu_launches": launches,
            "cuda_graph": captured,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": UNIT,
                         "frac": round(achieved / peak, 4), "peak_source": f"of {which} (MEASURED_PEAKS.json hbm_gbs)",
                         "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                         "kernel": "gemv_q4_kernel" if fmt == FMT_Q4 else "gemv_q8_kernel",
                         "bytes_per_launch": round(per_launch_bytes), "us_per_launch": round(per_launch_us, 3),
                         "traffic": NCU_TRAFFIC.get(args.fmt) if (world == 1 and args.model == "qwen3-8b" and args.batch == 1
                                                                   and not args.plan_kernel) else None},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(shape, fmt)
        if world == 1 and not args.no_decode and args.batch == 1 and not args.plan_kernel:
            chain.graph = None
            line["decode"] = decode_tokens_per_s(args.model)
        print(json.dumps(line))
    if world > 1:
        # A captured graph that holds NCCL nodes must go before the communicator does (destroying the
        # process group first blocks forever); a watchdog ends the process if teardown still stalls.
        sys.stdout.flush()
        dist.barrier()
        torch.cuda.synchronize()
        chain.graph = None
        del chain
        torch.cuda.synchronize()
        watchdog = threading.Timer(30.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        dist.destroy_process_group()
        watchdog.cancel()


# DRAM bytes per launch of the GEMV kernel (dram__bytes_read.sum + dram__bytes_write.sum averaged
# over 298 launches of the default workload, single ncu pass; summary:
# profiles/gemv_q4_qwen3_decode_launch_list.md).  Only meaningful for the default Qwen3-8B-shaped
# Q4 workload with one launch per GEMV.
NCU_TRAFFIC = {"q4": 32620000, "q8": None}

if __name__ == "__main__":
    main()
