#!/usr/bin/env python
"""Benchmark of the Q4 dequantize-fused decode GEMVs (metric: HBM GB/s of the quantized GEMV path).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--fmt q4|q8] [--impl reference]

Workload: every quantized GEMV of one Qwen3-8B-shaped decode token (36 layers x {q|k|v, o, gate|up,
down} + lm_head, 145 GEMVs, 4.73 GB of packed Q4 weights), chained through their data (each GEMV
consumes its predecessor's output) and column-sharded over N GPUs with an all-gather of activations
after each GEMV.  A step is one token; `value` is the algorithmic bytes all ranks move per step
divided by the step time (max over ranks, CUDA events, barrier and synchronize on both sides).
Weights are resident; per-step weight bytes exceed L2 by 4-37x, so every step streams from HBM
without an explicit flush.

`e2e` is the same step through host buffers: pinned host activations are copied in and the
logits are copied out inside the timed region.  `--impl reference` times the CPU restatement of
meganeura's own kernel math (oracle/) on the host cores; the reference itself needs a Rust
toolchain and a Vulkan device, neither of which exists here.

Every line carries `parity_check` (the measured results against the CPU oracle, the stand-alone
kernels and, on several GPUs, the unsharded chain).  Further keys unless --no-extras: on one GPU
`other_mode`, `batch8`, `gemm` (512x4096x14336 Q8 prefill GEMM), `gemv_cases`, `decode` /
`decode_<model>` (whole-model greedy decode through Graph / Session); on several GPUs `batch8`
(8 rows over the column shards, peer-memory all-gather with NCCL timed beside it) and
`decode_sharded` (the whole model column-sharded over the ranks, tokens checked against the
unsharded model).
"""
from __future__ import annotations

import argparse
import hashlib
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
FALLBACK_BF16_TFLOPS = 1590.0
FMT_Q4, FMT_Q8 = 2, 3

# name, layers, hidden, q_dim, kv_dim, ffn, vocab (examples/qwen3.rs:91-105, src/models/smollm2.rs:35-47)
SHAPES = {"qwen3-8b": ("qwen3-8b", 36, 4096, 4096, 1024, 12288, 151936),
          "smollm2-135m": ("smollm2-135m", 30, 576, 576, 192, 1536, 49152)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", FALLBACK_BF16_TFLOPS)), "measured"
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


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
# This part imports nothing from the product package: shapes, byte counts and data come from here
# and from oracle/ (the checker), so the reference arm's process loads only the oracle library.

def cpu_layer_gemvs(shape):
    """(k, n, residual, source vector) of the GEMVs of one layer, in launch order."""
    _, _, hidden, q_dim, kv_dim, ffn, _ = shape
    return [(hidden, q_dim + 2 * kv_dim, False, "h"), (q_dim, hidden, True, "h"),
            (hidden, 2 * ffn, False, "h"), (ffn, hidden, True, "f")]


def cpu_gemv_bytes(fmt, k, n, residual):
    return k * n // 32 * (20 if fmt == FMT_Q4 else 36) + 4 * k + 4 * n * (2 if residual else 1)


def cpu_layer_buffers(shape, fmt, layers, seed=0):
    """Host packed weights + activations for `layers` layers of the workload (distinct bytes per GEMV)."""
    import numpy as np
    from oracle import oracle as O
    rng = np.random.Generator(np.random.PCG64(seed))
    xs = {"h": rng.standard_normal((1, shape[2])).astype(np.float32),
          "f": rng.standard_normal((1, shape[5])).astype(np.float32)}
    items = []
    for layer in range(layers):
        for j, (k, n, residual, src) in enumerate(cpu_layer_gemvs(shape)):
            n0 = 256 if n % 256 == 0 else n
            base = O.synth_weights(fmt, k, n0, seed=layer * 16 + j)
            nb = k // 32 * n0
            reps = n // n0
            w = np.tile(base, reps) if fmt == FMT_Q8 else np.concatenate([np.tile(base[: nb * 4], reps), np.tile(base[nb * 4:], reps)])
            items.append((k, n, residual, src, w))
    return xs, items


def cpu_pass(coracle, fmt, xs, items, threads):
    """One pass of the oracle's f32 matmul over the buffers; returns (seconds, algorithmic bytes)."""
    t0 = time.perf_counter()
    nbytes = 0
    for k, n, residual, src, w in items:
        coracle.matmul(fmt, xs[src], w, k, n, wide=False, variant=0, nthreads=threads)
        nbytes += cpu_gemv_bytes(fmt, k, n, residual)
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


def cpu_timed(coracle, fmt, xs, items, threads, warmups, repeats):
    """Median GB/s over `repeats` passes after `warmups` untimed ones."""
    for _ in range(warmups):
        cpu_pass(coracle, fmt, xs, items, threads)
    rates, secs = [], []
    for _ in range(repeats):
        sec, nbytes = cpu_pass(coracle, fmt, xs, items, threads)
        rates.append(nbytes / sec / 1e9)
        secs.append(sec)
    rates.sort()
    return rates[len(rates) // 2], sum(secs), nbytes


def cpu_baseline(shape, fmt):
    coracle = build_fast_oracle()
    threads = os.cpu_count() or 1
    layers = 4                                         # 0.48 GB of distinct packed weights: well beyond the host caches
    xs, items = cpu_layer_buffers(shape, fmt, layers)
    value, total_s, nbytes = cpu_timed(coracle, fmt, xs, items, threads, warmups=3, repeats=7)
    one = items[: len(items) // layers]
    single, single_s, _ = cpu_timed(coracle, fmt, xs, one, 1, warmups=1, repeats=5)
    return {"value": round(value, 3), "unit": UNIT, "cores": threads, "kind": "port",
            "single_thread": round(single, 3),
            "sample": f"{layers} of {shape[1]} layers of the workload ({nbytes / 1e6:.0f} MB of GEMV bytes per pass), "
                      f"3 warm-ups, median of 7 passes ({total_s:.2f} s timed) on {threads} threads; single-thread figure: "
                      f"1 layer, median of 5 ({single_s:.2f} s); C restatement of the reference kernel math, f32"}


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
    layers = max(1, min(shape[1], int(90.0 / max(sec1 * total_steps, 1e-3))))
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
    sample = (f"each step = {layers} of {shape[1]} layers ({nbytes / args.steps / 1e6:.0f} MB of GEMV bytes) on "
              f"{threads} host threads; C restatement of meganeura's quantized matmul math "
              "(the Rust/WGSL reference needs cargo and Vulkan: unavailable on this box)")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(shape, fmt, args.batch, args.gpus, "plan"),
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------- GPU arm

def cuda_timed(fn, launches, warmup=3):
    """Average milliseconds per call of fn over `launches` calls (CUDA events on the current stream)."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / launches


def decode_tokens_per_s(model: str, steps: int = 128, context: int = 2048):
    """Whole-model greedy decode through Graph / build_inference_session / Session: every operator
    of the step (embedding, norms, RoPE, cache writes, attention, SwiGLU, the quantized GEMVs and
    the greedy pick) runs on the GPU from one captured CUDA graph per token; the host only launches.
    KV caches are pre-filled to `context` positions; weights are seeded N(0, 0.02^2) matrices run
    through the quantizer, distinct for every tensor of every layer."""
    import numpy as np
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
    first = s.read_output(cfg.vocab_size)
    finite = bool(np.isfinite(first).all())
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
    last = s.read_output(cfg.vocab_size)
    finite = finite and bool(np.isfinite(last).all())
    plan = s.plan().dispatches
    kv_bytes = 2 * cfg.num_hidden_layers * cfg.kv_dim * 4 * (context + steps // 2)
    distinct = int(len(set(int(t) for t in tokens)))
    out = {"model": f"{cfg.name}-shaped, seeded N(0,0.02^2) weights through the quantizer", "tokens_per_s": round(steps / dt, 1),
           "ms_per_token": round(dt / steps * 1e3, 4), "steps": steps, "kv_context": context, "batch": 1,
           "launches_per_token": len(plan) + 1, "greedy_pick": "device", "timing": "host wall clock around launch + final token read",
           "weight_plus_kv_gbs": round((M.packed_weight_bytes(cfg) + kv_bytes) / (dt / steps) / 1e9, 1),
           "distinct_tokens": distinct, "logits_finite": finite, "build_s": round(build_s, 1)}
    if distinct <= 1 or not finite:
        out["invalid"] = "degenerate decode: one distinct token or non-finite logits"
    return out


def decode_sharded_tokens_per_s(model: str, rank: int, world: int, steps: int = 128, context: int = 2048):
    """The same whole-model greedy decode column-sharded over `world` GPUs: every rank holds its
    column range of every projection and its heads' KV cache and runs its own captured CUDA graph;
    slices travel through all_gathers over peer memory (four per layer and the logits).  Timed by
    the host clock on every rank (launch of `steps` tokens to the last token read), max over ranks.
    Checked: every rank picked the same tokens, and they are the tokens the unsharded model picks
    on rank 0's GPU (the logits are bit-identical by construction)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from meganeura_b200 import decode_model as M
    cfg = M.QWEN3_8B if model == "qwen3-8b" else M.SMOLLM2_135M
    try:
        M.check_world(cfg, world)
    except ValueError as e:
        return {"skipped": str(e)}
    if cfg is M.SMOLLM2_135M:
        context = 128
    max_seq = context + steps + 8
    dec = M.DecodeSession(cfg, max_seq, seed=3, greedy_history=max_seq, rank=rank, world=world)
    dec.fill_caches(context)
    s = dec.session
    dist.barrier()
    dec.set_position(1, context)
    s.step()
    s.wait()
    s.capture()
    dec.set_position(1, context)
    for _ in range(3):
        s.step()
    s.wait()
    dec.set_position(1, context)
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        s.step()
    s.wait()
    tokens = np.asarray(s.read_tokens(context, steps), dtype=np.int64)
    dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
    dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    dt = float(dt.item())
    timeout = False
    try:
        dec.check_exchange()
    except Exception:
        timeout = True
    finite = bool(np.isfinite(s.read_output(cfg.vocab_size)).all())
    mine = torch.from_numpy(tokens).cuda()
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    same = all(bool(torch.equal(t, mine)) for t in everyone)
    flag = torch.tensor([1 if timeout else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    launches = len(s.plan().dispatches) + 2
    del dec, s
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    ref = M.DecodeSession(cfg, max_seq, seed=3, greedy_history=max_seq)
    ref.fill_caches(context)
    ref.set_position(1, context)
    for _ in range(steps):
        ref.step()
    ref.session.wait()
    want = np.asarray(ref.session.read_tokens(context, steps), dtype=np.int64)
    distinct = int(len(set(int(t) for t in tokens)))
    out = {"model": f"{cfg.name}-shaped, column-sharded over {world} GPUs", "tokens_per_s": round(steps / dt, 1),
           "ms_per_token": round(dt / steps * 1e3, 4), "steps": steps, "kv_context": context, "batch": 1,
           "launches_per_token": launches, "all_gathers_per_token": 4 * cfg.num_hidden_layers + 1,
           "timing": "host wall clock, launch of the first token to the last token read, max over ranks",
           "same_tokens_on_every_rank": same, "tokens_equal_unsharded_model": bool(np.array_equal(tokens, want)),
           "distinct_tokens": distinct, "logits_finite": finite, "wait_ran_out": bool(flag.item())}
    if not (same and out["tokens_equal_unsharded_model"] and finite) or out["wait_ran_out"] or distinct <= 1:
        out["invalid"] = "sharded decode differs from the unsharded model, is degenerate, or a wait ran out"
    return out


def gemm_case(peak_tflops, which):
    """BASELINE config 3: Q8 prefill GEMM 512 x 4096 x 14336, bf16 activations, on the tcgen05 kernel."""
    import torch
    from meganeura_b200 import ops, synth
    m, k, n = 512, 4096, 14336
    base, n0, reps = synth.synth_weights_tiled(FMT_Q8, k, n, 1)
    w = synth.tile_columns(FMT_Q8, torch.from_numpy(base).cuda(), k, n0, reps)
    a = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    c = torch.empty((m, n), device="cuda")
    ms = cuda_timed(lambda: ops.matmul(FMT_Q8, a, w, k, n, out=c, route="gemm"), 50, warmup=5)
    ops.device_status()
    tf = 2.0 * m * k * n / (ms * 1e-3) / 1e12
    return {"shape": f"Q8 {m}x{k}x{n}, bf16 activations, f32 accumulate", "us": round(ms * 1e3, 2), "launches": 50,
            "tflops": round(tf, 1), "flops": "2*M*K*N (the kernel executes twice that for its hi/lo weight split)",
            "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peak_tflops, "unit": "TFLOP/s",
                         "frac": round(tf / peak_tflops, 4), "peak_source": f"of {which} (bf16_tflops, burst)"}}


def gemv_cases(peak):
    """BASELINE configs 0 and 1 in the streaming regime: each launch reads a different weight copy
    (copies x bytes >= 4 x L2), launches replayed from a CUDA graph."""
    import torch
    from meganeura_b200 import ops, synth
    out = []
    for fmt, k, n in [(FMT_Q8, 576, 1536), (FMT_Q4, 576, 576), (FMT_Q4, 576, 192), (FMT_Q4, 576, 1536), (FMT_Q4, 1536, 576),
                      (FMT_Q4, 576, 3072), (FMT_Q4, 576, 49152)]:
        w = torch.from_numpy(synth.synth_weights(fmt, k, min(n, 1536), 7)).cuda()
        if n > 1536:
            w = synth.tile_columns(fmt, w, k, 1536, n // 1536)
        nbytes = w.numel()
        copies = max(2, min(1024, int(520e6 // nbytes) + 1))
        ws = [w] + [w.clone() for _ in range(copies - 1)]
        x = torch.randn((1, k), device="cuda")
        y = torch.empty((1, n), device="cuda")
        ops.matmul(fmt, x, ws[0], k, n, out=y, route="gemv")
        torch.cuda.synchronize()
        graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for wc in ws:
                    ops.matmul(fmt, x, wc, k, n, out=y, route="gemv")
        ms = cuda_timed(graph.replay, 5, warmup=2)
        us = ms * 1e3 / copies
        alg = nbytes + 4 * (k + n)
        out.append({"shape": f"{'Q4' if fmt == FMT_Q4 else 'Q8'} {k}x{n}", "us": round(us, 3), "gbs": round(alg / us / 1e3, 1),
                    "frac": round(alg / us / 1e3 / peak, 4), "weight_copies": copies})
    return out


def workload_config(shape, fmt, batch, gpus, mode, exchange="peer"):
    if gpus > 1:
        how = ("slices stored into every peer's gathered vector by the persistent kernel (NVLink stores, {value, stamp} elements)"
               if mode == "plan" else
               ("slices pushed into every peer's buffer by the GEMV kernels" if exchange == "peer" else "NCCL all-gather"))
        par = f"columns sharded x{gpus}, all-gather of activations after every GEMV: {how}"
    else:
        par = "single GPU"
    return {
        "workload": f"{shape[0]}-shaped decode token, all {'Q4' if fmt == FMT_Q4 else 'Q8'} GEMVs "
                    f"({shape[1]} layers x q|k|v,o,gate|up,down + lm_head), chained through their data, batch {batch}",
        "weights": "seeded N(0, 0.02^2) f32 matrices through the reference's quantizer (periodic extension of 256-column bases)",
        "activations": "f32 N(0,1) token vector, seeded; every other GEMV reads its predecessor's output",
        "parallelism": par,
        "l2": "no flush needed: each step streams its weights once, 4-37x the 126 MB L2",
        "launch": ("one persistent cooperative kernel per token (mgq_plan), replayed from a CUDA graph" if mode == "plan"
                   else "one kernel per GEMV, one CUDA graph per token"),
    }


def parity_check(chain, coracle_threads=8):
    """The chain's results against the CPU oracle and against an independent GPU path.

    (1) layer 0, op by op, against the f64 oracle fed with its own previous output; (2) the last op
    (lm_head) against the oracle fed with the activations the GPU used; (3) the whole chain's logits
    against the same chain run as one launch per GEMV (different kernels, same weights)."""
    import numpy as np
    import torch
    from oracle import oracle as O
    co = O.COracle()
    fmt = chain.fmt
    worst = 0.0
    chain.step()
    torch.cuda.synchronize()
    want = chain.x0.cpu().numpy()
    for i in range(min(4, len(chain.ops_list))):
        op = chain.ops_list[i]
        sp = op["spec"]
        add = op["addend"].cpu().numpy() if op["addend"] is not None else None
        full = co.matmul(fmt, want[:, : sp.k], op["w"].cpu().numpy(), sp.k, op["n_loc"], addend=add, wide=True, nthreads=coracle_threads)
        worst = max(worst, O.rel_l2(op["y"].cpu().numpy(), full))
        want = full.astype(np.float32)
    head = chain.ops_list[-1]
    x_used = chain.ops_list[-2]["y"][:, : head["spec"].k].cpu().numpy()
    cols = 4096                                             # a strip of the lm_head is enough for the oracle
    w_strip = O.shard_columns_np(fmt, head["w"].cpu().numpy(), head["spec"].k, head["n_loc"], head["n_loc"] - cols, head["n_loc"])
    strip = co.matmul(fmt, x_used, w_strip, head["spec"].k, cols, wide=True, nthreads=coracle_threads)
    worst = max(worst, O.rel_l2(head["y"][:, -cols:].cpu().numpy(), strip))
    logits_plan = chain.logits_view().clone()
    finite = bool(torch.isfinite(logits_plan).all())
    mode, graph = chain.mode, chain.graph
    chain.mode, chain.graph = ("launches" if mode == "plan" else "plan"), None
    chain.step()
    torch.cuda.synchronize()
    logits_launch = chain.logits_view().clone()
    chain.mode, chain.graph = mode, graph
    chain.step()                                            # leave the measured mode's results in the buffers
    torch.cuda.synchronize()
    rel = float((logits_plan.double() - logits_launch.double()).norm() / logits_launch.double().norm())
    # every GEMV of the chain on its own: the stand-alone GEMV kernel fed with the activations the measured run used
    from meganeura_b200 import ops
    per_op = 0.0
    for i, op in enumerate(chain.ops_list):
        sp = op["spec"]
        x_in = chain.x0 if i == 0 else chain.ops_list[i - 1]["y"][:, : sp.k]
        ref = ops.matmul(fmt, x_in, op["w"], sp.k, op["n_loc"], addend=op["addend"], route="gemv")
        per_op = max(per_op, float((op["y"].double() - ref.double()).norm() / ref.double().norm()))
    # per-op results are held to 1e-4; the whole chain of 145 dependent GEMVs multiplies rounding differences
    # between the two kernels (f32 summation order), so its end-to-end figure is held to 1e-3
    ok = finite and worst <= 1e-4 and per_op <= 1e-4 and rel <= 1e-3
    return {"ok": ok, "rel_l2_vs_oracle": float(f"{worst:.3e}"), "max_rel_l2_per_op_vs_gemv_kernel": float(f"{per_op:.3e}"),
            "rel_l2_chain_vs_other_mode": float(f"{rel:.3e}"),
            "tolerance": 1e-4, "chain_tolerance": 1e-3, "logits_finite": finite,
            "what": "layer 0 op by op and a 4096-column strip of lm_head vs the f64 CPU oracle; every GEMV vs the stand-alone kernel on the same activations; final logits vs the other way of running the chain"}


def parity_check_sharded(chain, shape_key, fmt, seed):
    """N > 1: every rank's gathered logits must equal the all-gather of the ranks' slices, be the same
    on every rank, and match the unsharded chain (same seeds) run on rank 0's GPU alone."""
    import torch
    import torch.distributed as dist
    from meganeura_b200 import decode_chain as dc
    world, rank = chain.world, chain.rank
    dist.barrier()                                  # ranks may be seconds apart here (rank 0 has just stopped its clock sampler)
    chain.step()
    torch.cuda.synchronize()
    timed_out = chain.check_error()
    mine = chain.head["y"][0].contiguous()
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    gathered = chain.logits_view().reshape(-1).contiguous()
    same_as_slices = bool(torch.equal(gathered, torch.cat(parts)))
    copies = [torch.empty_like(gathered) for _ in range(world)]
    dist.all_gather(copies, gathered)
    same_on_all = all(bool(torch.equal(c, copies[0])) for c in copies)
    finite = bool(torch.isfinite(gathered).all())
    rel, exact, where = None, None, None
    if rank == 0:
        shape = dc.QWEN3_8B if shape_key == "qwen3-8b" else dc.SMOLLM2_135M
        single = dc.DecodeGemvChain(shape, fmt, rank=0, world=1, seed=seed, mode=chain.mode if chain.mode == "plan" else "launches")
        single.step()
        torch.cuda.synchronize()
        ref = single.logits_view().reshape(-1)
        rel = float((gathered.double() - ref.double()).norm() / ref.double().norm())
        exact = bool(torch.equal(gathered, ref))
        where = None
        if not exact:                                   # name the first GEMV whose slice on this rank differs
            where = "input vector" if not torch.equal(single.x0, chain.x0) else None
            for i, (a, b) in enumerate(zip(chain.ops_list, single.ops_list)):
                if where:
                    break
                off_c = off_s = 0
                for gw in a["spec"].groups:
                    per = gw // world
                    if not torch.equal(a["y"][0, off_c:off_c + per], b["y"][0, off_s + rank * per: off_s + (rank + 1) * per]):
                        where = f"op {i} ({a['spec'].name})"
                        break
                    off_c += per
                    off_s += gw
        del single
    flag = torch.tensor([1 if (same_as_slices and same_on_all and finite and not timed_out) else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ok = bool(flag.item()) and (rel is None or rel <= 1e-4)
    return {"ok": ok, "rel_l2_vs_single_gpu": rel, "bit_exact_vs_single_gpu": exact, "first_difference": where if rank == 0 else None,
            "gathered_equals_all_gather_of_slices": same_as_slices,
            "identical_on_all_ranks": same_on_all, "logits_finite": finite, "tolerance": 1e-4,
            "what": "gathered logits vs NCCL all-gather of the ranks' slices, across ranks, and vs the unsharded chain on rank 0's GPU"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--fmt", choices=["q4", "q8"], default="q4")
    ap.add_argument("--model", choices=["qwen3-8b", "smollm2-135m"], default="qwen3-8b")
    ap.add_argument("--impl", choices=["mgq", "reference"], default="mgq")
    ap.add_argument("--mode", choices=["auto", "plan", "launches"], default="auto",
                    help="plan: one persistent kernel per token; launches: one kernel per GEMV; auto (default): on one GPU "
                         "whichever of the two is faster in a short calibration, on several GPUs the persistent kernel")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="launches mode on several GPUs: slices pushed over NVLink by the GEMV kernels (default) or NCCL all-gather")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the extra keys (gemm, gemv_cases, batch8, per_gemv_launches, decode)")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-model decode tokens/s measurement")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "mgq" else args.warmup
    shape_t = SHAPES[args.model]
    fmt = FMT_Q4 if args.fmt == "q4" else FMT_Q8

    if args.impl == "reference":
        run_reference(args, shape_t, fmt)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path (use --impl reference for the CPU arm)")
    from meganeura_b200 import decode_chain as dc
    shape = dc.QWEN3_8B if args.model == "qwen3-8b" else dc.SMOLLM2_135M
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    mode = args.mode if args.batch == 1 else "launches"
    calibration = None
    if mode == "auto":
        mode = "plan"
    exchange = args.exchange if mode == "launches" else "peer"
    chain = dc.DecodeGemvChain(shape, fmt, batch=args.batch, rank=rank, world=world, seed=0, mode=mode, exchange=exchange)
    captured = chain.capture()
    if args.mode == "auto" and world == 1 and args.batch == 1:
        # both ways of running the token, a few steps each; the faster one is what gets measured
        ms_plan = cuda_timed(chain.step, 8, warmup=3)
        chain.mode, chain.graph = "launches", None
        chain.capture()
        ms_launch = cuda_timed(chain.step, 8, warmup=3)
        calibration = {"plan_ms": round(ms_plan, 4), "launches_ms": round(ms_launch, 4)}
        if ms_plan <= ms_launch:
            chain.mode, chain.graph = "plan", None
            captured = chain.capture()
        mode = chain.mode

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
    if chain.check_error():
        raise SystemExit("a bounded device-side wait ran out (MGQ_ERR_TIMEOUT): results are invalid")

    launches_per_step = chain.launches_per_step
    check = parity_check_sharded(chain, args.model, fmt, 0) if world > 1 else (parity_check(chain) if args.batch == 1 else None)

    bytes_rank = chain.bytes_per_step()
    total_bytes = bytes_rank * world
    ms_step = ms_dev / args.steps
    value = total_bytes / (ms_step * 1e-3) / 1e9
    e2e_value = total_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    launches = launches_per_step * args.steps * 2               # device-timed steps + end-to-end steps

    if rank == 0:
        peak, peak_tf, which = measured_peaks()
        achieved = bytes_rank / (ms_step * 1e-3) / 1e9
        kernel = "chain_kernel (persistent plan)" if mode == "plan" else ("gemv_q4_kernel" if fmt == FMT_Q4 else "gemv_q8_kernel")
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(shape_t, fmt, args.batch, world, mode, exchange),
            "tokens_per_s": round(args.batch / (ms_step * 1e-3), 1),
            "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": chain.h2d_bytes(),
                    "d2h_bytes_per_step": chain.d2h_bytes(), "ms_per_step": round(ms_e2e / args.steps, 4),
                    "tokens_per_s": round(args.batch / (ms_e2e / args.steps * 1e-3), 1)},
            "gpu_launches": launches, "launches_per_step": launches_per_step, "mode": mode, "mode_calibration": calibration,
            "cuda_graph": captured,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": UNIT,
                         "frac": round(achieved / peak, 4), "peak_source": f"of {which} (MEASURED_PEAKS.json hbm_gbs)",
                         "frac_of_nominal_8000": round(achieved / 8000.0, 4), "kernel": kernel,
                         "bytes_per_launch": round(bytes_rank / launches_per_step),
                         "us_per_launch": round(ms_step * 1e3 / launches_per_step, 3),
                         "traffic": None},
            "clocks": clocks,
            "parity_check": check,
            "logits_sha1": hashlib.sha1(chain.logits_view().contiguous().cpu().numpy().tobytes()).hexdigest(),
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(shape_t, fmt)
        if world == 1 and args.batch == 1 and not args.no_extras:
            # The extra measurements must never cost the line above them: whatever goes wrong in one of them is
            # recorded under "extras_error" and the line is printed with the extras measured so far.
            try:
                # the same chain run the other way (one launch per GEMV with programmatic dependent launch, or the
                # persistent plan kernel), CUDA graph, same weights
                other = "launches" if mode == "plan" else "plan"
                chain.mode, chain.graph = other, None
                chain.capture()
                ms_l = cuda_timed(chain.step, args.steps, warmup=args.warmup)
                line["other_mode"] = {"mode": other, "ms_per_step": round(ms_l, 4), "gbs": round(bytes_rank / ms_l / 1e6, 1),
                                      "frac": round(bytes_rank / ms_l / 1e6 / peak, 4), "launches_per_step": chain.launches_per_step}
                chain.graph = None
                del chain
                torch.cuda.empty_cache()
                b8 = dc.DecodeGemvChain(shape, fmt, batch=8, seed=0, mode="launches")
                b8.capture()
                ms8 = cuda_timed(b8.step, max(5, args.steps // 2), warmup=3)
                line["batch8"] = {"ms_per_step": round(ms8, 4), "tokens_per_s": round(8 / (ms8 * 1e-3), 1),
                                  "weight_gbs": round(b8.bytes_per_step() / ms8 / 1e6, 1), "kernel": "gemv_mma_kernel (8 rows per pass over W)"}
                b8.graph = None
                del b8
                torch.cuda.empty_cache()
                line["gemm"] = gemm_case(peak_tf, which)
                line["gemv_cases"] = gemv_cases(peak)
                if not args.no_decode:
                    line["decode"] = decode_tokens_per_s(args.model)
                    other = "smollm2-135m" if args.model == "qwen3-8b" else "qwen3-8b"
                    line["decode_" + other.split("-")[0]] = decode_tokens_per_s(other)
            except Exception as exc:
                line["extras_error"] = repr(exc)[:300]
    sharded, batch8, extras_error = None, None, None
    if world > 1 and args.batch == 1 and not args.no_extras:
        # The extra measurements must never cost the line above them.  They hold collectives, so an error on one
        # rank can leave the others waiting: rank 0 arms a timer that prints the line as it stands and ends the
        # process if the extras have not come back in time; an exception is recorded and the line is printed.
        def give_up():
            line["extras_error"] = "the extra measurements did not finish in 420 s"
            print(json.dumps(line), flush=True)
            os._exit(0)
        extras_timer = threading.Timer(420.0, give_up) if rank == 0 else None
        if extras_timer is not None:
            extras_timer.daemon = True
            extras_timer.start()
        try:
            chain.graph = None
            # eight tokens per step over the same column shards: the 8-row GEMV kernel, then an all-gather kernel that stores
            # the rank's rows into every peer's gathered vector and unpacks the whole; NCCL all-gathers timed beside it
            b8 = dc.DecodeGemvChain(shape, fmt, batch=8, rank=rank, world=world, seed=0, mode="launches", exchange="peer")
            b8.capture()
            dist.barrier()
            ms8 = torch.tensor([cuda_timed(b8.step, max(5, args.steps // 2), warmup=3)], device="cuda")
            dist.all_reduce(ms8, op=dist.ReduceOp.MAX)
            ms8 = float(ms8.item())
            bad8 = torch.tensor([1 if b8.check_error() else 0], device="cuda")
            dist.all_reduce(bad8, op=dist.ReduceOp.MAX)
            peer_logits = b8.logits_view().clone()
            bytes8 = b8.bytes_per_step()
            b8.graph = None
            del b8
            torch.cuda.empty_cache()
            b8 = dc.DecodeGemvChain(shape, fmt, batch=8, rank=rank, world=world, seed=0, mode="launches", exchange="nccl")
            b8.capture()
            dist.barrier()
            ms8n = torch.tensor([cuda_timed(b8.step, max(5, args.steps // 2), warmup=3)], device="cuda")
            dist.all_reduce(ms8n, op=dist.ReduceOp.MAX)
            same8 = torch.tensor([1 if bool(torch.equal(peer_logits, b8.logits_view())) else 0], device="cuda")
            dist.all_reduce(same8, op=dist.ReduceOp.MIN)
            batch8 = {"ms_per_step": round(ms8, 4), "tokens_per_s": round(8 / (ms8 * 1e-3), 1),
                      "weight_gbs": round(bytes8 * world / ms8 / 1e6, 1), "exchange": "all-gather kernel over peer memory",
                      "kernel": "gemv_mma_kernel (8 rows per pass over W)", "nccl_ms_per_step": round(float(ms8n.item()), 4),
                      "logits_equal_nccl_path": bool(same8.item()), "wait_ran_out": bool(bad8.item())}
            if not batch8["logits_equal_nccl_path"] or batch8["wait_ran_out"]:
                batch8["invalid"] = "the two exchange paths disagree or a wait ran out"
            b8.graph = None
            del b8
            torch.cuda.empty_cache()
            if not args.no_decode:
                sharded = decode_sharded_tokens_per_s(args.model, rank, world)
        except Exception as exc:
            extras_error = repr(exc)[:300]
        if extras_timer is not None:
            extras_timer.cancel()
    if rank == 0:
        if batch8 is not None:
            line["batch8"] = batch8
        if sharded is not None:
            line["decode_sharded"] = sharded
        if extras_error is not None:
            line["extras_error"] = extras_error
        print(json.dumps(line))
        if check is not None and not check["ok"]:
            sys.stdout.flush()
            if world == 1:
                raise SystemExit("parity check failed: " + json.dumps(check))
    if world > 1:
        # A captured graph that holds NCCL nodes must go before the communicator does (destroying the
        # process group first blocks forever); a watchdog ends the process if teardown still stalls.
        sys.stdout.flush()
        bad = check is not None and not check["ok"]
        watchdog = threading.Timer(60.0, lambda: os._exit(1 if bad else 0))
        watchdog.daemon = True
        watchdog.start()
        dist.barrier()
        torch.cuda.synchronize()
        try:
            chain.graph = None
        except NameError:
            pass
        dist.destroy_process_group()
        watchdog.cancel()
        if bad:
            raise SystemExit("parity check failed")


if __name__ == "__main__":
    main()
