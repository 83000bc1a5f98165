"""Single-kernel timing cases (also the commands the ncu summaries under profiles/ were made with).

    python -m meganeura_b200.kernel_cases gemv q4 4096x151936 [--launches 3] [--rows 1]
    python -m meganeura_b200.kernel_cases gemm q8 512x4096x14336 [--launches 3]
    python -m meganeura_b200.kernel_cases sweep q4            # the SmolLM2-135M decode shapes
    python -m meganeura_b200.kernel_cases decode qwen3-8b --layers 4 --steps 4 [--context 2048]
    python -m meganeura_b200.kernel_cases chain q4 --layers 4 [--launches 3] [--no-head] [--mode plan|launches]

`gemv` rotates through enough distinct weight copies to exceed L2 several times over and replays
the launches from a CUDA graph, so the printed GB/s is a streaming (cold-cache) figure; with
--launches N it only issues N plain launches (what a profiler capture wants).
"""
from __future__ import annotations

import argparse

import torch

from . import ops, synth
from ._lib import FMT_Q4, FMT_Q8

SMOLLM2_SHAPES = [(576, 576), (576, 192), (576, 1536), (1536, 576), (576, 49152), (576, 3072)]


def _weights(fmt, k, n, seed=1):
    base, n0, reps = synth.synth_weights_tiled(fmt, k, n, seed)
    return synth.tile_columns(fmt, torch.from_numpy(base).cuda(), k, n0, reps)


def gemv_case(fmt, k, n, rows=1, launches=0, peak_gbs=None, hot=False):
    """hot=True keeps ONE weight copy (L2-resident for small shapes); the default rotates copies so
    that every launch streams from HBM."""
    w = _weights(fmt, k, n)
    nbytes = w.numel()
    copies = 1 if (launches or hot) else max(2, min(64, int(600e6 // nbytes) + 1))
    ws = [w] + [w.clone() for _ in range(copies - 1)]
    x = torch.randn((rows, k), device="cuda")
    y = torch.empty((rows, n), device="cuda")
    for i in range(max(launches, 3)):
        ops.matmul(fmt, x, ws[i % copies], k, n, out=y, route="gemv")
    torch.cuda.synchronize()
    if launches:
        return None
    per_graph = max(copies, 8)
    graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for i in range(per_graph):
                ops.matmul(fmt, x, ws[i % copies], k, n, out=y, route="gemv")
    alg = nbytes + 4 * rows * (k + n)
    reps = max(3, int(30e3 / max(1.0, alg / 3e6 * per_graph)))
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * per_graph)
    gbs = alg / us / 1e3
    tail = f" ({gbs / peak_gbs * 100:.1f}% of {peak_gbs:.0f})" if peak_gbs else ""
    print(f"gemv {'Q4' if fmt == FMT_Q4 else 'Q8'} m={rows} {k}x{n}: {nbytes / 1e6:.2f} MB packed, {us:.2f} us/launch, "
          f"{gbs:.1f} GB/s{tail}  [{'hot: ' if hot else ''}{copies} weight cop{'y' if copies == 1 else 'ies'}, {per_graph} launches per graph]")
    return gbs


def gemm_case(fmt, m, k, n, launches=0):
    w = _weights(fmt, k, n)
    a = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    c = torch.empty((m, n), device="cuda")
    for _ in range(max(launches, 3)):
        ops.matmul(fmt, a, w, k, n, out=c, route="gemm")
    torch.cuda.synchronize()
    ops.device_status()
    if launches:
        return None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        ops.matmul(fmt, a, w, k, n, out=c, route="gemm")
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 20
    tf = 2.0 * m * k * n / us / 1e6
    print(f"gemm {'Q4' if fmt == FMT_Q4 else 'Q8'} bf16 {m}x{k}x{n}: {us:.1f} us, {tf:.1f} TFLOP/s "
          f"(2*M*K*N; the kernel executes twice that for the hi/lo weight split)")
    return tf


def chain_case(fmt, layers, launches, head=True, peak_gbs=None, mode="plan"):
    """The decode GEMV chain (Qwen3-8B shapes, `layers` layers, optionally without the lm_head) as one
    persistent plan kernel per token (mode "plan") or one kernel per GEMV (mode "launches"): `launches`
    plain tokens for a profiler, else a timed loop."""
    from . import decode_chain as dc
    chain = dc.DecodeGemvChain(dc.QWEN3_8B, fmt, layers=layers, mode=mode)
    if not head:
        chain.ops_list.pop()
    nbytes = sum(dc.gemv_bytes(fmt, 1, op["spec"].k, op["n_loc"], op["spec"].residual) for op in chain.ops_list)
    for _ in range(max(launches, 3)):
        chain._launch_all()
    if chain.check_error():
        raise RuntimeError("a bounded device-side wait ran out")
    if launches:
        return None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        chain._launch_all()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 20
    gbs = nbytes / us / 1e3
    tail = f" ({gbs / peak_gbs * 100:.1f}% of {peak_gbs:.0f})" if peak_gbs else ""
    info = chain.plan.info() if chain.plan is not None else {"kernels_per_token": chain.launches_per_step}
    print(f"chain {'Q4' if fmt == FMT_Q4 else 'Q8'} {layers} layers{' + lm_head' if head else ''} ({mode}): {len(chain.ops_list)} GEMVs, "
          f"{nbytes / 1e6:.1f} MB, {us:.1f} us per token, {gbs:.1f} GB/s{tail}  {info}")
    return gbs


def decode_case(model, layers, steps, context):
    """A few whole decode steps of a shortened model through the session (plain launches, no graph):
    what a profiler capture of the decode-step operators wants."""
    import time
    from dataclasses import replace
    from . import decode_model as M
    cfg = replace(M.QWEN3_8B if model == "qwen3-8b" else M.SMOLLM2_135M, num_hidden_layers=layers)
    dec = M.DecodeSession(cfg, context + steps + 8, seed=3, greedy_history=context + steps + 8)
    dec.fill_caches(context)
    dec.set_position(1, context)
    dec.step()
    dec.session.wait()
    t0 = time.perf_counter()
    for _ in range(steps):
        dec.step()
    dec.session.wait()
    print(f"decode {cfg.name}, {layers} layers, context {context}: {(time.perf_counter() - t0) / steps * 1e3:.3f} ms/token "
          f"({len(dec.session.plan().dispatches) + 1} launches, no graph)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["gemv", "gemm", "sweep", "decode", "chain"])
    ap.add_argument("fmt", help="q4 | q8, or the model for `decode` (qwen3-8b | smollm2-135m)")
    ap.add_argument("shape", nargs="?", default="")
    ap.add_argument("--launches", type=int, default=0)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--peak-gbs", type=float, default=None)
    ap.add_argument("--hot", action="store_true", help="one weight copy: the L2-resident regime for small shapes")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--no-head", action="store_true", help="chain: leave the lm_head out (a small profiler case)")
    ap.add_argument("--mode", choices=["plan", "launches"], default="plan", help="chain: persistent kernel or one kernel per GEMV")
    args = ap.parse_args()
    if args.kind == "decode":
        if args.fmt not in ("qwen3-8b", "smollm2-135m"):
            ap.error("decode takes qwen3-8b or smollm2-135m")
        return decode_case(args.fmt, args.layers, args.steps, args.context)
    if args.fmt not in ("q4", "q8"):
        ap.error("format must be q4 or q8")
    fmt = FMT_Q4 if args.fmt == "q4" else FMT_Q8
    warm = torch.randn(8192, 8192, device="cuda")          # bring the clocks up
    for _ in range(10):
        warm @ warm
    torch.cuda.synchronize()
    del warm
    if args.kind == "chain":
        chain_case(fmt, args.layers, args.launches, head=not args.no_head, peak_gbs=args.peak_gbs, mode=args.mode)
    elif args.kind == "sweep":
        for k, n in SMOLLM2_SHAPES:
            gemv_case(fmt, k, n, peak_gbs=args.peak_gbs, hot=args.hot)
    elif args.kind == "gemv":
        k, n = (int(v) for v in args.shape.split("x"))
        gemv_case(fmt, k, n, rows=args.rows, launches=args.launches, peak_gbs=args.peak_gbs, hot=args.hot)
    else:
        m, k, n = (int(v) for v in args.shape.split("x"))
        gemm_case(fmt, m, k, n, launches=args.launches)


if __name__ == "__main__":
    main()
