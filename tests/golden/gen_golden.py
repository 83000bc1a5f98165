"""Regenerates tests/golden/q4q8_golden.npz.

The reference (Rust + WGSL) cannot run in this environment, so these vectors come from the
numpy restatement in oracle/oracle.py, which follows src/runtime.rs:2035-2215 line by line.
Inputs are the reference's own test formulas where it has them:

  ident_*   q4_roundtrip_identity   src/runtime.rs:2222-2242   32x1, (i-16)*0.1
  mat_*     q4_roundtrip_matrix     src/runtime.rs:2245-2266   32x4, ((i%17)-8)*0.05
  smoke_*   q4_matmul_correctness   tests/gpu_smoke.rs:2705-2712 formulas at m=6, k=64, n=12
  synth_*   seeded weights with the benchmark's distributions (64x8), x ~ N(0,1)

Run:  python tests/golden/gen_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402


def main():
    out = {}
    ident = ((np.arange(32, dtype=np.float32) - np.float32(16.0)) * np.float32(0.1)).reshape(32, 1)
    mat = (((np.arange(128) % 17).astype(np.float32) - np.float32(8.0)) * np.float32(0.05)).reshape(32, 4)
    m, k, n = 6, 64, 12
    a = (((np.arange(m * k) % 7).astype(np.float32) - np.float32(3.0)) * np.float32(0.5)).reshape(m, k)
    i = np.arange(k * n)
    b = ((i % 11).astype(np.float32) - np.float32(5.0)) * np.float32(0.3)
    b = np.where(i % 1000 == 0, b * np.float32(5.0), b).astype(np.float32).reshape(k, n)
    for name, w in (("ident", ident), ("mat", mat), ("smoke", b)):
        out[f"{name}_w"] = w
        out[f"{name}_q4"] = O.quantize_q4_np(w)
        out[f"{name}_q8"] = O.quantize_q8_np(w)
        out[f"{name}_dq4"] = O.dequantize_q4_np(out[f"{name}_q4"], *w.shape)
        out[f"{name}_dq8"] = O.dequantize_q8_np(out[f"{name}_q8"], *w.shape)
    out["smoke_a"] = a
    out["smoke_c_q4"] = O.matmul_f64_np(O.FMT_Q4, a, out["smoke_q4"], k, n)
    out["smoke_c_q8"] = O.matmul_f64_np(O.FMT_Q8, a, out["smoke_q8"], k, n)
    rng = np.random.Generator(np.random.PCG64(20240))
    x = rng.standard_normal((2, 64)).astype(np.float32)
    d = rng.standard_normal((2, 8)).astype(np.float32)
    out["synth_x"] = x
    out["synth_addend"] = d
    for fmt, tag in ((O.FMT_Q4, "q4"), (O.FMT_Q8, "q8")):
        w = O.synth_weights(fmt, 64, 8, seed=7 + fmt)
        out[f"synth_{tag}"] = w
        out[f"synth_y_{tag}"] = O.matmul_f64_np(fmt, x, w, 64, 8, addend=d)
        out[f"synth_shard_{tag}"] = O.shard_columns_np(fmt, w, 64, 8, 4, 8)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "q4q8_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
