"""Seeded synthetic packed weights in the reference's byte layout (data generation only).

The benchmark configurations describe weights by their codes and scales, not by f32 values:
codes uniform (Q8: int8 in [-127,127]; Q4: nibbles 0..15 with offset 8), one scale per
32-element block drawn log-uniform in [1e-3, 1e-1].  The layout stores binary16 scales
(src/codegen.rs:748-805 of meganeura), so the drawn scale is rounded to binary16 and that value
is the weight's scale; Q4 offset 8 is the header m = -8*d, exact in binary16.
"""
from __future__ import annotations

import numpy as np

from ._lib import FMT_Q4, FMT_Q8


def pack_q4(codes: np.ndarray, d_bits: np.ndarray, m_bits: np.ndarray) -> np.ndarray:
    """codes [K,N] uint8 (0..15); d_bits, m_bits [N, K/32] uint16 -> [headers][nibbles] bytes."""
    k, n = codes.shape
    bpc = k // 32
    hdr = d_bits.astype(np.uint32) | (m_bits.astype(np.uint32) << 16)
    q = codes.reshape(bpc, 32, n)
    nib = (q[:, 0::2, :] | (q[:, 1::2, :] << 4)).astype(np.uint8)            # [b, 16, n]
    nib = np.ascontiguousarray(nib.transpose(2, 0, 1))                        # block = n*bpc + b
    return np.concatenate([np.ascontiguousarray(hdr).reshape(-1).view(np.uint8), nib.reshape(-1)])


def pack_q8(codes: np.ndarray, scale_bits: np.ndarray) -> np.ndarray:
    """codes [K,N] int8; scale_bits [N, K/32] uint16 -> 36-byte blocks."""
    k, n = codes.shape
    bpc = k // 32
    out = np.zeros((n, bpc, 36), dtype=np.uint8)
    out[:, :, 0:2] = np.ascontiguousarray(scale_bits.astype(np.uint16))[:, :, None].view(np.uint8).reshape(n, bpc, 2)
    out[:, :, 4:] = np.ascontiguousarray(codes.reshape(bpc, 32, n).transpose(2, 0, 1)).view(np.uint8)
    return out.reshape(-1)


def synth_weights(fmt: int, k: int, n: int, seed: int) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed))
    bpc = k // 32
    scale = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=(n, bpc))).astype(np.float32).astype(np.float16)
    if fmt == FMT_Q8:
        codes = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
        return pack_q8(codes, scale.view(np.uint16))
    if fmt != FMT_Q4:
        raise ValueError("format must be Q4 or Q8")
    codes = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    m = (np.float16(-8.0) * scale).astype(np.float16)
    return pack_q4(codes, scale.view(np.uint16), m.view(np.uint16))


def tile_columns(fmt: int, packed, k: int, n: int, reps: int):
    """The packed [k, n] weight repeated `reps` times along N (numpy array or torch tensor).

    Columns are independent in both layouts, so the result is a valid packed [k, n*reps] weight.
    """
    nb = (k // 32) * n
    if isinstance(packed, np.ndarray):
        if fmt == FMT_Q8:
            return np.tile(packed, reps)
        return np.concatenate([np.tile(packed[: nb * 4], reps), np.tile(packed[nb * 4:], reps)])
    import torch
    if fmt == FMT_Q8:
        return packed.repeat(reps)
    return torch.cat([packed[: nb * 4].repeat(reps), packed[nb * 4:].repeat(reps)])


def synth_weights_tiled(fmt: int, k: int, n: int, seed: int, base_cols: int = 512):
    """Large synthetic weight built from a seeded base of about `base_cols` columns (host array).

    Returns (base, n0, reps) with n0*reps == n; use tile_columns on the host or on the device.
    """
    reps = 1
    for r in range(max(1, n // base_cols), 0, -1):
        if n % r == 0 and (n // r) % 4 == 0:
            reps = r
            break
    n0 = n // reps
    return synth_weights(fmt, k, n0, seed), n0, reps
