"""CPU oracle for the Q4/Q8 quantized matmul path -- TEST INFRASTRUCTURE ONLY.

Two independent restatements of the reference algorithm live here:

* ``COracle``: ctypes binding of ``mgq_oracle.c`` (plain C, the timed CPU baseline);
* the ``*_np`` functions: a vectorised numpy restatement used to cross-check the C
  file and to generate the byte fixtures committed under ``tests/golden/``.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` may import this module.  The product package never does.

Reference locations (paths inside the meganeura tree):
  quantize/dequantize Q4  src/runtime.rs:2035-2138
  quantize/dequantize Q8  src/runtime.rs:2143-2215
  shader f16 decode       src/codegen.rs:739-746
  matmul semantics        src/shaders/matmul.wgsl:42-108

Parity pin: see the header of ``mgq_oracle.c`` (the reference cannot be built here;
pinned on the reference's own formula-generated tests, tolerance-based).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

FMT_Q4 = 2
FMT_Q8 = 3

_HERE = os.path.dirname(os.path.abspath(__file__))


def build(force: bool = False, arch: str = "") -> str:
    """Compile mgq_oracle.c into liborc.so next to it (gcc only)."""
    so = os.path.join(_HERE, "liborc.so")
    src = os.path.join(_HERE, "mgq_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        cmd = ["gcc", "-O3", "-fPIC", "-ffp-contract=off", "-shared"]
        if arch:
            cmd.append(arch)
        cmd += ["-o", so, src, "-lm", "-lpthread"]
        subprocess.run(cmd, check=True)
    return so


def packed_bytes(fmt: int, k: int, n: int) -> int:
    blocks = (k * n + 31) // 32
    return blocks * (20 if fmt == FMT_Q4 else 36)


# --------------------------------------------------------------------------- numpy

def _round_half_away(v: np.ndarray) -> np.ndarray:
    """Rust f32::round(): halves go away from zero (np.round is half-to-even)."""
    v = v.astype(np.float32)
    return (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.float32)


def f16_bits_to_f32_shader_np(bits: np.ndarray) -> np.ndarray:
    bits = bits.astype(np.uint32)
    sign = (bits >> 15) & 1
    expo = (bits >> 10) & 0x1F
    mant = bits & 0x3FF
    out = (sign << 31) | ((expo + 112) << 23) | (mant << 13)
    out = np.where(expo == 0, sign << 31, out).astype(np.uint32)
    return out.view(np.float32)


def quantize_q4_np(data: np.ndarray) -> np.ndarray:
    """[K,N] f32 -> packed bytes, src/runtime.rs:2035-2102."""
    data = np.ascontiguousarray(data, dtype=np.float32)
    k, n = data.shape
    assert k % 32 == 0
    bpc = k // 32
    blk = data.reshape(bpc, 32, n)                     # [b, i, col]
    bmin = blk.min(axis=1)
    bmax = blk.max(axis=1)
    with np.errstate(divide="ignore", invalid="ignore"):
        d = np.where(bmax > bmin, (bmax - bmin) / np.float32(15.0), np.float32(1.0)).astype(np.float32)
        d_inv = np.where(d > 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    m = bmin.astype(np.float32)
    q = _round_half_away((blk - m[:, None, :]) * d_inv[:, None, :])
    q = np.clip(q, 0.0, 15.0).astype(np.uint8)         # [b, i, col]
    hdr = d.astype(np.float16).view(np.uint16).astype(np.uint32) | (
        m.astype(np.float16).view(np.uint16).astype(np.uint32) << 16)   # [b, col]
    hdr = np.ascontiguousarray(hdr.T)                  # block = col*bpc + b
    nib = q[:, 0::2, :] | (q[:, 1::2, :] << 4)         # [b, 16, col]
    nib = np.ascontiguousarray(nib.transpose(2, 0, 1)) # [col, b, 16]
    return np.concatenate([hdr.reshape(-1).view(np.uint8), nib.reshape(-1)])


def dequantize_q4_np(buf: np.ndarray, k: int, n: int, shader: bool = False) -> np.ndarray:
    bpc = k // 32
    nb = bpc * n
    hdr = buf[: nb * 4].view(np.uint32).reshape(n, bpc)
    if shader:
        d = f16_bits_to_f32_shader_np(hdr & 0xFFFF)
        m = f16_bits_to_f32_shader_np(hdr >> 16)
    else:
        d = (hdr & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32)
        m = (hdr >> 16).astype(np.uint16).view(np.float16).astype(np.float32)
    by = buf[nb * 4: nb * 20].reshape(n, bpc, 16)
    q = np.empty((n, bpc, 32), dtype=np.float32)
    q[:, :, 0::2] = by & 0xF
    q[:, :, 1::2] = by >> 4
    w = q * d[:, :, None] + m[:, :, None]              # f32 multiply then add, like the source
    return np.ascontiguousarray(w.reshape(n, k).T)


def quantize_q8_np(data: np.ndarray) -> np.ndarray:
    """[K,N] f32 -> packed bytes, src/runtime.rs:2143-2188."""
    data = np.ascontiguousarray(data, dtype=np.float32)
    k, n = data.shape
    assert k % 32 == 0
    bpc = k // 32
    blk = data.reshape(bpc, 32, n)
    absmax = np.abs(blk).max(axis=1)
    scale = np.where(absmax > 0, absmax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    inv = (np.float32(1.0) / scale).astype(np.float32)
    q = np.clip(_round_half_away(blk * inv[:, None, :]), -128.0, 127.0).astype(np.int8)
    out = np.zeros((n, bpc, 36), dtype=np.uint8)
    out[:, :, 0:2] = scale.astype(np.float16).view(np.uint16).T[:, :, None].view(np.uint8).reshape(n, bpc, 2)
    out[:, :, 4:] = q.transpose(2, 0, 1).view(np.uint8)
    return out.reshape(-1)


def dequantize_q8_np(buf: np.ndarray, k: int, n: int, shader: bool = False) -> np.ndarray:
    bpc = k // 32
    blk = buf.reshape(n, bpc, 36)
    sbits = np.ascontiguousarray(blk[:, :, 0:2]).view(np.uint16).reshape(n, bpc)
    scale = f16_bits_to_f32_shader_np(sbits) if shader else sbits.view(np.float16).astype(np.float32)
    q = np.ascontiguousarray(blk[:, :, 4:]).view(np.int8).astype(np.float32)
    w = q * scale[:, :, None]
    return np.ascontiguousarray(w.reshape(n, k).T)


def pack_q4_np(codes: np.ndarray, d_bits: np.ndarray, m_bits: np.ndarray) -> np.ndarray:
    """codes [K,N] uint8 in 0..15; d_bits/m_bits [N, K/32] uint16 -> packed bytes."""
    k, n = codes.shape
    bpc = k // 32
    hdr = d_bits.astype(np.uint32) | (m_bits.astype(np.uint32) << 16)
    q = codes.reshape(bpc, 32, n).astype(np.uint8)
    nib = q[:, 0::2, :] | (q[:, 1::2, :] << 4)
    nib = np.ascontiguousarray(nib.transpose(2, 0, 1))
    return np.concatenate([np.ascontiguousarray(hdr).reshape(-1).view(np.uint8), nib.reshape(-1)])


def pack_q8_np(codes: np.ndarray, scale_bits: np.ndarray) -> np.ndarray:
    """codes [K,N] int8; scale_bits [N, K/32] uint16 -> packed bytes."""
    k, n = codes.shape
    bpc = k // 32
    out = np.zeros((n, bpc, 36), dtype=np.uint8)
    out[:, :, 0:2] = np.ascontiguousarray(scale_bits.astype(np.uint16))[:, :, None].view(np.uint8).reshape(n, bpc, 2)
    out[:, :, 4:] = np.ascontiguousarray(codes.reshape(bpc, 32, n).transpose(2, 0, 1)).view(np.uint8)
    return out.reshape(-1)


def dequantize_np(fmt: int, buf: np.ndarray, k: int, n: int, shader: bool = False) -> np.ndarray:
    return (dequantize_q4_np if fmt == FMT_Q4 else dequantize_q8_np)(buf, k, n, shader)


def matmul_f64_np(fmt: int, a: np.ndarray, buf: np.ndarray, k: int, n: int, addend=None) -> np.ndarray:
    w = dequantize_np(fmt, buf, k, n).astype(np.float64)
    c = a.astype(np.float64) @ w
    if addend is not None:
        c = c + addend.astype(np.float64)
    return c


def shard_columns_np(fmt: int, buf: np.ndarray, k: int, n: int, n0: int, n1: int) -> np.ndarray:
    bpc = k // 32
    nb = bpc * n
    if fmt == FMT_Q8:
        return buf[n0 * bpc * 36: n1 * bpc * 36].copy()
    return np.concatenate([buf[n0 * bpc * 4: n1 * bpc * 4], buf[nb * 4 + n0 * bpc * 16: nb * 4 + n1 * bpc * 16]])


# --------------------------------------------------------------------------- C binding

_u8p = ctypes.POINTER(ctypes.c_uint8)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)


def _p(arr: np.ndarray, typ):
    return arr.ctypes.data_as(typ)


class COracle:
    """ctypes view of liborc.so (built on demand)."""

    def __init__(self, so: str | None = None):
        self.lib = ctypes.CDLL(so or build())
        L = self.lib
        sz = ctypes.c_size_t
        L.orc_packed_bytes.restype = sz
        L.orc_packed_bytes.argtypes = [ctypes.c_int, sz, sz]
        for name in ("orc_quantize_q4", "orc_quantize_q8"):
            getattr(L, name).argtypes = [_f32p, sz, sz, _u8p]
        for name in ("orc_dequantize_q4", "orc_dequantize_q8"):
            getattr(L, name).argtypes = [_u8p, sz, sz, _f32p]
        L.orc_f16_bits_to_f32_ieee.restype = ctypes.c_float
        L.orc_f16_bits_to_f32_ieee.argtypes = [ctypes.c_uint16]
        L.orc_f16_bits_to_f32_shader.restype = ctypes.c_float
        L.orc_f16_bits_to_f32_shader.argtypes = [ctypes.c_uint16]
        L.orc_f32_to_f16_bits.restype = ctypes.c_uint16
        L.orc_f32_to_f16_bits.argtypes = [ctypes.c_float]
        L.orc_matmul_f32.argtypes = [ctypes.c_int, _f32p, _u8p, _f32p, _f32p, sz, sz, sz, ctypes.c_int, ctypes.c_int]
        L.orc_matmul_f64.argtypes = [ctypes.c_int, _f32p, _u8p, _f32p, _f64p, sz, sz, sz, ctypes.c_int, ctypes.c_int]
        L.orc_pack_q4.argtypes = [_u8p, ctypes.POINTER(ctypes.c_uint16), ctypes.POINTER(ctypes.c_uint16), sz, sz, _u8p]
        L.orc_pack_q8.argtypes = [ctypes.POINTER(ctypes.c_int8), ctypes.POINTER(ctypes.c_uint16), sz, sz, _u8p]
        L.orc_shard_columns.argtypes = [ctypes.c_int, _u8p, sz, sz, sz, sz, _u8p]
        u32p = ctypes.POINTER(ctypes.c_uint32)
        for name in ("orc_dequant_q4_shader", "orc_dequant_q8_shader"):
            f = getattr(L, name)
            f.restype = ctypes.c_float
            f.argtypes = [u32p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32]

    def packed_bytes(self, fmt, k, n):
        return int(self.lib.orc_packed_bytes(fmt, k, n))

    def quantize(self, fmt, data: np.ndarray) -> np.ndarray:
        data = np.ascontiguousarray(data, dtype=np.float32)
        k, n = data.shape
        out = np.empty(packed_bytes(fmt, k, n), dtype=np.uint8)
        fn = self.lib.orc_quantize_q4 if fmt == FMT_Q4 else self.lib.orc_quantize_q8
        rc = fn(_p(data, _f32p), k, n, _p(out, _u8p))
        if rc:
            raise ValueError(f"oracle quantize failed rc={rc}")
        return out

    def dequantize(self, fmt, buf: np.ndarray, k, n) -> np.ndarray:
        out = np.empty((k, n), dtype=np.float32)
        fn = self.lib.orc_dequantize_q4 if fmt == FMT_Q4 else self.lib.orc_dequantize_q8
        rc = fn(_p(buf, _u8p), k, n, _p(out, _f32p))
        if rc:
            raise ValueError(f"oracle dequantize failed rc={rc}")
        return out

    def dequant_shader_elem(self, fmt, buf: np.ndarray, kk, nn, k, n) -> float:
        fn = self.lib.orc_dequant_q4_shader if fmt == FMT_Q4 else self.lib.orc_dequant_q8_shader
        return float(fn(buf.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), kk, nn, k, n))

    def matmul(self, fmt, a: np.ndarray, buf: np.ndarray, k, n, addend=None, wide=True, variant=0, nthreads=1):
        a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1, k)
        m = a.shape[0]
        add_p = None
        if addend is not None:
            addend = np.ascontiguousarray(addend, dtype=np.float32)
            add_p = _p(addend, _f32p)
        if wide:
            c = np.empty((m, n), dtype=np.float64)
            rc = self.lib.orc_matmul_f64(fmt, _p(a, _f32p), _p(buf, _u8p), add_p, _p(c, _f64p), m, k, n, variant, nthreads)
        else:
            c = np.empty((m, n), dtype=np.float32)
            rc = self.lib.orc_matmul_f32(fmt, _p(a, _f32p), _p(buf, _u8p), add_p, _p(c, _f32p), m, k, n, variant, nthreads)
        if rc:
            raise ValueError(f"oracle matmul failed rc={rc}")
        return c

    def pack_q4(self, codes, d_bits, m_bits):
        k, n = codes.shape
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        d_bits = np.ascontiguousarray(d_bits, dtype=np.uint16)
        m_bits = np.ascontiguousarray(m_bits, dtype=np.uint16)
        out = np.empty(packed_bytes(FMT_Q4, k, n), dtype=np.uint8)
        rc = self.lib.orc_pack_q4(_p(codes, _u8p), d_bits.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)),
                                  m_bits.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), k, n, _p(out, _u8p))
        assert rc == 0
        return out

    def pack_q8(self, codes, scale_bits):
        k, n = codes.shape
        codes = np.ascontiguousarray(codes, dtype=np.int8)
        scale_bits = np.ascontiguousarray(scale_bits, dtype=np.uint16)
        out = np.empty(packed_bytes(FMT_Q8, k, n), dtype=np.uint8)
        rc = self.lib.orc_pack_q8(codes.ctypes.data_as(ctypes.POINTER(ctypes.c_int8)),
                                  scale_bits.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), k, n, _p(out, _u8p))
        assert rc == 0
        return out

    def shard_columns(self, fmt, buf, k, n, n0, n1):
        out = np.empty(packed_bytes(fmt, k, n1 - n0), dtype=np.uint8)
        rc = self.lib.orc_shard_columns(fmt, _p(buf, _u8p), k, n, n0, n1, _p(out, _u8p))
        assert rc == 0
        return out


# --------------------------------------------------------------------------- synthetic inputs

def synth_weights(fmt: int, k: int, n: int, seed: int):
    """Seeded packed weights with the benchmark's distributions.

    Codes uniform (Q8: int8 in [-127,127]; Q4: nibbles 0..15), one scale per 32-element
    block drawn log-uniform in [1e-3, 1e-1] in f32 and rounded to f16 (the layout stores
    f16 scales).  Q4 uses offset 8: m = -8*d, exact in f16.  Returns packed bytes.
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    bpc = k // 32
    scale = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=(n, bpc))).astype(np.float32).astype(np.float16)
    if fmt == FMT_Q8:
        codes = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
        return pack_q8_np(codes, scale.view(np.uint16))
    codes = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    m = (np.float16(-8.0) * scale).astype(np.float16)
    return pack_q4_np(codes, scale.view(np.uint16), m.view(np.uint16))


def rel_l2(got: np.ndarray, want: np.ndarray) -> float:
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    den = float(np.linalg.norm(want))
    return float(np.linalg.norm(got - want)) / (den if den > 0 else 1.0)
