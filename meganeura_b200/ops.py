"""Array-level entry points over the C ABI (numpy for host data, torch for device data).

These are thin argument marshallers: every computation happens in libmgq.
"""
from __future__ import annotations

import numpy as np

from . import _lib
from ._lib import A_BF16, A_F32, FMT_Q4, FMT_Q8, check, lib


def set_option(name: str, value: int) -> None:
    """Runtime option of the library (mgq_set_option), e.g. "gemv.serial_dispatch"."""
    check(lib.mgq_set_option(name.encode(), int(value)))


def device_status() -> None:
    """Raises MgqError(MGQ_ERR_TIMEOUT) if a bounded device-side wait ran out (mgq_device_status)."""
    check(lib.mgq_device_status())


def packed_bytes(fmt: int, k: int, n: int) -> int:
    return int(lib.mgq_packed_bytes(fmt, k, n))


def quantize(fmt: int, w: np.ndarray) -> np.ndarray:
    """Host quantizer: row-major [K,N] f32 -> packed bytes (quantize_q4_0 / quantize_q8_0)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.ndim != 2:
        raise ValueError("weights must be 2-D [K, N]")
    k, n = w.shape
    out = np.empty(packed_bytes(fmt, k, n) if k % 32 == 0 else 1, dtype=np.uint8)
    fn = lib.mgq_quantize_q4 if fmt == FMT_Q4 else lib.mgq_quantize_q8
    check(fn(w.ctypes.data, k, n, out.ctypes.data))
    return out


def dequantize(fmt: int, packed: np.ndarray, k: int, n: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty((k, n), dtype=np.float32)
    fn = lib.mgq_dequantize_q4 if fmt == FMT_Q4 else lib.mgq_dequantize_q8
    check(fn(packed.ctypes.data, k, n, out.ctypes.data))
    return out


def shard_columns(fmt: int, packed: np.ndarray, k: int, n: int, n0: int, n1: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(packed_bytes(fmt, k, max(n1 - n0, 0)) or 1, dtype=np.uint8)
    check(lib.mgq_shard_columns(fmt, packed.ctypes.data, k, n, n0, n1, out.ctypes.data))
    return out


def _stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def matmul(fmt: int, a, w, k: int, n: int, addend=None, out=None, stream=None, route: str = "auto"):
    """c = a . dequant(w) (+ addend) on torch CUDA tensors.

    a: [m,k] float32 or bfloat16; w: uint8 tensor holding the packed weight; returns float32 [m,n].
    route: "auto" (mgq_matmul), "gemv" (mgq_gemv) or "gemm" (mgq_gemm).
    """
    import torch
    if not (a.is_cuda and w.is_cuda):
        raise ValueError("matmul takes CUDA tensors; the library has no CPU path")
    a2 = a.reshape(-1, k)
    if not a2.is_contiguous():
        a2 = a2.contiguous()
    m = a2.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    a_dtype = A_BF16 if a2.dtype == torch.bfloat16 else A_F32
    if a2.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("activations must be float32 or bfloat16")
    add_p = addend.data_ptr() if addend is not None else None
    sp = _stream_ptr(stream)
    if route == "gemv":
        check(lib.mgq_gemv(fmt, a2.data_ptr(), w.data_ptr(), add_p, out.data_ptr(), m, k, n, sp))
    elif route == "gemm":
        check(lib.mgq_gemm(fmt, a2.data_ptr(), a_dtype, w.data_ptr(), add_p, out.data_ptr(), m, k, n, sp))
    else:
        check(lib.mgq_matmul(fmt, a2.data_ptr(), a_dtype, w.data_ptr(), add_p, out.data_ptr(), m, k, n, sp))
    return out


class Plan:
    """A static list of single-row GEMVs executed by one persistent kernel (mgq_plan_*).

    ops: iterable of (fmt, x, w, addend_or_None, y, k, n, wait_for) with torch CUDA tensors; the
    tensors are kept alive by the plan.  With `links` (one (push_ptr, wait_ptr) pair of device
    addresses or None per op) the plan uses caller-owned gathered vectors (mgq_plan_create_linked):
    `epoch_ptr` / `error_ptr` are the token index and timeout flag in local device memory and
    `final` = (vector address, length) is the gathered vector that must be complete when a launch ends.
    """

    def __init__(self, ops_list, links=None, epoch_ptr=None, error_ptr=None, final=None, keep=None):
        import ctypes
        self._keep = [keep]
        arr = (_lib.PlanOp * len(ops_list))()
        for i, (fmt, x, w, addend, y, k, n, wait_for) in enumerate(ops_list):
            self._keep.append((x, w, addend, y))
            arr[i] = _lib.PlanOp(fmt, x.data_ptr() if x is not None else None, w.data_ptr(),
                                 addend.data_ptr() if addend is not None else None, y.data_ptr(), 1, k, n, wait_for)
        handle = ctypes.c_void_p()
        if links is None:
            check(lib.mgq_plan_create(arr, len(ops_list), ctypes.byref(handle)))
        else:
            larr = (_lib.PlanLink * len(ops_list))()
            for i, (push_ptr, wait_ptr) in enumerate(links):
                larr[i] = _lib.PlanLink(push_ptr, wait_ptr)
            fvec, flen = final if final is not None else (None, 0)
            check(lib.mgq_plan_create_linked(arr, larr, len(ops_list), epoch_ptr, error_ptr, fvec, flen, ctypes.byref(handle)))
        self._h = handle
        self.count = len(ops_list)

    def launch(self, stream=None) -> None:
        check(lib.mgq_plan_launch(self._h, _stream_ptr(stream)))

    def check(self, stream=None) -> None:
        check(lib.mgq_plan_check(self._h, _stream_ptr(stream)))

    def info(self) -> dict:
        import ctypes
        g, t, c, s = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_size_t()
        check(lib.mgq_plan_info(self._h, ctypes.byref(g), ctypes.byref(t), ctypes.byref(c), ctypes.byref(s)))
        return {"grid": g.value, "threads": t.value, "ring_slots": c.value, "smem_bytes": s.value}

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.mgq_plan_destroy(self._h)
            self._h = None


def matmul_host(fmt: int, a: np.ndarray, w_dev_ptr: int, k: int, n: int, addend: np.ndarray | None = None) -> np.ndarray:
    """Host activations in, host result out, device-resident weight (mgq_matmul_host)."""
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1, k)
    m = a.shape[0]
    out = np.empty((m, n), dtype=np.float32)
    add_p = None
    if addend is not None:
        addend = np.ascontiguousarray(addend, dtype=np.float32)
        add_p = addend.ctypes.data
    check(lib.mgq_matmul_host(fmt, a.ctypes.data, A_F32, w_dev_ptr, add_p, out.ctypes.data, m, k, n))
    return out


__all__ = ["Plan", "set_option", "device_status", "packed_bytes", "quantize", "dequantize", "shard_columns", "matmul", "matmul_host",
           "FMT_Q4", "FMT_Q8", "A_F32", "A_BF16"]
_ = _lib
