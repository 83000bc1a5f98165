"""ctypes binding of libmgq (the C ABI declared in include/mgq.h).

The shared library is built in-tree by ``meganeura_b200/csrc/Makefile``.  There is no
fallback: if the library is missing the import fails, and every call that needs a GPU
returns ``MGQ_ERR_CUDA`` (raised here as :class:`MgqError`) when none is usable.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libmgq.so")

FMT_F32, FMT_F16, FMT_Q4, FMT_Q8 = 0, 1, 2, 3
A_F32, A_BF16 = 0, 1
GEMV_MAX_M = 16

STATUS_NAMES = {
    0: "MGQ_OK", 1: "MGQ_ERR_NULL", 2: "MGQ_ERR_SHAPE", 3: "MGQ_ERR_FORMAT", 4: "MGQ_ERR_CUDA",
    5: "MGQ_ERR_NAME", 6: "MGQ_ERR_SIZE", 7: "MGQ_ERR_ALIGN", 8: "MGQ_ERR_STATE", 9: "MGQ_ERR_TIMEOUT",
}


class MgqError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
            "(nvcc, sm_100a).  There is no CPU fallback.")
    return ctypes.CDLL(LIB_PATH)


lib = _load()

_sz, _u32, _int, _vp = ctypes.c_size_t, ctypes.c_uint32, ctypes.c_int, ctypes.c_void_p
_f32p = ctypes.POINTER(ctypes.c_float)
_u8p = ctypes.POINTER(ctypes.c_uint8)
_szp = ctypes.POINTER(ctypes.c_size_t)

# name -> (restype, argtypes).  Every symbol include/mgq.h declares is listed here.
SIGNATURES = {
    "mgq_last_error": (ctypes.c_char_p, []),
    "mgq_version": (ctypes.c_char_p, []),
    "mgq_set_option": (_int, [ctypes.c_char_p, ctypes.c_long]),
    "mgq_packed_bytes": (_sz, [_int, _sz, _sz]),
    "mgq_quantize_q4": (_int, [_vp, _sz, _sz, _vp]),
    "mgq_quantize_q8": (_int, [_vp, _sz, _sz, _vp]),
    "mgq_dequantize_q4": (_int, [_vp, _sz, _sz, _vp]),
    "mgq_dequantize_q8": (_int, [_vp, _sz, _sz, _vp]),
    "mgq_shard_columns": (_int, [_int, _vp, _sz, _sz, _sz, _sz, _vp]),
    "mgq_buffer_create": (_int, [_sz, ctypes.POINTER(_vp)]),
    "mgq_buffer_destroy": (_int, [_vp]),
    "mgq_buffer_upload": (_int, [_vp, _vp, _sz, _vp]),
    "mgq_buffer_download": (_int, [_vp, _vp, _sz, _vp]),
    "mgq_device_status": (_int, []),
    "mgq_gemv": (_int, [_int, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "mgq_gemv_f16": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "mgq_convert_f16": (_int, [_vp, _sz, _vp]),
    "mgq_gemv_bt": (_int, [_vp, _vp, _vp, _u32, _u32, _vp]),
    "mgq_graph_matmul_bt": (_int, [_vp, _int, _int]),
    "mgq_graph_parameter_f16": (_int, [_vp, ctypes.c_char_p, _szp, _sz]),
    "mgq_embedding": (_int, [_vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "mgq_rms_norm": (_int, [_vp, _vp, _vp, _u32, _u32, ctypes.c_float, _vp]),
    "mgq_rope_dynamic": (_int, [_vp, _vp, _vp, _u32, _u32, _u32, ctypes.c_float, _vp]),
    "mgq_rope_cache_write": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, ctypes.c_float, _u32, _vp]),
    "mgq_cache_write": (_int, [_vp, _vp, _vp, _u32, _u32, _vp]),
    "mgq_swiglu": (_int, [_vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "mgq_cached_attention_workspace": (_sz, [_u32, _u32, _u32]),
    "mgq_cached_attention": (_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, _vp]),
    "mgq_argmax_workspace": (_sz, []),
    "mgq_argmax": (_int, [_vp, _u32, _vp, _vp, _vp, _vp, _vp, _u32, _vp]),
    "mgq_gemv_exchange": (_int, [_int, _vp, _vp, _vp, _vp, _u32, _u32, _vp, _vp, _vp, _vp, _vp]),
    "mgq_exchange_finish": (_int, [_vp, _u32, _vp, _vp, _vp, _vp]),
    "mgq_exchange_all_gather": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _vp, _vp, _vp]),
    "mgq_exchange_all_gather_rows": (_int, [_vp, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mgq_gemm": (_int, [_int, _vp, _int, _vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "mgq_matmul": (_int, [_int, _vp, _int, _vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "mgq_matmul_host": (_int, [_int, _vp, _int, _vp, _vp, _vp, _u32, _u32, _u32]),
    "mgq_plan_create": (_int, [_vp, _sz, ctypes.POINTER(_vp)]),
    "mgq_plan_create_linked": (_int, [_vp, _vp, _sz, _vp, _vp, _vp, _u32, ctypes.POINTER(_vp)]),
    "mgq_plan_launch": (_int, [_vp, _vp]),
    "mgq_plan_check": (_int, [_vp, _vp]),
    "mgq_plan_info": (_int, [_vp, ctypes.POINTER(_u32), ctypes.POINTER(_u32), ctypes.POINTER(_u32), _szp]),
    "mgq_plan_destroy": (None, [_vp]),
    "mgq_plan_run_static": (_int, [_vp, _sz, _vp]),
    "mgq_graph_new": (_vp, []),
    "mgq_graph_free": (None, [_vp]),
    "mgq_graph_input": (_int, [_vp, ctypes.c_char_p, _szp, _sz]),
    "mgq_graph_parameter": (_int, [_vp, ctypes.c_char_p, _szp, _sz]),
    "mgq_graph_parameter_q4": (_int, [_vp, ctypes.c_char_p, _szp, _sz]),
    "mgq_graph_parameter_q8": (_int, [_vp, ctypes.c_char_p, _szp, _sz]),
    "mgq_graph_matmul": (_int, [_vp, _int, _int]),
    "mgq_graph_add": (_int, [_vp, _int, _int]),
    "mgq_graph_input_u32": (_int, [_vp, ctypes.c_char_p, _szp, _sz]),
    "mgq_graph_embedding": (_int, [_vp, _int, _int]),
    "mgq_graph_rms_norm": (_int, [_vp, _int, _int, ctypes.c_float]),
    "mgq_graph_rope_dynamic_offset": (_int, [_vp, _int, ctypes.c_float, _int, _u32]),
    "mgq_graph_cache_write": (_int, [_vp, _int, _int, _int]),
    "mgq_graph_cached_attention": (_int, [_vp, _int, _int, _int, _int, _u32, _u32, _u32]),
    "mgq_graph_swiglu": (_int, [_vp, _int, _int]),
    "mgq_graph_swiglu_concat": (_int, [_vp, _int]),
    "mgq_graph_all_gather": (_int, [_vp, _int, _u32]),
    "mgq_graph_slice_columns": (_int, [_vp, _int, _u32, _u32]),
    "mgq_graph_set_outputs": (_int, [_vp, ctypes.POINTER(_int), _sz]),
    "mgq_build_inference_session": (_int, [_vp, ctypes.POINTER(_vp)]),
    "mgq_session_free": (None, [_vp]),
    "mgq_session_set_parameter": (_int, [_vp, ctypes.c_char_p, _vp, _sz]),
    "mgq_session_upload_param": (_int, [_vp, ctypes.c_char_p, _vp, _sz]),
    "mgq_session_set_input": (_int, [_vp, ctypes.c_char_p, _vp, _sz]),
    "mgq_session_save_checkpoint": (_int, [_vp, ctypes.c_char_p]),
    "mgq_session_load_checkpoint": (_int, [_vp, ctypes.c_char_p]),
    "mgq_session_set_input_u32": (_int, [_vp, ctypes.c_char_p, _vp, _sz]),
    "mgq_session_step": (_int, [_vp]),
    "mgq_session_capture": (_int, [_vp]),
    "mgq_session_enable_greedy": (_int, [_vp, _sz, ctypes.c_char_p, ctypes.c_char_p, _u32]),
    "mgq_session_read_tokens": (_int, [_vp, _u32, _vp, _sz]),
    "mgq_session_wait": (_int, [_vp]),
    "mgq_session_read_output": (_int, [_vp, _vp, _sz]),
    "mgq_session_read_output_by_index": (_int, [_vp, _sz, _vp, _sz]),
    "mgq_session_num_dispatches": (_int, [_vp]),
    "mgq_session_dispatch_info": (_int, [_vp, _sz, ctypes.POINTER(_int), ctypes.POINTER(_u32), ctypes.POINTER(_u32),
                                         ctypes.POINTER(_int), ctypes.c_char_p, _sz]),
    "mgq_session_launch_count": (ctypes.c_uint64, [_vp]),
    "mgq_session_set_profiling": (_int, [_vp, _int]),
    "mgq_session_gpu_timings": (_int, [_vp, _vp, _sz]),
    "mgq_session_dump_gpu_timings": (_int, [_vp, ctypes.c_char_p, _sz]),
    "mgq_session_num_groups": (_int, [_vp]),
    "mgq_session_num_exchanges": (_int, [_vp]),
    "mgq_session_exchange_info": (_int, [_vp, _sz, ctypes.POINTER(_u32), ctypes.POINTER(_u32)]),
    "mgq_session_bind_exchange": (_int, [_vp, _sz, _vp, _vp]),
    "mgq_session_bind_exchange_state": (_int, [_vp, _vp, _vp, _vp]),
    "mgq_session_check_exchange": (_int, [_vp]),
    "mgq_barrier_groups": (_int, [_vp, _vp, _sz, _int]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


class PlanOp(ctypes.Structure):
    """mgq_plan_op"""
    _fields_ = [("fmt", ctypes.c_int), ("x", _vp), ("w", _vp), ("addend", _vp), ("y", _vp),
                ("m", _u32), ("k", _u32), ("n", _u32), ("wait_for", _u32)]


class PlanLink(ctypes.Structure):
    """mgq_plan_link"""
    _fields_ = [("push_dev", _vp), ("wait_vec", _vp)]


class ExchangePush(ctypes.Structure):
    """mgq_exchange_push (built on the host, copied to device memory)"""
    _fields_ = [("world", _u32), ("rank", _u32), ("gather_cols", _u32), ("reserved", _u32),
                ("dst", ctypes.c_uint64 * 8)]


def last_error() -> str:
    return lib.mgq_last_error().decode()


def check(status: int) -> None:
    if status != 0:
        raise MgqError(status, last_error())
