"""Graph / build_inference_session / Session with meganeura's names, over the C ABI.

The graph, the plan and the session live in C++ (csrc/mgq_session.cpp); this module only holds
handles.  Method names and argument meaning follow meganeura (src/graph.rs:714-795,
src/train.rs:380-389, src/runtime.rs:2327-2345, 2612-2643, 2786-2791, 2835-2959) so tests read
like the reference's (tests/gemv_parity.rs, tests/gpu_smoke.rs:2680-2771).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from enum import IntEnum

import numpy as np

from ._lib import check, last_error, lib, MgqError


class ShaderEntry(IntEnum):
    MatMul = 0
    FusedMatMulAdd = 1
    MatMulGemv = 2
    MatMulGemvAdd = 3
    Add = 4
    Embedding = 5
    RmsNorm = 6
    RoPEDynamic = 7
    CacheWrite = 8
    CachedAttention = 9
    SwiGLU = 10
    SwiGLUConcat = 11
    RoPECacheWrite = 12
    AllGather = 13
    MatMulGemvBT = 14


class WeightFormat(IntEnum):
    F32 = 0
    F16 = 1
    Q4 = 2
    Q8 = 3


@dataclass
class Dispatch:
    shader: ShaderEntry
    workgroups: tuple
    params: tuple
    weight_format: WeightFormat
    label: str


@dataclass
class ExecutionPlan:
    dispatches: list


def _shape(shape):
    arr = (ctypes.c_size_t * len(shape))(*[int(s) for s in shape])
    return arr, len(shape)


def _node(rc: int) -> int:
    if rc < 0:
        raise MgqError(-rc, last_error())
    return rc


class Graph:
    def __init__(self):
        self._h = lib.mgq_graph_new()

    def __del__(self):
        if getattr(self, "_h", None):
            lib.mgq_graph_free(self._h)
            self._h = None

    def input(self, name: str, shape) -> int:
        return _node(lib.mgq_graph_input(self._h, name.encode(), *_shape(shape)))

    def parameter(self, name: str, shape) -> int:
        return _node(lib.mgq_graph_parameter(self._h, name.encode(), *_shape(shape)))

    def parameter_q4(self, name: str, shape) -> int:
        return _node(lib.mgq_graph_parameter_q4(self._h, name.encode(), *_shape(shape)))

    def parameter_q8(self, name: str, shape) -> int:
        return _node(lib.mgq_graph_parameter_q8(self._h, name.encode(), *_shape(shape)))

    def parameter_f16(self, name: str, shape) -> int:
        return _node(lib.mgq_graph_parameter_f16(self._h, name.encode(), *_shape(shape)))

    def matmul(self, a: int, b: int) -> int:
        return _node(lib.mgq_graph_matmul(self._h, a, b))

    def add(self, a: int, b: int) -> int:
        return _node(lib.mgq_graph_add(self._h, a, b))

    def input_u32(self, name: str, shape) -> int:
        return _node(lib.mgq_graph_input_u32(self._h, name.encode(), *_shape(shape)))

    def embedding(self, indices: int, table: int) -> int:
        return _node(lib.mgq_graph_embedding(self._h, indices, table))

    def rms_norm(self, x: int, weight: int, eps: float) -> int:
        return _node(lib.mgq_graph_rms_norm(self._h, x, weight, eps))

    def rope_dynamic_offset(self, x: int, theta: float, offset_input: int, head_dim: int) -> int:
        return _node(lib.mgq_graph_rope_dynamic_offset(self._h, x, theta, offset_input, head_dim))

    def cache_write(self, new_kv: int, cache: int, kv_pos: int) -> int:
        return _node(lib.mgq_graph_cache_write(self._h, new_kv, cache, kv_pos))

    def cached_attention(self, q: int, k_cache: int, v_cache: int, kv_pos: int, num_heads: int, num_kv_heads: int,
                         head_dim: int) -> int:
        return _node(lib.mgq_graph_cached_attention(self._h, q, k_cache, v_cache, kv_pos, num_heads, num_kv_heads, head_dim))

    def swiglu(self, gate: int, up: int) -> int:
        return _node(lib.mgq_graph_swiglu(self._h, gate, up))

    def swiglu_concat(self, x: int) -> int:
        return _node(lib.mgq_graph_swiglu_concat(self._h, x))

    def matmul_bt(self, a: int, b: int) -> int:
        """Graph::matmul_bt (src/graph.rs:809-817): a [M, K] @ b[N, K]^T, b an f32 parameter."""
        return _node(lib.mgq_graph_matmul_bt(self._h, a, b))

    def all_gather(self, x: int, world: int) -> int:
        """This rank's [1, n] slice -> the whole [1, n * world] vector, rank-major (column-sharded
        models; no reference counterpart: the reference is single-device)."""
        return _node(lib.mgq_graph_all_gather(self._h, x, world))

    def slice_columns(self, x: int, first: int, count: int) -> int:
        """Columns [first, first + count) of a [1, n] node, as a view."""
        return _node(lib.mgq_graph_slice_columns(self._h, x, first, count))

    def set_outputs(self, ids) -> None:
        arr = (ctypes.c_int * len(ids))(*ids)
        check(lib.mgq_graph_set_outputs(self._h, arr, len(ids)))


class Session:
    def __init__(self, handle):
        self._h = handle

    def __del__(self):
        if getattr(self, "_h", None):
            lib.mgq_session_free(self._h)
            self._h = None

    def set_parameter(self, name: str, data) -> None:
        data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        check(lib.mgq_session_set_parameter(self._h, name.encode(), data.ctypes.data, data.size))

    def upload_param(self, name: str, raw) -> None:
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        check(lib.mgq_session_upload_param(self._h, name.encode(), raw.ctypes.data, raw.size))

    def set_input(self, name: str, data) -> None:
        data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        check(lib.mgq_session_set_input(self._h, name.encode(), data.ctypes.data, data.size))

    def save_checkpoint(self, path) -> None:
        check(lib.mgq_session_save_checkpoint(self._h, str(path).encode()))

    def load_checkpoint(self, path) -> None:
        check(lib.mgq_session_load_checkpoint(self._h, str(path).encode()))

    def set_input_u32(self, name: str, data) -> None:
        data = np.ascontiguousarray(data, dtype=np.uint32).reshape(-1)
        check(lib.mgq_session_set_input_u32(self._h, name.encode(), data.ctypes.data, data.size))

    def step(self) -> None:
        check(lib.mgq_session_step(self._h))

    def capture(self) -> None:
        """Capture the dispatch list into a CUDA graph (after at least one ordinary step)."""
        check(lib.mgq_session_capture(self._h))

    def enable_greedy(self, output_index: int, token_input: str, pos_input: str, history_cap: int) -> None:
        """Pick the next token on the device after every step and feed it (and position + 1) back."""
        check(lib.mgq_session_enable_greedy(self._h, output_index, token_input.encode(), pos_input.encode(), history_cap))

    def read_tokens(self, first_pos: int, count: int) -> np.ndarray:
        out = np.empty(count, dtype=np.uint32)
        check(lib.mgq_session_read_tokens(self._h, first_pos, out.ctypes.data, count))
        return out

    def wait(self) -> None:
        check(lib.mgq_session_wait(self._h))

    def read_output(self, length: int) -> np.ndarray:
        out = np.empty(length, dtype=np.float32)
        check(lib.mgq_session_read_output(self._h, out.ctypes.data, length))
        return out

    def read_output_by_index(self, index: int, length: int) -> np.ndarray:
        out = np.empty(length, dtype=np.float32)
        check(lib.mgq_session_read_output_by_index(self._h, index, out.ctypes.data, length))
        return out

    def plan(self) -> ExecutionPlan:
        count = lib.mgq_session_num_dispatches(self._h)
        dispatches = []
        for i in range(count):
            shader, wf = ctypes.c_int(), ctypes.c_int()
            wg, pr = (ctypes.c_uint32 * 3)(), (ctypes.c_uint32 * 4)()
            label = ctypes.create_string_buffer(128)
            check(lib.mgq_session_dispatch_info(self._h, i, ctypes.byref(shader), wg, pr, ctypes.byref(wf), label, 128))
            dispatches.append(Dispatch(ShaderEntry(shader.value), tuple(wg), tuple(pr), WeightFormat(wf.value), label.value.decode()))
        return ExecutionPlan(dispatches)

    def launch_count(self) -> int:
        return int(lib.mgq_session_launch_count(self._h))

    def set_profiling(self, enabled: bool) -> None:
        """Session::set_profiling: the next steps run one timed dispatch at a time (no graph replay)."""
        check(lib.mgq_session_set_profiling(self._h, 1 if enabled else 0))

    def gpu_timings(self):
        """Microseconds of every dispatch of the last profiled step."""
        import numpy as np
        n = int(lib.mgq_session_num_dispatches(self._h))
        out = np.zeros(n, dtype=np.float32)
        check(lib.mgq_session_gpu_timings(self._h, out.ctypes.data, n))
        return out

    def dump_gpu_timings(self) -> str:
        """Session::dump_gpu_timings: per-label totals of the last profiled step, largest first."""
        buf = ctypes.create_string_buffer(16384)
        check(lib.mgq_session_dump_gpu_timings(self._h, buf, len(buf)))
        return buf.value.decode()

    def num_groups(self) -> int:
        """Session::num_groups: barrier groups of the dispatch list."""
        n = int(lib.mgq_session_num_groups(self._h))
        if n < 0:
            check(-n)
        return n

    # ---- column-sharded sessions (graphs with all_gather nodes)
    def exchange_slices(self):
        """Floats this rank contributes to each all_gather, in execution order."""
        n = int(lib.mgq_session_num_exchanges(self._h))
        if n < 0:
            check(-n)
        out = []
        for i in range(n):
            slice_len, world = ctypes.c_uint32(), ctypes.c_uint32()
            check(lib.mgq_session_exchange_info(self._h, i, ctypes.byref(slice_len), ctypes.byref(world)))
            out.append(int(slice_len.value))
        return out

    def bind_exchanges(self, exchange) -> None:
        """Binds every all_gather to a PeerExchange built from exchange_slices() (kept alive here)."""
        for i in range(len(exchange.gather_sizes)):
            check(lib.mgq_session_bind_exchange(self._h, i, exchange.push_ptr(i), exchange.vec_ptr(i)))
        check(lib.mgq_session_bind_exchange_state(self._h, exchange.epoch_ptr, exchange.error_ptr, exchange.local + exchange.off_blocks))
        self._exchange = exchange

    def check_exchange(self) -> None:
        check(lib.mgq_session_check_exchange(self._h))


def build_inference_session(graph: Graph) -> Session:
    handle = ctypes.c_void_p()
    check(lib.mgq_build_inference_session(graph._h, ctypes.byref(handle)))
    return Session(handle)
