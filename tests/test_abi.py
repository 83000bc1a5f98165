"""CPU tests of the C ABI: every declared symbol is exported, host-side functions match the
oracle byte for byte, and bad arguments give status codes instead of crashes."""
import ctypes
import os
import re

import numpy as np
import pytest

import meganeura_b200 as mg
from meganeura_b200 import _lib, ops
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mgq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mgq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 30
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in names:
        assert hasattr(raw, name), f"{name} declared in include/mgq.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_static_library_is_built():
    assert os.path.exists(os.path.join(os.path.dirname(_lib.LIB_PATH), "libmgq.a"))


def test_packed_bytes_matches_size_bytes():
    # src/graph.rs:52-68
    assert ops.packed_bytes(mg.FMT_Q8, 576, 1536) == 995328
    assert ops.packed_bytes(mg.FMT_Q4, 576, 49152) == 17694720
    assert ops.packed_bytes(mg.FMT_Q8, 4096, 14336) == 66060288
    assert ops.packed_bytes(mg.FMT_Q4, 4096, 12288) == 31457280
    assert ops.packed_bytes(0, 64, 64) == 0


@pytest.mark.parametrize("k,n", [(32, 1), (64, 4), (576, 192), (1024, 100)])
def test_host_quantizers_match_oracle(coracle, k, n):
    rng = np.random.default_rng(k + n)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    w[:32, 0] = 0.0
    for fmt in (mg.FMT_Q4, mg.FMT_Q8):
        packed = ops.quantize(fmt, w)
        assert (packed == coracle.quantize(fmt, w)).all()
        assert (ops.dequantize(fmt, packed, k, n) == coracle.dequantize(fmt, packed, k, n)).all()


def test_golden_bytes_from_library(golden):
    for name in ("ident", "mat", "smoke"):
        w = golden[f"{name}_w"]
        assert (ops.quantize(mg.FMT_Q4, w) == golden[f"{name}_q4"]).all()
        assert (ops.quantize(mg.FMT_Q8, w) == golden[f"{name}_q8"]).all()
        assert (ops.dequantize(mg.FMT_Q4, golden[f"{name}_q4"], *w.shape) == golden[f"{name}_dq4"]).all()
        assert (ops.dequantize(mg.FMT_Q8, golden[f"{name}_q8"], *w.shape) == golden[f"{name}_dq8"]).all()


def test_shard_columns_matches_oracle(coracle, golden):
    for fmt, tag in ((mg.FMT_Q4, "q4"), (mg.FMT_Q8, "q8")):
        assert (ops.shard_columns(fmt, golden[f"synth_{tag}"], 64, 8, 4, 8) == golden[f"synth_shard_{tag}"]).all()
        w = O.synth_weights(fmt, 128, 24, seed=2)
        assert (ops.shard_columns(fmt, w, 128, 24, 6, 18) == coracle.shard_columns(fmt, w, 128, 24, 6, 18)).all()


def test_bad_arguments_return_status():
    with pytest.raises(mg.MgqError) as e:
        ops.quantize(mg.FMT_Q4, np.zeros((33, 4), np.float32))      # K % 32 != 0
    assert e.value.status == 2 and "multiple of 32" in str(e.value)
    with pytest.raises(mg.MgqError) as e:
        ops.shard_columns(mg.FMT_Q4, np.zeros(160, np.uint8), 64, 4, 2, 9)
    assert e.value.status == 2
    with pytest.raises(mg.MgqError) as e:
        ops.shard_columns(0, np.zeros(160, np.uint8), 64, 4, 0, 2)
    assert e.value.status == 3
    assert _lib.lib.mgq_quantize_q8(None, 32, 1, None) == 1
    # kernel entry points validate before touching the device
    assert _lib.lib.mgq_gemv(mg.FMT_Q4, None, None, None, None, 1, 64, 4, None) == 1
    assert _lib.lib.mgq_gemv(7, 16, 16, None, 16, 1, 64, 4, None) == 3
    assert _lib.lib.mgq_gemv(mg.FMT_Q4, 16, 16, None, 16, 1, 48, 4, None) == 2
    assert _lib.lib.mgq_gemv(mg.FMT_Q4, 16, 16, None, 16, 17, 64, 4, None) == 2
    assert _lib.lib.mgq_gemm(mg.FMT_Q8, 16, 5, 16, None, 16, 64, 64, 4, None) == 3
    assert _lib.lib.mgq_gemm(mg.FMT_Q8, 16, 0, 8, None, 16, 64, 64, 4, None) == 7


def test_graph_builder_checks():
    g = mg.Graph()
    a = g.input("a", [1, 64])
    with pytest.raises(mg.MgqError):
        g.parameter_q4("w", [48, 8])                 # rows not a multiple of 32
    w = g.parameter_q8("w", [64, 8])
    with pytest.raises(mg.MgqError):
        g.matmul(w, a)                               # inner dimensions / quantized lhs
    bad = g.parameter_q4("w2", [32, 8])
    with pytest.raises(mg.MgqError):
        g.matmul(a, bad)                             # 64 vs 32
    c = g.matmul(a, w)
    g.set_outputs([c])
    with pytest.raises(mg.MgqError):
        g.set_outputs([99])


def test_barrier_groups_follow_the_reference_rules():
    """reorder_by_level + compute_groups (src/runtime.rs:1202-1256) on plain buffer-id lists."""
    import ctypes
    import numpy as np
    from meganeura_b200 import _lib

    def groups(dispatches, reorder=1):
        n = len(dispatches)
        ins = np.full((n, 4), -1, dtype=np.int32)
        outs = np.full((n, 4), -1, dtype=np.int32)
        for i, (i_ids, o_ids) in enumerate(dispatches):
            ins[i, :len(i_ids)] = i_ids
            outs[i, :len(o_ids)] = o_ids
        return _lib.lib.mgq_barrier_groups(ins.ctypes.data, outs.ctypes.data, n, reorder)

    assert groups([]) == 0
    assert groups([([0], [1])]) == 1
    # a chain: every dispatch reads what the one before wrote -> one group each
    assert groups([([0], [1]), ([1], [2]), ([2], [3])]) == 3
    # q, k, v read the same input and write different buffers: one group; attention reads all three: a second one
    assert groups([([0, 10], [1]), ([0, 11], [2]), ([0, 12], [3]), ([1, 2, 3], [4])]) == 2
    # level reordering pulls an independent late dispatch forward into the first group ...
    late = [([0], [1]), ([1], [2]), ([0], [5])]
    assert groups(late, reorder=1) == 2
    # ... without it the list order decides, which here gives the same count but a hazard-free third dispatch
    assert groups(late, reorder=0) == 2
    # extra outputs count as writes (merged RoPE + cache write): a reader of the second output starts a new group
    assert groups([([0], [1, 2]), ([2], [3])]) == 2
    # write-after-write alone is no hazard in the reference's rule (only reads of dirty buffers split groups)
    assert groups([([0], [1]), ([0], [1])]) == 1
    _ = ctypes


def test_new_entry_points_check_their_arguments_without_a_gpu():
    """Argument errors are reported before any CUDA call."""
    from meganeura_b200._lib import MgqError, check, lib
    for call in (lambda: lib.mgq_gemv_bt(None, None, None, 64, 8, None),
                 lambda: lib.mgq_exchange_all_gather(None, None, None, None, 4, 8, None, None, None),
                 lambda: lib.mgq_exchange_all_gather_rows(None, 4, 1, 4, 2, None, None, None, None, None, None)):
        with pytest.raises(MgqError):
            check(call())
