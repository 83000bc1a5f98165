"""The Graph / build_inference_session / Session surface on the GPU, written like the reference's
tests (tests/gemv_parity.rs, tests/gpu_smoke.rs:2680-2771)."""
import numpy as np
import pytest

import meganeura_b200 as mg
from meganeura_b200 import Graph, ShaderEntry, WeightFormat, build_inference_session
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def run_gpu_gemv(fmt, a_data, b_data, k, n, coracle):
    g = Graph()
    a = g.input("a", [1, k])
    b = (g.parameter_q4 if fmt == O.FMT_Q4 else g.parameter_q8)("b", [k, n])
    c = g.matmul(a, b)
    g.set_outputs([c])
    session = build_inference_session(g)
    plan = session.plan()
    gemv_count = sum(1 for d in plan.dispatches if d.shader == ShaderEntry.MatMulGemv)
    if n % 4 == 0:                                            # routing rule, tests/gemv_parity.rs:32-52
        assert gemv_count == 1
        assert plan.dispatches[0].workgroups == (n // 4, 1, 1)
        assert plan.dispatches[0].label == f"MatMulGemv[1x{n}x{k}]"
    else:
        assert gemv_count == 0
        assert plan.dispatches[0].shader == ShaderEntry.MatMul
        assert plan.dispatches[0].workgroups == ((n + 63) // 64, 1, 1)
    assert plan.dispatches[0].params == (1, k, n, 0)
    assert plan.dispatches[0].weight_format == (WeightFormat.Q4 if fmt == O.FMT_Q4 else WeightFormat.Q8)
    session.set_input("a", a_data)
    session.set_parameter("b", b_data)                        # quantizes on upload
    session.step()
    session.wait()
    out = session.read_output(n)
    want = coracle.matmul(fmt, a_data.reshape(1, k), coracle.quantize(fmt, b_data), k, n)
    assert O.rel_l2(out, want) <= 1e-4
    return out


@pytest.mark.parametrize("fmt", [O.FMT_Q4, O.FMT_Q8])
@pytest.mark.parametrize("k,n,seed", [(64, 64, 1), (576, 576, 2), (576, 1536, 3), (1536, 576, 4), (128, 300, 7), (128, 257, 8), (128, 1, 9)])
def test_gemv_shapes(coracle, fmt, k, n, seed):
    # data generators of tests/gemv_parity.rs:74-82
    i = np.arange(k, dtype=np.uint32)
    a = np.sin((i ^ np.uint32(seed)).astype(np.float32) * np.float32(0.003)).astype(np.float32)
    j = np.arange(k * n, dtype=np.uint32)
    b = np.cos((j ^ np.uint32(seed * 31)).astype(np.float32) * np.float32(0.0007)).astype(np.float32).reshape(k, n)
    run_gpu_gemv(fmt, a, b, k, n, coracle)


@pytest.mark.parametrize("fmt", [O.FMT_Q4, O.FMT_Q8])
def test_fused_matmul_add_and_raw_upload(coracle, fmt):
    k, n = 576, 576
    g = Graph()
    a = g.input("a", [1, k])
    d = g.input("d", [1, n])
    w = (g.parameter_q4 if fmt == O.FMT_Q4 else g.parameter_q8)("w", [k, n])
    out = g.add(g.matmul(a, w), d)
    g.set_outputs([out])
    s = build_inference_session(g)
    plan = s.plan()
    assert [x.shader for x in plan.dispatches] == [ShaderEntry.MatMulGemvAdd]      # MatMul+Add fused
    assert plan.dispatches[0].label == f"MatMulGemvAdd[1x{n}x{k}]"
    packed = O.synth_weights(fmt, k, n, seed=17)
    rng = np.random.default_rng(1)
    x, dd = rng.standard_normal(k).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    s.upload_param("w", packed)                                # pre-packed bytes, no quantization
    s.set_input("a", x)
    s.set_input("d", dd)
    s.step(); s.wait()
    got = s.read_output(n)
    want = coracle.matmul(fmt, x.reshape(1, k), packed, k, n, addend=dd.reshape(1, n))
    assert O.rel_l2(got, want) <= 1e-4
    assert s.launch_count() == 1
    # zero-filled buffers: before any upload a fresh session returns zeros
    s2 = build_inference_session(g)
    s2.step(); s2.wait()
    assert (s2.read_output(n) == 0).all()


def test_matmul_output_is_not_fused(coracle):
    # a matmul that is itself a graph output keeps its own dispatch (src/optimize.rs:748-752)
    k, n = 64, 8
    g = Graph()
    a = g.input("a", [1, k]); d = g.input("d", [1, n])
    w = g.parameter_q8("w", [k, n])
    mm = g.matmul(a, w)
    out = g.add(mm, d)
    g.set_outputs([out, mm])
    s = build_inference_session(g)
    assert [x.shader for x in s.plan().dispatches] == [ShaderEntry.MatMulGemv, ShaderEntry.Add]
    packed = O.synth_weights(O.FMT_Q8, k, n, seed=3)
    x = np.linspace(-1, 1, k, dtype=np.float32); dd = np.ones(n, np.float32)
    s.upload_param("w", packed); s.set_input("a", x); s.set_input("d", dd)
    s.step(); s.wait()
    mmv = s.read_output_by_index(1, n)
    assert np.allclose(s.read_output(n), mmv + 1.0)
    assert O.rel_l2(mmv, coracle.matmul(O.FMT_Q8, x.reshape(1, k), packed, k, n)) <= 1e-4


def test_q4_matmul_correctness_session(coracle):
    # tests/gpu_smoke.rs:2680-2771 through the session, m=6 (routes to the tiled MatMul entry)
    m, k, n = 6, 1024, 2048
    g = Graph()
    a = g.input("a", [m, k]); b = g.parameter_q4("b", [k, n])
    g.set_outputs([g.matmul(a, b)])
    s = build_inference_session(g)
    assert s.plan().dispatches[0].shader == ShaderEntry.MatMul
    assert s.plan().dispatches[0].workgroups == (32, 1, 1)
    a_data = (((np.arange(m * k) % 7).astype(np.float32) - 3.0) * 0.5).astype(np.float32)
    i = np.arange(k * n)
    b_data = ((i % 11).astype(np.float32) - np.float32(5.0)) * np.float32(0.3)
    b_data = np.where(i % 1000 == 0, b_data * np.float32(5.0), b_data).astype(np.float32)
    s.set_input("a", a_data); s.set_parameter("b", b_data)
    s.step(); s.wait()
    got = s.read_output(m * n).reshape(m, n)
    deq = coracle.dequantize(O.FMT_Q4, coracle.quantize(O.FMT_Q4, b_data.reshape(k, n)), k, n)
    cpu = a_data.reshape(m, k) @ deq
    assert np.count_nonzero(np.isnan(got)) == 0
    assert np.abs(got - cpu).max() < 0.1


def test_errors_are_statuses():
    g = Graph()
    a = g.input("a", [1, 64]); w = g.parameter_q4("w", [64, 8])
    g.set_outputs([g.matmul(a, w)])
    s = build_inference_session(g)
    with pytest.raises(mg.MgqError) as e:
        s.set_parameter("nope", np.zeros(512, np.float32))
    assert e.value.status == 5 and "unknown parameter" in str(e.value)
    with pytest.raises(mg.MgqError) as e:
        s.set_parameter("w", np.zeros(100, np.float32))
    assert e.value.status == 6
    with pytest.raises(mg.MgqError):
        s.upload_param("w", np.zeros(7, np.uint8))
    g2 = Graph()
    a2 = g2.input("a", [1, 64]); w2 = g2.parameter("w", [64, 8])
    g2.set_outputs([g2.matmul(a2, w2)])
    with pytest.raises(mg.MgqError) as e:
        build_inference_session(g2)                            # f32 weights are not on this path
    assert e.value.status == 3


def test_matmul_host_round_trip(coracle):
    from meganeura_b200 import ops
    from gpu_util import to_dev
    k, n = 576, 1536
    packed = O.synth_weights(O.FMT_Q8, k, n, seed=1)
    wd = to_dev(packed)
    x = np.random.default_rng(0).standard_normal((1, k)).astype(np.float32)
    got = ops.matmul_host(O.FMT_Q8, x, wd.data_ptr(), k, n)
    assert O.rel_l2(got, coracle.matmul(O.FMT_Q8, x, packed, k, n)) <= 1e-4


def test_profiling_surface_and_groups():
    """set_profiling / dump_gpu_timings / num_groups (src/runtime.rs:1965-1967, 2798-2832, 4192-4199):
    per-dispatch times add up to about the step, the report lists every label, groups follow the
    dependency levels of the decode graph."""
    import time
    import torch
    import meganeura_b200 as mg
    from meganeura_b200 import decode_model as M
    cfg = M.small(M.SMOLLM2_135M, 2, 4096)
    dec = M.DecodeSession(cfg, 64, seed=5)
    s = dec.session
    dec.set_position(3, 0)
    s.step(); s.wait()
    n = len(s.plan().dispatches)
    # the decode graph is a chain except for what the fusions merged: one group per dispatch here
    assert 1 <= s.num_groups() <= n
    s.set_profiling(True)
    dec.set_position(4, 1)
    s.step(); s.wait()                                   # first profiled step creates the events
    dec.set_position(5, 2)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    s.step(); s.wait()
    wall_us = (time.perf_counter() - t0) * 1e6
    times = s.gpu_timings()
    assert times.shape == (n,) and (times > 0).all()
    total = float(times.sum())
    assert 0.3 * wall_us <= total <= 1.2 * wall_us, f"dispatch times {total:.0f} us vs step {wall_us:.0f} us"
    report = s.dump_gpu_timings()
    assert report.startswith("--- GPU pass timings (%d passes" % n)
    for d in s.plan().dispatches:
        assert d.label in report
    s.set_profiling(False)
    dec.set_position(6, 3)
    s.step(); s.wait()
    assert np.isfinite(s.read_output(cfg.vocab_size)).all()
    _ = mg
