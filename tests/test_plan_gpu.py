"""The persistent plan kernel (mgq_plan_*): chains of dependent GEMVs in one launch, against the
oracle run op by op."""
import numpy as np
import pytest

from oracle import oracle as O
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


def _chain(coracle, fmts, dims, addend_at=(), seed=0, replays=1):
    """dims = [k0, n1, n2, ...]; op i maps dims[i] -> dims[i+1] and reads the previous op's output."""
    import torch
    from meganeura_b200 import ops
    rng = np.random.Generator(np.random.PCG64(seed))
    x0 = rng.standard_normal((1, dims[0])).astype(np.float32)
    bufs = [to_dev(x0)] + [torch.full((1, n), 7.0, dtype=torch.float32, device="cuda") for n in dims[1:]]
    packed, addends, plan_ops = [], [], []
    for i in range(len(dims) - 1):
        k, n, fmt = dims[i], dims[i + 1], fmts[i % len(fmts)]
        w = O.synth_weights(fmt, k, n, seed=seed * 31 + i)
        packed.append(w)
        add = rng.standard_normal((1, n)).astype(np.float32) if i in addend_at else None
        addends.append(add)
        plan_ops.append((fmt, bufs[i], to_dev(w), to_dev(add) if add is not None else None, bufs[i + 1], k, n, i))
    plan = ops.Plan(plan_ops)
    for _ in range(replays):
        plan.launch()
    plan.check()
    # oracle, fed with its own previous output (f64 accumulate, rounded to f32 between ops)
    want = x0
    for i in range(len(dims) - 1):
        k, n, fmt = dims[i], dims[i + 1], fmts[i % len(fmts)]
        want = coracle.matmul(fmt, want, packed[i], k, n, addend=addends[i], wide=True, nthreads=8).astype(np.float32)
        got = bufs[i + 1].cpu().numpy()
        assert np.isfinite(got).all()
        err = O.rel_l2(got, want)
        assert err <= 1e-4, f"op {i} ({k}x{n}, fmt {fmt}): rel-L2 {err:.3e}"
    return plan


@pytest.mark.parametrize("dataflow", [0, 1])
@pytest.mark.parametrize("fmts", [(O.FMT_Q4,), (O.FMT_Q8,), (O.FMT_Q4, O.FMT_Q8)])
def test_dependent_chain(coracle, fmts, dataflow):
    """dataflow 0: consumers wait on arrival counters and read plain vectors; 1: {value, stamp} vectors."""
    from meganeura_b200 import ops
    ops.set_option("plan.dataflow", dataflow)
    try:
        _chain(coracle, fmts, [512, 1024, 768, 4096, 256, 576, 1536, 576], addend_at=(1, 4, 6), replays=2)
    finally:
        ops.set_option("plan.dataflow", 0)


@pytest.mark.parametrize("dataflow", [0, 1])
def test_qwen_layer_shapes(coracle, dataflow):
    # one layer of the benchmark's shapes, each op consuming its predecessor's output
    from meganeura_b200 import ops
    ops.set_option("plan.dataflow", dataflow)
    try:
        _chain(coracle, (O.FMT_Q4,), [4096, 12288, 4096, 6144, 4096, 12288, 4096], addend_at=(1, 5))
    finally:
        ops.set_option("plan.dataflow", 0)


def test_small_ops_leave_ctas_idle(coracle):
    # fewer column groups than CTAs: most CTAs only take part in the barriers
    _chain(coracle, (O.FMT_Q4, O.FMT_Q8), [256, 288, 256, 320, 288, 4096], addend_at=(0,))


def test_replay_rearms_the_barriers(coracle):
    plan = _chain(coracle, (O.FMT_Q8, O.FMT_Q4), [1024, 2048, 1024], replays=5)
    info = plan.info()
    assert info["threads"] == 800 and info["grid"] >= 100 and info["ring_slots"] >= 3


def test_plan_inside_cuda_graph(coracle):
    import torch
    from meganeura_b200 import ops
    k, n = 4096, 4096
    w1, w2 = O.synth_weights(O.FMT_Q4, k, n, 1), O.synth_weights(O.FMT_Q4, n, 1024, 2)
    x = np.random.default_rng(0).standard_normal((1, k)).astype(np.float32)
    xd, y1, y2 = to_dev(x), torch.zeros((1, n), device="cuda"), torch.zeros((1, 1024), device="cuda")
    plan = ops.Plan([(O.FMT_Q4, xd, to_dev(w1), None, y1, k, n, 0), (O.FMT_Q4, y1, to_dev(w2), None, y2, n, 1024, 1)])
    plan.launch(); plan.check()
    ref = y2.clone()
    g, s = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            plan.launch()
    y2.zero_()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    plan.check()
    assert bool((y2 == ref).all())
    want = coracle.matmul(O.FMT_Q4, coracle.matmul(O.FMT_Q4, x, w1, k, n).astype(np.float32), w2, n, 1024)
    assert O.rel_l2(y2.cpu().numpy(), want) <= 1e-4


def test_plain_vectors_wait_on_arrival_counters(coracle):
    """An op whose activations are not a range of an earlier op's output (here: a copy made by the
    test in a separate buffer is NOT used; the op reads a buffer that op 0 writes through an alias the
    plan cannot see) still honours wait_for through the per-op arrival counters."""
    import torch
    from meganeura_b200 import ops
    k, n, n2 = 1024, 2048, 512
    rng = np.random.Generator(np.random.PCG64(3))
    x0 = rng.standard_normal((1, k)).astype(np.float32)
    w1, w2, w3 = (O.synth_weights(O.FMT_Q4, k, n, 11), O.synth_weights(O.FMT_Q8, k, n2, 12), O.synth_weights(O.FMT_Q4, n2, 256, 13))
    xd = to_dev(x0)
    y1 = torch.zeros((1, n), device="cuda"); y2 = torch.zeros((1, n2), device="cuda"); y3 = torch.zeros((1, 256), device="cuda")
    # op 1 reads the external input again but must wait for op 0 (wait_for = 1): counter path
    plan = ops.Plan([(O.FMT_Q4, xd, to_dev(w1), None, y1, k, n, 0),
                     (O.FMT_Q8, xd, to_dev(w2), None, y2, k, n2, 1),
                     (O.FMT_Q4, y2, to_dev(w3), None, y3, n2, 256, 2)])
    for _ in range(3):
        plan.launch()
    plan.check()
    assert O.rel_l2(y1.cpu().numpy(), coracle.matmul(O.FMT_Q4, x0, w1, k, n, wide=True)) <= 1e-4
    want2 = coracle.matmul(O.FMT_Q8, x0, w2, k, n2, wide=True).astype(np.float32)
    assert O.rel_l2(y2.cpu().numpy(), want2) <= 1e-4
    assert O.rel_l2(y3.cpu().numpy(), coracle.matmul(O.FMT_Q4, want2, w3, n2, 256, wide=True)) <= 1e-4


@pytest.mark.parametrize("dataflow", [0, 1])
def test_consumer_of_a_column_range(coracle, dataflow):
    """The consumer takes columns [256, 256+512) of its producer's output (not the leading ones)."""
    import torch
    from meganeura_b200 import ops
    ops.set_option("plan.dataflow", dataflow)
    k, n, k2, n2 = 512, 1024, 512, 384
    rng = np.random.Generator(np.random.PCG64(4))
    x0 = rng.standard_normal((1, k)).astype(np.float32)
    w1, w2 = O.synth_weights(O.FMT_Q8, k, n, 21), O.synth_weights(O.FMT_Q4, k2, n2, 22)
    y1 = torch.zeros((1, n), device="cuda"); y2 = torch.zeros((1, n2), device="cuda")
    try:
        plan = ops.Plan([(O.FMT_Q8, to_dev(x0), to_dev(w1), None, y1, k, n, 0),
                         (O.FMT_Q4, y1[:, 256:256 + k2], to_dev(w2), None, y2, k2, n2, 1)])
    finally:
        ops.set_option("plan.dataflow", 0)
    plan.launch(); plan.launch()
    plan.check()
    mid = coracle.matmul(O.FMT_Q8, x0, w1, k, n, wide=True).astype(np.float32)
    assert O.rel_l2(y1.cpu().numpy(), mid) <= 1e-4
    assert O.rel_l2(y2.cpu().numpy(), coracle.matmul(O.FMT_Q4, mid[:, 256:256 + k2], w2, k2, n2, wide=True)) <= 1e-4


def test_wide_and_narrow_ops_share_one_plan(coracle):
    plan = _chain(coracle, (O.FMT_Q4, O.FMT_Q8), [4096, 1536, 12288, 576, 1024], addend_at=(2,), replays=2)
    assert plan.info()["threads"] == 800


def test_wait_that_nothing_satisfies_times_out(coracle):
    """A linked op whose gathered vector nobody fills: the waits run into their time limit (set to
    1 ms here), the launch ends, the error is reported and the next correct launch works."""
    import ctypes
    import torch
    import meganeura_b200 as mg
    from meganeura_b200 import _lib, ops
    k, n = 1024, 256
    w = to_dev(O.synth_weights(O.FMT_Q4, k, n, 31))
    state = torch.zeros(64, dtype=torch.uint8, device="cuda")               # [epoch u64][error u32]
    vec = torch.zeros(k * 8, dtype=torch.uint8, device="cuda")               # stamps stay 0: never valid
    y = torch.zeros((1, n), device="cuda")
    ops.set_option("plan.peer_deadline_us", 1000)
    try:
        plan = ops.Plan([(O.FMT_Q4, None, w, None, y, k, n, 0)], links=[(None, vec.data_ptr())],
                        epoch_ptr=state.data_ptr(), error_ptr=state.data_ptr() + 8)
        plan.launch()
        with pytest.raises(mg.MgqError) as e:
            plan.check()
        assert e.value.status == 9                                          # MGQ_ERR_TIMEOUT
    finally:
        ops.set_option("plan.peer_deadline_us", 0)
    x = to_dev(np.ones((1, k), dtype=np.float32))
    good = ops.Plan([(O.FMT_Q4, x, w, None, y, k, n, 0)])
    good.launch(); good.check()
    assert O.rel_l2(y.cpu().numpy(), coracle.matmul(O.FMT_Q4, np.ones((1, k), np.float32), w.cpu().numpy(), k, n)) <= 1e-4
    _ = ctypes, _lib


def test_plan_rejects_what_it_cannot_run():
    import torch
    import meganeura_b200 as mg
    from meganeura_b200 import ops
    x = torch.zeros((1, 64), device="cuda"); y = torch.zeros((1, 8), device="cuda")
    w = torch.zeros(64 * 8 // 32 * 20, dtype=torch.uint8, device="cuda")
    with pytest.raises(mg.MgqError) as e:
        ops.Plan([(O.FMT_Q4, x, w, None, y, 64, 8, 0)])          # K < 256
    assert e.value.status == 2
    with pytest.raises(mg.MgqError) as e:
        ops.Plan([(0, x, w, None, y, 64, 8, 0)])
    assert e.value.status == 3
