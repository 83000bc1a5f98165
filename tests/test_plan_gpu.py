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


@pytest.mark.parametrize("fmts", [(O.FMT_Q4,), (O.FMT_Q8,), (O.FMT_Q4, O.FMT_Q8)])
def test_dependent_chain(coracle, fmts):
    _chain(coracle, fmts, [512, 1024, 768, 4096, 256, 576, 1536, 576], addend_at=(1, 4, 6))


def test_qwen_layer_shapes(coracle):
    # one layer of the benchmark's shapes, each op consuming its predecessor's output
    _chain(coracle, (O.FMT_Q4,), [4096, 12288, 4096, 6144, 4096, 12288, 4096], addend_at=(1, 5))


def test_small_ops_leave_ctas_idle(coracle):
    # fewer column groups than CTAs: most CTAs only take part in the barriers
    _chain(coracle, (O.FMT_Q4, O.FMT_Q8), [256, 288, 256, 320, 288, 4096], addend_at=(0,))


def test_replay_rearms_the_barriers(coracle):
    plan = _chain(coracle, (O.FMT_Q8, O.FMT_Q4), [1024, 2048, 1024], replays=5)
    info = plan.info()
    assert info["threads"] == 384 and info["grid"] >= 100


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
