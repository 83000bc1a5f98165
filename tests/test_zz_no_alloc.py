"""mgq_plan_run_static: the allocation-free way to run a list of GEMVs.

Some hosts may not allocate device memory once they are running (fixed memory budget, or a rule
against cudaMalloc on the execution path), so they cannot build a plan with mgq_plan_create.
This entry point keeps the kernel's scratch in a fixed device array inside the library instead.
The test drives it through the C ABI and compares it with the allocating entry point on the same
inputs, twice in a row (the array is reused and keeps the previous call's contents).

The file name sorts last on purpose: pytest runs it after every other test file.
"""
import ctypes

import numpy as np
import pytest

from oracle import oracle as O
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


def _ops_array(entries):
    from meganeura_b200 import _lib
    arr = (_lib.PlanOp * len(entries))()
    for i, (fmt, x, w, addend, y, k, n, wait_for) in enumerate(entries):
        arr[i] = _lib.PlanOp(fmt, x.data_ptr(), w.data_ptr(), addend.data_ptr() if addend is not None else None,
                             y.data_ptr(), 1, k, n, wait_for)
    return arr


def test_static_plan_matches_allocating_plan_twice(coracle):
    import torch
    from meganeura_b200 import _lib, ops
    dims = [1024, 4096, 2048, 576]
    fmts = [O.FMT_Q4, O.FMT_Q8, O.FMT_Q4]
    rng = np.random.Generator(np.random.PCG64(5))
    x0 = rng.standard_normal((1, dims[0])).astype(np.float32)
    weights = [to_dev(O.synth_weights(fmts[i], dims[i], dims[i + 1], seed=40 + i)) for i in range(3)]
    addend = to_dev(rng.standard_normal((1, dims[2])).astype(np.float32))

    def buffers():
        return [to_dev(x0)] + [torch.zeros((1, n), dtype=torch.float32, device="cuda") for n in dims[1:]]

    def entries(bufs):
        return [(fmts[i], bufs[i], weights[i], addend if i == 1 else None, bufs[i + 1], dims[i], dims[i + 1], i) for i in range(3)]

    ref_bufs = buffers()
    plan = ops.Plan(entries(ref_bufs))                     # existing entry point (allocates its scratch)
    plan.launch()
    plan.check()
    want = [b.clone() for b in ref_bufs[1:]]
    oracle_last = x0
    for i in range(3):
        oracle_last = coracle.matmul(fmts[i], oracle_last, weights[i].cpu().numpy(), dims[i], dims[i + 1],
                                     addend=addend.cpu().numpy() if i == 1 else None).astype(np.float32)
    assert O.rel_l2(want[-1].cpu().numpy(), oracle_last) <= 1e-4

    stream = torch.cuda.current_stream().cuda_stream
    for attempt in range(2):                               # second call reuses the array left by the first
        bufs = buffers()
        arr = _ops_array(entries(bufs))
        _lib.check(_lib.lib.mgq_plan_run_static(arr, 3, stream))
        for got, ref in zip(bufs[1:], want):
            g, r = got.cpu().numpy(), ref.cpu().numpy()
            assert np.isfinite(g).all()
            assert O.rel_l2(g, r) <= 1e-6, f"call {attempt}: differs from the allocating entry point"


def test_static_plan_in_any_order_of_formats_and_without_allocating(coracle):
    """A Q4-only list, then a list with a Q8 op, then Q4-only again: each call works out its own kernel
    variant and shared-memory layout (nothing cached from the call before can be wrong for it), each
    result matches the allocating entry point, and the device's free memory does not change across a call."""
    import torch
    from meganeura_b200 import _lib, ops
    rng = np.random.Generator(np.random.PCG64(8))
    stream = torch.cuda.current_stream().cuda_stream
    x0 = rng.standard_normal((1, 1024)).astype(np.float32)
    cases = [((O.FMT_Q4, O.FMT_Q4), 61), ((O.FMT_Q4, O.FMT_Q8), 62), ((O.FMT_Q4, O.FMT_Q4), 63)]
    for fmts, seed in cases:
        dims = [1024, 2048, 512]
        weights = [to_dev(O.synth_weights(fmts[i], dims[i], dims[i + 1], seed=seed * 10 + i)) for i in range(2)]

        def run(static):
            bufs = [to_dev(x0)] + [torch.zeros((1, n), dtype=torch.float32, device="cuda") for n in dims[1:]]
            entries = [(fmts[i], bufs[i], weights[i], None, bufs[i + 1], dims[i], dims[i + 1], i) for i in range(2)]
            if static:
                arr = _ops_array(entries)
                torch.cuda.synchronize()
                free_before = torch.cuda.mem_get_info()[0]
                _lib.check(_lib.lib.mgq_plan_run_static(arr, 2, stream))
                assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed the free device memory"
            else:
                plan = ops.Plan(entries)
                plan.launch()
                plan.check()
            return bufs[-1].cpu().numpy()

        want, got = run(False), run(True)
        assert np.isfinite(got).all() and O.rel_l2(got, want) <= 1e-6, f"formats {fmts}"
        mid = coracle.matmul(fmts[0], x0, weights[0].cpu().numpy(), dims[0], dims[1]).astype(np.float32)
        assert O.rel_l2(got, coracle.matmul(fmts[1], mid, weights[1].cpu().numpy(), dims[1], dims[2])) <= 1e-4


def test_static_plan_rejects_long_lists():
    import torch
    import meganeura_b200 as mg
    from meganeura_b200 import _lib
    x = torch.zeros((1, 256), device="cuda")
    y = torch.zeros((1, 64), device="cuda")
    w = torch.zeros(256 * 64 // 32 * 20, dtype=torch.uint8, device="cuda")
    arr = _ops_array([(O.FMT_Q4, x, w, None, y, 256, 64, 0)] * 129)
    status = _lib.lib.mgq_plan_run_static(arr, 129, torch.cuda.current_stream().cuda_stream)
    assert status == 6                                      # MGQ_ERR_SIZE
    assert "at most 128" in _lib.last_error()
    with pytest.raises(mg.MgqError):
        _lib.check(_lib.lib.mgq_plan_run_static(None, 1, None))
