"""GEMV with 3..16 rows: the integer tensor-core kernel that reads the weights once per 8 rows
(mgq_gemv routes there for k % 256 == 0), against the f64 oracle and against the two-rows-at-a-time
streaming kernels."""
import numpy as np
import pytest

from oracle import oracle as O
from gpu_util import check_against_oracle, run_matmul, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", [O.FMT_Q4, O.FMT_Q8])
@pytest.mark.parametrize("m,k,n", [(3, 256, 64), (4, 4096, 1024), (8, 4096, 4096), (8, 1536, 576), (5, 12288, 512),
                                   (9, 4096, 256), (16, 2048, 1000), (8, 4096, 24), (7, 768, 100), (8, 8192, 2052)])
def test_batched_gemv_matches_oracle(coracle, fmt, m, k, n):
    rng = np.random.Generator(np.random.PCG64(m * 1000 + n))
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[0, :32] *= 1e-3                                     # blocks of very different magnitude
    x[m - 1, 32:64] *= 1e3
    packed = O.synth_weights(fmt, k, n, seed=k + n)
    addend = rng.standard_normal((m, n)).astype(np.float32) if n % 3 == 0 else None
    got = run_matmul(fmt, x, packed, k, n, addend=addend, route="gemv")
    check_against_oracle(coracle, fmt, x, packed, k, n, got, addend=addend)


def test_batched_kernel_agrees_with_streaming_kernels(coracle):
    from meganeura_b200 import ops
    fmt, m, k, n = O.FMT_Q4, 8, 4096, 2048
    rng = np.random.Generator(np.random.PCG64(77))
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((k, n)).astype(np.float32) * 0.05
    packed = coracle.quantize(fmt, w)                     # real quantizer output: arbitrary minima and scales
    a = run_matmul(fmt, x, packed, k, n, route="gemv")
    ops.set_option("gemv.batch_mma", 0)
    try:
        b = run_matmul(fmt, x, packed, k, n, route="gemv")
    finally:
        ops.set_option("gemv.batch_mma", 1)
    assert O.rel_l2(a, b) < 2e-6                          # same fixed-point activations, other summation order
    check_against_oracle(coracle, fmt, x, packed, k, n, a)


def test_rows_are_independent_and_zero_rows_stay_zero():
    fmt, k, n = O.FMT_Q8, 4096, 512
    rng = np.random.Generator(np.random.PCG64(5))
    packed = O.synth_weights(fmt, k, n, seed=9)
    x = rng.standard_normal((6, k)).astype(np.float32)
    x[2] = 0.0
    full = run_matmul(fmt, x, packed, k, n, route="gemv")
    assert (full[2] == 0.0).all()
    single = run_matmul(fmt, x[4:5], packed, k, n, route="gemv")         # one row: the streaming kernel
    assert O.rel_l2(full[4], single[0]) < 2e-6


def test_sliced_batch_survives_a_larger_later_call(coracle):
    """K > 4096 runs in K-slices whose partial sums live in a library-owned buffer.  A CUDA graph that
    captured a launch must keep working after a later, larger call has made the library allocate a
    bigger buffer: the old one is never freed or moved."""
    import torch
    from meganeura_b200 import ops
    k, n = 12288, 512
    w = to_dev(O.synth_weights(O.FMT_Q4, k, n, seed=77))
    rng = np.random.Generator(np.random.PCG64(78))
    x4 = to_dev(rng.standard_normal((4, k)).astype(np.float32))
    y4 = torch.zeros((4, n), device="cuda")
    ops.matmul(O.FMT_Q4, x4, w, k, n, out=y4, route="gemv")                 # first use sizes the buffer (before capture)
    torch.cuda.synchronize()
    want = y4.clone()
    g, s = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            ops.matmul(O.FMT_Q4, x4, w, k, n, out=y4, route="gemv")
    n_big = 4096
    w_big = to_dev(O.synth_weights(O.FMT_Q4, k, n_big, seed=79))
    x16 = to_dev(rng.standard_normal((16, k)).astype(np.float32))
    big = ops.matmul(O.FMT_Q4, x16, w_big, k, n_big, route="gemv")          # needs a larger partial-sum buffer
    torch.cuda.synchronize()
    y4.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y4, want)
    ref = coracle.matmul(O.FMT_Q4, x16.cpu().numpy(), w_big.cpu().numpy(), k, n_big)
    assert O.rel_l2(big.cpu().numpy(), ref) <= 1e-4
