"""The tcgen05/TMEM GEMM (bf16 activations, M >= 64, K % 128 == 0) against the oracle."""
import numpy as np
import pytest

from oracle import oracle as O
from gpu_util import check_against_oracle, run_matmul

pytestmark = pytest.mark.gpu


def _case(coracle, fmt, m, k, n, addend=False, seed=0):
    import torch
    from meganeura_b200 import ops
    rng = np.random.Generator(np.random.PCG64(seed + m + k + n))
    w = O.synth_weights(fmt, k, n, seed=seed + 1)
    xb = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    x = xb.float().cpu().numpy()                                   # the bf16 values are the inputs
    d = rng.standard_normal((m, n)).astype(np.float32) if addend else None
    got = run_matmul(fmt, xb, w, k, n, addend=d, route="gemm")
    ops.device_status()                                            # no bounded wait ran out
    return check_against_oracle(coracle, fmt, x, w, k, n, got, addend=d)


@pytest.mark.parametrize("fmt", [O.FMT_Q8, O.FMT_Q4])
def test_single_tile(coracle, fmt):
    _case(coracle, fmt, 128, 128, 128)


@pytest.mark.parametrize("fmt", [O.FMT_Q8, O.FMT_Q4])
@pytest.mark.parametrize("m,k,n", [(128, 512, 256), (64, 256, 128), (200, 1024, 264), (512, 1024, 512), (130, 4096, 200)])
def test_shapes(coracle, fmt, m, k, n):
    _case(coracle, fmt, m, k, n)


@pytest.mark.parametrize("fmt", [O.FMT_Q8, O.FMT_Q4])
def test_addend_and_ragged_n(coracle, fmt):
    _case(coracle, fmt, 192, 512, 380, addend=True)
    _case(coracle, fmt, 100, 256, 130, addend=True)               # N % 4 != 0: scalar stores


def test_prefill_config_slice(coracle):
    # the prefill configuration's K and M (512 tokens, K = 4096) on a 1024-column slice of N = 14336
    err = _case(coracle, O.FMT_Q8, 512, 4096, 1024)
    assert err < 2e-5


def test_tiled_kernel_agrees(coracle):
    # the same inputs through the CUDA-core kernel ("gemm.force_tiled") give the same answer within tolerance
    import torch
    from meganeura_b200 import ops
    m, k, n = 128, 512, 256
    w = O.synth_weights(O.FMT_Q8, k, n, seed=3)
    xb = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    wd = torch.from_numpy(w).cuda()
    tc = ops.matmul(O.FMT_Q8, xb, wd, k, n, route="gemm")
    ops.set_option("gemm.force_tiled", 1)
    try:
        tiled = ops.matmul(O.FMT_Q8, xb, wd, k, n, route="gemm")
    finally:
        ops.set_option("gemm.force_tiled", 0)
    torch.cuda.synchronize()
    assert float((tc.double() - tiled.double()).norm() / tiled.double().norm()) < 2e-5
