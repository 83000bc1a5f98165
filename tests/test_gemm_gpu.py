"""GPU parity of the dequantize-fused GEMM (M > 16, f32 or bf16 activations) against the oracle."""
import numpy as np
import pytest

from oracle import oracle as O
from gpu_util import check_against_oracle, run_matmul

pytestmark = pytest.mark.gpu

FMTS = [O.FMT_Q4, O.FMT_Q8]


def _x(m, k, seed):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal((m, k)).astype(np.float32)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,k,n", [(17, 64, 4), (63, 96, 70), (64, 576, 192), (65, 1024, 130), (128, 1024, 2048), (6, 1024, 2048)])
def test_f32_activations(coracle, fmt, m, k, n):
    w = O.synth_weights(fmt, k, n, seed=m + k + n)
    x = _x(m, k, 1)
    got = run_matmul(fmt, x, w, k, n, route="gemm")
    check_against_oracle(coracle, fmt, x, w, k, n, got)


@pytest.mark.parametrize("fmt", FMTS)
def test_addend(coracle, fmt):
    m, k, n = 70, 576, 200
    w = O.synth_weights(fmt, k, n, seed=4)
    x, d = _x(m, k, 5), _x(m, n, 6)
    got = run_matmul(fmt, x, w, k, n, addend=d, route="gemm")
    check_against_oracle(coracle, fmt, x, w, k, n, got, addend=d)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,k,n", [(64, 256, 128), (512, 1024, 512), (200, 4096, 264)])
def test_bf16_activations(coracle, fmt, m, k, n):
    import torch
    w = O.synth_weights(fmt, k, n, seed=m ^ n)
    xb = torch.from_numpy(_x(m, k, 2)).cuda().to(torch.bfloat16)
    x = xb.float().cpu().numpy()                              # the bf16 values are the inputs
    got = run_matmul(fmt, xb, w, k, n, route="gemm")
    check_against_oracle(coracle, fmt, x, w, k, n, got)


def test_reference_q4_matmul_correctness(coracle):
    # tests/gpu_smoke.rs:2680-2771: m=6, k=1024, n=2048, weights quantized on upload,
    # GPU result within 0.1 of the CPU product over dequantize(quantize(b)).
    m, k, n = 6, 1024, 2048
    a = (((np.arange(m * k) % 7).astype(np.float32) - 3.0) * 0.5).astype(np.float32).reshape(m, k)
    i = np.arange(k * n)
    b = ((i % 11).astype(np.float32) - np.float32(5.0)) * np.float32(0.3)
    b = np.where(i % 1000 == 0, b * np.float32(5.0), b).astype(np.float32).reshape(k, n)
    from meganeura_b200 import ops
    packed = ops.quantize(O.FMT_Q4, b)
    cpu = coracle.matmul(O.FMT_Q4, a, packed, k, n, wide=False, nthreads=8)
    for route in ("auto", "gemm"):
        got = run_matmul(O.FMT_Q4, a, packed, k, n, route=route)
        assert np.abs(got - cpu).max() < 0.1
        check_against_oracle(coracle, O.FMT_Q4, a, packed, k, n, got)
