"""GPU parity of the dequantize-fused GEMV against the oracle (through the C ABI)."""
import numpy as np
import pytest

from oracle import oracle as O
from gpu_util import check_against_oracle, run_matmul, tile_columns, to_dev

pytestmark = pytest.mark.gpu

FMTS = [O.FMT_Q4, O.FMT_Q8]


def _x(m, k, seed):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal((m, k)).astype(np.float32)


def test_golden_fixture(golden, coracle):
    for fmt, tag in ((O.FMT_Q4, "q4"), (O.FMT_Q8, "q8")):
        got = run_matmul(fmt, golden["synth_x"], golden[f"synth_{tag}"], 64, 8, addend=golden["synth_addend"], route="gemv")
        assert O.rel_l2(got, golden[f"synth_y_{tag}"]) <= 1e-5
        got = run_matmul(fmt, golden["smoke_a"], golden[f"smoke_{tag}"], 64, 12, route="gemv")
        assert O.rel_l2(got, golden[f"smoke_c_{tag}"]) <= 1e-5


def test_config0_q8_576x1536(coracle):
    # the benchmark's first configuration: y[1x1536] = x[1x576] . dequant(W[576x1536]), Q8
    k, n = 576, 1536
    w = O.synth_weights(O.FMT_Q8, k, n, seed=1)
    x = _x(1, k, 2)
    got = run_matmul(O.FMT_Q8, x, w, k, n, route="gemv")
    check_against_oracle(coracle, O.FMT_Q8, x, w, k, n, got)


@pytest.mark.parametrize("k,n", [(576, 576), (576, 192), (576, 1536), (1536, 576), (576, 49152), (576, 3072)])
def test_smollm2_q4_sweep(coracle, k, n):
    w = O.synth_weights(O.FMT_Q4, k, n, seed=k + n)
    x = _x(1, k, k * 7 + n)
    got = run_matmul(O.FMT_Q4, x, w, k, n, route="gemv")
    check_against_oracle(coracle, O.FMT_Q4, x, w, k, n, got)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("k,n,m", [
    (32, 4, 1), (32, 8, 2), (64, 12, 1), (64, 4, 7), (96, 20, 3), (576, 8, 1), (1024, 2048, 6),
    (1056, 36, 1),            # bpc = 33: idle lanes in every column group
    (4096, 1024, 1), (4096, 4096, 1), (4096, 24576, 1), (12288, 4096, 1), (12288, 512, 2),
    (16384, 64, 1),           # bpc = 512
    (32768, 16, 1),           # bpc = 1024: one column per 1024-thread CTA
    (4096, 1024, 8), (4096, 256, 16), (3072, 1024, 5),
])
def test_shape_grid(coracle, fmt, k, n, m):
    w = O.synth_weights(fmt, k, n, seed=k ^ (n << 3) ^ m)
    x = _x(m, k, 99 + k + n + m)
    got = run_matmul(fmt, x, w, k, n, route="gemv")
    check_against_oracle(coracle, fmt, x, w, k, n, got)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("k,n,m", [(576, 576, 1), (1536, 576, 1), (4096, 4096, 1), (4096, 4096, 4)])
def test_addend(coracle, fmt, k, n, m):
    # MatMulGemvAdd: + src[idx] (src/shaders/matmul_gemv_add.wgsl:48-50)
    w = O.synth_weights(fmt, k, n, seed=5)
    x = _x(m, k, 6)
    d = _x(m, n, 7)
    got = run_matmul(fmt, x, w, k, n, addend=d, route="gemv")
    check_against_oracle(coracle, fmt, x, w, k, n, got, addend=d)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("k,n", [(64, 1), (64, 3), (96, 5), (576, 6), (128, 257), (128, 300)])
def test_ragged_n(coracle, fmt, k, n):
    # N not a multiple of 4 (the reference sends these to the tiled kernel; tests/gemv_parity.rs:107-113)
    w = O.synth_weights(fmt, k, n, seed=n)
    x = _x(2, k, n + 1)
    got = run_matmul(fmt, x, w, k, n, route="gemv")
    check_against_oracle(coracle, fmt, x, w, k, n, got)


@pytest.mark.parametrize("fmt", FMTS)
def test_quantized_real_weights(coracle, fmt):
    # weights produced by the quantizer itself (asymmetric Q4 with m != -8d, flat blocks, zeros)
    k, n = 1024, 512
    rng = np.random.default_rng(8)
    wf = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    wf[:32, 0] = 0.0
    wf[32:64, 1] = 0.5
    packed = coracle.quantize(fmt, wf)
    x = _x(1, k, 9)
    got = run_matmul(fmt, x, packed, k, n, route="gemv")
    check_against_oracle(coracle, fmt, x, packed, k, n, got)


@pytest.mark.parametrize("fmt", FMTS)
def test_activation_extremes(coracle, fmt):
    # tiny, huge and mixed-magnitude activations keep f32-level accuracy
    k, n = 4096, 256
    w = O.synth_weights(fmt, k, n, seed=3)
    base = _x(1, k, 4)
    for scale in (1e-6, 1e6):
        x = (base * np.float32(scale)).astype(np.float32)
        got = run_matmul(fmt, x, w, k, n, route="gemv")
        check_against_oracle(coracle, fmt, x, w, k, n, got)
    x = base.copy()
    x[0, ::97] *= 1000.0
    x[0, 5] = 0.0
    got = run_matmul(fmt, x, w, k, n, route="gemv")
    check_against_oracle(coracle, fmt, x, w, k, n, got)


@pytest.mark.parametrize("fmt", FMTS)
def test_linearity_and_zero_at_full_size(fmt):
    # size-independent properties at the largest decode shape (no CPU oracle pass needed):
    # W.(a*x1 + x2) == a*W.x1 + W.x2 within f32 rounding, and W.0 == 0 exactly.
    import torch
    from meganeura_b200 import ops
    k, n0, reps = 4096, 4748, 32                              # 32 * 4748 = 151936 columns (Qwen3 vocabulary)
    n = n0 * reps
    w = tile_columns(fmt, to_dev(O.synth_weights(fmt, k, n0, seed=12)), k, n0, reps)
    g = torch.Generator(device="cuda").manual_seed(1)
    x1 = torch.randn((1, k), device="cuda", generator=g)
    x2 = torch.randn((1, k), device="cuda", generator=g)
    y1 = ops.matmul(fmt, x1, w, k, n, route="gemv")
    y2 = ops.matmul(fmt, x2, w, k, n, route="gemv")
    y3 = ops.matmul(fmt, 2.0 * x1 + x2, w, k, n, route="gemv")
    ref = 2.0 * y1.double() + y2.double()
    assert float((y3.double() - ref).norm() / ref.norm()) < 1e-5
    y0 = ops.matmul(fmt, torch.zeros((1, k), device="cuda"), w, k, n, route="gemv")
    assert float(y0.abs().max()) == 0.0
    assert bool((y1[0, :n0] == y1[0, n - n0:]).all())          # repeated columns give identical results


@pytest.mark.parametrize("fmt", FMTS)
def test_column_shards_are_bit_exact(fmt):
    # a column range run as its own weight reproduces the unsharded columns bit for bit
    k, n, world = 4096, 2048, 8
    w = O.synth_weights(fmt, k, n, seed=21)
    x = _x(1, k, 22)
    full = run_matmul(fmt, x, w, k, n, route="gemv")
    from meganeura_b200 import ops
    for r in (0, 3, 7):
        n0, n1 = r * n // world, (r + 1) * n // world
        part = run_matmul(fmt, x, ops.shard_columns(fmt, w, k, n, n0, n1), k, n1 - n0, route="gemv")
        assert (part == full[:, n0:n1]).all()


def test_subnormal_scales_follow_cpu_dequantize(coracle):
    # binary16 subnormal scales: the library decodes IEEE like dequantize_q8_0 (src/runtime.rs:2204);
    # the WGSL helper would flush them to zero (src/codegen.rs:781).
    k, n = 64, 8
    rng = np.random.default_rng(2)
    codes = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    sb = np.full((n, 2), 0x0200, dtype=np.uint16)            # 2^-15, subnormal
    w = O.pack_q8_np(codes, sb)
    x = _x(1, k, 3)
    got = run_matmul(O.FMT_Q8, x, w, k, n, route="gemv")
    check_against_oracle(coracle, O.FMT_Q8, x, w, k, n, got)
    assert np.abs(got).max() > 0
