"""CPU tests of the oracle: the reference's own known-answer tests restated, the golden
fixtures, and agreement of the two restatements (C and numpy)."""
import numpy as np
import pytest

from oracle import oracle as O

FMTS = [(O.FMT_Q4, "q4"), (O.FMT_Q8, "q8")]


def test_q4_roundtrip_identity(coracle):
    # src/runtime.rs:2222-2242: 32x1 column, (i-16)*0.1, every element within 0.3
    data = ((np.arange(32, dtype=np.float32) - 16.0) * 0.1).astype(np.float32).reshape(32, 1)
    dec = coracle.dequantize(O.FMT_Q4, coracle.quantize(O.FMT_Q4, data), 32, 1)
    assert np.all(np.abs(data - dec) < 0.3)


def test_q4_roundtrip_matrix(coracle):
    # src/runtime.rs:2245-2266: 32x4, ((i%17)-8)*0.05, max error below 0.3
    data = (((np.arange(128) % 17).astype(np.float32) - 8.0) * 0.05).astype(np.float32).reshape(32, 4)
    dec = coracle.dequantize(O.FMT_Q4, coracle.quantize(O.FMT_Q4, data), 32, 4)
    assert np.abs(data - dec).max() < 0.3


def test_q4_decode_f16_matches_half_crate(coracle):
    # src/runtime.rs:2268-2290: the shader's decode equals IEEE for these six patterns
    for bits in [0x3C00, 0x4000, 0x3800, 0xBC00, 0x0000, 0x7BFF]:
        expected = float(np.array([bits], dtype=np.uint16).view(np.float16).astype(np.float32)[0])
        assert abs(expected - coracle.lib.orc_f16_bits_to_f32_shader(bits)) < 1e-6
        assert expected == coracle.lib.orc_f16_bits_to_f32_ieee(bits)


def test_f16_decode_all_patterns(coracle):
    bits = np.arange(65536, dtype=np.uint32)
    ieee = np.array([coracle.lib.orc_f16_bits_to_f32_ieee(int(b)) for b in bits], dtype=np.float32)
    want = bits.astype(np.uint16).view(np.float16).astype(np.float32)
    same = (ieee.view(np.uint32) == want.view(np.uint32)) | (np.isnan(ieee) & np.isnan(want))
    assert same.all()
    shader = np.array([coracle.lib.orc_f16_bits_to_f32_shader(int(b)) for b in bits], dtype=np.float32)
    expo = (bits >> 10) & 0x1F
    normal = (expo != 0) & (expo != 31)
    assert (shader[normal] == want[normal]).all()          # identical on every normal binary16
    assert (shader[expo == 0] == 0).all()                  # subnormals flushed to +-0
    assert (O.f16_bits_to_f32_shader_np(bits) .view(np.uint32) == shader.view(np.uint32)).all()


def test_f16_encode_round_to_nearest_even(coracle):
    rng = np.random.default_rng(3)
    vals = (rng.standard_normal(20000) * np.exp(rng.uniform(-20, 12, 20000))).astype(np.float32)
    vals = np.concatenate([vals, np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 6.1e-5, 5.96e-8, 2.98e-8], np.float32)])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([coracle.lib.orc_f32_to_f16_bits(float(v)) for v in vals], dtype=np.uint16)
    assert (got == want).all()


def test_q4_matmul_correctness_formulas(coracle):
    # tests/gpu_smoke.rs:2680-2771 with its own inputs (m=6,k=1024,n=2048): the f32 matmul over
    # dequantize(quantize(b)) must sit within 0.1 of the same product accumulated in f64, and the
    # quantization error against the f32 weights must stay small.
    m, k, n = 6, 1024, 2048
    a = (((np.arange(m * k) % 7).astype(np.float32) - 3.0) * 0.5).astype(np.float32).reshape(m, k)
    i = np.arange(k * n)
    b = ((i % 11).astype(np.float32) - np.float32(5.0)) * np.float32(0.3)
    b = np.where(i % 1000 == 0, b * np.float32(5.0), b).astype(np.float32).reshape(k, n)
    packed = coracle.quantize(O.FMT_Q4, b)
    assert packed.size == k * n // 32 * 20
    c32 = coracle.matmul(O.FMT_Q4, a, packed, k, n, wide=False, nthreads=4)
    c64 = coracle.matmul(O.FMT_Q4, a, packed, k, n, wide=True, nthreads=4)
    assert np.abs(c32 - c64).max() < 0.1
    deq = coracle.dequantize(O.FMT_Q4, packed, k, n)
    step = (b.reshape(k // 32, 32, n).max(1) - b.reshape(k // 32, 32, n).min(1)) / 15.0
    assert (np.abs(deq - b).reshape(k // 32, 32, n) <= step[:, None, :] * 0.5 + 2e-2).all()


@pytest.mark.parametrize("name", ["ident", "mat", "smoke"])
def test_golden_bytes(coracle, golden, name):
    w = golden[f"{name}_w"]
    k, n = w.shape
    for fmt, tag in FMTS:
        packed = coracle.quantize(fmt, w)
        assert (packed == golden[f"{name}_{tag}"]).all()
        assert (coracle.dequantize(fmt, packed, k, n) == golden[f"{name}_d{tag}"]).all()


def test_golden_matmul(coracle, golden):
    a = golden["smoke_a"]
    for fmt, tag in FMTS:
        c = coracle.matmul(fmt, a, golden[f"smoke_{tag}"], 64, 12)
        assert np.allclose(c, golden[f"smoke_c_{tag}"], rtol=0, atol=1e-12)
        y = coracle.matmul(fmt, golden["synth_x"], golden[f"synth_{tag}"], 64, 8, addend=golden["synth_addend"])
        assert np.allclose(y, golden[f"synth_y_{tag}"], rtol=0, atol=1e-12)
        sh = coracle.shard_columns(fmt, golden[f"synth_{tag}"], 64, 8, 4, 8)
        assert (sh == golden[f"synth_shard_{tag}"]).all()


def test_appendix_offsets(coracle):
    # K=64, N=4: element (k=37, n=2) lives in block 5, position 5.
    k, n = 64, 4
    codes8 = np.zeros((k, n), dtype=np.int8)
    codes8[37, 2] = -77
    sb = np.full((n, 2), 0x3C00, dtype=np.uint16)           # scale 1.0
    p8 = coracle.pack_q8(codes8, sb)
    assert p8.size == 288 and p8[189] == np.uint8(-77 & 0xFF) and p8[180] == 0x00 and p8[181] == 0x3C
    codes4 = np.zeros((k, n), dtype=np.uint8)
    codes4[37, 2] = 0xB
    p4 = coracle.pack_q4(codes4, sb, np.zeros((n, 2), np.uint16))
    assert p4.size == 160 and p4[114] == 0xB0
    assert (p4 == O.pack_q4_np(codes4, sb, np.zeros((n, 2), np.uint16))).all()
    assert (p8 == O.pack_q8_np(codes8, sb)).all()
    assert coracle.dequant_shader_elem(O.FMT_Q4, p4, 37, 2, k, n) == 11.0
    assert coracle.dequant_shader_elem(O.FMT_Q8, p8, 37, 2, k, n) == -77.0


@pytest.mark.parametrize("k,n", [(32, 1), (64, 4), (576, 192), (1024, 64)])
def test_c_and_numpy_restatements_agree(coracle, k, n):
    rng = np.random.default_rng(k * 131 + n)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    w[:32, 0] = 0.25                                        # a flat block: d = 1.0 branch
    x = rng.standard_normal((3, k)).astype(np.float32)
    for fmt, _ in FMTS:
        packed = coracle.quantize(fmt, w)
        np_packed = (O.quantize_q4_np if fmt == O.FMT_Q4 else O.quantize_q8_np)(w)
        assert (packed == np_packed).all()
        assert (coracle.dequantize(fmt, packed, k, n) == O.dequantize_np(fmt, packed, k, n)).all()
        assert np.allclose(coracle.matmul(fmt, x, packed, k, n), O.matmul_f64_np(fmt, x, packed, k, n), rtol=1e-12, atol=1e-12)
        # shader-variant dequant equals the CPU variant whenever scales are normal binary16
        c0 = coracle.matmul(fmt, x, packed, k, n, variant=0)
        c1 = coracle.matmul(fmt, x, packed, k, n, variant=1)
        assert (c0 == c1).all()


def test_sharded_columns_reassemble(coracle):
    k, n, world = 128, 24, 4
    x = np.random.default_rng(5).standard_normal((2, k)).astype(np.float32)
    for fmt, _ in FMTS:
        w = O.synth_weights(fmt, k, n, seed=11)
        full = coracle.matmul(fmt, x, w, k, n)
        parts = []
        for r in range(world):
            n0, n1 = r * n // world, (r + 1) * n // world
            sh = coracle.shard_columns(fmt, w, k, n, n0, n1)
            assert sh.size == O.packed_bytes(fmt, k, n1 - n0)
            parts.append(coracle.matmul(fmt, x, sh, k, n1 - n0))
        assert (np.concatenate(parts, axis=1) == full).all()
