"""CPU checks for the decode-step widening: the numpy restatement of the shaders is self-consistent,
and the graph builder rejects what meganeura's builder rejects (src/graph.rs asserts)."""
import numpy as np
import pytest

from oracle import decode_oracle as D


def test_attention_direct_matches_online_softmax_form():
    rng = np.random.Generator(np.random.PCG64(3))
    for heads, kv_heads, dim, pos in [(9, 3, 64, 0), (9, 3, 64, 37), (8, 2, 128, 70), (4, 4, 64, 5)]:
        q = rng.standard_normal((1, heads * dim)).astype(np.float32)
        kc = rng.standard_normal((96, kv_heads * dim)).astype(np.float32)
        vc = rng.standard_normal((96, kv_heads * dim)).astype(np.float32)
        a = D.cached_attention(q, kc, vc, pos, heads, kv_heads, dim)
        b = D.cached_attention_online(q, kc, vc, pos, heads, kv_heads, dim)
        assert np.abs(a - b).max() < 2e-6


def test_rope_is_a_rotation_and_identity_at_position_zero():
    rng = np.random.Generator(np.random.PCG64(4))
    x = rng.standard_normal((1, 256)).astype(np.float32)
    assert np.allclose(D.rope(x, 1e4, 0, 64), x)
    r = D.rope(x, 1e6, 1234, 128)
    for h in range(2):
        assert abs(np.linalg.norm(r[0, h * 128:(h + 1) * 128]) - np.linalg.norm(x[0, h * 128:(h + 1) * 128])) < 1e-5
    # half-split pairing: element i rotates with element i + head_dim/2
    one = np.zeros((1, 64), dtype=np.float32)
    one[0, 3] = 1.0
    r = D.rope(one, 1e4, 7, 64)
    assert np.count_nonzero(np.abs(r) > 1e-12) == 2 and abs(r[0, 3 + 32]) > 0


def test_rms_norm_and_swiglu_formulas():
    x = np.array([[3.0, -4.0, 0.0, 0.0]], dtype=np.float32)
    w = np.array([1.0, 2.0, 1.0, 1.0], dtype=np.float32)
    y = D.rms_norm(x, w, 0.0)
    assert np.allclose(y, [[3 / 2.5, -8 / 2.5, 0, 0]])
    assert np.allclose(D.swiglu(np.array([[0.0, 2.0]]), np.array([[5.0, 3.0]])), [[0.0, 2.0 / (1 + np.exp(-2.0)) * 3.0]])


def test_graph_builder_rejects_what_the_reference_rejects():
    import meganeura_b200 as mg
    g = mg.Graph()
    ids = g.input_u32("token_ids", [1])
    pos = g.input_u32("kv_pos", [1])
    xf = g.input("x", [1, 64])
    table = g.parameter("table", [100, 64])
    w = g.parameter("w", [64])
    cache = g.parameter("cache", [16, 64])
    g.embedding(ids, table)
    with pytest.raises(mg.MgqError):
        g.embedding(xf, table)                       # indices must be U32
    with pytest.raises(mg.MgqError):
        g.rms_norm(xf, table, 1e-5)                  # weight must be 1D
    with pytest.raises(mg.MgqError):
        g.rope_dynamic_offset(xf, 1e4, pos, 48)      # dim must be divisible by head_dim
    with pytest.raises(mg.MgqError):
        g.rope_dynamic_offset(xf, 1e4, xf, 32)       # offset must be a U32 input
    with pytest.raises(mg.MgqError):
        g.cache_write(g.input("two", [2, 64]), cache, pos)     # new_kv must have seq_len=1
    with pytest.raises(mg.MgqError):
        g.cached_attention(xf, cache, cache, pos, 2, 1, 64)    # q dim mismatch
    with pytest.raises(mg.MgqError):
        g.swiglu_concat(g.input("odd", [1, 63]))     # SwiGLUConcat requires even N
    assert g.rms_norm(xf, w, 1e-5) > 0
    assert g.cached_attention(xf, cache, cache, pos, 1, 1, 64) > 0


def test_decode_graph_builds_for_both_model_shapes():
    import meganeura_b200 as mg
    from meganeura_b200 import decode_model as M
    for cfg in (M.small(M.SMOLLM2_135M, 2, 512), M.small(M.QWEN3_8B, 1, 512)):
        g = mg.Graph()
        logits, kc, vc = M.build_decode_graph(g, cfg, 32)
        assert len(kc) == len(vc) == cfg.num_hidden_layers and logits > 0
    assert M.packed_weight_bytes(M.QWEN3_8B) == 4730060800
