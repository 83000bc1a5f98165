"""Whole decode steps through Graph / build_inference_session / Session against the CPU decode
oracle, teacher-forced on a fixed token sequence (with random weights a free-running greedy
sequence diverges at the first near-tie, after which logits are not comparable).

Bars: relative L2 <= 1e-4 per logits vector and max-abs logit error <= 1e-2.
"""
from dataclasses import replace

import numpy as np
import pytest

from oracle import decode_oracle as D
from oracle import oracle as O

pytestmark = pytest.mark.gpu

MAX_SEQ = 96


def _configs():
    from meganeura_b200 import decode_model as M
    smol = M.small(M.SMOLLM2_135M, 2, 2048)                       # real layer shape: 576 / 9 heads / 3 KV heads / 64 / 1536
    qwen = replace(M.QWEN3_8B, name="qwen3-like", vocab_size=1024, hidden_size=512, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, intermediate_size=1024)   # head_dim 128, all Q4
    return {"smollm2": smol, "qwen3": qwen}


def _build(cfg, seed, greedy_history=0):
    """A session and the matching oracle with seeded f32 weights quantized by the reference's rules."""
    import meganeura_b200 as mg
    from meganeura_b200 import decode_model as M
    g = mg.Graph()
    logits, _, _ = M.build_decode_graph(g, cfg, MAX_SEQ)
    g.set_outputs([logits])
    s = mg.build_inference_session(g)
    rng = np.random.Generator(np.random.PCG64(seed))
    weights = {}
    table = rng.standard_normal((cfg.vocab_size, cfg.hidden_size)).astype(np.float32)
    s.set_parameter("model.embed_tokens.weight", table)
    weights["model.embed_tokens.weight"] = table
    for name in M.norm_weights(cfg):
        w = (1.0 + 0.1 * rng.standard_normal(cfg.hidden_size)).astype(np.float32)
        s.set_parameter(name, w)
        weights[name] = w
    for name, fmt, k, n in M.quantized_weights(cfg):
        w = (rng.standard_normal((k, n)) * (1.5 / np.sqrt(k))).astype(np.float32)
        s.set_parameter(name, w)                                   # quantizes on upload
        packed = O.quantize_q4_np(w) if fmt == O.FMT_Q4 else O.quantize_q8_np(w)
        weights[name] = (fmt, packed, k, n)
    if greedy_history:
        s.enable_greedy(0, "token_ids", "kv_pos", greedy_history)
    return s, D.DecodeOracle(cfg, weights, MAX_SEQ)


@pytest.mark.parametrize("which", ["smollm2", "qwen3"])
def test_teacher_forced_decode_matches_oracle(which):
    cfg = _configs()[which]
    s, oracle = _build(cfg, seed=11)
    rng = np.random.Generator(np.random.PCG64(5))
    tokens = rng.integers(0, cfg.vocab_size, size=10)
    worst_rel, worst_abs = 0.0, 0.0
    for pos, tok in enumerate(tokens):
        s.set_input_u32("token_ids", [tok])
        s.set_input_u32("kv_pos", [pos])
        s.step()
        s.wait()
        got = s.read_output(cfg.vocab_size).astype(np.float64)
        want = oracle.step(int(tok), pos)
        assert np.isfinite(got).all()
        worst_rel = max(worst_rel, O.rel_l2(got, want))
        worst_abs = max(worst_abs, np.abs(got - want).max())
    assert worst_rel <= 1e-4, f"rel-L2 {worst_rel:.3e}"
    assert worst_abs <= 1e-2, f"max-abs logit error {worst_abs:.3e}"


def test_plan_follows_the_fusion_rules():
    import meganeura_b200 as mg
    from meganeura_b200 import decode_model as M, ops
    from meganeura_b200.graph import ShaderEntry as S
    cfg = M.small(M.SMOLLM2_135M, 1, 512)

    def dispatches(horizontal, rope_cache):
        ops.set_option("session.horizontal_fusion", horizontal)
        ops.set_option("session.fuse_rope_cache", rope_cache)
        try:
            g = mg.Graph()
            logits, _, _ = M.build_decode_graph(g, cfg, 32)
            g.set_outputs([logits])
            return mg.build_inference_session(g).plan().dispatches
        finally:
            ops.set_option("session.horizontal_fusion", 2)
            ops.set_option("session.fuse_rope_cache", 1)

    rope_cache = [S.RoPEDynamic, S.RoPEDynamic, S.CacheWrite, S.CacheWrite]
    attn = [S.CachedAttention, S.MatMulGemvAdd, S.RmsNorm]
    end = [S.MatMulGemvAdd, S.RmsNorm, S.MatMulGemv]
    # nothing merged: the dispatch list the reference produces without its gate|up fusion
    none = [d.shader for d in dispatches(0, 0)]
    assert none == [S.Embedding, S.RmsNorm, S.MatMulGemv, S.MatMulGemv, S.MatMulGemv] + rope_cache + attn + \
        [S.MatMulGemv, S.MatMulGemv, S.SwiGLU] + end
    # the reference's own fusion: gate|up -> one GEMV + SwiGLUConcat (src/optimize.rs:776-879)
    ref = dispatches(1, 0)
    assert [d.shader for d in ref] == [S.Embedding, S.RmsNorm, S.MatMulGemv, S.MatMulGemv, S.MatMulGemv] + rope_cache + attn + \
        [S.MatMulGemv, S.SwiGLUConcat] + end
    gate_up = ref[12]
    assert gate_up.params == (1, 576, 3072, 0) and gate_up.workgroups == (768, 1, 1) and gate_up.weight_format == mg.WeightFormat.Q4
    assert ref[9].label == "CachedAttention[9x64]" and ref[9].workgroups == (1, 9, 1)
    # default: q|k|v in one GEMV, RoPE and cache writes in one launch
    full = dispatches(2, 1)
    assert [d.shader for d in full] == [S.Embedding, S.RmsNorm, S.MatMulGemv, S.RoPECacheWrite] + attn + \
        [S.MatMulGemv, S.SwiGLUConcat] + end
    assert full[2].params == (1, 576, 576 + 192 + 192, 0) and full[2].weight_format == mg.WeightFormat.Q8
    assert full[3].params == (576, 192, 64, 32)


def test_fusion_modes_give_the_same_logits():
    from meganeura_b200 import ops
    cfg = _configs()["smollm2"]
    outs = []
    for mode, rope_cache in ((0, 0), (1, 0), (2, 1)):
        ops.set_option("session.horizontal_fusion", mode)
        ops.set_option("session.fuse_rope_cache", rope_cache)
        try:
            s, _ = _build(cfg, seed=21)
        finally:
            ops.set_option("session.horizontal_fusion", 2)
            ops.set_option("session.fuse_rope_cache", 1)
        for pos, tok in enumerate([5, 17, 900]):
            s.set_input_u32("token_ids", [tok])
            s.set_input_u32("kv_pos", [pos])
            s.step()
        s.wait()
        outs.append(s.read_output(cfg.vocab_size))
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])    # columns are independent: bit-identical


def test_device_greedy_loop_and_graph_replay_match_host_loop():
    cfg = _configs()["qwen3"]
    steps = 12
    # host loop: argmax on the host, token and position written back every step
    s, _ = _build(cfg, seed=31)
    tok, host_tokens = 7, []
    for pos in range(steps):
        s.set_input_u32("token_ids", [tok])
        s.set_input_u32("kv_pos", [pos])
        s.step()
        s.wait()
        tok = int(np.argmax(s.read_output(cfg.vocab_size)))
        host_tokens.append(tok)
    # device loop: one warm-up step, reset, capture, then replays with no host round trip
    s2, _ = _build(cfg, seed=31, greedy_history=MAX_SEQ)
    s2.set_input_u32("token_ids", [7])
    s2.set_input_u32("kv_pos", [0])
    s2.step()
    s2.wait()
    s2.capture()
    s2.set_input_u32("token_ids", [7])
    s2.set_input_u32("kv_pos", [0])
    for _ in range(steps):
        s2.step()
    s2.wait()
    assert list(s2.read_tokens(0, steps)) == host_tokens
    assert s2.launch_count() > 0


def test_checkpoint_round_trip_in_the_reference_file_layout(tmp_path):
    """save_checkpoint writes what the reference writes (safetensors, every parameter buffer a flat F32
    tensor of byte_len/4 under its name, src/runtime.rs:4205-4273); an independent safetensors reader
    sees the packed bytes, and a file from an independent writer loads back."""
    from safetensors.numpy import load_file, save_file
    from meganeura_b200 import decode_model as M
    cfg = _configs()["smollm2"]
    s, _ = _build(cfg, seed=41)
    s.set_input_u32("token_ids", [3])
    s.set_input_u32("kv_pos", [0])
    s.step()
    s.wait()
    want = s.read_output(cfg.vocab_size)
    path = tmp_path / "ckpt.safetensors"
    s.save_checkpoint(path)
    tensors = load_file(str(path))
    # every parameter of the graph is there, members of concatenated weights under their own names
    names = {n for n, _, _, _ in M.quantized_weights(cfg)} | set(M.norm_weights(cfg)) | {"model.embed_tokens.weight"}
    names |= {f"kv_cache.layer.{i}.{kv}" for i in range(cfg.num_hidden_layers) for kv in "kv"}
    assert set(tensors) == names
    rng = np.random.Generator(np.random.PCG64(41))
    rng.standard_normal((cfg.vocab_size, cfg.hidden_size))                  # same draw order as _build
    for _ in M.norm_weights(cfg):
        rng.standard_normal(cfg.hidden_size)
    name, fmt, k, n = M.quantized_weights(cfg)[0]
    w = (rng.standard_normal((k, n)) * (1.5 / np.sqrt(k))).astype(np.float32)
    packed = O.quantize_q8_np(w) if fmt == O.FMT_Q8 else O.quantize_q4_np(w)
    assert tensors[name].dtype == np.float32 and tensors[name].shape == (packed.size // 4,)
    assert np.array_equal(tensors[name].view(np.uint8), packed)
    # a second session restores from a file written by the independent writer
    other = tmp_path / "other.safetensors"
    save_file(tensors, str(other), metadata={"adam_step": "0"})
    s2, _ = _build(cfg, seed=99)                                            # different weights
    s2.load_checkpoint(other)
    s2.set_input_u32("token_ids", [3])
    s2.set_input_u32("kv_pos", [0])
    s2.step()
    s2.wait()
    assert np.array_equal(s2.read_output(cfg.vocab_size), want)
    with pytest.raises(Exception):
        s2.load_checkpoint(tmp_path / "missing.safetensors")


def test_all_gather_graph_on_one_rank_matches_the_plain_graph():
    """The column-sharded graph built for a single rank (every all_gather stores into and waits on this
    GPU's own vectors; o, down and the lm_head push their columns from inside the GEMV) gives the plain
    graph's logits bit for bit, eagerly, after capture, and with the fused push switched off."""
    from meganeura_b200 import decode_model as M, ops
    from meganeura_b200.graph import ShaderEntry as S
    cfg = _configs()["qwen3"]
    plain = M.DecodeSession(cfg, MAX_SEQ, seed=3)
    outs = {}
    for fuse in (1, 0):
        ops.set_option("session.fuse_exchange", fuse)
        try:
            sharded = M.DecodeSession(cfg, MAX_SEQ, seed=3, gather_always=True)
        finally:
            ops.set_option("session.fuse_exchange", 1)
        shaders = [d.shader for d in sharded.session.plan().dispatches]
        assert shaders.count(S.AllGather) == 4 * cfg.num_hidden_layers + 1
        assert sharded.session.exchange_slices()[:4] == [cfg.q_dim, cfg.hidden_size, cfg.intermediate_size, cfg.hidden_size]
        for dec in (plain, sharded):
            dec.fill_caches(20, seed=9)
        got = []
        for step, (tok, pos) in enumerate([(5, 20), (77, 21), (901, 22), (3, 23)]):
            if step == 2:
                sharded.session.capture()
            want = None
            for dec in (plain, sharded):
                dec.set_position(tok, pos)
                dec.step()
                if dec is plain:
                    want = dec.logits()
            sharded.check_exchange()
            assert np.array_equal(sharded.logits(), want), f"fuse_exchange={fuse}, step {step}"
            got.append(want)
        outs[fuse] = got
    assert np.isfinite(outs[1][-1]).all()


def test_unbound_all_gather_is_refused():
    import meganeura_b200 as mg
    from meganeura_b200 import decode_model as M
    cfg = _configs()["qwen3"]
    g = mg.Graph()
    logits, _, _ = M.build_decode_graph(g, cfg, 32, gather_always=True)
    g.set_outputs([logits])
    s = mg.build_inference_session(g)
    with pytest.raises(Exception, match="bind"):
        s.step()


def test_tied_embeddings_use_the_transposed_gemv():
    """tie_word_embeddings (the reference's default for SmolLM2, src/models/smollm2.rs:45, 413-414): the
    lm_head is matmul_bt(x, embed_tokens), lowered to MatMulGemvBT with params [m, n, k, 0]."""
    from meganeura_b200.graph import ShaderEntry as S
    cfg = replace(_configs()["smollm2"], tie_word_embeddings=True)
    s, oracle = _build(cfg, seed=13)
    last = s.plan().dispatches[-1]
    assert last.shader == S.MatMulGemvBT and last.params == (1, cfg.vocab_size, cfg.hidden_size, 0)
    assert last.label == f"MatMulGemvBT[1x{cfg.vocab_size}x{cfg.hidden_size}]" and last.workgroups == (cfg.vocab_size, 1, 1)
    worst = 0.0
    for pos, tok in enumerate([9, 1500, 77]):
        s.set_input_u32("token_ids", [tok])
        s.set_input_u32("kv_pos", [pos])
        s.step()
        s.wait()
        got = s.read_output(cfg.vocab_size).astype(np.float64)
        worst = max(worst, O.rel_l2(got, oracle.step(int(tok), pos)))
    assert worst <= 1e-4, f"rel-L2 {worst:.3e}"


@pytest.mark.parametrize("k,n", [(576, 49152), (4096, 1001), (64, 7), (2048, 2)])
def test_gemv_bt_matches_float64(k, n):
    import ctypes
    import torch
    from meganeura_b200._lib import check, lib
    rng = np.random.Generator(np.random.PCG64(k + n))
    x = rng.standard_normal(k).astype(np.float32)
    b = rng.standard_normal((n, k)).astype(np.float32)
    xd, bd = torch.from_numpy(x).cuda(), torch.from_numpy(b).cuda()
    y = torch.full((n + 8,), 123.0, device="cuda")
    check(lib.mgq_gemv_bt(xd.data_ptr(), bd.data_ptr(), y.data_ptr(), k, n, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    want = b.astype(np.float64) @ x.astype(np.float64)
    assert O.rel_l2(y[:n].cpu().numpy().astype(np.float64), want) <= 1e-5
    assert bool((y[n:] == 123.0).all())                       # nothing written past the end
    with pytest.raises(Exception):
        check(lib.mgq_gemv_bt(xd.data_ptr(), bd.data_ptr(), y.data_ptr(), 6, n, None))
