"""The benchmark configurations at their full sizes (the other test files use reduced shapes).

  * SmolLM2-135M-architecture decode: all 30 layers, vocabulary 49152, weights ~ N(0, 0.02^2) quantized
    on upload (MLP Q4; attention and the untied lm_head Q8), teacher-forced tokens against the CPU
    decode oracle: rel-L2 <= 1e-4 and max-abs logit error <= 1e-2 per token.
  * Q8 prefill GEMM 512 x 4096 x 14336 (bf16 activations, tcgen05 kernel) at full size; the f64 oracle
    is evaluated on a seeded sample of columns taken from every 112-column strip plus the whole last
    strip: rel-L2 <= 1e-4.
  * A Qwen3-8B-shaped layer pair (hidden 4096, 32 query / 8 KV heads of 128, FFN 12288, Q4) with a
    small vocabulary, teacher-forced at context >= 1024.
"""
from dataclasses import replace

import numpy as np
import pytest

from oracle import decode_oracle as D
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _build(cfg, max_seq, seed, std=0.02):
    import meganeura_b200 as mg
    from meganeura_b200 import decode_model as M
    g = mg.Graph()
    logits, _, _ = M.build_decode_graph(g, cfg, max_seq)
    g.set_outputs([logits])
    s = mg.build_inference_session(g)
    rng = np.random.Generator(np.random.PCG64(seed))
    weights = {}
    table = rng.standard_normal((cfg.vocab_size, cfg.hidden_size), dtype=np.float32)
    s.set_parameter("model.embed_tokens.weight", table)
    weights["model.embed_tokens.weight"] = table
    for name in M.norm_weights(cfg):
        w = np.ones(cfg.hidden_size, dtype=np.float32)
        s.set_parameter(name, w)
        weights[name] = w
    for name, fmt, k, n in M.quantized_weights(cfg):
        w = rng.standard_normal((k, n), dtype=np.float32) * np.float32(std)
        s.set_parameter(name, w)                                   # quantizes on upload (mgq_quantize_q4 / q8)
        packed = O.quantize_q4_np(w) if fmt == O.FMT_Q4 else O.quantize_q8_np(w)
        weights[name] = (fmt, packed, k, n)
    return s, D.DecodeOracle(cfg, weights, max_seq)


def _teacher_forced(s, oracle, cfg, tokens, first_pos=0):
    worst_rel, worst_abs = 0.0, 0.0
    for i, tok in enumerate(tokens):
        pos = first_pos + i
        s.set_input_u32("token_ids", [int(tok)])
        s.set_input_u32("kv_pos", [pos])
        s.step()
        s.wait()
        got = s.read_output(cfg.vocab_size).astype(np.float64)
        want = oracle.step(int(tok), pos)
        assert np.isfinite(got).all()
        worst_rel = max(worst_rel, O.rel_l2(got, want))
        worst_abs = max(worst_abs, float(np.abs(got - want).max()))
    return worst_rel, worst_abs


def test_smollm2_135m_full_model_decode():
    from meganeura_b200 import decode_model as M
    cfg = M.SMOLLM2_135M                                           # 30 layers, vocab 49152
    s, oracle = _build(cfg, 32, seed=31)
    tokens = np.random.Generator(np.random.PCG64(7)).integers(0, cfg.vocab_size, size=8)
    rel, err = _teacher_forced(s, oracle, cfg, tokens)
    assert rel <= 1e-4, f"rel-L2 {rel:.3e}"
    assert err <= 1e-2, f"max-abs logit error {err:.3e}"


def test_qwen3_8b_layer_shape_at_long_context():
    from meganeura_b200 import decode_model as M
    cfg = replace(M.QWEN3_8B, name="qwen3-8b-2l", num_hidden_layers=2, vocab_size=2048)
    context, max_seq = 1024, 1040
    s, oracle = _build(cfg, max_seq, seed=41)
    # a pre-filled context: the same seeded rows in the session's caches and in the oracle's
    rng = np.random.Generator(np.random.PCG64(43))
    for i in range(cfg.num_hidden_layers):
        for kind, cache in (("k", oracle.k_cache), ("v", oracle.v_cache)):
            rows = np.zeros((max_seq, cfg.kv_dim), dtype=np.float32)
            rows[:context] = rng.standard_normal((context, cfg.kv_dim), dtype=np.float32) * np.float32(0.1)
            s.set_parameter(f"kv_cache.layer.{i}.{kind}", rows)
            cache[i][:] = rows
    tokens = np.random.Generator(np.random.PCG64(9)).integers(0, cfg.vocab_size, size=8)
    rel, err = _teacher_forced(s, oracle, cfg, tokens, first_pos=context)
    assert rel <= 1e-4, f"rel-L2 {rel:.3e}"
    assert err <= 1e-2, f"max-abs logit error {err:.3e}"


def test_prefill_gemm_full_size(coracle):
    import torch
    from meganeura_b200 import ops
    m, k, n = 512, 4096, 14336
    rng = np.random.Generator(np.random.PCG64(51))
    w = O.synth_weights(O.FMT_Q8, k, n, seed=52)
    a = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).cuda().to(torch.bfloat16)
    c = ops.matmul(O.FMT_Q8, a, torch.from_numpy(w).cuda(), k, n, route="gemm")
    torch.cuda.synchronize()
    ops.device_status()
    got = c.cpu().numpy()
    assert np.isfinite(got).all()
    strip = 112                                                    # the kernel's column strip per CTA
    cols = []
    for s0 in range(0, n, strip):                                  # two seeded columns out of every strip ...
        width = min(strip, n - s0)
        cols += sorted(int(v) for v in (s0 + rng.choice(width, size=2, replace=False)))
    last0 = (n - 1) // strip * strip
    cols = sorted(set(cols) | set(range(last0, n)))                # ... and the whole last strip
    assert len(cols) >= 256
    a_f32 = a.float().cpu().numpy()
    # the sampled columns as a packed weight of their own (a block never spans columns)
    packed = np.concatenate([O.shard_columns_np(O.FMT_Q8, w, k, n, cidx, cidx + 1) for cidx in cols])
    want = coracle.matmul(O.FMT_Q8, a_f32, packed, k, len(cols), wide=True, nthreads=8)
    sample = got[:, cols]
    assert O.rel_l2(sample, want) <= 1e-4
    for r in range(0, m, 37):
        assert O.rel_l2(sample[r], want[r]) <= 1e-4
