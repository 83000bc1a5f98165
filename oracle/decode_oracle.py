"""TEST INFRASTRUCTURE ONLY -- CPU restatement (numpy) of the operators between the quantized
matmuls of a meganeura decode step, and of the whole single-token decode graph.

Only tests/, __graft_entry__.smoke() and the CPU-baseline legs of bench.py may import this module;
the product path never does.

Each function restates one reference shader (paths inside the meganeura tree):
  embedding        src/shaders/embedding.wgsl
  rms_norm         src/shaders/rms_norm.wgsl           (mean of squares, + eps, rsqrt, * weight)
  rope             src/shaders/rope_dynamic.wgsl        (HF half-split inside each head)
  cache_write      src/shaders/cache_write.wgsl
  cached_attention src/shaders/cached_attention.wgsl    (scale 1/sqrt(head_dim), softmax over 0..kv_pos)
  swiglu           src/shaders/swiglu_concat.wgsl       (gate * sigmoid(gate) * up)
  decode_step      src/models/smollm2.rs:315-421        (build_decode_graph)
The matmuls use the dequantized weights of oracle.py (the reference's CPU dequantizers) in f64.

Parity status: these shaders have no golden vectors in the reference (its decode tests compare
against a HuggingFace checkpoint that is not available offline), so this restatement is pinned by
source only: "parity unpinned" for the decode-step operators.
"""
from __future__ import annotations

import numpy as np

from . import oracle as O


def embedding(ids, table):
    return np.asarray(table)[np.asarray(ids, dtype=np.int64)]


def rms_norm(x, weight, eps):
    x = np.asarray(x, dtype=np.float64)
    ms = (x * x).mean(axis=-1, keepdims=True)
    return x / np.sqrt(ms + eps) * np.asarray(weight, dtype=np.float64)


def rope(x, theta, pos_offset, head_dim):
    """x [seq, dim]; position of row r is r + pos_offset; pairs (i, i + head_dim/2) inside each head."""
    x = np.asarray(x, dtype=np.float64)
    seq, dim = x.shape
    half = head_dim // 2
    out = x.copy()
    pair = np.arange(half)
    # the shader evaluates pow / cos / sin in f32
    inv_freq = np.power(np.float32(theta), (-2.0 * pair.astype(np.float32) / np.float32(head_dim)).astype(np.float32)).astype(np.float32)
    for r in range(seq):
        angle = (np.float32(r + pos_offset) * inv_freq).astype(np.float32)
        c, s = np.cos(angle.astype(np.float64)), np.sin(angle.astype(np.float64))
        for h in range(dim // head_dim):
            b = h * head_dim
            v0, v1 = x[r, b:b + half], x[r, b + half:b + head_dim]
            out[r, b:b + half] = v0 * c - v1 * s
            out[r, b + half:b + head_dim] = v0 * s + v1 * c
    return out


def cache_write(cache, new_kv, kv_pos):
    cache[kv_pos, :] = np.asarray(new_kv).reshape(-1)
    return cache


def cached_attention(q, k_cache, v_cache, kv_pos, num_heads, num_kv_heads, head_dim):
    q = np.asarray(q, dtype=np.float64).reshape(num_heads, head_dim)
    kv_len = kv_pos + 1
    group = num_heads // num_kv_heads
    out = np.zeros((num_heads, head_dim))
    for h in range(num_heads):
        kvh = h // group
        k = np.asarray(k_cache[:kv_len, kvh * head_dim:(kvh + 1) * head_dim], dtype=np.float64)
        v = np.asarray(v_cache[:kv_len, kvh * head_dim:(kvh + 1) * head_dim], dtype=np.float64)
        score = k @ q[h] / np.sqrt(float(head_dim))
        w = np.exp(score - score.max())
        out[h] = (w[:, None] * v).sum(axis=0) / w.sum()
    return out.reshape(1, num_heads * head_dim)


def cached_attention_online(q, k_cache, v_cache, kv_pos, num_heads, num_kv_heads, head_dim):
    """The shader's own formulation (one running max / sum per head), in f32 like the shader."""
    q = np.asarray(q, dtype=np.float32).reshape(num_heads, head_dim)
    group = num_heads // num_kv_heads
    scale = np.float32(1.0) / np.sqrt(np.float32(head_dim))
    out = np.zeros((num_heads, head_dim), dtype=np.float32)
    for h in range(num_heads):
        kvh = h // group
        acc = np.zeros(head_dim, dtype=np.float32)
        mx, sm = np.float32(-1e30), np.float32(0.0)
        for t in range(kv_pos + 1):
            krow = np.asarray(k_cache[t, kvh * head_dim:(kvh + 1) * head_dim], dtype=np.float32)
            vrow = np.asarray(v_cache[t, kvh * head_dim:(kvh + 1) * head_dim], dtype=np.float32)
            score = np.float32(np.dot(q[h], krow)) * scale
            new_max = max(mx, score)
            corr, wgt = np.exp(mx - new_max, dtype=np.float32), np.exp(score - new_max, dtype=np.float32)
            sm = sm * corr + wgt
            acc = acc * corr + wgt * vrow
            mx = new_max
        out[h] = acc / (sm if sm != 0 else np.float32(1.0))
    return out.reshape(1, num_heads * head_dim)


def swiglu(gate, up):
    gate = np.asarray(gate, dtype=np.float64)
    return gate / (1.0 + np.exp(-gate)) * np.asarray(up, dtype=np.float64)


class DecodeOracle:
    """Whole-model single-token decode on the CPU (f64 between ops), following build_decode_graph.

    `weights`: name -> f32 array for norm weights and the embedding table, and name -> (fmt, packed
    bytes, k, n) for the quantized projections, with the HuggingFace-style names the reference uses.
    """

    def __init__(self, cfg, weights, max_seq):
        self.cfg, self.max_seq = cfg, max_seq
        self.w = {}
        for name, val in weights.items():
            if isinstance(val, tuple):
                fmt, packed, k, n = val
                self.w[name] = O.dequantize_np(fmt, np.asarray(packed), k, n).astype(np.float64)       # [k, n]
            else:
                self.w[name] = np.asarray(val, dtype=np.float64)
        kv_dim = cfg.num_key_value_heads * cfg.head_dim
        self.k_cache = [np.zeros((max_seq, kv_dim)) for _ in range(cfg.num_hidden_layers)]
        self.v_cache = [np.zeros((max_seq, kv_dim)) for _ in range(cfg.num_hidden_layers)]

    def step(self, token, pos):
        c = self.cfg
        x = embedding([token], self.w["model.embed_tokens.weight"]).astype(np.float64)
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}"
            h = rms_norm(x, self.w[f"{p}.input_layernorm.weight"], c.rms_norm_eps)
            q = h @ self.w[f"{p}.self_attn.q_proj.weight"]
            k = h @ self.w[f"{p}.self_attn.k_proj.weight"]
            v = h @ self.w[f"{p}.self_attn.v_proj.weight"]
            q = rope(q, c.rope_theta, pos, c.head_dim)
            k = rope(k, c.rope_theta, pos, c.head_dim)
            cache_write(self.k_cache[i], k, pos)
            cache_write(self.v_cache[i], v, pos)
            attn = cached_attention(q, self.k_cache[i], self.v_cache[i], pos, c.num_attention_heads, c.num_key_value_heads, c.head_dim)
            x = x + attn @ self.w[f"{p}.self_attn.o_proj.weight"]
            h = rms_norm(x, self.w[f"{p}.post_attention_layernorm.weight"], c.rms_norm_eps)
            ffn = swiglu(h @ self.w[f"{p}.mlp.gate_proj.weight"], h @ self.w[f"{p}.mlp.up_proj.weight"])
            x = x + ffn @ self.w[f"{p}.mlp.down_proj.weight"]
        x = rms_norm(x, self.w["model.norm.weight"], c.rms_norm_eps)
        if "lm_head.weight" not in self.w:
            # tied embeddings: logits = x . embed^T (g.matmul_bt(x, embed_weight), src/models/smollm2.rs:413-414)
            return (x @ self.w["model.embed_tokens.weight"].T).reshape(-1)
        return (x @ self.w["lm_head.weight"]).reshape(-1)
