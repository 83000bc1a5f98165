"""Single-token decode graphs of the two model shapes the benchmarks name, built through the
Graph mirror exactly like meganeura builds them (src/models/smollm2.rs:315-421 build_decode_graph;
examples/qwen3.rs:243-310 uses the same layer without q/k-norm), with the projections declared as
quantized parameters.

    token_ids, kv_pos (u32 inputs) -> embedding -> N x [rms_norm, q/k/v matmul, rope(q), rope(k),
    cache_write(k), cache_write(v), cached_attention, o matmul + residual, rms_norm, gate/up matmul,
    swiglu, down matmul + residual] -> rms_norm -> lm_head matmul

The session fuses o/down with their residual adds, q|k|v and gate|up into single GEMVs.

With world > 1 the same builder makes ONE RANK'S part of the column-sharded model (no reference
counterpart, the reference is single-device): every projection holds this rank's column range,
attention works on this rank's query heads and their KV heads, and four all_gathers per layer
(attention output, hidden state after o, SwiGLU output, hidden state after down) plus one for the
logits put the slices together over peer memory.  Columns never share a quantization block, each
head is local to one rank and the gathers are rank-major, so every rank computes, bit for bit, the
logits of the unsharded model.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np

from . import synth
from ._lib import FMT_Q4, FMT_Q8
from .graph import Graph, Session, build_inference_session


@dataclass(frozen=True)
class DecoderConfig:
    name: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    attn_fmt: int
    mlp_fmt: int
    head_fmt: int
    tie_word_embeddings: bool = False       # lm_head = embed_tokens^T through matmul_bt (src/models/smollm2.rs:29-30, 413-414)

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim


# src/models/smollm2.rs:35-47; MLP Q4, attention and an untied lm_head Q8
SMOLLM2_135M = DecoderConfig("smollm2-135m", 49152, 576, 30, 9, 3, 64, 1536, 1e-5, 1e4, FMT_Q8, FMT_Q4, FMT_Q8)
# examples/qwen3.rs:91-105 (8B variant); every projection and the lm_head Q4
QWEN3_8B = DecoderConfig("qwen3-8b", 151936, 4096, 36, 32, 8, 128, 12288, 1e-6, 1e6, FMT_Q4, FMT_Q4, FMT_Q4)


def small(cfg: DecoderConfig, layers: int, vocab: int) -> DecoderConfig:
    """The same layer shape with fewer layers and a smaller vocabulary (for tests)."""
    return replace(cfg, name=f"{cfg.name}-{layers}l", num_hidden_layers=layers, vocab_size=vocab)


def _qparam(g: Graph, fmt: int, name: str, shape):
    return g.parameter_q4(name, shape) if fmt == FMT_Q4 else g.parameter_q8(name, shape)


def check_world(cfg: DecoderConfig, world: int) -> None:
    for what, n in (("KV heads", cfg.num_key_value_heads), ("query heads", cfg.num_attention_heads)):
        if n % world != 0:
            raise ValueError(f"{n} {what} do not divide over {world} ranks")
    for what, n in (("hidden size", cfg.hidden_size), ("intermediate size", cfg.intermediate_size), ("vocabulary", cfg.vocab_size)):
        if n % (4 * world) != 0:
            raise ValueError(f"{what} {n}: each rank's slice must be a multiple of 4 columns ({world} ranks)")


def build_decode_graph(g: Graph, cfg: DecoderConfig, max_seq_len: int, rank: int = 0, world: int = 1, gather_always: bool = False):
    """Returns (logits, k_cache_params, v_cache_params), like the reference's build_decode_graph.
    world > 1: this rank's part of the column-sharded model (gather_always builds the same graph,
    all_gathers included, for a single rank)."""
    check_world(cfg, world)
    sharded = world > 1 or gather_always
    hidden, ffn = cfg.hidden_size, cfg.intermediate_size
    q_loc, kv_loc, ffn_loc, hid_loc, vocab_loc = (cfg.q_dim // world, cfg.kv_dim // world, ffn // world, hidden // world,
                                                  cfg.vocab_size // world)
    heads_loc, kv_heads_loc = cfg.num_attention_heads // world, cfg.num_key_value_heads // world

    def gather(x):
        return g.all_gather(x, world) if sharded else x

    def mine(x):                     # this rank's columns of a whole hidden-state vector
        return g.slice_columns(x, rank * hid_loc, hid_loc) if sharded else x

    token_ids = g.input_u32("token_ids", [1])
    kv_pos = g.input_u32("kv_pos", [1])
    embed = g.parameter("model.embed_tokens.weight", [cfg.vocab_size, hidden])
    x = g.embedding(token_ids, embed)
    k_caches, v_caches = [], []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        h = g.rms_norm(x, g.parameter(f"{p}.input_layernorm.weight", [hidden]), cfg.rms_norm_eps)
        wq = _qparam(g, cfg.attn_fmt, f"{p}.self_attn.q_proj.weight", [hidden, q_loc])
        wk = _qparam(g, cfg.attn_fmt, f"{p}.self_attn.k_proj.weight", [hidden, kv_loc])
        wv = _qparam(g, cfg.attn_fmt, f"{p}.self_attn.v_proj.weight", [hidden, kv_loc])
        q, k, v = g.matmul(h, wq), g.matmul(h, wk), g.matmul(h, wv)
        q = g.rope_dynamic_offset(q, cfg.rope_theta, kv_pos, cfg.head_dim)
        k = g.rope_dynamic_offset(k, cfg.rope_theta, kv_pos, cfg.head_dim)
        k_cache = g.parameter(f"kv_cache.layer.{i}.k", [max_seq_len, kv_loc])
        v_cache = g.parameter(f"kv_cache.layer.{i}.v", [max_seq_len, kv_loc])
        k_caches.append(k_cache)
        v_caches.append(v_cache)
        g.cache_write(k, k_cache, kv_pos)
        g.cache_write(v, v_cache, kv_pos)
        attn = gather(g.cached_attention(q, k_cache, v_cache, kv_pos, heads_loc, kv_heads_loc, cfg.head_dim))
        wo = _qparam(g, cfg.attn_fmt, f"{p}.self_attn.o_proj.weight", [cfg.q_dim, hid_loc])
        x = gather(g.add(mine(x), g.matmul(attn, wo)))
        h = g.rms_norm(x, g.parameter(f"{p}.post_attention_layernorm.weight", [hidden]), cfg.rms_norm_eps)
        w_gate = _qparam(g, cfg.mlp_fmt, f"{p}.mlp.gate_proj.weight", [hidden, ffn_loc])
        w_up = _qparam(g, cfg.mlp_fmt, f"{p}.mlp.up_proj.weight", [hidden, ffn_loc])
        w_down = _qparam(g, cfg.mlp_fmt, f"{p}.mlp.down_proj.weight", [ffn, hid_loc])
        ffn_out = gather(g.swiglu(g.matmul(h, w_gate), g.matmul(h, w_up)))
        x = gather(g.add(mine(x), g.matmul(ffn_out, w_down)))
    x = g.rms_norm(x, g.parameter("model.norm.weight", [hidden]), cfg.rms_norm_eps)
    if cfg.tie_word_embeddings:
        if sharded:
            raise ValueError("tied embeddings are not column-sharded (the table is indexed by rows)")
        logits = g.matmul_bt(x, embed)
    else:
        logits = gather(g.matmul(x, _qparam(g, cfg.head_fmt, "lm_head.weight", [hidden, vocab_loc])))
    return logits, k_caches, v_caches


def quantized_weights(cfg: DecoderConfig):
    """(name, fmt, k, n) of every quantized projection, in graph order."""
    out = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        out += [(f"{p}.self_attn.q_proj.weight", cfg.attn_fmt, cfg.hidden_size, cfg.q_dim),
                (f"{p}.self_attn.k_proj.weight", cfg.attn_fmt, cfg.hidden_size, cfg.kv_dim),
                (f"{p}.self_attn.v_proj.weight", cfg.attn_fmt, cfg.hidden_size, cfg.kv_dim),
                (f"{p}.self_attn.o_proj.weight", cfg.attn_fmt, cfg.q_dim, cfg.hidden_size),
                (f"{p}.mlp.gate_proj.weight", cfg.mlp_fmt, cfg.hidden_size, cfg.intermediate_size),
                (f"{p}.mlp.up_proj.weight", cfg.mlp_fmt, cfg.hidden_size, cfg.intermediate_size),
                (f"{p}.mlp.down_proj.weight", cfg.mlp_fmt, cfg.intermediate_size, cfg.hidden_size)]
    if not cfg.tie_word_embeddings:
        out.append(("lm_head.weight", cfg.head_fmt, cfg.hidden_size, cfg.vocab_size))
    return out


def norm_weights(cfg: DecoderConfig):
    names = []
    for i in range(cfg.num_hidden_layers):
        names += [f"model.layers.{i}.input_layernorm.weight", f"model.layers.{i}.post_attention_layernorm.weight"]
    return names + ["model.norm.weight"]


def packed_weight_bytes(cfg: DecoderConfig) -> int:
    from .ops import packed_bytes
    return sum(packed_bytes(fmt, k, n) for _, fmt, k, n in quantized_weights(cfg))


class DecodeSession:
    """A decode session with the weights the benchmark configurations describe for whole-model
    decode: seeded f32 matrices ~ N(0, 0.02^2) run through the reference's quantizer, a different
    seed for every tensor of every layer, norm weights 1, a seeded N(0,1) embedding table.  A
    projection of N columns is the periodic extension of a quantized base of `base_cols` columns
    (the lm_head of an eighth of the vocabulary), so the 30 GB of f32 an 8B-parameter model would
    need are never materialised and start-up stays in seconds."""

    def __init__(self, cfg: DecoderConfig, max_seq_len: int, seed: int = 0, greedy_history: int = 0, base_cols: int = 256,
                 rank: int = 0, world: int = 1, group=None, gather_always: bool = False):
        """world > 1 (under torch.distributed, one process per GPU): this rank's part of the sharded
        model, holding its column range of the very same weights, with the all_gathers bound to a
        symmetric-memory PeerExchange.  gather_always: the sharded graph for a single rank."""
        from . import ops
        self.cfg, self.max_seq_len, self.rank, self.world = cfg, max_seq_len, rank, world
        g = Graph()
        logits, self.k_caches, self.v_caches = build_decode_graph(g, cfg, max_seq_len, rank, world, gather_always)
        g.set_outputs([logits])
        self.session: Session = build_inference_session(g)
        s = self.session
        self.exchange = None
        slices = s.exchange_slices()
        if slices:
            if world > 1:
                from .exchange import PeerExchange
                self.exchange = PeerExchange(slices, rank, world, group)
            else:
                from .exchange import LocalExchange
                self.exchange = LocalExchange(slices)
            s.bind_exchanges(self.exchange)
        rng = np.random.Generator(np.random.PCG64(seed))
        table = rng.standard_normal((cfg.vocab_size, cfg.hidden_size), dtype=np.float32)
        s.set_parameter("model.embed_tokens.weight", table)
        ones = np.ones(cfg.hidden_size, dtype=np.float32)
        for name in norm_weights(cfg):
            s.set_parameter(name, ones)
        for idx, (name, fmt, k, n) in enumerate(quantized_weights(cfg)):
            cols = n
            if name == "lm_head.weight":
                while cols > 8192 and cols % 2 == 0 and (cols // 2) % 4 == 0:
                    cols //= 2
            else:
                while cols > base_cols and cols % 2 == 0 and (cols // 2) % 4 == 0:
                    cols //= 2
            wrng = np.random.Generator(np.random.PCG64(seed * 1000003 + 17 * idx + 1))
            w = wrng.standard_normal((k, cols), dtype=np.float32) * np.float32(0.02)
            packed = synth.tile_columns(fmt, ops.quantize(fmt, w), k, cols, n // cols)
            if world > 1:
                per = n // world
                packed = ops.shard_columns(fmt, packed, k, n, rank * per, (rank + 1) * per)
            s.upload_param(name, packed)
        if greedy_history:
            s.enable_greedy(0, "token_ids", "kv_pos", greedy_history)

    def fill_caches(self, upto: int, seed: int = 1, scale: float = 0.1) -> None:
        """Pretend `upto` tokens were already decoded: cache rows [0, upto) get N(0,1)*scale (a sharded
        rank keeps the columns of its own KV heads of the same rows)."""
        rng = np.random.Generator(np.random.PCG64(seed))
        kv_loc = self.cfg.kv_dim // self.world
        for i in range(self.cfg.num_hidden_layers):
            for kind in ("k", "v"):
                rows = np.zeros((self.max_seq_len, self.cfg.kv_dim), dtype=np.float32)
                rows[:upto] = rng.standard_normal((upto, self.cfg.kv_dim), dtype=np.float32) * scale
                mine = np.ascontiguousarray(rows[:, self.rank * kv_loc:(self.rank + 1) * kv_loc])
                self.session.set_parameter(f"kv_cache.layer.{i}.{kind}", mine)

    def set_position(self, token: int, pos: int) -> None:
        self.session.set_input_u32("token_ids", [token])
        self.session.set_input_u32("kv_pos", [pos])

    def step(self) -> None:
        self.session.step()

    def logits(self) -> np.ndarray:
        self.session.wait()
        return self.session.read_output(self.cfg.vocab_size)

    def check_exchange(self) -> None:
        """Raises if a wait for another rank ran out in an earlier step (sharded sessions)."""
        self.session.check_exchange()
