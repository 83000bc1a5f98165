"""Host-side sharding logic, including a world_size-2 gloo run on CPU.

The per-shard GEMV is computed by the oracle here (the product has no CPU kernels); what is
under test is the product's shard bookkeeping and the all-gather reassembly."""
import os
import socket

import numpy as np
import pytest

from meganeura_b200 import decode_chain as dc, ops, sharding, synth
from oracle import oracle as O


def test_synth_matches_oracle_generator():
    for fmt in (O.FMT_Q4, O.FMT_Q8):
        assert (synth.synth_weights(fmt, 96, 12, 5) == O.synth_weights(fmt, 96, 12, 5)).all()
        base, n0, reps = synth.synth_weights_tiled(fmt, 128, 4096, 1)
        full = synth.tile_columns(fmt, base, 128, n0, reps)
        assert n0 * reps == 4096 and full.size == ops.packed_bytes(fmt, 128, 4096)
        d = O.dequantize_np(fmt, full, 128, 4096)
        assert (d[:, 3 * n0:4 * n0] == O.dequantize_np(fmt, base, 128, n0)).all()


@pytest.mark.parametrize("fmt", [O.FMT_Q4, O.FMT_Q8])
@pytest.mark.parametrize("groups", [1, 2, (32, 16, 16)])
def test_shard_packed_selects_the_planned_columns(fmt, groups):
    k, n, world = 64, 64, 4
    w = synth.synth_weights(fmt, k, n, 3)
    dq = O.dequantize_np(fmt, w, k, n)
    plan = sharding.GatherPlan(n, world, groups)
    seen = []
    for r in range(world):
        sh = sharding.shard_packed(fmt, w, k, n, r, world, groups=groups)
        cols = plan.columns(r)
        assert (O.dequantize_np(fmt, sh, k, n // world) == dq[:, cols]).all()
        seen.append(cols)
    assert sorted(np.concatenate(seen).tolist()) == list(range(n))


def test_shard_errors():
    w = synth.synth_weights(O.FMT_Q4, 64, 24, 3)
    with pytest.raises(ValueError):
        sharding.shard_packed(O.FMT_Q4, w, 64, 24, 0, 4)          # 6 columns per rank: not a multiple of 4
    with pytest.raises(ValueError):
        sharding.shard_range(10, 0, 4)


def test_workload_byte_counts():
    # per-token packed weight bytes of the Qwen3-8B-shaped model in Q4: 36 * 120 586 240 + 388 956 160
    total = 0
    for sp in dc.layer_specs(dc.QWEN3_8B):
        total += 36 * ops.packed_bytes(O.FMT_Q4, sp.k, sp.n)
    total += ops.packed_bytes(O.FMT_Q4, 4096, 151936)
    assert total == 4730060800
    one = dc.step_bytes(dc.QWEN3_8B, O.FMT_Q4, 1, 1)
    assert total < one < total * 1.01
    assert abs(dc.step_bytes(dc.QWEN3_8B, O.FMT_Q4, 1, 8) * 8 - one) < one * 0.02


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, fmt, groups, m, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        k, n = 128, 64
        w = synth.synth_weights(fmt, k, n, 9)
        x = np.random.Generator(np.random.PCG64(4)).standard_normal((m, k)).astype(np.float32)
        co = O.COracle()
        shard = sharding.shard_packed(fmt, w, k, n, rank, world, groups=groups)
        local = co.matmul(fmt, x, shard, k, n // world, wide=False)
        full = sharding.all_gather_columns(torch.from_numpy(local), sharding.GatherPlan(n, world, groups))
        want = co.matmul(fmt, x, w, k, n, wide=False)
        q.put((rank, bool((full.numpy() == want).all())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("groups,m", [(1, 1), (2, 1), (1, 3), (2, 2), ((32, 16, 16), 2)])
def test_all_gather_reassembles_columns_gloo(groups, m):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, O.FMT_Q4, groups, m, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, True), (1, True)]


def test_sharded_decode_graph_builds_for_every_rank():
    """Host side of the column-sharded session: every rank's graph builds with the sliced shapes, the
    all_gather / slice_columns builders check their arguments, and a model whose heads or widths do
    not divide over the ranks is refused before anything is built."""
    from dataclasses import replace
    import meganeura_b200 as mg
    from meganeura_b200 import decode_model as M
    cfg = replace(M.QWEN3_8B, name="t", vocab_size=4096, hidden_size=512, num_hidden_layers=2,
                  num_attention_heads=4, num_key_value_heads=2, intermediate_size=1024)
    for world in (1, 2):
        for rank in range(world):
            g = mg.Graph()
            logits, k_caches, v_caches = M.build_decode_graph(g, cfg, 64, rank, world)
            g.set_outputs([logits])
            assert len(k_caches) == len(v_caches) == 2
    with pytest.raises(ValueError, match="KV heads"):
        M.build_decode_graph(mg.Graph(), cfg, 64, 0, 4)
    with pytest.raises(ValueError, match="multiple of 4"):
        M.build_decode_graph(mg.Graph(), replace(cfg, vocab_size=4100), 64, 0, 2)
    g = mg.Graph()
    x = g.input("x", [1, 64])
    assert g.all_gather(x, 2) >= 0 and g.slice_columns(x, 32, 32) >= 0
    for bad in (lambda: g.all_gather(x, 0), lambda: g.all_gather(x, 9), lambda: g.slice_columns(x, 48, 32),
                lambda: g.slice_columns(x, 2, 8), lambda: g.all_gather(g.input("m", [2, 64]), 2)):
        with pytest.raises(Exception):
            bad()


def _sharded_decode_worker(rank, world, port, q):
    """One rank of the column-sharded decoder in numpy: its column range of every projection, its heads'
    caches, and the five kinds of all-gather of decode_model.build_decode_graph, over gloo."""
    from dataclasses import replace
    import torch
    import torch.distributed as dist
    from oracle import decode_oracle as D
    from meganeura_b200 import decode_model as M
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = replace(M.QWEN3_8B, name="t", vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=64, intermediate_size=512)
        max_seq = 16
        rng = np.random.Generator(np.random.PCG64(21))
        weights = {"model.embed_tokens.weight": rng.standard_normal((cfg.vocab_size, cfg.hidden_size)).astype(np.float32)}
        for name in M.norm_weights(cfg):
            weights[name] = (1.0 + 0.1 * rng.standard_normal(cfg.hidden_size)).astype(np.float32)
        dense = {}
        for name, fmt, k, n in M.quantized_weights(cfg):
            w = (rng.standard_normal((k, n)) * (1.5 / np.sqrt(k))).astype(np.float32)
            packed = O.quantize_q4_np(w) if fmt == O.FMT_Q4 else O.quantize_q8_np(w)
            weights[name] = (fmt, packed, k, n)
            dense[name] = O.dequantize_np(fmt, packed, k, n).astype(np.float64)
        whole = D.DecodeOracle(cfg, weights, max_seq)

        def gather(local):                                   # rank-major concatenation, like the all_gather node
            parts = [torch.empty_like(torch.from_numpy(local)) for _ in range(world)]
            dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(local)))
            return np.concatenate([p.numpy() for p in parts], axis=-1)

        def mine(w):                                         # this rank's column range of a [k, n] weight
            per = w.shape[1] // world
            return w[:, rank * per:(rank + 1) * per]

        heads, kv_heads = cfg.num_attention_heads // world, cfg.num_key_value_heads // world
        kv_loc, hid_loc = cfg.kv_dim // world, cfg.hidden_size // world
        k_cache = [np.zeros((max_seq, kv_loc)) for _ in range(cfg.num_hidden_layers)]
        v_cache = [np.zeros((max_seq, kv_loc)) for _ in range(cfg.num_hidden_layers)]
        ok = True
        for pos, tok in enumerate([3, 200, 77]):
            x = D.embedding([tok], weights["model.embed_tokens.weight"]).astype(np.float64)
            for i in range(cfg.num_hidden_layers):
                p = f"model.layers.{i}"
                h = D.rms_norm(x, weights[f"{p}.input_layernorm.weight"].astype(np.float64), cfg.rms_norm_eps)
                qv = D.rope(h @ mine(dense[f"{p}.self_attn.q_proj.weight"]), cfg.rope_theta, pos, cfg.head_dim)
                kv = D.rope(h @ mine(dense[f"{p}.self_attn.k_proj.weight"]), cfg.rope_theta, pos, cfg.head_dim)
                vv = h @ mine(dense[f"{p}.self_attn.v_proj.weight"])
                D.cache_write(k_cache[i], kv, pos)
                D.cache_write(v_cache[i], vv, pos)
                attn = gather(D.cached_attention(qv, k_cache[i], v_cache[i], pos, heads, kv_heads, cfg.head_dim))
                x_mine = x[:, rank * hid_loc:(rank + 1) * hid_loc]
                x = gather(x_mine + attn @ mine(dense[f"{p}.self_attn.o_proj.weight"]))
                h = D.rms_norm(x, weights[f"{p}.post_attention_layernorm.weight"].astype(np.float64), cfg.rms_norm_eps)
                ffn = gather(D.swiglu(h @ mine(dense[f"{p}.mlp.gate_proj.weight"]), h @ mine(dense[f"{p}.mlp.up_proj.weight"])))
                x_mine = x[:, rank * hid_loc:(rank + 1) * hid_loc]
                x = gather(x_mine + ffn @ mine(dense[f"{p}.mlp.down_proj.weight"]))
            x = D.rms_norm(x, weights["model.norm.weight"].astype(np.float64), cfg.rms_norm_eps)
            logits = gather(x @ mine(dense["lm_head.weight"])).reshape(-1)
            want = whole.step(tok, pos)
            ok = ok and float(np.abs(logits - want).max()) <= 1e-9 * max(1.0, float(np.abs(want).max()))
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_sharded_decode_math_matches_the_whole_model_gloo():
    """The sharding of decode_model.build_decode_graph (heads per rank, column ranges, rank-major gathers)
    written out with the CPU oracle's operators on two gloo ranks reproduces the unsharded oracle."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sharded_decode_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, True), (1, True)]
