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
