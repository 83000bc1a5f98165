"""Run under torch.distributed.run on 2+ GPUs (see test_exchange_multigpu.py).

Every rank builds its part of a column-sharded decoder (Graph / build_inference_session with
all_gather nodes bound to symmetric memory) and, on its own GPU, the unsharded model with the same
seeded weights and caches.  Checked on every rank, bit for bit: the logits of teacher-forced steps
(eager and replayed from a CUDA graph), and a free-running greedy sequence picked on the device.
MGQ_CHECK_MODEL=qwen3-8b runs the full-size Qwen3-8B shape instead of the small one.
"""
import os
import sys
from dataclasses import replace

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import numpy as np
    import torch
    import torch.distributed as dist
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from meganeura_b200 import decode_model as M
    if os.environ.get("MGQ_CHECK_MODEL") == "qwen3-8b":
        cfg, max_seq, ctx, steps = M.QWEN3_8B, 1024, 512, 6
    else:
        cfg = replace(M.QWEN3_8B, name="qwen3-like", vocab_size=2048 * world, hidden_size=1024, num_hidden_layers=3,
                      num_attention_heads=8, num_key_value_heads=8, intermediate_size=2048)
        max_seq, ctx, steps = 96, 24, 6
    failures = []
    plain = M.DecodeSession(cfg, max_seq, seed=5, greedy_history=max_seq)
    shard = M.DecodeSession(cfg, max_seq, seed=5, greedy_history=max_seq, rank=rank, world=world)
    for dec in (plain, shard):
        dec.fill_caches(ctx, seed=2)
    dist.barrier()

    # teacher-forced steps: the same token and position on both, logits compared after every step
    rng = np.random.Generator(np.random.PCG64(7))
    tokens = rng.integers(0, cfg.vocab_size, size=steps)
    for i, tok in enumerate(tokens):
        if i == 3:
            shard.session.capture()
        for dec in (plain, shard):
            dec.set_position(int(tok), ctx + i)
            dec.step()
        want, got = plain.logits(), shard.logits()
        try:
            shard.check_exchange()
        except Exception as e:
            failures.append(f"step {i}: {e}")
            break
        if not np.isfinite(want).all():
            failures.append(f"step {i}: the unsharded logits are not finite")
        if not np.array_equal(want, got):
            rel = float(np.linalg.norm(want.astype(np.float64) - got) / max(np.linalg.norm(want.astype(np.float64)), 1e-30))
            failures.append(f"step {i}: sharded logits differ from the unsharded model (rel-L2 {rel:.3e}, expected bit-exact)")
            break

    # free-running greedy decode, the token picked on the device of every rank
    if not failures:
        n = 12
        for dec in (plain, shard):
            dec.set_position(11, ctx + steps)
        for _ in range(n):
            plain.step()
            shard.step()
        plain.session.wait()
        shard.session.wait()
        a = list(plain.session.read_tokens(ctx + steps, n))
        b = list(shard.session.read_tokens(ctx + steps, n))
        try:
            shard.check_exchange()
        except Exception as e:
            failures.append(f"greedy: {e}")
        if a != b:
            failures.append(f"greedy tokens differ: {a} vs {b}")
    dist.barrier()
    torch.cuda.synchronize()
    print(f"rank {rank}: {'OK' if not failures else 'FAIL ' + '; '.join(failures)}", flush=True)
    os._exit(1 if failures else 0)


if __name__ == "__main__":
    main()
