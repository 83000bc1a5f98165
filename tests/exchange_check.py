"""Run under torch.distributed.run on 2+ GPUs (see test_exchange_multigpu.py): checks that the fused
peer exchange leaves, on every rank, the gathered vectors an NCCL all-gather of the ranks' output
slices gives -- eagerly and when the token is replayed from a CUDA graph."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from meganeura_b200 import decode_chain as dc
    chain = dc.DecodeGemvChain(dc.QWEN3_8B, 2, rank=rank, world=world, layers=2, exchange="peer")
    failures = []

    def check(tag):
        torch.cuda.synchronize()
        if chain.peer.error():
            failures.append(f"{tag}: a bounded wait ran out")
            return
        for i, op in enumerate(chain.ops_list):
            g = op["gather_cols"]
            if not g:
                continue
            mine = op["y"][0, :g].contiguous()
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            if not bool((chain.peer.gathered(i) == torch.cat(parts)).all()):
                failures.append(f"{tag}: op {i} gathered vector differs")
                return

    chain._launch_all()
    check("eager 1")
    chain._launch_all()
    check("eager 2")
    if not failures and chain.capture():
        for _ in range(3):
            chain.step()
        check("graph replay")
    # a GEMV that consumes the gathered vector itself (x = None): op A pushes its whole slice, op B reads it
    if not failures:
        from meganeura_b200 import ops, synth
        from meganeura_b200.exchange import PeerExchange
        k0, na, nb = 1024, 4096, 512                      # A: k0 -> na (sharded), B: na -> nb (sharded)
        pe = PeerExchange([na // world, 0], rank, world)
        wa = torch.from_numpy(synth.synth_weights(2, k0, na // world, seed=100 + rank)).cuda()
        wb = torch.from_numpy(synth.synth_weights(3, na, nb // world, seed=200 + rank)).cuda()
        x0 = torch.randn((1, k0), generator=torch.Generator().manual_seed(7)).cuda()
        ya = torch.zeros((1, na // world), device="cuda")
        yb = torch.zeros((1, nb // world), device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        for token in range(2):
            pe.gemv(2, x0, wa, None, ya, k0, na // world, 0, None, stream)
            pe.gemv(3, None, wb, None, yb, na, nb // world, 1, 0, stream)
            pe.finish(0, stream)
            torch.cuda.synchronize()
            if pe.error():
                failures.append("consume: a bounded wait ran out")
                break
            full = pe.gathered(0).contiguous().view(1, na)
            want = ops.matmul(3, full, wb, na, nb // world, route="gemv")
            torch.cuda.synchronize()
            if not bool((yb == want).all()):
                failures.append(f"consume token {token}: result differs from a GEMV over the gathered values")
                break
            x0 = x0 * 1.5
    dist.barrier()
    torch.cuda.synchronize()
    chain.graph = None
    print(f"rank {rank}: {'OK' if not failures else 'FAIL ' + '; '.join(failures)}", flush=True)
    os._exit(1 if failures else 0)        # skip communicator teardown (it can stall after graph capture)


if __name__ == "__main__":
    main()
