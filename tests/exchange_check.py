"""Run under torch.distributed.run on 2+ GPUs (see test_exchange_multigpu.py).

Checks the column-sharded decode chain on every rank, for the persistent plan kernel (slices stored
into every peer's gathered vector by the kernel), for one launch per GEMV with the fused peer
exchange, and for one launch per GEMV with NCCL all-gathers:
  * every gathered vector equals an NCCL all-gather of the ranks' output slices, bit for bit;
  * the final logits equal the logits of the unsharded chain (same seeds) computed on this rank's
    own GPU: bit for bit for the plan kernel (the summation order depends on K only), within 1e-4
    for the other two (different kernels);
  * eagerly, twice in a row (stamps only grow), and replayed from a CUDA graph.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    layers = int(os.environ.get("MGQ_CHECK_LAYERS", "2"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from meganeura_b200 import decode_chain as dc
    failures = []

    single = dc.DecodeGemvChain(dc.QWEN3_8B, 2, rank=0, world=1, layers=layers, mode="plan")
    single.step()
    torch.cuda.synchronize()
    if single.check_error():
        failures.append("single-GPU plan: a bounded wait ran out")
    want = single.logits_view().reshape(-1).clone()
    single.mode = "launches"
    single.step()
    torch.cuda.synchronize()
    want_launch = single.logits_view().reshape(-1).clone()
    del single

    def check(chain, tag, exact):
        torch.cuda.synchronize()
        if chain.check_error():
            failures.append(f"{tag}: a bounded wait ran out")
            return
        for i, op in enumerate(chain.ops_list):
            g = op["gather_cols"]
            mine = op["y"][0, :g].contiguous()
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            full = op["full"].reshape(-1) if op["full"] is not None else None
            if full is not None and not bool(torch.equal(full.contiguous(), torch.cat(parts))):
                failures.append(f"{tag}: op {i} gathered vector differs from the all-gather of the slices")
                return
        got = chain.logits_view().reshape(-1)
        ref = want if exact else want_launch
        rel = float((got.double() - ref.double()).norm() / ref.double().norm())
        if exact and not bool(torch.equal(got.contiguous(), ref)):
            failures.append(f"{tag}: logits differ from the unsharded chain (rel-L2 {rel:.3e}, expected bit-exact)")
        elif rel > 1e-4:
            failures.append(f"{tag}: logits differ from the unsharded chain by rel-L2 {rel:.3e}")

    for mode, exchange, exact in (("plan", "peer", True), ("launches", "peer", False), ("launches", "nccl", False)):
        chain = dc.DecodeGemvChain(dc.QWEN3_8B, 2, rank=rank, world=world, layers=layers, mode=mode, exchange=exchange)
        tag = f"{mode}/{exchange}"
        chain._launch_all()
        check(chain, tag + " eager 1", exact)
        chain._launch_all()
        check(chain, tag + " eager 2", exact)
        if not failures and exchange == "peer" and chain.capture():
            for _ in range(3):
                chain.step()
            check(chain, tag + " graph replay", exact)
        dist.barrier()
        torch.cuda.synchronize()
        chain.graph = None
        del chain
        if failures:
            break
    # a batch of 8 rows: the 8-row GEMV kernel with the all-gather kernel over peer memory, against the same chain
    # with NCCL all-gathers (bit for bit: same GEMV kernel, different transport) and against the unsharded chain
    if not failures:
        single8 = dc.DecodeGemvChain(dc.QWEN3_8B, 2, batch=8, rank=0, world=1, layers=layers, mode="launches")
        single8.step()
        torch.cuda.synchronize()
        want8 = single8.logits_view().clone()
        del single8
        got = {}
        for exchange in ("peer", "nccl"):
            chain = dc.DecodeGemvChain(dc.QWEN3_8B, 2, batch=8, rank=rank, world=world, layers=layers, mode="launches", exchange=exchange)
            chain._launch_all()
            chain._launch_all()
            if exchange == "peer" and chain.capture():
                chain.step()
                chain.step()
            torch.cuda.synchronize()
            if chain.check_error():
                failures.append(f"batch 8 / {exchange}: a bounded wait ran out")
            got[exchange] = chain.logits_view().clone()
            dist.barrier()
            chain.graph = None
            del chain
        if not failures:
            if not bool(torch.equal(got["peer"], got["nccl"])):
                failures.append("batch 8: the peer all-gather and the NCCL all-gather give different logits")
            rel = float((got["peer"].double() - want8.double()).norm() / want8.double().norm())
            if rel > 1e-4:
                failures.append(f"batch 8: logits differ from the unsharded chain by rel-L2 {rel:.3e}")
    dist.barrier()
    torch.cuda.synchronize()
    print(f"rank {rank}: {'OK' if not failures else 'FAIL ' + '; '.join(failures)}", flush=True)
    os._exit(1 if failures else 0)        # skip communicator teardown (it can stall after graph capture)


if __name__ == "__main__":
    main()
