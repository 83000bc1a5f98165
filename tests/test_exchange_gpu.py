"""mgq_gemv_exchange on ONE GPU: a rank whose only peer is itself.

The push, stamp and poll code is the code the multi-GPU path runs (tests/test_exchange_multigpu.py
covers 2 ranks); here the gathered vector lives in ordinary device memory, so no second GPU and no
symmetric-memory rendezvous is needed.  Results must equal the plain mgq_gemv bit for bit.
"""
import ctypes

import numpy as np
import pytest

from oracle import oracle as O
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


class _SelfExchange:
    """[epoch u64][error u32][blocks_done u32] pad to 256, then one {value, stamp} vector per op."""

    def __init__(self, lengths):
        import torch
        from meganeura_b200 import _lib
        self.offsets, off = [], 256
        for n in lengths:
            self.offsets.append(off)
            off += (8 * n + 255) // 256 * 256
        self.buf = torch.zeros(off, dtype=torch.uint8, device="cuda")
        self.lengths = lengths
        descs = (_lib.ExchangePush * len(lengths))()
        for i, n in enumerate(lengths):
            descs[i].world, descs[i].rank, descs[i].gather_cols = 1, 0, n
            descs[i].dst[0] = self.buf.data_ptr() + self.offsets[i]
        self.descs = torch.from_numpy(np.frombuffer(bytes(descs), dtype=np.uint8).copy()).cuda()
        self.desc_size = ctypes.sizeof(_lib.ExchangePush)

    def push(self, i):
        return self.descs.data_ptr() + i * self.desc_size

    def vec(self, i):
        return self.buf.data_ptr() + self.offsets[i]

    epoch = property(lambda self: self.buf.data_ptr())
    error = property(lambda self: self.buf.data_ptr() + 8)
    blocks = property(lambda self: self.buf.data_ptr() + 12)

    def values(self, i):
        import torch
        n = self.lengths[i]
        return self.buf[self.offsets[i]: self.offsets[i] + 8 * n].view(torch.float32).view(n, 2)[:, 0]

    def stamps(self, i):
        import torch
        n = self.lengths[i]
        return self.buf[self.offsets[i]: self.offsets[i] + 8 * n].view(torch.int32).view(n, 2)[:, 1]

    def error_word(self):
        import torch
        torch.cuda.synchronize()
        return int(self.buf[8:12].view(torch.int32).item())

    def epoch_value(self):
        import torch
        torch.cuda.synchronize()
        return int(self.buf[0:8].view(torch.int64).item())


@pytest.mark.parametrize("fmt", [O.FMT_Q4, O.FMT_Q8])
@pytest.mark.parametrize("dims", [(1024, 2048, 1536), (576, 1536, 576), (4096, 3072, 4096), (4096, 512, 768), (12288, 512, 18992)])
def test_chained_gemvs_through_gathered_vectors(fmt, dims):
    """op0 pushes its output; op1 waits for it and takes its activations from the gathered vector;
    op1's own output is pushed too and closes the step.  Two steps in a row: stamps only grow."""
    import torch
    from meganeura_b200 import ops
    from meganeura_b200._lib import check, lib
    k0, n0, n1 = dims
    rng = np.random.Generator(np.random.PCG64(11))
    w0 = to_dev(O.synth_weights(fmt, k0, n0, seed=3))
    w1 = to_dev(O.synth_weights(fmt, n0, n1, seed=4))
    addend = to_dev(rng.standard_normal((1, n1)).astype(np.float32))
    ex = _SelfExchange([n0, n1])
    stream = torch.cuda.current_stream().cuda_stream
    for step in range(2):
        x = to_dev(rng.standard_normal((1, k0)).astype(np.float32))
        want0 = ops.matmul(fmt, x, w0, k0, n0)
        want1 = ops.matmul(fmt, want0, w1, n0, n1, addend=addend)
        y0 = torch.zeros((1, n0), dtype=torch.float32, device="cuda")
        y1 = torch.zeros((1, n1), dtype=torch.float32, device="cuda")
        check(lib.mgq_gemv_exchange(fmt, x.data_ptr(), w0.data_ptr(), None, y0.data_ptr(), k0, n0,
                                    ex.push(0), None, ex.epoch, ex.error, stream))
        check(lib.mgq_gemv_exchange(fmt, None, w1.data_ptr(), addend.data_ptr(), y1.data_ptr(), n0, n1,
                                    ex.push(1), ex.vec(0), ex.epoch, ex.error, stream))
        check(lib.mgq_exchange_finish(ex.vec(1), n1, ex.epoch, ex.error, ex.blocks, stream))
        assert ex.error_word() == 0
        assert ex.epoch_value() == step + 1
        assert torch.equal(y0, want0) and torch.equal(y1, want1)
        assert torch.equal(ex.values(0), want0[0]) and torch.equal(ex.values(1), want1[0])
        assert bool((ex.stamps(0) == step + 1).all()) and bool((ex.stamps(1) == step + 1).all())


def test_wait_that_nothing_satisfies_times_out_cleanly():
    """A consumer whose producer never ran: the bounded poll gives up, raises the error word and the
    kernel returns; the context stays usable and the next correct step works."""
    import torch
    from meganeura_b200 import ops
    from meganeura_b200._lib import check, lib
    fmt, k, n = O.FMT_Q4, 1024, 64
    w = to_dev(O.synth_weights(fmt, k, n, seed=9))
    ex = _SelfExchange([k])
    y = torch.zeros((1, n), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    ops.set_option("gemv.wait_us", 1000)                       # the default allows for peers that launch seconds apart
    try:
        check(lib.mgq_gemv_exchange(fmt, None, w.data_ptr(), None, y.data_ptr(), k, n,
                                    None, ex.vec(0), ex.epoch, ex.error, stream))
        assert ex.error_word() == 1                            # synchronises: the kernel has returned
    finally:
        ops.set_option("gemv.wait_us", 0)
    ex.buf[8:12].zero_()
    x = to_dev(np.ones((1, k), dtype=np.float32))
    want = ops.matmul(fmt, x, w, k, n)
    torch.cuda.synchronize()
    assert torch.isfinite(want).all()


def test_all_gather_rows_two_ranks_emulated_on_one_gpu():
    """mgq_exchange_all_gather_rows with both ranks' gathered vectors on this GPU: rank 0 stores only,
    then rank 1 stores and waits (nothing waits for a later launch).  Both vectors must hold the slices
    rank-major, and the unpacked matrix must be the row-major [rows, world * cols] whole; then a second
    token (stamps grow), and a wait for a slice that nobody stores, which must end in the error word."""
    import torch
    from meganeura_b200 import _lib, ops
    from meganeura_b200._lib import check, lib
    rows, cols, pitch, world = 8, 96, 160, 2
    total = world * rows * cols
    buf = torch.zeros(256 + 2 * 8 * total + 512, dtype=torch.uint8, device="cuda")
    vec = [buf.data_ptr() + 256, buf.data_ptr() + 256 + 8 * total + 256]
    descs = (_lib.ExchangePush * world)()
    for r in range(world):
        descs[r].world, descs[r].rank, descs[r].gather_cols = world, r, rows * cols
        for q in range(world):
            descs[r].dst[q] = vec[q]
    dev_descs = torch.from_numpy(np.frombuffer(bytes(descs), dtype=np.uint8).copy()).cuda()
    push = [dev_descs.data_ptr() + r * ctypes.sizeof(_lib.ExchangePush) for r in range(world)]
    epoch, error, blocks = buf.data_ptr(), buf.data_ptr() + 8, buf.data_ptr() + 12
    stream = torch.cuda.current_stream().cuda_stream
    rng = torch.Generator(device="cpu").manual_seed(3)
    for token in range(2):
        slices = [torch.randn((rows, pitch), generator=rng).cuda() for _ in range(world)]
        out = torch.full((rows, world * cols), -1.0, device="cuda")
        check(lib.mgq_exchange_all_gather_rows(slices[0].data_ptr(), pitch, rows, cols, world, push[0], vec[0], None, epoch, error, stream))
        check(lib.mgq_exchange_all_gather_rows(slices[1].data_ptr(), pitch, rows, cols, world, push[1], vec[1], out.data_ptr(),
                                               epoch, error, stream))
        check(lib.mgq_exchange_finish(None, 0, epoch, error, blocks, stream))
        torch.cuda.synchronize()
        want = torch.cat([s[:, :cols] for s in slices], dim=1)
        assert torch.equal(out, want)
        for q in range(world):                                   # both ranks' vectors hold the same gathered data
            off = vec[q] - buf.data_ptr()
            pairs = buf[off: off + 8 * total].view(torch.float32).view(world, rows, cols, 2)
            assert torch.equal(pairs[..., 0], torch.stack([s[:, :cols] for s in slices]))
            assert bool((buf[off: off + 8 * total].view(torch.int32).view(-1, 2)[:, 1] == token + 1).all())
        assert int(buf[8:12].view(torch.int32).item()) == 0
    # third token: rank 0 never stores; rank 1's wait must give up and say so
    ops.set_option("gemv.wait_us", 2000)
    try:
        out = torch.zeros((rows, world * cols), device="cuda")
        check(lib.mgq_exchange_all_gather_rows(slices[1].data_ptr(), pitch, rows, cols, world, push[1], vec[1], out.data_ptr(),
                                               epoch, error, stream))
        torch.cuda.synchronize()
        assert int(buf[8:12].view(torch.int32).item()) == 1
    finally:
        ops.set_option("gemv.wait_us", 0)
    with pytest.raises(Exception):
        check(lib.mgq_exchange_all_gather_rows(slices[1].data_ptr(), cols - 1, rows, cols, world, push[1], vec[1], out.data_ptr(),
                                               epoch, error, stream))
