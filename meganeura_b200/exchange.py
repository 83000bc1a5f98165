"""Peer-memory exchange for column-sharded GEMVs (the fused all-gather of mgq_gemv_exchange).

One symmetric allocation per rank (torch.distributed._symmetric_memory: same layout on every
rank, every rank can address every other rank's copy over NVLink) holds the token index, the
error word and, for each exchanging op, the gathered vector as 8-byte {value, stamp} elements:

    [ epoch u64 ][ error u32 ][ blocks_done u32 ] ... pad to 256 ... [ gathered vectors ... ]

No TMA multicast and no multimem are involved: producers use plain 64-bit stores into the
consumer GPU's own memory; consumers only read local memory.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from ._lib import check, lib


class PeerExchange:
    def __init__(self, gather_sizes, rank: int, world: int, group=None):
        """gather_sizes[i]: floats each rank contributes to op i's gathered vector (0: op does not exchange)."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        if world > 8:
            raise ValueError("at most 8 ranks")
        self.rank, self.world = rank, world
        self.n_ops = len(gather_sizes)
        self.gather_sizes = list(gather_sizes)
        self.off_epoch, self.off_error, self.off_blocks = 0, 8, 12
        off = 256
        self.off_gather = []
        for g in self.gather_sizes:
            self.off_gather.append(off)
            off += (8 * g * world + 255) // 256 * 256
        self.nbytes = off
        grp = group if group is not None else dist.group.WORLD
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm_mem.rendezvous(self.buf, grp)
        self.buf.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.local = self.ptrs[rank]
        descs = (_lib.ExchangePush * self.n_ops)()             # push descriptors, in ordinary device memory
        for i, g in enumerate(self.gather_sizes):
            d = descs[i]
            d.world, d.rank, d.gather_cols = world, rank, g
            for p in range(world):
                d.dst[p] = self.ptrs[p] + self.off_gather[i]
        raw = np.frombuffer(bytes(descs), dtype=np.uint8).copy()
        self.desc_dev = torch.from_numpy(raw).cuda()
        self.desc_size = ctypes.sizeof(_lib.ExchangePush)

    def push_ptr(self, op: int):
        return self.desc_dev.data_ptr() + op * self.desc_size if self.gather_sizes[op] else None

    def vec_ptr(self, op: int) -> int:
        return self.local + self.off_gather[op]

    def vec_len(self, op: int) -> int:
        return self.gather_sizes[op] * self.world

    @property
    def epoch_ptr(self) -> int:
        return self.local + self.off_epoch

    @property
    def error_ptr(self) -> int:
        return self.local + self.off_error

    def gathered(self, op: int):
        """This rank's copy of op's gathered values as a float32 tensor [world * gather] (strided view)."""
        import torch
        n = self.vec_len(op)
        pairs = self.buf[self.off_gather[op]: self.off_gather[op] + 8 * n].view(torch.float32).view(n, 2)
        return pairs[:, 0]

    def gemv(self, fmt, x, w, addend, y, k, n, op: int, wait_op, stream_ptr):
        wait_ptr = None
        if wait_op is not None:
            if self.vec_len(wait_op) != k:
                raise ValueError(f"op {op} consumes a gathered vector of {self.vec_len(wait_op)} elements but K={k}")
            wait_ptr = self.vec_ptr(wait_op)
        check(lib.mgq_gemv_exchange(fmt, x.data_ptr() if x is not None else None, w.data_ptr(),
                                    addend.data_ptr() if addend is not None else None,
                                    y.data_ptr(), k, n, self.push_ptr(op), wait_ptr,
                                    self.epoch_ptr, self.error_ptr, stream_ptr))

    def all_gather_rows(self, op: int, slice_t, rows: int, cols: int, out_t, stream_ptr):
        """Stores this rank's [rows, cols] slice (a view with any row stride) into every rank's gathered vector of
        `op`, waits for the whole vector and writes the row-major [rows, world * cols] matrix to out_t."""
        if rows * cols != self.gather_sizes[op]:
            raise ValueError(f"op {op} gathers {self.gather_sizes[op]} values per rank, got {rows}x{cols}")
        check(lib.mgq_exchange_all_gather_rows(slice_t.data_ptr(), slice_t.stride(0), rows, cols, self.world, self.push_ptr(op),
                                               self.vec_ptr(op), out_t.data_ptr(), self.epoch_ptr, self.error_ptr, stream_ptr))

    def finish(self, last_op, stream_ptr):
        last = self.vec_ptr(last_op) if last_op is not None else None
        length = self.vec_len(last_op) if last_op is not None else 0
        check(lib.mgq_exchange_finish(last, length, self.epoch_ptr, self.error_ptr, self.local + self.off_blocks, stream_ptr))

    def error(self) -> int:
        import torch
        torch.cuda.synchronize()
        return int(self.buf[self.off_error: self.off_error + 4].view(torch.int32).item())


class LocalExchange:
    """The same layout in ordinary device memory for a single rank (world 1): every all_gather then
    stores into and reads from this GPU's own vectors.  Exercises the exchange path without peers."""

    def __init__(self, gather_sizes):
        import torch
        self.rank, self.world = 0, 1
        self.gather_sizes = list(gather_sizes)
        self.n_ops = len(self.gather_sizes)
        self.off_epoch, self.off_error, self.off_blocks = 0, 8, 12
        off = 256
        self.off_gather = []
        for g in self.gather_sizes:
            self.off_gather.append(off)
            off += (8 * g + 255) // 256 * 256
        self.buf = torch.zeros(off, dtype=torch.uint8, device="cuda")
        self.local = self.buf.data_ptr()
        descs = (_lib.ExchangePush * self.n_ops)()
        for i, g in enumerate(self.gather_sizes):
            descs[i].world, descs[i].rank, descs[i].gather_cols = 1, 0, g
            descs[i].dst[0] = self.local + self.off_gather[i]
        self.desc_dev = torch.from_numpy(np.frombuffer(bytes(descs), dtype=np.uint8).copy()).cuda()
        self.desc_size = ctypes.sizeof(_lib.ExchangePush)
        torch.cuda.synchronize()

    def push_ptr(self, op: int):
        return self.desc_dev.data_ptr() + op * self.desc_size

    def vec_ptr(self, op: int) -> int:
        return self.local + self.off_gather[op]

    @property
    def epoch_ptr(self) -> int:
        return self.local + self.off_epoch

    @property
    def error_ptr(self) -> int:
        return self.local + self.off_error
