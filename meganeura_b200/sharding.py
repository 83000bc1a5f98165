"""Column sharding of packed weights across the GPUs of one node, plus the all-gather that
reassembles a sharded GEMV's output.

meganeura itself is single-device (one Session = one device, src/runtime.rs:1513-1531), so this
module has no reference counterpart.  It relies on one property of the reference layout: a
32-element block never spans two columns (block = n*(K/32) + k/32, src/codegen.rs:753, 788), so
any column range of a packed weight is itself a valid packed weight and every rank runs the
unchanged GEMV on its slice.  Rank r of `world` owns columns [r*N/world, (r+1)*N/world) of every
column group; a weight made of several groups (gate|up) is split group by group so that
element-wise combinations of the groups stay local to a rank.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import ops


def shard_range(n: int, rank: int, world: int) -> tuple[int, int]:
    if n % world != 0:
        raise ValueError(f"N={n} is not divisible by world size {world}")
    per = n // world
    return rank * per, (rank + 1) * per


def _group_sizes(n: int, groups) -> list[int]:
    if isinstance(groups, int):
        if n % groups != 0:
            raise ValueError("column groups must be equal")
        return [n // groups] * groups
    sizes = [int(g) for g in groups]
    if sum(sizes) != n:
        raise ValueError("group sizes must add up to N")
    return sizes


def shard_packed(fmt: int, packed: np.ndarray, k: int, n: int, rank: int, world: int, groups=1) -> np.ndarray:
    """This rank's columns of a packed [k, n] host weight, as one self-contained packed weight.

    `groups` is a count of equal column groups or a list of group widths (q|k|v, gate|up): the
    rank takes its slice of each group and the slices are concatenated in group order.
    """
    sizes = _group_sizes(n, groups)
    parts, start = [], 0
    for gn in sizes:
        if gn % world != 0 or (gn // world) % 4 != 0:
            raise ValueError(f"each rank's slice of a group must be a multiple of 4 columns (N={gn}, world={world})")
        n0, n1 = shard_range(gn, rank, world)
        parts.append(ops.shard_columns(fmt, packed, k, n, start + n0, start + n1))
        start += gn
    if len(parts) == 1:
        return parts[0]
    return concat_columns(fmt, parts, k)


def concat_columns(fmt: int, parts, k: int) -> np.ndarray:
    """Concatenate packed weights that share K along the column axis (host arrays)."""
    from ._lib import FMT_Q8
    if fmt == FMT_Q8:
        return np.concatenate(parts)
    bpc = k // 32
    hdrs, nibs = [], []
    for p in parts:
        nb = p.size // 20
        assert nb % bpc == 0
        hdrs.append(p[: nb * 4])
        nibs.append(p[nb * 4:])
    return np.concatenate(hdrs + nibs)


@dataclass
class GatherPlan:
    """Where each rank's slice lands in the gathered [m, n] output (row-major)."""
    n: int
    world: int
    groups: object = 1          # count of equal groups, or a list of group widths

    def sizes(self) -> list[int]:
        return _group_sizes(self.n, self.groups)

    def columns(self, rank: int) -> np.ndarray:
        out, start = [], 0
        for gn in self.sizes():
            n0, n1 = shard_range(gn, rank, self.world)
            out.append(np.arange(start + n0, start + n1))
            start += gn
        return np.concatenate(out)


def all_gather_columns(local, plan: GatherPlan, group=None, out=None):
    """All-gather of a [m, n/world] slice into the full [m, n] tensor on every rank.

    `local` is a torch tensor (CUDA with the nccl backend, CPU with gloo).  For m == 1 and a
    single column group the gathered buffer is already in column order; otherwise the slices are
    scattered to their columns.
    """
    import torch
    import torch.distributed as dist
    world = plan.world
    m = local.shape[0]
    per = local.shape[1]
    if world == 1:
        return local
    flat = torch.empty((world, m, per), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat.view(-1), local.contiguous().view(-1), group=group)
    sizes = plan.sizes()
    if len(sizes) == 1:
        res = flat.permute(1, 0, 2).reshape(m, plan.n)
    else:
        pieces, off = [], 0
        for gn in sizes:                                  # slice of group g from every rank, in rank order
            w = gn // world
            pieces.append(flat[:, :, off:off + w].permute(1, 0, 2).reshape(m, gn))
            off += w
        res = torch.cat(pieces, dim=1)
    if out is not None:
        out.copy_(res)
        return out
    return res.contiguous()
