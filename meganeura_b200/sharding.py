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


def shard_packed(fmt: int, packed: np.ndarray, k: int, n: int, rank: int, world: int, groups: int = 1) -> np.ndarray:
    """This rank's columns of a packed [k, n] host weight, as one self-contained packed weight.

    With groups > 1 the weight is a concatenation of `groups` equal column groups; the rank takes
    its slice of each group and the slices are concatenated in group order.
    """
    if n % groups != 0:
        raise ValueError("column groups must be equal")
    gn = n // groups
    if (gn // world) % 4 != 0 or gn % world != 0:
        raise ValueError(f"each rank's slice of a group must be a multiple of 4 columns (N={gn}, world={world})")
    parts = []
    for g in range(groups):
        n0, n1 = shard_range(gn, rank, world)
        parts.append(ops.shard_columns(fmt, packed, k, n, g * gn + n0, g * gn + n1))
    if groups == 1:
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
    groups: int = 1

    def columns(self, rank: int) -> np.ndarray:
        gn = self.n // self.groups
        out = []
        for g in range(self.groups):
            n0, n1 = shard_range(gn, rank, self.world)
            out.append(np.arange(g * gn + n0, g * gn + n1))
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
    if plan.groups == 1:
        res = flat.permute(1, 0, 2).reshape(m, plan.n)
    else:
        gper = per // plan.groups
        res = flat.view(world, m, plan.groups, gper).permute(1, 2, 0, 3).reshape(m, plan.n)
    if out is not None:
        out.copy_(res)
        return out
    return res.contiguous()
