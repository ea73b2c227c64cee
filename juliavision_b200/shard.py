"""Sharding layer: independent units (images, sequences, GEMM token rows) are split into
contiguous ranges across the GPUs of one box; weights are replicated; nothing is exchanged
while computing.  The optional final gather of output shards goes through torch.distributed
(NCCL over NVLink on GPUs, gloo in CPU tests).  New surface — the reference is single-device.
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

from . import _lib
from ._lib import check


def shard_range(total: int, world: int, rank: int, align: int = 1) -> Tuple[int, int]:
    """[begin, end) of `total` units owned by `rank`; split points are multiples of `align`."""
    b, e = C.c_int64(), C.c_int64()
    check(_lib.lib().b200_shard_range(total, world, rank, align, C.byref(b), C.byref(e)))
    return b.value, e.value


def shard_range_py(total: int, world: int, rank: int, align: int = 1) -> Tuple[int, int]:
    """The same arithmetic without the library (host-side planning before any GPU exists)."""
    if not (world > 0 and 0 <= rank < world and total >= 0 and align > 0):
        raise ValueError("shard_range: bad argument")
    units = (total + align - 1) // align
    per, rem = divmod(units, world)
    ub = per * rank + min(rank, rem)
    ue = ub + per + (1 if rank < rem else 0)
    return min(ub * align, total), min(ue * align, total)


def gather_shards(local, total: int, world: int, align: int = 1, group=None):
    """All-gather variable-length shards along axis 0 into the full array on every rank.

    `local` is a torch tensor holding this rank's [begin,end) rows.  Uses
    torch.distributed.all_gather on equal-sized padded buffers, then trims.
    """
    import torch
    import torch.distributed as dist

    sizes = [shard_range_py(total, world, r, align) for r in range(world)]
    maxn = max(e - b for b, e in sizes)
    pad = torch.zeros((maxn,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    bufs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(bufs, pad, group=group)
    return torch.cat([bufs[r][: e - b] for r, (b, e) in enumerate(sizes)], dim=0)
