"""Batch x head sharding across the GPUs of one box.

Every (batch, head) slice of the attention is independent in forward and
backward, so a multi-GPU run gives rank ``r`` of ``P`` a contiguous range of the
flattened ``B*H`` slices and needs no collective on the data path; a gather of
the outputs is used only to verify a sharded run against an unsharded one.
"""
from __future__ import annotations

from typing import Tuple

import torch


def bh_range(n_slices: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous ``[lo, hi)`` of the ``n_slices`` flattened (batch, head) slices owned
    by ``rank``; the first ``n_slices % world`` ranks take one extra slice."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(n_slices, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_bh(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank-local view ``[1, n_local, N, d]`` of ``x [B, H, N, d]`` (B and H flattened)."""
    B, H = x.shape[:2]
    flat = x.reshape(B * H, *x.shape[2:])
    lo, hi = bh_range(B * H, rank, world)
    return flat[lo:hi].unsqueeze(0)


def gather_bh(local: torch.Tensor, n_slices: int, group=None) -> torch.Tensor:
    """All-gather rank-local ``[1, n_local, ...]`` results back into ``[n_slices, ...]``
    (verification only).  Works with unequal shard sizes by padding to the largest."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    sizes = [bh_range(n_slices, r, world) for r in range(world)]
    biggest = max(hi - lo for lo, hi in sizes)
    body = local.squeeze(0)
    pad = torch.zeros((biggest,) + tuple(body.shape[1:]), dtype=body.dtype, device=body.device)
    pad[: body.shape[0]] = body
    out = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(out, pad, group=group)
    return torch.cat([t[: hi - lo] for t, (lo, hi) in zip(out, sizes)], dim=0)
