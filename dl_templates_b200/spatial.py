"""Spatial sharding: the rows of the token grid split across the GPUs of one box, with halo exchange.

The reference has no counterpart; batch x head sharding (``sharding.py``) needs no communication and is what
multi-GPU runs normally use.  Splitting the grid itself is for a single (batch, head) problem too large or too
latency-bound for one GPU.  Rank ``r`` owns a contiguous band of grid rows ``[r0, r1)`` (all token columns, all
batches and heads).  A query row interacts with the ``row_size`` tile rows either side of it
(src/tiled_swa.py:701-713: the window is truncated at the grid border, never shifted), so:

* forward and dQ of the own rows need K and V of the rows ``[r0 - row_size, r1 + row_size)``;
* dK and dV of the own rows need Q, dO, the softmax statistic and delta of the same extended band.

Every rank therefore runs the unmodified kernels on its EXTENDED band (own rows plus halo rows, with the tokens'
own packed RoPE indices, so the angles are those of the full grid) and keeps the own rows of the results.  What
the kernels compute for the halo rows themselves is discarded: their windows are cut at the edge of the band.  For
the backward pass the halo rows of O and of the softmax statistic -- wrong locally for that reason -- are replaced
by their owners' values before the kernels run, which makes every (query, key) pair inside the band exact.

Halo rows travel with point-to-point send / receive (NCCL on GPUs, gloo in the CPU tests) INTO LOCAL BUFFERS; the
kernels never see a peer's memory.  Per step and rank: 2 x row_size rows of q, k, v (forward), of o, the statistic
and dO (backward).  Halo rows cost compute as well: (r1 - r0 + 2 row_size) / (r1 - r0) of the own work.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch


def row_range(t_height: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous ``[r0, r1)`` of the ``t_height`` grid rows owned by ``rank``; the first
    ``t_height % world`` ranks take one extra row."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(t_height, world)
    r0 = rank * base + min(rank, extra)
    return r0, r0 + base + (1 if rank < extra else 0)


class RowShard:
    """Geometry of one rank's band.  ``W`` = tokens per grid row (``t_width * b_size``).

    ``recvs`` / ``sends``: lists of ``(peer, a, b)`` -- grid rows ``[a, b)`` of the extended band that ``peer`` owns,
    resp. own rows that lie in ``peer``'s extended band -- ordered by peer; a halo may span several peers when
    bands are thinner than ``row_size``."""

    def __init__(self, t_height: int, W: int, row_size: int, rank: int, world: int):
        self.t_height, self.W, self.row_size, self.rank, self.world = t_height, W, row_size, rank, world
        self.r0, self.r1 = row_range(t_height, rank, world)
        if self.r1 <= self.r0:
            raise ValueError("more ranks than grid rows")
        self.e0, self.e1 = max(0, self.r0 - row_size), min(t_height, self.r1 + row_size)
        self.recvs: List[Tuple[int, int, int]] = []
        self.sends: List[Tuple[int, int, int]] = []
        for peer in range(world):
            if peer == rank:
                continue
            p0, p1 = row_range(t_height, peer, world)
            a, b = max(self.e0, p0), min(self.e1, p1)
            if a < b:
                self.recvs.append((peer, a, b))
            q0, q1 = max(0, p0 - row_size), min(t_height, p1 + row_size)
            a, b = max(self.r0, q0), min(self.r1, q1)
            if a < b:
                self.sends.append((peer, a, b))

    @property
    def rows_own(self) -> int:
        return self.r1 - self.r0

    @property
    def rows_ext(self) -> int:
        return self.e1 - self.e0

    def own_tokens(self) -> slice:
        """Token range of the own rows inside a tensor of the extended band."""
        return slice((self.r0 - self.e0) * self.W, (self.r1 - self.e0) * self.W)

    def ext_tokens_global(self) -> slice:
        """Token range of the extended band inside a tensor of the full grid."""
        return slice(self.e0 * self.W, self.e1 * self.W)

    def own_tokens_global(self) -> slice:
        return slice(self.r0 * self.W, self.r1 * self.W)


def embed_rows(shard: RowShard, own: torch.Tensor) -> torch.Tensor:
    """A tensor of the extended band ``[B, H, rows_ext * W, ...]`` with ``own`` (``[B, H, rows_own * W, ...]``) copied into
    its own rows; the halo rows are uninitialised.  Callers that build their inputs inside such a tensor in the
    first place (``ext_inputs=True`` below) save this copy."""
    ext = torch.empty(own.shape[:2] + (shard.rows_ext * shard.W,) + own.shape[3:], dtype=own.dtype, device=own.device)
    ext[:, :, shard.own_tokens()] = own
    return ext


def exchange_halo(shard: RowShard, ext_tensors: Sequence[torch.Tensor], group=None) -> None:
    """Fill the halo rows of tensors of the extended band (``[B, H, rows_ext * W, ...]``, own rows valid) IN PLACE with
    their owners' rows, and serve the peers' halos from the own rows.  One batch of point-to-point operations for
    all tensors; rows are packed into and received in local staging buffers (a row range of a ``[B, H, N, ...]``
    tensor is not contiguous), so only halo-sized copies are made."""
    import torch.distributed as dist

    W = shard.W
    ops, landing = [], []
    for ti, t in enumerate(ext_tensors):
        for peer, a, b in shard.sends:
            buf = t[:, :, (a - shard.e0) * W:(b - shard.e0) * W].contiguous()
            ops.append(dist.P2POp(dist.isend, buf, peer, group=group))
        for peer, a, b in shard.recvs:
            buf = torch.empty(t.shape[:2] + ((b - a) * W,) + t.shape[3:], dtype=t.dtype, device=t.device)
            ops.append(dist.P2POp(dist.irecv, buf, peer, group=group))
            landing.append((ti, a, b, buf))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    for ti, a, b, buf in landing:
        ext_tensors[ti][:, :, (a - shard.e0) * W:(b - shard.e0) * W] = buf


def _default_kernels():
    from . import tiled_swa as ts

    def fwd(q, k, v, rope, win, sm_scale):
        if rope is None:
            o, lse = ts.swa_forward(q, k, v, None, *win, sm_scale)
            return o, lse, q, k
        return ts.swa_forward_rot(q, k, v, rope, *win, sm_scale)

    def bwd(q_in, k_in, v, o, lse, do, rope, win, sm_scale):
        if rope is None:
            return ts.swa_backward(q_in, k_in, v, o, lse, do, None, *win, sm_scale)
        return ts.swa_backward_rot(q_in, k_in, v, o, lse, do, rope, *win, sm_scale)

    return fwd, bwd


def spatial_forward(shard: RowShard, q, k, v, rope, b_size: int, t_width: int, row_size: int, col_size: int,
                    sm_scale: float, group=None, exchange: Optional[Callable] = None, kernels=None,
                    ext_inputs: bool = False):
    """Forward of this rank's band.  ``q, k, v``: own rows ``[B, H, rows_own * W, d]``, or -- ``ext_inputs`` --
    tensors of the extended band whose own rows are filled (their halo rows are then written in place, and no
    band-sized copy is made).  ``rope``: ``None`` or ``(idx, row_cs, col_cs)`` with ``idx`` of the FULL grid.
    ``exchange(list of extended tensors)`` fills halo rows in place (default: :func:`exchange_halo` over
    ``group``).  Returns ``(o_own, saved)``; ``saved`` goes to :func:`spatial_backward`."""
    if shard.W != t_width * b_size or shard.row_size != row_size:
        raise ValueError("shard geometry does not match the call")
    exchange = exchange or (lambda ts_: exchange_halo(shard, ts_, group))
    fwd, _ = kernels or _default_kernels()
    q_ext, k_ext, v_ext = (q, k, v) if ext_inputs else (embed_rows(shard, t) for t in (q, k, v))
    exchange([q_ext, k_ext, v_ext])
    rope_ext = None if rope is None else (rope[0][shard.ext_tokens_global()].contiguous(), rope[1], rope[2])
    win = (b_size, shard.rows_ext, t_width, row_size, col_size)
    o_ext, lse_ext, q_in, k_in = fwd(q_ext, k_ext, v_ext, rope_ext, win, sm_scale)
    saved = dict(q_in=q_in, k_in=k_in, v_ext=v_ext, o_ext=o_ext, lse_ext=lse_ext, rope_ext=rope_ext, win=win,
                 sm_scale=sm_scale)
    return o_ext[:, :, shard.own_tokens()], saved


def spatial_backward(shard: RowShard, saved: dict, do, group=None, exchange: Optional[Callable] = None,
                     kernels=None, ext_inputs: bool = False):
    """Backward of this rank's band: ``do`` = own rows of dO (or, ``ext_inputs``, a tensor of the extended band with
    its own rows filled).  Returns ``dq, dk, dv`` of the own rows (views of band-sized tensors).  The halo rows of
    the saved O and softmax statistic are overwritten in place with their owners' values."""
    exchange = exchange or (lambda ts_: exchange_halo(shard, ts_, group))
    _, bwd = kernels or _default_kernels()
    do_ext = do if ext_inputs else embed_rows(shard, do)
    # halo rows of O and of the softmax statistic come from their owners (locally their windows were cut)
    exchange([saved["o_ext"], saved["lse_ext"], do_ext])
    dq, dk, dv = bwd(saved["q_in"], saved["k_in"], saved["v_ext"], saved["o_ext"], saved["lse_ext"], do_ext,
                     saved["rope_ext"], saved["win"], saved["sm_scale"])
    own = shard.own_tokens()
    return dq[:, :, own], dk[:, :, own], dv[:, :, own]


class SpatialTiledSwaRope2D(torch.autograd.Function):
    """``o_own = SpatialTiledSwaRope2D.apply(q, k, v, idx, row_cs, col_cs, b_size, t_height, t_width, row_size,
    col_size, sm_scale, group)`` -- the argument order of ``TiledSwaRope2D`` plus the process group; ``q, k, v`` hold
    this rank's rows of the grid (``row_range(t_height, rank, world)``), ``t_height`` and ``idx`` are those of the
    full grid.  ``idx`` may be ``None`` (no RoPE)."""

    kernels = None      # (forward, backward) callables standing in for the CUDA entries; the CPU tests set it

    @staticmethod
    def forward(ctx, q, k, v, idx, row_cs, col_cs, b_size, t_height, t_width, row_size, col_size, sm_scale,
                group=None):
        import torch.distributed as dist

        shard = RowShard(t_height, t_width * b_size, row_size, dist.get_rank(group), dist.get_world_size(group))
        rope = None if idx is None else (idx, row_cs, col_cs)
        o, saved = spatial_forward(shard, q, k, v, rope, b_size, t_width, row_size, col_size, sm_scale, group,
                                   kernels=SpatialTiledSwaRope2D.kernels)
        rope_ext = saved["rope_ext"] or ()
        ctx.save_for_backward(saved["q_in"], saved["k_in"], saved["v_ext"], saved["o_ext"], saved["lse_ext"], *rope_ext)
        ctx.shard, ctx.group, ctx.win, ctx.sm_scale = shard, group, saved["win"], saved["sm_scale"]
        return o.contiguous()

    @staticmethod
    def backward(ctx, do):
        q_in, k_in, v_ext, o_ext, lse_ext, *rope_ext = ctx.saved_tensors
        saved = dict(q_in=q_in, k_in=k_in, v_ext=v_ext, o_ext=o_ext, lse_ext=lse_ext,
                     rope_ext=tuple(rope_ext) if rope_ext else None, win=ctx.win, sm_scale=ctx.sm_scale)
        dq, dk, dv = spatial_backward(ctx.shard, saved, do, ctx.group, kernels=SpatialTiledSwaRope2D.kernels)
        return (dq.contiguous(), dk.contiguous(), dv.contiguous()) + (None,) * 10
