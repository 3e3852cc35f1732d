"""Spatial sharding on CPU: gloo ranks own bands of grid rows, exchange halo rows point to point and run a CPU
stand-in for the kernels on their extended bands; the own rows of O, dQ, dK, dV must equal the oracle's full-grid
result.  This is about the partition, the halo index arithmetic and the exchange (including halos that span more
than one neighbour and ranks at the grid border), not about kernel arithmetic: the stand-in keeps the kernels'
contract -- backward takes the softmax statistic and O as inputs instead of recomputing them."""
import importlib.util
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import swa_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _spatial():
    # the module needs no CUDA library; load the file directly instead of importing the package
    spec = importlib.util.spec_from_file_location("spatial", os.path.join(ROOT, "dl_templates_b200", "spatial.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def cpu_kernels():
    """(fwd, bwd) with the call contract of the CUDA entries: fwd returns (o, lse, q_rot, k_rot); bwd takes the
    rotated q / k, O and lse of every row of the band and returns gradients of the un-rotated q, k and of v."""
    def fwd(q, k, v, rope, win, sm):
        qr, kr = (q, k) if rope is None else (orc.rope2d_ref(q, *rope), orc.rope2d_ref(k, *rope))
        s = torch.einsum("bhnd,bhmd->bhnm", qr, kr) * sm + orc.window_mask(*win)
        lse = torch.logsumexp(s, dim=-1)
        return torch.exp(s - lse[..., None]) @ v, lse, qr, kr

    def bwd(qr, kr, v, o, lse, do, rope, win, sm):
        s = torch.einsum("bhnd,bhmd->bhnm", qr, kr) * sm + orc.window_mask(*win)
        p = torch.exp(s - lse[..., None])
        delta = (o * do).sum(-1, keepdim=True)
        dv = p.transpose(-1, -2) @ do
        ds = p * (do @ v.transpose(-1, -2) - delta)
        dq, dk = ds @ kr * sm, ds.transpose(-1, -2) @ qr * sm
        if rope is not None:
            dq, dk = orc.rope2d_ref(dq, *rope, inverse=True), orc.rope2d_ref(dk, *rope, inverse=True)
        return dq, dk, dv

    return fwd, bwd


def _worker(rank, world, port, case, ret):
    sp = _spatial()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b, th, tw, rs, cs, with_rope = case
        B, H, d = 1, 2, 8
        N, W = th * tw * b, tw * b
        q, k, v, do = (t.double() for t in orc.seeded_inputs(B, H, N, d, d, torch.float32, seed=5))
        idx = orc.encode_idx(th, W)
        idx[3] = -1
        tab_r, tab_c = orc.make_cs_table(d // 4, th).double(), orc.make_cs_table(d // 4, W).double()
        rope = (idx, tab_r, tab_c) if with_rope else None
        if with_rope:
            want = orc.fused_ref(q, k, v, do, idx, tab_r, tab_c, b, th, tw, rs, cs, 0.3)
        else:
            want = list(orc.tiled_swa_bwd_ref(q, k, v, do, b, th, tw, rs, cs, 0.3))      # o, dq, dk, dv
        shard = sp.RowShard(th, W, rs, rank, world)
        own = shard.own_tokens_global()
        o, saved = sp.spatial_forward(shard, q[:, :, own], k[:, :, own], v[:, :, own], rope, b, tw, rs, cs, 0.3,
                                      kernels=cpu_kernels())
        dq, dk, dv = sp.spatial_backward(shard, saved, do[:, :, own], kernels=cpu_kernels())
        err = max((g - w[:, :, own]).abs().max().item() for g, w in zip((o, dq, dk, dv), want))
        # the same through the autograd surface
        sp.SpatialTiledSwaRope2D.kernels = cpu_kernels()
        ql, kl, vl = (t[:, :, own].clone().requires_grad_(True) for t in (q, k, v))
        ropes = rope if rope is not None else (None, None, None)
        o2 = sp.SpatialTiledSwaRope2D.apply(ql, kl, vl, *ropes, b, th, tw, rs, cs, 0.3, None)
        o2.backward(do[:, :, own])
        err = max([err] + [(g - w[:, :, own]).abs().max().item() for g, w in zip((o2.detach(), ql.grad, kl.grad, vl.grad), want)])
        flag = torch.tensor([err])
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if rank == 0:
            ret.put(float(flag.item()))
    finally:
        dist.destroy_process_group()


# (b_size, t_height, t_width, row_size, col_size, RoPE): bands thinner than the reach (halo from two neighbours),
# uneven split, tiles of several tokens, no RoPE
CASES = [((1, 8, 5, 2, 1, True), 2), ((1, 7, 4, 3, 2, True), 3), ((2, 6, 3, 1, 1, True), 2), ((1, 9, 4, 2, 2, False), 4)]


@pytest.mark.parametrize("case,world", CASES)
@pytest.mark.timeout(180)
def test_row_sharded_equals_full_grid_over_gloo(case, world):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(150)
        assert p.exitcode == 0
    assert ret.get(timeout=5) < 1e-9


def test_partition_and_halo_lists():
    sp = _spatial()
    for th, world, rs in ((8, 2, 2), (7, 3, 3), (16, 4, 1), (5, 5, 2), (128, 8, 6)):
        shards = [sp.RowShard(th, 3, rs, r, world) for r in range(world)]
        assert shards[0].r0 == 0 and shards[-1].r1 == th
        for a, b in zip(shards, shards[1:]):
            assert a.r1 == b.r0
        for s in shards:
            assert s.e0 == max(0, s.r0 - rs) and s.e1 == min(th, s.r1 + rs)
            got = sorted(r for _, a, b in s.recvs for r in range(a, b))
            assert got == [r for r in range(s.e0, s.e1) if not (s.r0 <= r < s.r1)]
            # what one rank expects to receive from a peer is exactly what that peer lists to send to it
            for peer, a, b in s.recvs:
                assert (s.rank, a, b) in shards[peer].sends
            assert sum(len(x.recvs) for x in shards) == sum(len(x.sends) for x in shards)
    with pytest.raises(ValueError):
        sp.RowShard(3, 3, 1, 3, 4)
