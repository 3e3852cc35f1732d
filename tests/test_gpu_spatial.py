"""Spatial sharding on the GPU kernels, on ONE GPU: the ranks of a row-sharded run are evaluated one after the other
with the halo exchange replaced by slicing from the full tensors (the exchange itself is covered over gloo on CPU,
tests/test_spatial_gloo.py).  What this checks is the numerical claim: a band evaluated on its extended rows with its
neighbours' O and softmax statistic spliced into the halo gives the full grid's O, dQ, dK, dV on the own rows."""
import pytest
import torch

from oracle import swa_oracle as orc
from swa_cases import tolerances

import dl_templates_b200 as swa
from dl_templates_b200 import spatial as sp

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("th,tw,b,rs,cs,world,rope_dims,dtype", [
    (40, 24, 1, 3, 2, 3, 64, torch.bfloat16),      # three bands, RoPE on all dims
    (26, 20, 1, 6, 6, 4, 32, torch.float16),       # bands (6-7 rows) as thin as the reach: halos from two neighbours
    (12, 5, 4, 1, 1, 2, 0, torch.bfloat16),        # tiles of four tokens, no RoPE
])
def test_row_sharded_bands_match_oracle_and_unsharded(th, tw, b, rs, cs, world, rope_dims, dtype):
    B, H, d = 1, 2, 64
    W, N = tw * b, th * tw * b
    q, k, v, do = orc.seeded_inputs(B, H, N, d, d, dtype, seed=11)
    idx = orc.encode_idx(th, W)
    idx[torch.arange(0, N, 7)] = -1
    rope_cpu = None
    if rope_dims:
        rope_cpu = (idx, orc.make_cs_table(rope_dims // 4, th), orc.make_cs_table(rope_dims // 4, W))
    Q, K, V, DO = (t.to(DEV) for t in (q, k, v, do))
    rope = None if rope_cpu is None else tuple(t.to(DEV) for t in rope_cpu)
    sm = d ** -0.5
    shards = [sp.RowShard(th, W, rs, r, world) for r in range(world)]

    # forward of every rank; the halo rows of q, k, v are cut from the full tensors
    outs, saved = [], []
    for s in shards:
        own = s.own_tokens_global()
        def take(ts_, s=s):                      # stands in for the exchange: fills the extended tensors in place
            for t, g in zip(ts_, (Q, K, V)):
                t.copy_(g[:, :, s.ext_tokens_global()])
        o, sv = sp.spatial_forward(s, Q[:, :, own], K[:, :, own], V[:, :, own], rope, b, tw, rs, cs, sm, exchange=take)
        outs.append(o)
        saved.append(sv)
    O = torch.cat(outs, dim=2)
    LSE = torch.cat([sv["lse_ext"][:, :, s.own_tokens()] for s, sv in zip(shards, saved)], dim=2)
    grads = []
    for s, sv in zip(shards, saved):
        def take(ts_, s=s):
            for t, g in zip(ts_, (O, LSE, DO)):
                t.copy_(g[:, :, s.ext_tokens_global()])
        grads.append(sp.spatial_backward(s, sv, DO[:, :, s.own_tokens_global()], exchange=take))
    swa.check_status()
    got = [O] + [torch.cat([g[i] for g in grads], dim=2) for i in range(3)]

    f = lambda t: t.float()
    if rope_cpu is not None:
        want = orc.fused_ref(f(q), f(k), f(v), f(do), *rope_cpu, b, th, tw, rs, cs, sm)
    else:
        want = list(orc.tiled_swa_bwd_ref(f(q), f(k), f(v), f(do), b, th, tw, rs, cs, sm))
    ma, mr = tolerances(dtype)
    for g, w, n in zip(got, want, ("o", "dq", "dk", "dv")):
        a, r = orc.max_abs(g.float().cpu(), w), orc.mean_rel(g.float().cpu(), w)
        assert a < ma and r < mr, f"{n}: max_abs={a:.3e} mean_rel={r:.3e}"

    # ... and against the unsharded run of the same kernels (tile origins differ, so not bitwise)
    if rope is not None:
        o1, l1, qr, kr = swa.swa_forward_rot(Q, K, V, rope, b, th, tw, rs, cs, sm)
        ref = [o1] + list(swa.swa_backward_rot(qr, kr, V, o1, l1, DO, rope, b, th, tw, rs, cs, sm))
    else:
        o1, l1 = swa.swa_forward(Q, K, V, None, b, th, tw, rs, cs, sm)
        ref = [o1] + list(swa.swa_backward(Q, K, V, o1, l1, DO, None, b, th, tw, rs, cs, sm))
    assert (LSE - l1).abs().max().item() < 1e-3
    for g, w, n in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert orc.mean_rel(g.float().cpu(), w.float().cpu()) < mr, n


def _nccl_worker(rank, world, port, ret):
    import os
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        th, tw, b, rs, cs, d = 48, 40, 1, 4, 3, 64
        q, k, v, do = orc.seeded_inputs(1, 3, th * tw, d, d, torch.bfloat16, seed=13)
        idx = orc.encode_idx(th, tw)
        rope = tuple(t.to(dev) for t in (idx, orc.make_cs_table(16, th), orc.make_cs_table(16, tw)))
        Q, K, V, DO = (t.to(dev) for t in (q, k, v, do))
        own = sp.RowShard(th, tw, rs, rank, world).own_tokens_global()
        ql, kl, vl = (t[:, :, own].clone().requires_grad_(True) for t in (Q, K, V))
        o = sp.SpatialTiledSwaRope2D.apply(ql, kl, vl, *rope, b, th, tw, rs, cs, d ** -0.5, None)
        o.backward(DO[:, :, own])
        swa.check_status()
        o1, l1, qr, kr = swa.swa_forward_rot(Q, K, V, rope, b, th, tw, rs, cs, d ** -0.5)
        ref = [o1] + list(swa.swa_backward_rot(qr, kr, V, o1, l1, DO, rope, b, th, tw, rs, cs, d ** -0.5))
        err = max(orc.mean_rel(g.float().cpu(), w[:, :, own].float().cpu())
                  for g, w in zip((o.detach(), ql.grad, kl.grad, vl.grad), ref))
        t = torch.tensor([err], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            ret.put(float(t.item()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_exchange_halos_over_nccl():
    """The autograd surface on two GPUs with the real exchange (NCCL send / receive into local buffers): every
    rank's rows of O, dQ, dK, dV against the unsharded run of the same kernels."""
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_nccl_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:                       # a rank that never came back must not outlive the test
        p.terminate()
        p.join(10)
    assert not alive and all(p.exitcode == 0 for p in procs)
    assert ret.get(timeout=5) < tolerances(torch.bfloat16)[1]
