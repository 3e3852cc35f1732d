"""Multi-rank host logic on CPU: two gloo ranks shard the flattened (batch, head) slices,
each evaluates its shard (with the CPU oracle standing in for the kernels -- this test
is about partitioning and the verification gather, not arithmetic), and the gathered
result must equal the unsharded one bitwise.  Also: an uneven split and a rank that
owns nothing."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import swa_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, H, ret):
    # the package's sharding helpers do not need the CUDA library; import the module file directly
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("sharding", os.path.join(root, "dl_templates_b200", "sharding.py"))
    sh = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sh)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        G, d = 6, 16
        q, k, v, _ = orc.seeded_inputs(B, H, G * G, d, d, torch.float32, seed=3)
        win = (1, G, G, 1, 2)
        full = orc.tiled_swa_ref(q, k, v, *win, 0.25).reshape(B * H, G * G, d)
        ql, kl, vl = (sh.shard_bh(t, rank, world) for t in (q, k, v))
        lo, hi = sh.bh_range(B * H, rank, world)
        assert ql.shape[1] == hi - lo
        if hi > lo:
            local = orc.tiled_swa_ref(ql, kl, vl, *win, 0.25)
        else:
            local = torch.zeros(1, 0, G * G, d)
        got = sh.gather_bh(local, B * H)
        ok = torch.equal(got, full)
        flag = torch.tensor([1 if ok else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            ret.put(int(flag.item()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,H,world", [(2, 3, 2), (1, 5, 2), (1, 1, 2)])
@pytest.mark.timeout(120)
def test_sharded_equals_unsharded_over_gloo(B, H, world):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, B, H, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    assert ret.get(timeout=5) == 1
