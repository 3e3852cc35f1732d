"""Generate the golden vectors under tests/golden/ from the reference's own code.

Usage:  python tests/golden/make_golden.py <path-to-reference-checkout>

The script imports, unmodified, the two PyTorch "ref" functions of the reference
(``tiled_swa_ref`` src/tiled_swa.py:693-717 and ``rope2d_ref``
src/fused_rope2d.py:204-225), with the modules they import but do not need on this
path (``natten``, the sibling ``rope2d`` the reference does not ship) replaced by
empty stand-ins, runs them on CPU on seeded inputs, takes gradients with autograd
(as the reference's own scripts do), and stores inputs and outputs as compressed
``.npz``.  The reference checkout is only needed to regenerate; the tests read
the stored files.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(ref_dir):
    for name in ("natten", "natten.na2d"):
        sys.modules[name] = types.ModuleType(name)
    for fn in ("use_fused_na", "use_autotuner", "use_kv_parallelism_in_fused_na"):
        setattr(sys.modules["natten"], fn, lambda *a, **k: None)
    sys.modules["natten.na2d"].na2d = None
    spec = importlib.util.spec_from_file_location("ref_tiled_swa", os.path.join(ref_dir, "src", "tiled_swa.py"))
    swa = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(swa)
    pkg = types.ModuleType("refpkg")
    pkg.__path__ = [os.path.join(ref_dir, "src")]
    sys.modules["refpkg"] = pkg
    stub = types.ModuleType("refpkg.rope2d")
    stub.FusedRotaryPositionEncodingContext = object
    sys.modules["refpkg.rope2d"] = stub
    spec = importlib.util.spec_from_file_location("refpkg.fused_rope2d", os.path.join(ref_dir, "src", "fused_rope2d.py"))
    rope = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rope)
    return swa, rope


def cs_table(n_rdim, max_len, theta):
    inv = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -(torch.arange(n_rdim, dtype=torch.float64) / n_rdim))
    ang = torch.outer(torch.arange(max_len, dtype=torch.float64), inv)
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32)


def swa_case(swa, rope, name, B, H, th, tw, b, row, col, dqk, dv, R, seed, drop=0.0, col_only_drop=False):
    g = torch.Generator().manual_seed(seed)
    N = th * tw * b
    q = torch.randn((B, H, N, dqk), generator=g)
    k = torch.randn((B, H, N, dqk), generator=g)
    v = torch.randn((B, H, N, dv), generator=g)
    do = torch.randn((B, H, N, dv), generator=g)
    sm_scale = dqk ** -0.5
    out = dict(q=q, k=k, v=v, do=do, meta=np.array([B, H, th, tw, b, row, col, dqk, dv, R], dtype=np.int64),
               sm_scale=np.float64(sm_scale))
    q0, k0, v0 = (t.clone().requires_grad_(True) for t in (q, k, v))
    if R > 0:
        # one packed index per token; tokens of a tile share the tile's (row, col)
        rows = torch.arange(th)[:, None, None].expand(th, tw, b)
        cols = torch.arange(tw)[None, :, None].expand(th, tw, b)
        idx = ((rows << 16) | cols).reshape(-1).to(torch.int32)
        if drop > 0:
            dr = torch.bernoulli(torch.full((N,), drop), generator=g).bool()
            idx[dr] = -1
        if col_only_drop:
            # a few tokens keep their row but lose the column half (0xFFFF) and vice versa
            idx[3] = int(idx[3]) | 0xFFFF                  # row kept, column half = -1
            idx[5] = -65536 | (int(idx[5]) & 0xFFFF)       # row half = -1, column kept
        row_cs, col_cs = cs_table(R, th, 10000.0), cs_table(R, tw, 10000.0)
        qr = rope.rope2d_ref(q0.reshape(B * H, N, dqk), idx, row_cs, col_cs).reshape(B, H, N, dqk)
        kr = rope.rope2d_ref(k0.reshape(B * H, N, dqk), idx, row_cs, col_cs).reshape(B, H, N, dqk)
        out.update(idx=idx, row_cs=row_cs, col_cs=col_cs)
    else:
        qr, kr = q0, k0
    o = swa.tiled_swa_ref(qr, kr, v0, b, th, tw, row, col, sm_scale)
    o.backward(do)
    out.update(o=o.detach(), dq=q0.grad, dk=k0.grad, dv=v0.grad)
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        **{k_: (v_.numpy() if isinstance(v_, torch.Tensor) else v_) for k_, v_ in out.items()})
    print(name, "o", tuple(o.shape), "max|o|", float(o.detach().abs().max()))


def rope_selftest_case(rope, name):
    """The layout of the reference's own self-test (src/fused_rope2d.py:230-268): 8x8
    grid + 16 trailing -1 tokens, R=8 of D=64, q taken as a strided view of a
    projection, table 1000^(-2i/R)."""
    g = torch.Generator().manual_seed(1)
    B, N, D, R, C = 8, 80, 64, 8, 128
    bases = torch.pow(1000, -2 * (torch.arange(R) / R))
    ind = torch.arange(0, 8)
    cs = torch.dstack([torch.cos(torch.outer(ind, bases)), torch.sin(torch.outer(ind, bases))])
    x = torch.randn((B, N, C), generator=g)
    idx = torch.bitwise_or(torch.arange(0, 8)[:, None] << 16, torch.arange(0, 8)[None, :]).to(torch.int32).flatten()
    idx = torch.concatenate([idx, torch.full((16,), -1, dtype=torch.int32)], dim=-1)
    w = torch.randn((C, D * 2), generator=g)
    qk = (x @ w).view((B, N, D, 2))
    q = qk[:, :, :, 0]
    y = rope.rope2d_ref(q, idx, cs, cs)
    gy = torch.randn(y.shape, generator=g)
    # gradient w.r.t. q itself (inverse rotation of gy): recompute with q as a leaf
    ql = q.detach().clone().requires_grad_(True)
    rope.rope2d_ref(ql, idx, cs, cs).backward(gy)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), idx=idx.numpy(), row_cs=cs.numpy(), col_cs=cs.numpy(),
                        q=q.detach().numpy(), y=y.detach().numpy(), gy=gy.numpy(), gq=ql.grad.numpy())
    print(name, "y", tuple(y.shape))


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    swa, rope = load_reference(sys.argv[1])
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    # first configuration of the benchmark spec: 16x16 grid, d=32, 7x7 window, fp32, RoPE on all dims
    swa_case(swa, rope, "cfg1_16x16_d32_w7_fp32", 1, 2, 16, 16, 1, 3, 3, 32, 32, 8, seed=0)
    # tiles of 16 tokens, non-square grid, mixed head dims (the regime of the reference's own kernels)
    swa_case(swa, rope, "b16_4x5_dqk16_dv32", 1, 2, 4, 5, 16, 1, 1, 16, 32, 0, seed=2)
    # non-square grid, row != col window, RoPE on the first 16 of 32 dims, 25% tokens without index
    swa_case(swa, rope, "g5x7_r2c1_partial_rope_drop", 2, 1, 5, 7, 1, 2, 1, 32, 16, 4, seed=3, drop=0.25,
             col_only_drop=True)
    # tiles of 2 tokens with RoPE
    swa_case(swa, rope, "b2_6x4_r1c2_rope", 1, 3, 6, 4, 2, 1, 2, 16, 16, 4, seed=4)
    # window larger than the grid (every query sees everything)
    swa_case(swa, rope, "g3x4_window_exceeds_grid", 1, 1, 3, 4, 1, 5, 5, 16, 16, 0, seed=5)
    # tensor-core-sized head dims on a small grid: d_qk=64, d_v=128, 5x5 window, RoPE on 32 dims
    swa_case(swa, rope, "g12x20_dqk64_dv128_w5", 1, 2, 12, 20, 1, 2, 2, 64, 128, 8, seed=6, drop=0.1)
    rope_selftest_case(rope, "rope_selftest_layout")


if __name__ == "__main__":
    main()
