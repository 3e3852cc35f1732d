"""Named problem sizes: the five configurations of the benchmark specification and
the headline target (128x128 grid, d=64, 13x13 window, bf16, forward + backward).

``rope_dims`` = how many leading q/k dims are rotated (4 * n_rdim); ``drop`` = fraction
of tokens whose packed index is -1 (no RoPE); all use one token per grid cell.
"""
import torch

CONFIGS = {
    "cfg1": dict(B=1, H=2, grid=16, d_qk=32, d_v=32, w=7, dtype=torch.float32, rope_dims=32, drop=0.0, bwd=True),
    "cfg2": dict(B=4, H=8, grid=64, d_qk=64, d_v=64, w=13, dtype=torch.bfloat16, rope_dims=64, drop=0.0, bwd=False),
    "cfg3": dict(B=8, H=12, grid=56, d_qk=64, d_v=64, w=7, dtype=torch.float16, rope_dims=64, drop=0.1, bwd=True),
    "cfg4": dict(B=4, H=8, grid=128, d_qk=64, d_v=128, w=15, dtype=torch.bfloat16, rope_dims=32, drop=0.0, bwd=True),
    "cfg5": dict(B=16, H=16, grid=256, d_qk=128, d_v=128, w=31, dtype=torch.bfloat16, rope_dims=128, drop=0.0,
                 bwd=True),
    "target": dict(B=16, H=16, grid=128, d_qk=64, d_v=64, w=13, dtype=torch.bfloat16, rope_dims=64, drop=0.0,
                   bwd=True),
}


def windowed_flops(bh: int, tokens: int, b_size: int, row_size: int, col_size: int, d_qk: int, d_v: int):
    """(forward, backward) FLOPs: forward ``2*N*w^2*(d_qk+d_v)`` per (batch, head),
    backward 2.5x that; truncation of the window at the grid border is ignored."""
    w2 = (2 * row_size + 1) * (2 * col_size + 1) * b_size
    fwd = 2.0 * bh * tokens * w2 * (d_qk + d_v)
    return fwd, 2.5 * fwd
