"""CPU oracle for the fused-RoPE 2D sliding-window attention path.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain PyTorch-on-CPU tensor
arithmetic, the algorithm of the reference project's two PyTorch "ref" functions

  * ``tiled_swa_ref``  -- src/tiled_swa.py:693-717 (dense [N,N] additive mask + softmax attention)
  * ``rope2d_ref``     -- src/fused_rope2d.py:204-225 (half-split 2D rotary embedding, -1 = identity)

so that the CUDA kernels of ``dl_templates_b200`` can be checked against it.  It is
imported only by the tests, by ``__graft_entry__.smoke()`` and by the CPU-baseline
leg of ``bench.py``; the product package never imports it and has no CPU fallback.

Pinning: ``tests/golden/make_golden.py`` runs the *reference's own* functions
(imported unmodified from the reference checkout) on seeded inputs and stores
their outputs; ``tests/test_oracle.py`` checks every function below against those
stored outputs.  The one unpinned item is the cos/sin *table formula*: the
reference imports it from a file it does not ship (src/fused_rope2d.py:8), so
``make_cs_table`` is this build's definition; kernels and oracle consume the same
table, so the choice cannot influence parity.

The softmax attention of the reference is ``torch.nn.functional.
scaled_dot_product_attention`` (src/tiled_swa.py:715) of the installed PyTorch; the
restatement spells it out as scores -> +mask -> softmax -> @v so that the forward
and the backward formulas are visible, and ``tiled_swa_ref_sdpa`` keeps the literal
SDPA form (the one timed as the CPU baseline).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

NEG_MASK = -1e6  # additive mask value of the reference, src/tiled_swa.py:712


# ----------------------------------------------------------------------------------------------
# RoPE-2D
# ----------------------------------------------------------------------------------------------

def encode_idx(height: int, width: int) -> torch.Tensor:
    """Packed per-token (row<<16)|col int32 index, row-major (src/fused_rope2d.py:173-183)."""
    rows = torch.arange(0, height)
    cols = torch.arange(0, width)
    return torch.bitwise_or(rows[:, None] << 16, cols).flatten().to(torch.int32)


def make_cs_table(n_rdim: int, max_len: int, theta: float = 10000.0) -> torch.Tensor:
    """cos/sin table ``[max_len, n_rdim, 2]`` (``[...,0]`` cos, ``[...,1]`` sin), fp32.

    Layout follows the tables the reference's self-test builds with ``dstack``
    (src/fused_rope2d.py:236-246).  Formula (unpinned, see module docstring):
    ``inv_freq_i = theta ** (-i / n_rdim)``.
    """
    inv = torch.pow(torch.tensor(float(theta), dtype=torch.float64),
                    -(torch.arange(n_rdim, dtype=torch.float64) / n_rdim))
    ang = torch.outer(torch.arange(max_len, dtype=torch.float64), inv)
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).contiguous()


def decode_idx(idx: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Split the packed index into int16 halves; -1 in a half means "no rotation"
    for that half (src/fused_rope2d.py:212-213)."""
    row = ((idx >> 16) & 0xFFFF).to(torch.int16)
    col = (idx & 0xFFFF).to(torch.int16)
    return row, col


def _cos_sin(idx_half: torch.Tensor, table: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(cos, sin) rows for one half; negative index -> (1, 0) (src/fused_rope2d.py:215-219)."""
    ok = (idx_half >= 0)[:, None]
    safe = idx_half.clamp(min=0).to(torch.int64)
    cos = torch.where(ok, table[safe, :, 0], torch.ones((), dtype=table.dtype))
    sin = torch.where(ok, table[safe, :, 1], torch.zeros((), dtype=table.dtype))
    return cos, sin


def rope2d_ref(x: torch.Tensor, idx: torch.Tensor, cs_row: torch.Tensor, cs_col: torch.Tensor,
               inverse: bool = False) -> torch.Tensor:
    """Out-of-place 2D rotary embedding on the last dim of ``x [..., N, C]``.

    Dims ``[0,R)`` pair with ``[R,2R)`` under the row angle, ``[2R,3R)`` with
    ``[3R,4R)`` under the column angle, dims ``>= 4R`` pass through
    (src/fused_rope2d.py:208-224).  ``inverse=True`` applies the transposed rotation,
    i.e. what the reference's backward kernel does to a gradient
    (src/fused_rope2d.py:114-115,121-122).
    """
    R = cs_row.shape[1]
    assert cs_col.shape[1] == R and x.shape[-1] >= 4 * R and idx.shape[0] == x.shape[-2]
    irow, icol = decode_idx(idx)
    rc, rs = _cos_sin(irow, cs_row)
    cc, cs = _cos_sin(icol, cs_col)
    if inverse:
        rs, cs = -rs, -cs
    rx0, rx1 = x[..., 0:R], x[..., R:2 * R]
    cx0, cx1 = x[..., 2 * R:3 * R], x[..., 3 * R:4 * R]
    ry0, ry1 = rx0 * rc - rx1 * rs, rx0 * rs + rx1 * rc
    cy0, cy1 = cx0 * cc - cx1 * cs, cx0 * cs + cx1 * cc
    return torch.cat([ry0, ry1, cy0, cy1, x[..., 4 * R:]], dim=-1)


# ----------------------------------------------------------------------------------------------
# Dense masked-softmax attention (the parity oracle proper)
# ----------------------------------------------------------------------------------------------

def window_mask(b_size: int, t_height: int, t_width: int, row_size: int, col_size: int,
                dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Additive ``[N,N]`` mask: 0 where the key's tile lies within ``row_size`` rows
    and ``col_size`` columns of the query's tile, -1e6 elsewhere; the window is
    truncated (not shifted) at the grid border (src/tiled_swa.py:701-713)."""
    n_tiles = t_height * t_width
    r = torch.arange(t_height)
    c = torch.arange(t_width)
    row_ok = (r[None, :] >= r[:, None] - row_size) & (r[None, :] <= r[:, None] + row_size)
    col_ok = (c[None, :] >= c[:, None] - col_size) & (c[None, :] <= c[:, None] + col_size)
    ok = row_ok[:, None, :, None] & col_ok[None, :, None, :]
    m = torch.where(ok, 0.0, NEG_MASK).to(dtype)
    N = n_tiles * b_size
    return m.reshape(n_tiles, 1, n_tiles, 1).expand(n_tiles, b_size, n_tiles, b_size).reshape(N, N)


def tiled_swa_ref(q, k, v, b_size, t_height, t_width, row_size, col_size, sm_scale: float = 1.0,
                  return_lse: bool = False):
    """Restatement of src/tiled_swa.py:693-717 with the softmax written out.

    ``q,k [B,H,N,d_qk]``, ``v [B,H,N,d_v]``; computes in the dtype of ``q``
    (pass fp32/fp64 copies for a high-precision ground truth).  ``lse`` is the
    natural-log logsumexp of the scaled, masked scores.
    """
    B, H, N, _ = q.shape
    assert N == t_height * t_width * b_size, "seqlen should match image size"
    mask = window_mask(b_size, t_height, t_width, row_size, col_size, q.dtype)
    s = torch.matmul(q, k.transpose(-1, -2)) * sm_scale + mask
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    o = torch.matmul(p, v)
    return (o, lse) if return_lse else o


def tiled_swa_ref_sdpa(q, k, v, b_size, t_height, t_width, row_size, col_size, sm_scale: float = 1.0):
    """The literal form of the reference: dense mask + ``scaled_dot_product_attention``
    (src/tiled_swa.py:712-715).  This is the function the CPU baseline times."""
    mask = window_mask(b_size, t_height, t_width, row_size, col_size, q.dtype)
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=sm_scale)


def tiled_swa_bwd_ref(q, k, v, do, b_size, t_height, t_width, row_size, col_size, sm_scale: float = 1.0):
    """Closed-form backward of the masked softmax attention (what autograd through
    src/tiled_swa.py:715 yields, and what the reference kernel spells out at
    src/tiled_swa.py:475-518,527-562): delta = rowsum(O*dO); dV = P^T dO;
    dP = dO V^T; dS = P*(dP-delta); dQ = scale*dS K; dK = scale*dS^T Q."""
    mask = window_mask(b_size, t_height, t_width, row_size, col_size, q.dtype)
    s = torch.matmul(q, k.transpose(-1, -2)) * sm_scale + mask
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, v)
    delta = (o * do).sum(-1, keepdim=True)
    dv = torch.matmul(p.transpose(-1, -2), do)
    dp = torch.matmul(do, v.transpose(-1, -2))
    ds = p * (dp - delta)
    dq = torch.matmul(ds, k) * sm_scale
    dk = torch.matmul(ds.transpose(-1, -2), q) * sm_scale
    return o, dq, dk, dv


# ----------------------------------------------------------------------------------------------
# Windowed O(N*w^2) form of the same arithmetic, for grids where [N,N] does not fit
# ----------------------------------------------------------------------------------------------

def _window_gather_index(b_size, t_height, t_width, row_size, col_size):
    """For every query token, the token indices of the (2R+1)(2C+1)*b keys of its
    untruncated window and a validity flag per slot (same predicate as
    ``window_mask``, enumerated per query instead of as an [N,N] matrix)."""
    tr = torch.arange(t_height)[:, None, None, None, None]
    tc = torch.arange(t_width)[None, :, None, None, None]
    dr = torch.arange(-row_size, row_size + 1)[None, None, :, None, None]
    dc = torch.arange(-col_size, col_size + 1)[None, None, None, :, None]
    s = torch.arange(b_size)[None, None, None, None, :]
    kr, kc = tr + dr, tc + dc
    ok = (kr >= 0) & (kr < t_height) & (kc >= 0) & (kc < t_width) & (s >= 0)
    tok = (kr.clamp(0, t_height - 1) * t_width + kc.clamp(0, t_width - 1)) * b_size + s
    n_tiles = t_height * t_width
    W = (2 * row_size + 1) * (2 * col_size + 1) * b_size
    tok = tok.expand(t_height, t_width, -1, -1, -1).reshape(n_tiles, 1, W).expand(n_tiles, b_size, W)
    ok = ok.expand(t_height, t_width, -1, -1, -1).reshape(n_tiles, 1, W).expand(n_tiles, b_size, W)
    return tok.reshape(n_tiles * b_size, W), ok.reshape(n_tiles * b_size, W)


def tiled_swa_windowed(q, k, v, do: Optional[torch.Tensor], b_size, t_height, t_width, row_size, col_size,
                       sm_scale: float = 1.0, chunk: int = 4096):
    """Same result as ``tiled_swa_ref`` / ``tiled_swa_bwd_ref`` but touching only the
    keys inside each query's window, query-chunked; used for grids whose dense
    mask is too large.  Returns ``(o, lse)`` or ``(o, lse, dq, dk, dv)``."""
    B, H, N, dqk = q.shape
    dv_ = v.shape[-1]
    tok, ok = _window_gather_index(b_size, t_height, t_width, row_size, col_size)
    o = torch.empty(B, H, N, dv_, dtype=q.dtype)
    lse = torch.empty(B, H, N, dtype=q.dtype)
    if do is not None:
        dq = torch.empty_like(q)
        dk = torch.zeros_like(k)
        dvv = torch.zeros_like(v)
    for n0 in range(0, N, chunk):
        n1 = min(N, n0 + chunk)
        t, m = tok[n0:n1], ok[n0:n1]
        kk = k[:, :, t]                      # [B,H,c,W,d]
        vv = v[:, :, t]
        s = torch.einsum("bhnd,bhnwd->bhnw", q[:, :, n0:n1], kk) * sm_scale
        s = s.masked_fill(~m, float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l[..., None])
        oc = torch.einsum("bhnw,bhnwd->bhnd", p, vv)
        o[:, :, n0:n1], lse[:, :, n0:n1] = oc, l
        if do is not None:
            doc = do[:, :, n0:n1]
            delta = (oc * doc).sum(-1, keepdim=True)
            dp = torch.einsum("bhnd,bhnwd->bhnw", doc, vv)
            ds = p * (dp - delta)
            dq[:, :, n0:n1] = torch.einsum("bhnw,bhnwd->bhnd", ds, kk) * sm_scale
            flat = t.reshape(-1)
            dk.index_add_(2, flat, (ds[..., None] * q[:, :, n0:n1, None, :]).reshape(B, H, -1, dqk) * sm_scale)
            dvv.index_add_(2, flat, (p[..., None] * doc[:, :, :, None, :]).reshape(B, H, -1, dv_))
    return (o, lse) if do is None else (o, lse, dq, dk, dvv)


# ----------------------------------------------------------------------------------------------
# The composed path: RoPE-2D on q and k, then windowed attention; gradients for the
# un-rotated q and k (the chain rule the reference gets from autograd: K4 -> K7).
# ----------------------------------------------------------------------------------------------

def fused_ref(q, k, v, do, idx, cs_row, cs_col, b_size, t_height, t_width, row_size, col_size, sm_scale,
              windowed: bool = False):
    """``o = swa(rope(q), rope(k), v)`` and, if ``do`` is given, ``dq, dk, dv``.

    ``idx is None`` skips the rotation.  Everything is evaluated in the dtype of the
    arguments; callers pass fp32/fp64 copies of the rounded low-precision inputs
    to get the ground truth.
    """
    if idx is not None:
        qr = rope2d_ref(q, idx, cs_row.to(q.dtype), cs_col.to(q.dtype))
        kr = rope2d_ref(k, idx, cs_row.to(q.dtype), cs_col.to(q.dtype))
    else:
        qr, kr = q, k
    args = (b_size, t_height, t_width, row_size, col_size, sm_scale)
    if do is None:
        if windowed:
            return tiled_swa_windowed(qr, kr, v, None, *args)[0]
        return tiled_swa_ref(qr, kr, v, *args)
    if windowed:
        o, _, dq, dk, dv = tiled_swa_windowed(qr, kr, v, do, *args)
    else:
        o, dq, dk, dv = tiled_swa_bwd_ref(qr, kr, v, do, *args)
    if idx is not None:
        dq = rope2d_ref(dq, idx, cs_row.to(q.dtype), cs_col.to(q.dtype), inverse=True)
        dk = rope2d_ref(dk, idx, cs_row.to(q.dtype), cs_col.to(q.dtype), inverse=True)
    return o, dq, dk, dv


# ----------------------------------------------------------------------------------------------
# Error metrics and seeded workloads
# ----------------------------------------------------------------------------------------------

def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return (a.double() - b.double()).abs().max().item()


def mean_rel(a: torch.Tensor, b: torch.Tensor) -> float:
    """mean|a-b| / mean|b| -- the mean-relative error the parity tolerance is stated in."""
    return ((a.double() - b.double()).abs().mean() / b.double().abs().mean().clamp_min(1e-30)).item()


def seeded_inputs(B, H, tokens, d_qk, d_v, dtype, seed: int = 0):
    """q, k, v, dO ~ N(0,1) drawn in fp32 from one CPU generator in that order, then
    rounded to ``dtype`` (so the oracle and the kernels see identical bits)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((B, H, tokens, d_qk), generator=g, dtype=torch.float32).to(dtype)
    k = torch.randn((B, H, tokens, d_qk), generator=g, dtype=torch.float32).to(dtype)
    v = torch.randn((B, H, tokens, d_v), generator=g, dtype=torch.float32).to(dtype)
    do = torch.randn((B, H, tokens, d_v), generator=g, dtype=torch.float32).to(dtype)
    return q, k, v, do


def windowed_flops(B, H, tokens, b_size, row_size, col_size, d_qk, d_v) -> Tuple[float, float]:
    """(forward, backward) FLOPs under the windowed convention: forward
    ``2*N*w^2*(d_qk+d_v)``, backward 2.5x that; border truncation ignored."""
    w2 = (2 * row_size + 1) * (2 * col_size + 1) * b_size
    fwd = 2.0 * B * H * tokens * w2 * (d_qk + d_v)
    return fwd, 2.5 * fwd
