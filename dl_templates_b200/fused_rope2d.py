"""Fused in-place 2D rotary position embedding: the call surface of the
reference's ``src/fused_rope2d.py`` on top of the sm_100a C-ABI library.

  ``RotaryPE2D.apply(x, idx, row_cs_buffer, col_cs_buffer) -> x``  (in place; src/fused_rope2d.py:124-168)
  ``FusedInplaceRotaryPositionEncoding2D(n_components, max_h, max_w)`` with ``encode_idx`` and
  ``forward(x, idx)``                                              (src/fused_rope2d.py:171-201)

Semantics follow ``rope2d_ref`` (src/fused_rope2d.py:204-225): ``idx[n] = (row<<16)|col``
with int16 halves, a negative half leaves that half of the token un-rotated; dims
``[0,R)``/``[R,2R)`` rotate by the row angle, ``[2R,3R)``/``[3R,4R)`` by the column angle,
dims ``>= 4R`` pass through.  The reference's Triton kernel substitutes (cos,sin) =
(1,1) resp. (0,0) for a negative half inside a partly-indexed token block
(src/fused_rope2d.py:53-54); that is not reproduced -- the oracle's pass-through is.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


def make_cs_table(n_rdim: int, max_len: int, theta: float = 10000.0, device=None) -> torch.Tensor:
    """cos/sin table ``[max_len, n_rdim, 2]`` fp32, ``inv_freq_i = theta**(-i/n_rdim)``.

    The reference takes this table from a module it does not ship
    (src/fused_rope2d.py:8), so the formula is this package's own; the layout is the
    one its self-test builds (src/fused_rope2d.py:236-246)."""
    inv = torch.pow(torch.tensor(float(theta), dtype=torch.float64),
                    -(torch.arange(n_rdim, dtype=torch.float64) / n_rdim))
    ang = torch.outer(torch.arange(max_len, dtype=torch.float64), inv)
    t = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).contiguous()
    return t.to(device) if device is not None else t


class FusedRotaryPositionEncodingContext(torch.nn.Module):
    """Holder of one ``cs_components [max_len, n_components, 2]`` table -- the object the
    reference module expects from its missing sibling (src/fused_rope2d.py:8,193-194)."""

    def __init__(self, n_components: int, max_len: int, theta: float = 10000.0):
        super().__init__()
        self.register_buffer("cs_components", make_cs_table(n_components, max_len, theta), persistent=False)


def rope2d_apply_(x: torch.Tensor, idx: torch.Tensor, row_cs: torch.Tensor, col_cs: torch.Tensor,
                  inverse: bool = False) -> torch.Tensor:
    """In-place rotation of ``x [batch, N, C]`` (any strides); returns ``x``."""
    if not x.is_cuda:
        raise RuntimeError("dl_templates_b200 runs on CUDA tensors only (sm_100a); there is no CPU path")
    B, N, n_dim = x.shape
    assert row_cs.shape[1] == col_cs.shape[1]
    assert idx.shape[0] == N
    with torch.cuda.device(x.device):
        rope = _lib.make_rope(idx, row_cs, col_cs)
        xs = (C.c_int64 * 3)(x.stride(0), x.stride(1), x.stride(2))
        code = _lib.lib.rope2d_apply(_lib.dtype_code(x.dtype), x.data_ptr(), B, N, n_dim, xs, C.byref(rope),
                                     1 if inverse else 0, _lib.stream_ptr(x.device))
    _lib.check(code, "rope2d_apply")
    return x


def rope2d_apply_to(x: torch.Tensor, idx: torch.Tensor, row_cs: torch.Tensor, col_cs: torch.Tensor,
                    inverse: bool = False) -> torch.Tensor:
    """``rope(x)`` (or the inverse rotation) of ``x [batch, N, C]`` in a new contiguous tensor, ``x`` untouched:
    one pass when the layout allows (fp16 / bf16, ``n_rdim % 8 == 0``, ``C % 8 == 0``, unit last stride, 16-byte
    aligned rows), else a copy followed by the in-place kernel."""
    if not x.is_cuda:
        raise RuntimeError("dl_templates_b200 runs on CUDA tensors only (sm_100a); there is no CPU path")
    B, N, n_dim = x.shape
    assert row_cs.shape[1] == col_cs.shape[1] and idx.shape[0] == N
    y = torch.empty((B, N, n_dim), dtype=x.dtype, device=x.device)
    rows16 = x.stride(2) == 1 and x.data_ptr() % 16 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0
    if x.dtype in (torch.float16, torch.bfloat16) and row_cs.shape[1] % 8 == 0 and n_dim % 8 == 0 and rows16:
        with torch.cuda.device(x.device):
            rope = _lib.make_rope(idx, row_cs, col_cs)
            xs = (C.c_int64 * 3)(x.stride(0), x.stride(1), x.stride(2))
            ys = (C.c_int64 * 3)(y.stride(0), y.stride(1), y.stride(2))
            code = _lib.lib.rope2d_apply_to(_lib.dtype_code(x.dtype), x.data_ptr(), y.data_ptr(), B, N, n_dim, xs, ys,
                                            C.byref(rope), 1 if inverse else 0, _lib.stream_ptr(x.device))
        _lib.check(code, "rope2d_apply_to")
        return y
    y.copy_(x)
    return rope2d_apply_(y, idx, row_cs, col_cs, inverse)


class RotaryPE2D(torch.autograd.Function):
    """``RotaryPE2D.apply(x, idx, row_cs_buffer, col_cs_buffer)``: rotates ``x [B,N,C]`` in
    place and returns it; backward applies the inverse rotation to a copy of the
    incoming gradient (src/fused_rope2d.py:126-168)."""

    @staticmethod
    def forward(ctx, x, idx, row_cs_buffer, col_cs_buffer):
        rope2d_apply_(x, idx, row_cs_buffer, col_cs_buffer, inverse=False)
        ctx.mark_dirty(x)
        ctx.save_for_backward(idx, row_cs_buffer, col_cs_buffer)
        return x

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, do):
        idx, row_cs_buffer, col_cs_buffer = ctx.saved_tensors
        dx = rope2d_apply_to(do, idx, row_cs_buffer, col_cs_buffer, inverse=True)   # clone + inverse rotation in one pass
        return dx, None, None, None


class FusedInplaceRotaryPositionEncoding2D(torch.nn.Module):
    """Module form (src/fused_rope2d.py:171-201): ``n_components // 2`` rotation pairs for
    rows and as many for columns, i.e. the first ``2 * n_components`` dims of ``x``
    are rotated."""

    @staticmethod
    def encode_idx(height: int, width: int) -> torch.Tensor:
        """Packed token indices of an image-like ``height x width`` grid, row-major
        (src/fused_rope2d.py:173-183)."""
        rows = torch.arange(0, height)
        cols = torch.arange(0, width)
        return torch.bitwise_or(rows[:, None] << 16, cols).flatten().to(torch.int32)

    def __init__(self, n_components: int, max_h: int, max_w: int, theta: float = 10000.0):
        super().__init__()
        self.max_h = max_h
        self.max_w = max_w
        self.row_components = n_components // 2
        self.col_components = n_components // 2
        self.row_buffer = FusedRotaryPositionEncodingContext(self.row_components, max_h, theta)
        self.col_buffer = FusedRotaryPositionEncodingContext(self.col_components, max_w, theta)

    def forward(self, x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        # x: [B, Head, N, C]  idx: [N]
        B, H, N, Cdim = x.shape
        x0 = x.reshape((-1, N, Cdim))
        return RotaryPE2D.apply(x0, idx, self.row_buffer.cs_components, self.col_buffer.cs_components).reshape(x.shape)
