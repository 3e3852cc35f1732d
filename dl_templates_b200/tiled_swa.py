"""Tiled 2D sliding-window attention: the call surface of the reference's
``src/tiled_swa.py`` on top of the sm_100a C-ABI library.

Same names and argument order as the reference:

  ``TiledSwa.apply(q, k, v, b_size, t_height, t_width, row_size, col_size, sm_scale)``   (src/tiled_swa.py:604)
  ``tiled_swa_fwd(q, k, v, b_size, t_height, t_width, row_size, col_size, sm_scale=1.0)`` (src/tiled_swa.py:564)

plus the composed entry the reference does not have (RoPE-2D and attention as one
autograd function; q and k stay untouched, their gradients come back un-rotated):

  ``TiledSwaRope2D.apply(q, k, v, idx, row_cs_buffer, col_cs_buffer, b_size, t_height,
  t_width, row_size, col_size, sm_scale)``

Layout: ``q, k [B,H,N,d_qk]``, ``v, o [B,H,N,d_v]``, ``N = t_height*t_width*b_size``,
token ``n = (tile_row*t_width + tile_col)*b_size + s``; a query attends every token
of every tile within ``row_size`` rows and ``col_size`` columns of its own tile,
truncated at the grid border (src/tiled_swa.py:76-79,212-214,704-710).

Departures from reference quirks (none changes the mathematics): outputs take the
dtype and device of ``q`` (the reference hard-codes fp16 on the default device,
src/tiled_swa.py:608-609); ``dq`` comes back in ``q.dtype`` (reference: fp32,
src/tiled_swa.py:656); backward works for every ``b_size`` (reference raises
below 16, src/tiled_swa.py:660-661); the saved softmax statistic is fp32.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import _lib

_status_words = {}
_status_mirrors = {}      # per device: (pinned host copy of the status word, event after the copy)


def _status(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] word the tensor-core kernels write to when one of their
    bounded waits gives up; stays zero in normal operation."""
    key = (device.type, device.index)
    if key not in _status_words:
        _status_words[key] = torch.zeros(1024, dtype=torch.int32, device=device)
    return _status_words[key]


def _raise_timeout(key, vals):
    raise RuntimeError(f"swa2d kernel reported a bounded-wait timeout on {key}: status={vals} "
                       "(its outputs are incomplete)")


def _watch_status(device: torch.device) -> None:
    """A timed-out kernel must not go unnoticed by callers that never synchronise on it: after every batch of
    launches the status word is copied to pinned host memory on the same stream (16 bytes, no synchronisation),
    and every later call first looks at the copies that have arrived."""
    key = (device.type, device.index)
    if key not in _status_mirrors:
        _status_mirrors[key] = (torch.zeros(4, dtype=torch.int32).pin_memory(), torch.cuda.Event())
    host, ev = _status_mirrors[key]
    host.copy_(_status(device)[:4], non_blocking=True)
    ev.record(torch.cuda.current_stream(device))


def _poll_status() -> None:
    """Raise if a status copy that has ALREADY arrived reports a timed-out wait (never blocks)."""
    for key, (host, ev) in _status_mirrors.items():
        if ev.query() and int(host[0]) != 0:
            vals = host.tolist()
            host.zero_()
            _status_words[key].zero_()
            _raise_timeout(key, vals)


def check_status(device=None) -> None:
    """Synchronise and raise if any kernel reported a timed-out wait."""
    for key, word in _status_words.items():
        vals = word[:4].cpu().tolist()
        if vals[0] != 0:
            word.zero_()
            if key in _status_mirrors:
                _status_mirrors[key][0].zero_()
            _raise_timeout(key, vals)


def _check_inputs(q, k, v, b_size, t_height, t_width):
    _poll_status()
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("dl_templates_b200 runs on CUDA tensors only (sm_100a); there is no CPU path")
    if q.dim() != 4 or k.shape != q.shape or v.shape[:3] != q.shape[:3]:
        raise ValueError("expected q,k [B,H,N,d_qk] and v [B,H,N,d_v]")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise TypeError("q, k, v must share a dtype")
    assert q.shape[2] == t_height * t_width * b_size, "seqlen should match image size"


def _geom(q, v, b_size, t_height, t_width, row_size, col_size, sm_scale, impl):
    B, H, N, d_qk = q.shape
    return _lib.make_geom(q.dtype, B, H, b_size, t_height, t_width, row_size, col_size, d_qk, v.shape[-1], sm_scale,
                          impl)


def _ref(x):
    return C.byref(x) if x is not None else None


def padded_head_dims(q, v, rope, b_size, t_height, t_width, row_size, col_size, sm_scale=1.0, impl="auto"):
    """``(d_qk', d_v')`` if zero-padding the head dims to 64 or 128 moves this problem from the SIMT kernels to
    the tensor-core kernels, else ``None``.  Padding q and k with zero columns leaves every score unchanged,
    padding v adds zero columns to O; the reference's own test shape (d = 32, b_size = 16,
    src/tiled_swa.py:736-746) is the case this exists for."""
    if impl != "auto" or q.dtype == torch.float32 or os.environ.get("SWA_NO_HEAD_PAD"):
        return None

    def up(d):
        return d if d in (64, 128) else 64 if d < 64 else 128 if d < 128 else None

    d_qk, d_v = q.shape[-1], v.shape[-1]
    p_qk, p_v = up(d_qk), up(d_v)
    if p_qk is None or p_v is None or (p_qk == d_qk and p_v == d_v):
        return None
    B, H, _, _ = q.shape
    r = _lib.make_rope(*rope) if rope is not None else None
    # head dims of 32 and 96 run on the tensor-core kernels as they are when no streamed row has to be rotated
    # (TMA zero-fills the missing half of the last 64-element chunk): nothing to pad then
    g0 = _lib.make_geom(q.dtype, B, H, b_size, t_height, t_width, row_size, col_size, d_qk, d_v, sm_scale, "auto")
    if all(_lib.lib.swa_select_impl(C.byref(g0), _ref(r), which) == _lib.IMPL_TC for which in (0, 1, 2)):
        return None
    g = _lib.make_geom(q.dtype, B, H, b_size, t_height, t_width, row_size, col_size, p_qk, p_v, sm_scale, "auto")
    for which in (0, 1, 2):
        if _lib.lib.swa_select_impl(C.byref(g), _ref(r), which) != _lib.IMPL_TC:
            return None
    return p_qk, p_v


def _pad_last(t, d):
    return t if t.shape[-1] == d else torch.nn.functional.pad(t, (0, d - t.shape[-1]))


def _tc_addressable(t) -> bool:
    """Unit last stride, positive strides that are multiples of 8 elements, 16-byte aligned base: what a tensor map
    of the tensor-core kernels can describe (fp32 runs on the SIMT kernels, which take any strides)."""
    st = t.stride()
    return st[-1] == 1 and min(st[:3]) > 0 and not any(x % 8 for x in st[:3]) and t.data_ptr() % 16 == 0


def _materialise(*tensors):
    """16-bit tensors the tensor-core kernels cannot address are copied once rather than sending the call to
    the SIMT kernels (two orders of magnitude slower); everything else is passed through untouched."""
    return tuple(t if t.dtype == torch.float32 or _tc_addressable(t) else t.contiguous() for t in tensors)


def _check_out(t, shape, like, what):
    if t.shape != shape or t.dtype != like.dtype or t.device != like.device:
        raise ValueError(f"{what}: expected shape {tuple(shape)}, dtype {like.dtype} on {like.device}")


def swa_forward(q, k, v, rope, b_size, t_height, t_width, row_size, col_size, sm_scale, impl="auto", out=None):
    """Launch the forward kernel; returns ``(o, lse)`` with ``lse`` fp32 ``[B,H,N]`` in
    the base-2 domain.  ``rope`` is ``None`` or ``(idx, row_cs, col_cs)``.  ``out``: an
    optional ``[B,H,N,d_v]`` tensor or strided view the kernel writes O into (e.g. a view
    of a ``[B,N,H*d_v]`` buffer for the output projection)."""
    _check_inputs(q, k, v, b_size, t_height, t_width)
    B, H, N, _ = q.shape
    q, k, v = _materialise(q, k, v)
    pad = padded_head_dims(q, v, rope, b_size, t_height, t_width, row_size, col_size, sm_scale, impl)
    if pad is not None:
        o_p, lse = swa_forward(_pad_last(q, pad[0]), _pad_last(k, pad[0]), _pad_last(v, pad[1]), rope, b_size, t_height,
                               t_width, row_size, col_size, sm_scale, impl)
        o_v = o_p[..., :v.shape[-1]]
        if out is None:
            return o_v.contiguous(), lse
        _check_out(out, o_v.shape, q, "out")
        out.copy_(o_v)
        return out, lse
    with torch.cuda.device(q.device):
        if out is None:
            o = torch.empty((B, H, N, v.shape[-1]), dtype=q.dtype, device=q.device)
        else:
            o = out
            _check_out(o, (B, H, N, v.shape[-1]), q, "out")
        lse = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
        g = _geom(q, v, b_size, t_height, t_width, row_size, col_size, sm_scale, impl)
        r = _lib.make_rope(*rope) if rope is not None else None
        tq, tk, tv, to = (_lib.tensor4(t) for t in (q, k, v, o))
        code = _lib.lib.swa_fwd(C.byref(g), _ref(r), C.byref(tq), C.byref(tk), C.byref(tv), C.byref(to),
                                lse.data_ptr(), _status(q.device).data_ptr(), _lib.stream_ptr(q.device))
    _lib.check(code, "swa_fwd")
    _watch_status(q.device)
    if os.environ.get("SWA_DEBUG_SYNC"):
        check_status()
    return o, lse


def swa_backward(q, k, v, o, lse, do, rope, b_size, t_height, t_width, row_size, col_size, sm_scale, impl="auto",
                 out=None):
    """Launch delta, dQ and dK/dV kernels; returns ``(dq, dk, dv)`` in the input dtype
    (gradients of the un-rotated q and k when ``rope`` is given).  ``out``: optional
    ``(dq, dk, dv)`` tensors or strided views to write into (e.g. the three slices of one
    packed ``[B,N,3,H,d]`` gradient buffer)."""
    _poll_status()        # e.g. the forward of this very step: its status copy has usually arrived by now
    B, H, N, _ = q.shape
    q, k, v, o, do = _materialise(q, k, v, o, do)   # e.g. the expanded (stride-0) gradient of ``o.sum()``
    pad = padded_head_dims(q, v, rope, b_size, t_height, t_width, row_size, col_size, sm_scale, impl)
    if pad is not None:
        grads = swa_backward(_pad_last(q, pad[0]), _pad_last(k, pad[0]), _pad_last(v, pad[1]), _pad_last(o, pad[1]), lse,
                             _pad_last(do, pad[1]), rope, b_size, t_height, t_width, row_size, col_size, sm_scale, impl)
        grads = tuple(g[..., :like.shape[-1]] for g, like in zip(grads, (q, k, v)))
        if out is None:
            return tuple(g.contiguous() for g in grads)
        for t, g, what in zip(out, grads, ("dq", "dk", "dv")):
            _check_out(t, g.shape, q, what)
            t.copy_(g)
        return tuple(out)
    with torch.cuda.device(q.device):
        if out is None:
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        else:
            dq, dk, dv = out
            for t, like, what in ((dq, q, "dq"), (dk, k, "dk"), (dv, v, "dv")):
                _check_out(t, like.shape, like, what)
        delta = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
        g = _geom(q, v, b_size, t_height, t_width, row_size, col_size, sm_scale, impl)
        r = _lib.make_rope(*rope) if rope is not None else None
        tq, tk, tv, to, tdo, tdq, tdk, tdv = (_lib.tensor4(t) for t in (q, k, v, o, do, dq, dk, dv))
        st, status = _lib.stream_ptr(q.device), _status(q.device).data_ptr()
        _lib.check(_lib.lib.swa_bwd_delta(C.byref(g), C.byref(to), C.byref(tdo), delta.data_ptr(), st),
                   "swa_bwd_delta")
        _lib.check(_lib.lib.swa_bwd_dq(C.byref(g), _ref(r), C.byref(tq), C.byref(tk), C.byref(tv), C.byref(tdo),
                                       lse.data_ptr(), delta.data_ptr(), C.byref(tdq), status, st), "swa_bwd_dq")
        _lib.check(_lib.lib.swa_bwd_dkdv(C.byref(g), _ref(r), C.byref(tq), C.byref(tk), C.byref(tv), C.byref(tdo),
                                         lse.data_ptr(), delta.data_ptr(), C.byref(tdk), C.byref(tdv), status, st),
                   "swa_bwd_dkdv")
    _watch_status(q.device)
    if os.environ.get("SWA_DEBUG_SYNC"):
        check_status()
    return dq, dk, dv


def swa_forward_rot(q, k, v, rope, b_size, t_height, t_width, row_size, col_size, sm_scale, impl="auto", out=None):
    """Forward with the rotation handed on (``swa_fwd_rot``): returns ``(o, lse, q_rot, k_rot)``.

    Every key row is rotated once by a streaming pass into ``k_rot``, every query tile is rotated on chip by the
    attention kernel, which stores the rotated rows to ``q_rot``; ``q`` and ``k`` stay untouched.  ``q_rot`` and
    ``k_rot`` are what ``swa_backward_rot`` takes in place of ``q`` and ``k`` -- the tensors the reference keeps for
    backward as well, since its RoPE rotates q and k in place (src/fused_rope2d.py:143-145).  ``rope`` =
    ``(idx, row_cs, col_cs)`` is required; ``out`` as in ``swa_forward``."""
    _check_inputs(q, k, v, b_size, t_height, t_width)
    B, H, N, _ = q.shape
    q, k, v = _materialise(q, k, v)
    with torch.cuda.device(q.device):
        if out is None:
            o = torch.empty((B, H, N, v.shape[-1]), dtype=q.dtype, device=q.device)
        else:
            o = out
            _check_out(o, (B, H, N, v.shape[-1]), q, "out")
        lse = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
        q_rot = torch.empty((B, H, N, q.shape[-1]), dtype=q.dtype, device=q.device)
        k_rot = torch.empty_like(q_rot)
        g = _geom(q, v, b_size, t_height, t_width, row_size, col_size, sm_scale, impl)
        r = _lib.make_rope(*rope)
        tq, tk, tv, to, tqr, tkr = (_lib.tensor4(t) for t in (q, k, v, o, q_rot, k_rot))
        code = _lib.lib.swa_fwd_rot(C.byref(g), C.byref(r), C.byref(tq), C.byref(tk), C.byref(tv), C.byref(to),
                                    lse.data_ptr(), C.byref(tqr), C.byref(tkr), _status(q.device).data_ptr(),
                                    _lib.stream_ptr(q.device))
    _lib.check(code, "swa_fwd_rot")
    _watch_status(q.device)
    if os.environ.get("SWA_DEBUG_SYNC"):
        check_status()
    return o, lse, q_rot, k_rot


def swa_backward_rot(q_rot, k_rot, v, o, lse, do, rope, b_size, t_height, t_width, row_size, col_size, sm_scale,
                     impl="auto", out=None):
    """Backward pass on the rotated copies ``swa_forward_rot`` left behind: delta, ``swa_bwd_dq_rot``,
    ``swa_bwd_dkdv_rot``.  Returns ``(dq, dk, dv)``, gradients of the UN-rotated q and k (the kernels rotate dq and
    dk back in their epilogues).  ``out`` as in ``swa_backward``."""
    _poll_status()
    B, H, N, _ = q_rot.shape
    q_rot, k_rot, v, o, do = _materialise(q_rot, k_rot, v, o, do)
    with torch.cuda.device(q_rot.device):
        if out is None:
            dq, dk, dv = torch.empty_like(q_rot), torch.empty_like(k_rot), torch.empty_like(v)
        else:
            dq, dk, dv = out
            for t, like, what in ((dq, q_rot, "dq"), (dk, k_rot, "dk"), (dv, v, "dv")):
                _check_out(t, like.shape, like, what)
        delta = torch.empty((B, H, N), dtype=torch.float32, device=q_rot.device)
        g = _geom(q_rot, v, b_size, t_height, t_width, row_size, col_size, sm_scale, impl)
        r = _lib.make_rope(*rope)
        tq, tk, tv, to, tdo, tdq, tdk, tdv = (_lib.tensor4(t) for t in (q_rot, k_rot, v, o, do, dq, dk, dv))
        st, status = _lib.stream_ptr(q_rot.device), _status(q_rot.device).data_ptr()
        _lib.check(_lib.lib.swa_bwd_delta(C.byref(g), C.byref(to), C.byref(tdo), delta.data_ptr(), st),
                   "swa_bwd_delta")
        _lib.check(_lib.lib.swa_bwd_dq_rot(C.byref(g), C.byref(r), C.byref(tq), C.byref(tk), C.byref(tv), C.byref(tdo),
                                           lse.data_ptr(), delta.data_ptr(), C.byref(tdq), status, st), "swa_bwd_dq_rot")
        _lib.check(_lib.lib.swa_bwd_dkdv_rot(C.byref(g), C.byref(r), C.byref(tq), C.byref(tk), C.byref(tv),
                                             C.byref(tdo), lse.data_ptr(), delta.data_ptr(), C.byref(tdk),
                                             C.byref(tdv), status, st), "swa_bwd_dkdv_rot")
    _watch_status(q_rot.device)
    if os.environ.get("SWA_DEBUG_SYNC"):
        check_status()
    return dq, dk, dv


def swa_backward_noalloc(q, k, v, o, lse, do, rope, b_size, t_height, t_width, row_size, col_size, sm_scale, dq, dk,
                         dv, impl="auto"):
    """Backward pass into caller-provided ``dq, dk, dv`` through ``swa_bwd_noalloc``: the library
    neither allocates nor frees anything, the softmax-delta scratch lives in a fixed array
    inside the library (limit: ``B*H*N <= _lib.NOALLOC_MAX_ROWS``).  Meant for callers that own
    no allocator (everything, outputs included, comes from memory they reserved up front).
    Calls on one device share that array, so do not let two of them overlap on the GPU; the
    first call on a device does a one-time address lookup and should come before any stream
    capture.  Returns ``(dq, dk, dv)``."""
    B, H, N, _ = q.shape
    g = _geom(q, v, b_size, t_height, t_width, row_size, col_size, sm_scale, impl)
    r = _lib.make_rope(*rope) if rope is not None else None
    tq, tk, tv, to, tdo, tdq, tdk, tdv = (_lib.tensor4(t) for t in (q, k, v, o, do, dq, dk, dv))
    with torch.cuda.device(q.device):
        code = _lib.lib.swa_bwd_noalloc(C.byref(g), _ref(r), C.byref(tq), C.byref(tk), C.byref(tv), C.byref(to),
                                        C.byref(tdo), lse.data_ptr(), C.byref(tdq), C.byref(tdk), C.byref(tdv),
                                        _status(q.device).data_ptr(), _lib.stream_ptr(q.device))
    _lib.check(code, "swa_bwd_noalloc")
    _watch_status(q.device)
    return dq, dk, dv


def selected_impl(q, v, rope, b_size, t_height, t_width, row_size, col_size, sm_scale=1.0, which=0, impl="auto"):
    """'tc' or 'simt': the kernel family a call with these shapes would run."""
    g = _geom(q, v, b_size, t_height, t_width, row_size, col_size, sm_scale, impl)
    r = _lib.make_rope(*rope) if rope is not None else None
    code = _lib.lib.swa_select_impl(C.byref(g), _ref(r), which)
    if code < 0:
        _lib.check(code, "swa_select_impl")
    return {_lib.IMPL_SIMT: "simt", _lib.IMPL_TC: "tc"}[code]


def tiled_swa_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, b_size: int, t_height: int, t_width: int,
                  row_size: int, col_size: int, sm_scale: float = 1.0) -> torch.Tensor:
    """Forward only, no autograd graph (src/tiled_swa.py:564-600)."""
    return swa_forward(q, k, v, None, b_size, t_height, t_width, row_size, col_size, sm_scale)[0]


class TiledSwa(torch.autograd.Function):
    """``TiledSwa.apply(q, k, v, b_size, t_height, t_width, row_size, col_size, sm_scale)``
    -- src/tiled_swa.py:602-689."""

    @staticmethod
    def forward(ctx, q, k, v, b_size: int, t_height: int, t_width: int, row_size: int, col_size: int,
                sm_scale: float):
        o, lse = swa_forward(q, k, v, None, b_size, t_height, t_width, row_size, col_size, sm_scale)
        ctx.save_for_backward(q, k, v, lse, o)
        ctx.win = (b_size, t_height, t_width, row_size, col_size, sm_scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, lse, o = ctx.saved_tensors
        dq, dk, dv = swa_backward(q, k, v, o, lse, do, None, *ctx.win)
        return dq, dk, dv, None, None, None, None, None, None


_rope_mode = os.environ.get("SWA_ROPE_MODE", "handoff")
_ROPE_MODES = ("handoff", "fused", "prerotate")


def set_rope_mode(mode: str) -> str:
    """How ``TiledSwaRope2D`` and ``TiledSwaPackedQKV`` apply the rotation; returns the previous mode.

    ``"handoff"`` (default): every q and k row is rotated exactly once, by a streaming pass that writes rotated
    copies (``swa_forward_rot``); all three attention kernels read the copies, which replace q and k among the
    tensors saved for backward (the reference keeps the same thing: its RoPE rotates q and k in place,
    src/fused_rope2d.py:143-145), and the backward kernels rotate dq and dk back in their epilogues
    (``swa_backward_rot``).  ``"fused"``: every kernel rotates the rows it streams in shared memory (no temporaries,
    but a row is rotated once per tile whose window holds it: 4.4x at a 13 x 13 window).  ``"prerotate"``: the
    reference's own composition (src/fused_rope2d.py:126-168 around src/tiled_swa.py:604) -- rotated copies,
    attention without RoPE, separate in-place inverse rotation of dq and dk.  A module-level switch like the
    reference's ``use_fused_na()`` / ``use_autotuner()`` toggles."""
    global _rope_mode
    if mode == "auto":
        mode = "handoff"
    if mode not in _ROPE_MODES:
        raise ValueError(f"rope mode must be one of {_ROPE_MODES}")
    prev, _rope_mode = _rope_mode, mode
    return prev


def _mode_for(q, v, rope, win) -> str:
    """The mode a call runs in: 'none' without RoPE; head dims that only reach the tensor-core kernels through
    zero padding take the fused path (the padding wrapper lives there)."""
    if rope is None:
        return "none"
    if _rope_mode == "handoff" and padded_head_dims(q, v, rope, *win) is not None:
        return "fused"
    return _rope_mode


def _flat3(x):
    return x.view(-1, x.shape[2], x.shape[3])


class TiledSwaRope2D(torch.autograd.Function):
    """RoPE-2D and the attention as one autograd function.

    Equivalent to ``TiledSwa.apply(rope(q, idx), rope(k, idx), v, ...)`` with
    ``rope`` = ``RotaryPE2D`` (src/fused_rope2d.py:124-168), but q and k are left
    unmodified and ``dq``/``dk`` are gradients of the un-rotated tensors (rotated back
    inside the backward kernels).  How the rotation itself is done: ``set_rope_mode``.
    ``idx`` may be ``None`` (no rotation).
    """

    @staticmethod
    def forward(ctx, q, k, v, idx: Optional[torch.Tensor], row_cs_buffer, col_cs_buffer, b_size: int,
                t_height: int, t_width: int, row_size: int, col_size: int, sm_scale: float):
        rope = None if idx is None else (idx, row_cs_buffer, col_cs_buffer)
        if rope is not None:
            assert idx.shape[0] == q.shape[2]
            assert row_cs_buffer.shape[1] == col_cs_buffer.shape[1]
        win = (b_size, t_height, t_width, row_size, col_size, sm_scale)
        ctx.mode = _mode_for(q, v, rope, win)
        if ctx.mode == "handoff":       # q, k below are the rotated copies: they are what backward needs
            o, lse, q, k = swa_forward_rot(q, k, v, rope, *win)
        elif ctx.mode == "prerotate":
            from .fused_rope2d import rope2d_apply_to
            q, k = (rope2d_apply_to(t.reshape(-1, t.shape[2], t.shape[3]) if t.is_contiguous() else
                                    t.contiguous().view(-1, t.shape[2], t.shape[3]), *rope).view(t.shape) for t in (q, k))
            o, lse = swa_forward(q, k, v, None, *win)
        else:
            o, lse = swa_forward(q, k, v, rope, *win)
        if rope is None:
            ctx.save_for_backward(q, k, v, lse, o)
        else:
            ctx.save_for_backward(q, k, v, lse, o, idx, row_cs_buffer, col_cs_buffer)
        ctx.win = (b_size, t_height, t_width, row_size, col_size, sm_scale)
        return o

    @staticmethod
    def backward(ctx, do):
        saved = ctx.saved_tensors
        q, k, v, lse, o = saved[:5]
        rope = tuple(saved[5:8]) if len(saved) == 8 else None
        if ctx.mode == "handoff":      # q, k are the rotated copies; dq, dk come back un-rotated
            dq, dk, dv = swa_backward_rot(q, k, v, o, lse, do, rope, *ctx.win)
        elif ctx.mode == "prerotate":  # q, k are the rotated copies
            from .fused_rope2d import rope2d_apply_
            dq, dk, dv = swa_backward(q, k, v, o, lse, do, None, *ctx.win)
            dq, dk = (t if t.is_contiguous() else t.contiguous() for t in (dq, dk))
            rope2d_apply_(_flat3(dq), *rope, inverse=True)
            rope2d_apply_(_flat3(dk), *rope, inverse=True)
        else:
            dq, dk, dv = swa_backward(q, k, v, o, lse, do, rope, *ctx.win)
        return (dq, dk, dv) + (None,) * 9


class TiledSwaPackedQKV(torch.autograd.Function):
    """The op between a packed QKV projection and the output projection, without the
    permute / contiguous copies either side of it.

    ``TiledSwaPackedQKV.apply(qkv, idx, row_cs_buffer, col_cs_buffer, b_size, t_height,
    t_width, row_size, col_size, sm_scale)`` takes ``qkv [B, N, 3, H, d]`` -- the output of
    one ``Linear(C, 3*H*d)`` viewed, the layout the reference's RoPE self-test slices its
    strided q and k from (src/fused_rope2d.py:259-262) -- and returns ``o [B, N, H*d]``,
    the layout the output projection consumes.  The kernels read q, k, v through strided
    tensor maps and write O, and in backward the three slices of one packed
    ``[B, N, 3, H, d]`` gradient, in place; ``idx`` may be ``None`` (no rotation).
    Same mathematics as ``TiledSwaRope2D`` on the permuted views.
    """

    @staticmethod
    def forward(ctx, qkv, idx: Optional[torch.Tensor], row_cs_buffer, col_cs_buffer, b_size: int, t_height: int,
                t_width: int, row_size: int, col_size: int, sm_scale: float):
        if qkv.dim() != 5 or qkv.shape[2] != 3:
            raise ValueError("expected qkv [B, N, 3, H, d]")
        B, N, _, H, d = qkv.shape
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        rope = None if idx is None else (idx, row_cs_buffer, col_cs_buffer)
        o_buf = torch.empty((B, N, H, d), dtype=qkv.dtype, device=qkv.device)
        win = (b_size, t_height, t_width, row_size, col_size, sm_scale)
        ctx.handoff = _mode_for(q, v, rope, win) == "handoff"
        if ctx.handoff:   # the rotated copies ([B,H,N,d]) are kept for backward; v is still read from the packed tensor
            _, lse, q_rot, k_rot = swa_forward_rot(q, k, v, rope, *win, out=o_buf.permute(0, 2, 1, 3))
            saved = (qkv, lse, o_buf, idx, row_cs_buffer, col_cs_buffer, q_rot, k_rot)
        else:
            _, lse = swa_forward(q, k, v, rope, *win, out=o_buf.permute(0, 2, 1, 3))
            saved = (qkv, lse, o_buf) if rope is None else (qkv, lse, o_buf, idx, row_cs_buffer, col_cs_buffer)
        ctx.save_for_backward(*saved)
        ctx.win = win
        return o_buf.view(B, N, H * d)

    @staticmethod
    def backward(ctx, do):
        saved = ctx.saved_tensors
        qkv, lse, o_buf = saved[:3]
        rope = tuple(saved[3:6]) if len(saved) >= 6 else None
        B, N, _, H, d = qkv.shape
        if do.stride(-1) != 1 or do.stride(1) % 8 or do.stride(0) % 8 or do.data_ptr() % 16:
            do = do.contiguous()
        do4 = do.view(B, N, H, d).permute(0, 2, 1, 3)
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        dqkv = torch.empty((B, N, 3, H, d), dtype=qkv.dtype, device=qkv.device)
        outs = tuple(dqkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        if ctx.handoff:
            swa_backward_rot(saved[6], saved[7], v, o_buf.permute(0, 2, 1, 3), lse, do4, rope, *ctx.win, out=outs)
        else:
            swa_backward(q, k, v, o_buf.permute(0, 2, 1, 3), lse, do4, rope, *ctx.win, out=outs)
        return (dqkv,) + (None,) * 9
