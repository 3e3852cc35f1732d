"""Host-side checks that need no GPU: the shared library loads, exports every
symbol the header declares, and rejects bad arguments before any launch."""
import ctypes as C
import os
import re

import pytest
import torch

from conftest import ROOT

import dl_templates_b200 as swa
from dl_templates_b200 import _lib
from dl_templates_b200.sharding import bh_range, shard_bh


def header_symbols():
    text = open(os.path.join(ROOT, "include", "swa2d.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(swa_[a-z_0-9]+|rope2d_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = header_symbols()
    assert set(names) == set(_lib.EXPORTS)
    for n in names:
        assert hasattr(_lib.lib, n), n
    assert _lib.lib.swa_version() == 2


def _geom(**kw):
    base = dict(dtype=torch.bfloat16, B=1, H=1, b_size=1, t_height=4, t_width=4, row_size=1, col_size=1, d_qk=64,
                d_v=64, sm_scale=1.0)
    base.update(kw)
    return _lib.make_geom(**base)


def test_rejects_bad_geometry_before_launch():
    g = _geom(d_qk=0)
    assert _lib.lib.swa_select_impl(C.byref(g), None, 0) < 0
    assert b"head dims" in _lib.lib.swa_last_error()
    g = _geom(row_size=-1)
    assert _lib.lib.swa_select_impl(C.byref(g), None, 0) < 0
    g = _geom(t_height=0)
    assert _lib.lib.swa_select_impl(C.byref(g), None, 0) < 0
    g = _geom()
    g.dtype = 7
    assert _lib.lib.swa_select_impl(C.byref(g), None, 0) < 0
    assert b"dtype" in _lib.lib.swa_last_error()


def test_rejects_null_tensors_before_launch():
    g = _geom()
    t = _lib.Tensor4()
    code = _lib.lib.swa_fwd(C.byref(g), None, C.byref(t), C.byref(t), C.byref(t), C.byref(t), None, None, None)
    assert code < 0 and b"NULL" in _lib.lib.swa_last_error()
    with pytest.raises(RuntimeError, match="NULL"):
        _lib.check(code, "swa_fwd")


def test_rejects_bad_rope():
    g = _geom(d_qk=32)
    idx = torch.zeros(16, dtype=torch.int32)
    tab = torch.zeros(4, 16, 2)
    r = _lib.make_rope(idx, tab, tab)  # 4*16 = 64 > d_qk
    assert _lib.lib.swa_select_impl(C.byref(g), C.byref(r), 0) < 0
    assert b"n_rdim" in _lib.lib.swa_last_error()


def test_cpu_tensors_raise():
    q = torch.zeros(1, 1, 16, 32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        swa.tiled_swa_fwd(q, q, q, 1, 4, 4, 1, 1)
    with pytest.raises(RuntimeError, match="no CPU path"):
        swa.rope2d_apply_(torch.zeros(1, 16, 32), torch.zeros(16, dtype=torch.int32), torch.zeros(4, 4, 2),
                          torch.zeros(4, 4, 2))


def test_unsupported_dtype_raises():
    with pytest.raises(TypeError):
        _lib.dtype_code(torch.float64)


def test_encode_idx_matches_reference_packing():
    idx = swa.FusedInplaceRotaryPositionEncoding2D.encode_idx(3, 5)
    assert idx.dtype == torch.int32 and idx.shape == (15,)
    assert idx[7].item() == (1 << 16) | 2


def test_module_tables():
    m = swa.FusedInplaceRotaryPositionEncoding2D(32, 16, 24)
    assert m.row_buffer.cs_components.shape == (16, 16, 2)
    assert m.col_buffer.cs_components.shape == (24, 16, 2)


def test_bh_range_partitions():
    for n, w in ((256, 8), (32, 4), (7, 3), (2, 4)):
        seen = []
        for r in range(w):
            lo, hi = bh_range(n, r, w)
            seen += list(range(lo, hi))
        assert seen == list(range(n))
    x = torch.arange(2 * 3 * 4 * 5).reshape(2, 3, 4, 5)
    parts = [shard_bh(x, r, 4) for r in range(4)]
    assert torch.equal(torch.cat([p.squeeze(0) for p in parts]), x.reshape(6, 4, 5))


def _plan(g, r, which):
    out = (C.c_int32 * 12)()
    code = _lib.lib.swa_describe_plan(C.byref(g), None if r is None else C.byref(r), which, out)
    return code, list(out)


def test_every_tile_plan_fits_shared_and_tensor_memory():
    """Sweep geometries through the planner (host only) and check the resource invariants the kernels rely on:
    the layout fits the dynamic shared memory it asks for, that stays within 227 KB, tensor memory within its
    512 columns, blocks are multiples of 16 tokens of at most 128, and the ring has at least two stages."""
    idx = torch.zeros(16, dtype=torch.int32)
    n_plans = 0
    for d_qk, d_v in ((64, 64), (128, 64), (64, 128), (128, 128), (32, 32), (32, 96), (96, 64)):
        for n_rdim, max_hw in ((0, 0), (8, 16), (16, 128), (32, 128), (32, 1024)):
            if 4 * n_rdim > d_qk:
                continue
            r = None
            if n_rdim:
                tab = torch.zeros(max_hw, n_rdim, 2)
                r = _lib.make_rope(idx, tab, tab)
            for (th, tw, bs) in ((128, 128, 1), (32, 32, 1), (16, 16, 4), (24, 40, 1), (9, 7, 2), (64, 16, 2)):
                for (rs, cs) in ((1, 1), (3, 3), (6, 6), (13, 13), (2, 9), (20, 4)):
                    for dt in (torch.bfloat16, torch.float16):
                        g = _geom(dtype=dt, b_size=bs, t_height=th, t_width=tw, row_size=rs, col_size=cs, d_qk=d_qk,
                                  d_v=d_v)
                        for which in ((0, 1, 2) if r is None else (0, 1, 2, 3, 4, 5)):
                            code, p = _plan(g, r, which)
                            if code != 0:
                                if which < 3:
                                    assert _lib.lib.swa_select_impl(C.byref(g), None if r is None else C.byref(r),
                                                                    which) != _lib.IMPL_TC
                                continue
                            th_, tw_, kr, kw, n, stages, nsb, nxb, tab_b, req, used, tmem = p
                            what = (d_qk, d_v, n_rdim, max_hw, th, tw, bs, rs, cs, which, p)
                            assert th_ * tw_ == 128 and th_ + tw_ <= 32, what
                            assert n == kr * kw and n % 16 == 0 and 16 <= n <= 128, what
                            assert 2 <= stages <= 8 and 2 <= nsb <= 4 and 1 <= nxb <= 2, what
                            assert used <= req <= 227 * 1024, what
                            assert tmem <= 512, what
                            assert (tab_b > 0) <= (n_rdim > 0), what
                            n_plans += 1
    assert n_plans > 500


def test_head_dims_the_tensor_core_kernels_take():
    """32, 64, 96, 128 where no streamed row is rotated (no RoPE, or the entries that take rotated copies); 64 and
    128 only for the kernels that rotate what they stream; anything else runs on the SIMT kernels."""
    idx = torch.zeros(16, dtype=torch.int32)
    tab = torch.zeros(64, 8, 2)
    r = _lib.make_rope(idx, tab, tab)
    out = (C.c_int32 * 12)()
    for d, plain, streamed in ((32, True, False), (64, True, True), (96, True, False), (128, True, True), (48, False, False),
                               (16, False, False), (160, False, False)):
        g = _geom(d_qk=d, d_v=d)
        assert (_lib.lib.swa_select_impl(C.byref(g), None, 0) == _lib.IMPL_TC) == plain, d
        if 32 <= d:
            assert (_lib.lib.swa_select_impl(C.byref(g), C.byref(r), 0) == _lib.IMPL_TC) == streamed, d
            assert (_lib.lib.swa_describe_plan(C.byref(g), C.byref(r), 3, out) == 0) == plain, d


def test_describe_plan_rejects_bad_arguments():
    g = _geom()
    assert _lib.lib.swa_describe_plan(C.byref(g), None, 0, None) < 0
    out = (C.c_int32 * 12)()
    assert _lib.lib.swa_describe_plan(C.byref(g), None, 3, out) < 0      # the hand-off kernels need a RoPE description
    assert _lib.lib.swa_describe_plan(C.byref(g), None, 6, out) < 0
    g32 = _geom(dtype=torch.float32)
    assert _lib.lib.swa_describe_plan(C.byref(g32), None, 0, out) < 0   # fp32 runs on the SIMT kernels


def test_planner_refuses_overrides_beyond_tensor_memory(monkeypatch):
    """The experiment knobs cannot produce a plan that overflows the 512 tensor-memory columns or the barrier
    arrays, or a block narrower than the halo: such a plan is refused on the host instead of being launched.  The
    library reads its knobs once per process, so every change is followed by swa_refresh_env."""
    g = _geom(t_height=128, t_width=128, row_size=6, col_size=6)
    assert _plan(g, None, 1)[0] == 0

    def knobs(**kw):
        for k in ("SWA_TC_NMAX", "SWA_TC_KR", "SWA_TC_KW", "SWA_TC_TH", "SWA_TC_NSB", "SWA_TC_STAGES"):
            monkeypatch.delenv(k, raising=False)
        for k, v in kw.items():
            monkeypatch.setenv("SWA_TC_" + k, str(v))
        _lib.lib.swa_refresh_env()

    try:
        knobs(NMAX=160, KR=8, KW=20, TH=16)
        assert _plan(g, None, 1)[0] < 0 and _plan(g, None, 2)[0] < 0      # 2 pairs x 2 x 160 columns do not fit
        knobs(NMAX=160, KR=8, KW=20, TH=16, NSB=2)
        code, p = _plan(g, None, 0)                                          # forward: 2 x 160 + 128 columns fit
        assert code == 0 and p[4] == 160 and p[11] == 448
        knobs(NMAX=160, KR=8, KW=20, TH=16, NSB=3)
        assert _plan(g, None, 0)[0] < 0
        knobs(TH=16, KR=4, KW=16)                                            # narrower than the 20-column halo
        assert _plan(g, None, 0)[0] < 0
        knobs(STAGES=9)
        assert _plan(g, None, 0)[0] < 0
    finally:
        knobs()
    assert _plan(g, None, 0)[0] == 0


def test_plans_are_cached_and_cheap():
    """The second request for a plan is a map lookup: far below the cost of the search (host-only timing, generous
    bound), and identical to the first."""
    import time
    g = _geom(t_height=96, t_width=80, row_size=5, col_size=7)
    _lib.lib.swa_refresh_env()
    t0 = time.perf_counter()
    first = _plan(g, None, 2)
    t1 = time.perf_counter()
    for _ in range(200):
        again = _plan(g, None, 2)
    t2 = time.perf_counter()
    assert again == first and first[0] == 0
    assert (t2 - t1) / 200 < 20e-6


def test_broadcast_strides_fall_back_to_simt():
    """A 16-bit tensor broadcast over batch or heads (stride 0) cannot be described by a tensor map: AUTO demotes the
    call to the SIMT kernels instead of failing in the map encoder; a forced tensor-core request is rejected."""
    g = _geom(B=2, H=3, t_height=16, t_width=16, row_size=2, col_size=2)
    ok = _lib.Tensor4()
    ok.ptr = 256
    for i, st in enumerate((3 * 256 * 64, 256 * 64, 64, 1)):
        ok.stride[i] = st
    bc = _lib.Tensor4()
    bc.ptr = 256
    for i, st in enumerate((0, 256 * 64, 64, 1)):
        bc.stride[i] = st
    lse = C.c_void_p(512)
    g_tc = _geom(B=2, H=3, t_height=16, t_width=16, row_size=2, col_size=2, impl="tc")
    before = _lib.launch_count()
    code = _lib.lib.swa_fwd(C.byref(g_tc), None, C.byref(bc), C.byref(ok), C.byref(ok), C.byref(ok), lse, None, None)
    assert code < 0 and b"positive strides" in _lib.lib.swa_last_error()
    assert _lib.launch_count() == before


def test_rope_mode_switch():
    """``set_rope_mode`` accepts the three modes (and 'auto' as an alias of the default), returns the previous one,
    rejects anything else; without RoPE a call has no mode (host-only check)."""
    from dl_templates_b200 import tiled_swa as ts
    prev = swa.set_rope_mode("fused")
    try:
        assert swa.set_rope_mode("auto") == "fused"
        assert swa.set_rope_mode("prerotate") == "handoff"
        q = torch.zeros(1, 1, 64 * 64, 64, dtype=torch.bfloat16)
        assert ts._mode_for(q, q, None, (1, 64, 64, 3, 3, 0.1)) == "none"
    finally:
        swa.set_rope_mode(prev)
    with pytest.raises(ValueError):
        swa.set_rope_mode("sometimes")


def test_noalloc_rejects_everything_before_its_first_launch():
    """swa_bwd_noalloc runs every check of the three calls it makes before the first of them: a NULL output, a bad
    RoPE description or a tensor-core request the dK/dV plan cannot serve is a negative return with nothing
    enqueued (the launch counter does not move; no GPU is needed to see that)."""
    g = _geom(t_height=16, t_width=16, row_size=2, col_size=2)
    t = _lib.Tensor4()
    t.ptr = 256
    for i, st in enumerate((16 * 16 * 64, 16 * 16 * 64, 64, 1)):
        t.stride[i] = st
    null = _lib.Tensor4()
    before = _lib.launch_count()
    args = [C.byref(t)] * 5
    lse = C.c_void_p(512)
    ok_outs = [C.byref(t)] * 3
    for bad in range(3):
        outs = list(ok_outs)
        outs[bad] = C.byref(null)
        assert _lib.lib.swa_bwd_noalloc(C.byref(g), None, *args, lse, *outs, None, None) < 0
        assert b"NULL" in _lib.lib.swa_last_error()
    bad_rope = _lib.Rope(1024, 0, 0, 16, 16, 16)                       # tables missing
    assert _lib.lib.swa_bwd_noalloc(C.byref(g), C.byref(bad_rope), *args, lse, *ok_outs, None, None) < 0
    bad_rope = _lib.Rope(1024, 2048, 4096, 24, 16, 16)                 # 4 * n_rdim > d_qk
    assert _lib.lib.swa_bwd_noalloc(C.byref(g), C.byref(bad_rope), *args, lse, *ok_outs, None, None) < 0
    assert _lib.lib.swa_bwd_noalloc(C.byref(g), None, *args, None, *ok_outs, None, None) < 0   # lse NULL
    g_tc = _geom(t_height=16, t_width=16, row_size=2, col_size=2, d_qk=48, impl="tc")          # no tensor-core kernel
    assert _lib.lib.swa_bwd_noalloc(C.byref(g_tc), None, *args, lse, *ok_outs, None, None) < 0
    assert _lib.launch_count() == before


def test_rot_entries_need_a_rope_description():
    """swa_fwd_rot / swa_bwd_*_rot exist for RoPE; without one they point at the plain entry points."""
    g = _geom(t_height=16, t_width=16, row_size=2, col_size=2)
    t = _lib.Tensor4()
    t.ptr = 256
    for i, st in enumerate((16 * 16 * 64, 16 * 16 * 64, 64, 1)):
        t.stride[i] = st
    p = C.c_void_p(512)
    before = _lib.launch_count()
    assert _lib.lib.swa_fwd_rot(C.byref(g), None, *([C.byref(t)] * 4), p, C.byref(t), C.byref(t), None, None) < 0
    assert b"RoPE" in _lib.lib.swa_last_error()
    assert _lib.lib.swa_bwd_dq_rot(C.byref(g), None, *([C.byref(t)] * 4), p, p, C.byref(t), None, None) < 0
    assert _lib.lib.swa_bwd_dkdv_rot(C.byref(g), None, *([C.byref(t)] * 4), p, p, C.byref(t), C.byref(t), None, None) < 0
    rope = _lib.Rope(1024, 2048, 4096, 16, 16, 16)
    assert _lib.lib.swa_fwd_rot(C.byref(g), C.byref(rope), *([C.byref(t)] * 4), p, C.byref(t), C.byref(t), None, None) < 0
    assert b"alias" in _lib.lib.swa_last_error()                      # q_rot / k_rot must be separate tensors
    assert _lib.launch_count() == before
