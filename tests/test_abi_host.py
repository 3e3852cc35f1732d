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
    return sorted(set(re.findall(r"\b(swa_[a-z_0-9]+|rope2d_apply)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = header_symbols()
    assert set(names) == set(_lib.EXPORTS)
    for n in names:
        assert hasattr(_lib.lib, n), n
    assert _lib.lib.swa_version() == 1


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
