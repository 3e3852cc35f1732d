"""The allocation-free backward entry point (``swa_bwd_noalloc``) against the regular
three-call backward, through the C ABI.

Some hosts of this library cannot allocate device memory around the op (all of it was
reserved up front by somebody else, or an allocation's device-wide synchronisation is
not acceptable where they run); for them the library keeps the one scratch vector the
backward pass needs in a fixed array of its own.  This file is collected last on
purpose: the entry point shares that array between calls, so its test runs after every
other test has had its turn, and it must pass both alone and after them.
"""
import ctypes as C

import pytest
import torch

from swa_cases import CONFIGS, make_case

import dl_templates_b200 as swa
from dl_templates_b200 import _lib
from dl_templates_b200 import tiled_swa as ts

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_both(cfg_name, B, H, grid=None):
    cfg = dict(CONFIGS[cfg_name])
    if grid:
        cfg["grid"] = grid
    c = make_case(cfg, B=B, H=H)
    rope = tuple(t.to(DEV) for t in (c["idx"], c["row_cs"], c["col_cs"]))
    q, k, v, do = (c[x].to(DEV) for x in ("q", "k", "v", "do"))
    o, lse = swa.swa_forward(q, k, v, rope, *c["win"], c["sm_scale"])
    want = swa.swa_backward(q, k, v, o, lse, do, rope, *c["win"], c["sm_scale"])
    # the caller of the allocation-free entry point brings its own outputs; poison them first
    outs = [torch.full_like(t, float("nan")) for t in (q, k, v)]
    g = ts._geom(q, v, *c["win"], c["sm_scale"], "auto")
    r = _lib.make_rope(*rope)
    t4 = [_lib.tensor4(t) for t in (q, k, v, o, do, *outs)]
    torch.cuda.synchronize()
    n_allocs = lambda: torch.cuda.memory_stats(DEV).get("allocation.all.allocated", 0)   # allocations so far (a count)
    before = n_allocs()
    code = _lib.lib.swa_bwd_noalloc(C.byref(g), C.byref(r), *(C.byref(t) for t in t4[:5]), lse.data_ptr(),
                                    *(C.byref(t) for t in t4[5:]), ts._status(torch.device(DEV)).data_ptr(),
                                    _lib.stream_ptr(torch.device(DEV)))
    assert code == 0, _lib.lib.swa_last_error().decode()
    torch.cuda.synchronize()
    assert n_allocs() == before, "the allocation-free entry point must not allocate device memory"
    swa.check_status()
    return want, outs


def test_noalloc_backward_matches_regular_backward_twice_in_a_row():
    # two calls in a row on different problems: the second sees the first one's leftovers in the scratch
    for cfg_name, B, H, grid in (("cfg2", 1, 3, None), ("cfg1", 1, 2, None), ("cfg4", 1, 2, 32)):
        want, got = _run_both(cfg_name, B, H, grid)
        for w, g_, name in zip(want, got, ("dq", "dk", "dv")):
            assert torch.isfinite(g_.float()).all(), name
            assert torch.equal(w, g_), f"{cfg_name} {name}: differs from the three-call backward"


def test_noalloc_rejects_oversized_problems():
    rows = _lib.NOALLOC_MAX_ROWS
    G = 128
    bh = rows // (G * G) + 1
    g = _lib.make_geom(torch.bfloat16, 1, bh, 1, G, G, 1, 1, 64, 64, 0.125)
    t = _lib.Tensor4()
    code = _lib.lib.swa_bwd_noalloc(C.byref(g), None, *(C.byref(t),) * 5, None, *(C.byref(t),) * 3, None, None)
    assert code < 0 and b"exceeds the built-in scratch" in _lib.lib.swa_last_error()
