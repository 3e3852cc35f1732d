"""The CPU oracle against the stored outputs of the reference's own functions."""
import pytest
import torch

from conftest import SWA_GOLDEN_CASES, load_golden
from oracle import swa_oracle as orc


def _args(m):
    return (m["b_size"], m["t_height"], m["t_width"], m["row_size"], m["col_size"])


@pytest.mark.parametrize("name", SWA_GOLDEN_CASES)
def test_fused_oracle_matches_reference_outputs(name):
    g = load_golden(name)
    m = g["meta"]
    idx = g.get("idx")
    o, dq, dk, dv = orc.fused_ref(g["q"], g["k"], g["v"], g["do"], idx, g.get("row_cs"), g.get("col_cs"),
                                  *_args(m), g["sm_scale"])
    for mine, ref in ((o, g["o"]), (dq, g["dq"]), (dk, g["dk"]), (dv, g["dv"])):
        assert orc.max_abs(mine, ref) < 2e-5
        assert orc.mean_rel(mine, ref) < 1e-5


@pytest.mark.parametrize("name", SWA_GOLDEN_CASES)
def test_windowed_form_equals_dense_form(name):
    g = load_golden(name)
    m = g["meta"]
    q, k, v, do = (g[x].double() for x in ("q", "k", "v", "do"))
    dense = orc.fused_ref(q, k, v, do, None, None, None, *_args(m), g["sm_scale"])
    win = orc.fused_ref(q, k, v, do, None, None, None, *_args(m), g["sm_scale"], windowed=True)
    for a, b in zip(dense, win):
        assert orc.max_abs(a, b) < 1e-10


def test_sdpa_form_equals_written_out_form():
    g = load_golden("cfg1_16x16_d32_w7_fp32")
    m = g["meta"]
    a = orc.tiled_swa_ref(g["q"], g["k"], g["v"], *_args(m), g["sm_scale"])
    b = orc.tiled_swa_ref_sdpa(g["q"], g["k"], g["v"], *_args(m), g["sm_scale"])
    assert orc.max_abs(a, b) < 1e-5


def test_rope_selftest_layout():
    g = load_golden("rope_selftest_layout")
    y = orc.rope2d_ref(g["q"], g["idx"], g["row_cs"], g["col_cs"])
    assert orc.max_abs(y, g["y"]) < 1e-6
    gq = orc.rope2d_ref(g["gy"], g["idx"], g["row_cs"], g["col_cs"], inverse=True)
    assert orc.max_abs(gq, g["gq"]) < 1e-6
    # tokens without an index pass through unchanged
    assert torch.equal(y[:, 64:], g["q"][:, 64:])


def test_rope_inverse_is_inverse():
    R, N = 4, 30
    idx = orc.encode_idx(5, 6)
    idx[7] = -1
    x = torch.randn(2, N, 24, dtype=torch.float64)
    t = orc.make_cs_table(R, 8).double()
    y = orc.rope2d_ref(x, idx, t, t)
    assert orc.max_abs(orc.rope2d_ref(y, idx, t, t, inverse=True), x) < 1e-6   # fp32 table: cos^2+sin^2 = 1 to ~1e-7
    assert torch.equal(y[..., 16:], x[..., 16:])


def test_encode_idx_and_table():
    idx = orc.encode_idx(3, 4)
    assert idx.dtype == torch.int32 and idx.tolist()[:5] == [0, 1, 2, 3, 1 << 16]
    t = orc.make_cs_table(8, 16, 10000.0)
    assert t.shape == (16, 8, 2) and torch.allclose(t[0, :, 0], torch.ones(8)) and float(t[0, :, 1].abs().max()) == 0
    assert abs(float(t[1, 0, 1]) - 0.8414709848) < 1e-6           # sin(1)
    assert abs(float(t[3, 4, 0]) - float(torch.cos(torch.tensor(3 * 10000.0 ** -0.5)))) < 1e-6


def test_flop_convention():
    fwd, bwd = orc.windowed_flops(4, 8, 4096, 1, 6, 6, 64, 64)
    assert abs(fwd - 5.671e9) / 5.671e9 < 1e-3 and bwd == 2.5 * fwd
