"""GPU parity: the CUDA path (through the Python surface over the C ABI) against
the CPU oracle and the stored reference outputs.

Ground truth for bf16/fp16 is the oracle evaluated in fp32 on the rounded inputs.
Tolerances: max-abs 2e-2 and mean-rel 5e-3 for bf16/fp16, 1e-4 for fp32.
"""
import ctypes as C

import pytest
import torch

from conftest import SWA_GOLDEN_CASES, load_golden
from oracle import swa_oracle as orc
from swa_cases import CONFIGS, make_case, tolerances

import dl_templates_b200 as swa

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


PATHS = ["handoff", "fused"]


def run_gpu(q, k, v, do, rope, win, sm_scale, impl="auto", path="fused"):
    """Forward (+ backward when ``do`` is given) through the ABI; returns CPU tensors.

    ``path`` (only matters with RoPE): ``"fused"`` = swa_fwd / swa_bwd_dq / swa_bwd_dkdv, every kernel rotates the rows
    it streams; ``"handoff"`` = swa_fwd_rot / swa_bwd_dq_rot / swa_bwd_dkdv_rot, rotated copies handed from forward to
    backward (the default of the autograd surfaces)."""
    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    rd = None if rope is None else tuple(t.to(DEV) for t in rope)
    if rd is not None and path == "handoff":
        o, lse, q_rot, k_rot = swa.swa_forward_rot(qd, kd, vd, rd, *win, sm_scale, impl=impl)
        outs = [o]
        if do is not None:
            outs += list(swa.swa_backward_rot(q_rot, k_rot, vd, o, lse, do.to(DEV), rd, *win, sm_scale, impl=impl))
        assert torch.equal(qd.cpu(), q) and torch.equal(kd.cpu(), k)       # q and k stay untouched
    else:
        o, lse = swa.swa_forward(qd, kd, vd, rd, *win, sm_scale, impl=impl)
        outs = [o]
        if do is not None:
            outs += list(swa.swa_backward(qd, kd, vd, o, lse, do.to(DEV), rd, *win, sm_scale, impl=impl))
    swa.check_status()
    return [t.float().cpu() for t in outs], lse.cpu()


def assert_close(got, want, dtype, names=("o", "dq", "dk", "dv"), what=""):
    ma, mr = tolerances(dtype)
    for g, w, n in zip(got, want, names):
        assert torch.isfinite(g).all(), f"{what} {n}: non-finite values"
        a, r = orc.max_abs(g, w), orc.mean_rel(g, w)
        assert a < ma and r < mr, f"{what} {n}: max_abs={a:.3e} (<{ma}) mean_rel={r:.3e} (<{mr})"


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("impl", ["auto", "simt"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", SWA_GOLDEN_CASES)
def test_golden_cases(name, dtype, impl, path):
    g = load_golden(name)
    m = g["meta"]
    win = (m["b_size"], m["t_height"], m["t_width"], m["row_size"], m["col_size"])
    q, k, v, do = (g[x].to(dtype) for x in ("q", "k", "v", "do"))
    rope = (g["idx"], g["row_cs"], g["col_cs"]) if "idx" in g else None
    if rope is None and path != PATHS[0]:
        pytest.skip("no RoPE in this case: both paths are the same call")
    got, _ = run_gpu(q, k, v, do, rope, win, g["sm_scale"], impl, path)
    if dtype == torch.float32:
        want = [g["o"], g["dq"], g["dk"], g["dv"]]      # the reference's own stored outputs
    else:
        want = orc.fused_ref(q.float(), k.float(), v.float(), do.float(), *(rope or (None, None, None)), *win,
                             g["sm_scale"])
    assert_close(got, want, dtype, what=f"{name}/{impl}/{path}")


def _config_check(cfg_name, B, H, impl="auto", windowed=False, path="handoff"):
    cfg = CONFIGS[cfg_name]
    c = make_case(cfg, B=B, H=H)
    rope = (c["idx"], c["row_cs"], c["col_cs"])
    do = c["do"] if cfg["bwd"] else None
    got, lse = run_gpu(c["q"], c["k"], c["v"], do, rope, c["win"], c["sm_scale"], impl, path)
    f = lambda t: None if t is None else t.float()
    want = orc.fused_ref(f(c["q"]), f(c["k"]), f(c["v"]), f(do), *rope, *c["win"], c["sm_scale"], windowed=windowed)
    if do is None:
        want = [want]
    assert_close(got, want, cfg["dtype"], what=f"{cfg_name}/{impl}/{path}")
    return got


@pytest.mark.parametrize("path", PATHS)
def test_config1_fp32_full(path):
    _config_check("cfg1", None, None, path=path)


@pytest.mark.parametrize("path", PATHS)
def test_config2_bf16_forward_full(path):
    _config_check("cfg2", None, None, path=path)


@pytest.mark.parametrize("path", PATHS)
def test_config3_fp16_dropped_idx(path):
    # 8 of the 96 (batch, head) slices: the dense oracle is O(N^2) per slice
    _config_check("cfg3", 2, 4, path=path)


@pytest.mark.parametrize("path", PATHS)
def test_config4_mixed_dims_slices(path):
    _config_check("cfg4", 1, 2, windowed=True, path=path)


@pytest.mark.parametrize("path", PATHS)
def test_target_config_slices(path):
    _config_check("target", 1, 2, windowed=True, path=path)


def test_lse_matches_oracle():
    c = make_case(CONFIGS["cfg1"])
    rope = (c["idx"], c["row_cs"], c["col_cs"])
    _, lse = run_gpu(c["q"], c["k"], c["v"], None, rope, c["win"], c["sm_scale"])
    qr = orc.rope2d_ref(c["q"], c["idx"], c["row_cs"], c["col_cs"])
    kr = orc.rope2d_ref(c["k"], c["idx"], c["row_cs"], c["col_cs"])
    _, want = orc.tiled_swa_ref(qr, kr, c["v"], *c["win"], c["sm_scale"], return_lse=True)
    assert orc.max_abs(lse * 0.6931471805599453, want) < 1e-4


def test_autograd_surface_matches_reference_order():
    """TiledSwa.apply / TiledSwaRope2D.apply / RotaryPE2D.apply compose as in the reference."""
    g = load_golden("g5x7_r2c1_partial_rope_drop")
    m = g["meta"]
    win = (m["b_size"], m["t_height"], m["t_width"], m["row_size"], m["col_size"])
    idx, rcs, ccs = (g[x].to(DEV) for x in ("idx", "row_cs", "col_cs"))
    want = [g["o"], g["dq"], g["dk"], g["dv"]]
    # (a) fused entry
    q, k, v = (g[x].to(DEV).requires_grad_(True) for x in ("q", "k", "v"))
    o = swa.TiledSwaRope2D.apply(q, k, v, idx, rcs, ccs, *win, g["sm_scale"])
    o.backward(g["do"].to(DEV))
    assert_close([t.detach().cpu() for t in (o, q.grad, k.grad, v.grad)], want, torch.float32, what="fused")
    # (b) the reference's own composition: in-place RoPE on q and k, then TiledSwa
    q, k, v = (g[x].to(DEV).requires_grad_(True) for x in ("q", "k", "v"))
    B, H, N, D = q.shape
    qr = swa.RotaryPE2D.apply(q.clone().reshape(B * H, N, D), idx, rcs, ccs).reshape(B, H, N, D)
    kr = swa.RotaryPE2D.apply(k.clone().reshape(B * H, N, D), idx, rcs, ccs).reshape(B, H, N, D)
    o = swa.TiledSwa.apply(qr, kr, v, *win, g["sm_scale"])
    o.backward(g["do"].to(DEV))
    assert_close([t.detach().cpu() for t in (o, q.grad, k.grad, v.grad)], want, torch.float32, what="composed")
    swa.check_status()


def test_strided_inputs():
    """q, k, v as strided views of one packed projection output [B, N, 3, H, d]."""
    torch.manual_seed(0)
    B, H, G, d = 2, 3, 12, 64
    N = G * G
    packed = torch.randn(B, N, 3, H, d).to(torch.bfloat16)
    q, k, v = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    assert not q.is_contiguous()
    do = torch.randn(B, H, N, d).to(torch.bfloat16)
    win = (1, G, G, 2, 2)
    pd = packed.to(DEV)
    qd, kd, vd = (pd[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    o, lse = swa.swa_forward(qd, kd, vd, None, *win, 0.125)
    dq, dk, dv = swa.swa_backward(qd, kd, vd, o, lse, do.to(DEV), None, *win, 0.125)
    swa.check_status()
    want = orc.fused_ref(q.float(), k.float(), v.float(), do.float(), None, None, None, *win, 0.125)
    assert_close([t.float().cpu() for t in (o, dq, dk, dv)], want, torch.bfloat16, what="strided")


@pytest.mark.parametrize("path", PATHS)
def test_bitwise_determinism(path):
    c = make_case(CONFIGS["cfg2"], B=1, H=2)
    rope = (c["idx"], c["row_cs"], c["col_cs"])
    a, _ = run_gpu(c["q"], c["k"], c["v"], c["do"], rope, c["win"], c["sm_scale"], path=path)
    b, _ = run_gpu(c["q"], c["k"], c["v"], c["do"], rope, c["win"], c["sm_scale"], path=path)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_rows_of_p_sum_to_one_and_linearity_in_v():
    """Size-independent properties on a full-size grid: with v = 1 the output is 1;
    the output is linear in v."""
    cfg = CONFIGS["target"]
    c = make_case(cfg, B=1, H=4)
    rope = tuple(t.to(DEV) for t in (c["idx"], c["row_cs"], c["col_cs"]))
    q, k, v = (c[x].to(DEV) for x in ("q", "k", "v"))
    ones = torch.ones_like(v)
    o1, _ = swa.swa_forward(q, k, ones, rope, *c["win"], c["sm_scale"])
    assert (o1.float() - 1).abs().max().item() < 1e-2
    v2 = torch.roll(v, 1, dims=2)
    oa, _ = swa.swa_forward(q, k, v, rope, *c["win"], c["sm_scale"])
    ob, _ = swa.swa_forward(q, k, v2, rope, *c["win"], c["sm_scale"])
    oc, _ = swa.swa_forward(q, k, (2 * v.float() + v2.float()).to(v.dtype), rope, *c["win"], c["sm_scale"])
    swa.check_status()
    assert (oc.float() - (2 * oa.float() + ob.float())).abs().max().item() < 6e-2


@pytest.mark.parametrize("path", PATHS)
def test_batch_head_slices_are_independent(path):
    """A sharded run must equal the unsharded one bitwise: computing slices [2:4) alone
    gives the same bits as those slices of the full call."""
    c = make_case(CONFIGS["cfg2"], B=1, H=4)
    rope = (c["idx"], c["row_cs"], c["col_cs"])
    full, _ = run_gpu(c["q"], c["k"], c["v"], c["do"], rope, c["win"], c["sm_scale"], path=path)
    part, _ = run_gpu(c["q"][:, 2:4], c["k"][:, 2:4], c["v"][:, 2:4], c["do"][:, 2:4], rope, c["win"], c["sm_scale"],
                      path=path)
    for x, y in zip(full, part):
        assert torch.equal(x[:, 2:4], y)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("b_size,G,wr,wc", [(2, 10, 2, 1), (4, 9, 1, 1), (16, 6, 1, 1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_tiles_of_several_tokens_on_the_tensor_core_path(b_size, G, wr, wc, dtype, path):
    """b_size > 1 (the reference's own regime is 16): every token of a tile attends every token of
    the tiles in the window; RoPE indices are per token (tokens of a tile share its coordinates)."""
    torch.manual_seed(b_size)
    B, H, d = 1, 2, 64
    N = G * G * b_size
    q, k, v, do = (torch.randn(B, H, N, d).to(dtype) for _ in range(4))
    rows = torch.arange(G)[:, None, None].expand(G, G, b_size)
    cols = torch.arange(G)[None, :, None].expand(G, G, b_size)
    idx = ((rows << 16) | cols).reshape(-1).to(torch.int32)
    idx[5] = -1
    tab = orc.make_cs_table(8, G)
    rope = (idx, tab, tab.clone())
    win = (b_size, G, G, wr, wc)
    qd, vd = q.to(DEV), v.to(DEV)
    assert swa.selected_impl(qd, vd, tuple(t.to(DEV) for t in rope), *win, 0.125) == "tc"
    got, _ = run_gpu(q, k, v, do, rope, win, 0.125, path=path)
    want = orc.fused_ref(q.float(), k.float(), v.float(), do.float(), *rope, *win, 0.125)
    assert_close(got, want, dtype, what=f"b_size={b_size}/{path}")


@pytest.mark.parametrize("path", PATHS)
def test_config5_geometry_on_a_smaller_grid(path):
    """d_qk = d_v = 128, 31x31 window, RoPE on all 128 dims (n_rdim 32) as in the largest configuration,
    on a 96x96 grid the windowed oracle finishes in seconds."""
    cfg = dict(CONFIGS["cfg5"])
    cfg["grid"] = 96
    c = make_case(cfg, B=1, H=1)
    rope = (c["idx"], c["row_cs"], c["col_cs"])
    got, _ = run_gpu(c["q"], c["k"], c["v"], c["do"], rope, c["win"], c["sm_scale"], path=path)
    want = orc.fused_ref(*(c[x].float() for x in ("q", "k", "v", "do")), *rope, *c["win"], c["sm_scale"], windowed=True)
    assert_close(got, want, cfg["dtype"], what=f"cfg5 geometry/{path}")


@pytest.mark.parametrize("path", PATHS)
def test_config5_full_size_against_oracle_on_cropped_bands(path):
    """The largest configuration at its stated size (256 x 256 grid, d = 128, 31 x 31 window, RoPE on all 128 dims,
    one (batch, head) slice) on the tensor-core kernels, compared with the oracle on three bands of grid rows (top
    border, interior, bottom border).  The window is truncated at the border, not shifted
    (src/tiled_swa.py:704-710), so the oracle evaluated on the rows [a - 30, b + 30) of the grid -- with the
    tokens' own packed indices, so the RoPE angles are those of the full grid -- reproduces the full-grid O, dQ
    (15 rows of reach) and dK, dV (15 more) of rows [a, b) exactly."""
    cfg = CONFIGS["cfg5"]
    G, half = cfg["grid"], (cfg["w"] - 1) // 2
    c = make_case(cfg, B=1, H=1)
    rope = (c["idx"], c["row_cs"], c["col_cs"])
    assert swa.selected_impl(c["q"].to(DEV), c["v"].to(DEV), tuple(t.to(DEV) for t in rope), *c["win"], c["sm_scale"],
                             which=2) == "tc"
    got, _ = run_gpu(c["q"], c["k"], c["v"], c["do"], rope, c["win"], c["sm_scale"], path=path)
    for a, b in ((0, 24), (116, 140), (G - 24, G)):
        lo, hi = max(0, a - 2 * half), min(G, b + 2 * half)
        rows = slice(lo * G, hi * G)
        crop = [c[x][:, :, rows].float() for x in ("q", "k", "v", "do")]
        want = orc.fused_ref(*crop, c["idx"][rows], c["row_cs"], c["col_cs"], 1, hi - lo, G, half, half, c["sm_scale"],
                             windowed=True)
        keep = slice((a - lo) * G, (b - lo) * G)
        full = slice(a * G, b * G)
        assert_close([t[:, :, full] for t in got], [t[:, :, keep] for t in want], cfg["dtype"],
                     what=f"cfg5 rows [{a},{b})/{path}")


def test_config5_full_grid_properties():
    """Full 256x256 grid of the largest configuration on two (batch, head) slices: with v = 1 the
    output is 1 (rows of P sum to 1 for all 65 536 queries, borders included), gradients are finite,
    dV sums to the sum of dO over the grid (columns of P^T dO), and two runs agree bitwise."""
    cfg = CONFIGS["cfg5"]
    c = make_case(cfg, B=1, H=2)
    rope = tuple(t.to(DEV) for t in (c["idx"], c["row_cs"], c["col_cs"]))
    q, k, do = (c[x].to(DEV) for x in ("q", "k", "do"))
    ones = torch.ones_like(c["v"]).to(DEV)
    o, lse = swa.swa_forward(q, k, ones, rope, *c["win"], c["sm_scale"])
    assert (o.float() - 1).abs().max().item() < 1e-2
    dq, dk, dv = swa.swa_backward(q, k, ones, o, lse, do, rope, *c["win"], c["sm_scale"])
    dq2, dk2, dv2 = swa.swa_backward(q, k, ones, o, lse, do, rope, *c["win"], c["sm_scale"])
    swa.check_status()
    for a, b in ((dq, dq2), (dk, dk2), (dv, dv2)):
        assert torch.isfinite(a.float()).all() and torch.equal(a, b)
    # sum_k dV[k, :] = sum_q (sum_k P[q, k]) dO[q, :] = sum_q dO[q, :]
    lhs, rhs = dv.double().sum(2), do.double().sum(2)
    rel = ((lhs - rhs).norm() / rhs.norm()).item()
    assert rel < 1e-2, rel


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("grid,w", [((21, 21), 7), ((37, 19), 5), ((9, 50), 9)])
def test_ragged_grids_tensor_core_path(grid, w, dtype, path="fused"):
    """Grids that are no multiple of the resident tile in rows or columns (partly empty tiles, one-block
    items), RoPE with dropped tokens and tokens whose row or column half alone is -1, forward + backward
    on the tcgen05 kernels against the oracle."""
    th, tw = grid
    N = th * tw
    q, k, v, do = orc.seeded_inputs(1, 3, N, 64, 64, dtype, 7)
    idx = orc.encode_idx(th, tw)
    gsel = torch.Generator().manual_seed(11)
    r = torch.rand(N, generator=gsel)
    idx[r < 0.05] = -1                                              # token not rotated at all
    row_only = (r >= 0.05) & (r < 0.10)
    idx[row_only] = (idx[row_only] & ~0xFFFF) | 0xFFFF              # column half -1: only the row angle applies
    col_only = (r >= 0.10) & (r < 0.15)
    idx[col_only] = idx[col_only] | -65536                          # row half -1
    idx = idx.to(torch.int32)
    tab_r, tab_c = orc.make_cs_table(16, th, 10000.0), orc.make_cs_table(16, tw, 10000.0)
    half = (w - 1) // 2
    win = (1, th, tw, half, half)
    rope = (idx, tab_r, tab_c)
    assert swa.selected_impl(q.to(DEV), v.to(DEV), tuple(t.to(DEV) for t in rope), *win, 0.125, which=1, impl="auto") == "tc"
    want = orc.fused_ref(q.float(), k.float(), v.float(), do.float(), *rope, *win, 0.125)
    for path in PATHS:
        got, _ = run_gpu(q, k, v, do, rope, win, 0.125, impl="tc", path=path)
        assert_close(got, want, dtype, what=f"ragged {grid}/{path}")


def test_random_shapes_tensor_core_vs_simt():
    """48 seeded random shapes (grid, b_size, window, head dims, dtype, RoPE width, dropped indices): wherever
    the tcgen05 kernels take the shape they must agree with the fp32-accumulate SIMT kernels (which the other
    tests pin to the oracle) to within the 16-bit rounding of the outputs; nothing may hang or be non-finite."""
    import random
    rnd = random.Random(3)
    n_tc = n_oracle = 0
    for case in range(48):
        th, tw = rnd.choice([5, 9, 16, 23, 31, 40, 47]), rnd.choice([6, 8, 13, 16, 24, 33, 50])
        b = rnd.choice([1, 1, 1, 2, 4])
        wr, wc = rnd.choice([0, 1, 2, 3, 6, 7, 12]), rnd.choice([0, 1, 2, 3, 6, 10])
        dqk, dv = rnd.choice([64, 64, 128]), rnd.choice([64, 64, 128])
        dtype = rnd.choice([torch.bfloat16, torch.float16])
        H = rnd.choice([1, 2, 3])
        R = rnd.choice([0, 8, 16, 32]) if dqk == 128 else rnd.choice([0, 8, 16])
        N = th * tw * b
        g = torch.Generator().manual_seed(100 + case)
        q, k = (torch.randn(1, H, N, dqk, generator=g).to(dtype).to(DEV) for _ in range(2))
        v, do = (torch.randn(1, H, N, dv, generator=g).to(dtype).to(DEV) for _ in range(2))
        rope = None
        if R:
            idx = orc.encode_idx(th, tw * b)
            idx[torch.rand(N, generator=g) < 0.05] = -1
            rope = (idx.to(DEV), orc.make_cs_table(R, max(th, 2)).to(DEV), orc.make_cs_table(R, max(tw * b, 2)).to(DEV))
        win, sc = (b, th, tw, wr, wc), dqk ** -0.5
        what = f"case {case}: grid {th}x{tw} b{b} w({wr},{wc}) d{dqk}/{dv} {dtype} R{R}"
        if swa.selected_impl(q, v, rope, *win, sc, which=2, impl="auto") != "tc":
            continue
        n_tc += 1
        o1, l1 = swa.swa_forward(q, k, v, rope, *win, sc, impl="simt")
        g1 = swa.swa_backward(q, k, v, o1, l1, do, rope, *win, sc, impl="simt")
        o2, _ = swa.swa_forward(q, k, v, rope, *win, sc, impl="tc")
        g2 = swa.swa_backward(q, k, v, o1, l1, do, rope, *win, sc, impl="tc")
        swa.check_status()
        for a, c, n in zip((o1, *g1), (o2, *g2), ("o", "dq", "dk", "dv")):
            assert torch.isfinite(c.float()).all(), f"{what} {n}: non-finite"
            err = (a.float() - c.float()).abs().max().item()
            assert err < 4e-2, f"{what} {n}: max abs {err:.3e}"
        if n_tc % 2 == 0 and N <= 3000 and wr + wc > 0:      # (a 1 x 1 window has dq = dk = 0: no relative error to speak of)
            # every second shape the tensor-core kernels take also goes to the oracle (windowed form of the same
            # arithmetic), on both paths: d_qk != d_v with 32 rotated pairs, wr != wc up to 12 / 10, three heads
            rope_cpu = (None, None, None) if rope is None else tuple(t.cpu() for t in rope)
            want = orc.fused_ref(q.float().cpu(), k.float().cpu(), v.float().cpu(), do.float().cpu(), *rope_cpu, *win, sc,
                                 windowed=True)
            for path in (PATHS if rope is not None else PATHS[:1]):
                got, _ = run_gpu(q.cpu(), k.cpu(), v.cpu(), do.cpu(), None if rope is None else rope_cpu, win, sc,
                                 impl="tc", path=path)
                assert_close(got, want, dtype, what=f"{what} vs oracle/{path}")
                n_oracle += 1
    assert n_tc >= 30 and n_oracle >= 12


def test_host_pipeline_matches_direct_calls():
    """Chunked, stream-pipelined host-buffer path (uneven last chunk, buffers reused) == direct calls, bitwise."""
    from dl_templates_b200.host_pipeline import HostPipeline
    c = make_case(CONFIGS["cfg2"], B=1, H=7)
    rope = tuple(t.to(DEV) for t in (c["idx"], c["row_cs"], c["col_cs"]))
    direct, _ = run_gpu(c["q"], c["k"], c["v"], c["do"], (c["idx"], c["row_cs"], c["col_cs"]), c["win"], c["sm_scale"],
                        path="handoff")
    host_in = [c[x].pin_memory() for x in ("q", "k", "v", "do")]
    outs = [torch.empty_like(c[x]).pin_memory() for x in ("v", "q", "k", "v")]
    pipe = HostPipeline(DEV, chunk_slices=2)
    for _ in range(2):                      # second run reuses the staging buffers
        pipe.run(*host_in, outs, rope, c["win"], c["sm_scale"])
        torch.cuda.synchronize()
    swa.check_status()
    for got, want in zip(outs, direct):
        assert torch.equal(got.float(), want)


def test_host_pipeline_back_to_back_runs_do_not_race():
    """Two runs on DIFFERENT inputs with nothing between them but the enqueue order: the copies of the second run into
    the staging buffers must wait for the kernels of the first run that still read them."""
    from dl_templates_b200.host_pipeline import HostPipeline
    c = make_case(CONFIGS["cfg2"], B=1, H=6)
    rope_cpu = (c["idx"], c["row_cs"], c["col_cs"])
    rope = tuple(t.to(DEV) for t in rope_cpu)
    ins_a = [c[x] for x in ("q", "k", "v", "do")]
    ins_b = [torch.roll(t, 1, dims=1) * 0.5 for t in ins_a]
    want_a, _ = run_gpu(*ins_a[:3], ins_a[3], rope_cpu, c["win"], c["sm_scale"], path="handoff")
    want_b, _ = run_gpu(*ins_b[:3], ins_b[3], rope_cpu, c["win"], c["sm_scale"], path="handoff")
    host_a, host_b = ([t.pin_memory() for t in ins] for ins in (ins_a, ins_b))
    outs_a, outs_b = ([torch.empty_like(c[x]).pin_memory() for x in ("v", "q", "k", "v")] for _ in range(2))
    pipe = HostPipeline(DEV, chunk_slices=2, n_buffers=2)
    for _ in range(3):
        pipe.run(*host_a, outs_a, rope, c["win"], c["sm_scale"])
        pipe.run(*host_b, outs_b, rope, c["win"], c["sm_scale"])
    torch.cuda.synchronize()
    swa.check_status()
    for got, want in zip(outs_a + outs_b, want_a + want_b):
        assert torch.equal(got.float(), want)


def test_outputs_stay_inside_their_rows():
    """Canary test: every output is a strided view into a poisoned buffer with guard rows either side and guard
    columns after every row; ragged grids (partly empty tiles at the right and bottom edges) on both paths.  After
    forward and backward the outputs match the oracle and every guard element still holds the poison."""
    POISON = -1234.0
    for (th, tw, w, dqk, dv, R) in ((21, 19, 7, 64, 64, 16), (9, 50, 9, 64, 128, 8), (37, 11, 5, 128, 64, 32),
                                    (19, 21, 5, 32, 64, 8), (13, 18, 7, 96, 32, 16)):    # half-filled last chunks
        N = th * tw
        q, k, v, do = orc.seeded_inputs(1, 2, N, dqk, dv, torch.bfloat16, 5)
        idx = orc.encode_idx(th, tw)
        rope_cpu = (idx, orc.make_cs_table(R, th), orc.make_cs_table(R, tw))
        rope = tuple(t.to(DEV) for t in rope_cpu)
        half = (w - 1) // 2
        win, sc = (1, th, tw, half, half), dqk ** -0.5
        want = orc.fused_ref(q.float(), k.float(), v.float(), do.float(), *rope_cpu, *win, sc)
        qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))

        def guarded(d):
            buf = torch.full((1, 2, N + 16, d + 8), POISON, dtype=torch.bfloat16, device=DEV)
            return buf, buf[:, :, 8:N + 8, :d]

        for path in PATHS:
            if path != "handoff" and (dqk % 64 or dv % 64):
                continue                 # the kernels that rotate streamed rows take head dims 64 and 128 only
            (bo, o), (bq, dq), (bk, dk), (bv, dv_) = guarded(dv), guarded(dqk), guarded(dqk), guarded(dv)
            if path == "handoff":
                _, lse, qr, kr = swa.swa_forward_rot(qd, kd, vd, rope, *win, sc, impl="tc", out=o)
                swa.swa_backward_rot(qr, kr, vd, o, lse, dod, rope, *win, sc, impl="tc", out=(dq, dk, dv_))
            else:
                _, lse = swa.swa_forward(qd, kd, vd, rope, *win, sc, impl="tc", out=o)
                swa.swa_backward(qd, kd, vd, o, lse, dod, rope, *win, sc, impl="tc", out=(dq, dk, dv_))
            swa.check_status()
            assert_close([t.float().cpu() for t in (o, dq, dk, dv_)], want, torch.bfloat16, what=f"canary {th}x{tw}/{path}")
            for buf, view, d in ((bo, o, dv), (bq, dq, dqk), (bk, dk, dqk), (bv, dv_, dv)):
                guard = buf.clone()
                guard[:, :, 8:N + 8, :d] = POISON
                assert bool((guard == POISON).all()), f"canary {th}x{tw}/{path}: a guard element was overwritten"


@pytest.mark.parametrize("d", [64, 32])
@pytest.mark.parametrize("with_rope", [True, False])
def test_packed_qkv_entry(with_rope, d):
    """qkv [B, N, 3, H, d] in, o [B, N, H*d] out, packed gradient back: against the oracle, and bit-identical to
    the [B, H, N, d] entry on contiguous copies (same kernels, same arithmetic order)."""
    torch.manual_seed(3)
    B, H, TH, TW = 2, 3, 20, 24
    N = TH * TW
    qkv = torch.randn(B, N, 3, H, d).to(torch.bfloat16)
    do = torch.randn(B, N, H * d).to(torch.bfloat16)
    win = (1, TH, TW, 3, 2)
    rope_cpu = rope_dev = (None, None, None)
    if with_rope:
        idx = swa.FusedInplaceRotaryPositionEncoding2D.encode_idx(TH, TW)
        idx[torch.rand(N) < 0.1] = -1
        tr, tc = swa.make_cs_table(d // 4, TH), swa.make_cs_table(d // 4, TW)
        rope_cpu = (idx, tr, tc)
        rope_dev = tuple(t.to(DEV) for t in rope_cpu)
    x = qkv.to(DEV).requires_grad_(True)
    o = swa.TiledSwaPackedQKV.apply(x, *rope_dev, *win, 0.125)
    assert o.shape == (B, N, H * d) and o.is_contiguous()
    o.backward(do.to(DEV))
    swa.check_status()
    assert x.grad.shape == qkv.shape and x.grad.is_contiguous()
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3).float() for i in range(3))
    do4 = do.view(B, N, H, d).permute(0, 2, 1, 3).float()
    want = orc.fused_ref(q, k, v, do4, *rope_cpu, *win, 0.125)
    got = [o.detach().view(B, N, H, d).permute(0, 2, 1, 3).float().cpu()]
    got += [x.grad[:, :, i].permute(0, 2, 1, 3).float().cpu() for i in range(3)]
    assert_close(got, want, torch.bfloat16, what="packed qkv")
    # the same problem through the [B, H, N, d] entry
    qc, kc, vc = (qkv[:, :, i].permute(0, 2, 1, 3).contiguous().to(DEV).requires_grad_(True) for i in range(3))
    if d == 64 or not with_rope:      # (with RoPE and d = 32 only the rotate-once entries are tensor-core shapes)
        assert swa.selected_impl(qc, vc, rope_dev if with_rope else None, *win) == "tc"
    o2 = swa.TiledSwaRope2D.apply(qc, kc, vc, *rope_dev, *win, 0.125)
    o2.backward(do.view(B, N, H, d).permute(0, 2, 1, 3).contiguous().to(DEV))
    swa.check_status()
    for a, b in zip(got, (o2.detach(), qc.grad, kc.grad, vc.grad)):
        assert torch.equal(a, b.float().cpu())


def test_reference_selftest_shape_runs_on_tensor_cores():
    """The shape of the reference's own self-test (src/tiled_swa.py:736-746: fp16, d = 32, 4x4-pixel tiles so
    b_size = 16, 16 x 16 tiles, one tile of reach) through the public autograd surface: the tensor-core kernels take
    d = 32 as it is (no padding by the Python layer); results against the oracle and against the SIMT kernels.  With
    RoPE on the kernels that rotate streamed rows the Python layer still pads to 64."""
    torch.manual_seed(0)
    B, H, d, bs, TH, TW = 1, 2, 32, 16, 16, 16
    N = bs * TH * TW
    q, k, v, do = (torch.randn(B, H, N, d).to(torch.float16) for _ in range(4))
    win = (bs, TH, TW, 1, 1)
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    assert swa.padded_head_dims(qd, vd, None, *win, 1.0) is None     # nothing to pad: the problem itself is eligible
    assert swa.selected_impl(qd, vd, None, *win) == "tc"
    idx = orc.encode_idx(TH, TW * bs).to(DEV)
    tab = orc.make_cs_table(8, TH * bs).to(DEV)
    assert swa.padded_head_dims(qd, vd, (idx, tab, tab), *win, 1.0) == (64, 64)
    o = swa.TiledSwa.apply(qd, kd, vd, *win, 1.0)
    o.backward(do.to(DEV))
    swa.check_status()
    got = [t.detach().float().cpu() for t in (o, qd.grad, kd.grad, vd.grad)]
    for t in got:
        assert t.shape == q.shape
    want = orc.fused_ref(q.float(), k.float(), v.float(), do.float(), None, None, None, *win, 1.0)
    assert_close(got, want, torch.float16, what="self-test shape")
    simt, _ = run_gpu(q, k, v, do, None, win, 1.0, impl="simt")
    assert_close(got, simt, torch.float16, what="self-test shape vs simt")


def test_rope_modes_agree():
    """The three ways ``TiledSwaRope2D`` can apply the rotation (``set_rope_mode``: rotated copies handed from forward
    to backward; every kernel rotating what it streams; the reference's own composition with separate passes)
    against the oracle and against each other; q and k stay unmodified in all of them."""
    c = make_case(CONFIGS["cfg3"], B=1, H=2)
    rope = tuple(t.to(DEV) for t in (c["idx"], c["row_cs"], c["col_cs"]))
    want = orc.fused_ref(c["q"].float(), c["k"].float(), c["v"].float(), c["do"].float(), c["idx"], c["row_cs"],
                         c["col_cs"], *c["win"], c["sm_scale"])
    results = {}
    for mode in ("handoff", "prerotate", "fused"):
        prev = swa.set_rope_mode(mode)
        try:
            q, k, v = (c[n].to(DEV).requires_grad_(True) for n in ("q", "k", "v"))
            o = swa.TiledSwaRope2D.apply(q, k, v, *rope, *c["win"], c["sm_scale"])
            o.backward(c["do"].to(DEV))
            swa.check_status()
        finally:
            swa.set_rope_mode(prev)
        assert torch.equal(q.detach().cpu(), c["q"]) and torch.equal(k.detach().cpu(), c["k"])
        results[mode] = [t.detach().float().cpu() for t in (o, q.grad, k.grad, v.grad)]
        assert_close(results[mode], want, c["q"].dtype, what=mode)
    assert_close(results["prerotate"], results["fused"], c["q"].dtype, what="prerotate vs fused")
    assert_close(results["handoff"], results["fused"], c["q"].dtype, what="handoff vs fused")


@pytest.mark.parametrize("bs,th,tw,rs,cs", [(16, 6, 6, 1, 2), (32, 4, 5, 2, 1), (8, 7, 9, 1, 5), (16, 5, 12, 0, 2)])
def test_wide_halo_runs_on_tensor_cores(bs, th, tw, rs, cs):
    """Windows whose halo is 65 to 96 token columns wide (the dK/dV kernel fits blocks of up to 96 tokens at d = 64) (tiles of 8 to 32 tokens with several tile columns of
    reach -- the regime of the reference's own self-test, b_size = 16) take the tensor-core kernels."""
    torch.manual_seed(bs + cs)
    B, H, d = 1, 2, 64
    N = bs * th * tw
    q, k, v, do = (torch.randn(B, H, N, d).to(torch.bfloat16) for _ in range(4))
    win = (bs, th, tw, rs, cs)
    idx = torch.arange(N, dtype=torch.int32) // bs          # every token of a tile shares the tile's position
    idx = ((idx // tw) << 16) | (idx % tw)
    rope = (idx.to(torch.int32), swa.make_cs_table(16, th), swa.make_cs_table(16, tw))
    rope_dev = tuple(t.to(DEV) for t in rope)
    for which in (0, 1, 2):
        assert swa.selected_impl(q.to(DEV), v.to(DEV), rope_dev, *win, 0.125, which=which) == "tc"
    got, _ = run_gpu(q, k, v, do, rope, win, 0.125)
    want = orc.fused_ref(q.float(), k.float(), v.float(), do.float(), *rope, *win, 0.125)
    assert_close(got, want, torch.bfloat16, what=f"wide halo b={bs} col={cs}")


@pytest.mark.parametrize("bs,th,tw,rs,cs,d_qk,d_v", [(16, 8, 12, 1, 4, 64, 64), (16, 6, 14, 2, 5, 64, 128),
                                                    (32, 5, 9, 1, 3, 128, 64), (4, 9, 60, 1, 25, 64, 64)])
def test_halos_wider_than_a_block_stay_on_tensor_cores(bs, th, tw, rs, cs, d_qk, d_v):
    """Halos of 150 to 250 token columns -- wider than any streamed block (128 tokens at most): kernel-9 / -11 sized
    windows over tiles of 16 or 32 tokens, the regime of the reference's own harness (src/tiled_swa.py:736-757).  The
    kernels without streamed rotation walk such a halo in several column blocks per row band; without RoPE and on
    the hand-off path nothing falls to the SIMT kernels any more."""
    torch.manual_seed(bs + cs)
    B, H = 1, 2
    N = bs * th * tw
    q, k = (torch.randn(B, H, N, d_qk).to(torch.bfloat16) for _ in range(2))
    v, do = (torch.randn(B, H, N, d_v).to(torch.bfloat16) for _ in range(2))
    win, sc = (bs, th, tw, rs, cs), d_qk ** -0.5
    idx = torch.arange(N, dtype=torch.int32) // bs          # every token of a tile shares the tile's position
    idx = (((idx // tw) << 16) | (idx % tw)).to(torch.int32)
    rope = (idx, swa.make_cs_table(16, th), swa.make_cs_table(16, tw))
    g = swa.tiled_swa._geom(q, v, *win, sc, "auto")
    plan = (C.c_int32 * 12)()
    r = swa._lib.make_rope(*rope)
    for which in (3, 4, 5):
        assert swa._lib.lib.swa_describe_plan(C.byref(g), C.byref(r), which, plan) == 0, "hand-off kernels must take it"
        assert plan[3] < (2 * cs + 1) * bs                  # block narrower than the halo: several column blocks
    for rp, path in ((None, "fused"), (rope, "handoff")):
        got, _ = run_gpu(q, k, v, do, rp, win, sc, impl="tc", path=path)
        want = orc.fused_ref(q.float(), k.float(), v.float(), do.float(), *(rp or (None, None, None)), *win, sc,
                             windowed=True)
        assert_close(got, want, torch.bfloat16, what=f"wide halo b={bs} col={cs} {path}")


def test_expanded_gradient_keeps_tensor_core_path():
    """``o.sum().backward()`` hands backward a stride-0 gradient; it is materialised once instead of pushing the
    whole backward pass onto the SIMT kernels, and the result matches an explicit tensor of ones."""
    torch.manual_seed(5)
    q, k, v = (torch.randn(1, 2, 32 * 32, 64, device=DEV).to(torch.bfloat16).requires_grad_(True) for _ in range(3))
    win = (1, 32, 32, 3, 3)
    swa.TiledSwa.apply(q, k, v, *win, 0.125).sum().backward()
    got = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    o = swa.TiledSwa.apply(q, k, v, *win, 0.125)
    o.backward(torch.ones_like(o))
    swa.check_status()
    for a, t in zip(got, (q, k, v)):
        assert torch.equal(a, t.grad)


def test_unaddressable_inputs_are_copied_not_demoted():
    """q, k, v with a non-unit last stride (a transposed [B,H,d,N] buffer): same result as contiguous copies."""
    torch.manual_seed(6)
    base = [torch.randn(1, 2, 64, 24 * 24, device=DEV).to(torch.bfloat16) for _ in range(3)]
    q, k, v = (t.transpose(-1, -2) for t in base)
    assert q.stride(-1) != 1
    win = (1, 24, 24, 2, 2)
    o1, l1 = swa.swa_forward(q, k, v, None, *win, 0.125)
    o2, l2 = swa.swa_forward(q.contiguous(), k.contiguous(), v.contiguous(), None, *win, 0.125)
    do = torch.randn_like(o2)
    g1 = swa.swa_backward(q, k, v, o1, l1, do, None, *win, 0.125)
    g2 = swa.swa_backward(q.contiguous(), k.contiguous(), v.contiguous(), o2, l2, do, None, *win, 0.125)
    swa.check_status()
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)


@pytest.mark.parametrize("d_qk,d_v,rope_dims,b,th,tw,rs,cs,dtype", [
    (32, 32, 0, 16, 16, 16, 1, 1, torch.float16),      # the reference's own self-test shape (src/tiled_swa.py:736-746)
    (32, 32, 32, 1, 24, 20, 3, 2, torch.bfloat16),     # RoPE on all 32 dims, rotate-once path
    (32, 96, 32, 1, 21, 19, 2, 3, torch.float16),      # different q/k and v dims, ragged grid
    (96, 64, 64, 2, 10, 9, 1, 2, torch.bfloat16),      # 96 = one and a half chunks, partial RoPE, tiles of two tokens
])
def test_head_dims_32_and_96_run_on_tensor_cores_as_they_are(monkeypatch, d_qk, d_v, rope_dims, b, th, tw, rs, cs, dtype):
    """Head dims of 32 and 96 through the C ABI itself, with the Python layer's zero-padding switched off: the
    tensor-core kernels without streamed rotation take them (TMA zero-fills the missing half of the last 64-element
    chunk, the epilogues store the real columns only)."""
    monkeypatch.setenv("SWA_NO_HEAD_PAD", "1")
    B, H, N, W = 1, 3, th * tw * b, tw * b
    q, k, v, do = orc.seeded_inputs(B, H, N, d_qk, d_v, dtype, seed=21)
    rope = None
    if rope_dims:
        idx = orc.encode_idx(th, W)
        idx[torch.arange(0, N, 5)] = -1
        rope = (idx, orc.make_cs_table(rope_dims // 4, th), orc.make_cs_table(rope_dims // 4, W))
    win, sm = (b, th, tw, rs, cs), d_qk ** -0.5
    g = swa._lib.make_geom(dtype, B, H, *win, d_qk, d_v, sm)
    r = swa._lib.make_rope(*(t.to(DEV) for t in rope)) if rope else None
    for which in ((3, 4, 5) if rope else (0, 1, 2)):
        out = (C.c_int32 * 12)()
        assert swa._lib.lib.swa_describe_plan(C.byref(g), C.byref(r) if r else None, which, out) == 0, "not a tensor-core shape"
    got, _ = run_gpu(q, k, v, do, rope, win, sm, path="handoff")
    f = lambda t: t.float()
    if rope:
        want = orc.fused_ref(f(q), f(k), f(v), f(do), *rope, *win, sm)
    else:
        want = list(orc.tiled_swa_bwd_ref(f(q), f(k), f(v), f(do), *win, sm))
    assert [t.shape[-1] for t in got] == [d_v, d_qk, d_qk, d_v]
    assert_close(got, want, dtype, what=f"d_qk={d_qk} d_v={d_v}")
