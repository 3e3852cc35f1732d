"""GPU parity of the stand-alone RoPE-2D against the oracle and the stored
outputs of the reference's own ``rope2d_ref``."""
import pytest
import torch

from conftest import load_golden
from oracle import swa_oracle as orc

import dl_templates_b200 as swa

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_selftest_layout_fp32_strided_views():
    """Layout of the reference's self-test (src/fused_rope2d.py:230-268): q is a
    stride-2 view, 16 trailing tokens have no index."""
    g = load_golden("rope_selftest_layout")
    B, N, D = g["q"].shape
    qk = torch.zeros(B, N, D, 2)
    qk[..., 0] = g["q"]
    qk[..., 1] = 7.0
    qk = qk.to(DEV)
    qv = qk[..., 0].requires_grad_(True)
    idx, rcs, ccs = (g[x].to(DEV) for x in ("idx", "row_cs", "col_cs"))
    x = qv.clone()          # RotaryPE2D works in place on its argument
    y = swa.RotaryPE2D.apply(x, idx, rcs, ccs)
    assert y.data_ptr() == x.data_ptr()
    y.backward(g["gy"].to(DEV))
    assert torch.allclose(y.detach().cpu(), g["y"], rtol=1e-2, atol=1e-2)     # the reference's own criterion
    assert orc.max_abs(y.detach().cpu(), g["y"]) < 1e-5
    assert orc.max_abs(qv.grad.cpu(), g["gq"]) < 1e-5
    assert float((qk[..., 1] - 7.0).abs().max()) == 0.0                       # the interleaved k half is untouched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("R,C", [(8, 32), (16, 64), (8, 64), (3, 20), (32, 128)])
def test_interleaved_missing_indices(dtype, R, C):
    torch.manual_seed(1)
    Gh, Gw, B = 9, 11, 5
    N = Gh * Gw + 3
    idx = torch.cat([orc.encode_idx(Gh, Gw), torch.full((3,), -1, dtype=torch.int32)])
    drop = torch.rand(N) < 0.2
    idx[drop] = -1
    idx[4] = int(idx[4]) | 0xFFFF if int(idx[4]) >= 0 else idx[4]       # column half missing only
    idx[9] = -65536 | (int(idx[9]) & 0xFFFF)                             # row half missing only
    rt, ct = orc.make_cs_table(R, Gh), orc.make_cs_table(R, Gw)
    x = torch.randn(B, N, C).to(dtype)
    want = orc.rope2d_ref(x.float(), idx, rt, ct)
    xd = x.to(DEV)
    swa.rope2d_apply_(xd, idx.to(DEV), rt.to(DEV), ct.to(DEV))
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert orc.max_abs(xd.float().cpu(), want) < tol
    back = swa.rope2d_apply_(xd, idx.to(DEV), rt.to(DEV), ct.to(DEV), inverse=True)
    assert orc.max_abs(back.float().cpu(), x.float()) < (1e-5 if dtype == torch.float32 else 6e-2)
    # tokens with no index at all are bit-identical
    none = (idx == -1)
    assert torch.equal(xd.cpu()[:, none], x[:, none])


def test_module_forward_4d():
    G, B, H, C = 8, 2, 3, 64
    m = swa.FusedInplaceRotaryPositionEncoding2D(32, G, G).to(DEV)
    idx = m.encode_idx(G, G).to(DEV)
    x = torch.randn(B, H, G * G, C, device=DEV)
    want = orc.rope2d_ref(x.cpu().reshape(B * H, G * G, C), idx.cpu(), m.row_buffer.cs_components.cpu(),
                          m.col_buffer.cs_components.cpu()).reshape(B, H, G * G, C)
    y = m(x, idx)
    assert orc.max_abs(y.cpu(), want) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("R,C", [(8, 32), (16, 64), (8, 64), (3, 20), (32, 128)])
def test_out_of_place_form(dtype, R, C):
    """``rope2d_apply_to``: same values as clone + in-place rotation (one-pass kernel for 16-bit types with
    n_rdim % 8 == 0, the two-step path otherwise), input untouched, strided input rows, inverse included."""
    torch.manual_seed(2)
    Gh, Gw, B = 7, 12, 4
    N = Gh * Gw + 2
    idx = torch.cat([orc.encode_idx(Gh, Gw), torch.full((2,), -1, dtype=torch.int32)])
    idx[torch.rand(N) < 0.2] = -1
    idx[5] = int(idx[5]) | 0xFFFF if int(idx[5]) >= 0 else idx[5]
    idx[8] = -65536 | (int(idx[8]) & 0xFFFF)
    rt, ct = orc.make_cs_table(R, Gh), orc.make_cs_table(R, Gw)
    packed = torch.randn(B, N, 3, C).to(dtype).to(DEV)
    x = packed[:, :, 1]                                   # rows of C elements at a stride of 3*C
    keep = packed.clone()
    dev = [t.to(DEV) for t in (idx, rt, ct)]
    for inverse in (False, True):
        y = swa.rope2d_apply_to(x, *dev, inverse=inverse)
        assert y.is_contiguous() and torch.equal(packed, keep)
        ref = swa.rope2d_apply_(x.clone(), *dev, inverse=inverse)
        if dtype == torch.float32:
            assert torch.equal(y, ref)
        else:
            assert orc.max_abs(y.float().cpu(), ref.float().cpu()) <= 2 ** -6 * float(ref.float().abs().max())
            want = orc.rope2d_ref(x.float().cpu(), idx, rt, ct) if not inverse else None
            if want is not None:
                assert orc.max_abs(y.float().cpu(), want) < 3e-2
        none = (idx == -1)
        assert torch.equal(y[:, none.to(DEV)], x[:, none.to(DEV)])
        assert torch.equal(y[..., 4 * R:], x[..., 4 * R:])
