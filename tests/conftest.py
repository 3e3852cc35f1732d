import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def load_golden(name):
    """Read one stored reference case as a dict of torch tensors / python scalars."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for k in z.files:
        a = z[k]
        out[k] = torch.from_numpy(a) if a.ndim > 0 else a.item()
    if "meta" in out:
        B, H, th, tw, b, row, col, dqk, dv, R = (int(x) for x in out["meta"])
        out["meta"] = dict(B=B, H=H, t_height=th, t_width=tw, b_size=b, row_size=row, col_size=col,
                           d_qk=dqk, d_v=dv, R=R)
    return out


SWA_GOLDEN_CASES = [
    "cfg1_16x16_d32_w7_fp32",
    "b16_4x5_dqk16_dv32",
    "g5x7_r2c1_partial_rope_drop",
    "b2_6x4_r1c2_rope",
    "g3x4_window_exceeds_grid",
    "g12x20_dqk64_dv128_w5",
]


@pytest.fixture
def golden():
    return load_golden
