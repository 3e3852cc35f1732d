"""Seeded workloads shared by the GPU parity tests, the smoke test and the bench."""
from __future__ import annotations

import torch

from oracle import swa_oracle as orc

from dl_templates_b200.workloads import CONFIGS  # noqa: F401


def make_case(cfg: dict, B=None, H=None, seed: int = 0):
    """CPU tensors of one configuration (optionally with fewer batch/head slices)."""
    B = cfg["B"] if B is None else B
    H = cfg["H"] if H is None else H
    G = cfg["grid"]
    N = G * G
    q, k, v, do = orc.seeded_inputs(B, H, N, cfg["d_qk"], cfg["d_v"], cfg["dtype"], seed)
    R = cfg["rope_dims"] // 4
    idx = orc.encode_idx(G, G)
    if cfg["drop"] > 0:
        g = torch.Generator().manual_seed(seed + 1000)
        idx[torch.bernoulli(torch.full((N,), cfg["drop"]), generator=g).bool()] = -1
    tab = orc.make_cs_table(R, G, 10000.0)
    half = (cfg["w"] - 1) // 2
    return dict(q=q, k=k, v=v, do=do, idx=idx, row_cs=tab, col_cs=tab.clone(),
                win=(1, G, G, half, half), sm_scale=cfg["d_qk"] ** -0.5)


def tolerances(dtype):
    """(max-abs, mean-rel) bounds of the parity requirement."""
    return (1e-4, 1e-4) if dtype == torch.float32 else (2e-2, 5e-3)
