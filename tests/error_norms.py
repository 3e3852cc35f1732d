#!/usr/bin/env python
"""Error norms of the CUDA path against the CPU oracle, one JSON line per configuration.

    python tests/error_norms.py [cfg1 cfg2 ... target]

Not a test (the parity tests assert the same bounds); this prints the figures themselves: max-abs and mean-rel
error of O, dQ, dK, dV on the default call path (rotated copies handed from forward to backward), on the seeded
inputs the parity tests use.  Slices per configuration are chosen so that the oracle finishes in seconds:
configurations 1 and 2 in full, 3 on 8 slices, 4 and the target on one slice (windowed form of the oracle), 5 on
one slice at its full 256 x 256 size, compared on three bands of rows (top border, interior, bottom border)
against the oracle evaluated on the band plus its reach.
"""
from __future__ import annotations

import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

from oracle import swa_oracle as orc  # noqa: E402
from swa_cases import CONFIGS, make_case  # noqa: E402

import dl_templates_b200 as swa  # noqa: E402

DEV = "cuda:0"
NAMES = ("o", "dq", "dk", "dv")
SLICES = {"cfg1": None, "cfg2": None, "cfg3": (1, 8), "cfg4": (1, 1), "target": (1, 1), "cfg5": (1, 1)}


def run(c, cfg):
    q, k, v = (c[x].to(DEV) for x in ("q", "k", "v"))
    rope = tuple(c[x].to(DEV) for x in ("idx", "row_cs", "col_cs"))
    o, lse, q_rot, k_rot = swa.swa_forward_rot(q, k, v, rope, *c["win"], c["sm_scale"])
    outs = [o]
    if cfg["bwd"]:
        outs += list(swa.swa_backward_rot(q_rot, k_rot, v, o, lse, c["do"].to(DEV), rope, *c["win"], c["sm_scale"]))
    swa.check_status()
    fam = swa.selected_impl(q, v, rope, *c["win"], c["sm_scale"])
    return [t.float().cpu() for t in outs], fam


def norms(got, want):
    ma = {n: orc.max_abs(g, w) for g, w, n in zip(got, want, NAMES)}
    mr = {n: orc.mean_rel(g, w) for g, w, n in zip(got, want, NAMES)}
    return ma, mr


def rounding_floor(want, dtype):
    """Max-abs error of the oracle's own result rounded to the output dtype: what any implementation that returns
    that dtype pays before its arithmetic is counted."""
    return {n: orc.max_abs(w.to(dtype).float(), w) for w, n in zip(want, NAMES)}


def one(name):
    cfg = CONFIGS[name]
    bh = SLICES[name]
    c = make_case(cfg) if bh is None else make_case(cfg, B=bh[0], H=bh[1])
    got, fam = run(c, cfg)
    f = lambda t: t.float()
    do = f(c["do"]) if cfg["bwd"] else None
    G, half = cfg["grid"], (cfg["w"] - 1) // 2
    if name == "cfg5":
        ma, mr, fl = {}, {}, {}
        for a, b in ((0, 24), (116, 140), (G - 24, G)):
            lo, hi = max(0, a - 2 * half), min(G, b + 2 * half)
            rows = slice(lo * G, hi * G)
            crop = [f(c[x][:, :, rows]) for x in ("q", "k", "v", "do")]
            want = orc.fused_ref(*crop, c["idx"][rows], c["row_cs"], c["col_cs"], 1, hi - lo, G, half, half,
                                 c["sm_scale"], windowed=True)
            keep, full = slice((a - lo) * G, (b - lo) * G), slice(a * G, b * G)
            a_, r_ = norms([t[:, :, full] for t in got], [t[:, :, keep] for t in want])
            f_ = rounding_floor([t[:, :, keep] for t in want], cfg["dtype"])
            for n in a_:
                ma[n] = max(ma.get(n, 0.0), a_[n])
                mr[n] = max(mr.get(n, 0.0), r_[n])
                fl[n] = max(fl.get(n, 0.0), f_[n])
        compared = "rows [0,24), [116,140), [232,256) of one slice"
    else:
        want = orc.fused_ref(f(c["q"]), f(c["k"]), f(c["v"]), do, c["idx"], c["row_cs"], c["col_cs"], *c["win"],
                             c["sm_scale"], windowed=cfg["grid"] ** 2 > 4096)
        if do is None:
            want = [want]
        ma, mr = norms(got, want)
        fl = rounding_floor(want, cfg["dtype"])
        compared = f"{c['q'].shape[0] * c['q'].shape[1]} (batch, head) slice(s), all tokens"
    print(json.dumps({"config": name, "dtype": str(cfg["dtype"]).replace("torch.", ""), "kernels": fam,
                      "compared": compared, "max_abs": ma, "mean_rel": mr, "output_rounding_max_abs": fl}), flush=True)


if __name__ == "__main__":
    for n in (sys.argv[1:] or ["cfg1", "cfg2", "cfg3", "cfg4", "target", "cfg5"]):
        one(n)
