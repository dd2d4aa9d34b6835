"""Regenerate ``stack_golden.pt``: packed expert tensors built by hi2's ``assemble`` and what hi2's
``build_stack`` makes of them (the stacked layout of routed experts), for a two-part group with a
smoothing vector per expert and a one-part group without.

    PYTHONPATH=<hi2 checkout>:<this repo> python tests/golden/make_golden_stack.py
"""

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from hi2 import encode as h_enc  # noqa: E402
from hi2 import format as h_fmt  # noqa: E402
from hi2 import stack as h_stack  # noqa: E402

CANDS = [(2, 16), (2, 64), (4, 32), (8, 32), (4, 16)]


def packed(g, rows, k, had, col_scale):
    w = torch.randn(rows, k, generator=g)
    d = torch.rand(k, generator=g) + 0.1
    pick = torch.randint(0, len(CANDS), (rows,), generator=g)
    pieces = []
    for ci, (nb, b) in enumerate(CANDS):
        idx = (pick == ci).nonzero().flatten()
        if idx.numel():
            e = h_enc.encode_rows(w[idx], d, nb, b, "fast")
            pieces.append((idx, e.codes, e.params, e.consts))
    nbits = torch.tensor([CANDS[i][0] for i in pick.tolist()])
    block = torch.tensor([CANDS[i][1] for i in pick.tolist()])
    return h_fmt.assemble(pieces, nbits, block, had, k, col_scale)


def fields(t):
    return dict(fields={f: getattr(t, f) for f in h_fmt.FIELDS}, shape=t.shape, col_scale=t.col_scale)


def main():
    g = torch.Generator().manual_seed(91)
    k = 128
    out = {}
    for group, rows_of_parts, scaled in (("gate_up", (5, 7), True), ("down", (9,), False)):
        experts = []
        for _ in range(3):
            had = (torch.rand(k // 16, generator=g) < 0.5).to(torch.uint8)
            cs = (torch.rand(k, generator=g) * 2 + 0.25).half() if scaled else None
            experts.append([packed(g, r, k, had, cs) for r in rows_of_parts])
        out[group] = dict(experts=[[fields(p) for p in parts] for parts in experts],
                          stack=h_stack.build_stack(experts), parts=h_stack.GROUPS[group])
    names = [f"model.layers.0.mlp.experts.{e}.{p}.hi2_{f}" for e in range(3) for p in ("gate_proj", "up_proj", "down_proj")
             for f in h_fmt.FIELDS] + [f"model.layers.0.self_attn.q_proj.hi2_{f}" for f in h_fmt.FIELDS]
    single, stacked = h_stack.hi2_bases(names)
    out["names"] = dict(names=names, single=single, stacked=stacked, groups=h_stack.stack_groups(single))
    path = Path(__file__).with_name("stack_golden.pt")
    torch.save(out, path)
    print(path, path.stat().st_size)


if __name__ == "__main__":
    main()
