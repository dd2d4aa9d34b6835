"""Regenerate ``dequant_golden.pt``: a mixed-row packed tensor (INT2/4/8, blocks 16/32/64, partial
rotation flags, a smoothing vector) built by hi2's ``assemble`` and what hi2's ``dequantize_stored``
and ``dequantize`` return for it.

    PYTHONPATH=<hi2 checkout>:<this repo> python tests/golden/make_golden_dequant.py
"""

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from hi2 import encode as h_enc  # noqa: E402
from hi2 import format as h_fmt  # noqa: E402


def main():
    g = torch.Generator().manual_seed(77)
    k, rows = 192, 40
    w = torch.randn(rows, k, generator=g) * torch.exp(0.5 * torch.randn(rows, 1, generator=g))
    d = torch.rand(k, generator=g) + 0.1
    cands = [(2, 16), (2, 64), (4, 32), (8, 32), (8, 64), (4, 16)]
    pick = torch.randint(0, len(cands), (rows,), generator=g)
    pieces = []
    for ci, (nb, b) in enumerate(cands):
        idx = (pick == ci).nonzero().flatten()
        if idx.numel():
            e = h_enc.encode_rows(w[idx], d, nb, b, "fast")
            pieces.append((idx, e.codes, e.params, e.consts))
    nbits = torch.tensor([cands[i][0] for i in pick.tolist()])
    block = torch.tensor([cands[i][1] for i in pick.tolist()])
    had = (torch.rand(k // 16, generator=g) < 0.6).to(torch.uint8)
    col_scale = (torch.rand(k, generator=g) * 2 + 0.25).half()
    out = {}
    for name, cs in (("scaled", col_scale), ("plain", None)):
        t = h_fmt.assemble(pieces, nbits, block, had, k, cs)
        out[name] = dict(fields={f: getattr(t, f) for f in h_fmt.FIELDS}, shape=t.shape, col_scale=t.col_scale,
                         stored=h_fmt.dequantize_stored(t), original=h_fmt.dequantize(t))
    path = Path(__file__).with_name("dequant_golden.pt")
    torch.save(out, path)
    print(path, path.stat().st_size)


if __name__ == "__main__":
    main()
