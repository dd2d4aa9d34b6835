"""Regenerate ``quality_golden.pt``: hi2's ``allocate_by_quality`` on seeded error tables (three
tensors, six candidates, one tensor with a sensitivity weight) at several error ratios.

    PYTHONPATH=<hi2 checkout>:<this repo> python tests/golden/make_golden_quality.py
"""

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from hi2 import allocate as h_alloc  # noqa: E402
from hi2.calibrate import ALL_CANDIDATES, TensorTable  # noqa: E402


def main():
    g = torch.Generator().manual_seed(123)
    tables = []
    for name, (r, k) in (("a", (300, 256)), ("b", (120, 512)), ("c", (77, 128))):
        base = torch.rand(r, generator=g) * 5 + 0.1
        # more bits and smaller blocks cost less error, with row-dependent noise
        sse = torch.stack([base * (0.02 if nb == 4 else 1.0) * (b / 32) ** 0.5 * (0.5 + torch.rand(r, generator=g))
                           for nb, b in ALL_CANDIDATES]).float()
        had = torch.ones(k // 16, dtype=torch.uint8)
        tables.append(TensorTable(name, (r, k), had, sse, list(ALL_CANDIDATES), float(base.sum()) * 3, 1000))
    sens = {"b": 2.5}
    out = {"tables": [dict(name=t.name, shape=t.shape, had=t.had, sse=t.sse, candidates=t.candidates, energy=t.energy,
                           n_tokens=t.n_tokens) for t in tables], "sens": sens, "cases": {}}
    for ratio in (1.0, 1.05, 1.5, 4.0, 0.9):
        a = h_alloc.allocate_by_quality(tables, ratio, sens)
        out["cases"][ratio] = dict(picks=a.picks, bpw=a.bpw, lam=a.lam, feasible=a.feasible, error_ratio=a.error_ratio,
                                   frac=a.frac_by_bits)
        print(ratio, a.bpw, a.lam, a.feasible, a.error_ratio)
    path = Path(__file__).with_name("quality_golden.pt")
    torch.save(out, path)
    print(path, path.stat().st_size)


if __name__ == "__main__":
    main()
