"""Regenerate ``transform_golden.pt``: what hi2 itself chooses as the shared transform
(``shared_transform``: smoothing exponent search, per-chunk rotation flags) for seeded inputs.

    PYTHONPATH=<hi2 checkout>:<this repo> python tests/golden/make_golden_transform.py
"""

import os
import sys
from pathlib import Path

import torch

os.environ.setdefault("HI2_LADDER_BACKEND", "torch")
ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from hi2 import calibrate as h_cal  # noqa: E402
from hi2.executor import Executor  # noqa: E402
from hi2.stats import ColumnStats  # noqa: E402

from tests.helpers import transform_case  # noqa: E402


def main():
    ex = Executor("cpu")
    out = []
    for seed, k, rows, mode, alpha, search in [(1, 256, (96, 40), "auto", 0.5, ()),
                                               (2, 512, (1500, 700), "auto", 0.5, (0.25, 0.75)),
                                               (3, 256, (64,), "on", 0.5, (0.0, 0.25, 1.0)),
                                               (4, 192, (80, 80, 80), "off", 0.0, ())]:
        ws, x = transform_case(seed, k, rows)
        stats = ColumnStats(k)
        stats.update(x)
        cfg = h_cal.Config(rotation=mode, smooth=alpha, smooth_search=search, effort="fast")
        s16, had = h_cal.shared_transform(ws, stats, cfg, ex)
        costs = {}
        for a in dict.fromkeys((alpha, *search)):
            s_a, had_a = h_cal._fixed_transform(ws, stats, cfg, ex, a)
            costs[a] = h_cal.transform_error(ws, stats, s_a, had_a, ex)
        out.append(dict(seed=seed, k=k, rows=rows, mode=mode, alpha=alpha, search=search, s16=s16, had=had, costs=costs))
    path = Path(__file__).with_name("transform_golden.pt")
    torch.save(out, path)
    print(path, path.stat().st_size)


if __name__ == "__main__":
    main()
