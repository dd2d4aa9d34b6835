"""Regenerate ``layerwise_golden.pt``: hi2's own ``calibrate_layerwise`` on a two-layer Llama-shaped
toy model (fp32, seeded) on the CPU: the model's weights, the calibration ids, and per Linear the
error table, smoothing vector, flags and token count, plus the second moment of every shared input.

    PYTHONPATH=<hi2 checkout>:<this repo> HI2_GPTQ_BACKEND=torch HI2_LADDER_BACKEND=torch \
        python tests/golden/make_golden_layerwise.py
"""

import os
import re
import sys
import tempfile
from pathlib import Path

import torch

os.environ.setdefault("HI2_GPTQ_BACKEND", "torch")
os.environ.setdefault("HI2_LADDER_BACKEND", "torch")
ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from hi2 import calibrate as h_cal  # noqa: E402
from hi2 import layerwise as h_lw  # noqa: E402
from hi2.executor import Executor  # noqa: E402

from tests.helpers import toy_llama  # noqa: E402


class Keep:
    """A sink that keeps the second moments instead of writing them."""

    def __init__(self):
        self.sigma, self.n, self.groups = {}, {}, []

    def hessians(self, lead, hess, linears):
        for ld, h in hess.items():
            self.sigma[linears[ld]] = h.S.clone()
            self.n[linears[ld]] = h.n

    def stats(self, leader, members, st):
        self.groups.append((leader, list(members)))

    def layer(self, *a):
        pass

    def expert_tokens(self, obj):
        pass


def main():
    model, ids = toy_llama()
    cfg = h_cal.Config(effort="fast")
    sink = Keep()
    with tempfile.TemporaryDirectory() as tmp:
        tables = h_lw.calibrate_layerwise(model, ids, cfg, Executor("cpu"), Path(tmp), None,
                                          re.compile("lm_head|embed"), sink=sink, log=lambda *_: None)
    out = {
        "state": {k: v.clone() for k, v in model.state_dict().items()},
        "ids": ids,
        "tables": {n: dict(sse=t.sse, energy=t.energy, had=t.had, col_scale=t.col_scale, n_tokens=t.n_tokens,
                           shape=t.shape) for n, t in tables.items()},
        "sigma": sink.sigma, "n": sink.n, "groups": sink.groups,
    }
    path = Path(__file__).with_name("layerwise_golden.pt")
    torch.save(out, path)
    print(path, path.stat().st_size, len(tables), "tables", sink.groups)


if __name__ == "__main__":
    main()
