"""Regenerate ``layerwise_moe_golden.pt``: hi2's own ``unfuse_experts`` and ``calibrate_layerwise`` on a
two-layer OLMoE-shaped toy model (fp32, seeded, fused 3-D expert parameters) on the CPU: the model's
weights as they were before unfusing, the calibration ids, and per Linear (every expert projection
among them) the error table, smoothing vector, flags and token count, plus the second moment of
every shared input after the top-up of experts below the token floor.

    PYTHONPATH=<hi2 checkout>:<this repo> HI2_GPTQ_BACKEND=torch HI2_LADDER_BACKEND=torch \
        python tests/golden/make_golden_layerwise_moe.py
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
from hi2 import moe as h_moe  # noqa: E402
from hi2.executor import Executor  # noqa: E402

from tests.golden.make_golden_layerwise import Keep  # noqa: E402
from tests.helpers import toy_olmoe  # noqa: E402


def main():
    model, ids = toy_olmoe()
    state = {k: v.clone() for k, v in model.state_dict().items()}
    with torch.no_grad():
        fused_logits = model(ids[:2], use_cache=False).logits
    assert h_moe.unfuse_experts(model) == 2
    with torch.no_grad():
        assert torch.equal(model(ids[:2], use_cache=False).logits, fused_logits)
    cfg = h_cal.Config(effort="fast")
    sink = Keep()
    with tempfile.TemporaryDirectory() as tmp:
        tables = h_lw.calibrate_layerwise(model, ids, cfg, Executor("cpu"), Path(tmp), None,
                                          re.compile("lm_head|embed"), sink=sink, log=lambda *_: None)
    out = {
        "state": state, "ids": ids, "logits": fused_logits,
        "tables": {n: dict(sse=t.sse, energy=t.energy, had=t.had, col_scale=t.col_scale, n_tokens=t.n_tokens,
                           shape=t.shape) for n, t in tables.items()},
        "sigma": sink.sigma, "n": sink.n, "groups": sink.groups,
    }
    path = Path(__file__).with_name("layerwise_moe_golden.pt")
    torch.save(out, path)
    print(path, path.stat().st_size, len(tables), "tables")
    print({n: t.n_tokens for n, t in tables.items() if "layers.0.mlp.experts" in n and "gate" in n})


if __name__ == "__main__":
    main()
