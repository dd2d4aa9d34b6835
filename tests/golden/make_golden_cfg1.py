"""Regenerate ``cfg1_golden.pt``: BASELINE config 1 (a 4096 x 4096 fp16 Linear, 2048 calibration
tokens, 3.0 bpw) through hi2 ITSELF on the CPU, reduced to a small fixture.

Run in a container that has the hi2 sources (about a minute on 8 cores):

    PYTHONPATH=<hi2 checkout>:<this repo> HI2_GPTQ_BACKEND=torch HI2_LADDER_BACKEND=torch \
        HI2_REFINE_BACKEND=torch python tests/golden/make_golden_cfg1.py

What is kept (0.3 MB): the smoothing vector, the whole error table ``sse [6, 4096]``, energy, the
allocator's picks, bpw and multiplier, the diagonal of the stored-basis Hessian and of the factor,
the three row constants of every row, and of the big buffers (6 MB of code words, 1.3 MB of
parameter bytes) a SHA-256 each plus the first 64 rows verbatim.  tests/test_oracle_cfg1.py checks
the CPU oracle against it at full size; the GPU tests check the kernels against the oracle.
"""

import hashlib
import os
import sys
from pathlib import Path

import torch

os.environ.setdefault("HI2_GPTQ_BACKEND", "torch")
os.environ.setdefault("HI2_LADDER_BACKEND", "torch")
os.environ.setdefault("HI2_REFINE_BACKEND", "torch")

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from hi2 import allocate as h_alloc  # noqa: E402
from hi2 import calibrate as h_cal  # noqa: E402
from hi2.executor import Executor  # noqa: E402
from hi2.hessian import HessianStats, inverse_factor, transform_sigma  # noqa: E402
from hi2.stats import ColumnStats  # noqa: E402

from tests.helpers import config1_inputs  # noqa: E402

HEAD = 64


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def main():
    w, x = config1_inputs()
    k = w.shape[1]
    ex = Executor("cpu")
    cfg = h_cal.Config()
    hess = HessianStats(k, "cpu")
    hess.update(x)
    stats = ColumnStats(k)
    stats.update(x)
    table = h_cal.build_table("w", w, stats, cfg, ex)
    alloc = h_alloc.allocate_global([table], 3.0)
    picks = alloc.picks["w"]
    req = h_cal.EncodeRequest(w, stats, table, picks, sigma=hess.mean(), sigma_id="x")
    (t,) = h_cal.encode_many([req], cfg, ex)
    hs = transform_sigma(hess.mean(), table.col_scale, table.had)
    u = inverse_factor(hs, cfg.damp)
    out = {
        "seed_note": "inputs: tests.helpers.config1_inputs()",
        "candidates": list(cfg.candidates),
        "col_scale": table.col_scale,
        "sse": table.sse,
        "energy": table.energy,
        "picks": picks.to(torch.int8),
        "bpw": alloc.bpw,
        "lam": alloc.lam,
        "feasible": alloc.feasible,
        "hs_diag": hs.diagonal().clone(),
        "u_diag": u.diagonal().clone(),
        "row_consts": t.row_consts,
        "row_nbits": t.row_nbits,
        "row_block": t.row_block,
        "code_off_head": t.code_off[: HEAD + 1].clone(),
        "param_off_head": t.param_off[: HEAD + 1].clone(),
        "codes_head": t.codes[: int(t.code_off[HEAD])].clone(),
        "params_head": t.blk_params[: 2 * int(t.param_off[HEAD])].clone(),
        "codes_total": int(t.codes.numel()),
        "params_total": int(t.blk_params.numel()),
        "sha": {"codes": sha(t.codes), "blk_params": sha(t.blk_params), "row_consts": sha(t.row_consts),
                "sse": sha(table.sse), "picks": sha(picks)},
    }
    path = Path(__file__).with_name("cfg1_golden.pt")
    torch.save(out, path)
    print(path, path.stat().st_size, "bytes; bpw", alloc.bpw)


if __name__ == "__main__":
    main()
