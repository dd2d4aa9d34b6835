"""Block encoder of the ladder format on B200: search, parameter bytes, nearest codes, error.

Same names, arguments and results as hi2/encode.py (``fit_ladder`` :53-92, ``quantize_params``
:95-119, ``Encoded`` :122-130, ``encode_rows`` :133-173); the arithmetic runs in two kernels of
``libhi2_b200.so`` per candidate (fit, then one pass per row).  ``_safe``/``_recon``/``_lsq`` are
the elementwise definitions other modules and tests import.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from . import ladder_kernel as _ladder

EFFORT = {
    "fast": dict(grid=(0.0, 0.06, 0.12), ls=1),
    "normal": dict(grid=(0.0, 0.04, 0.08, 0.12, 0.16, 0.20), ls=2),
    "max": dict(grid=(0.0, 0.025, 0.05, 0.075, 0.10, 0.125, 0.15, 0.20), ls=4),
}
CHUNK_ELEMS = 1 << 24  # kept for interface compatibility; the kernels need no row chunking


def _safe(step: torch.Tensor) -> torch.Tensor:
    return torch.where(step == 0, torch.ones_like(step), step)


def _recon(wb, lo, step, n):
    c = torch.round((wb - lo.unsqueeze(-1)) / _safe(step).unsqueeze(-1)).clamp(0, n - 1)
    return lo.unsqueeze(-1) + c * step.unsqueeze(-1), c


def _lsq(c, w, d):
    """Weighted least squares ``w ~ lo + c * step`` per block (definition only; the fit kernel
    carries the same formulas)."""
    sd, sc, scc = d.sum(-1), (d * c).sum(-1), (d * c * c).sum(-1)
    sw, scw = (d * w).sum(-1), (d * c * w).sum(-1)
    det = sd * scc - sc * sc
    ok = det.abs() > 1e-20
    step = torch.where(ok, (sd * scw - sc * sw) / torch.where(ok, det, torch.ones_like(det)),
                       torch.zeros_like(det))
    lo = torch.where(ok, (sw - step * sc) / sd.clamp_min(1e-20), w.mean(-1))
    return lo, step


def fit_ladder(wb: torch.Tensor, db: torch.Tensor, n: int, effort: str = "normal"):
    """Per-block ``(lo, step)`` minimising ``sum d * (w_hat - w)^2`` for ``wb [N, nb, B]`` and
    ``db`` broadcastable to ``[1, nb, B]``."""
    cfg = EFFORT[effort]
    rows, nb, b = wb.shape
    w = wb.reshape(rows, nb * b)
    if w.dtype != torch.float32 or w.stride(1) != 1:
        w = w.float().contiguous()
    d = db.to(wb.device, torch.float32).expand(1, nb, b).reshape(-1).contiguous()
    return _ladder.fit(w, d, cfg["grid"], cfg["ls"], n, b)


def quantize_params(lo: torch.Tensor, step: torch.Tensor):
    """``(lo_u8, step_u8, consts[N, 3])`` with ``consts = (lo_min, lo_scale, step_scale)`` in
    fp16, bytes computed against the rounded constants."""
    _lib.need_cuda(lo, step)
    nb = lo.shape[1]
    out = _ladder.quantize_rows(lo.float(), step.float(), 8, 16, nb * 16)
    return out["params"][..., 0].contiguous(), out["params"][..., 1].contiguous(), out["consts"]


@dataclass
class Encoded:
    codes: torch.Tensor  # uint8 [N, K]
    params: torch.Tensor  # uint8 [N, nb, 2]
    consts: torch.Tensor  # fp16 [N, 3]
    sse: torch.Tensor  # float32 [N], activation-weighted squared error
    comp: torch.Tensor | None = None  # values the codes were rounded from (GPTQ)


def encode_rows(w: torch.Tensor, d: torch.Tensor, nbits: int, block: int, effort: str = "normal",
                *, want_codes: bool = True, want_energy: bool = False, row_group=None) -> Encoded:
    """Quantise ``w [N, K]`` (stored basis) at ``(nbits, block)`` under column weights ``d [K]``, or
    ``d [G, K]`` with ``row_group [N]`` naming every row's vector (default: ``G`` equal groups of
    consecutive rows).

    ``want_codes=False`` skips the code bytes (the tables only read ``sse``); ``want_energy``
    attaches ``energy [N] = sum d * w^2`` as attribute ``energy`` of the result."""
    dev = _lib.need_cuda(w)
    n_rows, k = w.shape
    cfg = EFFORT[effort]
    if w.dtype != torch.float32 or w.stride(1) != 1:
        w = w.float().contiguous()
    d = d.to(dev, torch.float32).contiguous()
    if d.dim() == 2 and d.shape[0] > 1 and row_group is None:  # the index is made once for both launches
        row_group = _ladder._row_d(d, n_rows, k, None, "encode_rows")
    lo, st = _ladder.fit(w, d, cfg["grid"], cfg["ls"], 2**nbits, block, row_group)
    out = _ladder.quantize_rows(lo, st, nbits, block, k, w, d, want_codes=want_codes, want_sse=True,
                                want_energy=want_energy, row_group=row_group)
    enc = Encoded(out.get("codes"), out["params"], out["consts"], out["sse"])
    if want_energy:
        enc.energy = out["energy"]
    return enc
