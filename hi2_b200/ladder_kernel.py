"""Ladder search kernels on B200 (interface of hi2/ladder_kernel.py:109-156).

``ladder_grid`` is the grid part of the fit as in the reference; ``fit`` adds the least-squares
refits and ``quantize_rows`` the row-wide parameter quantisation, decode, code assignment and
error, so one candidate of the tables costs two launches.
"""

from __future__ import annotations

import torch

from . import _lib
from .gptq_kernel import kernel_dir, supported  # noqa: F401  (re-exported like the reference)


def load():
    return _lib.load()


def available(dev: torch.device) -> bool:
    return supported(dev) and load() is not None


def failure() -> str | None:
    return _lib.failure()


def ladder_grid(wb: torch.Tensor, db: torch.Tensor, grid: tuple, n: int):
    """``(lo, step, err)`` per ``(row, block)``, all ``[N, nb]`` float32."""
    dev = _lib.need_cuda(wb, db)
    wb = wb.contiguous().float()
    db = db.contiguous().float()
    rows, nb, b = wb.shape
    lo = torch.empty(rows, nb, dtype=torch.float32, device=dev)
    st = torch.empty(rows, nb, dtype=torch.float32, device=dev)
    err = torch.empty(rows, nb, dtype=torch.float32, device=dev)
    _lib.call(
        "hi2_ladder_grid", _lib.ptr(wb), _lib.ptr(db), _lib.host_floats(grid), len(grid), int(n),
        rows, nb, b, _lib.ptr(lo), _lib.ptr(st), _lib.ptr(err), _lib.stream(dev),
    )
    return lo, st, err


def _row_d(d: torch.Tensor, rows: int, k: int, row_group, what: str):
    """None for one weight vector ``d [K]``.  For ``d [G, K]`` the int32 index ``[N]`` of every row's
    vector: ``row_group`` as given, or, without one, ``G`` equal groups of consecutive rows."""
    if d.dim() == 1 or d.numel() == k:
        return None
    if d.dim() != 2 or d.shape[1] != k:
        raise ValueError(f"{what}: d must be [K] or [G, K]")
    if row_group is not None:
        if row_group.numel() != rows:
            raise ValueError(f"{what}: row_group must name a vector for every row")
        return row_group.to(d.device, torch.int32).contiguous()
    if rows % d.shape[0]:
        raise ValueError(f"{what}: without row_group the rows must be a multiple of the number of vectors")
    return torch.arange(d.shape[0], device=d.device, dtype=torch.int32).repeat_interleave(rows // d.shape[0])


def fit(w: torch.Tensor, d: torch.Tensor, grid: tuple, refits: int, n: int, block: int, row_group=None):
    """Grid search plus ``refits`` least-squares refits (hi2/encode.py:53-92) on rows
    ``w [N, K]`` (fp32, unit column stride); returns ``lo, step [N, K / block]``.  ``d`` is ``[K]``,
    or ``[G, K]`` with ``row_group [N]`` naming every row's vector (default: ``G`` equal groups of
    consecutive rows)."""
    dev = _lib.need_cuda(w, d)
    rows, k = w.shape
    if w.dtype != torch.float32 or w.stride(1) != 1:
        raise ValueError("fit: w must be fp32 with unit column stride")
    group = _row_d(d, rows, k, row_group, "fit")
    d = d.contiguous()
    lo = torch.empty(rows, k // block, dtype=torch.float32, device=dev)
    st = torch.empty(rows, k // block, dtype=torch.float32, device=dev)
    _lib.call(
        "hi2_fit_ladder_grouped", _lib.ptr(w), w.stride(0), _lib.ptr(d), _lib.ptr(group), _lib.host_floats(grid), len(grid),
        int(refits), int(n), rows, k, int(block), _lib.ptr(lo), _lib.ptr(st), _lib.stream(dev),
    )
    return lo, st


def quantize_rows(lo, step, nbits: int, block: int, k: int, w=None, d=None, *, want_params=True,
                  want_decoded=False, ldp: int | None = None, want_codes=False, want_sse=False,
                  want_energy=False, row_group=None):
    """Row-wide quantisation of ladders ``lo, step [N, K/block]`` (hi2/encode.py:95-119), decode
    (hi2/format.py:45-60) and, on request, nearest codes / weighted error / energy of ``w``
    (hi2/encode.py:146-157).  Returns a dict of the requested tensors."""
    dev = _lib.need_cuda(lo, step, w, d)
    rows, nb = lo.shape
    lo, step = lo.contiguous(), step.contiguous()
    out = {}
    if want_params:
        out["params"] = torch.empty(rows, nb, 2, dtype=torch.uint8, device=dev)
        out["consts"] = torch.empty(rows, 3, dtype=torch.float16, device=dev)
    if want_decoded:
        ldp = ldp or nb
        # padding stays zero, as the reference's padded ladders do (hi2/hessian.py:279-287)
        make = torch.zeros if ldp != nb else torch.empty
        out["lo_d"] = make(rows, ldp, dtype=torch.float32, device=dev)
        out["step_d"] = make(rows, ldp, dtype=torch.float32, device=dev)
    if want_codes:
        out["codes"] = torch.empty(rows, k, dtype=torch.uint8, device=dev)
    if want_sse:
        out["sse"] = torch.empty(rows, dtype=torch.float32, device=dev)
    if want_energy:
        out["energy"] = torch.empty(rows, dtype=torch.float32, device=dev)
    ldw, group = 0, None
    if w is not None:
        if w.dtype != torch.float32 or w.stride(1) != 1:
            raise ValueError("quantize_rows: w must be fp32 with unit column stride")
        ldw = w.stride(0)
        group = _row_d(d, rows, k, row_group, "quantize_rows")
        d = d.contiguous().float()
    _lib.call(
        "hi2_quantize_rows_grouped", _lib.ptr(lo), _lib.ptr(step), _lib.ptr(w), ldw, _lib.ptr(d), _lib.ptr(group), int(nbits),
        rows, k, int(block), _lib.ptr(out.get("params")), _lib.ptr(out.get("consts")),
        _lib.ptr(out.get("lo_d")), _lib.ptr(out.get("step_d")), ldp or nb, _lib.ptr(out.get("codes")),
        _lib.ptr(out.get("sse")), _lib.ptr(out.get("energy")), _lib.stream(dev),
    )
    return out
