"""Global allocation of ``(nbits, block)`` per row on B200 (hi2/allocate.py:212-261).

The cost tables never leave the device: each multiplier of the bisection is one kernel launch
(first-minimum argmin of ``cost + lam * bits`` in fp64 plus the exact sum of the picked bits) and
a few bytes back to the host, which keeps the reference's bisection (geometric midpoints in
Python floats, 80 iterations) and therefore its picks bit for bit; five bisection steps share
one launch and one read-back.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib

ROW_OVERHEAD_BITS = 48 + 2 + 1  # row constants + block-size flag + width flag


def candidate_row_bits(nbits: int, block: int, k: int) -> float:
    return nbits * k + 16 * k / block


def row_overhead_bits(t) -> int:
    widths = len({nb for nb, _ in t.candidates})
    return ROW_OVERHEAD_BITS - 1 + max(1, math.ceil(math.log2(max(widths, 1))))


def _overhead(tables) -> int:
    return sum(
        row_overhead_bits(t) * t.shape[0]
        + t.shape[1] // 16
        + (16 * t.shape[1] if t.col_scale is not None else 0)
        for t in tables
    )


@dataclass
class Allocation:
    picks: dict  # name -> candidate index per row (int64, on the device of the tables)
    bpw: float
    lam: float
    feasible: bool
    error_ratio: float = float("nan")
    frac_by_bits: dict | None = None


class _Flat:
    """Costs and bits of all tables side by side, ``[C, sum R]`` fp64 on the device."""

    def __init__(self, tables, sens, dev):
        self.dev = dev
        cmax = max(len(t.candidates) for t in tables)
        costs, bits, self.spans, self.per_table = [], [], [], []
        off = 0
        for t in tables:
            r, k = t.shape
            scale = sens.get(t.name, 1.0) / max(float(t.energy), 1e-30)
            # fp32 product with the scalar rounded to fp32 first, then widened: what
            # `scalar * float32_tensor` followed by `.double()` gives
            cost = (t.sse.to(dev, torch.float32) * scale).double()
            b = torch.tensor(
                [candidate_row_bits(nb, bl, k) for nb, bl in t.candidates],
                dtype=torch.float64, device=dev,
            )
            self.per_table.append((t, cost, b))
            pad = cmax - cost.shape[0]
            costs.append(torch.cat([cost, torch.full((pad, r), float("inf"), dtype=torch.float64,
                                                      device=dev)]))
            bits.append(torch.cat([b, torch.zeros(pad, dtype=torch.float64, device=dev)])
                        .unsqueeze(1).expand(cmax, r))
            self.spans.append((t.name, off, off + r))
            off += r
        self.cost = torch.cat(costs, 1).contiguous()
        self.bits = torch.cat(bits, 1).contiguous()
        self.rows = off
        self.picks = torch.empty(off, dtype=torch.int64, device=dev)
        self.total = torch.zeros(1, dtype=torch.float64, device=dev)

    def solve(self, lam: float):
        """``(picks [sum R] on the device, total picked bits)`` for one multiplier."""
        self.total.zero_()
        picks = torch.empty_like(self.picks)
        _lib.call(
            "hi2_allocate_solve", _lib.ptr(self.cost), _lib.ptr(self.bits), self.cost.shape[0],
            self.rows, float(lam), _lib.ptr(picks), _lib.ptr(self.total), _lib.stream(self.dev),
        )
        return picks, float(self.total.item())

    def bits_of(self, lams: list[float]) -> list[float]:
        """Total picked bits under each of up to 32 multipliers, one launch and one read-back."""
        import ctypes

        totals = torch.zeros(len(lams), dtype=torch.float64, device=self.dev)
        arr = (ctypes.c_double * len(lams))(*lams)
        _lib.call(
            "hi2_allocate_bits", _lib.ptr(self.cost), _lib.ptr(self.bits), self.cost.shape[0], self.rows,
            arr, len(lams), _lib.ptr(totals), _lib.stream(self.dev),
        )
        return totals.tolist()

    def split(self, picks):
        return {name: picks[a:b].clone() for name, a, b in self.spans}


def _summary(flat: _Flat, picks):
    """``(error / floor, fraction of rows by width)`` with two read-backs for all tables."""
    err = flat.cost.gather(0, picks[None])[0].sum()
    floor = flat.cost.min(0).values.sum()
    widths = sorted({nb for t, _, _ in flat.per_table for nb, _ in t.candidates})
    nbits = torch.cat([
        torch.tensor([nb for nb, _ in t.candidates], device=flat.dev)[picks[a:b]]
        for (t, _, _), (_, a, b) in zip(flat.per_table, flat.spans)
    ])
    counts = torch.stack([(nbits == nb).sum() for nb in widths])
    head = torch.stack([err, floor]).tolist()
    counts = counts.tolist()
    return head[0] / max(head[1], 1e-30), {nb: n / max(flat.rows, 1) for nb, n in zip(widths, counts)}


def allocate_global(tables, target_bpw: float, sensitivity: dict | None = None,
                    iters: int = 80) -> Allocation:
    """Minimise ``sum_t s_t * sse_t / energy_t`` under a model-wide bits-per-weight target."""
    sens = sensitivity or {}
    dev = _lib.need_cuda(*[t.sse for t in tables])
    total_w = sum(t.shape[0] * t.shape[1] for t in tables)
    overhead = _overhead(tables)
    budget = target_bpw * total_w - overhead
    flat = _Flat(tables, sens, dev)

    slopes = []
    for _t, cost, bits in flat.per_table:
        span_b = (bits.max() - bits.min()).clamp_min(1e-9)
        slopes.append(2 * ((cost.max(0).values - cost.min(0).values) / span_b).max())
    lam_hi = max(1.0, max(torch.stack(slopes).tolist()))  # one read-back for all tables
    lo, hi = lam_hi * 1e-12, lam_hi

    def done(p, b, lam, ok):
        ratio, frac = _summary(flat, p)
        return Allocation(flat.split(p), (b + overhead) / total_w, lam, ok, ratio, frac)

    picks, bits_total = flat.solve(hi)
    if bits_total > budget:  # even the cheapest assignment is over target
        return done(picks, bits_total, hi, False)
    best = flat.solve(lo)
    if best[1] <= budget:  # even the most accurate one fits
        return done(best[0], best[1], lo, True)
    # The reference bisects one multiplier per step.  The next five steps can only visit the 31
    # midpoints of a depth-5 tree, so their bit totals are fetched in one launch and the steps are
    # then taken on the host exactly as the reference takes them (same Python-float midpoints).
    best_lam = hi
    left = iters
    while left > 0:
        depth = min(5, left)
        nodes = {(): (lo, hi)}  # path of outcomes (True = fits) -> bracket before that step
        lams, order = [], []
        for level in range(depth):
            for path in [q for q in nodes if len(q) == level]:
                a, b = nodes[path]
                mid = (a * b) ** 0.5
                order.append(path)
                lams.append(mid)
                nodes[path + (True,)] = (a, mid)
                nodes[path + (False,)] = (mid, b)
        totals = dict(zip(order, zip(lams, flat.bits_of(lams))))
        path = ()
        for _ in range(depth):
            mid, b = totals[path]
            fits = b <= budget
            if fits:
                hi, bits_total, best_lam = mid, b, mid
            else:
                lo = mid
            path = path + (fits,)
        left -= depth
    if best_lam != lam_hi:
        picks, bits_total = flat.solve(best_lam)
    return done(picks, bits_total, best_lam, True)
