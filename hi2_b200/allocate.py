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


def restrict(t, keep):
    """``t`` with only the candidates ``(nbits, block)`` that ``keep`` accepts (hi2/allocate.py:49-59):
    picks made over the result index its shorter candidate list, which is also what the encoder
    reads.  ``t`` itself when nothing or everything would go."""
    import dataclasses

    kept = [i for i, cand in enumerate(t.candidates) if keep(cand)]
    if not kept or len(kept) == len(t.candidates):
        return t
    rows = torch.tensor(kept, device=t.sse.device)
    return dataclasses.replace(t, sse=t.sse.index_select(0, rows), candidates=[t.candidates[i] for i in kept])


def force_int8(tables: dict, sens: dict | None, top: int):
    """The whole-tensor INT8 rule of hi2/allocate.py:62-76: among the tensors that have INT8
    candidates, the ``top`` most sensitive ones keep ONLY those, every other tensor loses them.
    Returns ``(tables, names of the chosen tensors)``."""
    sens = sens or {}
    eligible = [n for n, t in tables.items() if any(nb == 8 for nb, _ in t.candidates)]
    chosen = sorted(eligible, key=lambda n: -sens.get(n, 1.0))[:top]
    out = {n: restrict(t, (lambda c: c[0] == 8) if n in chosen else (lambda c: c[0] != 8)) for n, t in tables.items()}
    return out, chosen


@dataclass
class Allocation:
    picks: dict  # name -> candidate index per row (int64, on the device of the tables)
    bpw: float
    lam: float
    feasible: bool
    error_ratio: float = float("nan")
    frac_by_bits: dict | None = None


class _Flat:
    """Costs and bits of all tables side by side, ``[C, sum R]`` fp64 on the device.  Built with a
    handful of launches and one read-back whatever the number of tables (a model has hundreds)."""

    def __init__(self, tables, sens, dev):
        self.dev = dev
        self.tables = list(tables)
        cmax = max(len(t.candidates) for t in tables)
        # energies: device scalars of local tables and plain numbers of gathered ones, read once
        lazy = [(i, t.energy) for i, t in enumerate(tables) if isinstance(t.energy, torch.Tensor)]
        energy = [0.0 if isinstance(t.energy, torch.Tensor) else float(t.energy) for t in tables]
        if lazy:
            for (i, _), v in zip(lazy, torch.stack([e.to(dev, torch.float64).reshape(()) for _, e in lazy]).tolist()):
                energy[i] = v
        rows = [t.shape[0] for t in tables]
        self.rows = sum(rows)
        self.spans, off = [], 0
        for t, r in zip(tables, rows):
            self.spans.append((t.name, off, off + r))
            off += r
        # Per table (a few numbers each, built on the host and uploaded as one small matrix): the bits
        # of every candidate, which candidates exist, their widths, and the table's scale; per row
        # they are gathered on the device through the row's table index.
        n_t = len(tables)
        desc = torch.zeros(n_t, 3 * cmax + 2, dtype=torch.float64)
        for i, (t, r, e) in enumerate(zip(tables, rows, energy)):
            k = t.shape[1]
            for ci, (nb, bl) in enumerate(t.candidates):
                desc[i, ci] = candidate_row_bits(nb, bl, k)
                desc[i, cmax + ci] = 1.0
                desc[i, 2 * cmax + ci] = nb
            # the fp32 number a Python scalar becomes in an fp32 product
            desc[i, 3 * cmax] = float(torch.tensor(sens.get(t.name, 1.0) / max(e, 1e-30), dtype=torch.float64).to(torch.float32))
            desc[i, 3 * cmax + 1] = r
        desc = _lib.upload(desc, dev)
        table_of_row = torch.repeat_interleave(torch.arange(n_t, device=dev), desc[:, 3 * cmax + 1].long(),
                                               output_size=self.rows)
        per_row = desc[table_of_row]  # [rows, 3 cmax + 2]
        self.bits = per_row[:, :cmax].T.contiguous()
        self.valid = per_row[:, cmax : 2 * cmax].T > 0.5
        self.nbits_of = per_row[:, 2 * cmax : 3 * cmax].T.long()
        scale_d = per_row[:, 3 * cmax].to(torch.float32)
        parts = []
        for t in tables:
            sse = t.sse.to(dev, torch.float32)
            if sse.shape[0] < cmax:
                pad = torch.full((cmax - sse.shape[0], sse.shape[1]), float("inf"), dtype=torch.float32, device=dev)
                sse = torch.cat([sse, pad])
            parts.append(sse)
        sse_all = parts[0] if len(parts) == 1 else torch.cat(parts, 1)
        # fp32 product with the scalar rounded to fp32 first, then widened: what
        # `scalar * float32_tensor` followed by `.double()` gives
        self.cost = (sse_all * scale_d[None]).double().contiguous()
        self.picks = torch.empty(self.rows, dtype=torch.int64, device=dev)
        self.total = torch.zeros(1, dtype=torch.float64, device=dev)

    def upper_multiplier(self) -> float:
        """``max(1, 2 * max over rows of (cost spread) / (bit spread of the row's table))``: one
        read-back (the reference takes the maximum table by table)."""
        neg, pos = float("-inf"), float("inf")
        hi = torch.where(self.valid, self.cost, torch.full_like(self.cost, neg)).max(0).values
        lo = torch.where(self.valid, self.cost, torch.full_like(self.cost, pos)).min(0).values
        bhi = torch.where(self.valid, self.bits, torch.full_like(self.bits, neg)).max(0).values
        blo = torch.where(self.valid, self.bits, torch.full_like(self.bits, pos)).min(0).values
        slope = 2 * ((hi - lo) / (bhi - blo).clamp_min(1e-9)).max()
        return max(1.0, float(slope.item()))

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
    floor = torch.where(flat.valid, flat.cost, torch.full_like(flat.cost, float("inf"))).min(0).values.sum()
    widths = sorted({nb for t in flat.tables for nb, _ in t.candidates})
    nbits = flat.nbits_of.gather(0, picks[None])[0]
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

    lam_hi = flat.upper_multiplier()
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


def allocate_by_quality(tables, max_error_ratio: float, sensitivity: dict | None = None,
                        iters: int = 80) -> Allocation:
    """The fewest bits whose weighted error stays within ``max_error_ratio`` times the best the allowed
    candidates can reach (1.0 = every row at its most accurate candidate); the model-wide bits per
    weight is the result, not an input (hi2/allocate.py:156-209).  Same geometric bisection on the
    multiplier as the reference, one solve and two small read-backs per step; ``feasible`` is False
    when even the most accurate assignment is over the error budget (then that assignment is
    returned)."""
    sens = sensitivity or {}
    dev = _lib.need_cuda(*[t.sse for t in tables])
    total_w = sum(t.shape[0] * t.shape[1] for t in tables)
    overhead = _overhead(tables)
    flat = _Flat(tables, sens, dev)
    best_cost = torch.where(flat.valid, flat.cost, torch.full_like(flat.cost, float("inf"))).min(0).values.sum()
    budget = max_error_ratio * float(best_cost.item())

    def solve(lam):
        picks, bits = flat.solve(lam)
        return picks, bits, float(flat.cost.gather(0, picks[None])[0].sum().item())

    lam_hi = flat.upper_multiplier()
    lo, hi = lam_hi * 1e-12, lam_hi  # a larger multiplier buys fewer bits with more error
    picks, bits_total, err = solve(lo)
    best_lam, feasible = lo, err <= budget
    if feasible:
        for _ in range(iters):
            mid = (lo * hi) ** 0.5
            p, b, e = solve(mid)
            if e <= budget:
                lo, picks, bits_total, best_lam = mid, p, b, mid
            else:
                hi = mid
    ratio, frac = _summary(flat, picks)
    return Allocation(flat.split(picks), (bits_total + overhead) / total_w, best_lam, feasible, ratio, frac)
