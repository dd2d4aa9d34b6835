"""Per-tensor tabulate and encode stages on one B200 (callers of the kernels; the shapes of
hi2/calibrate.py:37-81, :96-111, :212-270, :274-424 with the device kept as the home of the data).

Differences from the reference's orchestration, none of which changes a result:

* one process drives one GPU, so there is no row sharding over an executor: the ``ex`` argument
  is accepted and ignored (matrices, not rows, are what ``hi2_b200.dist`` spreads over GPUs);
* weights are cast, scaled and rotated in one kernel pass, straight from bf16 / fp16;
* a table costs two launches per candidate and returns ``sse`` on the device;
* the Hessian of a shared input is transformed and factorised once per ``sigma_id``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import _lib
from .encode import encode_rows
from .format import GROUP, HI2Tensor, assemble, fwht_groups
from .stats import ColumnStats

ALL_CANDIDATES = [(nb, b) for nb in (2, 4) for b in (16, 32, 64)]
INT8_CANDIDATES = [(8, 32), (8, 64)]
SELECTABLE = ALL_CANDIDATES + INT8_CANDIDATES


ROTATION_ROWS = 1024  # rows sampled to decide the rotation per 64-column chunk
CHUNK = 64


@dataclass
class Config:
    candidates: list = field(default_factory=lambda: list(ALL_CANDIDATES))
    rotation: str = "on"  # on | off | auto (per 64-column chunk, decided on a row sample)
    smooth: float = 0.5
    smooth_search: tuple = ()
    rounding: str = "gptq"  # gptq | nearest
    sequential: bool = False
    damp: float = 0.01
    act_order: bool = False
    refine_passes: int = 0
    effort: str = "normal"
    expert_min_tokens: float = 2.0


@dataclass
class TensorTable:
    name: str
    shape: tuple
    had: torch.Tensor  # uint8 [K/16]
    sse: torch.Tensor  # float32 [C, R] (on the device)
    candidates: list
    energy: float | torch.Tensor  # sum d * w^2; a 0-dim device tensor until someone reads it
    n_tokens: int
    col_scale: torch.Tensor | None = None  # fp16 [K]; on the device when the table was built there
    # the (smoothing vector, flags) objects handed to build_table, when it was handed some: tables and
    # factor jobs made from the same objects are recognised as sharing a transform without reading
    # the vector back from the device
    transform_ref: tuple | None = None


def candidate_row_bits(nbits: int, block: int, k: int) -> float:
    return nbits * k + 16 * k / block


def _weights(stats: ColumnStats | None, k: int, flags, device, inv_scale=None) -> torch.Tensor:
    if stats is None:
        return torch.ones(k, device=device)
    return stats.diag(flags, inv_scale).to(device)


def smoothing_scale(stats: ColumnStats | None, alpha: float) -> torch.Tensor | None:
    """fp16 smoothing vector ``s_j = clamp((d_j / geomean d)^(alpha/2), 0.05, 20)`` or None."""
    if alpha <= 0 or stats is None or stats.n == 0:
        return None
    d = stats.diag().clamp_min(1e-12)
    s = (d / d.log().mean().exp()).pow(alpha / 2).clamp(0.05, 20.0)
    return s.to(torch.float16)


def _sample_rows(w: torch.Tensor) -> torch.Tensor:
    """Every (R // 1024)-th row, at most 1024 of them (hi2/calibrate.py:125)."""
    r = w.shape[0]
    return w[torch.arange(0, r, max(1, r // ROTATION_ROWS), device=w.device)[:ROTATION_ROWS]]


def _chunk_errors(wt, d, enc, block: int) -> torch.Tensor:
    """Weighted error of an encode per 64-column chunk, summed over the rows
    (hi2/calibrate.py:140-157): codes and parameter bytes come from the kernels, the fp16 decode
    and the sums are elementwise tensor math on the device."""
    from .format import decode_params, ladder_dequantize

    r, k = wt.shape
    lo, step = decode_params(enc.params[..., 0], enc.params[..., 1], enc.consts[:, 0:1], enc.consts[:, 1:2],
                             enc.consts[:, 2:3])
    rec = ladder_dequantize(enc.codes.reshape(r, k // block, block), lo.float(), step.float(), torch.float32).float()
    return (d.reshape(1, k // block, block) * (rec - wt.reshape(r, k // block, block)) ** 2).sum((0, 2))


def choose_rotation(w: torch.Tensor, stats: ColumnStats | None, cfg: Config, device=None,
                    inv_scale: torch.Tensor | None = None) -> torch.Tensor:
    """Rotation flags ``[K/16]`` uint8, uniform over rows (hi2/calibrate.py:114-137).  ``auto``
    encodes a sample of the rows at INT2 / block 64 (effort fast) with and without the rotation
    and keeps, per 64-column chunk, whichever leaves the smaller activation-weighted error."""
    k = w.shape[1]
    ng = k // GROUP
    if cfg.rotation == "off":
        return torch.zeros(ng, dtype=torch.uint8)
    if cfg.rotation == "on":
        return torch.ones(ng, dtype=torch.uint8)
    if cfg.rotation != "auto":
        raise ValueError(f"rotation must be on, off or auto (got {cfg.rotation!r})")
    dev = _lib.need_cuda(w) if device is None else torch.device(device)
    ws = _sample_rows(w).to(dev, torch.float32)
    err = []
    for rot in (0, 1):
        fl = torch.full((ng,), rot, dtype=torch.uint8)
        wt = fwht_groups(ws, fl) if rot else ws
        d = _weights(stats, k, fl, dev, inv_scale)
        err.append(_chunk_errors(wt, d, encode_rows(wt, d, 2, CHUNK, "fast"), CHUNK))
    return (err[1] < err[0]).to(torch.uint8).repeat_interleave(CHUNK // GROUP).cpu()


def _fixed_transform(ws: list, stats: ColumnStats | None, cfg: Config, alpha: float):
    """``(smoothing vector for exponent alpha, flags)`` (hi2/calibrate.py:160-170); with ``auto``
    the flags are chosen on the smoothed rows of all the Linears together."""
    s16 = smoothing_scale(stats, alpha)
    if cfg.rotation != "auto":
        return s16, choose_rotation(ws[0], stats, cfg)
    dev = _lib.need_cuda(*ws)
    scale = None if s16 is None else s16.to(dev, torch.float32)
    # the reference samples the rows of the Linears stacked on top of each other; the same rows are
    # picked here without stacking the full matrices
    total = sum(w.shape[0] for w in ws)
    idx = torch.arange(0, total, max(1, total // ROTATION_ROWS))[:ROTATION_ROWS]
    parts, off = [], 0
    for w in ws:
        mine = idx[(idx >= off) & (idx < off + w.shape[0])] - off
        if mine.numel():
            rows = w[mine.to(w.device)].float()
            parts.append(rows if scale is None else rows * scale)
        off += w.shape[0]
    return s16, choose_rotation(torch.cat(parts), stats, cfg, dev, None if scale is None else 1.0 / scale)


def transform_error(ws: list, stats: ColumnStats, s16, had: torch.Tensor) -> float:
    """Weighted INT2 / block-32 error (effort fast) of a row sample of ``ws`` under one transform,
    relative to their weighted energy (hi2/calibrate.py:173-191)."""
    dev = _lib.need_cuda(*ws)
    inv = None if s16 is None else 1.0 / s16.to(dev, torch.float32)
    sse = energy = None
    for w in ws:
        wt = stored_rows(_sample_rows(w), s16, had)
        d = _weights(stats, w.shape[1], had, dev, inv)
        enc = encode_rows(wt, d, 2, 32, "fast", want_codes=False, want_energy=True)
        sse = enc.sse.sum() if sse is None else sse + enc.sse.sum()
        energy = enc.energy.sum() if energy is None else energy + enc.energy.sum()
    return float(sse) / max(float(energy), 1e-30)


def shared_transform(ws: list, stats: ColumnStats | None, cfg: Config, ex=None):
    """``(smoothing vector, rotation flags)`` for Linears that read the same input (q/k/v,
    gate/up): one vector from the shared statistics, one set of flags chosen on their rows
    together; with ``cfg.smooth_search`` the exponent with the lowest :func:`transform_error`
    wins, the first one on a tie (hi2/calibrate.py:194-209)."""
    del ex
    if not cfg.smooth_search or stats is None or stats.n == 0:
        return _fixed_transform(ws, stats, cfg, cfg.smooth)
    best = None
    for alpha in dict.fromkeys((cfg.smooth, *cfg.smooth_search)):
        s16, had = _fixed_transform(ws, stats, cfg, alpha)
        err = transform_error(ws, stats, s16, had)
        if best is None or err < best[0]:
            best = (err, s16, had)
    return best[1], best[2]


def stored_rows(w: torch.Tensor, s16: torch.Tensor | None, had: torch.Tensor) -> torch.Tensor:
    """``H(W * s)`` as fp32 ``[R, K]``: cast, smoothing multiply and rotation in one pass."""
    if w.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        w = w.float()
    scale = None if s16 is None else s16.to(w.device, torch.float32)
    return fwht_groups(w, had, col_scale=scale, out_dtype=torch.float32)


def build_table(name: str, w: torch.Tensor, stats: ColumnStats | None, cfg: Config, ex=None,
                transform=None, n_tokens: int | None = None) -> TensorTable:
    """Activation-weighted squared error of every row at every candidate ``(nbits, block)``."""
    del ex
    dev = _lib.need_cuda(w)
    r, k = w.shape
    if transform is None and cfg.smooth_search:
        transform = shared_transform([w], stats, cfg)
    if transform is None:
        s16 = smoothing_scale(stats, cfg.smooth)
        if cfg.rotation in ("on", "off"):
            had = choose_rotation(w, stats, cfg)
        else:  # the flags are chosen on the smoothed rows
            scale = None if s16 is None else s16.to(dev, torch.float32)
            rows = _sample_rows(w).float()
            had = choose_rotation(rows if scale is None else rows * scale, stats, cfg, dev,
                                  None if scale is None else 1.0 / scale)
    else:
        s16, had = transform
        s16 = None if s16 is None else s16.clone()
        had = had.clone()
    given = tuple(transform) if transform is not None else None
    wt = stored_rows(w, s16, had)
    inv = None if s16 is None else 1.0 / s16.to(dev, torch.float32)
    d = _weights(stats, k, had, dev, inv)
    sse, energy = [], None
    for i, (nb, b) in enumerate(cfg.candidates):
        enc = encode_rows(wt, d, nb, b, cfg.effort, want_codes=False, want_energy=(i == 0))
        sse.append(enc.sse)
        if i == 0:
            energy = enc.energy
    # nothing is read back here: the smoothing vector stays where it was computed (the device) and
    # the energy is a device scalar, so the host can queue the next table while this one runs
    return TensorTable(
        name, (r, k), had.cpu(), torch.stack(sse), list(cfg.candidates), energy.sum(),
        n_tokens if n_tokens is not None else (stats.n if stats else 0), s16,
        transform_ref=given,
    )


def build_tables_grouped(items: list, cfg: Config) -> list:
    """:func:`build_table` for several tensors of ONE shape that read different inputs (the experts of
    a layer): ``items`` holds ``(name, w [R, K], stats, (smoothing vector, flags), n_tokens)`` per
    tensor.  The stored rows of all of them lie one after the other in one buffer, their column
    weights form a ``[G, K]`` matrix, and every candidate costs two launches for the whole group
    instead of two per tensor; per row the arithmetic is that of :func:`build_table`.  Tables come
    back in the order of ``items`` (their ``sse`` are views of the group's table)."""
    if cfg.smooth_search or len(items) < 2 or any(it[3] is None for it in items):
        return [build_table(name, w, st, cfg, transform=tr, n_tokens=n) for name, w, st, tr, n in items]
    dev = _lib.need_cuda(*[it[1] for it in items])
    r, k = items[0][1].shape
    if any(tuple(it[1].shape) != (r, k) for it in items):
        raise ValueError("build_tables_grouped: the tensors of a group must have one shape")
    wt = torch.empty(len(items) * r, k, dtype=torch.float32, device=dev)
    d = torch.empty(len(items), k, dtype=torch.float32, device=dev)
    kept = []
    for e, (_, w, st, (s16, had), _) in enumerate(items):
        if w.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            w = w.float()
        scale = None if s16 is None else s16.to(dev, torch.float32)
        fwht_groups(w, had, col_scale=scale, out_dtype=torch.float32, out=wt[e * r : (e + 1) * r])
        d[e] = _weights(st, k, had, dev, None if scale is None else 1.0 / scale)
        kept.append((None if s16 is None else s16.clone(), had.clone()))
    row_group = torch.arange(len(items), device=dev, dtype=torch.int32).repeat_interleave(r)
    sse, energy = [], None
    for i, (nb, b) in enumerate(cfg.candidates):
        enc = encode_rows(wt, d, nb, b, cfg.effort, want_codes=False, want_energy=(i == 0), row_group=row_group)
        sse.append(enc.sse)
        if i == 0:
            energy = enc.energy
    sse = torch.stack(sse)
    out = []
    for e, (name, _, st, tr, n) in enumerate(items):
        rows = slice(e * r, (e + 1) * r)
        out.append(TensorTable(name, (r, k), kept[e][1].cpu(), sse[:, rows], list(cfg.candidates), energy[rows].sum(),
                               n if n is not None else (st.n if st else 0), kept[e][0], transform_ref=tuple(tr)))
    return out


@dataclass
class EncodeRequest:
    """One tensor for :func:`encode_many`; requests with the same ``sigma_id``, smoothing vector
    and flags share one transformed Hessian and one factor."""

    w: torch.Tensor  # [R, K] original basis (any float dtype, on the device)
    stats: ColumnStats | None
    table: TensorTable
    picks: torch.Tensor  # [R] candidate index per row
    sigma: torch.Tensor | None = None  # [K, K] mean second moment, or a raw sum with sigma_n
    sigma_id: str | None = None
    comp_out: dict | None = None
    sigma_n: int = 1  # divide sigma by this (lets the raw sum be passed without a copy)
    groups: tuple | None = None  # (row order, rows per candidate) from :func:`group_rows`


def _transform_key(col_scale, had):
    cs = None if col_scale is None else col_scale.detach().cpu().to(torch.float16).numpy().tobytes()
    return cs, had.detach().cpu().to(torch.uint8).numpy().tobytes()


def _job_key(job):
    if job.transform_key is None:
        job.transform_key = _transform_key(*job.transform)
    return job.transform_key


REFINE_STREAMS = 8
_refine_streams: dict = {}


def _refine_stream(dev: torch.device, i: int) -> torch.cuda.Stream:
    """Side streams for the refinement loops, made once per device and reused (the caching allocator
    keeps a pool per stream)."""
    key = (dev.index, i)
    if key not in _refine_streams:
        _refine_streams[key] = torch.cuda.Stream(dev)
    return _refine_streams[key]


def _factor_key(req: EncodeRequest, i: int):
    t = req.table
    sid = req.sigma_id if req.sigma_id is not None else f"#{i}"
    if t.transform_ref is not None:  # no read-back: the objects the table was built from stand for their content
        return (sid, "ref", id(t.transform_ref[0]), id(t.transform_ref[1]))
    return (sid, *_transform_key(t.col_scale, t.had))


def _same_transform(t: TensorTable, job) -> bool:
    """Whether a factor job started earlier belongs to the transform of table ``t``."""
    ref = t.transform_ref
    if ref is not None and job.transform is not None and ref[0] is job.transform[0] and ref[1] is job.transform[1]:
        return True
    return _job_key(job) == _transform_key(t.col_scale, t.had)


def group_rows(reqs: list) -> None:
    """Rows of every request grouped by candidate, with ONE read-back for all of them: a stable sort
    of the picks and their histogram, left in ``req.groups``.  (A ``nonzero()`` per request and
    candidate costs a host synchronisation each: 42 per decoder layer, 1152 per layer of 64 experts;
    so does ``torch.bincount``.)  :func:`encode_many` calls this for requests that come without;
    a caller that encodes a model in several calls groups all requests once, while the device is idle
    after the allocation anyway, and the calls then start without waiting for the device."""
    todo = [r for r in reqs if r.groups is None]
    if not todo:
        return
    hist, by_dev = [], {}
    for i, r in enumerate(todo):
        dev = _lib.need_cuda(r.w)
        picks = r.picks if r.picks.device == dev else _lib.upload(r.picks, dev)
        c = len(r.table.candidates)
        hist.append((picks[None, :] == torch.arange(c, device=dev)[:, None]).sum(1))
        r.groups = (torch.argsort(picks, stable=True), None)
        by_dev.setdefault(dev, []).append(i)
    cmax = max(h.numel() for h in hist)
    for idxs in by_dev.values():
        table = torch.stack([torch.nn.functional.pad(hist[i], (0, cmax - hist[i].numel())) for i in idxs])
        for i, row in zip(idxs, table.tolist()):
            todo[i].groups = (todo[i].groups[0], row)


def factor_for(sigma, sigma_n, col_scale, had, cfg: Config):
    """Enqueue basis change and inverse factor of one shared input on the current stream.
    Returns ``(d, job, hs)``: ladder weights ``diag(Hs)``, the :class:`FactorJob`, and ``Hs``."""
    from .hessian import FactorJob, transform_sigma

    if cfg.act_order:
        raise NotImplementedError("prefactoring with act_order: let encode_many factorise")
    hs, d = transform_sigma(sigma, col_scale, had, denom=float(max(sigma_n, 1)), return_diag=True)
    d_ready = torch.cuda.Event()
    d_ready.record()
    job = FactorJob(hs, cfg.damp)
    job.d_ready = d_ready
    # A factor belongs to ONE (input, smoothing vector, flags).  The key is only made when someone
    # compares it (encode_many): reading the smoothing vector back here would make the host wait
    # for the factorisation that was just enqueued.
    job.transform = (col_scale, had)
    job.transform_key = None
    return d, job, hs


def encode_many(reqs: list[EncodeRequest], cfg: Config, ex=None, to_host: bool = True,
                factors: dict | None = None, timing: list | None = None) -> list[HI2Tensor]:
    """Encode several tensors with their allocator picks (hi2/calibrate.py:297-424): all GPTQ
    candidate groups of all tensors go through one batched column loop; the Hessian transform
    and factorisation happen once per distinct input."""
    del ex
    from .hessian import GptqJob, encode_jobs_gptq, inverse_factor, transform_sigma

    # ``factors`` (optional): {sigma_id: (d, FactorJob, hs)} from :func:`factor_for`, started earlier
    # on side streams so the factorisations overlap the tables
    ready = factors or {}
    factors = {}
    waits: dict = {}
    pieces: dict[int, list] = {}
    jobs, where, refine_with = [], [], []
    stored: dict[int, torch.Tensor] = {}
    group_rows(reqs)
    for ri, r in enumerate(reqs):
        dev = _lib.need_cuda(r.w)
        t = r.table
        had, k = t.had, t.shape[1]
        wt = stored_rows(r.w, t.col_scale, had)
        stored[ri] = wt
        use_gptq = cfg.rounding == "gptq" and r.sigma is not None
        if use_gptq:
            fk = _factor_key(r, ri)
            if fk not in factors and r.sigma_id in ready and _same_transform(t, ready[r.sigma_id][1]):
                # started earlier on a side stream for this very (input, smoothing vector, flags):
                # order after it on the device, never on the host, so the narrow matrices are rounded
                # while the widest factor is still being computed.  d is complete at d_ready; U only
                # at job.done, which every GptqJob below carries as its ``wait`` event.
                d, job, hs = ready[r.sigma_id]
                torch.cuda.current_stream(dev).wait_event(job.d_ready)
                if cfg.refine_passes and hs is None:  # the prefactoring released it
                    hs = transform_sigma(r.sigma.to(dev), t.col_scale, had, denom=float(max(r.sigma_n, 1)))
                factors[fk] = (d, job.first_attempt(), None, hs if cfg.refine_passes else None)
                waits[fk] = job
            if fk not in factors:
                hs, d = transform_sigma(r.sigma.to(dev), t.col_scale, had, denom=float(max(r.sigma_n, 1)),
                                        return_diag=True)
                perm = None
                if cfg.act_order:
                    perm = torch.argsort(d, descending=True)
                    hs = hs[perm][:, perm].contiguous()
                u = inverse_factor(hs, cfg.damp)
                keep = hs if cfg.refine_passes and perm is None else None
                factors[fk] = (d, u, perm, keep)
            d, u, perm, hs_keep = factors[fk]
        else:
            inv = None if t.col_scale is None else 1.0 / t.col_scale.to(dev, torch.float32)
            d = _weights(r.stats, k, had, dev, inv)
        out = pieces.setdefault(ri, [])
        (order, counts), off = r.groups, 0
        for ci, (nb, b) in enumerate(t.candidates):
            n_ci = int(counts[ci])
            rows = order[off : off + n_ci]  # ascending row indices of this candidate (the sort is stable)
            off += n_ci
            if n_ci == 0:
                continue
            if use_gptq:
                jobs.append(GptqJob(wt[rows], d, u, nb, b, perm, waits[fk].done if fk in waits else None))
                where.append((ri, rows))
                refine_with.append(hs_keep if r.comp_out is None else None)
                out.append(None)
            else:
                enc = encode_rows(wt[rows], d, nb, b, cfg.effort)
                out.append((rows, enc.codes, enc.params, enc.consts, nb, b))
    want = any(reqs[ri].comp_out is not None for ri, _ in where)
    encs = encode_jobs_gptq(jobs, cfg.effort, comp=want, timing=timing) if jobs else []
    if any(not job.succeeded() for job in waits.values()):
        # a first attempt met a non-positive pivot: redo everything on the synchronous path, which
        # retries with more damping (hi2/hessian.py:78-86)
        return encode_many(reqs, cfg, to_host=to_host, factors=None, timing=timing)
    if cfg.refine_passes:
        for job in waits.values():
            torch.cuda.current_stream().wait_event(job.done)
    if any(h is not None for h in refine_with):
        from .refine import refine_groups

        # Rows that share a transformed Hessian (all candidates of a tensor, and all tensors reading
        # the same input) go through one column loop; the loops of different inputs are chains of
        # short dependent launches, so they run side by side on streams, nothing read back in between.
        by_hs: dict[int, list[int]] = {}
        for x in range(len(where)):
            if refine_with[x] is not None:
                by_hs.setdefault(id(refine_with[x]), []).append(x)
        # longest loops first, each on the stream with the least work so far: a loop costs its number
        # of column blocks times a step that grows with rows x width
        def cost(xs):
            k = jobs[xs[0]].w.shape[1]
            return (k / 128) * (0.1 + 3e-9 * k * sum(jobs[x].w.shape[0] for x in xs))

        load = [0.0] * REFINE_STREAMS
        pending = []
        for xs in sorted(by_hs.values(), key=cost, reverse=True):
            dev = _lib.need_cuda(jobs[xs[0]].w)
            si = load.index(min(load))
            load[si] += cost(xs)
            main, side = torch.cuda.current_stream(dev), _refine_stream(dev, si)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                new, status = refine_groups([(jobs[x].w, encs[x], jobs[x].nbits, jobs[x].block) for x in xs],
                                            refine_with[xs[0]], cfg.refine_passes, wait=False)
            pending.append((xs, new, status, main, side))
        for xs, new, status, main, side in pending:
            main.wait_stream(side)
            for x, codes in zip(xs, new):
                codes.record_stream(main)
                encs[x] = type(encs[x])(codes, encs[x].params, encs[x].consts, encs[x].sse, encs[x].comp)
        words = [st for _, _, st, _, _ in pending if st is not None]
        if words and any(torch.cat(words).tolist()):
            raise RuntimeError("refine: a bounded device-side wait ran out in a tensor-core product")
    slot = {ri: iter([j for j, p in enumerate(pieces[ri]) if p is None]) for ri in pieces}
    comps: dict[int, list] = {}
    for (ri, rows), enc, job in zip(where, encs, jobs):
        pieces[ri][next(slot[ri])] = (rows, enc.codes, enc.params, enc.consts, job.nbits, job.block)
        if reqs[ri].comp_out is not None:
            comps.setdefault(ri, []).append((rows, enc.comp))
    out = []
    flags: dict = {}  # one out-of-ladder flag per device for all tensors, read once
    for ri, r in enumerate(reqs):
        t = r.table
        bad = None
        if pieces.get(ri):
            dev = _lib.need_cuda(r.w)
            if dev not in flags:
                flags[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
            bad = flags[dev]
        if r.comp_out is not None:
            full = stored[ri].clone()  # nearest rounding: the stored-basis weights themselves
            for rows, c in comps.get(ri, []):
                full[rows] = c
            r.comp_out["comp"] = full
        cand = torch.tensor(t.candidates)
        picks = r.picks.cpu()
        out.append(
            assemble(pieces[ri], cand[picks, 0], cand[picks, 1], t.had, t.shape[1], t.col_scale,
                     to_host=to_host, bad=bad, wait=False)
        )
    if any(int(f.item()) for f in flags.values()):  # also the one wait for the copies to the host queued above
        raise ValueError("code outside the ladder")
    return out


def encode_with_picks(w, stats, table, picks, cfg: Config, ex=None, sigma=None, comp_out=None) -> HI2Tensor:
    """Encode rows with the candidate index ``picks[r]`` chosen by the allocator."""
    req = EncodeRequest(w, stats, table, picks, sigma, comp_out=comp_out)
    return encode_many([req], cfg, ex)[0]
