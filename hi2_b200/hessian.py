"""Hessian statistics and error-compensated rounding on B200 (interface of hi2/hessian.py).

``HessianStats`` (:26-47), ``transform_sigma`` (:50-68), ``inverse_factor`` (:71-86), ``GptqJob``
(:178-188), ``encode_jobs_gptq`` (:359-416) and ``encode_rows_gptq`` (:419-443) keep the
reference's names, arguments and results.  Underneath:

* the second moment is a TMA-fed tcgen05 product with fp32 accumulation (csrc/hessian.cu);
* the basis change is one tile kernel (csrc/sigma.cu);
* the inverse factor is one fp64 blocked factorisation plus triangular inverse (csrc/cholinv.cu)
  with the reference's damping retries driven from here;
* GPTQ fits the ladders once (csrc/ladder.cu), then runs the whole column loop, block kernel and
  trailing update per 128 columns, as one enqueue without host synchronisation (csrc/gptq.cu).

There is no torch loop: ``backend="torch"`` raises.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from . import _lib, gptq_kernel
from . import ladder_kernel as _ladder
from .encode import EFFORT, Encoded
from .format import GROUP

BLOCK_COLUMNS = 128  # lazy-update block of GPTQ
ROW_ELEMS = 1 << 26  # rows per unit, as in the reference (results do not depend on it)
BATCH_ELEMS = int(os.environ.get("HI2_BATCH_ELEMS", 1 << 27))

class _Scratch:
    """Grow-only scratch buffers, one per (device, stream): a kernel's scratch is only ever touched
    by work queued on the stream it was allocated for, so when a buffer is outgrown and dropped the
    caching allocator (which hands a block back only to later work of the same stream) cannot give
    it to anybody while its last user is still running, and two streams never share a buffer.  The
    registry belongs to the process, not to a call, but holds nothing a caller could observe."""

    def __init__(self):
        self._buffers: dict = {}

    def get(self, dev: torch.device, nbytes: int) -> torch.Tensor:
        stream = torch.cuda.current_stream(dev)
        key = (stream.device.index, stream.cuda_stream)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < nbytes:
            self._buffers.pop(key, None)
            del buf
            buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
            self._buffers[key] = buf
        return buf


_scratch = _Scratch()


def _workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch of at least ``nbytes`` for a kernel launched on the current stream of ``dev``."""
    return _scratch.get(dev, nbytes)


_side_streams: dict = {}


def _side_stream(dev: torch.device, i: int) -> torch.cuda.Stream:
    """Side streams are created once per device and reused (the caching allocator pools memory
    per stream)."""
    key = (dev.index, i)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(dev)
    return _side_streams[key]


class HessianStats:
    """Full second moment ``sum x x^T`` of a Linear's input (fp32, ``[K, K]``)."""

    def __init__(self, k: int, device="cuda", out: torch.Tensor | None = None):
        """``out`` (optional): a contiguous fp32 ``[k, k]`` tensor to accumulate into (it is zeroed),
        e.g. one slice of a stack that a reduce-scatter will sum over the ranks."""
        self.k = k
        if out is not None:
            if out.shape != (k, k) or out.dtype != torch.float32 or not out.is_contiguous():
                raise ValueError("out must be a contiguous fp32 [k, k] tensor")
            self.S = out.zero_()
        else:
            self.S = torch.zeros(k, k, dtype=torch.float32, device=device)
        self.n = 0
        self._unchecked: list = []  # status words of launches whose outcome nobody has read yet

    def check(self) -> None:
        """Raise if a launch made with ``defer_check=True`` gave up on a bounded device-side wait
        (synchronises with those launches)."""
        pending, self._unchecked = self._unchecked, []
        if not pending:
            return
        for status in torch.cat([w.reshape(1) for w in pending]).tolist():  # one read-back for all launches
            if status:
                raise RuntimeError(
                    f"hessian_accumulate: a bounded device-side wait ran out (status {status})"
                )

    @staticmethod
    def check_all(many) -> None:
        """:meth:`check` for several accumulators with ONE read-back (a layer of experts has hundreds)."""
        words = [w for h in many for w in h._unchecked]
        for h in many:
            h._unchecked = []
        if words and any(torch.cat(words).tolist()):
            raise RuntimeError("hessian_accumulate: a bounded device-side wait ran out")

    @torch.no_grad()
    def update(self, x: torch.Tensor, chunk: int = 4096, defer_check: bool = False) -> None:
        """``S += x^T x`` for ``x [..., K]``.  bf16 / fp16 activations feed the tensor cores
        directly (their products are exact in fp32); anything else is taken as fp32.  ``chunk``
        is accepted for compatibility: the kernel splits the tokens itself.  The tensor-core
        kernel leaves a status word; reading it costs a synchronisation, which callers that
        pipeline several inputs postpone with ``defer_check=True`` and settle with :meth:`check`."""
        del chunk
        dev = _lib.need_cuda(self.S)
        x = x.reshape(-1, self.k)
        if x.device != dev:
            x = x.to(dev)
        if x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            x = x.float()
        x = x.contiguous()
        tokens = x.shape[0]
        if tokens == 0:
            return
        lib = _lib.load()
        dt = _lib.DTYPES[x.dtype]
        need = lib.hi2_hessian_workspace_bytes(tokens, self.k, dt)
        ws = _workspace(dev, need) if need else None
        _lib.call(
            "hi2_hessian_accumulate", _lib.ptr(x), dt, tokens, self.k, _lib.ptr(self.S),
            _lib.ptr(ws), ws.numel() if ws is not None else 0, _lib.stream(dev),
        )
        if ws is not None:
            self._unchecked.append(ws[:4].view(torch.int32).clone())  # the scratch is shared
            if not defer_check:
                self.check()
        self.n += tokens

    def merge(self, other: "HessianStats") -> None:
        self.S += other.S.to(self.S.device)
        self.n += other.n

    def mean(self) -> torch.Tensor:
        return self.S / max(self.n, 1)


def transform_sigma(sigma: torch.Tensor, col_scale: torch.Tensor | None, had: torch.Tensor,
                    denom: float = 1.0, return_diag: bool = False):
    """``Hs = T (sigma / denom) T^T`` with ``T = R diag(1/s)``, symmetrised.  ``denom`` and
    ``return_diag`` are additions: the division of a raw sum by its token count and the
    diagonal of the result come out of the same pass."""
    dev = _lib.need_cuda(sigma)
    k = sigma.shape[0]
    s = sigma if sigma.dtype == torch.float32 else sigma.float()
    s = s.contiguous()
    hs = torch.empty(k, k, dtype=torch.float32, device=dev)
    diag = torch.empty(k, dtype=torch.float32, device=dev) if return_diag else None
    cs = None
    if col_scale is not None:
        cs = _lib.upload(col_scale, dev, torch.float16)
    flags = _lib.upload(had, dev, torch.uint8)
    if flags.numel() != k // GROUP:
        raise ValueError(f"had has {flags.numel()} entries, expected {k // GROUP}")
    _lib.call(
        "hi2_transform_sigma", _lib.ptr(s), float(denom), _lib.ptr(cs), _lib.ptr(flags), k,
        _lib.ptr(hs), _lib.ptr(diag), _lib.stream(dev),
    )
    return (hs, diag) if return_diag else hs


class FactorJob:
    """One damped inverse factor in flight.  ``FactorJob(hs, damp)`` enqueues the first attempt
    on the current stream (its own scratch, so several jobs may run on different streams at
    once) and returns; :meth:`result` waits for that attempt and, in the rare case of a
    non-positive pivot, repeats with ten times the damping as hi2/hessian.py:78-86 does."""

    def __init__(self, hs: torch.Tensor, damp: float = 0.01, workspace: torch.Tensor | None = None):
        self.dev = _lib.need_cuda(hs)
        self.k = hs.shape[0]
        h = hs if hs.dtype == torch.float32 else hs.float()
        self.h = h.contiguous()
        self.damp = damp
        self.mean = self.h.diagonal().mean().clamp_min(1e-12)
        need = _lib.load().hi2_inverse_factor_workspace_bytes(self.k)
        self.ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=self.dev)
        if self.ws.numel() < need:
            raise ValueError("inverse factor workspace too small")
        self.u = torch.empty(self.k, self.k, dtype=torch.float32, device=self.dev)
        self.info = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.stream = torch.cuda.current_stream(self.dev)
        self.attempt = 0
        self._launch()
        self.done = torch.cuda.Event()  # the first attempt has finished on the device
        self.done.record(self.stream)

    def first_attempt(self) -> torch.Tensor:
        """``U`` of the first attempt WITHOUT waiting for it: consumers order themselves after
        ``self.done`` on their stream and call :meth:`succeeded` once the work is enqueued."""
        return self.u

    def succeeded(self) -> bool:
        """Whether the first attempt met no non-positive pivot (synchronises with it)."""
        self.done.synchronize()
        return int(self.info.item()) == 0 and bool(torch.isfinite(self.u.diagonal()).all())

    def release_scratch(self) -> None:
        """Drop the damped input and the scratch of the attempt in flight (about five times the
        bytes of ``U``).  Both were allocated on the stream the attempt runs on, so the caching
        allocator hands them out again only to later work of that stream.  A job released this
        way cannot retry: a caller that finds :meth:`succeeded` false factorises again from the
        second moment."""
        self.h = None
        self.ws = None

    def _launch(self) -> None:
        self.lam = (self.damp * self.mean * 10**self.attempt).to(torch.float32).reshape(1)
        self.info.zero_()
        _lib.call(
            "hi2_inverse_factor", _lib.ptr(self.h), _lib.ptr(self.lam), self.k, _lib.ptr(self.u),
            _lib.ptr(self.ws), self.ws.numel(), _lib.ptr(self.info), _lib.stream(self.dev),
        )

    def result(self) -> torch.Tensor:
        if self.h is None:
            raise RuntimeError("FactorJob.result() after release_scratch(): use first_attempt()/succeeded()")
        with torch.cuda.stream(self.stream):
            while True:
                last = int(self.info.item())
                if last < 0:
                    raise RuntimeError("inverse_factor: a bounded device-side wait ran out")
                if last == 0 and bool(torch.isfinite(self.u.diagonal()).all()):
                    self.ws = None
                    return self.u
                self.attempt += 1
                if self.attempt >= 6:
                    raise RuntimeError(
                        f"Hessian is not factorisable even with heavy damping: non-positive pivot {last - 1}"
                    )
                self._launch()


def inverse_factor(hs: torch.Tensor, damp: float = 0.01) -> torch.Tensor:
    """Upper Cholesky factor ``U`` of ``(Hs + damp * mean(diag) I)^-1``; the damping is raised
    tenfold (up to five times) when the factorisation meets a non-positive pivot."""
    dev = _lib.need_cuda(hs)
    need = _lib.load().hi2_inverse_factor_workspace_bytes(hs.shape[0])
    return FactorJob(hs, damp, _workspace(dev, need)).result()


@dataclass
class GptqJob:
    """One call of :func:`encode_rows_gptq`: rows ``w [N, K]`` (stored basis), ladder weights
    ``d [K]``, factor ``u [K, K]`` (of the permuted Hessian when ``perm`` is set)."""

    w: torch.Tensor
    d: torch.Tensor
    u: torch.Tensor
    nbits: int
    block: int
    perm: torch.Tensor | None = None
    wait: torch.cuda.Event | None = None  # ``u`` is complete once this event has passed


@dataclass
class _Unit:
    job: int
    s: int
    rows: int
    wc: torch.Tensor | None  # [n, K] fp32 working copy, columns in rounding order
    src: torch.Tensor  # [n, K] fp32 original rows
    params: torch.Tensor
    consts: torch.Tensor
    lo_d: torch.Tensor  # [n, K/16] fp32 decoded, zero padded
    step_d: torch.Tensor
    blk_of: torch.Tensor  # [K] int32 block of each column in rounding order
    codes: torch.Tensor | None = None
    comp: torch.Tensor | None = None


def _prepare(ji: int, job: GptqJob, s: int, step_rows: int, effort: str) -> _Unit:
    dev = job.w.device
    k = job.w.shape[1]
    cfg = EFFORT[effort]
    src = job.w[s : s + step_rows]
    if src.dtype != torch.float32 or not src.is_contiguous():
        src = src.float().contiguous()
    d = job.d.to(dev, torch.float32).contiguous()
    lo, st = _ladder.fit(src, d, cfg["grid"], cfg["ls"], 2**job.nbits, job.block)
    q = _ladder.quantize_rows(lo, st, job.nbits, job.block, k, want_decoded=True, ldp=k // GROUP)
    cols = torch.arange(k, device=dev)
    if job.perm is not None:
        cols = job.perm.to(dev)
        wc = src[:, cols].contiguous()
    else:
        wc = src.clone()
    return _Unit(ji, s, src.shape[0], wc, src, q["params"], q["consts"], q["lo_d"], q["step_d"],
                 (cols // job.block).to(torch.int32))


# Row units of several jobs are prepared together when there are many small ones (a layer of experts
# has a thousand): jobs of one width that share (nbits, block) and keep their column order.
PREPARE_TOGETHER_MIN = 4
PREPARE_TOGETHER_MAX_ELEMS = 1 << 22  # mean size of a unit up to which gathering them into one buffer pays


def _prepare_together(pieces: list, jobs: list, step_rows: int, effort: str) -> list:
    """``_prepare`` for the units ``pieces = [(job index, first row)]`` of jobs with one width,
    ``(nbits, block)`` and no column permutation: their rows are gathered into one buffer, the ladder
    search runs once over all of them with the column weights of each unit's job
    (``d [units, K]`` and a row index), the parameter bytes and decoded ladders are made in one
    launch, and every unit gets views.  Per row the arithmetic is that of :func:`_prepare`."""
    first = jobs[pieces[0][0]]
    dev, k = first.w.device, first.w.shape[1]
    cfg = EFFORT[effort]
    srcs = []
    for ji, s0 in pieces:
        src = jobs[ji].w[s0 : s0 + step_rows]
        srcs.append(src if src.dtype == torch.float32 else src.float())
    sizes = [x.shape[0] for x in srcs]
    rows = torch.cat(srcs)
    d = torch.stack([jobs[ji].d.to(dev, torch.float32) for ji, _ in pieces])
    row_group = _lib.upload(torch.repeat_interleave(torch.arange(len(pieces), dtype=torch.int32), torch.tensor(sizes)), dev)
    lo, st = _ladder.fit(rows, d, cfg["grid"], cfg["ls"], 2**first.nbits, first.block, row_group)
    q = _ladder.quantize_rows(lo, st, first.nbits, first.block, k, want_decoded=True, ldp=k // GROUP)
    work = rows.clone()
    blk_of = (torch.arange(k, device=dev) // first.block).to(torch.int32)
    units, off = [], 0
    for (ji, s0), n in zip(pieces, sizes):
        cut = slice(off, off + n)
        units.append(_Unit(ji, s0, n, work[cut], rows[cut], q["params"][cut], q["consts"][cut], q["lo_d"][cut],
                           q["step_d"][cut], blk_of))
        off += n
    return units


# factors at least this wide take the tensor-core trailing update (below it the FMA product wins)
TC_MIN_K = 512


def _round_units(units: list[_Unit], jobs: list[GptqJob], want_comp: bool, splits: dict, checks: list) -> None:
    """All ``units`` (same K, same device) through one enqueue of the column loop.  ``splits``
    caches the TF32 split of each distinct factor over one :func:`encode_jobs_gptq` call;
    ``checks`` collects the device status words to be read once everything is enqueued."""
    dev, k = units[0].wc.device, units[0].wc.shape[1]
    for ev in {id(jobs[x.job].wait): jobs[x.job].wait for x in units if jobs[x.job].wait is not None}.values():
        torch.cuda.current_stream(dev).wait_event(ev)  # factors still in flight on a side stream
    sizes = [x.rows for x in units]
    total = sum(sizes)
    if len(units) == 1:
        wc, lo, st = units[0].wc, units[0].lo_d, units[0].step_d
    else:
        wc = torch.cat([x.wc for x in units])
        lo = torch.cat([x.lo_d for x in units])
        st = torch.cat([x.step_d for x in units])
    offs = [0]
    for n in sizes:
        offs.append(offs[-1] + n)
    row_grp = _lib.upload(torch.repeat_interleave(
        torch.arange(len(units), dtype=torch.int32), torch.tensor(sizes)
    ), dev)
    us = [jobs[x.job].u.to(dev, torch.float32).contiguous() for x in units]
    u_ptrs = _lib.upload(torch.tensor([u.data_ptr() for u in us], dtype=torch.int64), dev)
    blk = torch.stack([x.blk_of for x in units]).contiguous()
    nmax = _lib.upload(torch.tensor([2 ** jobs[x.job].nbits - 1 for x in units], dtype=torch.float32), dev)
    codes = torch.empty(total, k, dtype=torch.uint8, device=dev)
    comp = torch.empty(total, k, dtype=torch.float32, device=dev) if want_comp else None
    err1 = torch.empty(total, BLOCK_COLUMNS, dtype=torch.float32, device=dev)
    # INT8 ladders are 64 times finer than INT2: the 3 x TF32 update (error ~1e-6 of |err||U|, ten
    # times an fp32 FMA chain) moves ~0.1 % of INT8 codes, so rows with 256 levels keep the FMA
    # product; for INT2 / INT4 the codes are the same
    if k >= TC_MIN_K and all(jobs[x.job].nbits <= 4 for x in units):
        parts = []
        for u in us:
            if u.data_ptr() not in splits:
                splits[u.data_ptr()] = (u, gptq_kernel.split_tf32_transposed(u))  # keeps u alive with its split
            parts.append(splits[u.data_ptr()][1])
        checks.append(gptq_kernel.gptq_round_tc(wc, err1, codes, lo, st, row_grp, u_ptrs, blk, nmax, comp,
                                                offs, parts))
    else:
        gptq_kernel.gptq_round(wc, err1, codes, lo, st, row_grp, u_ptrs, blk, nmax, comp, offs, us)
    for x, o, n in zip(units, offs, sizes):
        x.codes = codes[o : o + n]
        x.comp = None if comp is None else comp[o : o + n]


def _finish(unit: _Unit, job: GptqJob) -> Encoded:
    dev = unit.src.device
    k = unit.src.shape[1]
    codes, comp = unit.codes, unit.comp
    if job.perm is not None:
        p = job.perm.to(dev)
        out = torch.empty_like(codes)
        out[:, p] = codes
        codes = out
        if comp is not None:
            c = torch.empty_like(comp)
            c[:, p] = comp
            comp = c
    codes = codes.contiguous()
    sse = torch.empty(unit.rows, dtype=torch.float32, device=dev)
    d = job.d.to(dev, torch.float32).contiguous()
    _lib.call(
        "hi2_ladder_sse", _lib.ptr(codes), _lib.ptr(unit.src), unit.src.stride(0), _lib.ptr(d),
        _lib.ptr(unit.lo_d), _lib.ptr(unit.step_d), unit.lo_d.shape[1], unit.rows, k, job.block,
        _lib.ptr(sse), _lib.stream(dev),
    )
    return Encoded(codes, unit.params, unit.consts, sse, comp)


def _use_kernel(dev: torch.device, backend: str) -> bool:
    if backend == "torch":
        raise RuntimeError("hi2_b200 has no torch loop: backend must be 'auto' or 'kernel'")
    if not gptq_kernel.available(dev):
        raise RuntimeError(f"gptq kernel unavailable on {dev}: {gptq_kernel.failure()}")
    return True


@torch.no_grad()
def encode_jobs_gptq(jobs: list[GptqJob], effort: str = "normal", backend: str | None = None,
                     comp: bool = False, timing: list | None = None) -> list[Encoded]:
    """:func:`encode_rows_gptq` for several jobs (tensors, experts, candidate groups) at once.

    Jobs are cut into row units; units with the same K on the same device are batched (up to
    ``BATCH_ELEMS`` weights) through one column loop.  With ``comp`` every result carries
    ``Encoded.comp``, the value each code was rounded from.  ``timing`` (optional list) receives one
    ``(K, rows, start event, end event)`` per width: the column loops of that width (block kernel +
    trailing updates) on their stream, for a caller that reports rows per second of the loop."""
    backend = backend or os.environ.get("HI2_GPTQ_BACKEND", "auto")
    # Widths are independent column loops of many short launches.  The jobs of one width are
    # prepared (ladders, parameter bytes) on the current stream and their column loop is then
    # handed to a side stream, widest first, so that the preparation of the next width and, e.g.,
    # the 86 blocks of a 4096 x 11008 matrix run beside the batches of the 4096-wide ones.
    # Nothing a side stream reads is released before the streams are joined, and status words are
    # read only after everything is enqueued.
    by_width: dict[tuple, list[int]] = {}
    for ji, job in enumerate(jobs):
        _lib.need_cuda(job.w, job.u)
        _use_kernel(job.w.device, backend)
        by_width.setdefault((job.w.device, job.w.shape[1]), []).append(ji)
    units: list[_Unit] = []
    splits: dict = {}
    checks: list = []
    joins = []
    for gi, ((dev, k), jis) in enumerate(sorted(by_width.items(), key=lambda kv: -kv[0][1])):
        step_rows = max(1, ROW_ELEMS // k)
        pieces = [(ji, s) for ji in jis for s in range(0, jobs[ji].w.shape[0], step_rows)]
        alike: dict[tuple, list[int]] = {}
        for at, (ji, _) in enumerate(pieces):
            if jobs[ji].perm is None:
                alike.setdefault((jobs[ji].nbits, jobs[ji].block), []).append(at)
        ready: dict[int, _Unit] = {}
        for members in alike.values():
            elems = sum(min(step_rows, jobs[pieces[at][0]].w.shape[0] - pieces[at][1]) for at in members) * k
            if len(members) >= PREPARE_TOGETHER_MIN and elems <= PREPARE_TOGETHER_MAX_ELEMS * len(members):
                for at, unit in zip(members, _prepare_together([pieces[at] for at in members], jobs, step_rows, effort)):
                    ready[at] = unit
        mine: list[_Unit] = [ready[at] if at in ready else _prepare(ji, jobs[ji], s, step_rows, effort)
                             for at, (ji, s) in enumerate(pieces)]
        units.extend(mine)
        bl: list[list[_Unit]] = [[]]
        for x in mine:
            if bl[-1] and sum(y.wc.numel() for y in bl[-1]) + x.wc.numel() > BATCH_ELEMS:
                bl.append([])
            bl[-1].append(x)
        main = torch.cuda.current_stream(dev)
        side = _side_stream(dev, gi + 1)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            if timing is not None:
                t0 = torch.cuda.Event(enable_timing=True)
                t0.record()
            for batch in bl:
                if batch:  # a width whose jobs have no rows leaves one empty batch
                    _round_units(batch, jobs, comp, splits, checks)
            if timing is not None:
                t1 = torch.cuda.Event(enable_timing=True)
                t1.record()
                timing.append((k, sum(x.rows for x in mine), t0, t1))
        joins.append((main, side))
    for main, side in joins:
        main.wait_stream(side)
    for x in units:
        x.wc = None
    units.sort(key=lambda x: (x.job, x.s))
    if any(int(st.item()) for st in checks):
        raise RuntimeError("gptq trailing update: a bounded device-side wait ran out")
    per_job: list[list[Encoded]] = [[] for _ in jobs]
    for x in units:
        per_job[x.job].append(_finish(x, jobs[x.job]))
    out = []
    for job, encs in zip(jobs, per_job):
        if len(encs) == 1:
            out.append(encs[0])
            continue
        if not encs:  # a job without rows: nothing was launched for it
            dev, k = job.w.device, job.w.shape[1]
            out.append(Encoded(
                torch.empty(0, k, dtype=torch.uint8, device=dev),
                torch.empty(0, k // job.block, 2, dtype=torch.uint8, device=dev),
                torch.empty(0, 3, dtype=torch.float16, device=dev),
                torch.empty(0, dtype=torch.float32, device=dev),
                torch.empty(0, k, dtype=torch.float32, device=dev) if comp else None,
            ))
            continue
        out.append(
            Encoded(
                *(torch.cat([getattr(o, f) for o in encs]) for f in ("codes", "params", "consts", "sse")),
                torch.cat([o.comp for o in encs]) if comp else None,
            )
        )
    return out


def encode_rows_gptq(w, d, u, nbits: int, block: int, effort: str = "normal", perm=None,
                     backend: str | None = None, comp: bool = True) -> Encoded:
    """Quantise ``w [N, K]`` (stored basis) with error compensation; ladders are fitted on the
    uncompensated weights with weights ``d`` and then fixed.  With ``perm`` the columns are
    rounded in that order while codes keep their original positions."""
    return encode_jobs_gptq([GptqJob(w, d, u, nbits, block, perm)], effort, backend, comp)[0]


def encode_rows_gptq_reference(w, d, u, nbits: int, block: int, effort: str = "normal",
                               perm=None) -> Encoded:
    """The reference keeps its original column loop under this name; here it is the same
    kernel path (there is one implementation), with ``comp`` always returned."""
    return encode_rows_gptq(w, d, u, nbits, block, effort, perm, comp=True)


__all__ = [
    "EFFORT",
    "GptqJob",
    "HessianStats",
    "encode_jobs_gptq",
    "encode_rows_gptq",
    "encode_rows_gptq_reference",
    "inverse_factor",
    "transform_sigma",
]
