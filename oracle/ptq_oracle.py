"""CPU oracle for the per-layer PTQ encode path (TEST INFRASTRUCTURE, not product code).

A restatement, on torch CPU tensors, of the arithmetic hi2 performs between the calibration
activations of a Linear and its packed ``rdna_hint_flex`` buffers.  Only ``tests/``, the smoke
check and the CPU-baseline / reference legs of ``bench.py`` may import this module; the product
package never does (it has no CPU path at all).

Pinning: every function below is compared with outputs of the reference itself (imported in the
build container, see ``tests/golden/make_golden.py``) through the fixtures under
``tests/golden/``.  Where the reference's result depends on the summation order of a CPU BLAS
(second moments, basis change, factorisation, block sums of the ladder search) the oracle uses
the same torch operators, so on the host that generated the fixtures it is bit-identical and
elsewhere it agrees to rounding.  The group rotation is written as an explicit left-to-right
sum, which is what the fixtures show the reference's ``[.,16] @ [16,16]`` product to be.

Reference locations (paths inside the hi2 project):
  hi2/format.py:22-41    rotation            -> hadamard16, rotate_groups
  hi2/hessian.py:26-47   second moment       -> SecondMoment
  hi2/stats.py:16-64     16x16 group moments -> GroupMoments
  hi2/calibrate.py:96-111 smoothing vector   -> smoothing_vector
  hi2/hessian.py:50-68   basis change        -> stored_basis_hessian
  hi2/hessian.py:71-86   damped inverse factor -> inverse_cholesky
  hi2/encode.py:18-92    ladder search       -> EFFORTS, search_ladder
  hi2/encode.py:95-119   parameter bytes     -> quantise_ladders
  hi2/format.py:45-69    decode              -> decode_ladders, reconstruct
  hi2/encode.py:133-173  nearest rows/tables -> nearest_rows
  hi2/hessian.py:89-175  fixed-ladder GPTQ   -> gptq_rows
  hi2/refine.py:44-106   +-1 refinement      -> refine_sweeps
  hi2/format.py:73-184   packing / layout    -> pack_words, unpack_words, assemble_flat
  hi2/allocate.py:79-261 allocation          -> allocate_rows
  hi2/calibrate.py:114-209 transform choice  -> pick_rotation, transform_cost, pick_transform
  hi2/format.py:195-239  inverse path        -> reconstruct_flat
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

GROUP = 16
LAZY = 128  # columns between two trailing updates (hi2/hessian.py:20, hi2/refine.py:20)
CHUNK_TOKENS = 4096
NEAREST_CHUNK = 1 << 24  # hi2/encode.py:23
GPTQ_CHUNK = 1 << 26  # hi2/hessian.py:21

EFFORTS = {
    "fast": ((0.0, 0.06, 0.12), 1),
    "normal": ((0.0, 0.04, 0.08, 0.12, 0.16, 0.20), 2),
    "max": ((0.0, 0.025, 0.05, 0.075, 0.10, 0.125, 0.15, 0.20), 4),
}

F16 = torch.float16
F32 = torch.float32
F64 = torch.float64


# --------------------------------------------------------------------------- rotation
def hadamard16(dtype=F64) -> torch.Tensor:
    """Order-16 Sylvester matrix over 4: entry (i, j) is (-1)^popcount(i & j) / 4."""
    idx = torch.arange(GROUP)
    par = torch.zeros(GROUP, GROUP, dtype=torch.int64)
    both = idx[:, None] & idx[None, :]
    for bit in range(4):
        par ^= (both >> bit) & 1
    return ((1 - 2 * par).to(F64) / 4.0).to(dtype)


def rotate_groups(x: torch.Tensor, flags: torch.Tensor) -> torch.Tensor:
    """Multiply every flagged run of 16 columns of ``x[..., K]`` by the matrix above.

    fp32 / fp64 inputs are transformed in their own precision, anything else in fp64 and rounded
    once.  Output element j of a group is ``((x0*h0j + x1*h1j) + x2*h2j) + ...`` (k ascending)."""
    k = x.shape[-1]
    if k % GROUP:
        raise ValueError(f"K={k} must be a multiple of {GROUP}")
    if flags.numel() != k // GROUP:
        raise ValueError(f"flags has {flags.numel()} entries, expected {k // GROUP}")
    work = x.dtype if x.dtype in (F32, F64) else F64
    xg = x.to(work).reshape(*x.shape[:-1], k // GROUP, GROUP)
    h = hadamard16(work)
    acc = xg[..., 0:1] * h[0]
    for t in range(1, GROUP):
        acc = acc + xg[..., t : t + 1] * h[t]
    keep = flags.to(torch.bool).reshape(-1, 1)
    return torch.where(keep, acc, xg).reshape(x.shape).to(x.dtype)


# --------------------------------------------------------------------------- statistics
class SecondMoment:
    """``S = sum_t x_t x_t^T`` in fp32, one product per run of 4096 tokens."""

    def __init__(self, k: int):
        self.k, self.n = k, 0
        self.S = torch.zeros(k, k, dtype=F32)

    def update(self, x: torch.Tensor, chunk: int = CHUNK_TOKENS) -> None:
        x = x.reshape(-1, self.k)
        for t0 in range(0, x.shape[0], chunk):
            part = x[t0 : t0 + chunk].to(F32)
            self.S += part.T @ part
        self.n += x.shape[0]

    def merge(self, other: "SecondMoment") -> None:
        self.S += other.S
        self.n += other.n

    def mean(self) -> torch.Tensor:
        return self.S / max(self.n, 1)


class GroupMoments:
    """The 16x16 diagonal blocks of the second moment, summed in fp64."""

    def __init__(self, k: int):
        if k % GROUP:
            raise ValueError(f"K={k} must be a multiple of {GROUP}")
        self.k, self.n = k, 0
        self.S = torch.zeros(k // GROUP, GROUP, GROUP, dtype=F64)

    def update(self, x: torch.Tensor) -> None:
        x = x.reshape(-1, self.k)
        for t0 in range(0, x.shape[0], CHUNK_TOKENS):
            part = x[t0 : t0 + CHUNK_TOKENS].to(F32)
            part = part.reshape(part.shape[0], self.k // GROUP, GROUP)
            self.S += torch.einsum("tgi,tgj->gij", part, part).double()
        self.n += x.shape[0]

    def merge(self, other: "GroupMoments") -> None:
        self.S += other.S
        self.n += other.n

    def diag(self, flags=None, inv_scale=None) -> torch.Tensor:
        """Per-column mean square of ``x * inv_scale`` after the flagged rotation (fp32)."""
        s = self.S / max(self.n, 1)
        if inv_scale is not None:
            inv = inv_scale.to(s.dtype).reshape(-1, GROUP)
            s = s * inv[:, :, None] * inv[:, None, :]
        plain = torch.diagonal(s, dim1=1, dim2=2)
        if flags is None:
            return plain.reshape(-1).float()
        h = hadamard16(F64)
        rot = torch.einsum("ij,gjk,ik->gi", h, s, h)
        return torch.where(flags.bool().reshape(-1, 1), rot, plain).reshape(-1).float()


def smoothing_vector(moments: GroupMoments | None, alpha: float):
    """fp16 ``s_j = clamp((d_j / geomean d)^(alpha/2), 0.05, 20)`` or None."""
    if alpha <= 0 or moments is None or moments.n == 0:
        return None
    d = moments.diag().clamp_min(1e-12)
    s = (d / d.log().mean().exp()).pow(alpha / 2).clamp(0.05, 20.0)
    return s.to(F16)


def stored_basis_hessian(sigma, col_scale, flags) -> torch.Tensor:
    """``T sigma T^T`` with ``T = R diag(1/s)``; symmetrised at the end."""
    k = sigma.shape[0]
    g = k // GROUP
    s = sigma.float()
    if col_scale is not None:
        inv = 1.0 / col_scale.float()
        s = s * inv[:, None] * inv[None, :]
    if bool(flags.any()):
        h = hadamard16(F32)
        m = torch.where(flags.bool().reshape(-1, 1, 1), h, torch.eye(GROUP, dtype=F32))
        t = s.reshape(g, GROUP, g, GROUP)
        t = torch.einsum("gij,gjhk->gihk", m, t)
        t = torch.einsum("gihk,hlk->gihl", t, m)
        s = t.reshape(k, k)
    return 0.5 * (s + s.T)


def inverse_cholesky(hs: torch.Tensor, damp: float = 0.01) -> torch.Tensor:
    """Upper ``U`` with ``U^T U = (hs + damp * mean(diag hs) * I)^-1``; the damping grows
    tenfold per failed attempt, six attempts in all."""
    k = hs.shape[0]
    level = hs.diagonal().mean().clamp_min(1e-12)
    eye = torch.eye(k, dtype=hs.dtype)
    err = None
    for attempt in range(6):
        h = hs + (damp * level * 10**attempt) * eye
        try:
            low = torch.linalg.cholesky(h)
            inv = torch.cholesky_inverse(low)
            return torch.linalg.cholesky(0.5 * (inv + inv.T), upper=True)
        except RuntimeError as e:
            err = e
    raise RuntimeError(f"Hessian is not factorisable even with heavy damping: {err}")


# --------------------------------------------------------------------------- ladders
def _nz(step):
    return torch.where(step == 0, torch.ones_like(step), step)


def _snap(wb, lo, step, n):
    c = torch.round((wb - lo.unsqueeze(-1)) / _nz(step).unsqueeze(-1)).clamp(0, n - 1)
    return lo.unsqueeze(-1) + c * step.unsqueeze(-1), c


def _block_error(wb, db, lo, step, n):
    rec, _ = _snap(wb, lo, step, n)
    return (db * (rec - wb) ** 2).sum(-1)


def grid_search(wb, db, n: int, grid) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Best ``(lo, step, err)`` over the range-shrink grid, first strict minimum wins."""
    mn, mx = wb.amin(-1), wb.amax(-1)
    span = mx - mn
    best = None
    for a in grid:
        for b in grid:
            lo = mn + a * span
            step = (mx - b * span - lo) / (n - 1)
            err = _block_error(wb, db, lo, step, n)
            if best is None:
                best = [lo, step, err]
                continue
            better = err < best[2]
            best = [torch.where(better, new, old) for new, old in zip((lo, step, err), best)]
    return best[0], best[1], best[2]


def _refit(c, w, d):
    sd = d.sum(-1)
    sc = (d * c).sum(-1)
    scc = (d * c * c).sum(-1)
    sw = (d * w).sum(-1)
    scw = (d * c * w).sum(-1)
    det = sd * scc - sc * sc
    ok = det.abs() > 1e-20
    step = torch.where(
        ok, (sd * scw - sc * sw) / torch.where(ok, det, torch.ones_like(det)), torch.zeros_like(det)
    )
    lo = torch.where(ok, (sw - step * sc) / sd.clamp_min(1e-20), w.mean(-1))
    return lo, step


def search_ladder(wb, db, n: int, effort: str = "normal"):
    """``(lo, step)`` per block of ``wb[N, nb, B]`` under weights ``db`` (broadcastable)."""
    grid, refits = EFFORTS[effort]
    lo, step, err = grid_search(wb, db, n, grid)
    dfull = db.expand_as(wb)
    for _ in range(refits):
        _, c = _snap(wb, lo, step, n)
        lo2, step2 = _refit(c, wb, dfull)
        err2 = _block_error(wb, db, lo2, step2, n)
        take = (err2 < err) & (step2 > 0)
        lo = torch.where(take, lo2, lo)
        step = torch.where(take, step2, step)
        err = torch.where(take, err2, err)
    return lo, step


def quantise_ladders(lo, step):
    """Bytes ``(lo_u8, step_u8)`` and fp16 row constants ``(lo_min, lo_scale, step_scale)``."""
    step = step.clamp_min(0)
    step_scale = (step.amax(-1, keepdim=True) / 255).to(F16)
    ss = step_scale.float()
    step_u8 = torch.where(
        ss > 0, torch.round(step / ss.clamp_min(1e-30)), torch.zeros_like(step)
    ).clamp(0, 255)
    lo_min = lo.amin(-1, keepdim=True).to(F16)
    lo_scale = ((lo.amax(-1, keepdim=True) - lo_min.float()).clamp_min(0) / 255).to(F16)
    ls = lo_scale.float()
    lo_u8 = torch.where(
        ls > 0, torch.round((lo - lo_min.float()) / ls.clamp_min(1e-30)), torch.zeros_like(lo)
    ).clamp(0, 255)
    consts = torch.cat([lo_min, lo_scale, step_scale], dim=-1)
    return lo_u8.to(torch.uint8), step_u8.to(torch.uint8), consts


def decode_ladders(lo_u8, step_u8, lo_min, lo_scale, step_scale):
    """fp16 ``lo = fma_f32(u, lo_scale, lo_min)`` and ``step = u * step_scale``."""
    lo = (lo_u8.double() * lo_scale.double() + lo_min.double()).float().to(F16)
    step = (step_u8.float() * step_scale.float()).to(F16)
    return lo, step


def reconstruct(codes, lo, step, dtype=F64):
    """``fp16(lo + code * step)``; ``codes`` carries a trailing block axis."""
    v = lo.to(dtype).unsqueeze(-1) + codes.to(dtype) * step.to(dtype).unsqueeze(-1)
    return v.to(F16)


def _decoded(lo_u8, step_u8, consts):
    lo, step = decode_ladders(lo_u8, step_u8, consts[:, 0:1], consts[:, 1:2], consts[:, 2:3])
    return lo.float(), step.float()


@dataclass
class Rows:
    codes: torch.Tensor  # u8 [N, K]
    params: torch.Tensor  # u8 [N, nb, 2]
    consts: torch.Tensor  # f16 [N, 3]
    sse: torch.Tensor  # f32 [N]
    comp: torch.Tensor | None = None


def _cat(parts, with_comp):
    if len(parts) == 1:
        return parts[0]
    names = ["codes", "params", "consts", "sse"] + (["comp"] if with_comp else [])
    return Rows(*(torch.cat([getattr(p, f) for p in parts]) for f in names))


def nearest_rows(w, d, nbits: int, block: int, effort: str = "normal") -> Rows:
    """Search, quantise the parameters, then round every weight to its decoded ladder."""
    n_rows, k = w.shape
    n = 2**nbits
    db = d.to(F32).reshape(1, k // block, block)
    per = max(1, NEAREST_CHUNK // k)
    parts = []
    for r0 in range(0, n_rows, per):
        wb = w[r0 : r0 + per].float().reshape(-1, k // block, block)
        lo, step = search_ladder(wb, db, n, effort)
        lo_u8, step_u8, consts = quantise_ladders(lo, step)
        lo_d, step_d = _decoded(lo_u8, step_u8, consts)
        codes = torch.where(
            step_d.unsqueeze(-1) == 0,
            torch.zeros_like(wb),
            torch.round((wb - lo_d.unsqueeze(-1)) / _nz(step_d).unsqueeze(-1)),
        ).clamp(0, n - 1)
        rec = reconstruct(codes, lo_d, step_d, F32).float()
        sse = (db * (rec - wb) ** 2).sum((-1, -2))
        parts.append(
            Rows(
                codes.reshape(-1, k).to(torch.uint8),
                torch.stack([lo_u8, step_u8], dim=-1),
                consts,
                sse,
            )
        )
    return _cat(parts, False)


# --------------------------------------------------------------------------- GPTQ
def gptq_rows(w, d, u, nbits: int, block: int, effort: str = "normal", perm=None, ladders=None,
              only_blocks=None) -> Rows:
    """Error-compensated rounding with ladders frozen beforehand.

    Columns are visited in ``perm`` order when given (``u`` then belongs to the permuted Hessian);
    codes and ``comp`` are reported at the original column positions.

    Two aids for the benchmark's bounded CPU sample (results are then NOT an encode): ``ladders``
    ``(lo_u8, step_u8, consts)`` skips the search, ``only_blocks`` (a set of 128-column block
    indices) visits only those blocks of the column loop."""
    n_rows, k = w.shape
    n = 2**nbits
    db = d.to(F32).reshape(1, k // block, block)
    per = max(1, GPTQ_CHUNK // k)
    order = list(range(k)) if perm is None else perm.tolist()
    parts = []
    for r0 in range(0, n_rows, per):
        src = w[r0 : r0 + per].float()
        work = src.clone()
        if ladders is None:
            lo, step = search_ladder(work.reshape(-1, k // block, block), db, n, effort)
            lo_u8, step_u8, consts = quantise_ladders(lo, step)
        else:
            lo_u8, step_u8, consts = (t[r0 : r0 + per] for t in ladders)
        lo_d, step_d = _decoded(lo_u8, step_u8, consts)
        if perm is not None:
            work = work[:, perm]
        codes = torch.zeros_like(work)
        comp = torch.zeros_like(work)
        for c0 in range(0, k, LAZY):
            if only_blocks is not None and c0 // LAZY not in only_blocks:
                continue
            c1 = min(c0 + LAZY, k)
            seg = work[:, c0:c1].clone()
            errs = torch.zeros_like(seg)
            tri = u[c0:c1, c0:c1]
            for i in range(c1 - c0):
                col_at = order[c0 + i]
                b = col_at // block
                lo_j, st_j = lo_d[:, b], step_d[:, b]
                col = seg[:, i]
                q = torch.round((col - lo_j) / _nz(st_j)).clamp(0, n - 1)
                q = torch.where(st_j == 0, torch.zeros_like(q), q)
                wq = (lo_j + q * st_j).to(F16).float()
                codes[:, col_at] = q
                comp[:, col_at] = col
                e = (col - wq) / tri[i, i]
                seg[:, i:] -= e[:, None] * tri[i, i:][None, :]
                errs[:, i] = e
            work[:, c1:] -= errs @ u[c0:c1, c1:]
        rec = reconstruct(codes.reshape(-1, k // block, block), lo_d, step_d, F32).float()
        diff = rec.reshape(-1, k) - src
        sse = (d * diff**2).sum(-1)
        parts.append(
            Rows(codes.to(torch.uint8), torch.stack([lo_u8, step_u8], dim=-1), consts, sse, comp)
        )
    return _cat(parts, True)


# --------------------------------------------------------------------------- refinement
def hessian_objective(w, codes, lo, step, hs, block) -> float:
    idx = torch.arange(w.shape[1]) // block
    e = (lo[:, idx] + codes.float() * step[:, idx]).half().float() - w
    return float((e @ hs * e).sum())


def refine_sweeps(w, codes, lo_x, st_x, top, hs, passes: int) -> torch.Tensor:
    """Move codes by one level while ``e hs e^T`` falls; per-column ladders ``lo_x/st_x [N,K]``,
    highest code per row ``top[N]``.  Returns fp32 codes."""
    n_rows, k = w.shape
    c = codes.float().clone()
    g = ((lo_x + c * st_x).half().float() - w) @ hs
    hd = hs.diagonal()
    rows = torch.arange(n_rows)
    signs = torch.tensor([[1.0], [-1.0]])
    for _ in range(passes):
        before = c.clone()
        for c0 in range(0, k, LAZY):
            c1 = min(c0 + LAZY, k)
            gseg = g[:, c0:c1].clone()
            moved = torch.zeros(n_rows, c1 - c0)
            hb = hs[c0:c1, c0:c1]
            for i in range(c1 - c0):
                j = c0 + i
                lo_j, st_j, cj = lo_x[:, j], st_x[:, j], c[:, j]
                cur = (lo_j + cj * st_j).half().float()
                cand = cj[None] + signs
                dw = (lo_j[None] + cand * st_j[None]).half().float() - cur[None]
                ok = (cand >= 0) & (cand <= top[None]) & (st_j > 0)[None]
                gain = torch.where(ok, -(2 * dw * gseg[:, i][None] + dw * dw * hd[j]), -torch.inf)
                best, which = gain.max(0)
                take = best > 0
                dwj = torch.where(take, dw[which, rows], 0.0)
                c[:, j] = cj + torch.where(take, signs[which, 0], 0.0)
                moved[:, i] = dwj
                gseg += dwj[:, None] * hb[i][None, :]
            g += moved @ hs[c0:c1]
        if bool((c == before).all()):
            break
    return c


def refine_groups(groups, hs, passes: int):
    """``groups`` = ``[(w, Rows, nbits, block)]`` of one tensor; one shared sweep."""
    cat = []
    for w, enc, nbits, block in groups:
        lo, step = _decoded(enc.params[..., 0], enc.params[..., 1], enc.consts)
        cat.append(
            (
                w,
                enc.codes.float(),
                lo.repeat_interleave(block, dim=1),
                step.repeat_interleave(block, dim=1),
                torch.full((w.shape[0],), float(2**nbits - 1)),
            )
        )
    joined = [torch.cat([p[i] for p in cat]) for i in range(5)]
    out = refine_sweeps(*joined, hs, passes)
    return [o.to(torch.uint8) for o in out.split([p[0].shape[0] for p in cat])]


# --------------------------------------------------------------------------- transform choice
SAMPLE_ROWS = 1024  # hi2/calibrate.py:32
CHUNK_COLS = 64  # hi2/calibrate.py:33


def _every_nth(w):
    r = w.shape[0]
    return w[torch.arange(0, r, max(1, r // SAMPLE_ROWS))[:SAMPLE_ROWS]]


def _column_weights(moments, k, flags, inv_scale=None):
    return torch.ones(k) if moments is None else moments.diag(flags, inv_scale)


def pick_rotation(w, moments, mode: str, inv_scale=None) -> torch.Tensor:
    """Flags ``[K/16]``: all, none, or (``auto``) per 64-column chunk whichever of rotated /
    unrotated leaves the smaller weighted INT2/B64 error on a row sample."""
    k = w.shape[1]
    groups = k // GROUP
    if mode == "off":
        return torch.zeros(groups, dtype=torch.uint8)
    if mode == "on":
        return torch.ones(groups, dtype=torch.uint8)
    sample = _every_nth(w).float()
    cost = []
    for rotated in (0, 1):
        flags = torch.full((groups,), rotated, dtype=torch.uint8)
        wt = rotate_groups(sample, flags) if rotated else sample
        d = _column_weights(moments, k, flags, inv_scale)
        enc = nearest_rows(wt, d, 2, CHUNK_COLS, "fast")
        lo, step = _decoded(enc.params[..., 0], enc.params[..., 1], enc.consts)
        rec = reconstruct(enc.codes.reshape(-1, k // CHUNK_COLS, CHUNK_COLS), lo, step, F32).float()
        wb = wt.reshape(-1, k // CHUNK_COLS, CHUNK_COLS)
        cost.append((d.reshape(1, -1, CHUNK_COLS) * (rec - wb) ** 2).sum((0, 2)))
    return (cost[1] < cost[0]).to(torch.uint8).repeat_interleave(CHUNK_COLS // GROUP)


def _transform_for(ws, moments, mode: str, alpha: float):
    s16 = smoothing_vector(moments, alpha)
    if mode != "auto":
        return s16, pick_rotation(ws[0], moments, mode)
    stacked = torch.cat([w.float() if s16 is None else w.float() * s16.float() for w in ws])
    return s16, pick_rotation(stacked, moments, mode, None if s16 is None else 1.0 / s16.float())


def transform_cost(ws, moments, s16, flags) -> float:
    """Weighted INT2/B32 error of a row sample under one transform over its weighted energy."""
    inv = None if s16 is None else 1.0 / s16.float()
    sse = energy = 0.0
    for w in ws:
        wt = _every_nth(w).float()
        if s16 is not None:
            wt = wt * s16.float()
        if bool(flags.any()):
            wt = rotate_groups(wt, flags)
        d = _column_weights(moments, w.shape[1], flags, inv)
        sse += float(nearest_rows(wt, d, 2, 32, "fast").sse.sum())
        energy += float((d * wt**2).sum())
    return sse / max(energy, 1e-30)


def pick_transform(ws, moments, mode: str, alpha: float, search=()):
    """``(smoothing vector, flags)`` shared by the Linears ``ws`` of one input; with ``search`` the
    exponent of lowest :func:`transform_cost`, the first on a tie."""
    if not search or moments is None or moments.n == 0:
        return _transform_for(ws, moments, mode, alpha)
    best = None
    for a in dict.fromkeys((alpha, *search)):
        s16, flags = _transform_for(ws, moments, mode, a)
        cost = transform_cost(ws, moments, s16, flags)
        if best is None or cost < best[0]:
            best = (cost, s16, flags)
    return best[1], best[2]


# --------------------------------------------------------------------------- packing
def pack_words(codes: torch.Tensor, nbits: int) -> torch.Tensor:
    """``[..., n]`` codes to ``[..., n*nbits/32]`` int32 words, first code in the low bits."""
    per = 32 // nbits
    n = codes.shape[-1]
    if n % per:
        raise ValueError(f"{n} codes is not a multiple of {per}")
    if int(codes.max()) >= 2**nbits or int(codes.min()) < 0:
        raise ValueError("code outside the ladder")
    c = codes.to(torch.int64).reshape(*codes.shape[:-1], n // per, per)
    shifts = torch.arange(per, dtype=torch.int64) * nbits
    word = (c << shifts).sum(-1)
    return torch.where(word >= 2**31, word - 2**32, word).to(torch.int32)


def unpack_words(words: torch.Tensor, nbits: int) -> torch.Tensor:
    per = 32 // nbits
    w = words.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(per, dtype=torch.int64) * nbits
    return ((w.unsqueeze(-1) >> shifts) & ((1 << nbits) - 1)).reshape(*words.shape[:-1], -1)


@dataclass
class Flat:
    codes: torch.Tensor  # i32
    code_off: torch.Tensor  # i32 [R+1], words
    blk_params: torch.Tensor  # u8
    param_off: torch.Tensor  # i32 [R+1], blocks
    row_consts: torch.Tensor  # f16 [R, 3]
    row_nbits: torch.Tensor  # u8 [R]
    row_block: torch.Tensor  # u8 [R]
    had: torch.Tensor  # u8 [K/16]
    shape: tuple
    col_scale: torch.Tensor | None = None


def assemble_flat(pieces, row_nbits, row_block, had, k: int, col_scale=None) -> Flat:
    """Scatter per-candidate pieces ``(rows, codes, params, consts)`` into the flat buffers."""
    r = row_nbits.numel()
    nb64, bl64 = row_nbits.to(torch.int64), row_block.to(torch.int64)
    code_off = torch.zeros(r + 1, dtype=torch.int64)
    code_off[1:] = torch.cumsum(k * nb64 // 32, 0)
    param_off = torch.zeros(r + 1, dtype=torch.int64)
    param_off[1:] = torch.cumsum(k // bl64, 0)
    codes = torch.zeros(int(code_off[-1]), dtype=torch.int32)
    params = torch.zeros(int(param_off[-1]) * 2, dtype=torch.uint8)
    consts = torch.zeros(r, 3, dtype=F16)
    for rows, c, p, rc in pieces:
        words = pack_words(c, int(nb64[rows[0]]))
        for i, row in enumerate(rows.tolist()):
            codes[code_off[row] : code_off[row + 1]] = words[i]
            params[2 * param_off[row] : 2 * param_off[row + 1]] = p[i].reshape(-1)
        consts[rows] = rc
    return Flat(
        codes,
        code_off.to(torch.int32),
        params,
        param_off.to(torch.int32),
        consts,
        row_nbits.to(torch.uint8),
        row_block.to(torch.uint8),
        had.to(torch.uint8).reshape(-1),
        (r, k),
        col_scale,
    )


def reconstruct_flat(flat, original: bool = True) -> torch.Tensor:
    """fp64 ``[R, K]`` reconstruction of a :class:`Flat` tensor, row by row: stored basis, or
    (``original``) rotated back and divided by the smoothing vector."""
    r, k = flat.shape
    out = torch.zeros(r, k, dtype=F64)
    for row in range(r):
        nb, bl = int(flat.row_nbits[row]), int(flat.row_block[row])
        codes = unpack_words(flat.codes[flat.code_off[row] : flat.code_off[row + 1]], nb)
        p = flat.blk_params[2 * flat.param_off[row] : 2 * flat.param_off[row + 1]].reshape(-1, 2)
        c = flat.row_consts[row]
        lo, step = decode_ladders(p[:, 0], p[:, 1], c[0], c[1], c[2])
        out[row] = reconstruct(codes.reshape(-1, bl), lo, step).double().reshape(-1)
    if original:
        out = rotate_groups(out, flat.had)
        if flat.col_scale is not None:
            out = out / flat.col_scale.double()
    return out


# --------------------------------------------------------------------------- allocation
@dataclass
class Table:
    name: str
    shape: tuple
    had: torch.Tensor
    sse: torch.Tensor  # f32 [C, R]
    candidates: list
    energy: float
    n_tokens: int = 0
    col_scale: torch.Tensor | None = None


@dataclass
class Allocation:
    picks: dict
    bpw: float
    lam: float
    feasible: bool


def _row_overhead(t: Table) -> int:
    widths = len({nb for nb, _ in t.candidates})
    return 50 + max(1, math.ceil(math.log2(max(widths, 1))))


def _first_min(v):
    best = v[0].clone()
    idx = torch.zeros(v.shape[1], dtype=torch.int64)
    for c in range(1, v.shape[0]):
        m = v[c] < best
        best = torch.where(m, v[c], best)
        idx.masked_fill_(m, c)
    return idx


def allocate_rows(tables, target_bpw: float, sensitivity=None, iters: int = 80) -> Allocation:
    """Lagrangian bisection of one multiplier over every row of every table (fp64)."""
    sens = sensitivity or {}
    cmax = max(len(t.candidates) for t in tables)
    costs, bits, spans, per_table = [], [], [], []
    off = 0
    for t in tables:
        k, r = t.shape[1], t.shape[0]
        cost = ((sens.get(t.name, 1.0) / max(t.energy, 1e-30)) * t.sse).double()
        b = torch.tensor([nb * k + 16 * k / bl for nb, bl in t.candidates], dtype=F64)
        per_table.append((cost, b))
        pad = cmax - cost.shape[0]
        costs.append(torch.cat([cost, torch.full((pad, r), float("inf"), dtype=F64)]))
        bits.append(torch.cat([b, torch.zeros(pad, dtype=F64)]).unsqueeze(1).expand(cmax, r))
        spans.append((t.name, off, off + r))
        off += r
    cost_all = torch.cat(costs, 1)
    bits_all = torch.cat(bits, 1).contiguous()
    total_w = sum(t.shape[0] * t.shape[1] for t in tables)
    overhead = sum(
        _row_overhead(t) * t.shape[0]
        + t.shape[1] // 16
        + (16 * t.shape[1] if t.col_scale is not None else 0)
        for t in tables
    )
    budget = target_bpw * total_w - overhead

    def solve(lam):
        p = _first_min(cost_all + lam * bits_all)
        pb = bits_all.gather(0, p[None])[0]
        total = 0.0
        for _, a, b in spans:
            total += pb[a:b].sum().item()
        return {name: p[a:b].clone() for name, a, b in spans}, total

    lam_hi = 1.0
    for cost, b in per_table:
        span_b = (b.max() - b.min()).clamp_min(1e-9)
        lam_hi = max(lam_hi, 2 * ((cost.max(0).values - cost.min(0).values) / span_b).max().item())
    lo, hi = lam_hi * 1e-12, lam_hi

    def done(p, b, lam, ok):
        return Allocation(p, (b + overhead) / total_w, lam, ok)

    picks, total = solve(hi)
    if total > budget:
        return done(picks, total, hi, False)
    rich = solve(lo)
    if rich[1] <= budget:
        return done(rich[0], rich[1], lo, True)
    lam = hi
    for _ in range(iters):
        mid = (lo * hi) ** 0.5
        p, b = solve(mid)
        if b <= budget:
            hi, picks, total, lam = mid, p, b, mid
        else:
            lo = mid
    return done(picks, total, lam, True)
