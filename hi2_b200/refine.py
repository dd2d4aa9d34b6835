"""Local code refinement after GPTQ on B200 (interface of hi2/refine.py:24-162).

A sweep visits the columns in blocks of 128: one launch of the block kernel decides every column
of the block for every row (csrc/refine.cu), one fp32-grade product (three TF32 tcgen05 products,
csrc/lazy_tc.cu; fp32 FMA for narrow inputs and 256-level rows) brings ``g = e Hs`` up to date for
the other columns.  Ladders are never touched.
"""

from __future__ import annotations

import torch

from . import _lib, refine_kernel
from .format import decode_params

BLOCK_COLUMNS = 128
GROUP_BLOCKS = 4  # blocks whose moves reach the far columns of g in one product
GROUP_MIN_ELEMS = 1 << 25  # rows x columns from which grouping pays (below, a step is a latency chain)
TC_MIN_K = 512  # inputs at least this wide take the tensor-core products


@torch.no_grad()
def objective(w, codes, lo, step, hs, block) -> float:
    """Sum over rows of ``e Hs e^T`` for the decoded codes."""
    idx = torch.arange(w.shape[1], device=w.device) // block
    e = ((lo[:, idx] + codes.float() * step[:, idx]).half().float() - w).contiguous()
    g = torch.empty_like(e)
    refine_kernel.gemm(e, hs.float().contiguous(), g)
    return float((g * e).sum())


def _expand(lo: torch.Tensor, step: torch.Tensor, block: int):
    """Per-column ladders ``[N, K]`` from the per-block ones ``[N, K / block]``."""
    return lo.repeat_interleave(block, dim=1), step.repeat_interleave(block, dim=1)


@torch.no_grad()
def _sweeps(w, codes, lo_x, st_x, top, hs, passes: int, use_tc: bool | None, wait: bool):
    """``(refined codes (float), status word or None)``.  With ``wait`` the host follows the device:
    it stops after a sweep that moved no code and raises on a raised status word.  Without, nothing
    is read back: every sweep is queued (one that moves nothing changes nothing) and the status
    word is left to the caller, so several tensors can be refined side by side on streams."""
    dev = _lib.need_cuda(w, codes, lo_x, st_x, top, hs)
    if not refine_kernel.available(dev):
        raise RuntimeError(f"refine kernel unavailable on {dev}: {refine_kernel.failure()}")
    n_rows, k = w.shape
    c = codes.float().contiguous().clone()
    lo_x, st_x = lo_x.float().contiguous(), st_x.float().contiguous()
    top = top.float().contiguous()
    hs = hs.float().contiguous()
    e = ((lo_x + c * st_x).half().float() - w.float()).contiguous()
    g = torch.empty(n_rows, k, dtype=torch.float32, device=dev)
    # The two products of a sweep, g = e Hs and g += dw Hs[b0:b1], run on the tensor cores as three
    # TF32 products (fp32-grade; Hs is symmetric, so its rows are the K-major right operand as they
    # lie).  Rows with 256 levels and narrow inputs keep the fp32 FMA product, as in the GPTQ path.
    if use_tc is None:
        use_tc = bool((top <= 15).all())
    use_tc = use_tc and k >= TC_MIN_K and k % 4 == 0
    status = None
    if use_tc:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        hs_split = refine_kernel.split_tf32(hs)
        refine_kernel.gemm_tc(refine_kernel.split_tf32(e), hs_split, g, status)
    else:
        refine_kernel.gemm(e, hs, g)
    del e
    # With tensor-core products the block kernel reads its slice of g in place and leaves the changes
    # as TF32 parts, and g is brought up to date lazily, as the GPTQ loop does: after a block only the
    # later blocks of its group of GROUP_BLOCKS need its moves now (a narrow product); the columns
    # outside the group take the moves of the whole group in one product with a reduction of up to
    # 512 (a 128 KiB tile of g is then read and written once per 100 MFLOP instead of once per 25);
    # the group's own columns at or before each block, needed by the next sweep only, follow per
    # column block.  The contributions to every g are the same, in another order.  Few rows make
    # every step a latency chain, where more launches cost more than the better products gain: then
    # a group is one block and its update one product.
    width = (GROUP_BLOCKS if n_rows * k >= GROUP_MIN_ELEMS else 1) * BLOCK_COLUMNS
    moves = torch.empty(2, n_rows, min(width, k), dtype=torch.float32, device=dev) if use_tc else None
    for _ in range(passes):
        start = c.clone() if wait else None
        if not use_tc:
            for b0 in range(0, k, BLOCK_COLUMNS):
                b1 = min(b0 + BLOCK_COLUMNS, k)
                gb = g[:, b0:b1].contiguous()
                dw_block = torch.empty(n_rows, b1 - b0, dtype=torch.float32, device=dev)
                refine_kernel.refine_block(gb, c, lo_x, st_x, top, hs, b0, b1 - b0, dw_block)
                refine_kernel.gemm(dw_block, hs[b0:b1], g, alpha=1.0, beta=1.0)
            if wait and bool((c == start).all()):
                break
            continue
        for g0 in range(0, k, width):
            g1 = min(g0 + width, k)
            for b0 in range(g0, g1, BLOCK_COLUMNS):
                b1 = min(b0 + BLOCK_COLUMNS, g1)
                dw = moves[:, :, b0 - g0 : b1 - g0]
                refine_kernel.refine_block_in_place(g, c, lo_x, st_x, top, hs, b0, b1 - b0, dw)
                if b1 < g1:
                    refine_kernel.gemm_tc(dw, hs_split[:, b1:g1, b0:b1], g[:, b1:g1], status, accumulate=True)
            if width == BLOCK_COLUMNS:  # groups of one block: the whole update in one product
                refine_kernel.gemm_tc(moves[:, :, : g1 - g0], hs_split[:, :, g0:g1], g, status, accumulate=True)
                continue
            group = moves[:, :, : g1 - g0]
            if g0 > 0:
                refine_kernel.gemm_tc(group, hs_split[:, :g0, g0:g1], g[:, :g0], status, accumulate=True)
            if g1 < k:
                refine_kernel.gemm_tc(group, hs_split[:, g1:, g0:g1], g[:, g1:], status, accumulate=True)
            for b0 in range(g0, g1, BLOCK_COLUMNS):
                b1 = min(b0 + BLOCK_COLUMNS, g1)
                refine_kernel.gemm_tc(moves[:, :, b0 - g0 : g1 - g0], hs_split[:, b0:b1, b0:g1], g[:, b0:b1], status,
                                      accumulate=True)
        if wait and bool((c == start).all()):
            break
    if wait and use_tc and int(status.item()):
        raise RuntimeError("refine: a bounded device-side wait ran out in a tensor-core product")
    return c, status


def refine_expanded(w, codes, lo_x, st_x, top, hs, passes: int) -> torch.Tensor:
    """Refined codes (float) of rows ``w [N, K]`` with per-column ladders ``lo_x``/``st_x`` and
    the highest code of each row ``top [N]``; stops early when a sweep moves no code."""
    return _sweeps(w, codes, lo_x, st_x, top, hs, passes, None, True)[0]


def refine_codes(w, codes, lo, step, hs, nbits: int, block: int, passes: int) -> torch.Tensor:
    """:func:`refine_expanded` for rows rounded at one ``(nbits, block)`` with decoded ladders
    ``lo``/``step [N, K / block]``; returns codes of the dtype of ``codes``."""
    lo_x, st_x = _expand(lo, step, block)
    top = torch.full((w.shape[0],), float(2**nbits - 1), device=w.device)
    return refine_expanded(w, codes, lo_x, st_x, top, hs, passes).to(codes.dtype)


def _decoded(enc):
    lo, step = decode_params(
        enc.params[..., 0], enc.params[..., 1], enc.consts[:, 0:1], enc.consts[:, 1:2],
        enc.consts[:, 2:3],
    )
    return lo.float(), step.float()


def refine_groups(groups, hs: torch.Tensor, passes: int, wait: bool = True):
    """One sweep over the rows of every ``(w, enc, nbits, block)`` group (rows of different
    candidates, and of different tensors that read the same input, share the column loop); returns
    the refined codes per group.  ``wait=False`` reads nothing back and returns ``(codes per group,
    status word or None)``: the caller checks the word once it has queued everything."""
    parts = []
    for w, enc, nbits, block in groups:
        lo, step = _decoded(enc)
        lo_x, st_x = _expand(lo, step, block)
        top = torch.full((w.shape[0],), float(2**nbits - 1), device=w.device)
        parts.append((w.float(), enc.codes.float(), lo_x, st_x, top))
    cat = [torch.cat([p[i] for p in parts]) for i in range(5)]
    out, status = _sweeps(*cat, hs, passes, max(g[2] for g in groups) <= 4, wait)
    sizes = [p[0].shape[0] for p in parts]
    codes = [c.to(groups[i][1].codes.dtype) for i, c in enumerate(out.split(sizes))]
    return codes if wait else (codes, status)


def refine_encoded(enc, w, hs, nbits: int, block: int, passes: int):
    """``enc`` with refined codes and a refreshed ``sse`` (weights ``diag(hs)``)."""
    (codes,) = refine_groups([(w, enc, nbits, block)], hs, passes)
    lo, step = _decoded(enc)
    dev = w.device
    k = w.shape[1]
    wf = w.float().contiguous()
    codes = codes.contiguous()
    d = hs.diagonal().float().contiguous()
    lo, step = lo.contiguous(), step.contiguous()
    sse = torch.empty(w.shape[0], dtype=torch.float32, device=dev)
    _lib.call(
        "hi2_ladder_sse", _lib.ptr(codes), _lib.ptr(wf), wf.stride(0), _lib.ptr(d), _lib.ptr(lo),
        _lib.ptr(step), lo.shape[1], w.shape[0], k, block, _lib.ptr(sse), _lib.stream(dev),
    )
    return type(enc)(codes, enc.params, enc.consts, sse, enc.comp)
