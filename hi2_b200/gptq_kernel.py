"""GPTQ column loop for one lazy-update block on B200 (interface of hi2/gptq_kernel.py).

``gptq_block`` keeps the reference's argument list (hi2/gptq_kernel.py:187-196) and buffer
contract: the caller allocates every tensor, ``u_ptrs`` holds device addresses of contiguous
``[K, K]`` fp32 factors, rows of several tensors share one launch through ``row_grp``.
There is no torch fallback: ``available`` is true on CUDA devices once the library loads, and
the entry points raise when it does not.
"""

from __future__ import annotations

from pathlib import Path

import torch

from . import _lib

BLOCK_COLUMNS = 128


def kernel_dir() -> Path:
    """Directory of the prebuilt library (the reference returns its JIT cache here)."""
    return _lib.LIB_PATH.parent


def supported(dev: torch.device) -> bool:
    """A CUDA device of compute capability 10.x (the library is built for sm_100a only)."""
    dev = torch.device(dev)
    if dev.type != "cuda" or torch.version.hip or not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_capability(dev)[0] == 10


def load():
    return _lib.load()


def available(dev: torch.device) -> bool:
    return supported(dev) and load() is not None


def failure() -> str | None:
    return _lib.failure()


def _check(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if t.dtype != dtype or not t.is_contiguous():
        raise ValueError(f"gptq_block: {name} must be a contiguous {dtype} tensor")


def gptq_block(wc, i1, length, err1, codes, lo, st, row_grp, u_ptrs, blk, nmax, comp=None) -> None:
    """Round columns ``[i1, i1 + length)`` of every row of ``wc [N, K]``; writes ``codes[:, j]``,
    ``err1 [N, length]`` and, when given, ``comp[:, j]`` (the value each code was rounded from)."""
    dev = _lib.need_cuda(wc, err1, codes, lo, st, row_grp, u_ptrs, blk, nmax, comp)
    for t, dt, name in ((wc, torch.float32, "wc"), (err1, torch.float32, "err1"),
                        (codes, torch.uint8, "codes"), (lo, torch.float32, "lo"),
                        (st, torch.float32, "st"), (row_grp, torch.int32, "row_grp"),
                        (u_ptrs, torch.int64, "u_ptrs"), (blk, torch.int32, "blk"),
                        (nmax, torch.float32, "nmax")):
        _check(t, dt, name)
    n, k = wc.shape
    if not (0 < length <= BLOCK_COLUMNS) or err1.shape[1] != length:
        raise ValueError("gptq_block: bad block length")
    if comp is not None and comp.numel() == 0:
        comp = None
    if comp is not None:
        _check(comp, torch.float32, "comp")
        if comp.shape != wc.shape:
            raise ValueError("gptq_block: comp must have the shape of wc")
    if n == 0:
        return
    _lib.call(
        "hi2_gptq_block", _lib.ptr(wc), n, k, int(i1), int(length), _lib.ptr(err1), _lib.ptr(codes),
        _lib.ptr(lo), _lib.ptr(st), lo.shape[1], _lib.ptr(row_grp), _lib.ptr(u_ptrs), _lib.ptr(blk),
        _lib.ptr(nmax), _lib.ptr(comp), _lib.stream(dev),
    )


def gptq_round(wc, err1, codes, lo, st, row_grp, u_ptrs, blk, nmax, comp, unit_rows, unit_u) -> None:
    """The whole column loop of hi2/hessian.py:267-315 in one call: for every lazy block the
    block kernel over all rows, then ``wc[o:o+n, i2:] -= err1[o:o+n] @ u[i1:i2, i2:]`` per unit.
    ``unit_rows`` are the ``len(units) + 1`` row offsets, ``unit_u`` the factor of each unit."""
    dev = _lib.need_cuda(wc, err1, codes, lo, st, row_grp, u_ptrs, blk, nmax, comp, *unit_u)
    n, k = wc.shape
    if n == 0:
        return
    for u in unit_u:
        _check(u, torch.float32, "u")
    _lib.call(
        "hi2_gptq_round", _lib.ptr(wc), n, k, _lib.ptr(err1), _lib.ptr(codes), _lib.ptr(lo),
        _lib.ptr(st), lo.shape[1], _lib.ptr(row_grp), _lib.ptr(u_ptrs), _lib.ptr(blk), _lib.ptr(nmax),
        _lib.ptr(comp), len(unit_u), _lib.host_i64(unit_rows),
        _lib.host_i64([u.data_ptr() for u in unit_u]), _lib.stream(dev),
    )


def split_tf32(x: torch.Tensor) -> torch.Tensor:
    """``[2, *x.shape]`` fp32: the TF32 parts ``hi = tf32(x)`` and ``lo = tf32(x - hi)`` (round to
    nearest), the operand form of the tensor-core trailing update."""
    dev = _lib.need_cuda(x)
    _check(x, torch.float32, "x")
    out = torch.empty(2, *x.shape, dtype=torch.float32, device=dev)
    _lib.call("hi2_split_tf32", _lib.ptr(x), _lib.ptr(out[0]), _lib.ptr(out[1]), x.numel(), _lib.stream(dev))
    return out


def split_tf32_transposed(x: torch.Tensor) -> torch.Tensor:
    """``[2, cols, rows]`` fp32: the TF32 parts of ``x^T`` for ``x [rows, cols]`` (the form in which
    the tensor-core trailing update takes the factor)."""
    dev = _lib.need_cuda(x)
    _check(x, torch.float32, "x")
    rows, cols = x.shape
    out = torch.empty(2, cols, rows, dtype=torch.float32, device=dev)
    _lib.call("hi2_split_tf32_transposed", _lib.ptr(x), _lib.ptr(out[0]), _lib.ptr(out[1]), rows, cols,
              _lib.stream(dev))
    return out


def gptq_round_tc(wc, err1, codes, lo, st, row_grp, u_ptrs, blk, nmax, comp, unit_rows, unit_u_split):
    """:func:`gptq_round` with the trailing update on the tensor cores (3 x TF32, fp32-grade).
    ``unit_u_split`` holds :func:`split_tf32_transposed` of each unit's factor.  Returns the device status
    word (int32 tensor): non-zero when a bounded device-side wait ran out."""
    dev = _lib.need_cuda(wc, err1, codes, lo, st, row_grp, u_ptrs, blk, nmax, comp, *unit_u_split)
    n, k = wc.shape
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    if n == 0:
        return status
    err_split = torch.empty(2, n, BLOCK_COLUMNS, dtype=torch.float32, device=dev)
    for u in unit_u_split:
        _check(u, torch.float32, "u_split")
        if u.shape != (2, k, k):
            raise ValueError("gptq_round_tc: a split factor must be [2, K, K]")
    _lib.call(
        "hi2_gptq_round_tc", _lib.ptr(wc), n, k, _lib.ptr(err1), _lib.ptr(err_split), _lib.ptr(codes),
        _lib.ptr(lo), _lib.ptr(st), lo.shape[1], _lib.ptr(row_grp), _lib.ptr(u_ptrs), _lib.ptr(blk),
        _lib.ptr(nmax), _lib.ptr(comp), len(unit_u_split), _lib.host_i64(unit_rows),
        _lib.host_i64([u.data_ptr() for u in unit_u_split]), _lib.ptr(status), _lib.stream(dev),
    )
    return status
