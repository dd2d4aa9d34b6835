"""One block of columns of the refinement sweep on B200 (interface of hi2/refine_kernel.py)."""

from __future__ import annotations

import torch

from . import _lib
from .gptq_kernel import kernel_dir, supported  # noqa: F401

BLOCK_COLUMNS = 128


def load():
    return _lib.load()


def available(dev: torch.device) -> bool:
    return supported(dev) and load() is not None


def failure() -> str | None:
    return _lib.failure()


def refine_block(gb, c, lo_x, st_x, top, hs, b0, length, dw_block) -> None:
    """Columns ``[b0, b0 + length)``: ``c [N, K]`` (fp32 codes) is updated in place and
    ``dw_block [N, length]`` receives the change of each decoded value (hi2/refine_kernel.py:173)."""
    dev = _lib.need_cuda(gb, c, lo_x, st_x, top, hs, dw_block)
    for t, name in ((gb, "gb"), (c, "c"), (lo_x, "lo"), (st_x, "st"), (top, "top"), (hs, "hs"),
                    (dw_block, "dw_block")):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError(f"refine_block: {name} must be a contiguous float32 tensor")
    n, k = c.shape
    if not (0 < length <= BLOCK_COLUMNS) or gb.shape[1] != length or dw_block.shape[1] != length:
        raise ValueError("refine_block: bad block length")
    if b0 < 0 or b0 + length > k or hs.shape != (k, k):
        raise ValueError("refine_block: block outside the row or hs of the wrong shape")
    if n == 0:
        return
    _lib.call(
        "hi2_refine_block", _lib.ptr(gb), int(length), _lib.ptr(c), _lib.ptr(lo_x), _lib.ptr(st_x),
        _lib.ptr(top), _lib.ptr(hs), n, k, int(b0), _lib.ptr(dw_block), _lib.stream(dev),
    )


def refine_block_in_place(g, c, lo_x, st_x, top, hs, b0, length, dw_split) -> None:
    """:func:`refine_block` reading the block's slice of ``g [N, K]`` where it lies and writing the
    changes as TF32 parts ``dw_split [2, N, length]``, the left operand of :func:`gemm_tc`;
    ``dw_split`` may be a column slice of a wider ``[2, N, W]`` buffer (unit column stride)."""
    dev = _lib.need_cuda(g, c, lo_x, st_x, top, hs, dw_split)
    for t, name in ((g, "g"), (c, "c"), (lo_x, "lo"), (st_x, "st"), (top, "top"), (hs, "hs")):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError(f"refine_block_in_place: {name} must be a contiguous float32 tensor")
    n, k = c.shape
    if not (0 < length <= BLOCK_COLUMNS) or g.shape != (n, k) or dw_split.shape != (2, n, length):
        raise ValueError("refine_block_in_place: bad block length or shape")
    if dw_split.dtype != torch.float32 or dw_split.stride(2) != 1 or (n > 1 and dw_split[0].stride(0) != dw_split[1].stride(0)):
        raise ValueError("refine_block_in_place: dw_split must be float32 with unit column stride")
    if b0 < 0 or b0 + length > k or hs.shape != (k, k):
        raise ValueError("refine_block_in_place: block outside the row or hs of the wrong shape")
    if n == 0:
        return
    _lib.call(
        "hi2_refine_block_in_place", _lib.ptr(g), int(length), _lib.ptr(c), _lib.ptr(lo_x), _lib.ptr(st_x),
        _lib.ptr(top), _lib.ptr(hs), n, k, int(b0), _lib.ptr(dw_split[0]), _lib.ptr(dw_split[1]),
        dw_split.stride(1), _lib.stream(dev),
    )


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, alpha=1.0, beta=0.0) -> None:
    """``out = alpha * a @ b + beta * out`` in fp32 FMA arithmetic; row-major views with unit
    column stride (row strides are passed as leading dimensions)."""
    dev = _lib.need_cuda(a, b, out)
    for t in (a, b, out):
        if t.dtype != torch.float32 or t.stride(1) != 1:
            raise ValueError("gemm: operands must be fp32 with unit column stride")
    m, kk = a.shape
    n = b.shape[1]
    if b.shape[0] != kk or out.shape != (m, n):
        raise ValueError("gemm: shape mismatch")
    _lib.call(
        "hi2_gemm_f32", 0, 0, m, n, kk, float(alpha), _lib.ptr(a), a.stride(0), _lib.ptr(b),
        b.stride(0), float(beta), _lib.ptr(out), out.stride(0), _lib.stream(dev),
    )


def split_tf32(x: torch.Tensor) -> torch.Tensor:
    """``[2, *x.shape]``: the TF32 parts ``hi = tf32(x)``, ``lo = tf32(x - hi)`` of a contiguous fp32
    tensor, the operand form of :func:`gemm_tc`."""
    dev = _lib.need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.numel() % 4:
        raise ValueError("split_tf32: a contiguous fp32 tensor with a multiple of 4 elements")
    out = torch.empty(2, *x.shape, dtype=torch.float32, device=dev)
    _lib.call("hi2_split_tf32", _lib.ptr(x), _lib.ptr(out[0]), _lib.ptr(out[1]), x.numel(), _lib.stream(dev))
    return out


def gemm_tc(a_split: torch.Tensor, bt_split: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
            accumulate: bool = False) -> None:
    """``out (+)= a @ bt^T`` with fp32-grade accuracy on the tensor cores; ``a_split [2, m, kk]`` and
    ``bt_split [2, n, kk]`` are TF32 parts (views with unit column stride are fine, both parts of an
    operand with the same row stride)."""
    dev = _lib.need_cuda(a_split, bt_split, out, status)
    _, m, kk = a_split.shape
    n = bt_split.shape[1]
    if bt_split.shape[2] != kk or out.shape != (m, n) or a_split.stride(2) != 1 or bt_split.stride(2) != 1:
        raise ValueError("gemm_tc: shape mismatch")
    _lib.call(
        "hi2_gemm_tf32x3", m, n, kk, _lib.ptr(a_split[0]), _lib.ptr(a_split[1]), a_split.stride(1),
        _lib.ptr(bt_split[0]), _lib.ptr(bt_split[1]), bt_split.stride(1), _lib.ptr(out), out.stride(0),
        1 if accumulate else 0, _lib.ptr(status), _lib.stream(dev),
    )
