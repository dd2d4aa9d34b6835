"""Rotation, packing and flat-buffer assembly of the ``rdna_hint_flex`` format on B200.

Same names and results as the functions of hi2/format.py that the PTQ encode path uses
(``fwht_groups`` :30-41, ``pack_codes`` :73-85, ``assemble`` :127-184); the work runs in
``libhi2_b200.so``.  ``decode_params`` / ``ladder_dequantize`` / ``unpack_codes`` are the
decoder-side definitions (hi2/format.py:45-69, :88-93) written with elementwise tensor ops; the
encode kernels carry their own copies of that arithmetic.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib

GROUP = 16


def hadamard16(dtype: torch.dtype = torch.float64, device="cpu") -> torch.Tensor:
    """Normalised order-16 Walsh-Hadamard matrix (symmetric, its own inverse)."""
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < GROUP:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (h / math.sqrt(GROUP)).to(dtype=dtype, device=device)


def fwht_groups(x: torch.Tensor, flags: torch.Tensor, col_scale: torch.Tensor | None = None,
                out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Transform the flagged 16-column groups of ``x[..., K]`` (an involution).

    Extensions over the reference signature, all optional: ``col_scale`` (``[K]``, multiplied
    in fp32 before the rotation, as ``W * s`` in hi2/calibrate.py:247-250), ``out_dtype``
    (``torch.float32`` lets a bf16/fp16 tensor be cast, scaled and rotated in one pass) and ``out``
    (a contiguous tensor of the result's shape and dtype to write into, e.g. a slice of a buffer
    that holds several tensors one after the other)."""
    k = x.shape[-1]
    if k % GROUP:
        raise ValueError(f"K={k} must be a multiple of {GROUP}")
    if flags.numel() != k // GROUP:
        raise ValueError(f"flags has {flags.numel()} entries, expected {k // GROUP}")
    dev = _lib.need_cuda(x)
    if x.dtype not in _lib.DTYPES:
        raise ValueError(f"unsupported dtype {x.dtype}")
    out_dtype = out_dtype or x.dtype
    xc = x.contiguous()
    if out is None:
        y = torch.empty(xc.shape, dtype=out_dtype, device=dev)
    else:
        if out.shape != xc.shape or out.dtype != out_dtype or out.device != dev or not out.is_contiguous():
            raise ValueError("fwht_groups: out must be a contiguous tensor of the result's shape, dtype and device")
        y = out
    fl = _lib.upload(flags, dev, torch.uint8)
    cs = None
    if col_scale is not None:
        cs = _lib.upload(col_scale, dev, torch.float32)
    rows = xc.numel() // k
    _lib.call(
        "hi2_rotate_groups", _lib.ptr(xc), _lib.DTYPES[x.dtype], _lib.ptr(y), _lib.DTYPES[out_dtype],
        _lib.ptr(fl), _lib.ptr(cs), rows, k, _lib.stream(dev),
    )
    return y


# ---- block parameters ---------------------------------------------------------------------
def decode_params(lo_u8, step_u8, lo_min, lo_scale, step_scale):
    """fp16 ``lo = fp16(fma_f32(u, lo_scale, lo_min))`` and ``step = fp16(u * step_scale)``."""
    lo = (lo_u8.double() * lo_scale.double() + lo_min.double()).float().to(torch.float16)
    step = (step_u8.float() * step_scale.float()).to(torch.float16)
    return lo, step


def ladder_dequantize(codes, lo, step, dtype=torch.float64):
    """``fp16(lo + code * step)`` with the sum formed in ``dtype``."""
    v = lo.to(dtype).unsqueeze(-1) + codes.to(dtype) * step.to(dtype).unsqueeze(-1)
    return v.to(torch.float16)


# ---- code packing ---------------------------------------------------------------------------
def pack_codes(codes: torch.Tensor, nbits: int) -> torch.Tensor:
    """``[..., n]`` codes -> ``[..., n * nbits / 32]`` int32, first code in the low bits."""
    per_word = 32 // nbits
    n = codes.shape[-1]
    if n % per_word:
        raise ValueError(f"{n} codes is not a multiple of {per_word}")
    dev = _lib.need_cuda(codes)
    if codes.dtype != torch.uint8:
        if codes.numel() and (int(codes.max()) >= 2**nbits or int(codes.min()) < 0):
            raise ValueError("code outside the ladder")
        codes = codes.to(torch.uint8)
    c = codes.contiguous()
    words = torch.empty(*c.shape[:-1], n // per_word, dtype=torch.int32, device=dev)
    bad = torch.zeros(1, dtype=torch.int32, device=dev)
    _lib.call(
        "hi2_pack_codes", _lib.ptr(c), _lib.ptr(words), c.numel() // max(n, 1), n, nbits,
        _lib.ptr(bad), _lib.stream(dev),
    )
    if int(bad.item()):
        raise ValueError("code outside the ladder")
    return words


def unpack_codes(words: torch.Tensor, nbits: int) -> torch.Tensor:
    """Inverse of :func:`pack_codes` (hi2/format.py:88-93): field ``i`` of a word occupies bits
    ``[i * nbits, (i + 1) * nbits)``.  Returns int64 codes ``[..., n_words * 32 / nbits]``."""
    shifts = torch.arange(0, 32, nbits, device=words.device)
    fields = (words.to(torch.int64).unsqueeze(-1) >> shifts) & (2**nbits - 1)
    return fields.flatten(-2)


# ---- tensor container ---------------------------------------------------------------------------
@dataclass
class HI2Tensor:
    """Flat per-tensor buffers (hi2/format.py:97-112)."""

    codes: torch.Tensor  # int32 [sum words_per_row]
    code_off: torch.Tensor  # int32 [R+1]
    blk_params: torch.Tensor  # uint8 [2 * sum K/B_r]
    param_off: torch.Tensor  # int32 [R+1], in blocks
    row_consts: torch.Tensor  # fp16 [R, 3]
    row_nbits: torch.Tensor  # uint8 [R]
    row_block: torch.Tensor  # uint8 [R]
    had: torch.Tensor  # uint8 [K/16]
    shape: tuple[int, int]
    col_scale: torch.Tensor | None = None


FIELDS = ("codes", "code_off", "blk_params", "param_off", "row_consts", "row_nbits", "row_block", "had")


def _to_pinned(t: torch.Tensor) -> torch.Tensor:
    """A copy of device tensor ``t`` in page-locked host memory, queued on the current stream (the
    caller synchronises before reading).  A plain ``.cpu()`` goes through pageable memory at a
    fraction of the link's speed and makes the host wait for every buffer in turn."""
    h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
    h.copy_(t, non_blocking=True)
    return h


def assemble(pieces, row_nbits, row_block, had, k: int, col_scale=None, stager=None,
             to_host: bool = True, bad: torch.Tensor | None = None, wait: bool = True) -> HI2Tensor:
    """Flat buffers from per-candidate pieces ``(rows, codes[r, K] u8, params[r, nb, 2] u8,
    consts[r, 3] fp16)``.  A piece may carry its ``(nbits, block)`` as fifth and sixth entry, which
    saves reading ``rows[0]`` back from the device; ``bad`` (optional, a device int32) collects the
    out-of-ladder flag for a caller that checks it once for several tensors instead of waiting
    for every one of them here.

    The packing and the scatters run on the device of the first piece.  As in the reference the
    result is returned on the host (``to_host=False`` keeps the three big buffers on the device,
    which is what a caller that overlaps the copy wants); the host buffers are page-locked, and with
    ``wait=False`` their copies are only queued on the current stream: the caller synchronises once
    for several tensors.  ``stager`` is accepted for signature compatibility and ignored."""
    del stager
    r = row_nbits.numel()
    nb = row_nbits.to("cpu", torch.int64)
    bl = row_block.to("cpu", torch.int64)
    code_off = torch.zeros(r + 1, dtype=torch.int64)
    code_off[1:] = torch.cumsum((k * nb) // 32, 0)
    param_off = torch.zeros(r + 1, dtype=torch.int64)
    param_off[1:] = torch.cumsum(k // bl, 0)
    if not pieces:
        dev = torch.device("cpu")
        codes = torch.zeros(int(code_off[-1]), dtype=torch.int32)
        params = torch.zeros(int(param_off[-1]) * 2, dtype=torch.uint8)
        consts = torch.zeros(r, 3, dtype=torch.float16)
    else:
        dev = _lib.need_cuda(*[p[1] for p in pieces])
        code_off_d, param_off_d = _lib.upload(code_off, dev), _lib.upload(param_off, dev)
        codes = torch.zeros(int(code_off[-1]), dtype=torch.int32, device=dev)
        params = torch.zeros(int(param_off[-1]) * 2, dtype=torch.uint8, device=dev)
        consts = torch.zeros(r, 3, dtype=torch.float16, device=dev)
        check_here = bad is None
        if check_here:
            bad = torch.zeros(1, dtype=torch.int32, device=dev)
        for piece in pieces:
            rows, c, p, rc = piece[:4]
            if rows.numel() == 0:
                continue
            if len(piece) >= 6:
                nbits, block = int(piece[4]), int(piece[5])
            else:
                first = int(rows[0])
                nbits, block = int(nb[first]), int(bl[first])
            rows_d = rows.to(dev, torch.int64).contiguous()
            c = c.to(dev, torch.uint8).contiguous()
            p = p.to(dev, torch.uint8).contiguous()
            rc = rc.to(dev, torch.float16).contiguous()
            _lib.call(
                "hi2_assemble_piece", _lib.ptr(rows_d), rows_d.numel(), _lib.ptr(c), _lib.ptr(p),
                _lib.ptr(rc), k, nbits, block, _lib.ptr(code_off_d), _lib.ptr(param_off_d),
                _lib.ptr(codes), _lib.ptr(params), _lib.ptr(consts), _lib.ptr(bad), _lib.stream(dev),
            )
        if check_here and int(bad.item()):
            raise ValueError("code outside the ladder")
    if to_host and codes.is_cuda:
        codes, params, consts = _to_pinned(codes), _to_pinned(params), _to_pinned(consts)
        if col_scale is not None and col_scale.is_cuda:
            col_scale = _to_pinned(col_scale)
        if wait:
            torch.cuda.current_stream(dev).synchronize()
    return HI2Tensor(
        codes=codes,
        code_off=code_off.to(torch.int32),
        blk_params=params,
        param_off=param_off.to(torch.int32),
        row_consts=consts,
        row_nbits=row_nbits.to("cpu", torch.uint8),
        row_block=row_block.to("cpu", torch.uint8),
        had=had.to("cpu", torch.uint8).reshape(-1),
        shape=(r, k),
        col_scale=col_scale.cpu() if (to_host and col_scale is not None and col_scale.is_cuda) else col_scale,
    )


# ---- the inverse path ---------------------------------------------------------------------------
def _dequantize(t: HI2Tensor, device, original: bool, dtype: torch.dtype) -> torch.Tensor:
    if dtype not in (torch.float64, torch.float32):
        raise ValueError("dequantize: dtype must be float64 or float32")
    dev = torch.device(device) if device is not None else (
        t.codes.device if t.codes.is_cuda else torch.device("cuda", torch.cuda.current_device()))
    if dev.type != "cuda":
        raise RuntimeError("hi2_b200 runs on CUDA devices only; there is no CPU path")
    r, k = t.shape
    out = torch.empty(r, k, dtype=dtype, device=dev)
    if r == 0:
        return out
    codes = _lib.upload(t.codes, dev, torch.int32)
    code_off = _lib.upload(t.code_off, dev, torch.int32)
    params = _lib.upload(t.blk_params, dev, torch.uint8)
    param_off = _lib.upload(t.param_off, dev, torch.int32)
    consts = _lib.upload(t.row_consts, dev, torch.float16)
    nbits = _lib.upload(t.row_nbits, dev, torch.uint8)
    block = _lib.upload(t.row_block, dev, torch.uint8)
    had = _lib.upload(t.had, dev, torch.uint8)
    cs = None if t.col_scale is None else _lib.upload(t.col_scale, dev, torch.float16)
    bad = torch.zeros(1, dtype=torch.int32, device=dev)
    _lib.call(
        "hi2_dequantize", _lib.ptr(codes), _lib.ptr(code_off), _lib.ptr(params), _lib.ptr(param_off),
        _lib.ptr(consts), _lib.ptr(nbits), _lib.ptr(block), _lib.ptr(had), _lib.ptr(cs), r, k, 1 if original else 0,
        _lib.ptr(out), _lib.DTYPES[dtype], _lib.ptr(bad), _lib.stream(dev),
    )
    if int(bad.item()):
        raise ValueError("dequantize: a row's code width or block size is not one of the format's")
    return out


def dequantize_stored(t: HI2Tensor, device=None, dtype: torch.dtype = torch.float64) -> torch.Tensor:
    """fp16 reconstruction in the stored (rotated, smoothed) basis as ``[R, K]`` on the device
    (hi2/format.py:195-228).  Every step is exact, so the float64 result equals the reference's."""
    return _dequantize(t, device, False, dtype)


def dequantize(t: HI2Tensor, device=None, dtype: torch.dtype = torch.float64) -> torch.Tensor:
    """Reconstruction in the original basis: the rotation is its own inverse and the smoothing
    vector is divided back out (hi2/format.py:231-239)."""
    return _dequantize(t, device, True, dtype)


# ---- the product a decode kernel computes, and the bit accounting of the format ---------------------
def reference_linear(x: torch.Tensor, t: HI2Tensor, device=None) -> torch.Tensor:
    """``x [M, K] @ W^T`` the way an inference kernel forms it (hi2/format.py:242-249): the
    activation is divided by the smoothing vector and rotated with the tensor's flags, then
    contracted with the stored-basis reconstruction.  fp64, on the device."""
    dev = torch.device(device) if device is not None else (x.device if x.is_cuda else torch.device("cuda", torch.cuda.current_device()))
    xd = x.to(dev, torch.float64)
    if t.col_scale is not None:
        xd = xd / t.col_scale.to(dev, torch.float64)
    return fwht_groups(xd.contiguous(), t.had) @ dequantize_stored(t, dev).T


def block_bits_per_weight(nbits: int, block: int) -> float:
    """Code bits plus the two parameter bytes of a block, per weight (row constants not counted)."""
    return nbits + 16 / block


def metadata_bits(row_nbits: torch.Tensor, row_block: torch.Tensor, had: torch.Tensor) -> int:
    """Bits a loader needs besides the buffers (hi2/format.py:253-265): the rotation flags (one bit when
    all groups agree, else one per group), per row ``ceil(log2(#code widths))`` bits when the rows
    use more than one width, and two more per row when they use more than one block size."""
    flags = had.reshape(-1)
    bits = 1 if flags.numel() == 0 or bool((flags == flags[0]).all()) else flags.numel()
    rows = row_nbits.numel()
    widths = int(torch.unique(row_nbits).numel())
    if widths > 1:
        bits += rows * math.ceil(math.log2(widths))
    if int(torch.unique(row_block).numel()) > 1:
        bits += 2 * rows
    return bits


def tensor_bpw(t: HI2Tensor) -> float:
    """Exact bits per weight of a packed tensor: codes and parameter bytes of every row, 48 bits of
    row constants per row, the metadata above, and 16 bits per column for a smoothing vector."""
    r, k = t.shape
    width, block = t.row_nbits.to(torch.float64), t.row_block.to(torch.float64)
    payload = float((width * k + 16 * k / block).sum())
    vector = 16 * k if t.col_scale is not None else 0
    return (payload + 48 * r + metadata_bits(t.row_nbits, t.row_block, t.had) + vector) / (r * k)
