"""ctypes binding of ``libhi2_b200.so`` (the C-ABI of ``include/hi2_b200.h``).

There is no fallback: a missing library raises at first use, and every entry point returns a
status that is turned into an exception here.
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import torch

# HI2_B200_LIB points at another build of the same library (kernel experiments)
LIB_PATH = Path(os.environ.get("HI2_B200_LIB") or Path(__file__).resolve().parent / "libhi2_b200.so")

OK, ERR_ARG, ERR_LAUNCH, ERR_NOT_PD, ERR_TIMEOUT, ERR_CODE_RANGE, ERR_WORKSPACE, ERR_DRIVER = range(8)
F32, F64, F16, BF16 = range(4)
DTYPES = {torch.float32: F32, torch.float64: F64, torch.float16: F16, torch.bfloat16: BF16}

_P, _I, _L, _Z, _F, _D = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_float, C.c_double

# name -> (restype, argtypes); mirrors include/hi2_b200.h line by line
SIGNATURES = {
    "hi2_abi_version": (_I, []),
    "hi2_last_error": (C.c_char_p, []),
    "hi2_launch_count": (C.c_longlong, []),
    "hi2_graph_launch_count": (C.c_longlong, []),
    "hi2_rotate_groups": (_I, [_P, _I, _P, _I, _P, _P, _L, _L, _P]),
    "hi2_pack_codes": (_I, [_P, _P, _L, _L, _I, _P, _P]),
    "hi2_assemble_piece": (_I, [_P, _L, _P, _P, _P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P]),
    "hi2_dequantize": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _I, _P, _I, _P, _P]),
    "hi2_ladder_grid": (_I, [_P, _P, _P, _I, _I, _L, _L, _I, _P, _P, _P, _P]),
    "hi2_fit_ladder": (_I, [_P, _L, _P, _P, _I, _I, _I, _L, _L, _I, _P, _P, _P]),
    "hi2_quantize_rows": (
        _I,
        [_P, _P, _P, _L, _P, _I, _L, _L, _I, _P, _P, _P, _P, _L, _P, _P, _P, _P],
    ),
    "hi2_fit_ladder_grouped": (_I, [_P, _L, _P, _P, _P, _I, _I, _I, _L, _L, _I, _P, _P, _P]),
    "hi2_quantize_rows_grouped": (
        _I,
        [_P, _P, _P, _L, _P, _P, _I, _L, _L, _I, _P, _P, _P, _P, _L, _P, _P, _P, _P],
    ),
    "hi2_gptq_block": (_I, [_P, _L, _L, _L, _I, _P, _P, _P, _P, _L, _P, _P, _P, _P, _P, _P]),
    "hi2_gptq_lazy_update": (_I, [_P, _L, _L, _L, _L, _P, _P, _P]),
    "hi2_gptq_round": (
        _I,
        [_P, _L, _L, _P, _P, _P, _P, _L, _P, _P, _P, _P, _P, _I, _P, _P, _P],
    ),
    "hi2_gptq_round_tc": (
        _I,
        [_P, _L, _L, _P, _P, _P, _P, _P, _L, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P],
    ),
    "hi2_gptq_lazy_update_tc": (_I, [_P, _L, _L, _L, _P, _P, _P, _P]),
    "hi2_split_tf32_transposed": (_I, [_P, _P, _P, _L, _L, _P]),
    "hi2_split_tf32": (_I, [_P, _P, _P, _L, _P]),
    "hi2_gemm_tf32x3": (_I, [_L, _L, _L, _P, _P, _L, _P, _P, _L, _P, _L, _I, _P, _P]),
    "hi2_ladder_sse": (_I, [_P, _P, _L, _P, _P, _P, _L, _L, _L, _I, _P, _P]),
    "hi2_refine_block": (_I, [_P, _I, _P, _P, _P, _P, _P, _L, _L, _L, _P, _P]),
    "hi2_refine_block_in_place": (_I, [_P, _I, _P, _P, _P, _P, _P, _L, _L, _L, _P, _P, _L, _P]),
    "hi2_gemm_f32": (_I, [_I, _I, _L, _L, _L, _F, _P, _L, _P, _L, _F, _P, _L, _P]),
    "hi2_hessian_workspace_bytes": (_Z, [_L, _L, _I]),
    "hi2_hessian_accumulate": (_I, [_P, _I, _L, _L, _P, _P, _Z, _P]),
    "hi2_hessian_status": (_I, [_P, _P]),
    "hi2_hessian_accumulate_noalloc": (_I, [_P, _I, _L, _L, _P, _P, _P]),
    "hi2_group_moments": (_I, [_P, _L, _P, _P]),
    "hi2_group_moments_update": (_I, [_P, _I, _L, _L, _P, _P]),
    "hi2_transform_sigma": (_I, [_P, _F, _P, _P, _L, _P, _P, _P]),
    "hi2_inverse_factor_workspace_bytes": (_Z, [_L]),
    "hi2_inverse_factor": (_I, [_P, _P, _L, _P, _P, _Z, _P, _P]),
    "hi2_allocate_solve": (_I, [_P, _P, _I, _L, _D, _P, _P, _P]),
    "hi2_allocate_bits": (_I, [_P, _P, _I, _L, _P, _I, _P, _P]),
}

_lock = threading.Lock()
_lib = None
_failed: str | None = None


def load():
    """The loaded library.  Raises ``RuntimeError`` when it is missing or lacks a symbol."""
    global _lib, _failed
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            _failed = f"{LIB_PATH} not found: build it with `python -m hi2_b200.build`"
            raise RuntimeError(_failed)
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as e:
                _failed = f"{LIB_PATH} does not export {name}"
                raise RuntimeError(_failed) from e
            fn.restype, fn.argtypes = res, args
        _lib = lib
        return lib


def failure() -> str | None:
    return _failed


def launch_count() -> int:
    return int(load().hi2_launch_count())


def graph_launch_count() -> int:
    return int(load().hi2_graph_launch_count())


def last_error() -> str:
    return load().hi2_last_error().decode(errors="replace")


def check(rc: int, what: str) -> None:
    if rc == OK:
        return
    msg = f"{what}: {last_error()} (status {rc})"
    if rc == ERR_ARG:
        raise ValueError(msg)
    raise RuntimeError(msg)


class StreamArg:
    """A stream handle that remembers its device: ``call`` makes that device current for the
    launch.  (ctypes passes ``_as_parameter_``.)"""

    __slots__ = ("_as_parameter_", "index")

    def __init__(self, handle: int, index: int):
        self._as_parameter_ = C.c_void_p(handle)
        self.index = index


def call(name: str, *args) -> None:
    """Invoke an ``int``-returning entry point and raise on a non-zero status.

    The entry points launch on the CUDA runtime's current device.  The reference's API names
    devices explicitly and drives several of them from one process (one thread each, sometimes
    without ``set_device``), so the device of the stream argument is made current around the call;
    a call whose tensors live on ``cuda:1`` never launches on ``cuda:0``."""
    fn = getattr(load(), name)
    for a in args:
        if isinstance(a, StreamArg):
            if a.index != torch.cuda.current_device():
                with torch.cuda.device(a.index):
                    check(fn(*args), name)
                return
            break
    check(fn(*args), name)


def ptr(t: torch.Tensor | None):
    """Device address of a tensor (``None`` -> null)."""
    if t is None:
        return None
    return C.c_void_p(t.data_ptr())


def stream(device=None) -> StreamArg:
    """The current CUDA stream of ``device`` (default: the current device), tagged with the
    device's index."""
    if _raw_stream is not None:  # the handle without building a Stream object: a few microseconds per launch
        dev = torch.device(device) if device is not None else None
        index = dev.index if dev is not None and dev.index is not None else torch.cuda.current_device()
        return StreamArg(_raw_stream(index), index)
    st = torch.cuda.current_stream(device)
    return StreamArg(st.cuda_stream, st.device.index)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def upload(t: torch.Tensor, dev: torch.device, dtype: torch.dtype | None = None) -> torch.Tensor:
    """``t`` on ``dev`` as a contiguous tensor of ``dtype``.  A host tensor goes through pinned
    memory with a non-blocking copy: a plain ``.to(device)`` of pageable memory makes the host wait
    for everything already queued on the stream, which stalls a pipeline for a few bytes of flags."""
    dtype = dtype or t.dtype
    if t.is_cuda:
        return t.to(dev, dtype).contiguous()
    return t.to(dtype).contiguous().pin_memory().to(dev, non_blocking=True)


def need_cuda(*tensors: torch.Tensor) -> torch.device:
    """All tensors on one CUDA device; this package has no CPU path."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "hi2_b200 runs on CUDA devices only (got a tensor on " f"{t.device}); there is no CPU path"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def host_floats(values):
    arr = (C.c_float * len(values))(*[float(v) for v in values])
    return arr


def host_i64(values):
    return (C.c_int64 * len(values))(*[int(v) for v in values])
