"""Per-group second moments on B200 (interface of hi2/stats.py:16-64).

hi2 keeps, next to the full second moment, the 16x16 diagonal blocks of it in fp64
(``ColumnStats``): enough for the exact diagonal in the rotated basis.  When the full second moment
is accumulated anyway they are read out of it (``from_second_moment``); ``update`` sums them from
activations directly for callers that keep no full second moment (data-free tables, nearest rounding).
"""

from __future__ import annotations

import torch

from . import _lib
from .format import GROUP, hadamard16


_basis: dict = {}


def _hadamard_on(dev: torch.device) -> torch.Tensor:
    """The fp64 rotation matrix on ``dev``, uploaded once per device: a fresh blocking copy per call
    would make the host wait for everything queued on the stream."""
    key = (dev.type, dev.index)
    if key not in _basis:
        _basis[key] = hadamard16(torch.float64, dev)
    return _basis[key]


class ColumnStats:
    def __init__(self, k: int, device="cuda"):
        if k % GROUP:
            raise ValueError(f"K={k} must be a multiple of {GROUP}")
        self.k = k
        self.S = torch.zeros(k // GROUP, GROUP, GROUP, dtype=torch.float64, device=device)
        self.n = 0

    @classmethod
    def from_second_moment(cls, s: torch.Tensor, n: int) -> "ColumnStats":
        """Blocks of an accumulated ``S [K, K]`` (fp32) covering ``n`` tokens."""
        out = cls(s.shape[0], s.device)
        out.add_second_moment(s, n)
        return out

    def add_second_moment(self, s: torch.Tensor, n: int) -> None:
        dev = _lib.need_cuda(s, self.S)
        if s.dtype != torch.float32 or not s.is_contiguous() or s.shape != (self.k, self.k):
            raise ValueError("second moment must be a contiguous fp32 [K, K] tensor")
        _lib.call("hi2_group_moments", _lib.ptr(s), self.k, _lib.ptr(self.S), _lib.stream(dev))
        self.n += n

    @torch.no_grad()
    def update(self, x: torch.Tensor) -> None:
        """Accumulate from activations ``x [..., K]`` (fp32 sums per 4096 tokens, fp64 total)."""
        dev = _lib.need_cuda(self.S)
        x = x.reshape(-1, self.k)
        if x.device != dev:
            x = x.to(dev)
        if x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            x = x.float()
        x = x.contiguous()
        _lib.call("hi2_group_moments_update", _lib.ptr(x), _lib.DTYPES[x.dtype], x.shape[0], self.k,
                  _lib.ptr(self.S), _lib.stream(dev))
        self.n += x.shape[0]

    def merge(self, other: "ColumnStats") -> None:
        self.S += other.S.to(self.S.device)
        self.n += other.n

    def diag(self, flags: torch.Tensor | None = None, inv_scale: torch.Tensor | None = None):
        """Mean square of every column of ``x * inv_scale`` after the flagged groups have been
        rotated: the diagonal of ``T_g M_g T_g^T`` per group, ``M_g`` the group's mean moment and
        ``T_g`` the rotation (or the identity).  fp64 throughout, returned as fp32 ``[K]``
        (hi2/stats.py:39-54)."""
        moment = self.S / max(self.n, 1)
        dev = moment.device
        if inv_scale is not None:
            # scale first (rows, then columns), then rotate: the order the reference rounds in
            v = inv_scale.to(dev, moment.dtype).reshape(-1, GROUP)
            moment = moment * v.unsqueeze(2) * v.unsqueeze(1)
        unrotated = moment.diagonal(dim1=-2, dim2=-1)
        if flags is None:
            return unrotated.flatten().float()
        basis = _hadamard_on(dev)
        # (T M T^T)_ii = sum_jk T_ij M_jk T_ik
        rotated = torch.einsum("ij,gjk,ik->gi", basis, moment, basis)
        chosen = torch.where(_lib.upload(flags, dev).reshape(-1, 1) != 0, rotated, unrotated)
        return chosen.flatten().float()

    def state(self) -> dict:
        return {"S": self.S.cpu(), "n": self.n, "k": self.k}

    @classmethod
    def from_state(cls, st: dict, device="cuda") -> "ColumnStats":
        c = cls(st["k"], device)
        c.S = st["S"].to(device)
        c.n = st["n"]
        return c
