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
        """``E[x_j^2]`` per column of ``x * inv_scale``, in the rotated basis where flagged."""
        s = self.S / max(self.n, 1)
        if inv_scale is not None:
            inv = inv_scale.to(s.device, s.dtype).reshape(-1, GROUP)
            s = s * inv[:, :, None] * inv[:, None, :]
        plain = torch.diagonal(s, dim1=1, dim2=2)
        if flags is None:
            return plain.reshape(-1).float()
        h = hadamard16(torch.float64, s.device)
        rot = ((h @ s) * h).sum(-1)  # diag(h s h) per group, h symmetric
        f = flags.to(s.device).bool().reshape(-1, 1)
        return torch.where(f, rot, plain).reshape(-1).float()

    def state(self) -> dict:
        return {"S": self.S.cpu(), "n": self.n, "k": self.k}

    @classmethod
    def from_state(cls, st: dict, device="cuda") -> "ColumnStats":
        c = cls(st["k"], device)
        c.S = st["S"].to(device)
        c.n = st["n"]
        return c
