"""Mixture-of-experts statistics on the device (hi2/moe.py:31-56, 152-156, 188-207;
hi2/layerwise.py:231-257).

The encode path treats every expert projection as its own matrix: its second moment sums only the
tokens routed to it, gate and up of one expert share that sum, and an expert that saw too few
tokens borrows the pooled sum of its layer for the missing ones.  This module holds that logic for
accumulators that live in HBM (``HessianStats`` / ``ColumnStats``), and the per-expert view of fused
3-D expert parameters (hi2/moe.py:53-121) that lets the calibration hooks see, expert by expert, the
tokens routed there.
"""

from __future__ import annotations

import re

import torch
from torch import nn

from .hessian import HessianStats
from .stats import ColumnStats

_EXPERT = re.compile(r"^(.*?\bexperts)\.(\d+)\.([^.]+)(?:\.weight)?$")
# projections of one expert that always see the same input (gate/up; Mixtral w1/w3)
_SAME_INPUT = {"up_proj": "gate_proj", "w3": "w1"}


def expert_parts(name: str):
    """``(group prefix, expert index, projection)`` of ``...experts.<E>.<proj>[.weight]``, else None."""
    m = _EXPERT.match(name)
    return None if m is None else (m.group(1), int(m.group(2)), m.group(3))


def group_key(name: str) -> str:
    """The name with the expert index replaced by ``*``: one key per layer and projection."""
    p = expert_parts(name)
    return name if p is None else f"{p[0]}.*.{p[2]}"


def sibling_leader(name: str):
    """For an expert ``up_proj`` (``w3``) the ``gate_proj`` (``w1``) whose input it shares."""
    p = expert_parts(name)
    if p is None or p[2] not in _SAME_INPUT:
        return None
    return f"{p[0]}.{p[1]}.{_SAME_INPUT[p[2]]}"


def blend(own_sum, own_n: int, avg_sum, avg_n: int, need: int):
    """``own + (need - n) * avg / avg_n`` and the new token count ``need``."""
    fill = (need - own_n) / max(avg_n, 1)
    return own_sum + fill * avg_sum.to(own_sum.device), need


def accumulate_routed(x: torch.Tensor, top_k_index: torch.Tensor, hess: list, stats: list | None = None):
    """Add to expert ``e``'s accumulators the tokens of ``x [T, K]`` whose ``top_k_index [T, k]``
    names ``e`` (each token once per expert, as the expert's Linear hook sees it)."""
    x = x.reshape(-1, x.shape[-1])
    idx = top_k_index.reshape(x.shape[0], -1)
    for e, h in enumerate(hess):
        rows = (idx == e).any(1).nonzero().squeeze(1)
        if rows.numel() == 0:
            continue
        xe = x.index_select(0, rows)
        if h is not None:
            h.update(xe)
        if stats is not None and stats[e] is not None:
            stats[e].update(xe)


def top_up(stats: dict, hess: dict | None, k_of: dict, min_tokens: float, all_reduce=None):
    """Top the leaders of every expert group up to ``min_tokens x widest input`` tokens with the
    group's pooled sums; returns the set of leaders that borrowed (hi2/layerwise.py:231-257).

    ``all_reduce`` (optional, ``tensor -> None`` in place): when the experts of a group are spread
    over several ranks each rank passes its own experts and the pooled sums and token totals are
    summed over the ranks through it before anybody borrows."""
    borrowed: set[str] = set()
    if min_tokens <= 0:
        return borrowed
    width: dict[tuple, int] = {}
    for n, k in k_of.items():
        p = expert_parts(n)
        if p is not None:
            width[p[:2]] = max(width.get(p[:2], 0), k)
    groups: dict[str, list[str]] = {}
    for ld in stats:
        if expert_parts(ld) is not None:
            groups.setdefault(group_key(ld), []).append(ld)
    for key in sorted(groups):  # the same order on every rank
        lds = groups[key]
        tot_n = sum(stats[ld].n for ld in lds)
        tot_s = sum(stats[ld].S for ld in lds)
        tot_h = sum(hess[ld].S for ld in lds) if hess else None
        if all_reduce is not None:
            count = torch.tensor([tot_n], dtype=torch.int64, device=tot_s.device)
            all_reduce(count)
            tot_n = int(count.item())
            tot_s = tot_s.clone()
            all_reduce(tot_s)
            if tot_h is not None:
                tot_h = tot_h.clone()
                all_reduce(tot_h)
        for ld in lds:
            need = int(min_tokens * width[expert_parts(ld)[:2]])
            if stats[ld].n >= need or tot_n == 0:
                continue
            st = stats[ld]
            st.S, st.n = blend(st.S, st.n, tot_s, tot_n, need)
            if hess:
                h = hess[ld]
                h.S, h.n = blend(h.S, h.n, tot_h, tot_n, need)
            borrowed.add(ld)
    return borrowed


def coverage(counts: dict, fallback) -> dict:
    """Report per layer and projection group (hi2/moe.py:159-182): how many experts, the least, median
    and most tokens an expert received, and the indices of the experts among ``fallback`` (the names
    that borrowed statistics).  Groups in natural order (``layers.2`` before ``layers.10``)."""
    import statistics

    groups: dict[str, list] = {}
    for name, tokens in counts.items():
        parts = expert_parts(name)
        if parts is not None:
            groups.setdefault(group_key(name), []).append((parts[1], tokens, name in fallback))

    def natural(key):
        return [int(piece) if piece.isdigit() else piece for piece in re.split(r"(\d+)", key)]

    report = {}
    for key in sorted(groups, key=natural):
        tokens = [n for _, n, _ in groups[key]]
        report[key] = {"experts": len(tokens), "min": min(tokens), "median": statistics.median(tokens), "max": max(tokens),
                       "fallback": sorted(e for e, _, borrowed in groups[key] if borrowed)}
    return report


# ---- per-expert views of fused experts -------------------------------------------------------------
def _linear_over(weight: torch.Tensor) -> nn.Linear:
    """An ``nn.Linear`` whose weight IS ``weight`` (a slice of the fused parameter; nothing is copied)."""
    lin = nn.Linear(weight.shape[1], weight.shape[0], bias=False, device="meta")
    lin.weight = nn.Parameter(weight, requires_grad=False)
    return lin


class _Expert(nn.Module):
    def __init__(self, gate, up, down):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = _linear_over(gate), _linear_over(up), _linear_over(down)


def is_fused_experts(mod: nn.Module) -> bool:
    """Experts stored as ``gate_up_proj [E, 2I, H]`` and ``down_proj [E, H, I]`` with an ``act_fn`` and no
    bias (the layout of recent ``transformers`` MoE blocks)."""
    gu, dn = getattr(mod, "gate_up_proj", None), getattr(mod, "down_proj", None)
    return (torch.is_tensor(gu) and torch.is_tensor(dn) and gu.dim() == 3 and dn.dim() == 3
            and hasattr(mod, "act_fn") and not getattr(mod, "has_bias", False))


class ExpertViews(nn.Module):
    """Drop-in for a fused-experts module: children ``0 .. E-1``, each with ``gate_proj`` / ``up_proj`` /
    ``down_proj`` Linears over slices of the fused parameters, and the fused module's call
    ``(hidden_states, top_k_index, top_k_weights)``.  The (token, slot) pairs are sorted by expert
    once (a stable sort keeps the token order inside an expert) and their counts read back once;
    every expert that received tokens then runs its three Linears on its own rows, gate and up on
    the SAME gathered tensor, so hooks on them see one shared input per expert."""

    def __init__(self, fused: nn.Module):
        super().__init__()
        gu, down = fused.gate_up_proj.data, fused.down_proj.data
        n_exp, twice, hidden = gu.shape
        inner = twice // 2
        if twice % 2 or tuple(down.shape) != (n_exp, hidden, inner):
            raise NotImplementedError(f"unsupported fused expert layout: gate_up {tuple(gu.shape)}, down {tuple(down.shape)}")
        for e in range(n_exp):
            self.add_module(str(e), _Expert(gu[e, :inner], gu[e, inner:], down[e]))
        self.n_experts = n_exp
        self.act_fn = fused.act_fn

    def __len__(self) -> int:
        return self.n_experts

    def __getitem__(self, e: int) -> nn.Module:
        return self.get_submodule(str(e))

    def forward(self, hidden_states, top_k_index, top_k_weights):
        x = hidden_states.reshape(-1, hidden_states.shape[-1])
        slots = top_k_index.shape[-1]
        chosen = top_k_index.reshape(-1)
        order = torch.argsort(chosen, stable=True)
        counts = (chosen[None, :] == torch.arange(self.n_experts, device=chosen.device)[:, None]).sum(1).tolist()
        share = top_k_weights.reshape(-1)
        out = torch.zeros_like(x)
        start = 0
        for e, n in enumerate(counts):
            pairs = order[start : start + n]
            start += n
            if n == 0:
                continue
            tokens = pairs // slots
            mine = x.index_select(0, tokens)
            ex = self[e]
            y = ex.down_proj(self.act_fn(ex.gate_proj(mine)) * ex.up_proj(mine))
            out.index_add_(0, tokens, (y * share[pairs, None]).to(out.dtype))
        return out.reshape(hidden_states.shape)


def unfuse_experts(model: nn.Module) -> int:
    """Replace every fused-experts module of ``model`` by :class:`ExpertViews` in place (the weights
    stay where they are); returns how many were replaced."""
    names = [n for n, m in model.named_modules() if is_fused_experts(m)]
    for n in names:
        model.set_submodule(n, ExpertViews(model.get_submodule(n)))
    return len(names)


def expert_weights(tables: dict, share_floor: float = 0.05) -> dict:
    """Allocation multiplier of every expert tensor (hi2/moe.py:188-207): an expert's share of its
    group's calibration tokens relative to an even split, floored at ``share_floor``, divided by
    the number of experts in the group, so a group weighs as much as one dense tensor."""
    members: dict[str, list[tuple[str, int]]] = {}
    for name, table in tables.items():
        if expert_parts(name) is not None:
            members.setdefault(group_key(name), []).append((name, table.n_tokens))
    weights: dict[str, float] = {}
    for group in members.values():
        experts = len(group)
        even = sum(tokens for _, tokens in group) / experts
        for name, tokens in group:
            relative = tokens / even if even > 0 else 1.0
            weights[name] = max(relative, share_floor) / experts
    return weights


__all__ = ["expert_parts", "group_key", "sibling_leader", "blend", "accumulate_routed", "top_up",
           "expert_weights", "coverage", "is_fused_experts", "ExpertViews", "unfuse_experts", "HessianStats", "ColumnStats"]
