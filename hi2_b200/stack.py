"""Stacked layout of routed-expert tensors (the arrays of hi2/stack.py:55-144 and its naming rules
:147-195), assembled where the packed buffers are: on the device, right after the encode.

The per-expert layout stores every expert projection as its own packed tensor.  The stacked layout
stores the experts of one layer and projection group (``gate_up``, ``down``; ``w13``, ``w2`` in
Mixtral's naming) as ONE flat container: the row buffers of all (expert, part) pieces one after the
other with the offsets rebased, ``had [E, K/16]`` and ``col_scale [E, K]`` with one row per expert
(the parts of a group share their transform), and ``part_off [E * P + 1]`` with the first row of
every piece.  Only the storage changes: :func:`split_stack` gives the pieces back byte for byte.

What differs from the reference: a stack is built with a handful of tensor operations over all
pieces at once, each array where its pieces live (the big buffers in HBM, the offsets on the host,
as the encode leaves them), and what must be looked at on the host (the two buffer totals for the
int32 check, whether device-resident transforms of an expert's parts agree) is read back together,
so that stacking the 64 experts of a layer costs no synchronisation per expert; the inverse likewise
reads its cut points back once.  Reading stacked checkpoints back from disk,
re-stacking existing checkpoints and their statistics stay with the reference.
"""

from __future__ import annotations

import torch

from .format import FIELDS, HI2Tensor
from .moe import expert_parts

LAYOUTS = ("per-expert", "stacked")
# group -> its parts in row order
GROUPS = {"gate_up": ("gate_proj", "up_proj"), "down": ("down_proj",), "w13": ("w1", "w3"), "w2": ("w2",)}
PART_GROUP = {part: (group, i) for group, parts in GROUPS.items() for i, part in enumerate(parts)}
MARK = "part_off"  # the array only a stack has
INT32_MAX = 2**31 - 1


class StackError(ValueError):
    """The group cannot be stored as a stack (the caller keeps it per expert)."""


def _check(experts) -> list:
    """Raises on what the host can see; returns, per expert and later part, a 0-dim tensor that is
    non-zero where a device-resident transform differs from the first part's (read back with the
    buffer totals)."""
    if not experts or not experts[0]:
        raise StackError("empty group")
    nparts, k = len(experts[0]), experts[0][0].shape[1]
    scaled = experts[0][0].col_scale is not None
    differs = []
    for e, parts in enumerate(experts):
        if len(parts) != nparts:
            raise StackError(f"expert {e} has {len(parts)} parts, expected {nparts}")
        for p in parts:
            if p.shape[1] != k:
                raise StackError(f"expert {e}: K={p.shape[1]}, expected {k}")
            if (p.col_scale is not None) != scaled:
                raise StackError("smoothing on for some experts only")
        for p in parts[1:]:  # the parts of a group read one input: one transform
            for name, a, b in (("rotation flags", p.had, parts[0].had), ("smoothing", p.col_scale, parts[0].col_scale)):
                if a is None:
                    continue
                if a.shape != b.shape:
                    raise StackError(f"expert {e}: parts have different {name}")
                if a.is_cuda or b.is_cuda:
                    differs.append((e, name, (a.to(b.device) != b).any()))
                elif not torch.equal(a, b):
                    raise StackError(f"expert {e}: parts have different {name}")
    return differs


def build_stack(experts: list[list[HI2Tensor]]) -> dict[str, torch.Tensor]:
    """``experts[e][p]`` (every part of every expert of one group) -> the arrays of the stack, keyed
    by field name without the ``hi2_`` prefix, each on the device its pieces are on.  Raises
    :class:`StackError` where the reference does: differing K or part count, a transform that differs
    between the parts of an expert, smoothing for some experts only, offsets that do not start at 0,
    a buffer beyond int32."""
    differs = _check(experts)
    pieces = [p for parts in experts for p in parts]
    rows = [p.shape[0] for p in pieces]

    def joined(field, flat=False):  # every array is put together where its first piece lives
        parts = [getattr(p, field) for p in pieces]
        return torch.cat([(t.reshape(-1) if flat else t).to(parts[0].device) for t in parts])

    out: dict[str, torch.Tensor] = {}
    checks = []
    for buf, off in (("codes", "code_off"), ("blk_params", "param_off")):
        where = getattr(pieces[0], off).device  # the host, for tensors that come out of assemble
        offs = [getattr(p, off).to(where, torch.int64) for p in pieces]
        ends = torch.stack([o[-1] for o in offs])
        first = torch.stack([o[0] for o in offs])
        base = torch.cumsum(ends, 0) - ends  # where each piece starts in the concatenated buffer
        shifted = torch.cat([o[:-1] for o in offs]) + torch.repeat_interleave(
            base, torch.tensor(rows, device=where), output_size=sum(rows))
        out[buf] = joined(buf, flat=True)
        out[off] = torch.cat([shifted, ends.sum().reshape(1)])
        checks += [ends.sum().cpu(), first.abs().max().cpu()]
    flags = [d.to("cpu", torch.int64) for _, _, d in differs]
    totals = torch.stack(checks + flags).tolist()  # read back together
    for (e, name, _), bad in zip(differs, totals[len(checks):]):
        if bad:
            raise StackError(f"expert {e}: parts have different {name}")
    for (buf, off), total, start in zip((("codes", "code_off"), ("blk_params", "param_off")), totals[0::2], totals[1::2]):
        if start != 0:
            raise StackError(f"{off} does not start at 0")
        if total > INT32_MAX:
            raise StackError(f"{off} total {total} exceeds int32")
        out[off] = out[off].to(torch.int32)
    for f in ("row_consts", "row_nbits", "row_block"):
        out[f] = joined(f)
    out[MARK] = torch.cumsum(torch.tensor([0, *rows], dtype=torch.int64), 0).to(torch.int32)
    out["had"] = torch.stack([parts[0].had.reshape(-1) for parts in experts])
    if experts[0][0].col_scale is not None:
        out["col_scale"] = torch.stack([parts[0].col_scale.reshape(-1) for parts in experts])
    return out


def stack_dims(d: dict[str, torch.Tensor], nparts: int) -> tuple[int, int]:
    """``(experts, K)`` of a stack, checked against ``part_off``."""
    e = d["had"].shape[0]
    if d[MARK].numel() != e * nparts + 1:
        raise ValueError(f"part_off has {d[MARK].numel()} entries, expected {e * nparts + 1}")
    return e, d["had"].shape[1] * 16


def split_stack(d: dict[str, torch.Tensor], nparts: int) -> list[list[HI2Tensor]]:
    """The pieces of a stack as fresh tensors, byte-identical to what was stacked."""
    n_exp, k = stack_dims(d, nparts)
    po = d[MARK].to("cpu", torch.int64)
    co, bo = d["code_off"].to(torch.int64), d["param_off"].to(torch.int64)
    at = po.to(co.device)
    cuts = torch.stack([co[at], bo[at]]).tolist()  # first code word and first block of every piece: one read-back
    po = po.tolist()
    out = []
    for e in range(n_exp):
        parts = []
        for p in range(nparts):
            i = e * nparts + p
            r0, r1 = po[i], po[i + 1]
            c0, c1, b0, b1 = cuts[0][i], cuts[0][i + 1], cuts[1][i], cuts[1][i + 1]
            parts.append(HI2Tensor(
                codes=d["codes"][c0:c1].clone(),
                code_off=(co[r0 : r1 + 1] - c0).to(d["code_off"].dtype),
                blk_params=d["blk_params"][2 * b0 : 2 * b1].clone(),
                param_off=(bo[r0 : r1 + 1] - b0).to(d["param_off"].dtype),
                row_consts=d["row_consts"][r0:r1].clone(),
                row_nbits=d["row_nbits"][r0:r1].clone(),
                row_block=d["row_block"][r0:r1].clone(),
                had=d["had"][e].clone(),
                shape=(r1 - r0, k),
                col_scale=d["col_scale"][e].clone() if "col_scale" in d else None,
            ))
        out.append(parts)
    return out


# ---- names ----------------------------------------------------------------------------------------
def member_base(pre: str, e: int, part: str) -> str:
    return f"{pre}.{e}.{part}"


def hi2_bases(names) -> tuple[list[str], list[str]]:
    """``(single, stacked)`` base names among the tensor names of a checkpoint: a stack is known by
    its ``part_off`` array, everything else with codes is a single tensor."""
    names = set(names)
    mark, codes = f".hi2_{MARK}", ".hi2_codes"
    stacked = sorted(n[: -len(mark)] for n in names if n.endswith(mark))
    single = sorted(set(n[: -len(codes)] for n in names if n.endswith(codes)) - set(stacked))
    return single, stacked


def stack_groups(single: list[str]) -> dict[str, list[list[str]]]:
    """``{stack base: members[e][p]}`` for the per-expert bases that form complete stacks: every part
    of the group present for every expert 0 .. E-1 (hi2/stack.py:168-186)."""
    seen: dict[tuple[str, str], dict[int, dict[str, str]]] = {}
    for base in single:
        ep = expert_parts(base)
        if ep is None or ep[2] not in PART_GROUP:
            continue
        pre, e, part = ep
        seen.setdefault((pre, PART_GROUP[part][0]), {}).setdefault(e, {})[part] = base
    out = {}
    for (pre, group), by_expert in seen.items():
        parts = GROUPS[group]
        complete = sorted(by_expert) == list(range(len(by_expert))) and all(
            set(found) == set(parts) for found in by_expert.values())
        if complete:
            out[f"{pre}.{group}"] = [[by_expert[e][p] for p in parts] for e in range(len(by_expert))]
    return out


def field_names(base: str, with_scale: bool, stacked: bool) -> list[str]:
    names = [f"{base}.hi2_{f}" for f in FIELDS]
    if with_scale:
        names.append(f"{base}.hi2_col_scale")
    if stacked:
        names.append(f"{base}.hi2_{MARK}")
    return names


def to_fields(t: HI2Tensor) -> dict[str, torch.Tensor]:
    d = {f: getattr(t, f) for f in FIELDS}
    if t.col_scale is not None:
        d["col_scale"] = t.col_scale
    return d


def from_fields(d: dict[str, torch.Tensor]) -> HI2Tensor:
    return HI2Tensor(**{f: d[f] for f in FIELDS}, shape=(d["row_nbits"].numel(), d["had"].numel() * 16),
                     col_scale=d.get("col_scale"))


def stack_packed(packed: dict[str, HI2Tensor]) -> tuple[dict[str, dict], dict[str, HI2Tensor]]:
    """Split the packed tensors of a shard (``{'<base>.weight': HI2Tensor}``) into ``(stacks, rest)``:
    ``stacks[stack base] = arrays`` for every expert group that is complete in the shard and can be
    stacked, ``rest`` everything else (groups that raise :class:`StackError` stay per expert)."""
    by_base = {name.removesuffix(".weight"): name for name in packed}
    stacks, used = {}, set()
    for stack, members in stack_groups(sorted(by_base)).items():
        try:
            stacks[stack] = build_stack([[packed[by_base[b]] for b in parts] for parts in members])
        except StackError:
            continue
        used.update(by_base[b] for parts in members for b in parts)
    return stacks, {n: t for n, t in packed.items() if n not in used}


__all__ = ["LAYOUTS", "GROUPS", "PART_GROUP", "MARK", "StackError", "build_stack", "split_stack", "stack_dims",
           "member_base", "hi2_bases", "stack_groups", "field_names", "to_fields", "from_fields", "stack_packed"]
