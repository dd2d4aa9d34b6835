"""Calibration propagation on the device: one decoder layer at a time, statistics taken straight
from the layer's own activations (hi2/layerwise.py:103-199 capture and hooks, :202-264 merge,
:323-361 layer pass, :559-694 ``calibrate_layerwise``).

What differs from the reference's driver, none of which changes a statistic:

* the hidden states of all calibration sequences stay in HBM as one ``[sequences, tokens, hidden]``
  tensor between layers (the reference round-trips them through host memory unless they fit its
  "resident" rule), and a Linear's forward pre-hook hands its input to the tensor-core second moment
  (:class:`hi2_b200.hessian.HessianStats`) without a copy: activations never cross PCIe;
* the 16 x 16 group moments are read out of the finished second moment instead of being summed in
  a second pass over the activations;
* several GPUs are several processes (``torch.distributed``): every rank runs every layer on ITS
  sequences (round-robin, as hi2/layerwise.py:336), the partial second moments of a layer are summed
  onto the rank that owns the layer (``layer mod world``), and only the owner tabulates it.  The
  reference runs one thread per device and adds the partial sums on its primary device.

Linears that receive the very same tensor (q/k/v, gate/up) share one accumulator, decided as in the
reference by the address and shape of the input among the inputs of the running batch.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field

import torch
from torch import nn

from . import dist as hd
from .calibrate import Config, TensorTable, build_table, factor_for, shared_transform
from .hessian import HessianStats
from .moe import expert_parts, sibling_leader, top_up
from .stats import ColumnStats


class _Halt(Exception):
    """Raised by the stand-in for layer 0 once it has seen its input."""


class _Recorder(nn.Module):
    """Takes the place of the first decoder layer while the model embeds the calibration ids:
    keeps the hidden states and the keyword arguments every layer is called with, then stops
    the forward pass."""

    def __init__(self, first: nn.Module, store: torch.Tensor, slots: list):
        super().__init__()
        self.first, self.store, self.slots, self.kwargs = first, store, slots, None

    def __getattr__(self, name):  # the model may read attributes of the layer it thinks it calls
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.first, name)

    def forward(self, hidden_states, *args, **kwargs):
        lo = self.slots.pop(0)
        self.store[lo : lo + hidden_states.shape[0]] = hidden_states.detach()
        if self.kwargs is None:
            self.kwargs = kwargs
        raise _Halt


def find_layers(model: nn.Module):
    """``(dotted path, ModuleList)`` of the decoder layers: the longest ``nn.ModuleList`` whose
    name ends in ``layers`` (``model.layers`` for Llama-style models)."""
    best = None
    for name, mod in model.named_modules():
        if isinstance(mod, nn.ModuleList) and name.split(".")[-1] in ("layers", "h", "blocks"):
            if best is None or len(mod) > len(best[1]):
                best = (name, mod)
    if best is None:
        raise ValueError("no decoder layer list found in the model")
    return best


def capture_inputs(model: nn.Module, layers: nn.ModuleList, ids: torch.Tensor, device, batch: int = 8):
    """Hidden states entering layer 0 for every calibration sequence, as ONE tensor
    ``[sequences, tokens, hidden]`` on ``device``, and the keyword arguments of a layer call
    (position embeddings, mask, ...) as captured for a batch of one sequence."""
    n_seq, tokens = ids.shape
    emb = model.get_input_embeddings()
    dtype = emb.weight.dtype
    store = torch.empty(n_seq, tokens, emb.weight.shape[1], dtype=dtype, device=device)
    slots: list = []
    rec = _Recorder(layers[0], store, slots)
    layers[0] = rec
    try:
        with torch.no_grad():
            # one sequence first: the kwargs kept are those of a batch of one, which expand to any batch
            for lo in [0, *range(1, n_seq, batch)]:
                hi = 1 if lo == 0 else min(lo + batch, n_seq)
                slots.append(lo)
                try:
                    model(ids[lo:hi].to(device), use_cache=False)
                except _Halt:
                    pass
    finally:
        layers[0] = rec.first
    kwargs = {k: v for k, v in (rec.kwargs or {}).items() if k != "past_key_values"}
    kwargs["use_cache"] = False
    return store, kwargs


def expand_batch(kwargs: dict, n: int) -> dict:
    """The batch-of-one tensors of the captured kwargs broadcast to ``n`` sequences (every
    sequence is its own causal window of the same length)."""

    def widen(v):
        if torch.is_tensor(v) and v.dim() >= 2 and v.shape[0] == 1:
            return v.expand(n, *v.shape[1:])
        if isinstance(v, (tuple, list)):
            return type(v)(widen(x) for x in v)
        return v

    return {k: widen(v) for k, v in kwargs.items()}


def run_layer(layer: nn.Module, hidden: torch.Tensor, kwargs: dict, linears, k_of: dict, batch: int = 32,
              want_hessian: bool = True):
    """Forward all sequences of ``hidden [S, T, H]`` through ``layer`` IN PLACE (its output replaces
    its input), ``batch`` sequences at a time, while forward pre-hooks accumulate the statistics of
    the Linears named in ``linears``.  Returns ``(stats, hess, leader_of)``: with ``want_hessian``
    only ``hess`` is filled during the pass (the group moments are read out of it afterwards by
    :func:`finish_stats`), else ``stats`` is summed directly."""
    dev = hidden.device
    stats: dict[str, ColumnStats] = {}
    hess: dict[str, HessianStats] = {}
    leader_of: dict[str, str] = {}
    seen: dict[tuple, str] = {}
    alive: list = []

    def hook_for(key):
        def hook(_mod, args):
            x = args[0].detach()
            tag = (x.data_ptr(), tuple(x.shape))
            lead = leader_of.get(key)
            if lead is None:  # first time this Linear runs: does it share its input with an earlier one?
                lead = leader_of[key] = seen.get(tag, key)
                if lead == key:
                    if want_hessian:
                        hess[key] = HessianStats(k_of[key], dev)
                    else:
                        stats[key] = ColumnStats(k_of[key], dev)
            if tag not in seen:
                seen[tag] = lead
                alive.append(x)  # keeps the address from being reused within this batch
            if lead == key and x.numel():
                if want_hessian:
                    hess[key].update(x, defer_check=True)
                else:
                    stats[key].update(x)

        return hook

    handles = [mod.register_forward_pre_hook(hook_for(n)) for n, mod in layer.named_modules() if n in linears]
    try:
        with torch.no_grad():
            for lo in range(0, hidden.shape[0], batch):
                part = hidden[lo : lo + batch]
                out = layer(part, **expand_batch(kwargs, part.shape[0]))
                part.copy_(out[0] if isinstance(out, tuple) else out)
                seen.clear()
                alive.clear()
    finally:
        for h in handles:
            h.remove()
    return stats, hess, leader_of


def leaders(linears, leader_of: dict) -> dict:
    """Leader of every Linear, also of those that never ran here (an expert without tokens follows
    its structural sibling, hi2/layerwise.py:213-218)."""
    lead = dict(leader_of)
    for n in linears:
        if n not in lead:
            sib = sibling_leader(n)
            lead[n] = lead.get(sib, sib) if sib in linears else n
    return lead


def finish_stats(lead: dict, linears, k_of: dict, stats: dict, hess: dict, dev, want_hessian: bool,
                 unchecked: list | None = None) -> None:
    """Make sure every leader has both accumulators (empty ones for Linears that saw no token) and,
    with full second moments, read the group moments out of them.  The status words of the
    second-moment launches are read here (a wait for the device), or, when the caller passes a list
    as ``unchecked``, left to it: the accumulators are appended and the caller settles them all with
    one ``HessianStats.check_all`` later."""
    for ld in dict.fromkeys(lead[n] for n in linears):
        if want_hessian:
            h = hess.setdefault(ld, HessianStats(k_of[ld], dev))
            if unchecked is None:
                h.check()
            else:
                unchecked.append(h)
            stats[ld] = ColumnStats.from_second_moment(h.S, h.n) if h.n else ColumnStats(k_of[ld], dev)
        else:
            stats.setdefault(ld, ColumnStats(k_of[ld], dev))


@dataclass
class DeviceSink:
    """Where ``calibrate_layerwise`` leaves the statistics the encode stage needs, kept in HBM
    (the reference writes them under its work directory, hi2/layerwise.py:382-398):
    ``sigma[leader tensor name] = (sum x x^T, tokens)`` and ``leader[tensor name]``."""

    sigma: dict = field(default_factory=dict)
    stats: dict = field(default_factory=dict)
    leader: dict = field(default_factory=dict)
    groups: list = field(default_factory=list)
    factors: dict = field(default_factory=dict)  # leader -> (d, FactorJob, None), started while tabulating

    def hessians(self, lead, hess, linears):
        for ld, h in hess.items():
            self.sigma[linears[ld]] = (h.S, h.n)

    def group(self, leader_name, member_names, st):
        self.stats[leader_name] = st
        self.groups.append((leader_name, list(member_names)))
        for m in member_names:
            self.leader[m] = leader_name


_factor_streams: dict = {}


def _factor_stream(device, i: int) -> torch.cuda.Stream:
    """High-priority side streams for the factor chains, made once per device and reused."""
    key = (torch.device(device).index, i)
    if key not in _factor_streams:
        _factor_streams[key] = torch.cuda.Stream(device, priority=-1)
    return _factor_streams[key]


def _eligible(name: str, shape, include, exclude) -> bool:
    if len(shape) != 2 or shape[1] % 64:
        return False
    if include and not any(re.search(p, name) for p in include):
        return False
    return not (exclude and any(re.search(p, name) for p in exclude))


def calibrate_layerwise(model: nn.Module, ids: torch.Tensor, cfg: Config, ex=None, workdir=None, include=None,
                        exclude=None, limit_layers: int | None = None, log=print, resolve=None,
                        sink: DeviceSink | None = None, device=None, batch: int = 32, prefactor: bool = True) -> dict:
    """``{checkpoint tensor name: TensorTable}`` for every eligible Linear of every decoder layer
    (of the layers this rank owns when several ranks run), statistics left in ``sink``.

    ``model`` must live on ``device`` (every rank holds the whole model); ``ids [sequences, tokens]``
    are the calibration ids of ALL ranks, of which rank r takes sequences ``r, r + world, ...``.
    With ``prefactor`` (and GPTQ rounding without act-order) the basis change and the inverse factor
    of every shared input are started on side streams as soon as its transform is known, so that they
    run beside the tables; the encode stage finds them in ``sink.factors``."""
    del ex, workdir
    sink = sink if sink is not None else DeviceSink()
    device = torch.device(device) if device is not None else next(model.parameters()).device
    rank, world = hd.rank(), hd.world_size()
    path, layers = find_layers(model)
    prefix = path + "."
    mine = ids[rank::world]
    hidden, kwargs = capture_inputs(model, layers, mine, device)
    log(f"captured {hidden.shape[0]} calibration sequences of {tuple(hidden.shape[1:])}")
    want_h = cfg.rounding == "gptq" and not cfg.sequential
    tables: dict = {}
    unchecked: list = []  # status words are read once, after the last layer: the host never waits in between
    for li, layer in enumerate(layers):
        if limit_layers is not None and li >= limit_layers:
            break
        linears = {}
        for n, mod in layer.named_modules():
            full = f"{prefix}{li}.{n}.weight"
            if isinstance(mod, nn.Linear) and _eligible(full, mod.weight.shape, include, exclude):
                ckpt = resolve(full) if resolve else full
                if ckpt is None:
                    log(f"warning: {full} has no tensor in the checkpoint; skipped")
                    continue
                linears[n] = ckpt
        k_of = {n: layer.get_submodule(n).in_features for n in linears}
        stats, hess, leader_of = run_layer(layer, hidden, kwargs, linears, k_of, batch, want_h)
        lead = leaders(linears, leader_of)
        owner = hd.owner_of(li, world)
        if world > 1:  # partial sums of this rank's sequences -> the layer's owner
            for ld in dict.fromkeys(lead[n] for n in linears):
                acc = (hess if want_h else stats).get(ld)
                if acc is None:  # never ran on this rank: contribute zeros
                    acc = (HessianStats if want_h else ColumnStats)(k_of[ld], device)
                    (hess if want_h else stats)[ld] = acc
                if want_h:
                    acc.check()
                count = torch.tensor([acc.n], dtype=torch.int64, device=device)
                torch.distributed.all_reduce(count)
                torch.distributed.reduce(acc.S, dst=owner)
                acc.n = int(count.item())
            if rank != owner:
                continue
        finish_stats(lead, linears, k_of, stats, hess, device, want_h, unchecked)
        counts = {n: stats[lead[n]].n for n in linears}
        borrowed = top_up({linears[ld]: st for ld, st in stats.items()},
                          {linears[ld]: h for ld, h in hess.items()} if want_h else None,
                          {linears[n]: k_of[n] for n in linears}, cfg.expert_min_tokens)
        if want_h:
            sink.hessians(lead, hess, linears)
        members: dict[str, list[str]] = {}
        for n in linears:
            members.setdefault(lead[n], []).append(n)
        for ld, names in members.items():
            st = stats[ld] if stats[ld].n > 0 else None
            ws = [layer.get_submodule(n).weight.detach() for n in names]
            transform = shared_transform(ws, st, cfg)
            sink.group(linears[ld], [linears[n] for n in names], st)
            if prefactor and want_h and not cfg.act_order and ld in hess and hess[ld].n > 0:
                side = _factor_stream(device, len(sink.factors) % 4)
                side.wait_stream(torch.cuda.current_stream(device))
                with torch.cuda.stream(side):
                    d, job, _ = factor_for(hess[ld].S, hess[ld].n, transform[0], transform[1], cfg)
                    job.release_scratch()
                sink.factors[linears[ld]] = (d, job, None)
            for n, w in zip(names, ws):
                if st is None:
                    log(f"warning: {linears[n]} saw no calibration tokens; data-free weights")
                tables[linears[n]] = build_table(linears[n], w, st, cfg, None, transform, counts[n])
        if borrowed:
            log(f"  layer {li}: {len(borrowed)} expert inputs topped up with the layer average")
        log(f"layer {li}: {len(linears)} linears tabulated")
    HessianStats.check_all(unchecked)
    return tables


def encode_layerwise(model: nn.Module, tables: dict, picks: dict, sink: DeviceSink, cfg: Config,
                     to_host: bool = True, groups_per_call: int = 8) -> dict:
    """Packed tensors of every tabulated Linear (this rank's) for the allocator's ``picks``; Linears
    that share an input share one basis change and one factor (hi2/calibrate.py:297-424)."""
    from .calibrate import EncodeRequest, encode_many

    weights = {name + ("" if name.endswith(".weight") else ".weight"): p for name, p in model.named_parameters()}
    out: dict = {}
    for g0 in range(0, len(sink.groups), groups_per_call):
        reqs, names = [], []
        for leader_name, member_names in sink.groups[g0 : g0 + groups_per_call]:
            sigma = sink.sigma.get(leader_name)
            for m in member_names:
                if m not in tables:
                    continue
                reqs.append(EncodeRequest(weights[m].detach(), sink.stats[leader_name], tables[m], picks[m],
                                          sigma=None if sigma is None else sigma[0], sigma_id=leader_name,
                                          sigma_n=1 if sigma is None else sigma[1]))
                names.append(m)
        if reqs:
            out.update(zip(names, encode_many(reqs, cfg, to_host=to_host, factors=sink.factors or None)))
    return out


__all__ = ["find_layers", "capture_inputs", "expand_batch", "run_layer", "leaders", "finish_stats", "DeviceSink",
           "calibrate_layerwise", "encode_layerwise", "expert_parts"]
