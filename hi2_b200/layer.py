"""One decoder layer through the whole encode path on one GPU: the call a user of this package
makes when the calibration activations of the layer's Linears are at hand.

    stats  = accumulate(inputs)                      second moments (tcgen05) + group moments
    tables = tabulate(weights, stats, cfg)           rotation + per-row error tables
    alloc  = allocate_global(tables, target_bpw)     (hi2_b200.allocate; all tables of the model)
    packed = encode(weights, stats, tables, alloc)   basis change, factor, GPTQ, packing

It is the order of hi2's pipeline (tabulate -> allocate -> encode, hi2/pipeline.py:1087-1252) with
the per-tensor stages of hi2/calibrate.py; Linears that read the same tensor (q/k/v, gate/up)
share one set of statistics, one smoothing vector and one factor, as in hi2/layerwise.py:140-154.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .calibrate import Config, EncodeRequest, TensorTable, build_table, build_tables_grouped, encode_many, smoothing_scale
from .format import GROUP, HI2Tensor
from .hessian import HessianStats
from .stats import ColumnStats


@dataclass
class SharedInput:
    """Calibration statistics of one distinct Linear input of width ``k``."""

    name: str
    k: int
    hessian: HessianStats
    moments: ColumnStats | None = None
    transform: tuple | None = None  # (fp16 smoothing vector or None, uint8 flags)


@dataclass
class LayerPlan:
    """Which weight reads which input: ``{"q": "attn_in", ...}``."""

    reads: dict = field(default_factory=dict)


def accumulate(inputs: dict, device, into: dict | None = None, defer_check: bool = False,
               storage: dict | None = None) -> dict:
    """``{input name: activations [tokens, k]}`` -> ``{input name: SharedInput}`` with the second
    moment summed (``into`` continues earlier sums: more tokens, or another rank's shard).  With
    ``defer_check`` the launches are not waited for; :func:`encode` settles their status.
    ``storage`` (optional) gives the ``[k, k]`` tensor a new input's sum is kept in."""
    out = into if into is not None else {}
    for name, x in inputs.items():
        k = x.shape[-1]
        if name not in out:
            where = None if storage is None else storage.get(name)
            out[name] = SharedInput(name, k, HessianStats(k, device, out=where))
        out[name].hessian.update(x, defer_check=defer_check)
    return out


def finish_statistics(shared: dict, cfg: Config, only: str | None = None) -> None:
    """Group moments, smoothing vector and rotation flags of every input, or of input ``only``
    (after all tokens, and after any cross-rank reduction of the second moments)."""
    for s in shared.values():
        if only is not None and s.name != only:
            continue
        s.moments = ColumnStats.from_second_moment(s.hessian.S, s.hessian.n)
        flags = torch.ones(s.k // GROUP, dtype=torch.uint8) if cfg.rotation == "on" else torch.zeros(
            s.k // GROUP, dtype=torch.uint8)
        s.transform = (smoothing_scale(s.moments, cfg.smooth), flags)


_side_streams: dict = {}


def _side_stream(device, i: int) -> torch.cuda.Stream:
    """Side streams are made once per device and reused: the caching allocator keeps a pool per
    stream, so a fresh stream every step would strand the factorisation scratch of the last one."""
    key = (torch.device(device).index, i)
    if key not in _side_streams:
        # high priority: the factorisation is a long chain of small kernels beside table kernels
        # that fill every SM, and a chain link should not queue behind a full grid
        _side_streams[key] = torch.cuda.Stream(device, priority=-1)
    return _side_streams[key]


def start_factors(shared: dict, cfg: Config, device, only: str | None = None, into: dict | None = None,
                  release_scratch: bool = False) -> dict:
    """Basis change and inverse factor of every input (or of input ``only``), each on a stream of
    its own, started now so they run beside the tables (which do not need them).  Pass the result
    to :func:`encode`.  ``release_scratch`` frees each factorisation's input and scratch as soon
    as it is enqueued (a model's worth of factors in flight would otherwise hold five times the
    bytes of the factors themselves); ``Hs`` is then not kept either, so not with refinement."""
    from .calibrate import factor_for

    main = torch.cuda.current_stream(device)
    out = into if into is not None else {}
    for i, s in enumerate(shared.values()):
        if only is not None and s.name != only:
            continue
        side = _side_stream(device, i % 8)  # a layer of experts has hundreds of inputs: eight chains at a time
        side.wait_stream(main)
        with torch.cuda.stream(side):
            d, job, hs = factor_for(s.hessian.S, s.hessian.n, s.transform[0], s.transform[1], cfg)
            if release_scratch:
                job.release_scratch()
                hs = None
            out[s.name] = (d, job, hs)
    return out


def tabulate(weights: dict, plan: LayerPlan, shared: dict, cfg: Config, only: str | None = None,
             into: dict | None = None, grouped: bool = False) -> dict:
    """Error tables of every weight ``{name: [R, K] tensor}`` (or of those reading input ``only``).
    ``grouped`` tabulates the weights of one shape together, a candidate at a time for all of them
    (:func:`hi2_b200.calibrate.build_tables_grouped`): what a layer of experts wants, whose hundreds
    of small tables are otherwise bound by the host's launch rate."""
    tables = into if into is not None else {}
    names = [n for n in weights if only is None or plan.reads[n] == only]
    if not grouped:
        for name in names:
            s = shared[plan.reads[name]]
            tables[name] = build_table(name, weights[name], s.moments, cfg, transform=s.transform)
        return tables
    by_shape: dict = {}
    for name in names:
        by_shape.setdefault((tuple(weights[name].shape), weights[name].dtype), []).append(name)
    for group in by_shape.values():
        items = [(n, weights[n], shared[plan.reads[n]].moments, shared[plan.reads[n]].transform, None) for n in group]
        for n, t in zip(group, build_tables_grouped(items, cfg)):
            tables[n] = t
    return {n: tables[n] for n in names} if into is None else tables


def encode(weights: dict, plan: LayerPlan, shared: dict, tables: dict, picks: dict, cfg: Config,
           to_host: bool = True, factors: dict | None = None, timing: list | None = None) -> dict:
    """Packed ``HI2Tensor`` of every weight for the allocator's ``picks``."""
    reqs, names = [], []
    for s in shared.values():
        s.hessian.check()
    for name, w in weights.items():
        s = shared[plan.reads[name]]
        reqs.append(EncodeRequest(w, s.moments, tables[name], picks[name], sigma=s.hessian.S,
                                  sigma_id=s.name, sigma_n=s.hessian.n))
        names.append(name)
    out = encode_many(reqs, cfg, to_host=to_host, factors=factors, timing=timing)
    return dict(zip(names, out))


def llama_plan() -> LayerPlan:
    """The seven matrices of a Llama-style decoder layer and the four tensors they read."""
    return LayerPlan({"q": "attn_in", "k": "attn_in", "v": "attn_in", "o": "attn_out",
                      "gate": "mlp_in", "up": "mlp_in", "down": "mlp_mid"})


def llama_shapes(hidden: int = 4096, ffn: int = 11008, kv_rows: int | None = None) -> tuple[dict, dict]:
    """``({weight: (rows, k)}, {input: k})`` of one decoder layer; ``kv_rows`` is the height of the
    k and v projections under grouped-query attention (default: ``hidden``)."""
    kv = hidden if kv_rows is None else kv_rows
    w = {"q": (hidden, hidden), "k": (kv, hidden), "v": (kv, hidden), "o": (hidden, hidden),
         "gate": (ffn, hidden), "up": (ffn, hidden), "down": (hidden, ffn)}
    x = {"attn_in": hidden, "attn_out": hidden, "mlp_in": hidden, "mlp_mid": ffn}
    return w, x


def keep_int8_for_most_sensitive(tables: list, fraction: float = 0.01) -> None:
    """Leave the INT8 candidates open only to the ``fraction`` of ALL rows whose best INT4 cost is
    largest, and close them for the rest, in place.  A closed INT8 entry is given the error of the
    row's best INT4 ladder: with equal error and more bits it can never be the allocator's argmin,
    while every number stays finite (an infinite entry would break the allocator's upper multiplier,
    hi2/allocate.py:233-240, in the reference as much as here).

    The reference has INT8 as a candidate for every row (hi2/calibrate.py:30-31, chosen by the
    allocator) or forced for whole tensors (hi2/allocate.py:62-76); "INT8 for the 1 % most
    sensitive rows" is the harness rule between the two: the allocator may spend 8 bits only where
    4 bits hurt most.  Cost is what the allocator minimises, ``sse / energy`` of the table
    (hi2/allocate.py:79-85).  The threshold is one quantile over the rows of all tables."""
    costs, best4 = [], []
    for t in tables:
        four = [i for i, (nb, _) in enumerate(t.candidates) if nb == 4]
        eight = [i for i, (nb, _) in enumerate(t.candidates) if nb == 8]
        if not four or not eight:
            best4.append(None)
            continue
        e = t.energy if isinstance(t.energy, torch.Tensor) else torch.tensor(float(t.energy), device=t.sse.device)
        floor4 = t.sse[four].min(0).values
        c = floor4 / e.to(t.sse.device, t.sse.dtype).clamp_min(1e-30)
        best4.append((c, eight, floor4))
        costs.append(c)
    if not costs:
        return
    allc = torch.cat(costs)
    keep = max(1, int(round(fraction * allc.numel())))
    threshold = torch.topk(allc, keep).values[-1]
    for t, item in zip(tables, best4):
        if item is None:
            continue
        c, eight, floor4 = item
        closed = c < threshold
        for i in eight:  # same error as the row's best INT4 ladder for more bits: never the argmin
            t.sse[i] = torch.where(closed, floor4, t.sse[i])


__all__ = ["SharedInput", "LayerPlan", "accumulate", "finish_statistics", "start_factors", "tabulate", "encode",
           "llama_plan", "llama_shapes", "keep_int8_for_most_sensitive", "Config", "TensorTable", "HI2Tensor"]
