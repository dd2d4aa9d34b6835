"""Benchmark of the PTQ encode path (Hessian + tables + allocation + GPTQ + pack).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config cfg3|cfg2|cfg1|...]

Default workload (``cfg3``, the configuration BASELINE.json's metric is quoted on): a whole
Llama-2-7B-shaped model, 32 decoder layers of seven bf16 matrices (hidden 4096, FFN 11008),
256 x 2048 synthetic calibration tokens per distinct input, 3.0 bpw, INT2/INT4 candidates.  One
step = the whole model through tabulate -> allocate -> encode.  Layer l is owned by rank
``l mod N`` (strong scaling: the model is fixed), the calibration tokens are sharded over the
ranks, partial second moments are summed onto the owner by one NCCL reduce-scatter per input and
group of N layers, the error tables are gathered once for the global allocation, and everything
else runs on the owner.  ``--config cfg2`` is one decoder layer per GPU at 128 x 2048 tokens and
2.5 bpw (weak scaling), ``cfg1`` the single 4096 x 4096 Linear the reference runs on CPU.

Prints ONE JSON line (rank 0).  ``value`` is rows of weight matrix encoded per second with all
inputs resident in HBM; ``e2e`` is the same through the public API from pinned host buffers with
the packed result copied back.  ``--impl reference`` times the CPU restatement of the reference
(oracle/) on the host cores on a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

CONFIGS = {
    # name: hidden, ffn, sequences, seq_len, activation spread, target bpw, weight dtype
    # BASELINE config 3, the one the metric is quoted on: a whole 7B-shaped model, 32 layers of the
    # config-2 shapes, 256 x 2048 calibration tokens per input, 3.0 bpw, layer l owned by rank l mod N
    "cfg3": dict(hidden=4096, ffn=11008, tokens=256 * 2048, spread=1.5, bpw=3.0, dtype="bf16", layers=32,
                 workload="llama2_7b_shape_32_layers_x_7_matrices_256x2048_tokens_3.0bpw"),
    # BASELINE config 4: Llama-3-70B shapes (GQA: k/v 1024 x 8192), 80 layers, 128 x 4096 tokens, INT8
    # candidates open to the 1 % most sensitive rows; 2.25 bpw is below the format's floor for these
    # shapes (INT2/B64 costs 2.25 bits before the per-row overhead), so the step records that
    # allocation as infeasible and encodes at 2.35 bpw.  80 layers hold 660 GB of second moments
    # and factors: they fit on 8 GPUs, one GPU takes --layers 8.
    "cfg4": dict(hidden=8192, ffn=28672, kv_rows=1024, tokens=128 * 4096, spread=1.5, bpw=2.35, bpw_infeasible=2.25,
                 int8_fraction=0.01, dtype="bf16", layers=80, layers_per_encode=2,
                 workload="llama3_70b_shape_80_layers_gqa_128x4096_tokens_2.35bpw_int8_top1pct"),
    # BASELINE config 5: OLMoE shapes, 16 layers of 64 experts (gate/up 1024 x 2048, down 2048 x 1024),
    # top-8 routing from a seeded random router with a per-expert bias (uneven token counts), per-expert
    # second moments over the routed tokens only, gate and up of an expert share theirs; expert e of
    # every layer is owned by rank e mod N
    "cfg5": dict(hidden=2048, expert_ffn=1024, experts=64, top_k=8, tokens=256 * 2048, spread=1.5, bpw=2.5, dtype="bf16",
                 moe_layers=16, router_bias=1.5, workload="olmoe_shape_16_layers_x_64_experts_top8_256x2048_tokens_2.5bpw"),
    "tiny_moe": dict(hidden=256, expert_ffn=128, experts=8, top_k=2, tokens=4096, spread=1.0, bpw=3.0, dtype="bf16",
                     moe_layers=2, router_bias=2.5, workload="tiny_moe_2_layers_x_8_experts_top2"),
    "cfg2": dict(hidden=4096, ffn=11008, tokens=128 * 2048, spread=1.5, bpw=2.5, dtype="bf16",
                 workload="llama_decoder_layer_7_matrices_4096x11008_128x2048_tokens_2.5bpw"),
    "cfg1": dict(hidden=4096, ffn=0, tokens=2048, spread=1.0, bpw=3.0, dtype="f16",
                 workload="single_linear_4096x4096_2048_tokens_3.0bpw"),
    # config 2 with 32768 tokens per input: small enough for an ncu capture, inputs still > L2
    "cfg2_32k": dict(hidden=4096, ffn=11008, tokens=32768, spread=1.5, bpw=2.5, dtype="bf16",
                     workload="llama_decoder_layer_7_matrices_4096x11008_32768_tokens_2.5bpw"),
    # small cases for the tests of this file (one layer; a four-layer model)
    "tiny": dict(hidden=512, ffn=1024, tokens=4096, spread=1.5, bpw=2.5, dtype="bf16",
                 workload="tiny_decoder_layer_512x1024_4096_tokens_2.5bpw"),
    "tiny_model": dict(hidden=512, ffn=1024, tokens=4096, spread=1.5, bpw=3.0, dtype="bf16", layers=4,
                       layers_per_encode=2, workload="tiny_model_4_layers_512x1024_4096_tokens_3.0bpw"),
    "tiny_gqa_int8": dict(hidden=512, ffn=1024, kv_rows=128, tokens=4096, spread=1.5, bpw=2.6, bpw_infeasible=2.25,
                          int8_fraction=0.01, dtype="bf16", layers=2, layers_per_encode=1,
                          workload="tiny_gqa_model_2_layers_int8_top1pct"),
}


def shapes_of(cfg):
    from hi2_b200.layer import LayerPlan, llama_plan, llama_shapes

    if cfg["ffn"] == 0:  # a single Linear (BASELINE config 1)
        return {"w": (cfg["hidden"], cfg["hidden"])}, {"x": cfg["hidden"]}, LayerPlan({"w": "x"})
    w, x = llama_shapes(cfg["hidden"], cfg["ffn"], cfg.get("kv_rows"))
    return w, x, llama_plan()


def candidates_of(cfg):
    from hi2_b200.calibrate import ALL_CANDIDATES, SELECTABLE

    return list(SELECTABLE if cfg.get("int8_fraction") else ALL_CANDIDATES)


def torch_dtype(name):
    return {"bf16": torch.bfloat16, "f16": torch.float16}[name]


def make_weights(cfg, shapes, layer, device):
    """Random-init weights N(0, 0.02); config 1 scales 0.1 % of the input columns by 20."""
    g = torch.Generator(device=device).manual_seed(1000 + layer)
    out = {}
    for name, (r, k) in shapes.items():
        w = torch.randn(r, k, generator=g, device=device) * 0.02
        if cfg["ffn"] == 0:
            cols = torch.randperm(k, generator=g, device=device)[: max(1, k // 1000)]
            w[:, cols] *= 20
        out[name] = w.to(torch_dtype(cfg["dtype"]))
    return out


def make_inputs(cfg, widths, layer, tokens, token0, device):
    """Synthetic activations: N(0,1) times a per-channel lognormal(0, spread) scale.  The channel
    scales depend on the layer only, the token noise on (layer, first token), so token shards of
    one layer are shards of one tensor."""
    out = {}
    for i, (name, k) in enumerate(widths.items()):
        gs = torch.Generator(device=device).manual_seed(77 + 13 * layer + i)
        scale = torch.exp(cfg["spread"] * torch.randn(1, k, generator=gs, device=device))
        gx = torch.Generator(device=device).manual_seed(5000 + 101 * layer + 7 * i + token0)
        x = torch.empty(tokens, k, dtype=torch_dtype(cfg["dtype"]), device=device)
        step = 16384
        for t0 in range(0, tokens, step):
            n = min(step, tokens - t0)
            x[t0 : t0 + n] = (torch.randn(n, k, generator=gx, device=device) * scale).to(x.dtype)
        out[name] = x
    return out


class Clocks:
    """Samples nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        for line in self.lines:
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])), mx.append(float(f[2])), power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------
# the B200 arm
# --------------------------------------------------------------------------------------------
class Job:
    """Resident workload of one rank: the weights of its own layer and its token shard of the
    calibration activations of every layer."""

    def __init__(self, cfg, rank, world, device):
        from hi2_b200 import dist as hd
        from hi2_b200.calibrate import ALL_CANDIDATES, Config

        self.cfg, self.rank, self.world, self.device = cfg, rank, world, device
        self.shapes, self.widths, self.plan = shapes_of(cfg)
        self.qcfg = Config(candidates=list(ALL_CANDIDATES))
        self.weights = make_weights(cfg, self.shapes, rank, device)
        lo, hi = hd.token_shard(cfg["tokens"], rank, world)
        self.inputs = [make_inputs(cfg, self.widths, layer, hi - lo, lo, device) for layer in range(world)]
        self.rows = sum(r for r, _ in self.shapes.values())
        self.host = None
        self.copy_stream = None
        self.stage_ms: dict = {}

    def input_order(self):
        """Widest input first (longest factorisation), then by the rows that read it, so the input
        that arrives last over PCIe has the least work hanging on it."""
        rows = {n: 0 for n in self.widths}
        for w, (r, _) in self.shapes.items():
            rows[self.plan.reads[w]] += r
        return sorted(self.widths, key=lambda n: (-self.widths[n], -rows[n]))

    # bytes one rank moves per step in the end-to-end measurement
    def h2d_bytes(self):
        n = sum(w.numel() * w.element_size() for w in self.weights.values())
        return n + sum(x.numel() * x.element_size() for layer in self.inputs for x in layer.values())

    def pin_host_copies(self):
        self.host = {"w": {k: v.cpu().pin_memory() for k, v in self.weights.items()},
                     "x": [{k: v.cpu().pin_memory() for k, v in layer.items()} for layer in self.inputs]}
        self.copy_stream = torch.cuda.Stream(self.device)

    def _mark(self, marks, name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append((name, ev))

    def step(self, from_host=False, to_host=False):
        from hi2_b200 import dist as hd
        from hi2_b200 import layer as L
        from hi2_b200.allocate import allocate_global
        from hi2_b200.calibrate import TensorTable

        marks: list = []
        ready = None
        if from_host:  # this step's inputs come over PCIe, overlapped with the kernels below
            ready = {}
            with torch.cuda.stream(self.copy_stream):
                for name, w in self.weights.items():
                    w.copy_(self.host["w"][name], non_blocking=True)
                ready["w"] = self.copy_stream.record_event()
                for name in self.input_order():  # the order of use
                    for layer, xs in enumerate(self.inputs):
                        xs[name].copy_(self.host["x"][layer][name], non_blocking=True)
                        ready[(layer, name)] = self.copy_stream.record_event()
        cur = torch.cuda.current_stream(self.device)
        # Inputs are taken widest first: the K = 11008 factorisation is the longest chain, so it
        # starts earliest and runs on its side stream beside everything that follows.
        order = self.input_order()
        self._mark(marks, "hessian")
        shared_all = [dict() for _ in self.inputs]
        pending, factors, tables = [], {}, {}
        mine = shared_all[self.rank]
        if ready is not None:
            cur.wait_event(ready["w"])
        def finish_input(name):  # statistics, the factor (on a side stream) and the tables of one input
            L.finish_statistics(mine, self.qcfg, only=name)
            L.start_factors(mine, self.qcfg, self.device, only=name, into=factors)
            L.tabulate(self.weights, self.plan, mine, self.qcfg, only=name, into=tables)

        # With one layer per rank the partial sums of an input are kept as one [world, K, K] stack and
        # summed by ONE reduce-scatter (every link carries (world - 1) / world of the stack once);
        # otherwise each layer's sum is reduced onto its owner.  The token total is known without
        # asking: the shards of dist.token_shard add up to it.
        scatter = self.world > 1 and len(self.inputs) == self.world
        if scatter and not hasattr(self, "stacks"):
            self.stacks = {n: torch.empty(self.world, k, k, dtype=torch.float32, device=self.device)
                           for n, k in self.widths.items()}
        for name in order:
            for layer, xs in enumerate(self.inputs):
                if ready is not None:
                    cur.wait_event(ready[(layer, name)])
                where = {name: self.stacks[name][layer]} if scatter else None
                L.accumulate({name: xs[name]}, self.device, into=shared_all[layer], defer_check=True, storage=where)
                s = shared_all[layer][name]  # partial sum of this rank's tokens -> the layer's owner
                if not scatter:
                    n, work = hd.reduce_second_moment(s.hessian.S, s.hessian.n, hd.owner_of(layer, self.world),
                                                      async_op=True, n_total=self.cfg["tokens"])
                    s.hessian.n = n
                    if work is not None:
                        pending.append(work)
            if scatter:
                own, work = hd.reduce_scatter_second_moments(self.stacks[name], async_op=True)
                mine[name].hessian.S, mine[name].hessian.n = own, self.cfg["tokens"]
                pending.append(work)
            if from_host:  # end to end: work on an input as soon as it has arrived
                for work in pending:
                    work.wait()
                pending = []
                finish_input(name)
        if not from_host:  # resident: the second moments first (their timing stays unshared)
            for work in pending:
                work.wait()
            self._mark(marks, "tables")
            for name in order:  # every factorisation starts before the first table kernel
                L.finish_statistics(mine, self.qcfg, only=name)
                L.start_factors(mine, self.qcfg, self.device, only=name, into=factors)
            for name in order:
                L.tabulate(self.weights, self.plan, mine, self.qcfg, only=name, into=tables)
        tables = {name: tables[name] for name in self.weights}
        self._mark(marks, "allocate")
        tag = f"L{self.rank}."
        for name, t in tables.items():
            t.name = tag + name
        # a few bytes per row: every rank allocates over every table and keeps its own picks
        everything = hd.gather_error_tables(list(tables.values()), TensorTable)
        alloc = allocate_global(everything, self.cfg["bpw"])
        picks = {name: alloc.picks[tag + name] for name in tables}
        self._mark(marks, "encode")
        packed = L.encode(self.weights, self.plan, mine, tables, picks, self.qcfg, to_host=to_host, factors=factors)
        for sh in shared_all:  # partial sums taken for other ranks' layers: settle their status too
            for s in sh.values():
                s.hessian.check()
        self._mark(marks, "end")
        self.last = dict(marks=marks, alloc=alloc, packed=packed)
        return packed

    def collect_stage_times(self):
        marks = self.last["marks"]
        for (name, a), (_, b) in zip(marks, marks[1:]):
            self.stage_ms[name] = self.stage_ms.get(name, 0.0) + a.elapsed_time(b)

    def d2h_bytes(self):
        from hi2_b200.format import FIELDS

        return sum(getattr(t, f).numel() * getattr(t, f).element_size()
                   for t in self.last["packed"].values() for f in FIELDS)


class ModelJob:
    """Resident workload of one rank for a whole model (BASELINE config 3): ``layers`` decoder
    layers, layer l owned by rank ``l mod world`` ("strong" scaling: the model is fixed).

    Inputs resident when the timed region starts: the bf16 weights of the owned layers and this
    rank's token shard of ONE set of synthetic calibration activations (four tensors, 24 GB at
    524 288 tokens), which stands in for the inputs of every layer: 32 distinct sets do not fit in
    HBM, and in the real pipeline a layer's inputs are produced on the device by the layer before
    it.  Every layer's second moments are computed from it anew; nothing is reused between layers.

    A step is the reference's three phases (hi2/pipeline.py:1087-1252):
      tabulate  per group of ``world`` consecutive layers: every rank accumulates the partial
                second moments of its tokens for all layers of the group, one reduce-scatter per
                input hands layer ``g * world + r`` to rank r; the owner then derives statistics,
                starts the four factorisations on side streams and builds the seven error tables;
      allocate  all tables of the model (1.36 M rows) gathered once, one global allocation;
      encode    per owned layer: basis change / factor (already in flight), GPTQ, packing.
    """

    def __init__(self, cfg, rank, world, device):
        from hi2_b200 import dist as hd
        from hi2_b200.calibrate import ALL_CANDIDATES, Config

        self.cfg, self.rank, self.world, self.device = cfg, rank, world, device
        self.n_layers = cfg["layers"]
        if self.n_layers % world:
            raise SystemExit(f"{self.n_layers} layers do not divide over {world} ranks")
        self.groups = self.n_layers // world
        self.owned = [g * world + rank for g in range(self.groups)]
        self.shapes, self.widths, self.plan = shapes_of(cfg)
        self.qcfg = Config(candidates=candidates_of(cfg), refine_passes=int(cfg.get("refine_passes", 0)))
        self.weights = {l: make_weights(cfg, self.shapes, l, device) for l in self.owned}
        lo, hi = hd.token_shard(cfg["tokens"], rank, world)
        self.inputs = make_inputs(cfg, self.widths, 0, hi - lo, lo, device)
        self.rows_layer = sum(r for r, _ in self.shapes.values())
        self.rows = self.rows_layer * self.n_layers  # whole model, all ranks
        self.specs = [(l % world, f"L{l}.{name}", shape, candidates_of(cfg), cfg["tokens"], True)
                      for l in range(self.n_layers) for name, shape in self.shapes.items()]
        self.stacks = None
        self.host = None
        self.copy_stream = None
        self.stage_ms: dict = {}
        self.hessian_ms = 0.0
        self.hessian_launches = 0
        self.gptq = {}  # K -> [rows, ms] over the timed steps

    def input_order(self):
        rows = {n: 0 for n in self.widths}
        for w, (r, _) in self.shapes.items():
            rows[self.plan.reads[w]] += r
        return sorted(self.widths, key=lambda n: (-self.widths[n], -rows[n]))

    def h2d_bytes(self):
        n = sum(w.numel() * w.element_size() for ws in self.weights.values() for w in ws.values())
        return n + sum(x.numel() * x.element_size() for x in self.inputs.values())

    def pin_host_copies(self):
        self.host = {"w": {l: {k: v.cpu().pin_memory() for k, v in ws.items()} for l, ws in self.weights.items()},
                     "x": {k: v.cpu().pin_memory() for k, v in self.inputs.items()}}
        self.copy_stream = torch.cuda.Stream(self.device)

    def _mark(self, marks, name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append((name, ev))

    def step(self, from_host=False, to_host=False):
        from hi2_b200 import dist as hd
        from hi2_b200 import layer as L
        from hi2_b200.allocate import allocate_global
        from hi2_b200.calibrate import EncodeRequest, TensorTable, encode_many, group_rows

        marks: list = []
        cur = torch.cuda.current_stream(self.device)
        order = self.input_order()
        ready = None
        if from_host:  # this step's inputs over PCIe, in the order of use, beside the kernels below
            ready = {}
            with torch.cuda.stream(self.copy_stream):
                for name in order:
                    self.inputs[name].copy_(self.host["x"][name], non_blocking=True)
                    ready[name] = self.copy_stream.record_event()
                for l in self.owned:
                    for name, w in self.weights[l].items():
                        w.copy_(self.host["w"][l][name], non_blocking=True)
                    ready[l] = self.copy_stream.record_event()
        if self.world > 1 and self.stacks is None:
            self.stacks = {n: torch.empty(self.world, k, k, dtype=torch.float32, device=self.device)
                           for n, k in self.widths.items()}
        self._mark(marks, "tabulate")
        state = {}
        hess_events = []
        for g, mine_l in enumerate(self.owned):
            shared_all = [dict() for _ in range(self.world)]
            mine = shared_all[self.rank]
            pending = []
            h0 = torch.cuda.Event(enable_timing=True)
            h0.record()
            for name in order:
                if ready is not None and g == 0:
                    cur.wait_event(ready[name])
                for r in range(self.world):  # this rank's tokens, for the layer rank r owns in this group
                    where = {name: self.stacks[name][r]} if self.world > 1 else None
                    L.accumulate({name: self.inputs[name]}, self.device, into=shared_all[r], defer_check=True,
                                 storage=where)
                if self.world > 1:
                    own, work = hd.reduce_scatter_second_moments(self.stacks[name], async_op=True)
                    mine[name].hessian.S, mine[name].hessian.n = own, self.cfg["tokens"]
                    pending.append(work)
            h1 = torch.cuda.Event(enable_timing=True)
            h1.record()
            hess_events.append((h0, h1))
            for work in pending:
                work.wait()
            if ready is not None:
                cur.wait_event(ready[mine_l])
            # The factorisations start here, on side streams, beside the table kernels.  (Starting them
            # beside the GPTQ column loops of the encode phase instead was measured: the tables gain
            # 16 ms per layer and the column loops lose 24.)
            factors, tables = {}, {}
            for name in order:
                L.finish_statistics(mine, self.qcfg, only=name)
                L.start_factors(mine, self.qcfg, self.device, only=name, into=factors, release_scratch=True)
            for name in order:
                L.tabulate(self.weights[mine_l], self.plan, mine, self.qcfg, only=name, into=tables)
            for name, t in tables.items():
                t.name = f"L{mine_l}.{name}"
            state[mine_l] = dict(shared=mine, others=[sh for i, sh in enumerate(shared_all) if i != self.rank],
                                 factors=factors, tables={name: tables[name] for name in self.shapes})
        self._mark(marks, "allocate")
        local = [state[l]["tables"][name] for l in self.owned for name in self.shapes]
        everything = hd.gather_tables_known_layout(local, self.specs, TensorTable)
        below_floor = None
        if self.cfg.get("int8_fraction"):
            L.keep_int8_for_most_sensitive(everything, self.cfg["int8_fraction"])
        if self.cfg.get("bpw_infeasible"):  # a target below the format's floor: the reference warns and
            probe = allocate_global(everything, self.cfg["bpw_infeasible"])  # takes the cheapest assignment
            below_floor = {"target_bpw": self.cfg["bpw_infeasible"], "feasible": probe.feasible, "bpw": probe.bpw,
                           "rows_by_width": probe.frac_by_bits}
        alloc = allocate_global(everything, self.cfg["bpw"])
        # the allocation has read results back: the status words are there
        L.HessianStats.check_all([s_in.hessian for st in state.values() for sh in [st["shared"], *st["others"]]
                                  for s_in in sh.values()])
        for st in state.values():
            st["others"] = None
        self._mark(marks, "encode")
        # Several layers per call: rows of equal width from all of them share the column loops, and the
        # host reads status words back once per call, not once per layer.
        packed, timing = {}, []
        per_call = self.cfg.get("layers_per_encode", 4)
        calls = []
        for c0 in range(0, len(self.owned), per_call):
            chunk = self.owned[c0 : c0 + per_call]
            reqs, keys, fac = [], [], {}
            for l in chunk:
                st = state[l]
                for name, w in self.weights[l].items():
                    s_in = st["shared"][self.plan.reads[name]]
                    reqs.append(EncodeRequest(w, s_in.moments, st["tables"][name], alloc.picks[f"L{l}.{name}"],
                                              sigma=s_in.hessian.S, sigma_id=f"L{l}.{s_in.name}",
                                              sigma_n=s_in.hessian.n))
                    keys.append((l, name))
                for iname, f in st["factors"].items():
                    fac[f"L{l}.{iname}"] = f
            calls.append((chunk, reqs, keys, fac))
        # rows by candidate for the whole model with one read-back, now that the device is idle anyway:
        # the calls below then start without waiting for it
        group_rows([r for _, reqs, _, _ in calls for r in reqs])
        while calls:
            chunk, reqs, keys, fac = calls.pop(0)
            out = encode_many(reqs, self.qcfg, to_host=to_host, factors=fac, timing=timing)
            for (l, name), t in zip(keys, out):
                packed.setdefault(l, {})[name] = t
            del reqs, fac
            for l in chunk:
                state[l] = None  # second moments and factors of the layer are free again
        self._mark(marks, "end")
        self.last = dict(marks=marks, alloc=alloc, packed=packed, hess_events=hess_events, timing=timing,
                         below_floor=below_floor)
        return packed

    def collect_stage_times(self):
        marks = self.last["marks"]
        for (name, a), (_, b) in zip(marks, marks[1:]):
            self.stage_ms[name] = self.stage_ms.get(name, 0.0) + a.elapsed_time(b)
        for a, b in self.last["hess_events"]:
            self.hessian_ms += a.elapsed_time(b)
            self.hessian_launches += len(self.widths) * self.world
        for k, rows, a, b in self.last["timing"]:
            acc = self.gptq.setdefault(k, [0, 0.0])
            acc[0] += rows
            acc[1] += a.elapsed_time(b)

    def d2h_bytes(self):
        from hi2_b200.format import FIELDS

        return sum(getattr(t, f).numel() * getattr(t, f).element_size()
                   for layer in self.last["packed"].values() for t in layer.values() for f in FIELDS)


class MoeJob:
    """Resident workload of one rank for a mixture-of-experts model (BASELINE config 5): the expert
    projections of ``moe_layers`` layers; expert ``e`` of every layer is owned by rank ``e mod world``.

    Resident when the timed region starts: the bf16 weights of the owned experts, one set of
    synthetic activations (hidden states ``[tokens, hidden]`` and expert-intermediate states
    ``[tokens, expert_ffn]``, standing in for every layer's) and a seeded random router per layer.
    A step, per layer: route (top-k of ``x W_r^T + bias``), per owned expert the second moments of
    the tokens routed to it (gate/up share one, hi2/layerwise.py:140-154; down has its own), the
    top-up of experts below ``expert_min_tokens x widest input`` tokens with the layer's pooled sums
    (hi2/moe.py:152-156, hi2/layerwise.py:243-258; pooled over the ranks), statistics, factors on
    side streams, tables; then ONE allocation over all expert tables weighted by
    ``max(n_e / mean n, 0.05) / E`` (hi2/moe.py:188-207), then the encode with the experts of a layer
    batched through the GPTQ column loops (row groups select their factor, hi2/hessian.py:267-315).
    The path has no exchange of activations: every rank routes the same resident tokens."""

    def __init__(self, cfg, rank, world, device):
        from hi2_b200 import layer as L
        from hi2_b200.calibrate import ALL_CANDIDATES, Config

        self.cfg, self.rank, self.world, self.device = cfg, rank, world, device
        self.n_layers, self.experts = cfg["moe_layers"], cfg["experts"]
        h, f = cfg["hidden"], cfg["expert_ffn"]
        self.owned = [e for e in range(self.experts) if e % world == rank]
        self.proj = {"gate_proj": (f, h), "up_proj": (f, h), "down_proj": (h, f)}
        self.reads = {"gate_proj": "in", "up_proj": "in", "down_proj": "mid"}
        self.qcfg = Config(candidates=list(ALL_CANDIDATES))
        dt = torch_dtype(cfg["dtype"])
        g = torch.Generator(device=device).manual_seed(4242)
        self.weights = {}
        for l in range(self.n_layers):
            for e in self.owned:
                ge = torch.Generator(device=device).manual_seed(100000 + 1000 * l + e)
                for p, (r, k) in self.proj.items():
                    self.weights[(l, e, p)] = (torch.randn(r, k, generator=ge, device=device) * 0.02).to(dt)
        x = make_inputs(cfg, {"in": h, "mid": f}, 0, cfg["tokens"], 0, device)
        self.x_in, self.x_mid = x["in"], x["mid"]
        self.router = [(torch.randn(self.experts, h, generator=g, device=device) / h**0.5).to(dt) for _ in range(self.n_layers)]
        self.bias = [cfg["router_bias"] * torch.randn(self.experts, generator=g, device=device) for _ in range(self.n_layers)]
        self.rows_layer = self.experts * sum(r for r, _ in self.proj.values())
        self.rows = self.rows_layer * self.n_layers
        self.specs = [(e % world, f"L{l}.experts.{e}.{p}", shape, list(ALL_CANDIDATES), 0, True)
                      for l in range(self.n_layers) for e in range(self.experts) for p, shape in self.proj.items()]
        self.widths = {"in": h, "mid": f}
        self.stage_ms: dict = {}
        self.gptq: dict = {}
        self.plan = L.LayerPlan({f"experts.{e}.{p}": f"experts.{e}.{self.reads[p]}" for e in self.owned for p in self.proj})

    def route(self, l):
        """Token indices per expert: ``(order [tokens * top_k] sorted by expert, counts [experts])``."""
        logits = (self.x_in @ self.router[l].T).float() + self.bias[l]
        top = torch.topk(logits, self.cfg["top_k"], dim=1).indices  # [tokens, top_k], distinct experts per token
        flat = top.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=self.experts)
        return order // self.cfg["top_k"], counts

    def _mark(self, marks, name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append((name, ev))

    def step(self, to_host=False):
        import torch.distributed as dist

        from hi2_b200 import dist as hd
        from hi2_b200 import layer as L
        from hi2_b200 import moe
        from hi2_b200.allocate import allocate_global
        from hi2_b200.calibrate import EncodeRequest, TensorTable, encode_many

        marks: list = []
        self._mark(marks, "tabulate")
        state, token_counts = {}, {}
        reduce = (lambda t: dist.all_reduce(t)) if self.world > 1 else None
        for l in range(self.n_layers):
            tokens_of, counts = self.route(l)
            counts = counts.tolist()  # the one read-back of the layer
            offs = [0]
            for c in counts:
                offs.append(offs[-1] + c)
            shared = {}
            for e in self.owned:
                rows = tokens_of[offs[e] : offs[e + 1]]
                if rows.numel():
                    L.accumulate({f"experts.{e}.in": self.x_in.index_select(0, rows),
                                  f"experts.{e}.mid": self.x_mid.index_select(0, rows)}, self.device, into=shared,
                                 defer_check=True)
                else:  # an expert without tokens: empty sums, filled by the top-up
                    from hi2_b200.hessian import HessianStats

                    for nm, k in (("in", self.cfg["hidden"]), ("mid", self.cfg["expert_ffn"])):
                        shared[f"experts.{e}.{nm}"] = L.SharedInput(f"experts.{e}.{nm}", k, HessianStats(k, self.device))
            L.HessianStats.check_all([s_in.hessian for s_in in shared.values()])
            for s_in in shared.values():
                s_in.moments = L.ColumnStats.from_second_moment(s_in.hessian.S, s_in.hessian.n)
            own_tokens = {name: s_in.hessian.n for name, s_in in shared.items()}
            # leaders named like the expert's first projection, so the grouping of hi2_b200.moe applies
            alias = {f"experts.{e}.in": f"L{l}.experts.{e}.gate_proj" for e in self.owned}
            alias.update({f"experts.{e}.mid": f"L{l}.experts.{e}.down_proj" for e in self.owned})
            borrowed = moe.top_up({alias[n]: s_in.moments for n, s_in in shared.items()},
                                  {alias[n]: s_in.hessian for n, s_in in shared.items()},
                                  {alias[n]: s_in.k for n, s_in in shared.items()}, self.qcfg.expert_min_tokens, reduce)
            weights = {f"experts.{e}.{p}": self.weights[(l, e, p)] for e in self.owned for p in self.proj}
            factors, tables = {}, {}
            for s_in in shared.values():
                flags = torch.ones(s_in.k // 16, dtype=torch.uint8)
                from hi2_b200.calibrate import smoothing_scale

                s_in.transform = (smoothing_scale(s_in.moments, self.qcfg.smooth), flags)
            L.start_factors(shared, self.qcfg, self.device, into=factors, release_scratch=True)
            L.tabulate(weights, self.plan, shared, self.qcfg, into=tables, grouped=True)
            for name, t in tables.items():
                t.name = f"L{l}.{name}"
                t.n_tokens = own_tokens[self.plan.reads[name]]  # an expert reports its own tokens (hi2/layerwise.py:230)
            state[l] = dict(shared=shared, factors=factors, tables=tables, weights=weights, borrowed=len(borrowed))
            token_counts[l] = counts
        self._mark(marks, "allocate")
        local = [state[l]["tables"][f"experts.{e}.{p}"] for l in range(self.n_layers) for e in self.owned for p in self.proj]
        specs = [(o, n, sh, c, token_counts[int(n.split(".")[0][1:])][int(n.split(".")[2])], sc)
                 for o, n, sh, c, _, sc in self.specs]
        everything = hd.gather_tables_known_layout(local, specs, TensorTable)
        share = moe.expert_weights({t.name: t for t in everything})
        alloc = allocate_global(everything, self.cfg["bpw"], sensitivity=share)
        self._mark(marks, "encode")
        packed, timing = {}, []
        for l in range(self.n_layers):
            st = state[l]
            reqs, keys = [], []
            for name, w in st["weights"].items():
                s_in = st["shared"][self.plan.reads[name]]
                reqs.append(EncodeRequest(w, s_in.moments, st["tables"][name], alloc.picks[f"L{l}.{name}"],
                                          sigma=s_in.hessian.S, sigma_id=s_in.name, sigma_n=s_in.hessian.n))
                keys.append((l, name))
            out = encode_many(reqs, self.qcfg, to_host=to_host, factors=st["factors"], timing=timing)
            for k_, t in zip(keys, out):
                packed[k_] = t
            state[l] = dict(borrowed=st["borrowed"])
        self._mark(marks, "end")
        self.last = dict(marks=marks, alloc=alloc, packed=packed, timing=timing, token_counts=token_counts,
                         borrowed=sum(st["borrowed"] for st in state.values()), share=share)
        return packed

    def collect_stage_times(self):
        marks = self.last["marks"]
        for (name, a), (_, b) in zip(marks, marks[1:]):
            self.stage_ms[name] = self.stage_ms.get(name, 0.0) + a.elapsed_time(b)
        for k, rows, a, b in self.last["timing"]:
            acc = self.gptq.setdefault(k, [0, 0.0])
            acc[0] += rows
            acc[1] += a.elapsed_time(b)


class PropagatedJob:
    """The whole-model workload with the calibration activations PRODUCED ON THE DEVICE: a
    Llama-shaped model (random init) and calibration token ids start in pinned host memory; a step
    copies the weights of the owned layers to the device (the owners then broadcast them over
    NVLink, every rank runs every layer), embeds the ids, runs the decoder layers one at a time over
    this rank's sequences with the statistics taken by forward pre-hooks
    (hi2_b200.layerwise.calibrate_layerwise), allocates over all tables, encodes every Linear from
    the statistics left in HBM, and copies the packed buffers back.  No activation crosses PCIe.
    The layer forward itself (library GEMMs and attention) is the caller's model, not this
    package's kernels; its time is inside the step."""

    def __init__(self, cfg, rank, world, device, heads=32, vocab=32000):
        from transformers import LlamaConfig, LlamaForCausalLM

        self.cfg, self.rank, self.world, self.device = cfg, rank, world, device
        seq_len = 2048 if cfg["tokens"] % 2048 == 0 else cfg["tokens"]
        self.sequences = cfg["tokens"] // seq_len
        mc = LlamaConfig(hidden_size=cfg["hidden"], intermediate_size=cfg["ffn"], num_hidden_layers=cfg["layers"],
                         num_attention_heads=heads, num_key_value_heads=heads, vocab_size=vocab,
                         max_position_embeddings=seq_len)
        dt = torch_dtype(cfg["dtype"])
        old = torch.get_default_dtype()
        torch.set_default_dtype(dt)
        try:
            torch.manual_seed(1234)  # the same model on every rank
            with torch.device(device):
                self.model = LlamaForCausalLM(mc).eval()
        finally:
            torch.set_default_dtype(old)
        self.layers = self.model.model.layers
        g = torch.Generator().manual_seed(99)
        self.ids_host = torch.randint(0, vocab, (self.sequences, seq_len), generator=g).pin_memory()
        self.owned = [l for l in range(cfg["layers"]) if l % world == rank]
        self.host = {l: [p.detach().cpu().pin_memory() for p in self.layers[l].parameters()] for l in self.owned}
        self.h2d = sum(t.numel() * t.element_size() for ts in self.host.values() for t in ts) + \
            self.ids_host.numel() * self.ids_host.element_size()
        self.rows = sum(p.shape[0] for l in range(cfg["layers"]) for n, p in self.layers[l].named_parameters()
                        if p.dim() == 2)
        from hi2_b200.calibrate import ALL_CANDIDATES, Config

        self.qcfg = Config(candidates=list(ALL_CANDIDATES))
        self.specs = None

    def step(self):
        import torch.distributed as dist

        from hi2_b200 import dist as hd
        from hi2_b200.allocate import allocate_global
        from hi2_b200.calibrate import ALL_CANDIDATES, TensorTable
        from hi2_b200.layerwise import DeviceSink, calibrate_layerwise, encode_layerwise

        for l in self.owned:
            for p, h in zip(self.layers[l].parameters(), self.host[l]):
                p.data.copy_(h, non_blocking=True)
        if self.world > 1:
            for l in range(self.cfg["layers"]):
                for p in self.layers[l].parameters():
                    dist.broadcast(p.data, src=l % self.world)
        ids = self.ids_host.to(self.device, non_blocking=True)
        sink = DeviceSink()
        t0 = torch.cuda.Event(enable_timing=True)
        t0.record()
        tables = calibrate_layerwise(self.model, ids, self.qcfg, exclude=["lm_head|embed"], sink=sink,
                                     log=lambda *_: None, device=self.device)
        t1 = torch.cuda.Event(enable_timing=True)
        t1.record()
        if self.specs is None:
            self.specs = [(l % self.world, f"model.layers.{l}.{n}.weight", tuple(m.weight.shape), list(ALL_CANDIDATES),
                           self.cfg["tokens"], True)
                          for l in range(self.cfg["layers"]) for n, m in self.layers[l].named_modules()
                          if isinstance(m, torch.nn.Linear)]
        local = [tables[name] for owner, name, *_ in self.specs if owner == self.rank]
        everything = hd.gather_tables_known_layout(local, self.specs, TensorTable)
        alloc = allocate_global(everything, self.cfg["bpw"])
        packed = encode_layerwise(self.model, tables, alloc.picks, sink, self.qcfg, to_host=True)
        self.last = dict(alloc=alloc, packed=packed, tabulate=(t0, t1))
        return packed

    def d2h_bytes(self):
        from hi2_b200.format import FIELDS

        return sum(getattr(t, f).numel() * getattr(t, f).element_size() for t in self.last["packed"].values()
                   for f in FIELDS)


def hessian_flops(widths, tokens):
    """(algorithmic 2 T K^2, issued by the upper-triangle 128 x 256 tiles) summed over the inputs."""
    algo = issued = 0.0
    for k in widths.values():
        nib, njb = -(-k // 128), -(-k // 256)
        tiles = sum(njb - (ib >> 1) for ib in range(nib))
        algo += 2.0 * tokens * k * k
        issued += 2.0 * tokens * tiles * 128 * 256
    return algo, issued


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return dict(hbm=p["hbm_gbs"], tensor=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    tensor_burst=p["bf16_tflops"], source="measured")
    return dict(hbm=6650.0, tensor=1400.0, tensor_burst=1590.0, source="fallback")


# --------------------------------------------------------------------------------------------
# the CPU arm: the oracle (a restatement of the reference's CPU path) on the host cores
# --------------------------------------------------------------------------------------------
_FACTOR_SECONDS: dict = {}  # width -> measured seconds of one full-size CPU factorisation (timed once per process)


def cpu_sample(cfg, threads: int, budget_s: float = 30.0) -> dict:
    """The oracle (a restatement of the reference's CPU path) on a BOUNDED sample of one layer of the
    workload, every stage scaled to the whole workload by the units it processes:

    * second moments and group moments: 4096 tokens per input (the reference's own chunk size, the
      product is in its efficient regime), scaled by tokens;
    * basis change and factorisation: FULL size per distinct input (the widest is timed once per
      process and its time reused, the others every call);
    * tables: a row sample of every matrix, all six candidates, scaled by rows (the search is
      elementwise over rows);
    * allocation: on the sampled tables (its cost is negligible either way);
    * GPTQ: ladders on a row sample (scaled by rows); the column loop on row groups of FULL size
      (the allocation's shares of the matrix: a column step costs the same for 32 rows as for
      2000, so a row sample would not do) over the first and the last 128-column block, whose mean
      is the mean cost of a block (the trailing update shrinks linearly), scaled by blocks;
    * packing: the sampled rows, scaled by rows.

    The row sample is sized so that the call takes about ``budget_s`` seconds.  Returns the
    extrapolated seconds per stage for ONE layer and their sum times the number of layers."""
    from oracle import ptq_oracle as po

    torch.set_num_threads(threads)
    shapes, widths, plan = shapes_of(cfg)
    cands = candidates_of(cfg)
    dt = torch_dtype(cfg["dtype"])
    g = torch.Generator().manual_seed(0)
    t = {k: 0.0 for k in ("hessian", "statistics", "tables", "allocate", "factor", "gptq_ladders", "gptq_columns", "pack")}
    tokens_s = min(4096, cfg["tokens"])
    # tables cost ~1.7 us per weight and candidate on 8 cores: keep them within about half of the budget
    weights_per_row = sum(k for _, k in shapes.values())
    rows_s = int(max(32, min(1024, 0.5 * budget_s / (1.0e-6 * 6 * weights_per_row) * threads / 8)))
    shared = {}
    for name, k in widths.items():
        x = (torch.randn(tokens_s, k, generator=g) * torch.exp(cfg["spread"] * torch.randn(1, k, generator=g))).to(dt)
        t0 = time.perf_counter()
        sm, gm = po.SecondMoment(k), po.GroupMoments(k)
        sm.update(x)
        gm.update(x)
        t["hessian"] += (time.perf_counter() - t0) * (cfg["tokens"] / tokens_s)
        t0 = time.perf_counter()
        s16 = po.smoothing_vector(gm, 0.5)
        had = torch.ones(k // 16, dtype=torch.uint8)
        d_tab = gm.diag(had, 1.0 / s16.float())
        t["statistics"] += time.perf_counter() - t0
        hs = po.stored_basis_hessian(sm.mean(), s16, had)
        widest = k == max(widths.values()) and k > 4096
        if widest and k in _FACTOR_SECONDS:
            u = _FACTOR_SECONDS[k][1]
            t["factor"] += _FACTOR_SECONDS[k][0]
        else:
            t0 = time.perf_counter()
            hs = po.stored_basis_hessian(sm.mean(), s16, had)
            u = po.inverse_cholesky(hs, 0.01)
            dtf = time.perf_counter() - t0
            t["factor"] += dtf
            if widest:
                _FACTOR_SECONDS[k] = (dtf, u)
        shared[name] = dict(s16=s16, had=had, d_tab=d_tab, u=u, d=hs.diagonal().clone())
    tables, stored = [], {}
    for name, (r, k) in shapes.items():
        s_in = shared[plan.reads[name]]
        rs = min(rows_s, r)
        w = (torch.randn(rs, k, generator=g) * 0.02).to(dt)
        t0 = time.perf_counter()
        wt = po.rotate_groups(w.float() * s_in["s16"].float(), s_in["had"])
        sse = torch.stack([po.nearest_rows(wt, s_in["d_tab"], nb, b).sse for nb, b in cands])
        energy = float((s_in["d_tab"] * wt**2).sum())
        t["tables"] += (time.perf_counter() - t0) * (r / rs)
        tables.append(po.Table(name, (rs, k), s_in["had"], sse, list(cands), energy, cfg["tokens"], s_in["s16"]))
        stored[name] = (wt, r / rs)
    t0 = time.perf_counter()
    alloc = po.allocate_rows(tables, cfg["bpw"])
    t["allocate"] += time.perf_counter() - t0
    groups = []
    for table in tables:
        s_in = shared[plan.reads[table.name]]
        wt, scale = stored[table.name]
        r, k = shapes[table.name]
        picks = alloc.picks[table.name]
        blocks = -(-k // 128)
        ends = {0, blocks - 1}
        pieces = []
        for ci, (nb, b) in enumerate(cands):
            rows = (picks == ci).nonzero().flatten()
            if rows.numel() == 0:
                continue
            # ladders of the sampled rows of this group (row-linear)
            t0 = time.perf_counter()
            lo, st = po.search_ladder(wt[rows].reshape(rows.numel(), k // b, b), s_in["d"].reshape(1, k // b, b), 2**nb)
            lad = po.quantise_ladders(lo, st)
            t["gptq_ladders"] += (time.perf_counter() - t0) * scale
            # the column loop at the group's FULL size, first and last block
            n_full = max(1, round(rows.numel() * scale))
            reps = -(-n_full // rows.numel())
            big = wt[rows].repeat(reps, 1)[:n_full]
            lad_big = tuple(x.repeat(reps, *([1] * (x.dim() - 1)))[:n_full] for x in lad)
            t0 = time.perf_counter()
            e = po.gptq_rows(big, s_in["d"], s_in["u"], nb, b, ladders=lad_big, only_blocks=ends)
            t["gptq_columns"] += (time.perf_counter() - t0) * (blocks / len(ends))
            groups.append((table.name, nb, b, n_full))
            pieces.append((rows, e.codes[: rows.numel()], e.params[: rows.numel()], e.consts[: rows.numel()]))
        t0 = time.perf_counter()
        nbits = torch.tensor([cands[i][0] for i in picks.tolist()])
        block = torch.tensor([cands[i][1] for i in picks.tolist()])
        po.assemble_flat(pieces, nbits, block, s_in["had"], k, s_in["s16"])
        t["pack"] += (time.perf_counter() - t0) * scale
    layers = cfg.get("layers", 1)
    per_layer = sum(t.values())
    return dict(seconds=per_layer * layers, seconds_per_layer=per_layer, layers=layers,
                stages={k: round(v, 3) for k, v in t.items()}, rows=sum(r for r, _ in shapes.values()) * layers,
                sample=f"one layer of {layers}: {tokens_s} of {cfg['tokens']} tokens per input; {rows_s} rows of each matrix "
                       f"for tables, ladders and packing; the GPTQ column loop on {len(groups)} row groups of full size "
                       f"(first and last 128-column block of each); basis change and factorisation at full size; every "
                       f"stage scaled by its units, the layer by {layers} (extrapolated)")


def cpu_config1_full(threads: int) -> dict:
    """BASELINE config 1 IN FULL on the host (the case the reference itself runs on a CPU): the
    oracle's whole chain for the 4096 x 4096 Linear with 2048 calibration tokens at 3.0 bpw, timed
    stage by stage, nothing sampled, nothing scaled."""
    from oracle import ptq_oracle as po

    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(2024)
    k = r = 4096
    w = torch.randn(r, k, generator=g) * 0.02
    w[:, torch.randperm(k, generator=g)[:4]] *= 20
    w = w.half()
    x = (torch.randn(2048, k, generator=g) * torch.exp(torch.randn(1, k, generator=g))).half()
    cands = [(nb, b) for nb in (2, 4) for b in (16, 32, 64)]
    st = {}
    t0 = time.perf_counter()
    sm, gm = po.SecondMoment(k), po.GroupMoments(k)
    sm.update(x)
    gm.update(x)
    st["hessian"] = time.perf_counter() - t0
    t0 = time.perf_counter()
    s16 = po.smoothing_vector(gm, 0.5)
    had = torch.ones(k // 16, dtype=torch.uint8)
    wt = po.rotate_groups(w.float() * s16.float(), had)
    d_tab = gm.diag(had, 1.0 / s16.float())
    sse = torch.stack([po.nearest_rows(wt, d_tab, nb, b).sse for nb, b in cands])
    table = po.Table("w", (r, k), had, sse, list(cands), float((d_tab * wt**2).sum()), 2048, s16)
    st["tables"] = time.perf_counter() - t0
    t0 = time.perf_counter()
    alloc = po.allocate_rows([table], 3.0)
    st["allocate"] = time.perf_counter() - t0
    t0 = time.perf_counter()
    hs = po.stored_basis_hessian(sm.mean(), s16, had)
    u = po.inverse_cholesky(hs, 0.01)
    st["factor"] = time.perf_counter() - t0
    t0 = time.perf_counter()
    d = hs.diagonal().clone()
    picks = alloc.picks["w"]
    pieces = []
    for ci, (nb, b) in enumerate(cands):
        rows = (picks == ci).nonzero().flatten()
        if rows.numel():
            e = po.gptq_rows(wt[rows], d, u, nb, b)
            pieces.append((rows, e.codes, e.params, e.consts))
    st["gptq"] = time.perf_counter() - t0
    t0 = time.perf_counter()
    cand = torch.tensor(cands)
    po.assemble_flat(pieces, cand[picks, 0], cand[picks, 1], had, k, s16)
    st["pack"] = time.perf_counter() - t0
    total = sum(st.values())
    return {"workload": CONFIGS["cfg1"]["workload"], "seconds": total, "rows_per_s": r / total,
            "stages_s": {k: round(v, 3) for k, v in st.items()}, "bpw": alloc.bpw, "sampled": False}


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference(args, cfg):
    """The CPU arm: the oracle on all host threads, one bounded sample of the workload per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    n = args.warmup + args.steps
    budget = max(8.0, min(30.0, 150.0 / max(1, n)))  # the whole run stays within a few minutes
    times = []
    walls = []
    for i in range(n):
        t0 = time.perf_counter()
        res = cpu_sample(cfg, threads, budget)
        if i >= args.warmup:
            times.append(res)
            walls.append(time.perf_counter() - t0)
    secs = sum(r["seconds"] for r in times) / len(times)
    value = res["rows"] / secs
    whole_model = "layers" in cfg
    line = {
        "impl": "reference", "metric": "ptq_encode_rows_per_s", "value": value, "unit": "rows/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3,
        "higher_is_better": True, "scaling": "strong" if whole_model else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": cfg["workload"], "layers": cfg.get("layers", 1), "tokens_per_input": cfg["tokens"],
                   "target_bpw": cfg["bpw"], "candidates": "int2,int4 x b16,b32,b64",
                   "note": "CPU restatement of the reference (oracle/) on the host cores; value and ms_per_step are the "
                           "full-workload figures EXTRAPOLATED from a bounded sample per step (see cpu_baseline.sample)"},
        "encode_wall_s": secs,
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": "port",
                         "sample": res["sample"], "stages_s_per_layer": res["stages"],
                         "sample_wall_s_per_step": round(sum(walls) / len(walls), 1)},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ncu capture of the second-moment kernel at 32768 tokens x 4096 columns
# (profiles/hessian_tc_kernel_k4096_32k_tokens.md): DRAM reads were 2.08 x the bytes of X (L2 absorbs
# the rest of the tile re-reads), DRAM writes the per-item output tiles.  Reads grow in proportion
# to the tokens, the tiles do not, so a full-size launch is scaled from those two figures.
# DRAM reads of the second-moment kernel as a multiple of the bytes of X, from ncu captures at
# 32768 tokens: 1.05 at K = 4096 (pair kernel, X of a wave fits in L2), 6.2 at K = 11008 (one-block
# kernel, banded tile schedule, ~13 waves of which the L2 absorbs half)
HESSIAN_READ_FACTOR = {4096: 1.05, 11008: 6.2}


def hessian_traffic(widths, tokens, elem_bytes=2):
    """Estimated DRAM bytes per launch, averaged over the launches of one step."""
    total = 0.0
    for k in widths.values():
        kblocks = -(-tokens // 64)
        cap = max(1, kblocks // 64)
        if 1024 <= k <= 8192:
            # CTA-pair kernel: 256 x 256 fp32 per (tile, token split); the split count follows the
            # kernel's plan (fewest waves per split, at most 512 MiB of tiles)
            nb = -(-k // 256)
            tiles, area = nb * (nb + 1) // 2, 256 * 256
            splits, best_cost = 1, float("inf")
            for sp in range(1, min(16, cap) + 1):
                if sp > 1 and sp * tiles * area * 4 > (512 << 20):
                    break
                cost = -(-tiles * sp // 74) / sp
                if cost < best_cost * 0.995:
                    splits, best_cost = sp, cost
        else:  # one-block kernel: 128 x 256 tiles
            nib, njb = -(-k // 128), -(-k // 256)
            tiles, area = sum(njb - (ib >> 1) for ib in range(nib)), 128 * 256
            splits = max(1, min(-(-148 * 6 // tiles), cap))
        factor = HESSIAN_READ_FACTOR.get(k, 1.05 if k <= 4096 else 6.2)
        total += factor * tokens * k * elem_bytes + splits * tiles * area * 4
    return total / max(1, len(widths))


def mem_available_bytes() -> int:
    try:
        for line in open("/proc/meminfo"):
            if line.startswith("MemAvailable"):
                return int(line.split()[1]) * 1024
    except OSError:
        pass
    return 0


def all_ranks_agree(flag: bool, world: int, device) -> bool:
    """True only if ``flag`` holds on EVERY rank.  A per-rank decision that steers collectives (whether
    the end-to-end leg runs: its steps reduce-scatter and gather) must be the same everywhere; free
    host memory is read at slightly different moments by ranks that are pinning buffers meanwhile."""
    if world == 1:
        return bool(flag)
    import torch.distributed as dist

    t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(int(t.item()))


def run_ours(args, cfg):
    import torch.distributed as dist

    from hi2_b200 import _lib
    from hi2_b200 import dist as hd

    rank, world, device = hd.init_from_env("cuda")
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}", file=sys.stderr)
    _lib.load()
    whole_model = "layers" in cfg
    job = ModelJob(cfg, rank, world, device) if whole_model else Job(cfg, rank, world, device)
    total_rows = job.rows if whole_model else job.rows * world

    def sync_all():
        torch.cuda.synchronize(device)
        hd.barrier()
        torch.cuda.synchronize(device)

    for _ in range(args.warmup):
        job.step()
    sync_all()
    clocks = Clocks(device.index or 0)
    if rank == 0:
        clocks.start()
    launches0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        job.step()
        torch.cuda.synchronize(device)
        job.collect_stage_times()
    ev1.record()
    sync_all()
    launches = _lib.launch_count() - launches0
    ms = torch.tensor([ev0.elapsed_time(ev1) / args.steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item())
    clock_info = clocks.stop() if rank == 0 else None
    alloc = job.last["alloc"]
    below_floor = job.last.get("below_floor") if whole_model else None

    # ---- end to end: pinned host buffers in, packed buffers out ------------------------------
    e2e = None
    need = job.h2d_bytes()
    if args.no_e2e:
        e2e = {"value": None, "unit": "rows/s", "h2d_bytes_per_step": need * world, "d2h_bytes_per_step": 0,
               "note": "skipped (--no-e2e)"}
    elif all_ranks_agree(mem_available_bytes() > 3 * need * max(1, int(os.environ.get("LOCAL_WORLD_SIZE", world))),
                         world, device):
        job.pin_host_copies()
        job.step(from_host=True, to_host=True)  # warm-up of the copy path
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            job.step(from_host=True, to_host=True)
        e1.record()
        sync_all()
        ems = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(ems, op=dist.ReduceOp.MAX)
        e2e = {"value": total_rows / (float(ems.item()) / 1e3), "unit": "rows/s",
               "ms_per_step": float(ems.item()), "h2d_bytes_per_step": need * world,
               "d2h_bytes_per_step": job.d2h_bytes() * world}
    else:
        e2e = {"value": None, "unit": "rows/s", "h2d_bytes_per_step": need * world, "d2h_bytes_per_step": 0,
               "note": "host memory too small to pin the inputs"}

    # ---- the same model with the activations produced on the device (calibration propagation) ----
    propagated = None
    if whole_model and not args.no_propagate and not cfg.get("kv_rows"):  # the toy model builder has no GQA case
        keep = dict(stage_ms=job.stage_ms, hessian_ms=job.hessian_ms, hessian_launches=job.hessian_launches,
                    gptq=job.gptq, widths=job.widths, rows_layer=job.rows_layer)
        job.weights = job.inputs = job.host = job.stacks = job.last = None  # free HBM and pinned memory
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        pj = PropagatedJob(cfg, rank, world, device)
        pj.step()
        sync_all()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        tab_ms = 0.0
        psteps = min(args.steps, 2)  # a step is 10-20 s: two are enough for a steady figure
        for _ in range(psteps):
            pj.step()
            torch.cuda.synchronize(device)
            tab_ms += pj.last["tabulate"][0].elapsed_time(pj.last["tabulate"][1])
        p1.record()
        sync_all()
        pms = torch.tensor([p0.elapsed_time(p1) / psteps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(pms, op=dist.ReduceOp.MAX)
        propagated = {"value": pj.rows / (float(pms.item()) / 1e3), "unit": "rows/s", "ms_per_step": float(pms.item()),
                      "steps": psteps, "forward_and_tabulate_ms": tab_ms / psteps, "achieved_bpw": pj.last["alloc"].bpw,
                      "h2d_bytes_per_step": pj.h2d * world, "d2h_bytes_per_step": pj.d2h_bytes() * world,
                      "note": "weights and token ids from pinned host memory, activations produced on the device by "
                              "the layer forwards (library GEMMs and attention, inside the step), packed buffers back"}
        job.stage_ms, job.hessian_ms, job.hessian_launches, job.gptq = (keep["stage_ms"], keep["hessian_ms"],
                                                                        keep["hessian_launches"], keep["gptq"])

    if rank != 0:
        return
    pk = peaks()
    stage = {k: v / args.steps for k, v in job.stage_ms.items()}
    if whole_model:
        # second moments: CUDA events around every layer group's launches (the reduce-scatters and the
        # previous layer's factorisations run beside them)
        stage["hessian"] = job.hessian_ms / args.steps
        n_launch = job.hessian_launches / args.steps
        tokens_per_launch = cfg["tokens"] // world
        algo, issued = hessian_flops(job.widths, tokens_per_launch)
        algo, issued = algo * n_launch / len(job.widths), issued * n_launch / len(job.widths)
    else:
        n_launch = len(job.widths) * world
        tokens_per_launch = cfg["tokens"] // world
        algo, issued = hessian_flops(job.widths, cfg["tokens"])
    hess_s = stage["hessian"] / 1e3
    achieved = issued / hess_s / 1e12
    roofline = {
        "kernel": "hessian_pair_kernel / hessian_tc_kernel (second moment X^T X, tcgen05 cta_group::2 up to K=8192, cta_group::1 beyond; fp32 accumulate)",
        "bound": "tensor", "achieved": achieved, "peak": pk["tensor"], "unit": "TFLOP/s",
        "frac": achieved / pk["tensor"], "peak_source": f"{pk['source']}, sustained (kernel timed inside a long step)",
        "effective": algo / hess_s / 1e12,
        "note": "achieved counts the flops issued (upper-triangle 256x256 tiles); effective counts 2*T*K^2",
        "traffic": hessian_traffic(job.widths, tokens_per_launch),
        "traffic_note": "bytes per launch, scaled from ncu captures at 32768 tokens (reads 1.05 x X at K=4096, 6.2 x X at K=11008, plus item tiles)",
        "algorithmic_bytes": sum(tokens_per_launch * k * 2 + 4 * k * k for k in job.widths.values()) / max(1, len(job.widths)),
        "launches_per_step": n_launch,
        "launch_ms": hess_s * 1e3 / max(1, n_launch),
    }
    cpu = None
    if world == 1 and not args.no_cpu_baseline and max(job.widths.values()) <= 16384:  # wider: minutes per factor
        threads = host_threads()
        t0 = time.perf_counter()
        res = cpu_sample(cfg, threads, 25.0)
        wall = time.perf_counter() - t0
        cpu = {"value": res["rows"] / res["seconds"], "unit": "rows/s", "cores": threads, "kind": "port",
               "sample": res["sample"], "sample_wall_s": round(wall, 1), "seconds_full_workload": res["seconds"],
               "stages_s_per_layer": res["stages"],
               "config1_in_full": None if args.no_config1 else cpu_config1_full(threads)}
    config = {"workload": cfg["workload"], "layers": cfg.get("layers", world), "rows_per_layer": job.rows_layer if whole_model else job.rows,
              "tokens_per_input": cfg["tokens"], "target_bpw": cfg["bpw"], "achieved_bpw": alloc.bpw,
              "candidates": "int2,int4 x b16,b32,b64" + (" + int8 x b32,b64 for the "
                                                          f"{cfg['int8_fraction']:.0%} most sensitive rows" if cfg.get("int8_fraction") else ""),
              "parallelism": (f"layer l on rank l mod {world}, token-sharded hessian, one reduce-scatter per input and layer group"
                              if whole_model else f"layer-per-gpu x{world}, token-sharded hessian"),
              "l2": "inputs larger than L2 (12-24 GB of activations per layer)"}
    if cfg.get("refine_passes"):
        config["refine_passes"] = cfg["refine_passes"]
    if whole_model:
        config["activations"] = ("one synthetic set (four tensors) stands in for the inputs of every layer; each layer's "
                                 "statistics are computed from it anew")
    line = {
        "metric": "ptq_encode_rows_per_s", "value": total_rows / (ms_per_step / 1e3), "unit": "rows/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if whole_model else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config,
        "encode_wall_s": ms_per_step / 1e3,
        "stage_ms": {k: round(v, 3) for k, v in stage.items()},
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
        "gpu_launches": launches, "clocks": clock_info,
    }
    if propagated is not None:
        line["propagated"] = propagated
    if whole_model and below_floor is not None:
        line["allocation_below_format_floor"] = below_floor
        line["rows_by_width"] = alloc.frac_by_bits
    if whole_model and job.gptq:
        # rows through the GPTQ column loop (block kernel + trailing updates) per second of that loop,
        # per width; the widths run beside each other on two streams
        line["gptq_rows_per_s"] = {str(k): rows / (ms / 1e3) for k, (rows, ms) in sorted(job.gptq.items())}
    emit(line)


def run_moe(args, cfg):
    """BASELINE config 5 (per-expert statistics and GPTQ, experts spread over the ranks): the resident
    step only; prints one line with the same keys as the default workload's where they apply."""
    import statistics

    import torch.distributed as dist

    from hi2_b200 import _lib
    from hi2_b200 import dist as hd

    rank, world, device = hd.init_from_env("cuda")
    _lib.load()
    job = MoeJob(cfg, rank, world, device)

    def sync_all():
        torch.cuda.synchronize(device)
        hd.barrier()
        torch.cuda.synchronize(device)

    for _ in range(args.warmup):
        job.step()
    sync_all()
    clocks = Clocks(device.index or 0)
    if rank == 0:
        clocks.start()
    launches0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        job.step()
        torch.cuda.synchronize(device)
        job.collect_stage_times()
    ev1.record()
    sync_all()
    launches = _lib.launch_count() - launches0
    ms = torch.tensor([ev0.elapsed_time(ev1) / args.steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clock_info = clocks.stop() if rank == 0 else None
    if rank != 0:
        return
    ms_per_step = float(ms.item())
    counts = [c for layer in job.last["token_counts"].values() for c in layer]
    alloc = job.last["alloc"]
    emit({
        "metric": "ptq_encode_rows_per_s", "value": job.rows / (ms_per_step / 1e3), "unit": "rows/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["workload"], "layers": cfg["moe_layers"], "experts": cfg["experts"], "top_k": cfg["top_k"],
                   "rows_per_layer": job.rows_layer, "tokens": cfg["tokens"], "target_bpw": cfg["bpw"],
                   "achieved_bpw": alloc.bpw, "parallelism": f"expert e on rank e mod {world}; no exchange of activations",
                   "tokens_per_expert": {"min": min(counts), "median": statistics.median(counts), "max": max(counts)},
                   "expert_inputs_topped_up": job.last["borrowed"],
                   "activations": "one synthetic set stands in for every layer's hidden and expert-intermediate states"},
        "encode_wall_s": ms_per_step / 1e3, "stage_ms": {k: round(v / args.steps, 3) for k, v in job.stage_ms.items()},
        "gptq_rows_per_s": {str(k): rows / (t / 1e3) for k, (rows, t) in sorted(job.gptq.items())},
        "roofline": None, "cpu_baseline": None,
        "e2e": {"value": None, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "not measured for this configuration (the default workload carries the end-to-end figure)"},
        "gpu_launches": launches, "clocks": clock_info,
    })


# --------------------------------------------------------------------------------------------
# per-kernel view: every hot kernel alone at the shapes of the workload, against the bound that
# limits it (python bench.py --kernels); not the line the contract asks for, a table beside it
# --------------------------------------------------------------------------------------------
def run_kernels(args, cfg):
    import torch

    from hi2_b200 import _lib, gptq_kernel, ladder_kernel
    from hi2_b200.encode import EFFORT
    from hi2_b200.format import fwht_groups, pack_codes
    from hi2_b200.hessian import HessianStats, inverse_factor, transform_sigma

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    _lib.load()
    pk = peaks()
    g = torch.Generator(device=dev).manual_seed(0)
    # larger than L2, and long enough to write that the host has queued the timed call before it ends
    flush = torch.empty(1 << 30, dtype=torch.uint8, device=dev)

    only = set(filter(None, (args.only or "").split(",")))

    def timed(fn, reps=5, warm=3, cold=True, tag=None):
        if only and tag not in only and tag != "always":  # not asked for: run once (later sections use its results), no timing
            fn()
            return float("nan")
        for _ in range(warm):
            fn()
        samples = []
        for _ in range(reps):
            if cold:
                flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            samples.append(a.elapsed_time(b))
        return sorted(samples)[len(samples) // 2]  # median, ms

    rows_out = []

    def add(name, bound, work, unit, ms, peak, note=""):
        if ms != ms:  # not timed (--only)
            return
        achieved = work / (ms * 1e-3)
        rows_out.append(dict(kernel=name, bound=bound, ms=round(ms, 4), achieved=achieved, unit=unit, peak=peak,
                             frac=achieved / peak if peak else None, note=note))

    # denominators the driver does not measure: cuBLAS fp32 (FFMA) and TF32 products, 8192^3
    a = torch.randn(8192, 8192, device=dev, generator=g)
    b = torch.randn(8192, 8192, device=dev, generator=g)
    torch.backends.cuda.matmul.allow_tf32 = False
    fp32_peak = 2 * 8192**3 / (timed(lambda: torch.matmul(a, b), cold=False, tag="always") * 1e-3) / 1e12
    torch.backends.cuda.matmul.allow_tf32 = True
    tf32_peak = 2 * 8192**3 / (timed(lambda: torch.matmul(a, b), cold=False, tag="always") * 1e-3) / 1e12
    torch.backends.cuda.matmul.allow_tf32 = False
    del a, b
    lane_peak = fp32_peak / 2  # fp32 instructions per second (T lane-ops/s): an FMA is two flops

    k, r_wide, k_wide = 4096, 11008, 11008
    tokens = cfg["tokens"]
    # second moment
    for kk in (k, k_wide):
        x = torch.randn(tokens, kk, device=dev, generator=g).bfloat16()
        h = HessianStats(kk, dev)
        ms = timed(lambda: h.update(x, defer_check=True), reps=5, warm=2, tag="hessian")
        h.check()
        nib, njb = -(-kk // 128), -(-kk // 256)
        tiles = sum(njb - (ib >> 1) for ib in range(nib))
        add(f"hessian_tc K={kk} T={tokens}", "tensor (bf16)", 2.0 * tokens * tiles * 128 * 256 / 1e12, "TFLOP/s", ms,
            pk["tensor_burst"], "issued flops, burst peak (timed alone)")
        sig = h.S / h.n
        if kk == k:
            sigma_small = sig
        del x, h
        # basis change and inverse factor of the same input
        s16 = (torch.rand(kk, device=dev, generator=g) + 0.5).half()
        had = torch.ones(kk // 16, dtype=torch.uint8, device=dev)
        ms = timed(lambda: transform_sigma(sig, s16, had, denom=1.0, return_diag=True), tag="sigma")
        add(f"transform_sigma K={kk}", "hbm", 8.0 * kk * kk / 1e9, "GB/s", ms, pk["hbm"])
        hs = transform_sigma(sig, None, had)
        ms = timed(lambda: inverse_factor(hs, 0.01), reps=3, warm=1, cold=False, tag="factor")
        add(f"inverse_factor K={kk}", "fp32-grade flops", (2.0 / 3.0) * kk**3 / 1e12, "TFLOP/s", ms, fp32_peak,
            "(2/3) K^3 against the cuBLAS fp32 peak; a chain of K/64 dependent leaves")
        if kk == k:
            u_small = inverse_factor(hs, 0.01)
        del sig, hs
    # rotation with the cast and the smoothing multiply fused
    wb = (torch.randn(r_wide, k, device=dev, generator=g) * 0.02).bfloat16()
    had = torch.ones(k // 16, dtype=torch.uint8, device=dev)
    s32 = torch.rand(k, device=dev, generator=g) + 0.5
    ms = timed(lambda: fwht_groups(wb, had, col_scale=s32, out_dtype=torch.float32), tag="rotate")
    add(f"rotate bf16->fp32 {r_wide}x{k}", "hbm", wb.numel() * 6.0 / 1e9, "GB/s", ms, pk["hbm"])
    w = fwht_groups(wb, had, col_scale=s32, out_dtype=torch.float32)
    d = torch.rand(k, device=dev, generator=g) + 0.05
    eff = EFFORT["normal"]
    ops_per_weight = 11 * len(eff["grid"]) ** 2 + 28 * eff["ls"] + 14  # fp32 operations of the reference's search
    for block in (16, 32, 64):
        ms = timed(lambda: ladder_kernel.fit(w, d, eff["grid"], eff["ls"], 4, block), tag="fit")
        add(f"fit_kernel<{block}> INT2 {r_wide}x{k}", "fp32 instruction issue", w.numel() * ops_per_weight / 1e12,
            "Tops/s", ms, lane_peak, f"{ops_per_weight} reference operations per weight; peak = cuBLAS fp32 flops / 2")
    lo, st = ladder_kernel.fit(w, d, eff["grid"], eff["ls"], 4, 32)
    ms = timed(lambda: ladder_kernel.quantize_rows(lo, st, 2, 32, k, w, d, want_codes=True, want_sse=True), tag="row")
    add(f"row_kernel<32> INT2 {r_wide}x{k}", "hbm", (w.numel() * 5.0 + lo.numel() * 10.0) / 1e9, "GB/s", ms, pk["hbm"],
        "reads fp32 rows, writes codes, parameter bytes and sse")
    ms = timed(lambda: ladder_kernel.quantize_rows(lo, st, 2, 32, k, w, d, want_codes=False, want_sse=True), tag="row")
    add(f"row_kernel<32> INT2 {r_wide}x{k}, table pass (no codes)", "hbm", (w.numel() * 4.0 + lo.numel() * 10.0) / 1e9,
        "GB/s", ms, pk["hbm"], "what a table entry costs: reads fp32 rows, writes parameter bytes and sse")
    q = ladder_kernel.quantize_rows(lo, st, 2, 32, k, w, d, want_codes=True, want_decoded=True, ldp=k // 16)
    words = torch.empty(r_wide, k // 16, dtype=torch.int32, device=dev)
    bad = torch.zeros(1, dtype=torch.int32, device=dev)
    ms = timed(lambda: _lib.call("hi2_pack_codes", _lib.ptr(q["codes"]), _lib.ptr(words), r_wide, k, 2, _lib.ptr(bad),
                                 _lib.stream(dev)), tag="pack")
    assert torch.equal(words, pack_codes(q["codes"], 2)) and int(bad.item()) == 0
    add(f"pack_codes INT2 {r_wide}x{k}", "hbm", w.numel() * 1.25 / 1e9, "GB/s", ms, pk["hbm"],
        "the C entry point alone (the Python wrapper also reads the out-of-range flag back)")
    # GPTQ: one 128-column segment and its trailing update, then the whole column loop
    n = r_wide
    wc = w.clone()
    codes = torch.empty(n, k, dtype=torch.uint8, device=dev)
    err1 = torch.empty(n, 128, device=dev)
    rg = torch.zeros(n, dtype=torch.int32, device=dev)
    up = torch.tensor([u_small.data_ptr()], dtype=torch.int64, device=dev)
    blk = (torch.arange(k, device=dev) // 32).to(torch.int32).reshape(1, k)
    nm = torch.tensor([3.0], device=dev)
    ms_blk = timed(lambda: gptq_kernel.gptq_block(wc, 0, 128, err1, codes, q["lo_d"], q["step_d"], rg, up, blk, nm),
                   cold=False, tag="gptq")
    add(f"gptq_block N={n} (128 columns)", "dependent chain", n * 128 * 140.0 / 1e12, "Tops/s", ms_blk, lane_peak,
        "140 reference operations per row and column")
    parts = gptq_kernel.split_tf32_transposed(u_small)
    ms_round = timed(lambda: gptq_kernel.gptq_round_tc(wc, err1, codes, q["lo_d"], q["step_d"], rg, up, blk, nm, None,
                                                        [0, n], [parts]), reps=3, warm=1, cold=False, tag="gptq")
    lazy_flops = float(n) * k * k * (1 - 128.0 / k)
    ms_lazy = ms_round - (k // 128) * ms_blk
    add(f"lazy_tc (all {k // 128 - 1} trailing updates, N={n})", "tensor (3xTF32)", 3 * lazy_flops / 1e12, "TFLOP/s",
        max(ms_lazy, 1e-3), tf32_peak, "three TF32 products per fp32-grade product; time = column loop minus segments")
    if ms_round == ms_round:
        rows_out.append(dict(kernel=f"GPTQ column loop N={n} K={k}", bound="chain + tensor", ms=round(ms_round, 3),
                             achieved=n / (ms_round * 1e-3), unit="rows/s", peak=None, frac=None,
                             note="segments + trailing updates"))
    # refinement: two sweeps over the rows of one 4096-wide matrix (the reference's CLI default for
    # calibrated GPTQ without QAD, hi2/__main__.py:164-172); 2 N K^2 flops for g = e Hs plus 2 N K^2 per sweep
    from hi2_b200.encode import Encoded
    from hi2_b200.refine import refine_groups

    n_ref = 4096
    hs_small = transform_sigma(sigma_small, None, had)
    enc = Encoded(codes[:n_ref].clone(), q["params"][:n_ref], q["consts"][:n_ref], torch.zeros(n_ref, device=dev))
    ms_ref = timed(lambda: refine_groups([(w[:n_ref], enc, 2, 32)], hs_small, 2), reps=3, warm=1, cold=False, tag="refine")
    add(f"refine, 2 sweeps, N={n_ref} K={k} (block kernel + 3xTF32 products)", "tensor (3xTF32) + chain",
        3 * 2.0 * n_ref * k * k * 3 / 1e12, "TFLOP/s", ms_ref, tf32_peak,
        "three TF32 products per fp32-grade product; includes the 32 block-kernel launches per sweep")
    if ms_ref == ms_ref and ms_round == ms_round:
        rows_out.append(dict(kernel=f"refine vs GPTQ column loop (same rows, K={k})", bound="ratio", ms=round(ms_ref, 3),
                             achieved=ms_ref / (ms_round * n_ref / n), unit="x the GPTQ column loop of the same rows",
                             peak=None, frac=None, note="the reference reports about 1.1x fused on its hardware"))
    emit({"kernels": rows_out, "peaks": {"hbm_gbs": pk["hbm"], "bf16_tflops_burst": pk["tensor_burst"],
                                         "bf16_tflops_sustained": pk["tensor"], "fp32_tflops_cublas": fp32_peak,
                                         "tf32_tflops_cublas": tf32_peak, "source": pk["source"]},
          "timing": "CUDA events, median of 3-5 calls after warm-up, a 1 GiB buffer written before each timed call"})


_RESULT = None  # the process's original stdout, kept for the one JSON line


def guard_stdout():
    """stdout carries exactly one JSON line.  Libraries print there too (NCCL writes its version
    banner to file descriptor 1 when NCCL_DEBUG asks for it), so descriptor 1 is pointed at stderr
    for the rest of the process and the line goes to a duplicate of the original."""
    global _RESULT
    sys.stdout.flush()
    _RESULT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(line: dict):
    out = _RESULT if _RESULT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    guard_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg3", choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="whole-model configs: take this many layers instead of all")
    ap.add_argument("--refine-passes", type=int, default=0,
                    help="whole-model configs: sweeps of the +-1 code refinement after GPTQ (the reference's CLI default is 2; "
                         "the headline metric is quoted without)")
    ap.add_argument("--no-config1", action="store_true", help="skip the full CPU run of config 1 in the cpu_baseline leg")
    ap.add_argument("--no-propagate", action="store_true",
                    help="skip the run with the activations produced on the device by layer forwards")
    ap.add_argument("--kernels", action="store_true", help="time every hot kernel alone against its bound")
    ap.add_argument("--only", default="", help="with --kernels: comma-separated sections to time (hessian, sigma, factor, "
                    "rotate, fit, row, pack, gptq, refine); the others run once, untimed, for their results")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.layers and "layers" in cfg:
        cfg["layers"] = args.layers
        cfg["workload"] += f"_first_{args.layers}_layers"
    if args.refine_passes and "layers" in cfg:
        cfg["refine_passes"] = args.refine_passes
        cfg["workload"] += f"_refine_{args.refine_passes}"
    if args.kernels:
        run_kernels(args, cfg)
    elif "moe_layers" in cfg:
        run_moe(args, cfg)
    elif args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
