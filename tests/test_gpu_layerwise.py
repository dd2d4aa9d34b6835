"""Calibration propagation on the device against hi2's own ``calibrate_layerwise`` run on the CPU
(tests/golden/layerwise_golden.pt: a two-layer Llama-shaped toy model, fp32): sharing groups, token
counts, second moments of every shared input, and the error tables built from them.  The layer
forward runs on another device than the fixture's, so the comparison is by tolerance (the
reference's own 1-vs-2-device test allows 1e-5 on one host; here 1e-4 on the moments, 2e-3 on
the tables)."""

import pathlib

import pytest
import torch

from tests.helpers import DEV, toy_llama

pytestmark = pytest.mark.gpu
GOLDEN = pathlib.Path(__file__).parent / "golden" / "layerwise_golden.pt"


def _norm_err(a, b):
    s = b.double().diagonal().clamp_min(1e-30).sqrt()
    return ((a.double().cpu() - b.double()) / (s[:, None] * s[None, :])).abs().max().item()


@pytest.fixture(scope="module")
def run():
    from hi2_b200.calibrate import Config
    from hi2_b200.layerwise import DeviceSink, calibrate_layerwise

    want = torch.load(GOLDEN, weights_only=False)
    model, ids = toy_llama()
    model.load_state_dict(want["state"])
    assert torch.equal(ids, want["ids"])
    model = model.to(DEV)
    sink = DeviceSink()
    tables = calibrate_layerwise(model, ids, Config(effort="fast"), exclude=["lm_head|embed"], sink=sink,
                                 log=lambda *_: None, batch=4)
    return model, tables, sink, want


def test_groups_counts_and_second_moments(run):
    _, tables, sink, want = run
    assert sink.groups == want["groups"]  # q/k/v and gate/up share their leader's accumulator
    assert set(tables) == set(want["tables"])
    for name, (s, n) in sink.sigma.items():
        assert n == want["n"][name] == 6 * 48
        assert _norm_err(s, want["sigma"][name]) < 1e-4, name


def test_tables_match_reference(run):
    _, tables, _, want = run
    for name, ref in want["tables"].items():
        t = tables[name]
        assert tuple(t.shape) == tuple(ref["shape"]) and t.n_tokens == ref["n_tokens"]
        assert torch.equal(t.had, ref["had"])
        assert torch.allclose(t.col_scale.cpu().float(), ref["col_scale"].float(), rtol=2e-3)
        assert abs(float(t.energy) - ref["energy"]) <= 2e-3 * ref["energy"]
        assert torch.allclose(t.sse.cpu().sum(1), ref["sse"].sum(1), rtol=2e-3), name


def test_encode_from_the_sink(run):
    """allocate over the propagated tables and encode every Linear from the statistics left in HBM."""
    from hi2_b200.allocate import allocate_global
    from hi2_b200.calibrate import Config
    from hi2_b200.layerwise import encode_layerwise

    model, tables, sink, _ = run
    alloc = allocate_global(list(tables.values()), 4.5)  # 64-wide rows: the per-row overhead alone is 0.8 bpw
    assert alloc.feasible
    packed = encode_layerwise(model, tables, alloc.picks, sink, Config(effort="fast"))
    assert set(packed) == set(tables)
    for name, t in packed.items():
        assert tuple(t.shape) == tuple(tables[name].shape) and int(t.code_off[-1]) == t.codes.numel()


def test_statistics_without_full_second_moment(run):
    """rounding='nearest' keeps only the group moments (summed directly from the activations)."""
    from hi2_b200.calibrate import Config
    from hi2_b200.layerwise import DeviceSink, calibrate_layerwise

    model, tables, _, want = run
    _, ids = toy_llama()
    # the run above propagated in place only its own copy of the hidden states: the model is untouched
    sink = DeviceSink()
    t2 = calibrate_layerwise(model, ids, Config(effort="fast", rounding="nearest"), exclude=["lm_head|embed"],
                             sink=sink, log=lambda *_: None, limit_layers=1)
    assert not sink.sigma and len(t2) == 7
    name = "model.layers.0.mlp.down_proj.weight"
    assert torch.allclose(t2[name].sse.cpu().sum(1), want["tables"][name]["sse"].sum(1), rtol=2e-3)


def test_propagation_through_routed_experts():
    """An OLMoE-shaped toy model with fused expert parameters: unfused into per-expert views, then the
    same propagation; every expert projection gets its own table from the tokens routed to it, gate
    and up of an expert share their accumulator, an expert below the token floor is topped up with
    the layer's pooled sum.  Checked twice: exactly, against what extra hooks on the expert Linears
    see in this very run (the routing of this device), and against hi2's own run on the CPU
    (tests/golden/layerwise_moe_golden.pt) - there by a looser tolerance for the expert inputs, since
    a token whose second and third router scores nearly tie may go to another expert on another
    device (one of 288 did when this was written)."""
    from hi2_b200.calibrate import Config
    from hi2_b200.layerwise import DeviceSink, calibrate_layerwise
    from hi2_b200.moe import expert_parts, unfuse_experts
    from tests.helpers import toy_olmoe

    want = torch.load(GOLDEN.with_name("layerwise_moe_golden.pt"), weights_only=False)
    model, ids = toy_olmoe()
    model.load_state_dict(want["state"])
    assert unfuse_experts(model) == 2
    model = model.to(DEV)
    seen: dict = {}
    hooks = []
    for name, mod in model.named_modules():
        if name.endswith(".gate_proj") and expert_parts(name) is not None:
            hooks.append(mod.register_forward_pre_hook(
                lambda _m, args, key=name + ".weight": seen.setdefault(key, []).append(args[0].detach().double().clone())))
    sink = DeviceSink()
    tables = calibrate_layerwise(model, ids, Config(effort="fast"), exclude=["lm_head|embed"], sink=sink,
                                 log=lambda *_: None, batch=4)
    for h in hooks:
        h.remove()
    assert sink.groups == want["groups"] and set(tables) == set(want["tables"])
    floor = 2 * 64  # expert_min_tokens x the widest input of an expert
    topped_up = 0
    for name, (s, n) in sink.sigma.items():
        if expert_parts(name) is None:  # attention inputs: every token, whatever the routing
            assert n == want["n"][name] == 6 * 48
            assert _norm_err(s, want["sigma"][name]) < (1e-4 if ".layers.0." in name else 2e-2), name
            continue
        own = torch.cat(seen[name]) if name in seen else torch.zeros(0, 64, dtype=torch.float64, device=DEV)
        assert tables[name].n_tokens == own.shape[0] and abs(own.shape[0] - want["tables"][name]["n_tokens"]) <= 3
        if own.shape[0] >= floor:  # exactly the tokens this device routed here
            assert n == own.shape[0]
            assert _norm_err(s, (own.T @ own).cpu()) < 1e-4, name
        else:
            topped_up += 1
            assert n == floor == want["n"][name]
        assert _norm_err(s, want["sigma"][name]) < 5e-2, name
    assert topped_up >= 1
    for name, ref in want["tables"].items():
        t = tables[name]
        assert tuple(t.shape) == tuple(ref["shape"]) and torch.equal(t.had, ref["had"])
        exact = expert_parts(name) is None and ".layers.0." in name
        assert torch.allclose(t.col_scale.cpu().float(), ref["col_scale"].float(), rtol=2e-3 if exact else 5e-2)
        assert torch.allclose(t.sse.cpu().sum(1), ref["sse"].sum(1), rtol=2e-3 if exact else 5e-2), name
