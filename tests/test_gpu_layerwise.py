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
