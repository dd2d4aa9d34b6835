"""Routed-token statistics per expert (hi2/moe.py:152-156, hi2/layerwise.py:231-257): the device
accumulators against the CPU restatement's second moments over the same routed tokens."""

import pytest
import torch

from hi2_b200 import moe
from hi2_b200.hessian import HessianStats
from hi2_b200.stats import ColumnStats
from oracle import ptq_oracle as po
from tests.helpers import activations

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _routing(tokens, experts, top_k, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(tokens, experts, generator=g)
    logits[:, 0] += 2.0  # one popular expert, the others sparse
    return logits.topk(top_k, dim=1).indices


def test_routed_second_moments_match_oracle():
    t, k, e = 3000, 128, 8
    x = activations(t, k, 11, dtype=torch.bfloat16)
    idx = _routing(t, e, 2, 5)
    hess = [HessianStats(k, DEV) for _ in range(e)]
    stats = [ColumnStats(k, DEV) for _ in range(e)]
    moe.accumulate_routed(x.to(DEV), idx.to(DEV), hess, stats)
    assert sum(h.n for h in hess) == 2 * t
    for ei in range(e):
        xe = x[(idx == ei).any(1)]
        o = po.SecondMoment(k)
        o.update(xe)
        assert hess[ei].n == o.n == stats[ei].n
        err = (hess[ei].S.cpu().double() - o.S.double()).norm() / o.S.double().norm()
        assert err < 1e-5  # both sides sum in fp32; the same bar as the dense second-moment tests
        og = po.GroupMoments(k)
        og.update(xe)
        assert (stats[ei].S.cpu() - og.S).norm() / og.S.norm() < 1e-6


def test_top_up_borrows_the_pooled_sum():
    t, k, e = 600, 64, 4
    x = activations(t, k, 3, dtype=torch.float32)
    idx = _routing(t, e, 1, 9)
    names = [f"layers.0.mlp.experts.{i}.gate_proj" for i in range(e)]
    hess = {n: HessianStats(k, DEV) for n in names}
    stats = {n: ColumnStats(k, DEV) for n in names}
    moe.accumulate_routed(x.to(DEV), idx.to(DEV), [hess[n] for n in names], [stats[n] for n in names])
    before = {n: (hess[n].S.clone(), hess[n].n, stats[n].S.clone()) for n in names}
    tot_h = sum(b[0] for b in before.values())
    tot_s = sum(b[2] for b in before.values())
    k_of = {n: k for n in names}
    k_of.update({n.replace("gate_proj", "down_proj"): 2 * k for n in names})
    need = int(2.0 * 2 * k)  # the widest input of the expert sets the floor
    borrowed = moe.top_up(stats, hess, k_of, 2.0)
    assert borrowed == {n for n in names if before[n][1] < need} and borrowed
    for n in names:
        s0, n0, g0 = before[n]
        if n in borrowed:
            fill = (need - n0) / t
            assert torch.equal(hess[n].S, s0 + fill * tot_h) and hess[n].n == need
            assert torch.equal(stats[n].S, g0 + fill * tot_s) and stats[n].n == need
        else:
            assert torch.equal(hess[n].S, s0) and hess[n].n == n0


def test_moe_job_routes_tops_up_and_encodes_per_expert():
    """bench.MoeJob on a toy mixture (8 experts, top-2, a strongly biased router): per-expert
    second moments over the routed tokens only (hi2 tests/test_moe.py:157-181 semantics), starved
    experts topped up with the pooled sums, allocation weighted by token share, every expert encoded."""
    import bench
    from hi2_b200 import moe
    from hi2_b200.hessian import HessianStats

    cfg = dict(bench.CONFIGS["tiny_moe"])
    dev = torch.device(DEV, torch.cuda.current_device())
    job = bench.MoeJob(cfg, 0, 1, dev)
    tokens_of, counts = job.route(0)
    counts = counts.tolist()
    assert sum(counts) == cfg["tokens"] * cfg["top_k"] and min(counts) < max(counts)
    # second moment of one expert = x_e^T x_e over exactly the tokens whose top-k names it
    e = max(range(8), key=lambda i: counts[i])
    off = sum(counts[:e])
    rows = tokens_of[off : off + counts[e]]
    logits = (job.x_in @ job.router[0].T).float() + job.bias[0]
    named = (torch.topk(logits, cfg["top_k"], dim=1).indices == e).any(1).nonzero().squeeze(1)
    assert torch.equal(rows.sort().values, named)
    h = HessianStats(cfg["hidden"], dev)
    h.update(job.x_in.index_select(0, rows))
    xe = job.x_in.index_select(0, named).double()
    ref = xe.T @ xe
    scale = ref.diagonal().clamp_min(1e-30).sqrt()
    assert ((h.S.double() - ref) / (scale[:, None] * scale[None, :])).abs().max().item() < 2e-5
    packed = job.step()
    torch.cuda.synchronize()
    assert len(packed) == cfg["moe_layers"] * 8 * 3
    need = int(2.0 * cfg["hidden"])
    starved = sum(1 for layer in job.last["token_counts"].values() for c in layer if c < need)
    assert job.last["borrowed"] == 2 * starved and starved > 0  # both inputs of a starved expert borrow
    alloc = job.last["alloc"]
    assert alloc.feasible and abs(alloc.bpw - cfg["bpw"]) < 0.02
    share = job.last["share"]
    layer0 = job.last["token_counts"][0]
    mean = sum(layer0) / 8
    for ex in range(8):
        assert abs(share[f"L0.experts.{ex}.down_proj"] - max(layer0[ex] / mean, 0.05) / 8) < 1e-12
    t = packed[(1, "experts.3.down_proj")]
    assert t.shape == (cfg["hidden"], cfg["expert_ffn"]) and int(t.code_off[-1]) == t.codes.numel()


def test_tables_of_a_group_of_experts_equal_tables_one_by_one():
    """``calibrate.build_tables_grouped`` (the stored rows of all experts in one buffer, column weights
    per group of rows, two launches per candidate for the whole group) against ``build_table`` per
    expert: ``sse``, energy, flags, smoothing vector bit for bit; and through ``layer.tabulate`` with
    mixed shapes, where only equal shapes are grouped."""
    import torch

    from hi2_b200 import layer as L
    from hi2_b200.calibrate import Config, build_table, build_tables_grouped
    from tests.helpers import DEV, activations, gen

    g = gen(5)
    cfg = Config(effort="fast")
    n_exp, r, k = 5, 72, 256  # 72 rows: a warp of the search kernel straddles two experts
    acts = {f"e{e}": activations(700 + 50 * e, k, 70 + e, spread=1.0, dtype=torch.bfloat16).to(DEV) for e in range(n_exp)}
    shared = L.accumulate(acts, DEV)
    L.finish_statistics(shared, cfg)
    ws = {f"e{e}": (torch.randn(r, k, generator=g) * 0.03).bfloat16().to(DEV) for e in range(n_exp)}
    items = [(n, ws[n], shared[n].moments, shared[n].transform, 123 + i) for i, n in enumerate(ws)]
    many = build_tables_grouped(items, cfg)
    for (name, w, st, tr, n), got in zip(items, many):
        want = build_table(name, w, st, cfg, transform=tr, n_tokens=n)
        assert got.name == name and got.n_tokens == n and got.shape == want.shape and got.candidates == want.candidates
        assert torch.equal(got.sse, want.sse) and torch.equal(got.energy, want.energy)
        assert torch.equal(got.had, want.had) and torch.equal(got.col_scale, want.col_scale)
        assert got.transform_ref[0] is tr[0] and got.transform_ref[1] is tr[1]
    # through the layer: three shapes, one of them alone in its group
    plan = L.LayerPlan({**{f"a{e}": f"e{e}" for e in range(n_exp)}, **{f"b{e}": f"e{e}" for e in range(2)}, "c": "e0"})
    weights = {**{f"a{e}": ws[f"e{e}"] for e in range(n_exp)},
               **{f"b{e}": (torch.randn(40, k, generator=g) * 0.03).bfloat16().to(DEV) for e in range(2)},
               "c": (torch.randn(24, k, generator=g) * 0.03).float().to(DEV)}
    one = L.tabulate(weights, plan, shared, cfg)
    grouped = L.tabulate(weights, plan, shared, cfg, grouped=True)
    assert list(grouped) == list(one)
    for name in one:
        assert torch.equal(grouped[name].sse, one[name].sse) and torch.equal(grouped[name].energy, one[name].energy), name
