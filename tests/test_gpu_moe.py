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
