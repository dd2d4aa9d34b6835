"""Refinement sweep on the GPU against the oracle's column loop."""

import pytest
import torch

from oracle import ptq_oracle as po
from tests.helpers import DEV, agreement, correlated_layer

pytestmark = pytest.mark.gpu


def _groups(seed, k=448, rows=(37, 20)):
    w, d, u, _, hs = correlated_layer(sum(rows), k, seed)
    out, r0 = [], 0
    for n, (nb, b) in zip(rows, ((2, 32), (4, 64))):
        part = w[r0 : r0 + n]
        out.append((part, po.gptq_rows(part, d, u, nb, b, "normal"), nb, b))
        r0 += n
    return out, hs


def _to_dev(groups):
    from hi2_b200.encode import Encoded

    return [
        (w.to(DEV), Encoded(e.codes.to(DEV), e.params.to(DEV), e.consts.to(DEV), e.sse.to(DEV)), nb, b)
        for w, e, nb, b in groups
    ]


def test_refine_groups_matches_oracle():
    from hi2_b200.refine import refine_groups

    groups, hs = _groups(11)
    want = po.refine_groups(groups, hs, 2)
    got = refine_groups(_to_dev(groups), hs.to(DEV), 2)
    for g, w_, (_, enc, nb, _) in zip(got, want, groups):
        assert g.dtype == torch.uint8
        assert agreement(g, w_) >= 0.999
        assert int(g.max()) <= 2**nb - 1
        assert (g.cpu().int() - enc.codes.int()).abs().max() <= 2


def test_refine_fixture(golden):
    from hi2_b200.encode import Encoded
    from hi2_b200.refine import refine_groups

    r = golden["refine"]
    groups = [
        (g["w"].to(DEV), Encoded(*(g["enc"][f].to(DEV) for f in ("codes", "params", "consts", "sse"))),
         g["nbits"], g["block"])
        for g in r["groups"]
    ]
    got = refine_groups(groups, r["hs"].to(DEV), 2)
    ok = sum(int((a.cpu() == b).sum()) for a, b in zip(got, r["codes"]))
    assert ok / sum(b.numel() for b in r["codes"]) >= 0.999


def test_sweep_never_raises_the_objective_and_converges():
    from hi2_b200.refine import objective, refine_codes

    groups, hs = _groups(12, k=256, rows=(40, 1))
    w, enc, nb, b = groups[0]
    lo, st = po._decoded(enc.params[..., 0], enc.params[..., 1], enc.consts)
    wd, hd, lod, std = w.to(DEV), hs.to(DEV), lo.to(DEV), st.to(DEV)
    c0 = enc.codes.to(DEV)
    before = objective(wd, c0, lod, std, hd, b)
    c1 = refine_codes(wd, c0, lod, std, hd, nb, b, 1)
    after1 = objective(wd, c1, lod, std, hd, b)
    assert after1 <= before * (1 + 1e-6)
    assert (c1.int() - c0.int()).abs().max() <= 1
    c9 = refine_codes(wd, c0, lod, std, hd, nb, b, 50)  # runs until a sweep moves nothing
    again = refine_codes(wd, c9, lod, std, hd, nb, b, 1)
    assert torch.equal(again, c9)
    assert objective(wd, c9, lod, std, hd, b) <= after1 * (1 + 1e-6)
    assert abs(before - po.hessian_objective(w, enc.codes, lo, st, hs, b)) <= 1e-4 * before


def test_refine_block_entry_point():
    """The per-block entry point with the reference's buffer contract; rows and columns that do
    not fill a thread block or a 128-column block."""
    from hi2_b200 import refine_kernel

    g = torch.Generator().manual_seed(4)
    n, k, b0, length = 37, 192, 128, 64
    a = torch.randn(k, k, generator=g)
    hs = (a @ a.T / k).to(DEV).contiguous()
    c = torch.randint(0, 4, (n, k), generator=g).float().to(DEV)
    lo = (torch.randn(n, k, generator=g) * 0.1).half().float().to(DEV)
    st = (torch.rand(n, k, generator=g) * 0.2).half().float().to(DEV)
    st[:, 130] = 0.0
    top = torch.full((n,), 3.0, device=DEV)
    gfull = torch.randn(n, k, generator=g).to(DEV)
    gb = gfull[:, b0 : b0 + length].contiguous()
    dwb = torch.full((n, length), 7.0, device=DEV)
    c_new = c.clone()
    refine_kernel.refine_block(gb, c_new, lo, st, top, hs, b0, length, dwb)
    # oracle: the same block by the plain loop
    cc, gg = c.cpu().clone(), gb.cpu().clone()
    hs_c, lo_c, st_c = hs.cpu(), lo.cpu(), st.cpu()
    moved = torch.zeros(n, length)
    for i in range(length):
        j = b0 + i
        cur = (lo_c[:, j] + cc[:, j] * st_c[:, j]).half().float()
        best = torch.full((n,), -float("inf"))
        pick = torch.zeros(n)
        dws = torch.zeros(n)
        for delta in (1.0, -1.0):
            cand = cc[:, j] + delta
            dw = (lo_c[:, j] + cand * st_c[:, j]).half().float() - cur
            ok = (cand >= 0) & (cand <= 3) & (st_c[:, j] > 0)
            gain = torch.where(ok, -(2 * dw * gg[:, i] + dw * dw * hs_c[j, j]), torch.tensor(-float("inf")))
            better = gain > best
            best = torch.where(better, gain, best)
            pick = torch.where(better, torch.tensor(delta), pick)
            dws = torch.where(better, dw, dws)
        take = best > 0
        cc[:, j] += torch.where(take, pick, torch.tensor(0.0))
        dwj = torch.where(take, dws, torch.tensor(0.0))
        moved[:, i] = dwj
        gg += dwj[:, None] * hs_c[j, b0 : b0 + length][None, :]
    assert torch.equal(c_new.cpu(), cc)
    assert torch.equal(dwb.cpu(), moved)
    assert torch.equal(c_new[:, :b0], c[:, :b0])


def test_refine_with_tensor_core_products():
    """K = 1024: the sweep's products g = e Hs and g += dw Hs[b0:b1] run as three TF32 tcgen05
    products; codes against the oracle's fp32 column loop, and the general product entry point
    against an fp64 product."""
    from hi2_b200 import refine_kernel
    from hi2_b200.refine import refine_groups

    groups, hs = _groups(23, k=1024, rows=(150, 70))
    want = po.refine_groups(groups, hs, 2)
    got = refine_groups(_to_dev(groups), hs.to(DEV), 2)
    for g, w_ in zip(got, want):
        assert agreement(g, w_) >= 0.999, agreement(g, w_)
    gen_ = torch.Generator().manual_seed(5)
    a = torch.randn(333, 1024, generator=gen_)
    b = torch.randn(517, 1024, generator=gen_)
    out = torch.full((333, 520), 7.0, device=DEV)  # a view with a wider leading dimension
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    view = out[:, :517]
    refine_kernel.gemm_tc(refine_kernel.split_tf32(a.to(DEV)), refine_kernel.split_tf32(b.to(DEV)), view, status)
    ref = a.double() @ b.double().T
    assert int(status.item()) == 0 and bool((out[:, 517:] == 7.0).all())
    assert ((view.double().cpu() - ref).abs().max() / ref.abs().max()).item() < 3e-6
    refine_kernel.gemm_tc(refine_kernel.split_tf32(a.to(DEV)), refine_kernel.split_tf32(b.to(DEV)), view, status,
                          accumulate=True)
    assert ((view.double().cpu() - 2 * ref).abs().max() / ref.abs().max()).item() < 6e-6


def test_block_kernel_mappings_agree():
    """The block entry point maps a lane to a row when the rows fill the SMs (>= 148 x 64) and a warp
    to a row below that: both must give the same codes and the same dw, bit for bit."""
    from hi2_b200 import refine_kernel

    g_ = torch.Generator().manual_seed(9)
    n, k, b0, length = 148 * 64 + 37, 256, 128, 128
    x = torch.randn(1024, k, generator=g_)
    hs = (x.T @ x / 1024).to(DEV).contiguous()
    c = torch.randint(0, 4, (n, k), generator=g_).float().to(DEV)
    lo = (torch.randn(n, k // 32, generator=g_) * 0.1).repeat_interleave(32, 1).to(DEV).contiguous()
    st = (torch.rand(n, k // 32, generator=g_) * 0.05 + 0.01).repeat_interleave(32, 1).to(DEV).contiguous()
    st[5] = 0.0  # a row that cannot move
    top = torch.full((n,), 3.0, device=DEV)
    gb = torch.randn(n, length, generator=g_).to(DEV) * 0.02
    outs = []
    for parts in ([slice(0, n)], [slice(0, 5000), slice(5000, n)]):  # one launch with a lane per row; two with a warp per row
        cc, dw = c.clone(), torch.zeros(n, length, device=DEV)
        for s in parts:
            cs, ds = cc[s].contiguous(), torch.empty(s.stop - s.start, length, device=DEV)
            refine_kernel.refine_block(gb[s].contiguous(), cs, lo[s].contiguous(), st[s].contiguous(), top[s].contiguous(),
                                       hs, b0, length, ds)
            cc[s], dw[s] = cs, ds
        outs.append((cc, dw))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert bool((outs[0][0] != c).any()) and torch.equal(outs[0][0][5], c[5])


def test_refinement_of_tensors_side_by_side_equals_one_by_one():
    """``encode_many`` with refinement: tensors that read the same input share one column loop, the
    loops of different inputs run on side streams with nothing read back in between.  Rows are
    refined independently of each other, so the result must equal encoding every tensor alone."""
    from hi2_b200 import layer as L
    from hi2_b200.allocate import allocate_global
    from hi2_b200.calibrate import Config, EncodeRequest, encode_many
    from tests.helpers import activations, gen

    g = gen(31)
    cfg = Config(effort="fast", refine_passes=2)
    plan = L.LayerPlan({"a": "x", "b": "x", "c": "y"})
    shapes = {"a": (96, 512), "b": (40, 512), "c": (64, 1024)}
    weights = {n: (torch.randn(r, k, generator=g) * 0.02).bfloat16().to(DEV) for n, (r, k) in shapes.items()}
    acts = {"x": activations(4096, 512, 5, spread=1.0, dtype=torch.bfloat16).to(DEV),
            "y": activations(4096, 1024, 6, spread=1.0, dtype=torch.bfloat16).to(DEV)}
    shared = L.accumulate(acts, DEV)
    L.finish_statistics(shared, cfg)
    tables = L.tabulate(weights, plan, shared, cfg)
    picks = allocate_global(list(tables.values()), 3.0).picks

    def request(n):
        s = shared[plan.reads[n]]
        return EncodeRequest(weights[n], s.moments, tables[n], picks[n], sigma=s.hessian.S, sigma_id=s.name,
                             sigma_n=s.hessian.n)

    together = encode_many([request(n) for n in shapes], cfg)
    alone = [encode_many([request(n)], cfg)[0] for n in shapes]
    plain = encode_many([request(n) for n in shapes], Config(effort="fast"))
    for t, u, p in zip(together, alone, plain):
        for f in ("codes", "blk_params", "row_consts", "row_nbits", "row_block", "code_off", "param_off"):
            assert torch.equal(getattr(t, f), getattr(u, f)), f
        assert torch.equal(t.blk_params, p.blk_params)  # ladders are never touched
    assert any(not torch.equal(t.codes, p.codes) for t, p in zip(together, plain))  # the sweeps did move codes


@pytest.mark.parametrize("n", [37, 148 * 64 + 5])
def test_block_in_place_equals_block_then_split(n):
    """The folded entry point (slice of g read where it lies, changes written as TF32 parts) against
    the plain one followed by the split, for both row mappings: same codes, same parts."""
    from hi2_b200 import refine_kernel

    g = torch.Generator().manual_seed(n)
    k, b0, length = 384, 128, 128
    a = torch.randn(k, k, generator=g)
    hs = (a @ a.T / k).to(DEV).contiguous()
    c = torch.randint(0, 16, (n, k), generator=g).float().to(DEV)
    lo = (torch.randn(n, k, generator=g) * 0.1).half().float().to(DEV)
    st = (torch.rand(n, k, generator=g) * 0.05).half().float().to(DEV)
    top = torch.full((n,), 15.0, device=DEV)
    gfull = torch.randn(n, k, generator=g).to(DEV)
    c1, c2 = c.clone(), c.clone()
    dwb = torch.empty(n, length, device=DEV)
    refine_kernel.refine_block(gfull[:, b0 : b0 + length].contiguous(), c1, lo, st, top, hs, b0, length, dwb)
    want = refine_kernel.split_tf32(dwb)
    parts = torch.full((2, n, length), 7.0, device=DEV)
    refine_kernel.refine_block_in_place(gfull, c2, lo, st, top, hs, b0, length, parts)
    assert torch.equal(c1, c2) and torch.equal(parts, want)
    assert bool((dwb != 0).any())


def test_grouped_updates_of_the_sweep_against_the_oracle(monkeypatch):
    """Tensors with many rows bring g up to date lazily, in groups of four blocks (near columns after
    every block, far columns once per group, the group's own columns for the next sweep): forced
    here on a small case whose width is no multiple of the group (1152 = 2 groups + 1 block), against
    the oracle's fp32 column loop and against the block-by-block update."""
    from hi2_b200 import refine
    from hi2_b200.refine import refine_groups

    groups, hs = _groups(29, k=1152, rows=(150, 70))
    want = po.refine_groups(groups, hs, 2)
    plain = refine_groups(_to_dev(groups), hs.to(DEV), 2)
    monkeypatch.setattr(refine, "GROUP_MIN_ELEMS", 0)
    got = refine_groups(_to_dev(groups), hs.to(DEV), 2)
    for g, w_, p in zip(got, want, plain):
        assert agreement(g, w_) >= 0.999, agreement(g, w_)
        assert agreement(g, p.cpu()) >= 0.9995
