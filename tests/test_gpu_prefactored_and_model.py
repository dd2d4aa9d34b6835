"""The pipelined encode (factors started ahead on side streams) and the whole-model job.

* ``layer.encode`` with ``start_factors`` must give exactly what the synchronous path gives, also
  when the factor is the LAST thing to finish (a wide input with few rows: tiny tables, long
  factorisation) - the column loop has to order itself after the factor on the device;
* a prefactored job belongs to one (input, smoothing vector, flags): a request with another
  transform on the same ``sigma_id`` must not receive it;
* a whole model through the bench's job class: layers batched through the encode, the global
  allocation over all tables, results equal to encoding layer by layer.
"""

import pytest
import torch

from tests.helpers import DEV, activations, gen

pytestmark = pytest.mark.gpu

FIELDS = ("codes", "code_off", "blk_params", "param_off", "row_consts", "row_nbits", "row_block", "had")


def _same(a, b):
    return all(torch.equal(getattr(a, f).cpu(), getattr(b, f).cpu()) for f in FIELDS)


@pytest.mark.parametrize("k,rows,tokens", [(512, 96, 4096), (4096, 16, 8192)])
def test_prefactored_encode_equals_synchronous(k, rows, tokens):
    from hi2_b200 import layer as L
    from hi2_b200.allocate import allocate_global
    from hi2_b200.calibrate import Config

    g = gen(k + rows)
    cfg = Config()
    plan = L.LayerPlan({"a": "x", "b": "x"})
    weights = {"a": (torch.randn(rows, k, generator=g) * 0.02).bfloat16().to(DEV),
               "b": (torch.randn(rows // 2, k, generator=g) * 0.02).bfloat16().to(DEV)}
    x = activations(tokens, k, 3, spread=1.0, dtype=torch.bfloat16).to(DEV)
    shared = L.accumulate({"x": x}, DEV)
    L.finish_statistics(shared, cfg)
    tables = L.tabulate(weights, plan, shared, cfg)
    alloc = allocate_global(list(tables.values()), 3.0)
    want = L.encode(weights, plan, shared, tables, alloc.picks, cfg)
    for release in (False, True):
        torch.cuda.synchronize()
        factors = L.start_factors(shared, cfg, DEV, release_scratch=release)
        got = L.encode(weights, plan, shared, tables, alloc.picks, cfg, factors=factors)  # no sync in between
        for name in weights:
            assert _same(got[name], want[name]), (name, release)


def test_prefactored_job_is_keyed_by_its_transform():
    from hi2_b200.calibrate import Config, EncodeRequest, build_table, encode_many, factor_for
    from hi2_b200.hessian import HessianStats
    from hi2_b200.stats import ColumnStats

    g = gen(11)
    k, r = 256, 48
    cfg = Config()
    w = (torch.randn(r, k, generator=g) * 0.02).half().to(DEV)
    x = activations(4096, k, 12, spread=1.2).to(DEV)
    h = HessianStats(k, DEV)
    h.update(x)
    stats = ColumnStats.from_second_moment(h.S, h.n)
    t_on = build_table("w", w, stats, cfg)  # smoothing vector + all groups rotated
    flags_off = torch.zeros(k // 16, dtype=torch.uint8)
    t_off = build_table("w", w, stats, cfg, transform=(None, flags_off))  # no smoothing, no rotation
    picks = torch.randint(0, 6, (r,), generator=g)
    fac = {"x": factor_for(h.S, h.n, t_on.col_scale, t_on.had, cfg)}  # factor of the FIRST transform only
    reqs = [EncodeRequest(w, stats, t_on, picks, sigma=h.S, sigma_id="x", sigma_n=h.n),
            EncodeRequest(w, stats, t_off, picks, sigma=h.S, sigma_id="x", sigma_n=h.n)]
    got = encode_many(reqs, cfg, factors=fac)
    want = [encode_many([q], cfg)[0] for q in reqs]
    assert _same(got[0], want[0]) and _same(got[1], want[1])
    assert not torch.equal(got[0].codes, got[1].codes)


def test_stream_argument_names_its_device():
    from hi2_b200 import _lib

    s = _lib.stream(torch.device(DEV, torch.cuda.current_device()))
    assert s.index == torch.cuda.current_device() and s._as_parameter_ is not None


def test_whole_model_job_equals_layer_by_layer():
    """bench.ModelJob on a four-layer toy model: one step, then every layer again through
    layer.encode with the same picks."""
    import bench
    from hi2_b200 import layer as L

    cfg = dict(bench.CONFIGS["tiny_model"])
    dev = torch.device(DEV, torch.cuda.current_device())
    job = bench.ModelJob(cfg, 0, 1, dev)
    packed = job.step()
    torch.cuda.synchronize()
    job.collect_stage_times()
    alloc = job.last["alloc"]
    assert alloc.feasible and abs(alloc.bpw - cfg["bpw"]) < 0.02
    assert len(alloc.picks) == cfg["layers"] * 7 and job.rows == cfg["layers"] * job.rows_layer
    assert set(job.gptq) == {512, 1024} and job.hessian_launches == cfg["layers"] * 4
    for l in range(cfg["layers"]):
        shared = L.accumulate(job.inputs, dev)
        L.finish_statistics(shared, job.qcfg)
        tables = L.tabulate(job.weights[l], job.plan, shared, job.qcfg)
        picks = {name: alloc.picks[f"L{l}.{name}"] for name in job.shapes}
        want = L.encode(job.weights[l], job.plan, shared, tables, picks, job.qcfg, to_host=False)
        for name in job.shapes:
            assert _same(packed[l][name], want[name]), (l, name)


def test_propagated_job_runs_the_whole_model():
    """bench.PropagatedJob on the toy model: weights and ids from pinned host memory, activations
    produced by the layer forwards on the device, every Linear tabulated, allocated and encoded."""
    import bench

    cfg = dict(bench.CONFIGS["tiny_model"])
    dev = torch.device(DEV, torch.cuda.current_device())
    job = bench.PropagatedJob(cfg, 0, 1, dev, heads=8, vocab=512)
    packed = job.step()
    torch.cuda.synchronize()
    assert len(packed) == cfg["layers"] * 7 and job.rows == cfg["layers"] * (4 * 512 + 2 * 1024 + 512)
    assert job.last["alloc"].feasible and abs(job.last["alloc"].bpw - cfg["bpw"]) < 0.02
    t = packed["model.layers.3.mlp.down_proj.weight"]
    assert t.shape == (512, 1024) and t.codes.device.type == "cpu" and int(t.code_off[-1]) == t.codes.numel()
    assert job.d2h_bytes() > 0 and job.h2d > 0


def test_whole_model_job_gqa_int8_rule_and_infeasible_target():
    """The config-4 mechanics on a toy model: grouped-query shapes (k/v shorter than q), INT8
    candidates open only to the 1 % most sensitive rows, a target below the format's floor recorded
    as infeasible with every row at INT2 (hi2/allocate.py:248-249), the encode at the feasible one."""
    import bench

    cfg = dict(bench.CONFIGS["tiny_gqa_int8"])
    dev = torch.device(DEV, torch.cuda.current_device())
    job = bench.ModelJob(cfg, 0, 1, dev)
    assert job.shapes["k"] == (128, 512) and len(job.qcfg.candidates) == 8
    packed = job.step()
    torch.cuda.synchronize()
    low = job.last["below_floor"]
    assert low["feasible"] is False and low["bpw"] > cfg["bpw_infeasible"] and low["rows_by_width"][2] == 1.0
    alloc = job.last["alloc"]
    assert alloc.feasible and abs(alloc.bpw - cfg["bpw"]) < 0.02
    share8 = alloc.frac_by_bits[8]
    assert 0.0 <= share8 <= cfg["int8_fraction"] + 1e-3, share8
    rows8 = sum(int((t.row_nbits == 8).sum()) for layer in packed.values() for t in layer.values())
    assert rows8 == round(share8 * job.rows)


def test_int8_rule_closes_all_but_the_most_sensitive_rows():
    from hi2_b200.calibrate import SELECTABLE, TensorTable
    from hi2_b200.layer import keep_int8_for_most_sensitive

    g = gen(5)
    tabs = []
    for i, r in enumerate((300, 700)):
        sse = torch.rand(8, r, generator=g) + 0.1
        sse[6:] *= 0.01  # INT8 is far more accurate
        tabs.append(TensorTable(f"t{i}", (r, 256), torch.ones(16, dtype=torch.uint8), sse.to(DEV), list(SELECTABLE), 1.0 + i, 10))
    before = [t.sse.clone() for t in tabs]
    keep_int8_for_most_sensitive(tabs, 0.01)
    cost = torch.cat([b[3:6].min(0).values / (1.0 + i) for i, b in enumerate(before)])
    top = set(torch.topk(cost, 10).indices.tolist())
    off = 0
    for t, b in zip(tabs, before):
        assert torch.equal(t.sse[:6], b[:6])
        for row in range(b.shape[1]):
            if off + row in top:
                assert torch.equal(t.sse[6:, row], b[6:, row])
            else:
                assert bool((t.sse[6:, row] == b[3:6, row].min()).all())
        off += b.shape[1]


def test_rows_grouped_by_candidate_with_one_read_back():
    """``group_rows``: per request the rows of each candidate in ascending order, candidates in
    order, counts on the host; picks given on the host or on the device; a candidate nobody picked;
    requests with different numbers of candidates; already grouped requests are left alone."""
    from hi2_b200.calibrate import EncodeRequest, TensorTable, group_rows

    g = gen(11)
    reqs = []
    for rows, cands, on_dev in ((257, [(2, 16), (2, 32), (4, 64)], True), (64, [(2, 64), (4, 16)], False),
                                (1000, [(2, 16), (2, 32), (2, 64), (4, 16), (4, 32), (4, 64)], True)):
        picks = torch.randint(0, len(cands), (rows,), generator=g)
        picks[picks == 1] = 0  # candidate 1 is never picked
        w = torch.zeros(rows, 32, device=DEV)
        table = TensorTable("t", (rows, 32), torch.ones(2, dtype=torch.uint8), torch.zeros(len(cands), rows, device=DEV),
                            cands, 0.0, 0)
        reqs.append(EncodeRequest(w, None, table, picks.to(DEV) if on_dev else picks))
    group_rows(reqs)
    for r in reqs:
        order, counts = r.groups
        picks = r.picks.cpu()
        assert counts[: len(r.table.candidates)] == [int((picks == c).sum()) for c in range(len(r.table.candidates))]
        assert sum(counts) == picks.numel() and counts[1] == 0
        want = torch.cat([torch.nonzero(picks == c).flatten() for c in range(len(r.table.candidates))])
        assert torch.equal(order.cpu(), want)
    before = [r.groups for r in reqs]
    group_rows(reqs)
    assert all(a is b for a, b in zip(before, [r.groups for r in reqs]))
