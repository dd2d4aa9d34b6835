"""No GPU needed: the library loads and exports what the header declares, the host logic of the
multi-GPU plan is right (two gloo ranks), and the package refuses CPU tensors."""

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "hi2_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hi2_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from hi2_b200 import _lib
    from hi2_b200.build import build

    build()
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), n
        assert n in _lib.SIGNATURES, f"{n} declared in the header but not bound in _lib.py"
    assert set(_lib.SIGNATURES) <= set(names)
    assert lib.hi2_abi_version() == 1


def test_argument_checks_need_no_device():
    """Bad shapes are refused before anything is launched."""
    from hi2_b200 import _lib

    lib = _lib.load()
    assert lib.hi2_rotate_groups(None, 0, None, 0, None, None, 4, 24, None) == _lib.ERR_ARG
    assert b"multiple of 16" in lib.hi2_last_error()
    assert lib.hi2_pack_codes(None, None, 1, 15, 2, None, None) == _lib.ERR_ARG
    assert lib.hi2_gptq_lazy_update(None, 0, 128, 0, 128, None, None, None) == _lib.OK
    assert lib.hi2_inverse_factor_workspace_bytes(1024) == 1024 * 1024 * 8 + 256
    assert lib.hi2_inverse_factor_workspace_bytes(4096) == 4096 * 4096 * 8 + 4 * 2048 * 2048 * 4 + 256
    assert lib.hi2_hessian_workspace_bytes(100, 64, _lib.BF16) == 0  # small: FMA path, no scratch
    need = lib.hi2_hessian_workspace_bytes(262144, 4096, _lib.BF16)
    assert need > 0 and need % 4 == 0


def test_cpu_tensors_are_refused_everywhere():
    from hi2_b200.encode import encode_rows
    from hi2_b200.format import fwht_groups, pack_codes
    from hi2_b200.hessian import HessianStats, inverse_factor, transform_sigma

    with pytest.raises(RuntimeError):
        fwht_groups(torch.zeros(2, 32), torch.ones(2))
    with pytest.raises(RuntimeError):
        pack_codes(torch.zeros(2, 32, dtype=torch.uint8), 2)
    with pytest.raises(RuntimeError):
        encode_rows(torch.zeros(2, 32), torch.ones(32), 2, 16)
    with pytest.raises(RuntimeError):
        transform_sigma(torch.eye(32), None, torch.ones(2))
    with pytest.raises(RuntimeError):
        inverse_factor(torch.eye(32))
    h = HessianStats(32, "cpu")
    with pytest.raises((RuntimeError, ValueError)):
        h.update(torch.zeros(4, 32))


def test_token_shards_and_owners():
    from hi2_b200 import dist as hd

    for tokens, world in ((10, 4), (262144, 8), (3, 8)):
        spans = [hd.token_shard(tokens, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == tokens
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    assert [hd.owner_of(i, 4) for i in range(6)] == [0, 1, 2, 3, 0, 1]


WORKER = r"""
import os, sys, torch
sys.path.insert(0, os.environ["HI2_ROOT"])
from hi2_b200 import dist as hd
rank, world, dev = hd.init_from_env("cpu", timeout_s=60)
k, tokens = 32, 101
g = torch.Generator().manual_seed(0)
x = torch.randn(tokens, k, generator=g)
lo, hi = hd.token_shard(tokens)
part = x[lo:hi]
full = x.T @ x
for owner in range(world):
    s = part.T @ part
    n, _ = hd.reduce_second_moment(s, part.shape[0], owner)
    assert n == tokens
    if rank == owner:
        assert torch.allclose(s, full, rtol=1e-5, atol=1e-4), (s - full).abs().max()
s = part.T @ part
assert hd.all_reduce_second_moment(s, part.shape[0]) == tokens
assert torch.allclose(s, full, rtol=1e-5, atol=1e-4)
n, _ = hd.reduce_second_moment(part.T @ part, part.shape[0], 0, n_total=tokens)  # no count exchange
assert n == tokens
# one input of `world` units, unit r owned by rank r: every rank's partial sums as one stack
units = [torch.randn(tokens, k, generator=g) for _ in range(world)]
stack = torch.stack([u[lo:hi].T @ u[lo:hi] for u in units])
own, work = hd.reduce_scatter_second_moments(stack, async_op=True)
work.wait()
assert torch.allclose(own, units[rank].T @ units[rank], rtol=1e-5, atol=1e-4)
tabs = hd.gather_tables([{"name": f"r{rank}", "sse": torch.full((2, 3), float(rank))}])
assert [t["name"] for t in tabs] == [f"r{i}" for i in range(world)]
from types import SimpleNamespace as NS
local = [NS(name=f"r{rank}.a", shape=(3 + rank, 64), candidates=[(2, 16), (4, 16)], energy=1.0 + rank, n_tokens=5,
            col_scale=None if rank else torch.ones(64), sse=torch.full((2, 3 + rank), float(rank))),
         NS(name=f"r{rank}.b", shape=(2, 32), candidates=[(2, 16)], energy=2.0, n_tokens=5, col_scale=None,
            sse=torch.full((1, 2), 10.0 + rank))]
every = hd.gather_error_tables(local, lambda **kw: NS(**kw))
assert [t.name for t in every] == ["r0.a", "r0.b", "r1.a", "r1.b"]
assert every[2 * rank] is local[0]
for r in range(world):
    a, b = every[2 * r], every[2 * r + 1]
    assert tuple(a.sse.shape) == (2, 3 + r) and bool((a.sse == float(r)).all()) and a.energy == 1.0 + r
    assert tuple(b.sse.shape) == (1, 2) and bool((b.sse == 10.0 + r).all())
    assert (a.col_scale is not None) == (r == 0) and b.col_scale is None
# the same tables through the fixed-layout gather: no metadata exchange, one all_gather
specs = [(r, f"r{r}.{x}", (3 + r, 64) if x == "a" else (2, 32), [(2, 16), (4, 16)] if x == "a" else [(2, 16)], 5,
          x == "a" and r == 0) for r in range(world) for x in "ab"]
every = hd.gather_tables_known_layout(local, specs, lambda **kw: NS(**kw))
assert [t.name for t in every] == ["r0.a", "r0.b", "r1.a", "r1.b"]
assert every[2 * rank] is local[0] and every[2 * rank + 1] is local[1]
for r in range(world):
    a, b = every[2 * r], every[2 * r + 1]
    assert tuple(a.sse.shape) == (2, 3 + r) and bool((a.sse == float(r)).all()) and float(a.energy) == 1.0 + r
    assert tuple(b.sse.shape) == (1, 2) and bool((b.sse == 10.0 + r).all()) and float(b.energy) == 2.0
    assert (a.col_scale is not None) == (r == 0) and b.col_scale is None
# layers interleaved over the ranks (layer l on rank l mod world), as a whole-model job lays them out
specs = [(l % world, f"L{l}", (2, 16), [(2, 16)], 7, False) for l in range(4)]
mine = [NS(name=f"L{l}", shape=(2, 16), candidates=[(2, 16)], energy=float(l), n_tokens=7, col_scale=None,
           sse=torch.full((1, 2), float(l))) for l in range(4) if l % world == rank]
every = hd.gather_tables_known_layout(mine, specs, lambda **kw: NS(**kw))
assert [t.name for t in every] == ["L0", "L1", "L2", "L3"]
assert all(float(t.energy) == float(l) and bool((t.sse == float(l)).all()) for l, t in enumerate(every))
hd.barrier()
print("ok", rank)
"""


def test_two_gloo_ranks_reduce_and_gather(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, HI2_ROOT=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT="29631",
               WORLD_SIZE="2", CUDA_VISIBLE_DEVICES="")
    procs = [
        subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        for r in range(2)
    ]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        assert "ok" in o


def test_expert_names_and_allocation_weights():
    """hi2/moe.py:31-56, 188-207 (tests/test_moe.py:236-250 checks the same split)."""
    from types import SimpleNamespace

    from hi2_b200 import moe

    n = "model.layers.3.mlp.experts.12.up_proj.weight"
    assert moe.expert_parts(n) == ("model.layers.3.mlp.experts", 12, "up_proj")
    assert moe.group_key(n) == "model.layers.3.mlp.experts.*.up_proj"
    assert moe.sibling_leader(n) == "model.layers.3.mlp.experts.12.gate_proj"
    assert moe.expert_parts("model.layers.3.mlp.gate.weight") is None
    assert moe.sibling_leader("model.layers.3.mlp.experts.12.down_proj") is None
    tables = {f"l.experts.{e}.down_proj": SimpleNamespace(n_tokens=c)
              for e, c in enumerate([300, 100, 0, 0])}
    tables["l.attn.q_proj"] = SimpleNamespace(n_tokens=400)
    w = moe.expert_weights(tables)
    assert "l.attn.q_proj" not in w
    assert w["l.experts.0.down_proj"] == 3.0 / 4 and w["l.experts.1.down_proj"] == 1.0 / 4
    assert w["l.experts.2.down_proj"] == 0.05 / 4
    own, need = moe.blend(torch.ones(2, 2), 10, torch.full((2, 2), 8.0), 40, 30)
    assert need == 30 and torch.equal(own, torch.full((2, 2), 5.0))


def test_host_side_helpers_need_no_device():
    """Argument checks that run before any kernel is launched."""
    from hi2_b200.hessian import HessianStats

    store = torch.ones(3, 8, 8)
    h = HessianStats(8, "cpu", out=store[1])
    assert h.S.data_ptr() == store[1].data_ptr() and not h.S.any() and bool(store[0].all())
    with pytest.raises(ValueError):
        HessianStats(8, "cpu", out=torch.zeros(8, 4))
    with pytest.raises(ValueError):
        HessianStats(8, "cpu", out=torch.zeros(8, 8, dtype=torch.float64))
    with pytest.raises(RuntimeError):
        h.update(torch.zeros(4, 8))  # no CPU path


def test_checkpoint_names_and_batches():
    """hi2/checkpoint.py:142-157 tensor names and :234-247 batching under a byte budget (host only)."""
    from types import SimpleNamespace

    from hi2_b200.checkpoint import batches, from_tensors, to_tensors
    from hi2_b200.format import FIELDS, HI2Tensor

    t = HI2Tensor(codes=torch.arange(8, dtype=torch.int32), code_off=torch.tensor([0, 4, 8], dtype=torch.int32),
                  blk_params=torch.zeros(16, dtype=torch.uint8), param_off=torch.tensor([0, 4, 8], dtype=torch.int32),
                  row_consts=torch.zeros(2, 3, dtype=torch.float16), row_nbits=torch.tensor([2, 2], dtype=torch.uint8),
                  row_block=torch.tensor([16, 16], dtype=torch.uint8), had=torch.ones(4, dtype=torch.uint8), shape=(2, 64),
                  col_scale=torch.ones(64, dtype=torch.float16))
    d = to_tensors(t, "model.layers.0.mlp.up_proj")
    assert set(d) == {f"model.layers.0.mlp.up_proj.hi2_{f}" for f in FIELDS} | {"model.layers.0.mlp.up_proj.hi2_col_scale"}
    back = from_tensors(d, "model.layers.0.mlp.up_proj")
    assert back.shape == (2, 64) and torch.equal(back.codes, t.codes) and back.col_scale is not None
    tables = {f"t{i}": SimpleNamespace(shape=(100, 256)) for i in range(5)}
    one = 4 * (256 * 256 + 3 * 100 * 256)
    assert [len(g) for g in batches(list(tables), tables, 2 * one)] == [2, 2, 1]
    assert [len(g) for g in batches(list(tables), tables, 1)] == [1] * 5


def test_install_wires_an_unmodified_hi2():
    """With a hi2 checkout importable (the build container has one; elsewhere the test is skipped),
    ``install()`` must put the replacements under hi2's module names BEFORE hi2.calibrate binds them,
    so that hi2's own ``build_table`` ends up in THIS package's ``encode_rows`` - which, on a machine
    without a GPU, refuses the CPU tensors it is given (there is no CPU path)."""
    import importlib
    import subprocess
    import sys

    ref = str(ROOT.parent / "reference")
    if not (ROOT.parent / "reference" / "hi2" / "calibrate.py").exists():
        pytest.skip("no hi2 checkout beside the repository")
    code = f"""
import sys
sys.path[:0] = [{str(ROOT)!r}, {ref!r}]
import torch
import hi2_b200.install as inst
done = inst.install()
assert "hi2.stats" in done and "hi2.format.assemble" in done
import hi2.calibrate as cal, hi2.encode, hi2.hessian, hi2.stats, hi2.format
import hi2_b200.encode, hi2_b200.hessian, hi2_b200.stats, hi2_b200.format
assert hi2.encode is hi2_b200.encode and hi2.hessian is hi2_b200.hessian and hi2.stats is hi2_b200.stats
assert cal.encode_rows is hi2_b200.encode.encode_rows and cal.ColumnStats is hi2_b200.stats.ColumnStats
assert hi2.format.fwht_groups is hi2_b200.format.fwht_groups and cal.fwht_groups is hi2_b200.format.fwht_groups
from hi2.executor import Executor
try:
    cal.build_table("w", torch.randn(8, 64), None, cal.Config(), Executor("cpu"))
except RuntimeError as e:
    assert "CUDA devices only" in str(e), e
else:
    raise SystemExit("hi2.calibrate.build_table did not reach the replaced kernels")
try:
    inst.install()
except RuntimeError as e:
    assert "before" in str(e)
else:
    raise SystemExit("a late install() was accepted")
print("wired")
"""
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "wired" in out.stdout, out.stdout + out.stderr


STALL_WORKER = """
import os, sys, time, datetime
sys.path.insert(0, os.environ["HI2_ROOT"])
import torch
import torch.distributed as dist
from hi2_b200 import dist as hd
rank, world, device = hd.init_from_env("cpu", timeout_s=4.0)
s = torch.ones(8, 8)
hd.reduce_second_moment(s, 3, 0, n_total=6)           # a step both ranks take
if rank == 1:
    time.sleep(30)                                     # a rank that stops answering between steps
    sys.exit(0)
t0 = time.time()
try:
    hd.reduce_second_moment(s, 3, 0, n_total=6)        # the survivor's next collective
    dist.barrier()
except Exception as e:                                 # the process-group timeout ends it with an error
    print("collective failed after %.1f s: %s" % (time.time() - t0, type(e).__name__))
    os._exit(7)
print("no error")
"""


def test_a_stalled_rank_ends_the_others_collective_by_timeout(tmp_path):
    """Failure detection without a GPU: one of two gloo ranks stops answering between steps; the
    other's next collective must end with an error within the process-group timeout that
    ``init_from_env(timeout_s=...)`` sets, not hang."""
    import time

    script = tmp_path / "stall.py"
    script.write_text(STALL_WORKER)
    env = dict(os.environ, HI2_ROOT=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT="29641", WORLD_SIZE="2",
               CUDA_VISIBLE_DEVICES="")
    t0 = time.time()
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    out0 = procs[0].communicate(timeout=120)[0]
    took = time.time() - t0
    procs[1].kill()
    procs[1].communicate()
    assert procs[0].returncode == 7 and "collective failed" in out0, out0
    assert took < 60, took


def test_stacked_expert_layout_against_the_reference_fixture():
    """``stack.build_stack`` / ``split_stack`` and the naming rules against what hi2's own functions
    made of the same packed tensors (``tests/golden/stack_golden.pt``): every array byte for byte,
    the inverse, and the refusals."""
    from hi2_b200 import stack
    from hi2_b200.format import FIELDS, HI2Tensor

    gold = torch.load(ROOT / "tests" / "golden" / "stack_golden.pt")

    def tensor(rec):
        return HI2Tensor(**rec["fields"], shape=tuple(rec["shape"]), col_scale=rec["col_scale"])

    for group in ("gate_up", "down"):
        experts = [[tensor(p) for p in parts] for parts in gold[group]["experts"]]
        want = gold[group]["stack"]
        got = stack.build_stack(experts)
        assert set(got) == set(want) and stack.GROUPS[group] == tuple(gold[group]["parts"])
        for f in want:
            assert got[f].dtype == want[f].dtype and torch.equal(got[f], want[f]), (group, f)
        back = stack.split_stack(got, len(experts[0]))
        for parts, again in zip(experts, back):
            for a, b in zip(parts, again):
                assert a.shape == b.shape and all(torch.equal(getattr(a, f), getattr(b, f)) for f in FIELDS)
                assert (a.col_scale is None) == (b.col_scale is None)
                assert a.col_scale is None or torch.equal(a.col_scale, b.col_scale)
    names = gold["names"]
    single, stacked = stack.hi2_bases(names["names"])
    assert single == names["single"] and stacked == names["stacked"]
    assert stack.stack_groups(single) == names["groups"]
    assert stack.hi2_bases([f"a.experts.gate_up.hi2_{f}" for f in (*FIELDS, stack.MARK)]) == ([], ["a.experts.gate_up"])
    # refusals: parts of one expert with different flags, smoothing for some experts only, unequal K
    experts = [[tensor(p) for p in parts] for parts in gold["gate_up"]["experts"]]
    experts[1][1].had = 1 - experts[1][1].had
    with pytest.raises(stack.StackError):
        stack.build_stack(experts)
    experts = [[tensor(p) for p in parts] for parts in gold["gate_up"]["experts"]]
    for p in experts[2]:
        p.col_scale = None
    with pytest.raises(stack.StackError):
        stack.build_stack(experts)
    with pytest.raises(stack.StackError):
        stack.build_stack([])
    # an incomplete group (expert 1 lacks up_proj) is not offered for stacking
    some = [n for n in single if not n.endswith("experts.1.up_proj")]
    assert "model.layers.0.mlp.experts.gate_up" not in stack.stack_groups(some)


def test_expert_views_run_the_fused_experts_forward():
    """``moe.unfuse_experts`` on an OLMoE-shaped toy model (fused 3-D expert parameters): the model's
    output is unchanged (and equals what the fixture's generator saw before it unfused), every expert
    projection becomes a Linear over a slice of the fused parameter (no copy), and gate and up of an
    expert are handed one and the same tensor."""
    from hi2_b200 import moe
    from tests.helpers import toy_olmoe

    gold = torch.load(ROOT / "tests" / "golden" / "layerwise_moe_golden.pt", weights_only=False)
    model, ids = toy_olmoe()
    model.load_state_dict(gold["state"])
    assert torch.equal(ids, gold["ids"])
    fused = model.model.layers[0].mlp.experts
    assert moe.is_fused_experts(fused) and not moe.is_fused_experts(model.model.layers[0].mlp)
    with torch.no_grad():
        before = model(ids[:2], use_cache=False).logits
    assert torch.equal(before, gold["logits"])
    assert moe.unfuse_experts(model) == 2 and moe.unfuse_experts(model) == 0
    views = model.model.layers[0].mlp.experts
    assert len(views) == 4 and views[3].down_proj.weight.data_ptr() == fused.down_proj[3].data_ptr()
    assert views[1].up_proj.weight.data_ptr() == fused.gate_up_proj[1, 32:].data_ptr()
    seen = {}
    hooks = [views[e].get_submodule(p).register_forward_pre_hook(
        lambda _m, args, key=(e, p): seen.setdefault(key, []).append((args[0].data_ptr(), tuple(args[0].shape))))
        for e in range(4) for p in ("gate_proj", "up_proj")]
    with torch.no_grad():
        after = model(ids[:2], use_cache=False).logits
    for h in hooks:
        h.remove()
    assert torch.equal(after, before)
    assert all(seen[(e, "gate_proj")] == seen[(e, "up_proj")] for e in range(4) if (e, "gate_proj") in seen)
    names = [n for n, _ in model.named_parameters() if ".experts." in n]
    assert "model.layers.1.mlp.experts.2.up_proj.weight" in names and moe.expert_parts(names[0]) is not None


def test_bit_accounting_and_table_restriction():
    """``format.block_bits_per_weight / metadata_bits / tensor_bpw`` on hand-made tensors (and against
    hi2's own functions when a checkout is beside the repository), ``allocate.restrict / force_int8``
    on tables."""
    from hi2_b200 import allocate, format as fmt
    from hi2_b200.calibrate import TensorTable

    assert fmt.block_bits_per_weight(2, 64) == 2.25 and fmt.block_bits_per_weight(4, 16) == 5.0
    nb = torch.tensor([2, 2, 4, 8], dtype=torch.uint8)
    bl = torch.tensor([16, 64, 32, 32], dtype=torch.uint8)
    same = torch.ones(8, dtype=torch.uint8)
    mixed = torch.tensor([1, 0, 1, 1, 0, 0, 1, 1], dtype=torch.uint8)
    assert fmt.metadata_bits(nb[:2], bl[:1].repeat(2), same) == 1  # one width, one block size, uniform flags
    assert fmt.metadata_bits(nb, bl, same) == 1 + 4 * 2 + 4 * 2  # three widths: 2 bits a row; blocks differ: 2 more
    assert fmt.metadata_bits(nb[1:3], bl[:1].repeat(2), mixed) == 8 + 2 * 1
    k = 128
    t = fmt.HI2Tensor(codes=torch.zeros(0, dtype=torch.int32), code_off=torch.zeros(5, dtype=torch.int32),
                      blk_params=torch.zeros(0, dtype=torch.uint8), param_off=torch.zeros(5, dtype=torch.int32),
                      row_consts=torch.zeros(4, 3, dtype=torch.float16), row_nbits=nb, row_block=bl, had=mixed,
                      shape=(4, k), col_scale=torch.ones(k, dtype=torch.float16))
    payload = sum(int(n) * k + 16 * k // int(b) for n, b in zip(nb, bl))
    want = (payload + 48 * 4 + (8 + 8 + 8) + 16 * k) / (4 * k)
    assert abs(fmt.tensor_bpw(t) - want) < 1e-12
    ref = ROOT.parent / "reference"
    if (ref / "hi2" / "format.py").exists():
        code = (f"import sys; sys.path.insert(0, {str(ref)!r}); import torch; from hi2 import format as f; "
                "nb=torch.tensor([2,2,4,8],dtype=torch.uint8); bl=torch.tensor([16,64,32,32],dtype=torch.uint8); "
                "h=torch.tensor([1,0,1,1,0,0,1,1],dtype=torch.uint8); print(f.metadata_bits(nb,bl,h), f.metadata_bits(nb,bl,torch.ones(8,dtype=torch.uint8)))")
        import subprocess
        import sys

        out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, check=True).stdout.split()
        assert [int(v) for v in out] == [fmt.metadata_bits(nb, bl, mixed), fmt.metadata_bits(nb, bl, same)]
    cands = [(2, 32), (4, 32), (8, 32), (8, 64)]
    tables = {n: TensorTable(n, (3, 64), same[:4], torch.arange(12.0).reshape(4, 3) + i, list(cands), 1.0, 10)
              for i, n in enumerate(("a", "b", "c"))}
    tables["d"] = TensorTable("d", (3, 64), same[:4], torch.zeros(2, 3), cands[:2], 1.0, 10)  # no INT8 candidates
    out, chosen = allocate.force_int8(tables, {"a": 0.5, "b": 3.0, "c": 2.0, "d": 9.0}, 1)
    assert chosen == ["b"] and out["b"].candidates == cands[2:] and torch.equal(out["b"].sse, tables["b"].sse[2:])
    assert out["a"].candidates == cands[:2] and out["c"].candidates == cands[:2] and out["d"] is tables["d"]
    assert allocate.restrict(tables["a"], lambda c: False) is tables["a"]  # nothing left: unchanged


def test_expert_coverage_report():
    from hi2_b200.moe import coverage

    counts = {f"m.layers.{l}.mlp.experts.{e}.gate_proj.weight": 10 * l + e for l in (2, 10) for e in range(4)}
    counts["m.layers.2.self_attn.q_proj.weight"] = 99  # not an expert tensor
    rep = coverage(counts, {"m.layers.10.mlp.experts.0.gate_proj.weight", "m.layers.10.mlp.experts.3.gate_proj.weight"})
    assert list(rep) == ["m.layers.2.mlp.experts.*.gate_proj", "m.layers.10.mlp.experts.*.gate_proj"]
    assert rep["m.layers.2.mlp.experts.*.gate_proj"] == {"experts": 4, "min": 20, "median": 21.5, "max": 23, "fallback": []}
    assert rep["m.layers.10.mlp.experts.*.gate_proj"]["fallback"] == [0, 3]
