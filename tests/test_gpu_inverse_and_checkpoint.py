"""The inverse path (dequantise on the device) and the streaming checkpoint writer.

* ``format.dequantize_stored`` / ``format.dequantize`` against hi2's own functions on a mixed-row
  packed tensor (tests/golden/dequant_golden.pt): equal in fp64, every step being exact;
* ``checkpoint.write_checkpoints`` on the toy Llama model of the propagation test: shards on disk
  with the format's tensor names, markers with the file digest, everything read back and
  dequantised on the device by ``verify_checkpoint``."""

import json
import pathlib

import pytest
import torch

from oracle import ptq_oracle as po
from tests.helpers import DEV, toy_llama

pytestmark = pytest.mark.gpu
GOLDEN = pathlib.Path(__file__).parent / "golden"


def test_dequantize_equals_reference():
    from hi2_b200.format import HI2Tensor, dequantize, dequantize_stored

    cases = torch.load(GOLDEN / "dequant_golden.pt", weights_only=False)
    for case in cases.values():
        t = HI2Tensor(**case["fields"], shape=case["shape"], col_scale=case["col_scale"])
        assert torch.equal(dequantize_stored(t).cpu(), case["stored"])
        assert torch.equal(dequantize(t).cpu(), case["original"])
        assert torch.equal(dequantize(t, dtype=torch.float32).cpu(), case["original"].float())
    bad = HI2Tensor(**{**case["fields"], "row_nbits": torch.full_like(case["fields"]["row_nbits"], 3)},
                    shape=case["shape"], col_scale=None)
    with pytest.raises(ValueError):
        dequantize(bad)


def test_reference_linear_and_bit_count():
    """``format.reference_linear`` (activation divided by the smoothing vector and rotated, contracted
    with the stored basis) equals the product with the original-basis reconstruction; ``tensor_bpw``
    counts what the buffers hold."""
    from hi2_b200.format import HI2Tensor, dequantize, metadata_bits, reference_linear, tensor_bpw

    cases = torch.load(GOLDEN / "dequant_golden.pt", weights_only=False)
    g = torch.Generator().manual_seed(3)
    for case in cases.values():
        t = HI2Tensor(**case["fields"], shape=case["shape"], col_scale=case["col_scale"])
        x = torch.randn(7, t.shape[1], generator=g, dtype=torch.float64)
        got = reference_linear(x, t, DEV)
        want = x.to(DEV) @ dequantize(t, DEV).T
        assert got.shape == (7, t.shape[0])
        assert ((got - want).abs().max() / want.abs().max()).item() < 1e-12
        bits = t.codes.numel() * 32 + t.blk_params.numel() * 8 + 48 * t.shape[0] + metadata_bits(t.row_nbits, t.row_block, t.had)
        bits += 16 * t.shape[1] if t.col_scale is not None else 0
        assert abs(tensor_bpw(t) - bits / (t.shape[0] * t.shape[1])) < 1e-12


def test_encode_then_dequantize_round_trip():
    """What the encoder packs is what the decoder reads: GPTQ-encode rows on the device, assemble,
    dequantise in the stored basis, and compare with the codes' own reconstruction."""
    from hi2_b200.format import assemble, dequantize_stored
    from hi2_b200.hessian import encode_rows_gptq
    from tests.helpers import correlated_layer

    w, d, u, _, _ = correlated_layer(48, 448, 3)
    pieces, want = [], torch.zeros(48, 448, dtype=torch.float64)
    nbits, block = torch.zeros(48, dtype=torch.int64), torch.zeros(48, dtype=torch.int64)
    for rows, (nb, b) in ((torch.arange(0, 20), (2, 32)), (torch.arange(20, 40), (4, 64)), (torch.arange(40, 48), (8, 32))):
        e = encode_rows_gptq(w[rows].to(DEV), d.to(DEV), u.to(DEV), nb, b)
        pieces.append((rows.to(DEV), e.codes, e.params, e.consts, nb, b))
        lo, st = po._decoded(e.params[..., 0].cpu(), e.params[..., 1].cpu(), e.consts.cpu())
        want[rows] = po.reconstruct(e.codes.cpu().reshape(rows.numel(), -1, b), lo, st).double().reshape(rows.numel(), -1)
        nbits[rows], block[rows] = nb, b
    t = assemble(pieces, nbits, block, torch.ones(28, dtype=torch.uint8), 448)
    assert torch.equal(dequantize_stored(t).cpu(), want)


def test_write_and_verify_checkpoint(tmp_path):
    from safetensors import safe_open

    from hi2_b200.allocate import allocate_global
    from hi2_b200.calibrate import Config
    from hi2_b200.checkpoint import file_digest, from_tensors, verify_checkpoint, write_checkpoints
    from hi2_b200.layerwise import DeviceSink, calibrate_layerwise

    model, ids = toy_llama()
    model = model.to(DEV)
    cfg = Config(effort="fast")
    sink = DeviceSink()
    tables = calibrate_layerwise(model, ids, cfg, exclude=["lm_head|embed"], sink=sink, log=lambda *_: None)
    alloc = allocate_global(list(tables.values()), 4.5)
    state = {n: p.detach() for n, p in model.named_parameters()}
    names = list(state)
    shards = {"model-00001-of-00002.safetensors": {n: state[n] for n in names[: len(names) // 2]},
              "model-00002-of-00002.safetensors": {n: state[n] for n in names[len(names) // 2 :]}}

    def sigma_of(name):
        leader = sink.leader[name]
        s, n = sink.sigma[leader]
        return s, n, leader, sink.stats[leader]

    assert len(sink.factors) == len(sink.groups)  # started beside the tables
    markers = write_checkpoints(shards, tables, alloc.picks, sigma_of, cfg, tmp_path, budget=1 << 18, log=lambda *_: None,
                                factors=sink.factors)
    assert set(markers) == set(shards)
    for shard, tensors in shards.items():
        path = tmp_path / shard
        saved = json.loads((tmp_path / (shard + ".done.json")).read_text())
        assert saved["sha256"] == file_digest(path) and saved["schema_version"] == 1
        with safe_open(str(path), "pt") as f:
            keys = set(f.keys())
            for n in tensors:
                if n in tables:
                    base = n.removesuffix(".weight")
                    assert f"{base}.hi2_codes" in keys and f"{base}.hi2_col_scale" in keys and n not in keys
                    t = from_tensors({k: f.get_tensor(k) for k in keys if k.startswith(base + ".hi2_")}, base)
                    assert tuple(t.shape) == tuple(tensors[n].shape)
                    assert abs(saved["tensors"][n]["bpw"] - (t.codes.numel() * 32 + t.blk_params.numel() * 8
                               + 48 * t.shape[0] + 16 * t.shape[1]) / (t.shape[0] * t.shape[1])) < 1e-9
                else:
                    assert n in keys  # norms and embeddings pass through
    errors = verify_checkpoint(tmp_path, shards, tables, log=lambda *_: None)
    assert set(errors) == set(tables) and max(errors.values()) < 0.35
    # a flipped byte is caught by the marker's digest
    path = tmp_path / "model-00001-of-00002.safetensors"
    raw = bytearray(path.read_bytes())
    raw[-1] ^= 1
    path.write_bytes(bytes(raw))
    with pytest.raises(ValueError):
        verify_checkpoint(tmp_path, shards, tables, log=lambda *_: None)


def test_stacked_expert_layout_through_the_writer(tmp_path):
    """``write_checkpoints(moe_layout="stacked")``: the experts of a layer are written as one stack
    per projection group (put together on the device), everything else as before; the stack splits
    back into exactly the tensors the per-expert layout writes; ``verify_checkpoint`` reads both."""
    from safetensors import safe_open

    from hi2_b200 import layer as L
    from hi2_b200 import stack
    from hi2_b200.allocate import allocate_global
    from hi2_b200.calibrate import Config, build_table
    from hi2_b200.checkpoint import from_tensors, verify_checkpoint, write_checkpoints
    from hi2_b200.format import FIELDS
    from tests.helpers import activations, gen

    g = gen(17)
    cfg = Config(effort="fast")
    hidden, ffn, n_exp = 256, 128, 3
    pre = "model.layers.0.mlp.experts"
    weights, reads = {}, {}
    for e in range(n_exp):
        for part, (r, k) in (("gate_proj", (ffn, hidden)), ("up_proj", (ffn, hidden)), ("down_proj", (hidden, ffn))):
            weights[f"{pre}.{e}.{part}.weight"] = (torch.randn(r, k, generator=g) * 0.05).bfloat16().to(DEV)
            reads[f"{pre}.{e}.{part}.weight"] = f"{e}.{'mid' if part == 'down_proj' else 'in'}"
    weights["model.layers.0.self_attn.q_proj.weight"] = (torch.randn(hidden, hidden, generator=g) * 0.05).bfloat16().to(DEV)
    reads["model.layers.0.self_attn.q_proj.weight"] = "attn"
    norm = {"model.layers.0.input_layernorm.weight": torch.ones(hidden, device=DEV)}
    acts = {f"{e}.in": activations(1024 + 64 * e, hidden, 40 + e, dtype=torch.bfloat16).to(DEV) for e in range(n_exp)}
    acts.update({f"{e}.mid": activations(1024 + 64 * e, ffn, 50 + e, dtype=torch.bfloat16).to(DEV) for e in range(n_exp)})
    acts["attn"] = activations(2048, hidden, 60, dtype=torch.bfloat16).to(DEV)
    shared = L.accumulate(acts, DEV)
    L.finish_statistics(shared, cfg)
    tables = {n: build_table(n, w, shared[reads[n]].moments, cfg, transform=shared[reads[n]].transform)
              for n, w in weights.items()}
    picks = allocate_global(list(tables.values()), 3.5).picks
    shards = {"model-00001-of-00001.safetensors": {**norm, **weights}}

    def sigma_of(name):
        s = shared[reads[name]]
        return s.hessian.S, s.hessian.n, reads[name], s.moments

    quiet = lambda *_: None  # noqa: E731
    write_checkpoints(shards, tables, picks, sigma_of, cfg, tmp_path / "flat", log=quiet)
    markers = write_checkpoints(shards, tables, picks, sigma_of, cfg, tmp_path / "stacked", log=quiet, moe_layout="stacked")
    (marker,) = markers.values()
    assert set(marker["tensors"]) == set(tables)  # every tensor is still reported under its own name
    shard_name = "model-00001-of-00001.safetensors"
    with safe_open(str(tmp_path / "stacked" / shard_name), "pt") as f, safe_open(str(tmp_path / "flat" / shard_name), "pt") as flat:
        keys, flat_keys = set(f.keys()), set(flat.keys())
        single, stacked = stack.hi2_bases(keys)
        assert stacked == [f"{pre}.down", f"{pre}.gate_up"] and single == ["model.layers.0.self_attn.q_proj"]
        assert "model.layers.0.input_layernorm.weight" in keys and not any(".experts.0." in k for k in keys)
        for base in stacked:
            group = base.rsplit(".", 1)[1]
            arrays = {k.rsplit(".hi2_", 1)[1]: f.get_tensor(k) for k in keys if k.startswith(base + ".hi2_")}
            assert set(arrays) == {*FIELDS, "col_scale", stack.MARK}
            pieces = stack.split_stack(arrays, len(stack.GROUPS[group]))
            assert len(pieces) == n_exp
            for e, parts in enumerate(pieces):
                for part, got in zip(stack.GROUPS[group], parts):
                    mb = stack.member_base(pre, e, part)
                    want = from_tensors({k: flat.get_tensor(k) for k in flat_keys if k.startswith(mb + ".hi2_")}, mb)
                    assert all(torch.equal(getattr(got, fld), getattr(want, fld)) for fld in FIELDS)
                    assert torch.equal(got.col_scale, want.col_scale)
    with pytest.raises(ValueError):
        write_checkpoints(shards, tables, picks, sigma_of, cfg, tmp_path / "x", log=quiet, moe_layout="rows")
    # random weights under correlated activations: GPTQ trades plain error for weighted error, so the
    # bound on the plain reconstruction error is loose here; what matters is that both layouts agree
    seen = {layout: verify_checkpoint(tmp_path / layout, shards, tables, rtol=0.9, log=quiet) for layout in ("flat", "stacked")}
    assert set(seen["flat"]) == set(tables) and seen["flat"] == seen["stacked"]
