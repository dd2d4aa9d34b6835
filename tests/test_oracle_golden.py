"""The CPU oracle against outputs of the reference itself (tests/golden/ptq_golden.pt).

Integer, byte and index results must be equal; floating-point results that go through a CPU
BLAS or a vectorised reduction are allowed the rounding of a different host."""

import pytest
import torch

from oracle import ptq_oracle as po

ROOT = __import__("pathlib").Path(__file__).resolve().parents[1]
TIGHT = dict(rtol=2e-6, atol=1e-7)


def close(a, b, **kw):
    kw = kw or TIGHT
    assert a.shape == b.shape and a.dtype == b.dtype
    assert torch.allclose(a.double(), b.double(), **kw), float((a.double() - b.double()).abs().max())


def same_rows(got, want, code_floor=1.0):
    agree = (got.codes == want["codes"]).float().mean().item()
    assert agree >= code_floor, agree
    assert (got.params == want["params"]).float().mean().item() >= code_floor
    close(got.consts, want["consts"], rtol=1e-3, atol=1e-6)
    close(got.sse, want["sse"], rtol=1e-4, atol=1e-6)
    if "comp" in want and code_floor == 1.0:
        close(got.comp, want["comp"], rtol=1e-5, atol=1e-6)


def test_hadamard_is_symmetric_involution():
    h = po.hadamard16()
    assert torch.equal(h, h.T)
    assert torch.equal(h @ h, torch.eye(16, dtype=torch.float64))


@pytest.mark.parametrize("name", ["f32", "f64", "f16", "bf16", "f32_all"])
def test_rotation_is_bit_exact(golden, name):
    rot = golden["rotation"]
    case = rot[name]
    flags = torch.ones(32, dtype=torch.uint8) if name == "f32_all" else rot["flags"]
    got = po.rotate_groups(case["x"], flags)
    assert got.dtype == case["y"].dtype
    assert torch.equal(got, case["y"])


def test_rotation_validates_shapes():
    with pytest.raises(ValueError):
        po.rotate_groups(torch.zeros(2, 24), torch.ones(1))
    with pytest.raises(ValueError):
        po.rotate_groups(torch.zeros(2, 32), torch.ones(3))


def test_second_moment_and_group_moments(golden):
    st = golden["stats"]
    sm = po.SecondMoment(64)
    sm.update(st["x"][:300], chunk=128)
    other = po.SecondMoment(64)
    other.update(st["x"][300:], chunk=128)
    sm.merge(other)
    assert sm.n == st["n"]
    close(sm.S, st["S"], rtol=1e-5, atol=1e-4)
    close(sm.mean(), st["mean"], rtol=1e-5, atol=1e-6)
    gm = po.GroupMoments(64)
    gm.update(st["x"])
    close(gm.S, st["G"], rtol=1e-6, atol=1e-6)
    close(gm.diag(), st["diag_plain"])
    close(gm.diag(st["had"]), st["diag_rot"])
    s16 = po.smoothing_vector(gm, 0.5)
    assert torch.equal(s16, st["s16"])
    close(gm.diag(st["had"], 1.0 / s16.float()), st["diag_rot_inv"])


def test_basis_change(golden):
    b = golden["basis"]
    close(po.stored_basis_hessian(b["sigma"], b["s16"], b["had"]), b["hs"], rtol=1e-5, atol=1e-6)
    close(po.stored_basis_hessian(b["sigma"], None, b["had"]), b["hs_noscale"], rtol=1e-5, atol=1e-6)
    plain = po.stored_basis_hessian(b["sigma"], None, torch.zeros(4, dtype=torch.uint8))
    close(plain, b["hs_plain"], rtol=1e-6, atol=1e-7)


def test_inverse_factor_and_damping_retry(golden):
    f = golden["factor"]
    close(po.inverse_cholesky(f["hs"], 0.01), f["u"], rtol=1e-4, atol=1e-5)
    close(po.inverse_cholesky(f["sing"], 1e-9), f["u_sing"], rtol=5e-2, atol=1e-2)
    with pytest.raises(RuntimeError):
        po.inverse_cholesky(-torch.eye(8), 0.01)


def test_ladder_search(golden):
    for case in golden["ladder"]:
        lo, st = po.search_ladder(case["wb"], case["db"], case["n"], case["effort"])
        close(lo, case["lo"], rtol=1e-6, atol=1e-6)
        close(st, case["step"], rtol=1e-6, atol=1e-6)


def test_parameter_bytes_and_decode(golden):
    p = golden["params"]
    lo_u8, st_u8, consts = po.quantise_ladders(p["lo"], p["step"])
    assert torch.equal(lo_u8, p["lo_u8"]) and torch.equal(st_u8, p["step_u8"])
    assert torch.equal(consts, p["consts"])
    lo_d, st_d = po.decode_ladders(lo_u8, st_u8, consts[:, 0:1], consts[:, 1:2], consts[:, 2:3])
    assert torch.equal(lo_d, p["lo_d"]) and torch.equal(st_d, p["step_d"])
    # known answers of the reference's format tests: fp32 fma then fp16; zero steps stay zero
    u = torch.arange(256)
    lo_min, lo_scale = torch.tensor(-0.37).half(), torch.tensor(0.00391).half()
    scale = torch.tensor(0.0123).half()
    lo, step = po.decode_ladders(u, u, lo_min, lo_scale, scale)
    assert torch.equal(lo, (u.double() * lo_scale.double() + lo_min.double()).float().half())
    assert torch.equal(step, (u.float() * scale.float()).half())
    lo_u8, st_u8, consts = po.quantise_ladders(
        torch.tensor([[0.5, -0.2, 0.1]]), torch.tensor([[0.0, 0.03, 0.0]])
    )
    _, dstep = po.decode_ladders(lo_u8, st_u8, consts[:, 0:1], consts[:, 1:2], consts[:, 2:3])
    assert dstep[0, 0] == 0 and dstep[0, 2] == 0


def test_reconstruction_rounds_once():
    g = torch.Generator().manual_seed(0)
    codes = torch.randint(0, 16, (4096,), generator=g)
    lo = (torch.randn(4096, generator=g) * 50).half()
    step = (torch.rand(4096, generator=g) * 16).half()
    got = po.reconstruct(codes.unsqueeze(-1), lo, step).squeeze(-1)
    assert torch.equal(got, (lo.double() + codes.double() * step.double()).half())


def test_nearest_rows(golden):
    near = golden["nearest"]
    for (nb, b, effort), want in near["cases"].items():
        same_rows(po.nearest_rows(near["w"], near["d"], nb, b, effort), want)


def test_gptq_rows(golden):
    for entry in golden["gptq"]:
        for (nb, b), want in entry["cases"].items():
            got = po.gptq_rows(entry["w"], entry["d"], entry["u"], nb, b, "normal", entry["perm"])
            same_rows(got, want)


def test_refinement(golden):
    r = golden["refine"]
    groups = [
        (g["w"], po.Rows(**g["enc"]), g["nbits"], g["block"]) for g in r["groups"]
    ]
    new = po.refine_groups(groups, r["hs"], 2)
    for got, want in zip(new, r["codes"]):
        assert torch.equal(got, want)
    # a sweep never raises the objective and moves a code by at most one level
    for (w, enc, nb, b), codes in zip(groups, new):
        lo, st = po._decoded(enc.params[..., 0], enc.params[..., 1], enc.consts)
        before = po.hessian_objective(w, enc.codes, lo, st, r["hs"], b)
        after = po.hessian_objective(w, codes, lo, st, r["hs"], b)
        assert after <= before * (1 + 1e-6)
        assert (codes.int() - enc.codes.int()).abs().max() <= 2  # two sweeps
        assert int(codes.max()) <= 2**nb - 1


def test_pack_known_answers(golden):
    for nb in (2, 4):
        one = torch.zeros(1, 32, dtype=torch.int64)
        one[0, 1] = 3 if nb == 2 else 9
        assert int(po.pack_words(one, nb)[0, 0]) == int(one[0, 1]) << nb
    with pytest.raises(ValueError):
        po.pack_words(torch.full((1, 16), 4), 2)
    with pytest.raises(ValueError):
        po.pack_words(torch.zeros(1, 15, dtype=torch.int64), 2)
    for nb in (2, 4, 8):
        case = golden["pack"][nb]
        words = po.pack_words(case["codes"], nb)
        assert words.dtype == torch.int32 and torch.equal(words, case["words"])
        assert torch.equal(po.unpack_words(words, nb), case["codes"])


def test_assemble_layout(golden):
    a = golden["pack"]["assemble"]
    flat = po.assemble_flat(a["pieces"], a["row_nbits"], a["row_block"], a["had"], a["k"])
    for name, want in a["out"].items():
        got = getattr(flat, name)
        assert got.dtype == want.dtype and torch.equal(got, want), name
    # offsets of the reference's layout test: rows (2,32) (4,64) (2,64) (4,32) at K=128
    nbits, block = torch.tensor([2, 4, 2, 4]), torch.tensor([32, 64, 64, 32])
    pieces = []
    for r in range(4):
        nb, b = int(nbits[r]), int(block[r])
        pieces.append(
            (
                torch.tensor([r]),
                torch.zeros(1, 128, dtype=torch.uint8),
                torch.zeros(1, 128 // b, 2, dtype=torch.uint8),
                torch.zeros(1, 3, dtype=torch.float16),
            )
        )
    flat = po.assemble_flat(pieces, nbits, block, torch.zeros(8), 128)
    assert flat.code_off.tolist() == [0, 8, 24, 32, 48]
    assert flat.param_off.tolist() == [0, 4, 6, 8, 12]
    assert flat.codes.numel() == 48 and flat.blk_params.numel() == 24


def test_allocation_is_bit_exact(golden):
    a = golden["allocate"]
    tables = [po.Table(**t) for t in a["tables"]]
    for target, want in a["results"].items():
        got = po.allocate_rows(tables, target, a["sens"])
        assert got.feasible == want["feasible"]
        assert got.lam == want["lam"] and got.bpw == want["bpw"]
        for name, p in want["picks"].items():
            assert torch.equal(got.picks[name], p)


def test_transform_choice_matches_reference():
    """Shared transform (rotation flags per 64-column chunk, smoothing exponent search) against what
    hi2 itself chose (tests/golden/transform_golden.pt, hi2/calibrate.py:114-209)."""
    from tests.helpers import transform_case

    cases = torch.load(ROOT / "tests" / "golden" / "transform_golden.pt", weights_only=False)
    assert {c["mode"] for c in cases} == {"auto", "on", "off"}
    for c in cases:
        ws, x = transform_case(c["seed"], c["k"], c["rows"])
        gm = po.GroupMoments(c["k"])
        gm.update(x)
        s16, had = po.pick_transform(ws, gm, c["mode"], c["alpha"], c["search"])
        assert (s16 is None and c["s16"] is None) or torch.equal(s16, c["s16"])
        assert torch.equal(had, c["had"])
        for alpha, want in c["costs"].items():
            s_a, had_a = po._transform_for(ws, gm, c["mode"], alpha)
            assert abs(po.transform_cost(ws, gm, s_a, had_a) - want) <= 1e-6 * want


def test_inverse_path_matches_reference():
    """Reconstruction of a mixed-row packed tensor against hi2's own dequantize / dequantize_stored
    (tests/golden/dequant_golden.pt): every step is exact in fp64, so the results are equal."""
    cases = torch.load(ROOT / "tests" / "golden" / "dequant_golden.pt", weights_only=False)
    for case in cases.values():
        flat = po.Flat(**case["fields"], shape=case["shape"], col_scale=case["col_scale"])
        assert torch.equal(po.reconstruct_flat(flat, original=False), case["stored"])
        assert torch.equal(po.reconstruct_flat(flat, original=True), case["original"])
