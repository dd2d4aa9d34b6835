"""Rotation and packing on the GPU: bit-exact against the oracle and the reference's fixtures."""

import pytest
import torch

from oracle import ptq_oracle as po
from tests.helpers import DEV, gen

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["f32", "f64", "f16", "bf16", "f32_all"])
def test_rotation_matches_reference_fixture(golden, name):
    from hi2_b200.format import fwht_groups

    rot = golden["rotation"]
    case = rot[name]
    flags = torch.ones(32, dtype=torch.uint8) if name == "f32_all" else rot["flags"]
    y = fwht_groups(case["x"].to(DEV), flags)
    assert y.dtype == case["y"].dtype
    assert torch.equal(y.cpu(), case["y"])


@pytest.mark.parametrize("shape", [(3, 64), (101, 10240), (1024, 4096), (257, 11008)])
@pytest.mark.parametrize("mode", ["on", "mixed", "off"])
def test_rotation_fp32_bit_exact(shape, mode):
    from hi2_b200.format import fwht_groups

    g = gen(shape[0] + shape[1])
    x = torch.randn(*shape, generator=g) * torch.exp(torch.randn(1, shape[1], generator=g))
    ng = shape[1] // 16
    flags = {"on": torch.ones(ng), "off": torch.zeros(ng),
             "mixed": (torch.rand(ng, generator=g) < 0.5).float()}[mode].to(torch.uint8)
    y = fwht_groups(x.to(DEV), flags)
    assert torch.equal(y.cpu(), po.rotate_groups(x, flags))
    # involution up to rounding, untouched groups identical
    off = (flags == 0).repeat_interleave(16)
    assert torch.equal(y.cpu()[:, off], x[:, off])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float64])
def test_rotation_other_dtypes(dtype):
    from hi2_b200.format import fwht_groups

    g = gen(5)
    x = (torch.randn(77, 1024, generator=g, dtype=torch.float64) * 4).to(dtype)
    flags = (torch.rand(64, generator=g) < 0.7).to(torch.uint8)
    y = fwht_groups(x.to(DEV), flags)
    assert y.dtype == dtype and torch.equal(y.cpu(), po.rotate_groups(x, flags))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_fused_cast_scale_rotate(dtype):
    """bf16 weights -> fp32, times the fp16 smoothing vector, rotated: one pass equals the
    reference's three steps (hi2/calibrate.py:243-251)."""
    from hi2_b200.format import fwht_groups

    g = gen(6)
    w = (torch.randn(130, 2048, generator=g) * 0.02).to(dtype)
    s16 = (torch.rand(2048, generator=g) * 3 + 0.1).half()
    flags = torch.ones(128, dtype=torch.uint8)
    want = po.rotate_groups(w.float() * s16.float(), flags)
    got = fwht_groups(w.to(DEV), flags, col_scale=s16.float().to(DEV), out_dtype=torch.float32)
    assert got.dtype == torch.float32 and torch.equal(got.cpu(), want)


def test_rotation_rejects_bad_shapes():
    from hi2_b200.format import fwht_groups

    with pytest.raises(ValueError):
        fwht_groups(torch.zeros(2, 24, device=DEV), torch.ones(1))
    with pytest.raises(ValueError):
        fwht_groups(torch.zeros(2, 32, device=DEV), torch.ones(3))
    assert fwht_groups(torch.zeros(0, 32, device=DEV), torch.ones(2)).shape == (0, 32)


def test_cpu_tensors_are_refused():
    from hi2_b200.format import fwht_groups

    with pytest.raises(RuntimeError):
        fwht_groups(torch.zeros(2, 32), torch.ones(2))


@pytest.mark.parametrize("nbits", [2, 4, 8])
def test_pack_matches_fixture_and_oracle(golden, nbits):
    from hi2_b200.format import pack_codes, unpack_codes

    case = golden["pack"][nbits]
    words = pack_codes(case["codes"].to(DEV), nbits)
    assert words.dtype == torch.int32 and torch.equal(words.cpu(), case["words"])
    g = gen(nbits)
    codes = torch.randint(0, 2**nbits, (513, 11008), generator=g, dtype=torch.uint8)
    words = pack_codes(codes.to(DEV), nbits)
    assert torch.equal(words.cpu(), po.pack_words(codes, nbits))
    assert torch.equal(unpack_codes(words, nbits).cpu(), codes.long())


def test_pack_known_answers_and_errors():
    from hi2_b200.format import pack_codes

    for nbits in (2, 4):
        one = torch.zeros(1, 32, dtype=torch.int64)
        one[0, 1] = 3 if nbits == 2 else 9
        assert int(pack_codes(one.to(DEV), nbits)[0, 0]) == int(one[0, 1]) << nbits
    top = torch.full((1, 16), 3, dtype=torch.uint8, device=DEV)
    assert int(pack_codes(top, 2)[0, 0]) == -1  # all ones wraps to a negative int32
    with pytest.raises(ValueError):
        pack_codes(torch.full((1, 16), 4, device=DEV), 2)
    with pytest.raises(ValueError):
        pack_codes(torch.full((1, 16), 4, dtype=torch.uint8, device=DEV), 2)
    with pytest.raises(ValueError):
        pack_codes(torch.zeros(1, 15, dtype=torch.uint8, device=DEV), 2)


def test_assemble_matches_fixture(golden):
    from hi2_b200.format import FIELDS, assemble

    a = golden["pack"]["assemble"]
    pieces = [(r, c.to(DEV), p.to(DEV), rc.to(DEV)) for r, c, p, rc in a["pieces"]]
    t = assemble(pieces, a["row_nbits"], a["row_block"], a["had"], a["k"])
    for name in FIELDS:
        got, want = getattr(t, name), a["out"][name]
        assert got.dtype == want.dtype and torch.equal(got.cpu(), want), name


def test_assemble_mixed_rows_against_oracle():
    from hi2_b200.format import FIELDS, assemble

    g = gen(21)
    r, k = 300, 1024
    cands = [(2, 16), (2, 64), (4, 32), (8, 64)]
    pick = torch.randint(0, len(cands), (r,), generator=g)
    nbits = torch.tensor([cands[i][0] for i in pick.tolist()])
    block = torch.tensor([cands[i][1] for i in pick.tolist()])
    pieces = []
    for ci, (nb, b) in enumerate(cands):
        rows = (pick == ci).nonzero().flatten()
        codes = torch.randint(0, 2**nb, (rows.numel(), k), generator=g, dtype=torch.uint8)
        params = torch.randint(0, 256, (rows.numel(), k // b, 2), generator=g, dtype=torch.uint8)
        consts = torch.randn(rows.numel(), 3, generator=g).half()
        pieces.append((rows, codes, params, consts))
    had = torch.ones(k // 16, dtype=torch.uint8)
    want = po.assemble_flat(pieces, nbits, block, had, k)
    got = assemble([(a, b.to(DEV), c.to(DEV), d.to(DEV)) for a, b, c, d in pieces], nbits, block, had, k)
    for name in FIELDS:
        assert torch.equal(getattr(got, name).cpu(), getattr(want, name)), name
