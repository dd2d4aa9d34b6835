"""Ladder search, parameter bytes and nearest rows on the GPU against the oracle.

The search's block sums are formed in the order of torch's CPU reduction (8-lane vectors, four
interleaved accumulators, lanes left to right), every quotient is the IEEE one, and no product is
fused, so on identical fp32 inputs the kernel returns the reference's ``(lo, step)`` BIT FOR BIT;
parameter bytes, row constants and nearest codes follow.  Bars: ladders, bytes, constants and
codes equal; the row error (a K-term fp32 sum added in another order) within 1e-5."""

import pytest
import torch

from oracle import ptq_oracle as po
from tests.helpers import CASES, DEV, gen, rel_close, weights

pytestmark = pytest.mark.gpu


def test_grid_matches_reference_grid():
    """101 x 640 x 16 is not a multiple of the thread block: tails must not be touched
    (the shape of the reference's kernel test)."""
    from hi2_b200 import ladder_kernel
    from hi2_b200.encode import EFFORT

    g = gen(0)
    wb = torch.randn(101, 640, 16, generator=g)
    db = torch.rand(640, 16, generator=g) + 0.5
    grid = EFFORT["normal"]["grid"]
    lo, st, err = ladder_kernel.ladder_grid(wb.to(DEV), db.to(DEV), grid, 4)
    lo_t, st_t, err_t = po.grid_search(wb, db.reshape(1, 640, 16), 4, grid)
    # the reference's own kernel test asks lo equal and step within 1e-6
    # (tests/test_ladder_kernel.py:47-60); here all three outputs are equal
    assert torch.equal(lo.cpu(), lo_t) and torch.equal(st.cpu(), st_t) and torch.equal(err.cpu(), err_t)


@pytest.mark.parametrize("block", [16, 32, 64])
@pytest.mark.parametrize("n", [4, 16, 256])
@pytest.mark.parametrize("effort", ["fast", "normal", "max"])
def test_fit_ladder(block, n, effort):
    from hi2_b200.encode import fit_ladder

    g = gen(block * 1000 + n)
    wb = torch.randn(67, 12, block, generator=g) * torch.exp(torch.randn(67, 12, 1, generator=g))
    wb[0, 0] = 0.25  # a constant block: step 0
    db = torch.rand(1, 12, block, generator=g) + 0.1
    lo, st = fit_ladder(wb.to(DEV), db.to(DEV), n, effort)
    lo_t, st_t = po.search_ladder(wb, db, n, effort)
    assert torch.equal(lo.cpu(), lo_t) and torch.equal(st.cpu(), st_t)
    assert st.cpu()[0, 0] == 0 and lo.cpu()[0, 0] == 0.25


def test_fit_ladder_fixture(golden):
    from hi2_b200.encode import fit_ladder

    for case in golden["ladder"]:  # outputs of the reference itself
        lo, st = fit_ladder(case["wb"].to(DEV), case["db"].to(DEV), case["n"], case["effort"])
        assert torch.equal(lo.cpu(), case["lo"]) and torch.equal(st.cpu(), case["step"]), (case["n"], case["effort"])


def test_quantize_params_is_exact(golden):
    from hi2_b200.encode import quantize_params

    p = golden["params"]
    lo_u8, st_u8, consts = quantize_params(p["lo"].to(DEV), p["step"].to(DEV))
    assert torch.equal(lo_u8.cpu(), p["lo_u8"]) and torch.equal(st_u8.cpu(), p["step_u8"])
    assert torch.equal(consts.cpu(), p["consts"])
    g = gen(3)
    lo = torch.randn(500, 688, generator=g) * 3
    st = torch.rand(500, 688, generator=g) * 0.2 - 0.01  # a few negative steps clamp to 0
    a, b, c = quantize_params(lo.to(DEV), st.to(DEV))
    a_t, b_t, c_t = po.quantise_ladders(lo, st)
    assert torch.equal(a.cpu(), a_t) and torch.equal(b.cpu(), b_t) and torch.equal(c.cpu(), c_t)


def _check_rows(got, want, nbits):
    assert torch.equal(got.params.cpu(), want.params) and torch.equal(got.consts.cpu(), want.consts)
    assert torch.equal(got.codes.cpu(), want.codes)
    assert rel_close(got.sse.cpu(), want.sse, 1e-5, 1e-9)


@pytest.mark.parametrize("nbits,block", CASES)
def test_encode_rows(nbits, block):
    from hi2_b200.encode import encode_rows

    k = 1024
    w = weights(129, k, nbits * 10 + block) * 0.05
    d = torch.rand(k, generator=gen(1)) + 0.05
    got = encode_rows(w.to(DEV), d.to(DEV), nbits, block, "normal")
    _check_rows(got, po.nearest_rows(w, d, nbits, block, "normal"), nbits)


def test_encode_rows_fixture(golden):
    from hi2_b200.encode import encode_rows

    near = golden["nearest"]
    for (nb, b, effort), want in near["cases"].items():  # outputs of the reference itself
        got = encode_rows(near["w"].to(DEV), near["d"].to(DEV), nb, b, effort)
        assert torch.equal(got.codes.cpu(), want["codes"]), (nb, b, effort)


def test_encode_rows_wide_and_strided():
    """K = 11008 (688 blocks of 16) and a row view with a stride."""
    from hi2_b200.encode import encode_rows

    k = 11008
    w = weights(40, k, 9) * 0.02
    d = torch.rand(k, generator=gen(2)) + 0.05
    wd = w.to(DEV)
    got = encode_rows(wd[::2], d.to(DEV), 2, 16, "normal")
    _check_rows(got, po.nearest_rows(w[::2], d, 2, 16, "normal"), 2)


def test_zero_step_and_constant_rows():
    from hi2_b200.encode import encode_rows

    w = torch.zeros(4, 256)
    w[1] = 0.5
    w[2, :128] = torch.linspace(-1, 1, 128)
    got = encode_rows(w.to(DEV), torch.ones(256, device=DEV), 2, 32, "fast")
    want = po.nearest_rows(w, torch.ones(256), 2, 32, "fast")
    assert torch.equal(got.codes.cpu(), want.codes)
    assert torch.equal(got.params.cpu(), want.params) and torch.equal(got.consts.cpu(), want.consts)
    assert float(got.sse[0]) == 0 and float(got.sse[1]) < 1e-6
    assert encode_rows(torch.zeros(0, 64, device=DEV), torch.ones(64, device=DEV), 2, 16).sse.numel() == 0
