"""GPTQ rounding on the GPU.  Given the oracle's factor U and the same fp32 rows, the in-block
arithmetic is operation-for-operation the reference's; only the fp32 trailing product and the
ladder-search sums differ in summation order.  Bars: >= 99.9 % codes, scales 1e-3, Hessian-
weighted error within 1 %."""

import pytest
import torch

from oracle import ptq_oracle as po
from tests.helpers import CASES, DEV, agreement, correlated_layer, rel_close, weighted_error

pytestmark = pytest.mark.gpu


def _compare(got, want, w, hs, block, floor=0.999):
    assert got.codes.dtype == torch.uint8 and got.codes.shape == want.codes.shape
    assert agreement(got.params, want.params) >= 0.999
    assert rel_close(got.consts.float(), want.consts.float(), 1e-3, 1e-6)
    assert agreement(got.codes, want.codes) >= floor, agreement(got.codes, want.codes)
    e_got = weighted_error(w, hs, got.codes, got.params, got.consts, block)
    e_want = weighted_error(w, hs, want.codes, want.params, want.consts, block)
    assert abs(e_got - e_want) <= 0.01 * e_want, (e_got, e_want)
    total = float(want.sse.sum())
    assert abs(float(got.sse.sum()) - total) <= 0.01 * total


@pytest.mark.parametrize("nbits,block", CASES)
@pytest.mark.parametrize("k", [192, 448, 1024])  # 192 and 448 end in a 64-column block
def test_gptq_matches_oracle(nbits, block, k):
    from hi2_b200.hessian import encode_rows_gptq

    w, d, u, _, hs = correlated_layer(200, k, nbits * 7 + block + k)
    got = encode_rows_gptq(w.to(DEV), d.to(DEV), u.to(DEV), nbits, block, "normal")
    want = po.gptq_rows(w, d, u, nbits, block, "normal")
    _compare(got, want, w, hs, block)
    same_rows = (got.codes.cpu() == want.codes).all(-1)
    assert rel_close(got.comp.cpu()[same_rows], want.comp[same_rows], 1e-3, 1e-4)


@pytest.mark.parametrize("nbits,block", [(2, 32), (4, 64)])
def test_gptq_act_order(nbits, block):
    from hi2_b200.hessian import encode_rows_gptq

    w, d, u, perm, hs_p = correlated_layer(64, 448, 5 + nbits, act_order=True)
    got = encode_rows_gptq(w.to(DEV), d.to(DEV), u.to(DEV), nbits, block, "normal", perm.to(DEV))
    want = po.gptq_rows(w, d, u, nbits, block, "normal", perm)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel())
    hs = hs_p[inv][:, inv]
    _compare(got, want, w, hs, block)


def test_gptq_fixture(golden):
    from hi2_b200.hessian import encode_rows_gptq

    ok = n = 0
    for entry in golden["gptq"]:
        perm = None if entry["perm"] is None else entry["perm"].to(DEV)
        for (nb, b), want in entry["cases"].items():
            got = encode_rows_gptq(entry["w"].to(DEV), entry["d"].to(DEV), entry["u"].to(DEV), nb, b,
                                   "normal", perm)
            ok += int((got.codes.cpu() == want["codes"]).sum())
            n += want["codes"].numel()
            assert rel_close(got.consts.float(), want["consts"].float(), 1e-3, 1e-6)
    assert ok / n >= 0.999, ok / n


def test_diagonal_hessian_gives_nearest_codes():
    """With U diagonal nothing is compensated: GPTQ must return the nearest codes."""
    from hi2_b200.encode import encode_rows
    from hi2_b200.hessian import encode_rows_gptq

    g = torch.Generator().manual_seed(3)
    w = torch.randn(50, 256, generator=g).to(DEV)
    d = (torch.rand(256, generator=g) + 0.5).to(DEV)
    u = torch.diag(d.rsqrt())
    a = encode_rows_gptq(w, d, u, 4, 32, "fast")
    b = encode_rows(w, d, 4, 32, "fast")
    assert torch.equal(a.codes, b.codes) and torch.equal(a.params, b.params)
    assert torch.allclose(a.sse, b.sse, rtol=1e-5)
    assert torch.equal(a.comp, w)


def test_batched_jobs_equal_single_calls(monkeypatch):
    """Several jobs, two widths, small units and batches: same results as one call each."""
    import hi2_b200.hessian as hm

    monkeypatch.setattr(hm, "ROW_ELEMS", 256 * 5)
    monkeypatch.setattr(hm, "BATCH_ELEMS", 256 * 23)
    jobs, refs = [], []
    for i, (nb, b) in enumerate(CASES):
        k = 256 if i % 3 else 128
        w, d, u, perm, _ = correlated_layer(13 + i, k, i, act_order=i % 2 == 1)
        perm = None if perm is None else perm.to(DEV)
        jobs.append(hm.GptqJob(w.to(DEV), d.to(DEV), u.to(DEV), nb, b, perm))
    monkeypatch.undo()
    for j in jobs:
        refs.append(hm.encode_rows_gptq(j.w, j.d, j.u, j.nbits, j.block, "fast", j.perm))
    monkeypatch.setattr(hm, "ROW_ELEMS", 256 * 5)
    monkeypatch.setattr(hm, "BATCH_ELEMS", 256 * 23)
    for got, ref in zip(hm.encode_jobs_gptq(jobs, "fast", comp=True), refs):
        for f in ("codes", "params", "consts", "sse", "comp"):
            assert torch.equal(getattr(got, f), getattr(ref, f)), f


def test_gptq_block_entry_point_matches_driver():
    """The reference-shaped per-block entry point (hi2/hessian.py:304-312 drives it) gives the
    same codes as the fused driver."""
    from hi2_b200 import gptq_kernel, ladder_kernel
    from hi2_b200.encode import EFFORT
    from hi2_b200.hessian import encode_rows_gptq

    w, d, u, _, _ = correlated_layer(37, 448, 77)
    w, d, u = w.to(DEV), d.to(DEV), u.to(DEV)
    ref = encode_rows_gptq(w, d, u, 2, 32, "normal")
    cfg = EFFORT["normal"]
    n, k = w.shape
    lo, st = ladder_kernel.fit(w, d, cfg["grid"], cfg["ls"], 4, 32)
    q = ladder_kernel.quantize_rows(lo, st, 2, 32, k, want_decoded=True, ldp=k // 16)
    wc = w.clone()
    codes = torch.zeros(n, k, dtype=torch.uint8, device=DEV)
    comp = torch.zeros(n, k, device=DEV)
    row_grp = torch.zeros(n, dtype=torch.int32, device=DEV)
    u_ptrs = torch.tensor([u.data_ptr()], dtype=torch.int64, device=DEV)
    blk = (torch.arange(k, device=DEV) // 32).to(torch.int32).reshape(1, k)
    nmax = torch.tensor([3.0], device=DEV)
    for i1 in range(0, k, 128):
        i2 = min(i1 + 128, k)
        err1 = torch.empty(n, i2 - i1, device=DEV)
        gptq_kernel.gptq_block(wc, i1, i2 - i1, err1, codes, q["lo_d"], q["step_d"], row_grp, u_ptrs,
                               blk, nmax, comp)
        if i2 < k:
            wc[:, i2:] -= err1 @ u[i1:i2, i2:]
    assert agreement(codes, ref.codes) >= 0.999
    with pytest.raises(ValueError):
        gptq_kernel.gptq_block(wc, 0, 129, torch.empty(n, 129, device=DEV), codes, q["lo_d"],
                               q["step_d"], row_grp, u_ptrs, blk, nmax)


def test_torch_backend_is_refused():
    from hi2_b200.hessian import encode_rows_gptq

    w, d, u, _, _ = correlated_layer(4, 128, 1)
    with pytest.raises(RuntimeError):
        encode_rows_gptq(w.to(DEV), d.to(DEV), u.to(DEV), 2, 32, backend="torch")
