"""GPTQ rounding on the GPU.

Two claims, tested apart.  (1) The column loop itself: given the oracle's factor U, the same fp32
rows AND the oracle's decoded ladders, the kernel's in-block arithmetic is operation for operation
the reference's and only the fp32 trailing product sums in a different order, so the codes must
be equal (>= 99.99 %).  (2) The whole encode_rows_gptq, ladders fitted by the kernels: the ladder
search returns the reference's ladders bit for bit (see test_gpu_ladder), so parameter bytes and
row constants must be EQUAL on every row, codes >= 99.99 % (the contract's bar is 99.9 %; 100 %
measured), Hessian-weighted error and sse within 1 % (1e-4 measured) of the oracle's."""

import pytest
import torch

from oracle import ptq_oracle as po
from tests.helpers import CASES, DEV, agreement, correlated_layer, ladder_report, rel_close, weighted_error

pytestmark = pytest.mark.gpu


def _compare(got, want, w, hs, block):
    assert got.codes.dtype == torch.uint8 and got.codes.shape == want.codes.shape
    rep = ladder_report(got, want)
    assert rep["rows_same"] == 1.0 and rep["params"] == 1.0, rep  # ladders: bytes and constants equal
    assert rep["codes"] >= 0.9999, rep
    e_got = weighted_error(w, hs, got.codes, got.params, got.consts, block)
    e_want = weighted_error(w, hs, want.codes, want.params, want.consts, block)
    assert abs(e_got - e_want) <= 0.01 * e_want, (e_got, e_want)
    total = float(want.sse.sum())
    assert abs(float(got.sse.sum()) - total) <= 0.01 * total
    return rep


def _round_with_ladders(w, u, lo_d, st_d, nbits, block, perm=None):
    """The C-ABI column loop on rows w with GIVEN decoded ladders [N, K/block] (CPU tensors in,
    codes and comp in rounding order out)."""
    from hi2_b200 import gptq_kernel

    n, k = w.shape
    ldp = k // 16
    lo = torch.zeros(n, ldp)
    st = torch.zeros(n, ldp)
    lo[:, : k // block], st[:, : k // block] = lo_d, st_d
    cols = torch.arange(k) if perm is None else perm
    wc = w[:, cols].contiguous().to(DEV)
    codes = torch.empty(n, k, dtype=torch.uint8, device=DEV)
    comp = torch.empty(n, k, device=DEV)
    err1 = torch.empty(n, 128, device=DEV)
    ud = u.to(DEV).contiguous()
    gptq_kernel.gptq_round(
        wc, err1, codes, lo.to(DEV), st.to(DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
        torch.tensor([ud.data_ptr()], dtype=torch.int64, device=DEV),
        (cols // block).to(torch.int32).reshape(1, k).to(DEV),
        torch.tensor([2.0**nbits - 1], device=DEV), comp, [0, n], [ud],
    )
    return codes.cpu(), comp.cpu()


@pytest.mark.parametrize("nbits,block", CASES)
@pytest.mark.parametrize("k", [192, 448, 1024])  # 192 and 448 end in a 64-column block
def test_column_loop_given_oracle_ladders(nbits, block, k):
    w, d, u, _, _ = correlated_layer(200, k, nbits * 7 + block + k)
    want = po.gptq_rows(w, d, u, nbits, block, "normal")
    lo_d, st_d = po._decoded(want.params[..., 0], want.params[..., 1], want.consts)
    codes, comp = _round_with_ladders(w, u, lo_d, st_d, nbits, block)
    assert agreement(codes, want.codes) >= 0.9999, agreement(codes, want.codes)
    rows = (codes == want.codes).all(-1)
    assert rel_close(comp[rows], want.comp[rows], 1e-4, 1e-4)


@pytest.mark.parametrize("nbits,block,k,rows", [(2, 32, 1024, 200), (4, 64, 2048, 333), (8, 32, 1024, 130),
                                                  (2, 16, 1280, 64)])
def test_column_loop_tensor_core_update_given_oracle_ladders(nbits, block, k, rows):
    """The trailing update as three TF32 tcgen05 products: same codes as the oracle's fp32 loop.
    Rows and columns that do not fill the 128 x 256 tiles, several column tiles, two units."""
    from hi2_b200 import gptq_kernel

    w, d, u, _, _ = correlated_layer(rows, k, nbits + block + k)
    want = po.gptq_rows(w, d, u, nbits, block, "normal")
    lo_d, st_d = po._decoded(want.params[..., 0], want.params[..., 1], want.consts)
    ldp = k // 16
    lo = torch.zeros(rows, ldp)
    st = torch.zeros(rows, ldp)
    lo[:, : k // block], st[:, : k // block] = lo_d, st_d
    ud = u.to(DEV).contiguous()
    ud2 = ud.clone()  # a second unit with its own copy of the factor
    split = [gptq_kernel.split_tf32_transposed(ud), gptq_kernel.split_tf32_transposed(ud2)]
    assert (split[0].sum(0).T - ud).abs().max() <= 1e-6 * ud.abs().max()
    half = rows // 2
    wc = w.contiguous().to(DEV)
    codes = torch.empty(rows, k, dtype=torch.uint8, device=DEV)
    comp = torch.empty(rows, k, device=DEV)
    err1 = torch.empty(rows, 128, device=DEV)
    grp = torch.cat([torch.zeros(half, dtype=torch.int32), torch.ones(rows - half, dtype=torch.int32)]).to(DEV)
    status = gptq_kernel.gptq_round_tc(
        wc, err1, codes, lo.to(DEV), st.to(DEV), grp,
        torch.tensor([ud.data_ptr(), ud2.data_ptr()], dtype=torch.int64, device=DEV),
        (torch.arange(k) // block).to(torch.int32).reshape(1, k).repeat(2, 1).contiguous().to(DEV),
        torch.tensor([2.0**nbits - 1] * 2, device=DEV), comp, [0, half, rows], split,
    )
    assert int(status.item()) == 0
    # 256 levels are sensitive to the ~1e-6 error of the split product; the encoder therefore keeps
    # the FMA update for INT8 rows (hi2_b200/hessian.py) and this case only documents the effect
    floor = 0.9999 if nbits <= 4 else 0.99
    assert agreement(codes, want.codes) >= floor, agreement(codes, want.codes)
    same = (codes.cpu() == want.codes).all(-1)
    assert rel_close(comp.cpu()[same], want.comp[same], 1e-4, 1e-4)


def test_column_loop_given_oracle_ladders_act_order():
    w, d, u, perm, _ = correlated_layer(64, 448, 9, act_order=True)
    want = po.gptq_rows(w, d, u, 4, 32, "normal", perm)
    lo_d, st_d = po._decoded(want.params[..., 0], want.params[..., 1], want.consts)
    codes_p, _ = _round_with_ladders(w, u, lo_d, st_d, 4, 32, perm)
    codes = torch.empty_like(codes_p)
    codes[:, perm] = codes_p
    assert agreement(codes, want.codes) >= 0.9999


@pytest.mark.parametrize("nbits,block", CASES)
@pytest.mark.parametrize("k", [192, 448, 1024])
def test_gptq_matches_oracle(nbits, block, k):
    from hi2_b200.hessian import encode_rows_gptq

    w, d, u, _, hs = correlated_layer(200, k, nbits * 7 + block + k)
    got = encode_rows_gptq(w.to(DEV), d.to(DEV), u.to(DEV), nbits, block, "normal")
    want = po.gptq_rows(w, d, u, nbits, block, "normal")
    rep = _compare(got, want, w, hs, block)
    assert rel_close(got.comp.cpu()[rep["same"]], want.comp[rep["same"]], 1e-4, 1e-4)


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
    """Against outputs of the reference itself (fixture): every row's ladder equal, codes >= 99.99 %."""
    from hi2_b200.hessian import encode_rows_gptq

    for entry in golden["gptq"]:
        perm = None if entry["perm"] is None else entry["perm"].to(DEV)
        for (nb, b), want in entry["cases"].items():
            got = encode_rows_gptq(entry["w"].to(DEV), entry["d"].to(DEV), entry["u"].to(DEV), nb, b,
                                   "normal", perm)
            rep = ladder_report(got, po.Rows(**want))
            assert rep["rows_same"] == 1.0 and rep["codes"] >= 0.9999, (nb, b, rep)


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


def test_many_small_jobs_prepared_together_equal_single_calls(monkeypatch):
    """A layer of experts: many small jobs of one width, several (nbits, block) among them, each with
    column weights and a factor of its own.  Their ladders are searched in one launch per
    (nbits, block) over a gathered buffer; results must equal one call per job, bit for bit.  Jobs
    with a column permutation, and kinds with fewer than four jobs, still go one by one."""
    import hi2_b200.hessian as hm

    k = 256
    jobs = []
    for i in range(14):
        nb, b = ((2, 32), (4, 64), (2, 16))[i % 3] if i < 12 else (4, 16)
        w, d, u, perm, _ = correlated_layer(9 + 3 * i, k, 100 + i, act_order=(i == 5))
        jobs.append(hm.GptqJob(w.to(DEV), d.to(DEV), u.to(DEV), nb, b, None if perm is None else perm.to(DEV)))
    refs = [hm.encode_rows_gptq(j.w, j.d, j.u, j.nbits, j.block, "fast", j.perm) for j in jobs]
    calls = []
    together = hm._prepare_together
    monkeypatch.setattr(hm, "_prepare_together", lambda pieces, *a: calls.append(len(pieces)) or together(pieces, *a))
    got = hm.encode_jobs_gptq(jobs, "fast", comp=True)
    assert sorted(calls) == [4, 4]  # (2, 32) lost job 5 to its permutation and (4, 16) has two jobs only
    for g_, ref in zip(got, refs):
        for f in ("codes", "params", "consts", "sse", "comp"):
            assert torch.equal(getattr(g_, f), getattr(ref, f)), f


def test_gptq_block_entry_point_matches_driver():
    """The reference-shaped per-block entry point (hi2/hessian.py:304-312 drives it) gives the
    same codes as the fused driver."""
    from hi2_b200 import _lib, gptq_kernel, ladder_kernel
    from hi2_b200.encode import EFFORT
    from hi2_b200.hessian import encode_rows_gptq

    w, d, u, _, _ = correlated_layer(37, 448, 77)
    w, d, u = w.to(DEV), d.to(DEV), u.to(DEV).contiguous()  # the entry point takes raw addresses
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
        if i2 < k:  # the trailing update through its own entry point (hi2/hessian.py:310-312)
            _lib.call("hi2_gptq_lazy_update", _lib.ptr(wc), n, k, i1, i2, _lib.ptr(err1), _lib.ptr(u),
                      _lib.stream(wc.device))
    assert torch.equal(codes, ref.codes) and torch.equal(comp, ref.comp)
    with pytest.raises(ValueError):
        gptq_kernel.gptq_block(wc, 0, 129, torch.empty(n, 129, device=DEV), codes, q["lo_d"],
                               q["step_d"], row_grp, u_ptrs, blk, nmax)


def test_torch_backend_is_refused():
    from hi2_b200.hessian import encode_rows_gptq

    w, d, u, _, _ = correlated_layer(4, 128, 1)
    with pytest.raises(RuntimeError):
        encode_rows_gptq(w.to(DEV), d.to(DEV), u.to(DEV), 2, 32, backend="torch")
