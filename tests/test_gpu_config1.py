"""BASELINE config 1 IN FULL on the GPU against the CPU oracle run beside it (4096 x 4096 fp16
Linear with 4 outlier columns, 2048 calibration tokens, six candidates, 3.0 bpw), stage by stage on
the oracle's own inputs, then end to end; and one wide matrix (K = 11008, a row sample) through
tables and GPTQ.  The oracle needs about a minute of host time per module.

Bars (the contract's): rotation, allocation and packing bit-exact; codes >= 99.9 %; parameter bytes and row constants (the scales) equal on every row; Hessian-weighted
error within 1 %.  The agreement per (nbits, block) is printed as a table."""

import pytest
import torch

from oracle import ptq_oracle as po
from tests.helpers import DEV, config1_inputs, gen, oracle_layer, rel_close, weighted_error

pytestmark = pytest.mark.gpu
CANDS = [(nb, b) for nb in (2, 4) for b in (16, 32, 64)]


@pytest.fixture(scope="module")
def cfg1():
    w, x = config1_inputs()
    return w, x, oracle_layer(w, x, CANDS, 3.0)


def _norm_err(a, b):
    s = b.double().diagonal().clamp_min(1e-30).sqrt()
    return ((a.double().cpu() - b.double()) / (s[:, None] * s[None, :])).abs().max().item()


def test_statistics_and_transform(cfg1):
    from hi2_b200.calibrate import smoothing_scale
    from hi2_b200.format import fwht_groups
    from hi2_b200.hessian import HessianStats, transform_sigma
    from hi2_b200.stats import ColumnStats

    w, x, ref = cfg1
    h = HessianStats(w.shape[1], DEV)
    h.update(x.to(DEV))
    assert h.n == x.shape[0] and _norm_err(h.S, ref["sm"].S) < 2e-5
    stats = ColumnStats.from_second_moment(h.S, h.n)
    s16 = smoothing_scale(stats, 0.5).cpu()
    assert ((s16.float() - ref["s16"].float()).abs() <= 1e-3 * ref["s16"].float()).all()  # scales: 1e-3
    assert (s16 == ref["s16"]).float().mean().item() >= 0.99  # fp16 of a value that differs by 1e-6
    # rotation with cast and smoothing multiply fused: bit-exact given the same fp32 inputs
    wt = fwht_groups(w.to(DEV), ref["had"], col_scale=ref["s16"].float().to(DEV), out_dtype=torch.float32)
    assert torch.equal(wt.cpu(), ref["wt"])
    hs = transform_sigma(ref["sm"].mean().to(DEV), ref["s16"], ref["had"])
    assert _norm_err(hs, ref["hs"]) < 2e-5 and torch.equal(hs, hs.T)


def test_tables_per_candidate_given_oracle_inputs(cfg1, capsys):
    """encode_rows of all 4096 rows at each of the six candidates on the oracle's rotated weights
    and column weights: ladders, codes and table entries."""
    from hi2_b200.encode import encode_rows

    w, x, ref = cfg1
    wt, d = ref["wt"].to(DEV), ref["d_tab"].to(DEV)
    lines = ["candidate   params==  consts==  codes==   max rel sse err"]
    for ci, (nb, b) in enumerate(CANDS):
        got = encode_rows(wt, d, nb, b, "normal")
        want = po.nearest_rows(ref["wt"], ref["d_tab"], nb, b, "normal")
        p = (got.params.cpu() == want.params).float().mean().item()
        c = (got.consts.cpu() == want.consts).float().mean().item()
        k = (got.codes.cpu() == want.codes).float().mean().item()
        e = ((got.sse.cpu() - want.sse).abs() / want.sse).max().item()
        lines.append(f"INT{nb}/B{b:<3}   {p:8.6f}  {c:8.6f}  {k:8.6f}  {e:.2e}")
        assert p == 1.0 and c == 1.0 and k == 1.0, lines[-1]
        assert rel_close(got.sse.cpu(), ref["table"].sse[ci], 1e-5)
    with capsys.disabled():
        print("\nconfig 1, nearest tables, GPU vs oracle on identical inputs\n" + "\n".join(lines))


def test_allocation_given_oracle_table(cfg1):
    from hi2_b200.allocate import allocate_global
    from hi2_b200.calibrate import TensorTable

    _, _, ref = cfg1
    t = ref["table"]
    table = TensorTable(t.name, t.shape, t.had, t.sse.to(DEV), t.candidates, t.energy, t.n_tokens, t.col_scale)
    got = allocate_global([table], 3.0)
    assert torch.equal(got.picks["w"].cpu(), ref["alloc"].picks["w"])
    assert got.bpw == ref["alloc"].bpw and got.lam == ref["alloc"].lam and got.feasible


def test_factor_gptq_and_packing_given_oracle_inputs(cfg1, capsys):
    from hi2_b200.format import assemble
    from hi2_b200.hessian import encode_rows_gptq, inverse_factor

    w, x, ref = cfg1
    # 2048 tokens for 4096 columns: the Hessian has rank 2048 and only the damping makes it definite
    # (condition ~1e5), so two fp32 factorisations differ from each other by 1e-4..1e-3 of max|U|.
    # The bar is therefore taken against an fp64 solution: as close to it as the reference's own
    # fp32 LAPACK chain is (within a factor 3), which is what "the reference's U" means here.
    u = inverse_factor(ref["hs"].to(DEV), 0.01)
    truth = po.inverse_cholesky(ref["hs"].double(), 0.01)
    scale = truth.abs().max()
    err_gpu = ((u.cpu().double() - truth).abs().max() / scale).item()
    err_ref = ((ref["u"].double() - truth).abs().max() / scale).item()
    assert err_gpu <= max(3 * err_ref, 2e-5), (err_gpu, err_ref)
    lines = ["candidate   rows   ladders==  codes==    e Hs e^T (gpu / oracle)"]
    pieces = []
    for rows, want, nb, b in ref["pieces"]:
        # the oracle's factor: this stage is the column loop, not the factorisation
        got = encode_rows_gptq(ref["wt"][rows].to(DEV), ref["d"].to(DEV), ref["u"].to(DEV), nb, b)
        lad = (got.params.cpu() == want.params).all(-1).all(-1) & (got.consts.cpu() == want.consts).all(-1)
        codes = (got.codes.cpu() == want.codes).float().mean().item()
        e_g = weighted_error(ref["wt"][rows], ref["hs"], got.codes, got.params, got.consts, b)
        e_o = weighted_error(ref["wt"][rows], ref["hs"], want.codes, want.params, want.consts, b)
        lines.append(f"INT{nb}/B{b:<3}   {rows.numel():5d}  {lad.float().mean().item():8.6f}  {codes:8.6f}   {e_g / e_o:.6f}")
        # the contract's bar; measured 99.98-100 % (a code the 3 x TF32 trailing update rounds the other
        # way changes the rest of its 4096-column row)
        assert bool(lad.all()) and codes >= 0.999 and abs(e_g - e_o) <= 0.01 * e_o, lines[-1]
        pieces.append((rows.to(DEV), got.codes, got.params, got.consts, nb, b))
    # with the GPU's own factor (another fp32 rounding of an ill-conditioned inverse, see above) the
    # codes are no longer "identical inputs"; what must hold is the error bar
    rows, want, nb, b = max(ref["pieces"], key=lambda p: p[0].numel())
    own = encode_rows_gptq(ref["wt"][rows].to(DEV), ref["d"].to(DEV), u, nb, b)
    same = (own.codes.cpu() == want.codes).float().mean().item()
    e_own = weighted_error(ref["wt"][rows], ref["hs"], own.codes, own.params, own.consts, b)
    e_o = weighted_error(ref["wt"][rows], ref["hs"], want.codes, want.params, want.consts, b)
    lines.append(f"own factor, INT{nb}/B{b}: codes== {same:.6f}, e Hs e^T ratio {e_own / e_o:.6f} "
                 f"(factor error vs fp64: gpu {err_gpu:.2e}, reference {err_ref:.2e})")
    with capsys.disabled():
        print("\nconfig 1, GPTQ per candidate group, GPU vs oracle on identical inputs\n" + "\n".join(lines))
    assert same >= 0.99 and abs(e_own - e_o) <= 0.01 * e_o, lines[-1]
    # packing / assembly: bit-exact given the oracle's pieces
    cand = torch.tensor(CANDS)
    picks = ref["alloc"].picks["w"]
    flat = assemble([(r.to(DEV), e.codes.to(DEV), e.params.to(DEV), e.consts.to(DEV), nb, b)
                     for r, e, nb, b in ref["pieces"]], cand[picks, 0], cand[picks, 1], ref["had"], w.shape[1], ref["s16"])
    for f in ("codes", "code_off", "blk_params", "param_off", "row_consts", "row_nbits", "row_block", "had"):
        assert torch.equal(getattr(flat, f).cpu(), getattr(ref["flat"], f)), f


def test_end_to_end_own_statistics(cfg1):
    """The GPU path alone (its own second moment, statistics, table, allocation, factor): bits per
    weight, picks, and the Hessian-weighted error of the packed result against the oracle's."""
    from hi2_b200.allocate import allocate_global
    from hi2_b200.calibrate import Config, EncodeRequest, build_table, encode_many
    from hi2_b200.format import unpack_codes
    from hi2_b200.hessian import HessianStats
    from hi2_b200.stats import ColumnStats

    w, x, ref = cfg1
    r, k = w.shape
    cfg = Config()
    h = HessianStats(k, DEV)
    h.update(x.to(DEV))
    stats = ColumnStats.from_second_moment(h.S, h.n)
    table = build_table("w", w.to(DEV), stats, cfg)
    assert rel_close(table.sse.sum(1), ref["table"].sse.sum(1), 2e-3)
    alloc = allocate_global([table], 3.0)
    assert alloc.feasible and abs(alloc.bpw - ref["alloc"].bpw) < 1e-3
    assert (alloc.picks["w"].cpu() == ref["alloc"].picks["w"]).float().mean().item() >= 0.98
    (t,) = encode_many([EncodeRequest(w.to(DEV), stats, table, alloc.picks["w"], sigma=h.S, sigma_id="x", sigma_n=h.n)], cfg)
    hs, wt = ref["hs"].double(), ref["wt"].double()
    err = 0.0
    for cand_nb, cand_b in CANDS:
        rows = ((t.row_nbits == cand_nb) & (t.row_block == cand_b)).nonzero().flatten()
        if rows.numel() == 0:
            continue
        words = torch.stack([t.codes[t.code_off[i] : t.code_off[i + 1]] for i in rows.tolist()])
        codes = unpack_codes(words, cand_nb)
        p = torch.stack([t.blk_params[2 * t.param_off[i] : 2 * t.param_off[i + 1]].reshape(-1, 2) for i in rows.tolist()])
        err += weighted_error(ref["wt"][rows], ref["hs"], codes, p, t.row_consts[rows], cand_b)
    err_ref = sum(weighted_error(ref["wt"][rows], ref["hs"], e.codes, e.params, e.consts, b)
                  for rows, e, _, b in ref["pieces"])
    assert abs(err - err_ref) <= 0.01 * err_ref, (err, err_ref)


def test_wide_matrix_row_sample():
    """K = 11008 (the down projection of config 2/3), 160 rows, 4096 tokens: nearest tables and
    GPTQ for three candidates against the oracle on identical inputs."""
    from hi2_b200.encode import encode_rows
    from hi2_b200.hessian import encode_rows_gptq

    k, rows, tokens = 11008, 160, 4096
    g = gen(31)
    w = (torch.randn(rows, k, generator=g) * 0.02).bfloat16().float()
    x = (torch.randn(tokens, k, generator=g) * torch.exp(1.5 * torch.randn(1, k, generator=g))).bfloat16()
    sm = po.SecondMoment(k)
    sm.update(x)
    had = torch.ones(k // 16, dtype=torch.uint8)
    hs = po.stored_basis_hessian(sm.mean(), None, had)
    u = po.inverse_cholesky(hs, 0.01)
    d = hs.diagonal().clone()
    wt = po.rotate_groups(w, had)
    for nb, b in [(2, 16), (2, 64), (4, 32)]:
        want = po.nearest_rows(wt, d, nb, b)
        got = encode_rows(wt.to(DEV), d.to(DEV), nb, b)
        assert torch.equal(got.params.cpu(), want.params) and torch.equal(got.codes.cpu(), want.codes)
        want = po.gptq_rows(wt, d, u, nb, b)
        got = encode_rows_gptq(wt.to(DEV), d.to(DEV), u.to(DEV), nb, b)
        assert torch.equal(got.params.cpu(), want.params) and torch.equal(got.consts.cpu(), want.consts)
        # 11008 dependent columns per row: one code that the fp32-grade (3 x TF32) trailing update
        # rounds the other way changes the rest of its row; the contract's bar, not a tighter one
        agree = (got.codes.cpu() == want.codes).float().mean().item()
        assert agree >= 0.999, (nb, b, agree)
        e_g = weighted_error(wt, hs, got.codes, got.params, got.consts, b)
        e_o = weighted_error(wt, hs, want.codes, want.params, want.consts, b)
        assert abs(e_g - e_o) <= 0.01 * e_o
