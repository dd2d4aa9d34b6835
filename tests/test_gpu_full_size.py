"""BASELINE-size shapes (hidden 4096, FFN 11008) through properties that need no CPU oracle run:
round trips, symmetry, inverse identities, monotone error, budget hit."""

import pytest
import torch

from tests.helpers import DEV

pytestmark = pytest.mark.gpu


def _gen(seed):
    return torch.Generator(device=DEV).manual_seed(seed)


def test_second_moment_k11008_against_fp64_columns():
    from hi2_b200.hessian import HessianStats

    g = _gen(1)
    k, tokens = 11008, 16384
    x = (torch.randn(tokens, k, generator=g, device=DEV) * torch.exp(1.5 * torch.randn(1, k, generator=g, device=DEV))).bfloat16()
    h = HessianStats(k, DEV)
    h.update(x)
    assert h.n == tokens and torch.equal(h.S, h.S.T)
    cols = torch.randint(0, k, (48,), generator=g, device=DEV)
    want = x.double().T[cols] @ x.double()  # 48 rows of the exact product
    scale = (x.double() ** 2).sum(0).sqrt()
    err = ((h.S[cols].double() - want) / (scale[cols, None] * scale[None, :])).abs().max().item()
    assert err < 2e-5, err


def test_second_moment_wide_input_off_the_tile_grid():
    """Inputs wider than 8192 columns (the one-block tensor-core kernel): K past a multiple of the
    256-wide tile, a token count that is no multiple of the stage, and a second call on top."""
    from hi2_b200.hessian import HessianStats

    g = _gen(3)
    k, tokens = 8208, 40000 + 37
    x = (torch.randn(tokens, k, generator=g, device=DEV) * torch.exp(torch.randn(1, k, generator=g, device=DEV))).bfloat16()
    h = HessianStats(k, DEV)
    h.update(x)
    h.update(x[:9000])
    assert h.n == tokens + 9000 and torch.equal(h.S, h.S.T)
    cols = torch.cat([torch.randint(0, k, (40,), generator=g, device=DEV),
                      torch.tensor([0, 255, 256, 8191, 8192, 8207], device=DEV)])
    xd = x.double()
    want = xd.T[cols] @ xd + xd[:9000].T[cols] @ xd[:9000]
    scale = ((xd**2).sum(0) + (xd[:9000] ** 2).sum(0)).sqrt()
    err = ((h.S[cols].double() - want) / (scale[cols, None] * scale[None, :])).abs().max().item()
    assert err < 2e-5, err


def test_inverse_factor_k11008_inverts_the_damped_hessian():
    from hi2_b200.hessian import HessianStats, inverse_factor, transform_sigma

    g = _gen(2)
    k = 11008
    x = (torch.randn(2 * k, k, generator=g, device=DEV) * torch.exp(torch.randn(1, k, generator=g, device=DEV))).bfloat16()
    h = HessianStats(k, DEV)
    h.update(x)
    del x
    s16 = (torch.rand(k, generator=g, device=DEV) + 0.5).half()
    hs, d = transform_sigma(h.S, s16, torch.ones(k // 16, dtype=torch.uint8), denom=float(h.n), return_diag=True)
    assert torch.equal(hs, hs.T) and torch.equal(d, hs.diagonal())
    u = inverse_factor(hs, 0.01)
    assert torch.equal(u, u.triu()) and bool((u.diagonal() > 0).all())
    lam = 0.01 * hs.diagonal().mean()
    v = torch.randn(k, 8, generator=g, device=DEV, dtype=torch.float64)
    hv = hs.double() @ v + lam.double() * v
    back = u.double().T @ (u.double() @ hv)  # U^T U (Hs + lam I) v = v
    assert ((back - v).norm() / v.norm()).item() < 1e-3


def test_rotation_involution_and_pack_round_trip_at_full_size():
    from hi2_b200.format import fwht_groups, pack_codes, unpack_codes

    g = _gen(3)
    w = torch.randn(11008, 4096, generator=g, device=DEV)
    flags = torch.ones(256, dtype=torch.uint8)
    back = fwht_groups(fwht_groups(w, flags), flags)
    assert (back - w).abs().max().item() < 2e-6 * w.abs().max().item()
    for nbits in (2, 4, 8):
        codes = torch.randint(0, 2**nbits, (4096, 11008), generator=g, device=DEV, dtype=torch.uint8)
        words = pack_codes(codes, nbits)
        assert words.shape == (4096, 11008 * nbits // 32)
        assert torch.equal(unpack_codes(words, nbits).to(torch.uint8), codes)


def test_config1_layer_gptq_beats_nearest_and_hits_the_budget():
    """BASELINE config 1: 4096 x 4096 fp16 weights with 0.1 % outlier columns, 2048 tokens, 3.0 bpw.
    GPTQ must lower the Hessian error of nearest rounding (the reference's own acceptance test asks
    for 3 %), the allocation must land on the target, the packed buffers must be consistent."""
    from hi2_b200.allocate import allocate_global
    from hi2_b200.calibrate import Config, EncodeRequest, build_table, encode_many, stored_rows
    from hi2_b200.format import unpack_codes
    from hi2_b200.hessian import HessianStats, transform_sigma
    from hi2_b200.stats import ColumnStats

    g = _gen(4)
    k = r = 4096
    w = torch.randn(r, k, generator=g, device=DEV) * 0.02
    w[:, torch.randperm(k, generator=g, device=DEV)[:4]] *= 20
    w = w.half()
    x = (torch.randn(2048, k, generator=g, device=DEV) * torch.exp(torch.randn(1, k, generator=g, device=DEV))).half()
    h = HessianStats(k, DEV)
    h.update(x)
    stats = ColumnStats.from_second_moment(h.S, h.n)
    cfg = Config()
    table = build_table("w", w, stats, cfg)
    alloc = allocate_global([table], 3.0)
    assert alloc.feasible and 2.99 < alloc.bpw <= 3.0
    picks = alloc.picks["w"]
    hs = transform_sigma(h.S, table.col_scale, table.had, denom=float(h.n)).double()
    wt = stored_rows(w, table.col_scale, table.had).double()

    def hessian_error(t):
        tot = 0.0
        rows = torch.arange(0, r, 16)  # every 16th row
        for row in rows.tolist():
            nb, b = int(t.row_nbits[row]), int(t.row_block[row])
            codes = unpack_codes(t.codes[t.code_off[row] : t.code_off[row + 1]], nb).double()
            p = t.blk_params[2 * t.param_off[row] : 2 * t.param_off[row + 1]].reshape(-1, 2).double()
            c = t.row_consts[row].double()
            lo = (p[:, 0] * c[1] + c[0]).float().half().double().repeat_interleave(b)
            st = (p[:, 1].float() * t.row_consts[row, 2].float()).half().double().repeat_interleave(b)
            e = (lo + codes * st).half().double().to(DEV) - wt[row]
            tot += float(e @ hs @ e)
        return tot

    req = EncodeRequest(w, stats, table, picks, sigma=h.S, sigma_id="x", sigma_n=h.n)
    (gptq,) = encode_many([req], cfg)
    (near,) = encode_many([EncodeRequest(w, stats, table, picks, sigma=None)], cfg)
    assert int(gptq.code_off[-1]) == gptq.codes.numel() and torch.equal(gptq.row_nbits, near.row_nbits)
    e_g, e_n = hessian_error(gptq), hessian_error(near)
    assert e_g < 0.97 * e_n, (e_g, e_n)


def test_widest_input_of_the_70b_shape():
    """K = 28672 (the FFN width of BASELINE config 4): second moment against exact columns, basis
    change, and the inverse factor through its defining identity.  The largest single matrices
    the path meets: S and U are 3.3 GB each."""
    from hi2_b200.hessian import HessianStats, inverse_factor, transform_sigma

    g = _gen(5)
    k, tokens = 28672, 32768
    x = (torch.randn(tokens, k, generator=g, device=DEV) * torch.exp(0.5 * torch.randn(1, k, generator=g, device=DEV))).bfloat16()
    h = HessianStats(k, DEV)
    h.update(x)
    assert h.n == tokens and torch.equal(h.S, h.S.T)
    cols = torch.randint(0, k, (16,), generator=g, device=DEV)
    want = x.double().T[cols] @ x.double()
    scale = (x.double() ** 2).sum(0).sqrt()
    err = ((h.S[cols].double() - want) / (scale[cols, None] * scale[None, :])).abs().max().item()
    assert err < 2e-5, err
    del x, want
    hs, d = transform_sigma(h.S, None, torch.ones(k // 16, dtype=torch.uint8), denom=float(h.n), return_diag=True)
    del h
    u = inverse_factor(hs, 0.01)
    assert torch.equal(u, u.triu()) and bool((u.diagonal() > 0).all())
    lam = 0.01 * hs.diagonal().mean()
    v = torch.randn(k, 4, generator=g, device=DEV)
    hv = (hs @ v + lam * v).double()
    back = (u.T.double() @ (u.double() @ hv)).float()
    rel = ((back - v).norm() / v.norm()).item()
    assert rel < 2e-3, rel


def test_empty_and_single_row_inputs():
    """Nothing to do is not an error (hi2/gptq_kernel.py:116), and one row is a full problem."""
    from hi2_b200.encode import encode_rows
    from hi2_b200.format import fwht_groups, pack_codes
    from hi2_b200.hessian import HessianStats, encode_rows_gptq, inverse_factor

    k = 256
    h = HessianStats(k, DEV)
    h.update(torch.zeros(0, k, device=DEV, dtype=torch.bfloat16))
    assert h.n == 0 and not h.S.any()
    g = _gen(6)
    x = torch.randn(600, k, generator=g, device=DEV).bfloat16()
    h.update(x)
    u = inverse_factor(h.S / h.n, 0.01)
    d = (h.S / h.n).diagonal().contiguous()
    none = encode_rows_gptq(torch.zeros(0, k, device=DEV), d, u, 2, 32)
    assert none.codes.shape == (0, k) and none.sse.numel() == 0
    one = encode_rows_gptq(torch.randn(1, k, generator=g, device=DEV) * 0.02, d, u, 4, 16)
    assert one.codes.shape == (1, k) and int(one.codes.max()) <= 15
    assert encode_rows(torch.zeros(0, k, device=DEV), d, 2, 16).codes.shape == (0, k)
    assert pack_codes(torch.zeros(0, k, dtype=torch.uint8, device=DEV), 2).shape == (0, k // 16)
    assert fwht_groups(torch.zeros(0, k, device=DEV), torch.ones(k // 16, dtype=torch.uint8)).shape == (0, k)
