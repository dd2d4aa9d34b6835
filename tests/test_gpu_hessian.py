"""Second moment, group moments, basis change and inverse factor on the GPU."""

import pytest
import torch

from oracle import ptq_oracle as po
from tests.helpers import DEV, activations, correlated_layer, gen, rel_close

pytestmark = pytest.mark.gpu


def _direct(x):
    xd = x.double()
    return xd.T @ xd


def _norm_err(got, want):
    """Largest error of a second moment relative to sqrt(S_ii S_jj)."""
    want = want.double().cpu()
    scale = want.diagonal().clamp_min(1e-30).sqrt()
    return ((got.double().cpu() - want) / (scale[:, None] * scale[None, :])).abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_second_moment_small_path(golden, dtype):
    """Small problems and fp32 activations take the exact fp32 FMA product."""
    from hi2_b200.hessian import HessianStats

    st = golden["stats"]
    x = st["x"].to(dtype)
    h = HessianStats(64, DEV)
    h.update(x[:300].to(DEV), chunk=128)
    other = HessianStats(64, DEV)
    other.update(x[300:].to(DEV))
    h.merge(other)
    assert h.n == st["n"]
    want = _direct(x)
    assert _norm_err(h.S, want) < 1e-5
    if dtype == torch.float16:
        assert torch.allclose(h.S.cpu(), st["S"], rtol=1e-4, atol=1e-4)
        assert torch.allclose(h.mean().cpu(), st["mean"], rtol=1e-4, atol=1e-4)
    assert torch.equal(h.S, h.S.T)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tokens,k", [(4096, 512), (5000, 448), (20000, 1024), (9000, 2304)])
def test_second_moment_tensor_core_path(dtype, tokens, k):
    """tcgen05 paths (the first two sizes take the one-block kernel, the last two the CTA-pair
    kernel with 256 x 256 tiles): tokens not a multiple of 64, K not a multiple of the tile,
    several token splits; accumulated on top of an existing sum; exactly symmetric."""
    from hi2_b200.hessian import HessianStats

    x = activations(tokens, k, tokens + k, spread=1.0, dtype=dtype)
    want = _direct(x)
    h = HessianStats(k, DEV)
    h.update(x.to(DEV))
    scale = want.diagonal().clamp_min(1e-30).sqrt()
    err = ((h.S.double().cpu() - want) / (scale[:, None] * scale[None, :])).abs().max().item()
    assert err < 2e-5, err
    assert torch.equal(h.S, h.S.T)
    h.update(x[:1000].to(DEV))  # a second call adds to the sum
    want2 = want + _direct(x[:1000])
    err = ((h.S.double().cpu() - want2) / (scale[:, None] * scale[None, :])).abs().max().item()
    assert err < 2e-5 and h.n == tokens + 1000
    # the oracle (fp32 products per 4096-token run) agrees within the reference's own tolerance
    o = po.SecondMoment(k)
    o.update(x)
    o.update(x[:1000])
    assert torch.allclose(h.S.cpu(), o.S, rtol=1e-4, atol=1e-4 * float(o.S.abs().max()))


def test_group_moments_and_diag(golden):
    from hi2_b200.hessian import HessianStats
    from hi2_b200.stats import ColumnStats
    from hi2_b200.calibrate import smoothing_scale

    st = golden["stats"]
    h = HessianStats(64, DEV)
    h.update(st["x"].to(DEV))
    c = ColumnStats.from_second_moment(h.S, h.n)
    blocks = torch.block_diag(*st["G"])
    got = torch.block_diag(*c.S.cpu())
    assert _norm_err(got, blocks) < 1e-5
    assert rel_close(c.diag(), st["diag_plain"], 1e-5)
    assert rel_close(c.diag(st["had"].to(DEV)), st["diag_rot"], 1e-5)
    s16 = smoothing_scale(c, 0.5)
    assert (s16.cpu() == st["s16"]).float().mean() >= 0.95  # fp16 rounding of a 1e-6-different input
    assert rel_close(s16.float(), st["s16"].float(), 1e-3)
    inv = 1.0 / st["s16"].float()
    assert rel_close(c.diag(st["had"].to(DEV), inv.to(DEV)), st["diag_rot_inv"], 1e-5)
    c2 = ColumnStats(64, DEV)
    c2.update(st["x"][:300].to(DEV))
    c2.update(st["x"][300:].to(DEV))
    assert c2.n == c.n and _norm_err(torch.block_diag(*c2.S.cpu()), blocks) < 1e-6


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_group_moments_from_activations(dtype):
    """Tokens beyond one 4096-run, K not a multiple of the 128-column block of a thread block."""
    from hi2_b200.stats import ColumnStats

    x = activations(9000, 208, 3, dtype=dtype)
    c = ColumnStats(208, DEV)
    c.update(x.to(DEV))
    o = po.GroupMoments(208)
    o.update(x)
    assert c.n == o.n
    assert _norm_err(torch.block_diag(*c.S.cpu()), torch.block_diag(*o.S)) < 1e-6
    flags = torch.ones(13, dtype=torch.uint8)
    assert rel_close(c.diag(flags.to(DEV)), o.diag(flags), 1e-5)


def test_transform_sigma_fixture(golden):
    from hi2_b200.hessian import transform_sigma

    b = golden["basis"]
    sig = b["sigma"].to(DEV)
    for cs, had, key in ((b["s16"], b["had"], "hs"), (None, b["had"], "hs_noscale"),
                         (None, torch.zeros(4, dtype=torch.uint8), "hs_plain")):
        hs = transform_sigma(sig, cs, had)
        assert torch.allclose(hs.cpu(), b[key], rtol=1e-5, atol=1e-6 * float(b[key].abs().max())), key
        assert torch.equal(hs, hs.T)


@pytest.mark.parametrize("k", [192, 1024, 2096])
def test_transform_sigma_against_oracle(k):
    from hi2_b200.hessian import transform_sigma

    g = gen(k)
    x = activations(3 * k, k, k, dtype=torch.float32)
    s = x.T @ x  # raw sum; the kernel divides by the token count on the fly
    n = x.shape[0]
    s16 = (torch.rand(k, generator=g) * 3 + 0.2).half()
    had = (torch.rand(k // 16, generator=g) < 0.6).to(torch.uint8)
    want = po.stored_basis_hessian(s / n, s16, had)
    hs, diag = transform_sigma(s.to(DEV), s16, had, denom=float(n), return_diag=True)
    tol = 1e-6 * float(want.abs().max())
    assert torch.allclose(hs.cpu(), want, rtol=2e-5, atol=tol)
    assert torch.equal(diag, hs.diagonal()) and torch.equal(hs, hs.T)


@pytest.mark.parametrize("k", [96, 192, 1024, 2096])
def test_inverse_factor(k):
    from hi2_b200.hessian import inverse_factor

    _, _, u_want, _, hs = correlated_layer(2, k, 31 + k)
    u = inverse_factor(hs.to(DEV), 0.01)
    assert torch.equal(u, u.triu()) and bool((u.diagonal() > 0).all())
    # the oracle is fp32 LAPACK, itself ~1.5e-5 of max|U| away from an fp64 solution; the kernel
    # (fp32 products, fp64 leaves) is as close to that solution as the oracle is
    rel = ((u.cpu() - u_want).abs().max() / u_want.abs().max()).item()
    assert rel < 6e-5, rel
    J = torch.arange(k - 1, -1, -1)
    lam64 = (0.01 * hs.diagonal().mean()).double()
    truth = torch.linalg.inv(torch.linalg.cholesky((hs.double() + lam64 * torch.eye(k, dtype=torch.float64))[J][:, J]))[J][:, J]
    ours = ((u.double().cpu() - truth).abs().max() / truth.abs().max()).item()
    theirs = ((u_want.double() - truth).abs().max() / truth.abs().max()).item()
    assert ours < max(3 * theirs, 2e-5), (ours, theirs)
    # U^T U (hs + lam I) = I
    lam = 0.01 * hs.diagonal().mean()
    prod = (u.double().cpu().T @ u.double().cpu()) @ (hs.double() + lam * torch.eye(k, dtype=torch.float64))
    assert (prod - torch.eye(k, dtype=torch.float64)).abs().max().item() < 1e-3


def test_inverse_factor_fixture_and_retry(golden):
    from hi2_b200.hessian import inverse_factor

    f = golden["factor"]
    u = inverse_factor(f["hs"].to(DEV), 0.01)
    assert torch.allclose(u.cpu(), f["u"], rtol=1e-4, atol=1e-5 * float(f["u"].abs().max()))
    # rank 6 of 40 with almost no damping: early attempts meet a non-positive pivot or an
    # ill-conditioned factor; the result must invert the damped matrix it settled on
    u = inverse_factor(f["sing"].to(DEV), 1e-9)
    assert bool(torch.isfinite(u).all())
    with pytest.raises(RuntimeError):
        inverse_factor(-torch.eye(32, device=DEV), 0.01)
