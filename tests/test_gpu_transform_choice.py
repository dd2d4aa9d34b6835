"""Transform selection on the GPU (hi2/calibrate.py:114-209): per-chunk rotation flags chosen on a
row sample, the smoothing exponent searched by the INT2/B32 error of the sample; against the
reference's own choices (fixture) and the oracle's."""

import pytest
import torch

from oracle import ptq_oracle as po
from tests.helpers import DEV, transform_case

pytestmark = pytest.mark.gpu


def _device_stats(x, k):
    from hi2_b200.stats import ColumnStats

    st = ColumnStats(k, DEV)
    st.update(x.to(DEV))
    return st


def test_shared_transform_matches_reference_choices():
    from hi2_b200.calibrate import Config, _fixed_transform, shared_transform, transform_error

    cases = torch.load(__import__("pathlib").Path(__file__).parent / "golden" / "transform_golden.pt", weights_only=False)
    for c in cases:
        ws, x = transform_case(c["seed"], c["k"], c["rows"])
        wd = [w.to(DEV) for w in ws]
        stats = _device_stats(x, c["k"])
        cfg = Config(rotation=c["mode"], smooth=c["alpha"], smooth_search=c["search"], effort="fast")
        s16, had = shared_transform(wd, stats, cfg)
        if c["s16"] is None:
            assert s16 is None
        else:  # the moments are summed in another order on the device: fp16 values, a few may sit on a boundary
            same = (s16.cpu() == c["s16"]).float().mean().item()
            assert same >= 0.98 and torch.allclose(s16.cpu().float(), c["s16"].float(), rtol=2e-3)
        agree = (had == c["had"]).float().mean().item()
        assert agree >= 0.97, (c["seed"], agree)  # a chunk whose two errors are within rounding may flip
        for alpha, want in c["costs"].items():
            s_a, had_a = _fixed_transform(wd, stats, cfg, alpha)
            got = transform_error(wd, stats, s_a, had_a)
            assert abs(got - want) <= 2e-3 * want, (alpha, got, want)


def test_choose_rotation_given_oracle_statistics():
    """Same statistics in (the oracle's fp64 group moments copied to the device): the flags must be
    the oracle's, chunk for chunk."""
    from hi2_b200.calibrate import Config, choose_rotation
    from hi2_b200.stats import ColumnStats

    for seed, k, rows in [(7, 512, (700,)), (8, 1024, (2100,))]:
        ws, x = transform_case(seed, k, rows)
        gm = po.GroupMoments(k)
        gm.update(x)
        want = po.pick_rotation(ws[0], gm, "auto")
        st = ColumnStats.from_state({"S": gm.S, "n": gm.n, "k": k}, DEV)
        got = choose_rotation(ws[0].to(DEV), st, Config(rotation="auto"))
        assert 0 < int(want.sum()) < want.numel()  # a mixed case
        assert (got == want).float().mean().item() >= 0.99
    assert int(choose_rotation(ws[0].to(DEV), st, Config(rotation="off")).sum()) == 0
    with pytest.raises(ValueError):
        choose_rotation(ws[0].to(DEV), st, Config(rotation="sometimes"))


def test_build_table_auto_rotation_and_search():
    from hi2_b200.calibrate import Config, build_table

    ws, x = transform_case(9, 256, (128,))
    stats = _device_stats(x, 256)
    t = build_table("w", ws[0].to(DEV), stats, Config(rotation="auto", smooth_search=(0.25, 0.75), effort="fast"))
    assert t.had.numel() == 16 and t.sse.shape == (6, 128) and bool(torch.isfinite(t.sse).all())
