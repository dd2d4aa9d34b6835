"""Regenerate ``ptq_golden.pt``: seeded inputs and the outputs hi2 itself gives for them.

Run in a container that has the hi2 sources:

    PYTHONPATH=<hi2 checkout> HI2_GPTQ_BACKEND=torch HI2_LADDER_BACKEND=torch \
        HI2_REFINE_BACKEND=torch python tests/golden/make_golden.py

The fixture is the pin for ``oracle/ptq_oracle.py`` (tests/test_oracle_golden.py) and a second
checker for the CUDA path (tests/test_gpu_*.py).  Nothing else reads hi2 at test time.
"""

import os
import sys
from pathlib import Path

import torch

os.environ.setdefault("HI2_GPTQ_BACKEND", "torch")
os.environ.setdefault("HI2_LADDER_BACKEND", "torch")
os.environ.setdefault("HI2_REFINE_BACKEND", "torch")

from hi2 import allocate as h_alloc  # noqa: E402
from hi2 import calibrate as h_cal  # noqa: E402
from hi2 import encode as h_enc  # noqa: E402
from hi2 import format as h_fmt  # noqa: E402
from hi2 import hessian as h_hes  # noqa: E402
from hi2 import refine as h_ref  # noqa: E402
from hi2 import stats as h_sta  # noqa: E402

CASES = [(2, 16), (2, 32), (2, 64), (4, 16), (4, 32), (4, 64), (8, 32), (8, 64)]


def gen(seed):
    return torch.Generator().manual_seed(seed)


def layer(rows, k, seed, act_order=False):
    """A correlated activation sample, its second moment and a weight tile with outlier
    columns (same recipe family as the reference's GPTQ tests, sizes kept small)."""
    g = gen(seed)
    mix = torch.randn(k, k, generator=g) * 0.1 + torch.eye(k)
    x = torch.randn(4 * k, k, generator=g) @ mix
    x *= torch.exp(0.5 * torch.randn(1, k, generator=g))
    hs = x.T @ x / x.shape[0]
    w = torch.randn(rows, k, generator=g) * torch.exp(0.4 * torch.randn(rows, 1, generator=g))
    w[:, :: max(1, k // 5)] *= 8
    d = hs.diagonal().clone()
    perm = None
    if act_order:
        perm = torch.argsort(d, descending=True)
        hs = hs[perm][:, perm]
    u = h_hes.inverse_factor(hs, 0.01)
    return w, d, u, perm, hs


def enc_dict(e):
    out = {"codes": e.codes, "params": e.params, "consts": e.consts, "sse": e.sse}
    if e.comp is not None:
        out["comp"] = e.comp
    return out


def main():
    out = {}

    # rotation -------------------------------------------------------------------------
    g = gen(1)
    flags = torch.tensor([1, 0, 1, 1, 0, 1], dtype=torch.uint8)
    rot = {"flags": flags}
    for name, dt in (("f32", torch.float32), ("f64", torch.float64), ("f16", torch.float16),
                     ("bf16", torch.bfloat16)):
        x = (torch.randn(7, 96, generator=g, dtype=torch.float64) * 3).to(dt)
        rot[name] = {"x": x, "y": h_fmt.fwht_groups(x, flags)}
    xb = torch.randn(33, 512, generator=g)
    rot["f32_all"] = {"x": xb, "y": h_fmt.fwht_groups(xb, torch.ones(32, dtype=torch.uint8))}
    out["rotation"] = rot

    # statistics -----------------------------------------------------------------------
    g = gen(2)
    k = 64
    x = (torch.randn(700, k, generator=g) * torch.exp(torch.randn(1, k, generator=g))).half()
    hstat = h_hes.HessianStats(k)
    hstat.update(x[:300], chunk=128)
    hstat.update(x[300:], chunk=128)
    cstat = h_sta.ColumnStats(k)
    cstat.update(x)
    had = torch.tensor([1, 0, 1, 1], dtype=torch.uint8)
    s16 = h_cal.smoothing_scale(cstat, 0.5)
    inv = 1.0 / s16.float()
    out["stats"] = {
        "x": x, "S": hstat.S, "n": hstat.n, "mean": hstat.mean(),
        "G": cstat.S, "diag_plain": cstat.diag(), "had": had,
        "diag_rot": cstat.diag(had), "diag_rot_inv": cstat.diag(had, inv), "s16": s16,
    }
    sigma = hstat.mean()
    out["basis"] = {
        "sigma": sigma, "s16": s16, "had": had,
        "hs": h_hes.transform_sigma(sigma, s16, had),
        "hs_noscale": h_hes.transform_sigma(sigma, None, had),
        "hs_plain": h_hes.transform_sigma(sigma, None, torch.zeros(4, dtype=torch.uint8)),
    }

    # inverse factor ---------------------------------------------------------------------
    _, _, u, _, hs = layer(4, 96, 3)
    g = gen(4)
    low = torch.randn(40, 6, generator=g)
    sing = low @ low.T  # rank 6 of 40: needs the damping to be factorisable
    out["factor"] = {"hs": hs, "u": u, "sing": sing, "u_sing": h_hes.inverse_factor(sing, 1e-9)}

    # ladder search ----------------------------------------------------------------------
    g = gen(5)
    lad = []
    for b in (16, 32, 64):
        for n in (4, 16, 256):
            for effort in ("fast", "normal", "max"):
                wb = torch.randn(9, 5, b, generator=g) * torch.exp(torch.randn(9, 5, 1, generator=g))
                wb[0, 0] = 0.25  # constant block
                db = torch.rand(1, 5, b, generator=g) + 0.1
                lo, st = h_enc.fit_ladder(wb, db, n, effort)
                lad.append({"wb": wb, "db": db, "n": n, "effort": effort, "lo": lo, "step": st})
    out["ladder"] = lad

    g = gen(6)
    lo = torch.randn(6, 12, generator=g)
    st = torch.rand(6, 12, generator=g) * 0.1
    st[1] = 0.0
    lo[2] = 0.5
    lo_u8, st_u8, consts = h_enc.quantize_params(lo, st)
    dlo, dst = h_fmt.decode_params(lo_u8, st_u8, consts[:, 0:1], consts[:, 1:2], consts[:, 2:3])
    out["params"] = {"lo": lo, "step": st, "lo_u8": lo_u8, "step_u8": st_u8, "consts": consts,
                     "lo_d": dlo, "step_d": dst}

    # nearest rows -----------------------------------------------------------------------
    g = gen(7)
    w = torch.randn(7, 192, generator=g) * torch.exp(0.5 * torch.randn(7, 1, generator=g))
    w[:, 5] *= 10
    d = torch.rand(192, generator=g) + 0.05
    near = {"w": w, "d": d, "cases": {}}
    for nb, b in CASES:
        for effort in ("fast", "normal"):
            near["cases"][(nb, b, effort)] = enc_dict(h_enc.encode_rows(w, d, nb, b, effort))
    out["nearest"] = near

    # GPTQ -------------------------------------------------------------------------------
    gp = []
    for act in (False, True):
        for k in (192, 256):
            w, d, u, perm, hs = layer(10, k, 100 + k + int(act), act)
            entry = {"w": w, "d": d, "u": u, "perm": perm, "cases": {}}
            for nb, b in CASES:
                if k % b:
                    continue
                e = h_hes.encode_rows_gptq_reference(w, d, u, nb, b, "normal", perm)
                entry["cases"][(nb, b)] = enc_dict(e)
            gp.append(entry)
    out["gptq"] = gp

    # refinement -------------------------------------------------------------------------
    w, d, u, _, hs = layer(9, 256, 11)
    groups, res = [], []
    for nb, b in ((2, 32), (4, 64)):
        rows = w[:5] if nb == 2 else w[5:]
        e = h_hes.encode_rows_gptq_reference(rows, d, u, nb, b, "normal")
        groups.append((rows, e, nb, b))
    new = h_ref.refine_groups(groups, hs, 2)
    out["refine"] = {
        "hs": hs,
        "groups": [{"w": gw, "enc": enc_dict(ge), "nbits": nb, "block": b}
                   for gw, ge, nb, b in groups],
        "codes": new,
    }

    # packing ----------------------------------------------------------------------------
    g = gen(12)
    pk = {}
    for nb in (2, 4, 8):
        c = torch.randint(0, 2**nb, (5, 128), generator=g)
        pk[nb] = {"codes": c, "words": h_fmt.pack_codes(c, nb)}
    r, k = 6, 128
    w = torch.randn(r, k, generator=g)
    nbits = torch.tensor([2, 4, 2, 4, 8, 2])
    block = torch.tensor([32, 64, 64, 32, 64, 16])
    pieces = []
    for nb in (2, 4, 8):
        for b in (16, 32, 64):
            rows = ((nbits == nb) & (block == b)).nonzero().flatten()
            if rows.numel():
                e = h_enc.encode_rows(w[rows], torch.ones(k), nb, b, "fast")
                pieces.append((rows, e.codes, e.params, e.consts))
    had = torch.tensor([1, 0, 1, 0, 1, 1, 0, 0], dtype=torch.uint8)
    t = h_fmt.assemble(pieces, nbits, block, had, k)
    pk["assemble"] = {
        "pieces": pieces, "row_nbits": nbits, "row_block": block, "had": had, "k": k,
        "out": {f: getattr(t, f) for f in h_fmt.FIELDS},
    }
    out["pack"] = pk

    # allocation -------------------------------------------------------------------------
    g = gen(13)
    tabs = []
    for i, (r, k, cands) in enumerate(
        [(40, 256, h_cal.ALL_CANDIDATES), (24, 512, h_cal.ALL_CANDIDATES),
         (16, 256, h_cal.ALL_CANDIDATES + h_cal.INT8_CANDIDATES)]
    ):
        base = torch.rand(1, r, generator=g) + 0.2
        bits = torch.tensor([nb + 16 / b for nb, b in cands]).reshape(-1, 1)
        sse = (base * 4.0 ** (-bits) * (1 + 0.3 * torch.rand(len(cands), r, generator=g))).float()
        cs = None if i == 1 else torch.ones(k, dtype=torch.float16)
        tabs.append(dict(name=f"t{i}", shape=(r, k), had=torch.ones(k // 16, dtype=torch.uint8),
                         sse=sse, candidates=list(cands), energy=float(3.0 + i), n_tokens=10,
                         col_scale=cs))
    tables = [h_cal.TensorTable(**t) for t in tabs]
    allocs = {}
    for target in (2.2, 2.6, 3.0, 4.5, 9.0):
        a = h_alloc.allocate_global(tables, target, {"t1": 2.0})
        allocs[target] = {"picks": a.picks, "bpw": a.bpw, "lam": a.lam, "feasible": a.feasible}
    out["allocate"] = {"tables": tabs, "sens": {"t1": 2.0}, "results": allocs}

    path = Path(__file__).with_name("ptq_golden.pt")
    torch.save(out, path)
    print(f"wrote {path} ({path.stat().st_size / 1024:.0f} KiB)", file=sys.stderr)


if __name__ == "__main__":
    main()
