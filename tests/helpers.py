"""Seeded inputs and comparison helpers shared by the GPU parity tests."""

import torch

from oracle import ptq_oracle as po

CASES = [(2, 16), (2, 32), (2, 64), (4, 16), (4, 32), (4, 64), (8, 32), (8, 64)]
DEV = "cuda"


def gen(seed):
    return torch.Generator().manual_seed(seed)


def weights(rows, k, seed, outliers=True):
    g = gen(seed)
    w = torch.randn(rows, k, generator=g) * torch.exp(0.4 * torch.randn(rows, 1, generator=g))
    if outliers:
        w[:, :: max(1, k // 5)] *= 8
    return w


def activations(tokens, k, seed, spread=1.0, dtype=torch.float16):
    g = gen(seed)
    x = torch.randn(tokens, k, generator=g) * torch.exp(spread * torch.randn(1, k, generator=g))
    return x.to(dtype)


def correlated_layer(rows, k, seed, act_order=False):
    """Weights, ladder weights d, factor u (oracle, CPU) and Hessian hs of a correlated input."""
    g = gen(seed)
    mix = torch.randn(k, k, generator=g) * 0.1 + torch.eye(k)
    x = torch.randn(4 * k, k, generator=g) @ mix
    x *= torch.exp(0.5 * torch.randn(1, k, generator=g))
    hs = x.T @ x / x.shape[0]
    w = weights(rows, k, seed + 1)
    d = hs.diagonal().clone()
    perm = None
    if act_order:
        perm = torch.argsort(d, descending=True)
        hs = hs[perm][:, perm]
    u = po.inverse_cholesky(hs, 0.01)
    return w, d, u, perm, hs


def agreement(a, b):
    return (a.cpu() == b.cpu()).float().mean().item()


def rel_close(a, b, rtol, atol=0.0):
    a, b = a.double().cpu(), b.double().cpu()
    return bool(((a - b).abs() <= atol + rtol * b.abs()).all())


def decoded(params, consts):
    lo, st = po.decode_ladders(params[..., 0].cpu(), params[..., 1].cpu(), consts[:, 0:1].cpu(),
                               consts[:, 1:2].cpu(), consts[:, 2:3].cpu())
    return lo.float(), st.float()


def weighted_error(w, hs, codes, params, consts, block):
    """Sum over rows of e Hs e^T for the stored-basis rows w (CPU, fp64)."""
    lo, st = decoded(params, consts)
    idx = torch.arange(w.shape[1]) // block
    rec = (lo[:, idx] + codes.cpu().float() * st[:, idx]).half().double()
    e = rec - w.double().cpu()
    return float(((e @ hs.double().cpu()) * e).sum())


def ladder_report(got, want):
    """How far two encodings of the same rows agree: share of rows whose ladders (parameter bytes
    and row constants) are identical, share of rows whose constants agree to 1e-3, share of equal
    parameter bytes and codes, and share of equal codes inside the rows with identical ladders."""
    gp, gc, gk = got.params.cpu(), got.consts.cpu(), got.codes.cpu()
    same = (gp == want.params).all(-1).all(-1) & (gc == want.consts).all(-1)
    cf, wf = gc.float(), want.consts.float()
    consts_ok = ((cf - wf).abs() <= 1e-3 * wf.abs() + 1e-6).all(-1)
    return dict(
        rows_same=same.float().mean().item(),
        consts_ok=consts_ok.float().mean().item(),
        params=(gp == want.params).float().mean().item(),
        codes=(gk == want.codes).float().mean().item(),
        codes_same_rows=(gk[same] == want.codes[same]).float().mean().item() if bool(same.any()) else 1.0,
        same=same,
    )


def config1_inputs(rows=4096, k=4096, tokens=2048, seed=2024):
    """BASELINE config 1: a 4096 x 4096 fp16 Linear, N(0, 0.02), 0.1 % of the input columns x 20;
    2048 tokens of fp16 activations, N(0, 1) times a per-channel lognormal(0, 1) scale."""
    g = gen(seed)
    w = torch.randn(rows, k, generator=g) * 0.02
    cols = torch.randperm(k, generator=g)[: max(1, k // 1000)]
    w[:, cols] *= 20
    x = torch.randn(tokens, k, generator=g) * torch.exp(torch.randn(1, k, generator=g))
    return w.half(), x.half()


def oracle_layer(w, x, candidates, target, keep_codes=True):
    """The reference's chain for one Linear on the CPU oracle: statistics, smoothing vector, table,
    allocation, basis change, factor, GPTQ per candidate group, flat-buffer assembly."""
    k = w.shape[1]
    sm = po.SecondMoment(k)
    sm.update(x)
    gm = po.GroupMoments(k)
    gm.update(x)
    s16 = po.smoothing_vector(gm, 0.5)
    had = torch.ones(k // 16, dtype=torch.uint8)
    wt = po.rotate_groups(w.float() * s16.float(), had)
    d_tab = gm.diag(had, 1.0 / s16.float())
    sse = torch.stack([po.nearest_rows(wt, d_tab, nb, b).sse for nb, b in candidates])
    table = po.Table("w", tuple(w.shape), had, sse, list(candidates), float((d_tab * wt**2).sum()),
                     x.shape[0], s16)
    alloc = po.allocate_rows([table], target)
    hs = po.stored_basis_hessian(sm.mean(), s16, had)
    u = po.inverse_cholesky(hs, 0.01)
    d = hs.diagonal().clone()
    pieces = []
    picks = alloc.picks["w"]
    for ci, (nb, b) in enumerate(candidates):
        rows = (picks == ci).nonzero().flatten()
        if rows.numel():
            pieces.append((rows, po.gptq_rows(wt[rows], d, u, nb, b), nb, b))
    cand = torch.tensor(candidates)
    flat = po.assemble_flat([(r, e.codes, e.params, e.consts) for r, e, _, _ in pieces], cand[picks, 0],
                            cand[picks, 1], had, k, s16)
    return dict(sm=sm, gm=gm, s16=s16, had=had, wt=wt, d_tab=d_tab, table=table, alloc=alloc, hs=hs, u=u, d=d,
                pieces=pieces, flat=flat)


def transform_case(seed, k, rows):
    """Linears that read one input (list of [R_i, K] fp32) and its activations: columns with very
    different scales, a few heavy-tailed groups, so that rotation helps some chunks and not others."""
    g = gen(1000 + seed)
    ws = []
    for r in rows:
        w = torch.randn(r, k, generator=g) * 0.05
        w[:, : k // 4] *= torch.exp(1.5 * torch.randn(1, k // 4, generator=g))  # spiky first quarter
        ws.append(w)
    x = torch.randn(2048, k, generator=g) * torch.exp(torch.randn(1, k, generator=g))
    return ws, x.half()


def toy_llama(layers=2, hidden=64, ffn=128, heads=2, vocab=256, sequences=6, tokens=48, seed=0):
    """A Llama-shaped fp32 toy model with seeded weights and seeded calibration ids."""
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers, num_attention_heads=heads,
                      num_key_value_heads=heads, vocab_size=vocab, max_position_embeddings=4 * tokens)
    torch.manual_seed(seed)
    model = LlamaForCausalLM(cfg).eval()
    ids = torch.randint(0, vocab, (sequences, tokens), generator=gen(seed + 1))
    return model, ids


def toy_olmoe(layers=2, hidden=64, ffn=32, heads=2, vocab=128, experts=4, top_k=2, sequences=6, tokens=48, seed=0):
    """An OLMoE-shaped fp32 toy model (fused 3-D expert parameters, as ``transformers`` stores them)
    with seeded weights and seeded calibration ids."""
    from transformers import OlmoeConfig, OlmoeForCausalLM

    cfg = OlmoeConfig(hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers, num_attention_heads=heads,
                      num_key_value_heads=heads, vocab_size=vocab, num_experts=experts, num_experts_per_tok=top_k,
                      max_position_embeddings=4 * tokens)
    torch.manual_seed(seed)
    model = OlmoeForCausalLM(cfg).eval()
    ids = torch.randint(0, vocab, (sequences, tokens), generator=gen(seed + 1))
    return model, ids
