"""Patadra on the GPU against the plain implementation of tests/patadra_oracle.py (float64): every mechanism alone,
then the model through the engine — whole prompts, token-by-token decoding, portions down to two tokens, mixed
batches against each request alone, reused pages, keys far away, at page borders and just inside / outside the
window, the first tokens, decoding far past the window, other sizes, greedy generation through the scheduler."""
import json
import math

import numpy as np
import pytest
import torch

import patadra_oracle as po

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
BOTH = [torch.float32, torch.bfloat16]


def _ops():
    from atoma_infer_b200 import hybrid_ops
    return hybrid_ops


@pytest.fixture(autouse=True)
def _reset_flags():
    yield
    if torch.cuda.is_available():
        _ops().debug_flags(0)


def nerr(got, want):
    got, want = torch.as_tensor(got).double().cpu(), torch.as_tensor(want).double().cpu()
    return float(((got - want) ** 2).mean().sqrt() / (want ** 2).mean().sqrt().clamp_min(1e-30))


def tol(dtype, f32=1e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


def model_close(got, want, dtype, f32=1e-5):
    """Whole-model comparison.  float32: the sharp one, over all rows.  bfloat16: rounding the router's input can flip the choice
    between two experts whose scores nearly tie, which changes that token's row (and, diluted, later ones) by far more than
    rounding does elsewhere — so the bound is on the typical row (median of the per-row errors), with a loose one on the whole."""
    if dtype == torch.float32:
        return nerr(got, want) < f32
    got, want = torch.as_tensor(got).double().cpu(), torch.as_tensor(want).double().cpu()
    rows = ((got - want) ** 2).mean(-1).sqrt() / (want ** 2).mean(-1).sqrt().clamp_min(1e-30)
    return float(rows.median()) < 8e-2 and nerr(got, want) < 0.5


def bf(t):
    """float32 values that bfloat16 holds exactly"""
    return t.to(torch.bfloat16).float()


# ------------------------------------------------------------------------------------------------
# row operators
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", BOTH)
def test_embedding_with_learned_positions(dtype):
    g = torch.Generator().manual_seed(0)
    table, pos = bf(torch.randn(20, 34, generator=g)), bf(torch.randn(50, 34, generator=g))
    toks, p = torch.tensor([3, 19, 0, 7, 7], dtype=torch.int32), torch.tensor([0, 1, 49, 17, 18], dtype=torch.int64)
    got = _ops().embed_learned(toks.to(DEV), p.to(DEV), table.to(dtype).to(DEV), pos.to(dtype).to(DEV))
    assert torch.equal(got.cpu(), po.embed(toks.long(), p, table, pos))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("width,groups", [(48, 1), (48, 3), (50, 2), (35, 5), (64, 64)])
def test_norm_over_groups_of_the_row(dtype, width, groups):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, width, generator=g) * 3
    x[:, : width // groups] *= 20          # a loud first group must not quieten the others
    w = 1 + 0.3 * torch.randn(width, generator=g)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    got = _ops().group_rmsnorm_rows(x.to(DEV), w.to(DEV), 0.0, groups, 1e-5, dtype)
    assert nerr(got, po.group_norm(x.double(), w.double(), groups, 1e-5)) < tol(dtype, 2e-6, 4e-3)
    got = _ops().group_rmsnorm_rows(x.to(DEV), w.to(DEV), 1.0, groups, 1e-5, dtype, rows=rows.to(DEV))
    assert nerr(got, po.group_norm(x.double()[rows.long()], 1 + w.double(), groups, 1e-5)) < tol(dtype, 2e-6, 4e-3)


@pytest.mark.parametrize("dtype", BOTH)
def test_gated_residual_update_with_the_next_norm(dtype):
    g = torch.Generator().manual_seed(2)
    T, W, groups, eps = 7, 50, 5, 1e-5
    x0 = torch.randn(T, W, generator=g) * 2
    wide = (torch.randn(T, 30 + W, generator=g)).to(dtype)            # the gate is a column slice of a wider projection
    y, bias, wn = torch.randn(T, W, generator=g).to(dtype), torch.randn(W, generator=g), 1 + 0.2 * torch.randn(W, generator=g)
    rs = torch.rand(T, generator=g)
    eo = torch.randn(12, W, generator=g).to(dtype)
    pr = torch.randint(0, 12, (T, 2), generator=g).to(torch.int32)
    wide_d = wide.to(DEV)
    # mixer form: gate, no experts
    x = x0.clone().to(DEV)
    h, xc = _ops().gated_residual_norm(x, y=y.to(DEV), gate=wide_d[:, 30:], gate_bias=bias.to(DEV), w_next=wn.to(DEV), groups=groups, eps=eps)
    want = x0.double() + y.double() * po.sigma(wide.double()[:, 30:] + bias.double())
    assert nerr(x, want) < 1e-6 and xc is None
    assert nerr(h, po.group_norm(want, wn.double(), groups, eps)) < tol(dtype, 2e-6, 4e-3)
    # feed-forward form: expert rows summed, shared output scaled per row, a cast copy, no norm
    x = x0.clone().to(DEV)
    h, xc = _ops().gated_residual_norm(x, y=y.to(DEV), gate=wide_d[:, 30:], gate_bias=bias.to(DEV), row_scale=rs.to(DEV),
                                       expert_out=eo.to(DEV), pair_row=pr.to(DEV), top=2, want_cast=True)
    v = y.double() * rs.double()[:, None] + eo.double()[pr.long()[:, 0]] + eo.double()[pr.long()[:, 1]]
    want = x0.double() + v * po.sigma(wide.double()[:, 30:] + bias.double())
    assert h is None and nerr(x, want) < 1e-6 and nerr(xc, want) < tol(dtype, 1e-7, 4e-3)
    # no gate at all
    x = x0.clone().to(DEV)
    _ops().gated_residual_norm(x, y=y.to(DEV))
    assert nerr(x, x0.double() + y.double()) < 1e-6


@pytest.mark.parametrize("dtype", BOTH)
def test_token_side_input(dtype):
    g = torch.Generator().manual_seed(3)
    T, W, D, parts, V, eps = 6, 40, 5, 3, 11, 1e-5
    toks = torch.randint(0, V, (T,), generator=g).to(torch.int32)
    table = bf(torch.randn(V, parts * D, generator=g))
    wide = bf(torch.randn(T, D + 3, generator=g))
    got = _ops().side_gate(wide.to(dtype).to(DEV)[:, :D], toks.to(DEV), table.to(dtype).to(DEV), 1, D)
    want = po.gelu_tanh(wide.double()[:, :D]) * table.double()[toks.long()][:, D:2 * D]
    assert nerr(got, want) < tol(dtype, 1e-6, 4e-3)
    # the whole mechanism from its operators: gate projection, table product, back projection, unit RMS, add, next norm
    x0 = torch.randn(T, W, generator=g)
    wg, wp, wn, w2 = bf(torch.randn(D, W, generator=g) / 6), bf(torch.randn(W, D, generator=g)), torch.rand(W, generator=g), 1 + torch.rand(W, generator=g)
    xc = x0.to(dtype).to(DEV)
    a = _ops().linear(xc, wg.to(dtype).to(DEV))
    y = _ops().linear(_ops().side_gate(a, toks.to(DEV), table.to(dtype).to(DEV), 2, D), wp.to(dtype).to(DEV))
    x = x0.clone().to(DEV)
    h = _ops().unitnorm_add_norm(y, x, wn.to(DEV), w2.to(DEV), 2, eps)
    want = x0.double() + po.side_input(xc.double().cpu(), toks.long(), table.double(), 2, D, wg.double(), wp.double(), wn.double(), eps)
    assert nerr(x, want) < tol(dtype, 2e-6, 5e-3)
    assert nerr(h, po.group_norm(want, w2.double(), 2, eps)) < tol(dtype, 2e-6, 6e-3)


@pytest.mark.parametrize("dtype", BOTH)
def test_clamped_activation_and_capped_logits(dtype):
    g = torch.Generator().manual_seed(4)
    gu = bf(torch.randn(5, 2 * 24 + 7, generator=g) * 3)
    for limit in (1.5, 0.0):
        got = _ops().glu_clamped(gu.to(dtype).to(DEV), 24, limit, 1.702, 1.0)
        a, u = gu.double()[:, :24], gu.double()[:, 24:48]
        if limit > 0:
            a, u = a.clamp(max=limit), u.clamp(-limit, limit)
        assert nerr(got, a * po.sigma(1.702 * a) * (u + 1)) < tol(dtype, 1e-6, 4e-3)
    lg = bf(torch.randn(3, 37, generator=g) * 20)
    lg[1, 5] = lg[1, 30] = 200.0
    out, tok = _ops().finish_logits_greedy(lg.to(dtype).to(DEV), 1.0, 9.0)
    assert nerr(out, 9.0 * torch.tanh(lg.double() / 9.0)) < 1e-6
    assert tok.tolist()[1] == 30 and tok.tolist()[0] == int(lg[0].argmax())
    out, _ = _ops().finish_logits_greedy(lg.to(dtype).to(DEV), 0.5, 0.0)
    assert nerr(out, lg.double() * 0.5) < 1e-7


# ------------------------------------------------------------------------------------------------
# latent attention
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", BOTH)
def test_latent_norms_and_cache_write(dtype):
    g = torch.Generator().manual_seed(5)
    T, qr, kr, eps = 6, 20, 12, 1e-5
    proj = bf(torch.randn(T, qr + kr + 9, generator=g) * 2)
    nq, nk = 1 + 0.3 * torch.randn(qr, generator=g), 1 + 0.3 * torch.randn(kr, generator=g)
    slots = torch.tensor([7, 0, -1, 33, 2, 5], dtype=torch.int64)
    cache = torch.full((40, kr), 77.0, dtype=dtype, device=DEV)
    cq = _ops().latent_norm_cache(proj.to(dtype).to(DEV), nq.to(DEV), nk.to(DEV), slots.to(DEV), cache, qr, kr, eps)
    assert nerr(cq, po.unit_rms(proj.double()[:, :qr], eps) * nq.double()) < tol(dtype, 2e-6, 4e-3)
    want = po.unit_rms(proj.double()[:, qr:qr + kr], eps) * nk.double()
    keep = slots >= 0
    assert nerr(cache[slots[keep].to(DEV)], want[keep]) < tol(dtype, 2e-6, 4e-3)
    untouched = torch.ones(40, dtype=torch.bool)
    untouched[slots[keep]] = False
    assert bool((cache[untouched.to(DEV)] == 77.0).all())


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("T,H,n,R", [(5, 3, 8, 16), (70, 2, 20, 33), (130, 1, 64, 72)])
def test_per_head_projections_to_and_from_the_latent_space(dtype, T, H, n, R):
    g = torch.Generator().manual_seed(6)
    w = bf(torch.randn(H * n, R, generator=g) / math.sqrt(R))
    q = bf(torch.randn(T, H * n, generator=g))
    got = _ops().head_project(q.to(dtype).to(DEV), w.to(dtype).to(DEV), H, n, R, True)
    want = torch.einsum("thj,hjr->thr", q.double().reshape(T, H, n), w.double().reshape(H, n, R))
    assert nerr(got, want) < 2e-6
    o = torch.randn(T, H, R, generator=g)
    got = _ops().head_project(o.to(DEV), w.to(dtype).to(DEV), H, n, R, False)
    want = torch.einsum("thr,hjr->thj", o.double(), w.double().reshape(H, n, R)).reshape(T, H * n)
    assert nerr(got, want) < tol(dtype, 2e-6, 4e-3)


def latent_attention_plain(q_lat, c, sink, scale, window, i):
    """One query at position i over the latents c[0 .. i] in float64: [H, R]."""
    lo = max(0, i - window + 1) if window > 0 else 0
    out = []
    for h in range(q_lat.shape[0]):
        s = (c[lo:i + 1] @ q_lat[h]) * scale
        if sink is None:
            p = torch.softmax(s, 0)
        else:
            p = po.windowed_sink_softmax(s, sink[h])
        out.append(p @ c[lo:i + 1])
    return torch.stack(out)


def paged_latents(g, seqs, R, bs, dtype, extra_pages=3):
    """seqs: (context, portion) per sequence -> device tensors of a mixed batch over a shuffled page pool full of garbage."""
    pages = sum(-(-(c + n) // bs) for c, n in seqs) + extra_pages
    order = torch.randperm(pages, generator=g).tolist()
    cache = bf(torch.randn(pages * bs, R, generator=g) * 50)          # what other requests left behind
    maxb = max(-(-(c + n) // bs) for c, n in seqs)
    bt = torch.zeros(len(seqs), maxb, dtype=torch.int32)
    lat, pos, tseq = [], [], []
    for b, (ctx, n) in enumerate(seqs):
        L = ctx + n
        c = bf(torch.randn(L, R, generator=g))
        for k in range(-(-L // bs)):
            bt[b, k] = order.pop()
        for j in range(L):
            cache[int(bt[b, j // bs]) * bs + j % bs] = c[j]
        lat.append(c)
        pos += list(range(ctx, L))
        tseq += [b] * n
    return (cache.to(dtype).to(DEV), bt.to(DEV), torch.tensor(pos, dtype=torch.int64, device=DEV),
            torch.tensor(tseq, dtype=torch.int32, device=DEV), lat)


def uses_tensor_cores(dtype, R, general):
    """bfloat16 caches with a latent size that is a multiple of 64 run the tensor-core kernel (queries and weights rounded to
    bfloat16 there); everything else, and everything under debug flag 2, runs the general float32 kernel."""
    return dtype == torch.bfloat16 and R % 64 == 0 and not general


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("H,R,window,sink", [(3, 16, 20, True), (1, 40, 0, True), (6, 24, 7, False), (4, 64, 33, True), (2, 8, 1, True),
                                             (5, 128, 20, True), (16, 64, 0, False), (3, 512, 50, True), (20, 192, 9, True), (40, 256, 30, True), (9, 1024, 12, True)])
def test_latent_attention_on_a_mixed_batch(dtype, general, H, R, window, sink):
    g = torch.Generator().manual_seed(7)
    seqs = [(0, 45), (37, 1), (16, 2), (90, 1), (0, 1), (15, 17)]
    cache, bt, pos, tseq, lat = paged_latents(g, seqs, R, 4, dtype)
    T = pos.numel()
    q = torch.randn(T, H, R, generator=g) * (4.0 / math.sqrt(R))
    sk = torch.randn(H, generator=g) if sink else None
    if general:
        _ops().debug_flags(2)
    got = _ops().latent_attention_paged(q.to(DEV), cache, pos, tseq, bt, sk.to(DEV) if sink else None, H, R, 4, window, 0.3,
                                        max(n for _, n in seqs))
    want = torch.stack([latent_attention_plain(q[t].double(), lat[int(tseq[t])].double(), sk.double() if sink else None, 0.3, window,
                                               int(pos[t])) for t in range(T)])
    assert nerr(got, want) < (1e-2 if uses_tensor_cores(dtype, R, general) else 3e-6)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("R", [32, 64])
@pytest.mark.parametrize("window", [0, 150, 700])
def test_latent_attention_decoding_over_long_contexts_with_split_keys(dtype, R, window):
    g = torch.Generator().manual_seed(8)
    H = 5
    seqs = [(900, 1), (3, 1), (0, 1), (257, 1)]
    cache, bt, pos, tseq, lat = paged_latents(g, seqs, R, 16, dtype)
    q = torch.randn(4, H, R, generator=g) * (4.0 / math.sqrt(R))
    sk = torch.randn(H, generator=g)
    want = torch.stack([latent_attention_plain(q[t].double(), lat[t].double(), sk.double(), 0.2, window, int(pos[t])) for t in range(4)])
    got = _ops().latent_attention_paged(q.to(DEV), cache, pos, tseq, bt, sk.to(DEV), H, R, 16, window, 0.2, 1)
    assert nerr(got, want) < (1e-2 if uses_tensor_cores(dtype, R, False) else 3e-6)
    _ops().debug_flags(2)          # the general kernel, unsplit
    one = _ops().latent_attention_paged(q.to(DEV), cache, pos, tseq, bt, sk.to(DEV), H, R, 16, window, 0.2, 1)
    assert nerr(one, want) < 3e-6


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("R", [16, 64])
@pytest.mark.parametrize("decode", [False, True])
def test_one_loud_key_is_seen_just_inside_the_window_and_not_just_outside(dtype, R, decode):
    """All latents are small but one, whose score towers over the rest when it is visible: the output then IS that latent.
    Placed at the window's first key, one before it, at page borders, hundreds of keys back, at the query, at position 0."""
    g = torch.Generator().manual_seed(9)
    H, bs, window, L = 2, 8, 96, 400
    u = torch.zeros(R)
    u[3] = 1.0
    for i, loud in [(399, 399 - 95), (399, 399 - 96), (399, 304), (399, 303), (200, 105), (200, 104), (95, 0), (96, 0), (399, 399),
                    (120, 64), (120, 63), (7, 0), (0, 0)]:
        c = bf(torch.randn(L, R, generator=g) * 0.05)
        c[loud] = 8.0 * u
        ctx = i if decode else max(0, i - 4)
        n = i + 1 - ctx
        pages = -(-(i + 1) // bs)
        order = torch.randperm(pages + 2, generator=g).tolist()
        bt = torch.tensor([order[:pages]], dtype=torch.int32)
        cache = bf(torch.randn((pages + 2) * bs, R, generator=g) * 9)
        for j in range(i + 1):
            cache[int(bt[0, j // bs]) * bs + j % bs] = c[j]
        q = torch.zeros(n, H, R)
        q[-1, :, 3] = 5.0
        pos = torch.arange(ctx, i + 1, dtype=torch.int64)
        got = _ops().latent_attention_paged(q.to(DEV), cache.to(dtype).to(DEV), pos.to(DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
                                            bt.to(DEV), torch.zeros(H, device=DEV), H, R, bs, window, 1.0, n)[-1].cpu()
        visible = 0 <= i - loud < window
        assert (abs(float(got[0, 3]) - 8.0) < 1e-3) == visible, (i, loud)
        want = latent_attention_plain(q[-1].double(), c.double(), torch.zeros(H, dtype=F64), 1.0, window, i)
        assert (got.double() - want).abs().max() < (2e-3 if uses_tensor_cores(dtype, R, False) else 1e-5), (i, loud)


@pytest.mark.parametrize("H,dim,R,window", [(3, 64, 64, 0), (2, 128, 128, 100), (5, 64, 192, 300), (1, 128, 64, 129)])
def test_long_portions_on_expanded_keys_and_values(H, dim, R, window):
    """Sequences with at least 128 tokens in the step: latents gathered from the pages, keys and values expanded, softmax with the
    window and the sink on the tensor-memory kernel; the other sequences' rows are left alone."""
    g = torch.Generator().manual_seed(12)
    seqs = [(0, 300), (37, 1), (200, 150), (16, 2), (500, 128)]
    cache, bt, pos, tseq, lat = paged_latents(g, seqs, R, 16, torch.bfloat16)
    T = pos.numel()
    wk, wv = bf(torch.randn(H * dim, R, generator=g) * 2 / math.sqrt(R)), bf(torch.randn(H * dim, R, generator=g) / math.sqrt(R))
    q = bf(torch.randn(T, H * dim, generator=g))
    sk = torch.randn(H, generator=g)
    qs = torch.tensor([0] + list(np.cumsum([n for _, n in seqs])), dtype=torch.int32)
    ctx = torch.tensor([c for c, _ in seqs], dtype=torch.int32)
    long_ = [(c, n) for c, n in seqs if n >= 128]
    max_keys = sum(n + (min(c, window - 1) if window else c) for c, n in long_)
    out = torch.full((T, H * dim), 7.0, dtype=torch.bfloat16, device=DEV)
    _ops().latent_attention_expanded(q.to(torch.bfloat16).to(DEV), cache, wk.to(torch.bfloat16).to(DEV), wv.to(torch.bfloat16).to(DEV), qs.to(DEV),
                                     ctx.to(DEV), bt, sk.to(DEV), H, dim, R, 16, window, dim ** -0.5, 128, max(n for _, n in seqs),
                                     max(c + n for c, n in seqs), max_keys, out=out)
    eye = torch.eye(H * dim, dtype=F64)
    for b, (c, n) in enumerate(seqs):
        rows = slice(int(qs[b]), int(qs[b + 1]))
        if n < 128:
            assert bool((out[rows] == 7.0).all()), b
            continue
        want = po.latent_attention_heads(q[rows].double(), lat[b].double(), eye, wk.double(), wv.double(), sk.double(), H, dim, dim,
                                         dim ** -0.5, window, first_query=c)
        assert nerr(out[rows], want) < 1.5e-2, b


def test_the_sink_takes_its_share_of_the_weights():
    """One key, score 0, sink s: the key's weight is 1 / (1 + e^s), counted once whatever the number of heads or tiles."""
    R = 8
    c = torch.ones(1, R)
    for s in (-2.0, 0.0, 3.0):
        got = _ops().latent_attention_paged(torch.zeros(1, 3, R, device=DEV), c.to(DEV), torch.zeros(1, dtype=torch.int64, device=DEV),
                                            torch.zeros(1, dtype=torch.int32, device=DEV), torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                                            torch.tensor([s, s, -30.0], device=DEV), 3, R, 1, 0, 1.0, 1).cpu()
        assert abs(float(got[0, 0, 0]) - 1 / (1 + math.exp(s))) < 1e-6 and abs(float(got[0, 2, 0]) - 1.0) < 1e-6


# ------------------------------------------------------------------------------------------------
# mixture of experts
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("E,top", [(5, 2), (12, 1), (3, 3), (40, 4)])
def test_router_scores_and_choice(dtype, E, top):
    g = torch.Generator().manual_seed(10)
    T, W = 9, 50
    h, wr, wg = bf(torch.randn(T, W, generator=g)), bf(torch.randn(E, W, generator=g) / 4), bf(torch.randn(W, generator=g) / 4)
    idx, wgt, rg = _ops().moe_route(h.to(dtype).to(DEV), wr.to(DEV), wg.to(DEV), top)
    want_idx, want_val = po.route(h.double(), wr.double(), top)
    assert torch.equal(idx.cpu().long(), want_idx)
    assert nerr(wgt, want_val) < 2e-6 and nerr(rg, po.sigma(h.double() @ wg.double())) < 2e-6
    _, wn, _ = _ops().moe_route(h.to(dtype).to(DEV), wr.to(DEV), None, top, renormalize=True)
    assert nerr(wn, want_val / want_val.sum(-1, keepdim=True)) < 2e-6


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("W", [64, 50])
def test_router_scores_do_not_depend_on_the_batch(dtype, W):
    """A token's scores are bit-identical whether it is routed in a decode-sized step or inside a prompt's portion (the two
    sizes run different tile shapes of the logits kernel)."""
    g = torch.Generator().manual_seed(13)
    h, wr, wg = bf(torch.randn(300, W, generator=g)), bf(torch.randn(9, W, generator=g) / 4), bf(torch.randn(W, generator=g) / 4)
    hd = h.to(dtype).to(DEV)
    i_all, w_all, g_all = _ops().moe_route(hd, wr.to(DEV), wg.to(DEV), 3)
    i_few, w_few, g_few = _ops().moe_route(hd[5:12].contiguous(), wr.to(DEV), wg.to(DEV), 3)
    assert torch.equal(i_all[5:12], i_few) and torch.equal(w_all[5:12], w_few) and torch.equal(g_all[5:12], g_few)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("T,E,top,W,ff,force_tmem", [(7, 5, 2, 48, 24, False), (150, 3, 1, 40, 70, False), (33, 12, 3, 50, 9, False),
                                                     (1, 4, 4, 64, 64, False), (1, 4, 4, 64, 64, True), (300, 4, 2, 128, 192, True),
                                                     (70, 6, 3, 72, 200, True), (700, 8, 2, 256, 136, False)])
def test_routed_experts_scale_their_input(dtype, T, E, top, W, ff, force_tmem):
    """bfloat16 steps of 1024 (token, expert) pairs and more run the tensor-memory products on 128-row tiles (forced for smaller
    steps by debug flag 8), smaller ones the warp-level products on 64-row tiles; float32 the plain kernel."""
    g = torch.Generator().manual_seed(11)
    h = bf(torch.randn(T, W, generator=g))
    wgu, wd = bf(torch.randn(E, 2 * ff, W, generator=g) * 2 / math.sqrt(W)), bf(torch.randn(E, W, ff, generator=g) / math.sqrt(ff))
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if T > 100:
        idx[:90] = torch.arange(1, 1 + top) % E      # crowded experts (more than one row tile) and, for E = 3, one that nobody chose
        if E == 3:
            idx[:] = 1
            idx[::7] = 2
    wgt = torch.rand(T, top, generator=g) + 0.2
    if force_tmem:
        _ops().debug_flags(8)
    got = _ops().moe_experts(h.to(dtype).to(DEV), idx.to(DEV), wgt.to(DEV), wgu.to(dtype).to(DEV), wd.to(dtype).to(DEV), 1.5, 1.702, 1.0)
    want = torch.zeros(T, W, dtype=F64)
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            x = h[t].double() * float(wgt[t, k])
            if dtype == torch.bfloat16:
                x = x.to(torch.bfloat16).double()      # the gathered row is stored in the activation format
            want[t] += po.expert(x, wgu[e, :ff].double(), wgu[e, ff:].double(), wd[e].double(), 1.5)
    assert nerr(got, want) < tol(dtype, 3e-6, 1e-2)
    # the weight on the output instead (another design's convention) is a different function
    other = _ops().moe_experts(h.to(dtype).to(DEV), idx.to(DEV), wgt.to(DEV), wgu.to(dtype).to(DEV), wd.to(dtype).to(DEV), 1.5, 1.702, 1.0,
                               scale_input=False)
    assert nerr(other, want) > 1e-2


# ------------------------------------------------------------------------------------------------
# the model through the engine
# ------------------------------------------------------------------------------------------------
def make_engine(tmp_path, cfg, weights, dtype, max_tokens=512, block_size=16, live=4, budget=2048):
    from atoma_infer_b200 import checkpoint
    from atoma_infer_b200.engine import Engine
    tmp_path.mkdir(exist_ok=True)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    checkpoint.write_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return Engine.from_model_dir(tmp_path, dtype=dtype, device=DEV, max_tokens=max_tokens, block_size=block_size,
                                 max_live_requests=live, max_num_batched_tokens=budget)


VARIANTS = {
    "base": dict(),
    "plain": dict(loop=None, side=0, softcap=0.0, groups=1, shared_ff=0, top=1, layers=2),
    "one_head_equal_dims": dict(heads=1, dim=16, vdim=16, q_rank=16, kv_rank=16, window=5, loop=(0, 2, 3), layers=2),
    "window_of_one": dict(window=1, experts=2, top=2, layers=2, loop=(0, 1, 1)),
    "window_beyond_the_prompt": dict(window=1000, layers=2, loop=(1, 2, 1), no_mlp_layers=(0,)),
    "heads_of_64": dict(width=64, groups=2, heads=2, dim=64, vdim=64, q_rank=32, kv_rank=64, window=150, layers=2, loop=(0, 1, 2), experts=4, ff=32,
                        shared_ff=32, max_positions=512),
    "odd_sizes": dict(width=50, vocab=37, heads=5, dim=6, vdim=10, q_rank=14, kv_rank=22, window=33, experts=7, top=3, ff=11,
                      shared_ff=13, groups=5, layers=4, loop=(1, 3, 2), side=3, no_mlp_layers=(2,)),
}


def build(name, seed=0):
    g = torch.Generator().manual_seed(200 + seed)
    cfg = po.random_config(**VARIANTS[name])
    return cfg, po.random_weights(cfg, g), g


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", list(VARIANTS))
def test_whole_prompt_matches_the_plain_model(tmp_path, dtype, name):
    cfg, w, g = build(name)
    toks = torch.randint(0, cfg["vocab"], (83,), generator=g).tolist()
    want, layers = po.forward(cfg, w, toks, return_layers=True)
    eng = make_engine(tmp_path, cfg, w, dtype)
    out = eng.step_forced([("a", toks, list(range(len(toks))))], want_residual_trace=True)
    assert out.residual_trace.shape[0] == len(po.run_order(cfg)) == len(layers)
    for i in range(len(layers)):
        assert model_close(out.residual_trace[i], layers[i], dtype, 5e-6), i
    assert model_close(out.logits, want, dtype)


@pytest.mark.parametrize("name", ["base", "odd_sizes", "window_of_one"])
def test_decoding_token_by_token_equals_the_whole_prompt(tmp_path, name):
    """70 single-token steps on pages of four tokens: every page border, the first tokens, and the window passing over decoded tokens."""
    cfg, w, g = build(name, 1)
    toks = torch.randint(0, cfg["vocab"], (70,), generator=g).tolist()
    want = po.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, torch.float32, max_tokens=128, block_size=4)
    got = [eng.step_forced([("a", [t], [0])]).logits.clone() for t in toks]
    assert nerr(torch.cat(got), want) < 1e-5


@pytest.mark.parametrize("dtype", BOTH)
def test_long_portions_beside_decoded_tokens(tmp_path, dtype):
    """Portions of 128 tokens and more (bfloat16: expanded keys and values on the tensor-memory kernel) in one step with short
    portions and single tokens (latent space), over a window that the long portions cross."""
    cfg, w, g = build("heads_of_64", 7)
    toks = {k: torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for k, n in (("a", 400), ("b", 40), ("c", 330))}
    want = {k: po.forward(cfg, w, t) for k, t in toks.items()}
    eng = make_engine(tmp_path, cfg, w, dtype, max_tokens=1024)
    steps = [[("a", 200), ("b", 3)], [("a", 130), ("b", 1), ("c", 129)], [("c", 200), ("a", 69), ("b", 36)], [("a", 1), ("c", 1)]]
    at, got = {k: 0 for k in toks}, {k: [] for k in toks}
    for step in steps:
        entries = []
        for k, n in step:
            entries.append((k, toks[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
        out = eng.step_forced(entries)
        r = 0
        for k, n in step:
            got[k].append(out.logits[r:r + n].clone())
            r += n
    for k in toks:
        assert at[k] == len(toks[k]) and model_close(torch.cat(got[k]), want[k], dtype), k


def test_long_decoding_far_past_the_window(tmp_path):
    cfg, w, g = build("one_head_equal_dims", 2)
    toks = torch.randint(0, cfg["vocab"], (230,), generator=g).tolist()
    want = po.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, torch.bfloat16, max_tokens=256, block_size=16)
    got = [eng.step_forced([("a", toks[:30], list(range(30)))]).logits.clone()]
    got += [eng.step_forced([("a", [t], [0])]).logits.clone() for t in toks[30:]]
    assert model_close(torch.cat(got), want, torch.bfloat16)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 2], [40, 2, 17, 1, 1, 2, 64, 5], [1, 130, 1, 1], [19, 20, 21]])
def test_portions_of_any_size_equal_the_whole_prompt(tmp_path, dtype, sizes):
    cfg, w, g = build("base", 3)
    n = sum(sizes)
    toks = torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
    want = po.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, dtype, block_size=16)
    got, at = [], 0
    for s in sizes:
        got.append(eng.step_forced([("a", toks[at:at + s], list(range(s)))]).logits.clone())
        at += s
    assert model_close(torch.cat(got), want, dtype)
    if dtype == torch.bfloat16:      # how the prompt was cut changes the result by rounding only
        whole = make_engine(tmp_path / "w", cfg, w, dtype).step_forced([("a", toks, list(range(n)))]).logits
        assert model_close(torch.cat(got), whole, dtype)


@pytest.mark.parametrize("dtype", BOTH)
def test_mixed_batches_with_reused_pages_equal_each_request_alone(tmp_path, dtype):
    """Five requests through a pool of 12 pages of 16, at most two live: later requests inherit the pages of ended ones (full of
    their latents, in every run's cache) and must not see them."""
    cfg, w, g = build("base", 4)
    lens = {"a": 70, "b": 9, "c": 55, "d": 33, "e": 60}
    toks = {k: torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for k, n in lens.items()}
    want = {k: po.forward(cfg, w, t) for k, t in toks.items()}
    eng = make_engine(tmp_path, cfg, w, dtype, max_tokens=12 * 16 - 2 * 16, block_size=16, live=2)
    assert eng.cache.blocks.capacity == 12
    steps = [[("a", 40), ("b", 3)], [("a", 2), ("b", 1)], [("b", 5), ("a", 27)], [("a", 1), ("c", 30)], [("c", 1), ("d", 2)],
             [("d", 31), ("c", 24)], [("e", 59)], [("e", 1)]]
    at, got = {k: 0 for k in lens}, {k: [] for k in lens}
    for step in steps:
        entries, end = [], []
        for k, n in step:
            entries.append((k, toks[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == lens[k]:
                end.append(k)
        out = eng.step_forced(entries, end)
        r = 0
        for k, n in step:
            got[k].append(out.logits[r:r + n].clone())
            r += n
    assert at == lens and eng.cache.live == 0
    for k in lens:
        assert model_close(torch.cat(got[k]), want[k], dtype), k


def test_a_changed_token_matters_inside_the_window_only(tmp_path):
    """One layer, window 12: the logits at position p feel the token at p - 11 and not the one at p - 12, in a prompt's portion
    and when decoded alone."""
    cfg = po.random_config(layers=1, loop=None, window=12, side=0)
    g = torch.Generator().manual_seed(77)
    w = po.random_weights(cfg, g)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=g).tolist()
    p = 39
    for decoded in (False, True):
        res = {}
        for name, j in (("same", None), ("inside", p - 11), ("outside", p - 12)):
            t = list(toks)
            if j is not None:
                t[j] = (t[j] + 1) % cfg["vocab"]
            eng = make_engine(tmp_path / f"{name}{decoded}", cfg, w, torch.float32)
            if decoded:
                eng.step_forced([("a", t[:p], [])])
                res[name] = eng.step_forced([("a", t[p:], [0])]).logits[0].clone()
            else:
                res[name] = eng.step_forced([("a", t, [p])]).logits[0].clone()
            assert nerr(res[name], po.forward(cfg, w, t)[p]) < 1e-5
        assert nerr(res["outside"], res["same"]) < 1e-6 and nerr(res["inside"], res["same"]) > 1e-3


def test_greedy_generation_through_the_scheduler(tmp_path):
    cfg, w, g = build("base", 5)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (19, 3, 41, 1)]
    eng = make_engine(tmp_path, cfg, w, torch.float32, max_tokens=256, block_size=8, live=2, budget=16)
    got = eng.generate(prompts, max_new_tokens=6)
    assert eng.cache.live == 0 and eng.cache.blocks.num_free == eng.cache.blocks.capacity
    for p, out in zip(prompts, got):
        assert len(out) == 6
        t = list(p)
        for tok in out:
            lg = po.forward(cfg, w, t)[-1]
            top = torch.topk(lg, 2).values
            if float(top[0] - top[1]) < 1e-3:
                break
            assert int(lg.argmax()) == tok
            t.append(tok)


def test_command_line_and_trace_replay(tmp_path, capsys, monkeypatch):
    import io
    from atoma_infer_b200 import checkpoint
    from atoma_infer_b200.__main__ import main
    cfg, w, g = build("plain", 6)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    checkpoint.write_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    assert main(["generate", "--model", str(tmp_path), "--prompt-ids", "3,4,5,6", "--max-new-tokens", "2", "--dtype", "float32",
                 "--max-tokens", "128", "--max-live", "2"]) == 0
    line = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines() if x.startswith("{")][0]
    lg = po.forward(cfg, w, [3, 4, 5, 6])[-1]
    if float(torch.topk(lg, 2).values[0] - torch.topk(lg, 2).values[1]) > 1e-3:
        assert line["generated"][0] == int(lg.argmax())
    toks = [5, 9, 2, 30, 11, 7]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:4], "want": [1, 3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[4:5], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[5:], "want": [0]}, {"id": "b", "tokens": toks[:2], "want": [1]}], "end": ["a", "b"]}]
    monkeypatch.setattr("sys.stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    out = tmp_path / "out"
    assert main(["trace", "--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"]) == 0
    assert [x for x in capsys.readouterr().out.split("\n") if x.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = po.forward(cfg, w, toks)
    assert not (out / "1.f32").exists()
    a = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    b = np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1)
    assert nerr(a, want[[1, 3]]) < 1e-5 and nerr(b, torch.stack([want[5], want[1]])) < 1e-5
