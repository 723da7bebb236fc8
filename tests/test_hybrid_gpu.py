"""Lilovik on the GPU against the plain implementation of tests/lilovik_oracle.py (float64): every operator
alone, then the model through the engine — whole prompts, token-by-token decoding, portions down to two
tokens, mixed batches against each request alone, reused pages and state slots, keys far away and at page
borders, long decoding, other sizes, and greedy generation through the scheduler."""
import json
import math

import numpy as np
import pytest
import torch

import lilovik_oracle as lo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from atoma_infer_b200 import hybrid_ops
    return hybrid_ops


@pytest.fixture(autouse=True)
def _reset_flags():
    yield
    if torch.cuda.is_available():
        _ops().debug_flags(0)


def nerr(got, want):
    """rms(got - want) / rms(want)"""
    got, want = torch.as_tensor(got).double().cpu(), torch.as_tensor(want).double().cpu()
    return float(((got - want) ** 2).mean().sqrt() / (want ** 2).mean().sqrt().clamp_min(1e-30))


TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


# ------------------------------------------------------------------------------------------------
# operators
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [48, 33])
def test_embedding_with_position_signal(dtype, width):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(20, width, generator=g).to(torch.bfloat16)
    toks = torch.tensor([3, 19, 0, 7, 7], dtype=torch.int32)
    pos = torch.tensor([0, 1, 517, 4095, 100000], dtype=torch.int64)
    inv = torch.tensor([10000.0 ** (-2.0 * i / width) for i in range((width + 1) // 2)], dtype=torch.float64)
    got = _ops().embed_sinusoid(toks.to(DEV), pos.to(DEV), table.to(dtype).to(DEV), inv.to(DEV))
    want = table.double()[toks.long()] + lo.sinusoid(pos.tolist(), width, torch.float64)
    assert (got.double().cpu() - want).abs().max() < 3e-7 * 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norms_and_the_fused_residual_update(dtype):
    g = torch.Generator().manual_seed(1)
    T, W, eps = 7, 50, 1e-5
    x = torch.randn(T, W, generator=g) * 3
    y = (torch.randn(T, W, generator=g) * 0.7).to(dtype)
    w1, w2 = torch.randn(W, generator=g) * 0.2, torch.randn(W, generator=g) * 0.2
    rows = torch.tensor([5, 0, 5], dtype=torch.int32)
    got = _ops().rmsnorm_rows(x.to(DEV), w1.to(DEV), 1.0, eps, dtype, rows.to(DEV))
    assert nerr(got, lo.norm_one_plus(x.double()[rows.long()], w1.double(), eps)) < TOL[dtype]
    got = _ops().rmsnorm_rows(x.to(DEV), w1.to(DEV), 0.0, eps, dtype)
    assert nerr(got, lo.rms(x.double(), eps) * w1.double()) < TOL[dtype]
    xd = x.to(DEV).clone()
    h = _ops().postnorm_add_prenorm(y.to(DEV), xd, w1.to(DEV), w2.to(DEV), eps, 1.0)
    x2 = x.double() + lo.norm_one_plus(y.double(), w1.double(), eps)
    assert nerr(xd, x2) < 2e-6                              # the residual stream is float32 in either format
    assert nerr(h, lo.norm_one_plus(x2, w2.double(), eps)) < TOL[dtype]
    xd = x.to(DEV).clone()
    assert _ops().postnorm_add_prenorm(y.to(DEV), xd, w1.to(DEV), None, eps, 1.0) is None
    assert nerr(xd, x2) < 2e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qk_norm_temperature_and_cache_write(dtype):
    g = torch.Generator().manual_seed(2)
    H, G, D, Dv, every, coef, eps = 4, 2, 8, 12, 8, 0.3, 1e-5
    pos = torch.tensor([0, 6, 7, 8, 14, 15, 16, 63, 64], dtype=torch.int64)     # (p + 1) / every crosses 1, 2 and 8
    T, n = pos.numel(), H * D + G * D + G * Dv
    qkv = torch.randn(T, n, generator=g).to(dtype)
    bias = torch.randn(n, generator=g) * 0.3
    qw, kw = 1 + 0.1 * torch.randn(H * D, generator=g), 1 + 0.1 * torch.randn(G * D, generator=g)
    slots = torch.tensor([5, 17, -1, 0, 30, 31, 2, 9, 11], dtype=torch.int64)
    kc = torch.full((32, G, D), 7.0, dtype=dtype, device=DEV)
    vc = torch.full((32, G, Dv), 7.0, dtype=dtype, device=DEV)
    q = _ops().qk_norm_cache(qkv.to(DEV), bias.to(DEV), qw.to(DEV), kw.to(DEV), pos.to(DEV), slots.to(DEV), kc, vc, H, G, D, Dv,
                             eps, coef, every)
    full = qkv.double() + bias.double()
    temp = torch.tensor([lo.query_temperature(int(p), coef, every) for p in pos], dtype=torch.float64)
    assert temp[1] == 1.0 and temp[2] > 1.0 and temp[7] > temp[5]
    assert nerr(q, lo.rms(full[:, :H * D], eps) * qw.double() * temp[:, None]) < TOL[dtype]
    wk = lo.rms(full[:, H * D:H * D + G * D], eps) * kw.double()
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            assert nerr(kc[s].reshape(-1), wk[t]) < TOL[dtype] and nerr(vc[s].reshape(-1), full[t, H * D + G * D:]) < TOL[dtype]
    untouched = [s for s in range(32) if s not in slots.tolist()]
    assert (kc[untouched] == 7).all() and (vc[untouched] == 7).all()


def _paged_batch(g, seqs, H, G, D, Dv, bs, dtype, scale_q=1.0, k_zero_dim=None):
    """seqs: list of (context, new tokens).  Returns device inputs of the attention operator and, per sequence, the
    float64 q / k / v the oracle reads.  Pages are handed out in a scrambled order and stale pages hold large values."""
    total = sum(c + n for c, n in seqs)
    nb = sum(-(-(c + n) // bs) for c, n in seqs) + 3
    perm = torch.randperm(nb, generator=g).tolist()
    kc = torch.full((nb * bs, G, D), 50.0, dtype=dtype)
    vc = torch.full((nb * bs, G, Dv), 50.0, dtype=dtype)
    mb = max(-(-(c + n) // bs) for c, n in seqs)
    bt = torch.zeros((len(seqs), mb), dtype=torch.int32)
    qs, pos, tseq, ref = [], [], [], []
    for b, (c, n) in enumerate(seqs):
        t = c + n
        k = torch.randn(t, G, D, generator=g).to(dtype)
        if k_zero_dim is not None:
            k[:, :, k_zero_dim] = 0
        v = torch.randn(t, G, Dv, generator=g).to(dtype)
        q = (torch.randn(n, H, D, generator=g) * scale_q).to(dtype)
        pages = [perm.pop() for _ in range(-(-t // bs))]
        bt[b, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        for j in range(t):
            kc[pages[j // bs] * bs + j % bs] = k[j]
            vc[pages[j // bs] * bs + j % bs] = v[j]
        qs.append(q.reshape(n, H * D))
        pos += list(range(c, t))
        tseq += [b] * n
        ref.append((q.double(), k.double(), v.double(), c))
    dev = lambda x: x.to(DEV)
    return (dev(torch.cat(qs)), dev(kc), dev(vc), dev(torch.tensor(pos, dtype=torch.int64)),
            dev(torch.tensor(tseq, dtype=torch.int32)), dev(bt), ref)


ATTN_SHAPES = [(4, 2, 16, 24), (4, 4, 32, 32), (6, 1, 8, 16), (2, 2, 64, 64), (8, 4, 80, 80), (3, 3, 20, 12),
               (32, 8, 64, 64), (16, 2, 128, 128), (12, 4, 32, 48), (32, 32, 128, 96), (36, 4, 16, 136)]   # the last rows spread heads over a cluster


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("H,G,D,Dv", ATTN_SHAPES)
def test_sigmoid_attention_on_a_mixed_batch(dtype, general, H, G, D, Dv):
    g = torch.Generator().manual_seed(3)
    bs, cap = 16, 5.0
    seqs = [(37, 90), (130, 1), (0, 70), (0, 1), (15, 2), (64, 1)]      # portions with and without context, decodes, first token
    q, kc, vc, pos, tseq, bt, ref = _paged_batch(g, seqs, H, G, D, Dv, bs, dtype)
    slopes = torch.tensor(lo.distance_slopes(H))
    pb = torch.randn(H, generator=g) - 2.0
    talk = torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)
    m = {"heads": H, "kv_heads": G, "scale": 0.3, "softcap": cap}
    _ops().debug_flags(2 if general else 0)
    out = _ops().sigmoid_attention_paged(q, kc, vc, pos, tseq, bt, slopes.to(DEV), pb.to(DEV), talk.to(DEV), H, G, D, Dv, bs,
                                         0.3, cap, max(n for _, n in seqs))
    t0 = 0
    for (qq, kk, vv, c), (_, n) in zip(ref, seqs):
        want = lo.attention_core(qq, kk, vv, m, pb.double(), talk.double(), first_position=c).reshape(n, H * Dv)
        assert nerr(out[t0:t0 + n], want) < (1e-5 if dtype == torch.float32 else 1e-2), (c, n)
        t0 += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("H,G,D,Dv", [(4, 2, 16, 24), (8, 4, 80, 80), (32, 8, 64, 64), (16, 2, 128, 128), (3, 3, 20, 12)])
def test_sigmoid_attention_on_a_decode_only_batch(dtype, general, H, G, D, Dv):
    """One query token per sequence, contexts from nothing to a thousand keys: the keys are split over CTAs and the splits'
    sums added."""
    g = torch.Generator().manual_seed(8)
    bs = 16
    seqs = [(300, 1), (0, 1), (65, 1), (1000, 1), (31, 1), (32, 1)]
    q, kc, vc, pos, tseq, bt, ref = _paged_batch(g, seqs, H, G, D, Dv, bs, dtype)
    slopes = torch.tensor(lo.distance_slopes(H))
    pb = torch.randn(H, generator=g) - 2.0
    talk = torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)
    m = {"heads": H, "kv_heads": G, "scale": 0.2, "softcap": 8.0}
    _ops().debug_flags(2 if general else 0)
    out = _ops().sigmoid_attention_paged(q, kc, vc, pos, tseq, bt, slopes.to(DEV), pb.to(DEV), talk.to(DEV), H, G, D, Dv, bs,
                                         0.2, 8.0, 1)
    for b, (qq, kk, vv, c) in enumerate(ref):
        want = lo.attention_core(qq, kk, vv, m, pb.double(), talk.double(), first_position=c).reshape(1, H * Dv)
        assert nerr(out[b:b + 1], want) < (1e-5 if dtype == torch.float32 else 1e-2), (b, c)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("general", [False, True])
def test_a_single_far_key_is_found_wherever_it_lies(dtype, general):
    """Head biases push every ordinary weight to ~0; one key is made to stand out by a q . k large enough to beat the distance
    bias from hundreds of positions away (the query looks along one dimension that every other key has at zero).  Its value
    must come through for keys at position 0, around page borders, far back, at the query itself — and must NOT when the key
    lies one position after the query (inside the same portion, already written to the cache)."""
    g = torch.Generator().manual_seed(4)
    H, G, D, Dv, bs = 4, 2, 16, 24, 16
    slopes = torch.tensor(lo.distance_slopes(H))
    pb = torch.full((H,), -14.0)
    talk = torch.eye(H) + 0.2 * torch.randn(H, H, generator=g)
    m = {"heads": H, "kv_heads": G, "scale": 1.0, "softcap": 0.0}
    _ops().debug_flags(2 if general else 0)
    for ctx, n, qrow in [(300, 1, 0), (250, 40, 17), (0, 200, 150)]:
        p = ctx + qrow
        for j in sorted({0, 1, bs - 1, bs, bs + 1, 127, 128, 129, p - bs, p - 1, p, p + 1}):
            if j < 0 or j >= ctx + n:
                continue
            q, kc, vc, pos, tseq, bt, ref = _paged_batch(g, [(ctx, n)], H, G, D, Dv, bs, dtype, scale_q=0.05, k_zero_dim=3)
            qq, kk, vv, _ = ref[0]
            big = torch.zeros(D)
            big[3] = 10.5
            qq[qrow] = big.repeat(H, 1)
            kk[j] = big.repeat(G, 1)
            q[qrow] = qq[qrow].reshape(-1).to(dtype)
            page = int(bt[0, j // bs])
            kc[page * bs + j % bs] = kk[j].to(dtype)
            out = _ops().sigmoid_attention_paged(q, kc, vc, pos, tseq, bt, slopes.to(DEV), pb.to(DEV), talk.to(DEV), H, G, D, Dv,
                                                 bs, 1.0, 0.0, n)
            want = lo.attention_core(qq, kk, vv, m, pb.double(), talk.double(), first_position=ctx).reshape(n, H * Dv)
            row = out[qrow].double().cpu()
            if j <= p:
                assert want[qrow].abs().max() > 0.3                       # the key is really seen by the oracle
                assert nerr(row, want[qrow]) < (1e-4 if dtype == torch.float32 else 2e-2), (ctx, n, j)
            else:
                assert want[qrow].abs().max() < 1e-2 and row.abs().max() < 1e-2, (ctx, n, j)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sequential", [False, True])
@pytest.mark.parametrize("S", [40, 33, 128])
def test_mingru_scan_carries_state_per_sequence(dtype, sequential, S):
    g = torch.Generator().manual_seed(5)
    lens = [(0, 300), (12, 1), (0, 1), (5, 131), (9, 2)]
    slots = torch.tensor([3, 0, 4, 1, 2], dtype=torch.int32)
    T = sum(n for _, n in lens)
    zxg = (torch.randn(T, 3 * S, generator=g) * 1.5).to(dtype)
    zxg[:, S:S + 4] = 0.0                                               # candidates exactly at the branch point
    bias = torch.cat([torch.randn(2 * S, generator=g) * 0.3, torch.zeros(S)])
    bias[S:S + 4] = 0.0
    state0 = torch.randn(5, S, generator=g)
    state = state0.clone().to(DEV)
    qs = torch.tensor([0] + list(np.cumsum([n for _, n in lens])), dtype=torch.int32)
    ctx = torch.tensor([c for c, _ in lens], dtype=torch.int32)
    _ops().debug_flags(4 if sequential else 0)
    out = _ops().mingru_scan(zxg.to(DEV), bias.to(DEV), state, slots.to(DEV), qs.to(DEV), ctx.to(DEV), max(n for _, n in lens))
    w = {"z": torch.eye(S, dtype=torch.float64), "x": torch.eye(S, dtype=torch.float64), "g": torch.eye(S, dtype=torch.float64),
         "o": torch.eye(S, dtype=torch.float64), "z.b": bias[:S].double(), "x.b": bias[S:2 * S].double()}
    for b, (c, n) in enumerate(lens):
        rows = slice(int(qs[b]), int(qs[b + 1]))
        z, u, gate = zxg[rows, :S].double(), zxg[rows, S:2 * S].double(), zxg[rows, 2 * S:].double()
        s = state0[slots[b]].double() if c > 0 else torch.zeros(S, dtype=torch.float64)
        want = []
        for t in range(n):
            zz = torch.sigmoid(z[t] + w["z.b"])
            uu = u[t] + w["x.b"]
            s = (1 - zz) * s + zz * torch.where(uu >= 0, uu + 0.5, torch.sigmoid(uu))
            want.append(s * gate[t] * torch.sigmoid(gate[t]))
        assert nerr(out[rows], torch.stack(want)) < (1e-5 if dtype == torch.float32 else 1e-2)
        assert nerr(state[slots[b]], s) < 1e-5                          # the state itself is float32 in either format


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_activations_projection_and_greedy_choice(dtype):
    g = torch.Generator().manual_seed(6)
    gu = (torch.randn(9, 2 * 24, generator=g) * 2).to(dtype)
    a, b = gu[:, :24].double(), gu[:, 24:].double()
    gelu = 0.5 * a * (1 + torch.tanh(math.sqrt(2 / math.pi) * (a + 0.044715 * a ** 3)))
    for act, want in ((0, a * torch.sigmoid(a) * b), (1, torch.relu(a) * b), (2, gelu * b)):
        assert nerr(_ops().glu(gu.to(DEV), act), want) < TOL[dtype]
    for T, N, K in [(5, 24, 40), (130, 72, 64), (3, 61, 50), (200, 8, 192), (1000, 1160, 328), (1, 50000, 72), (257, 96, 136),
                    (64, 24, 1032), (129, 8, 8), (2, 16, 4096)]:
        x, w = torch.randn(T, K, generator=g).to(dtype), (torch.randn(N, K, generator=g) * K ** -0.5).to(dtype)
        assert nerr(_ops().linear(x.to(DEV), w.to(DEV)), x.double() @ w.double().T) < (max(1e-6, 2e-7 * K ** 0.5) if dtype == torch.float32 else 6e-3), (T, N, K)
    lg = torch.randn(4, 37, generator=g).to(dtype)
    lg[1, 5] = lg[1, 30] = 9.0                                          # a tie: the last index wins
    out, tok = _ops().scale_logits_greedy(lg.to(DEV), 0.5)
    assert torch.equal(out.cpu(), lg.float() * 0.5)
    assert tok.cpu().tolist() == [int(lg[0].float().argmax()), 30, int(lg[2].float().argmax()), int(lg[3].float().argmax())]


@pytest.mark.parametrize("act", [0, 1, 2])
@pytest.mark.parametrize("T,ff,K", [(1, 264, 384), (37, 40, 64), (128, 1024, 512)])
def test_gate_up_projection_with_the_activation_in_its_epilogue(act, T, ff, K):
    g = torch.Generator().manual_seed(7)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * ff, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    got = _ops().gate_up_act(x.to(DEV), w.to(DEV), act)
    gate = (x.double() @ w[:ff].double().T).to(torch.bfloat16).double()      # the projections are rounded before the activation
    up = (x.double() @ w[ff:].double().T).to(torch.bfloat16).double()
    f = {0: gate * torch.sigmoid(gate), 1: torch.relu(gate),
         2: 0.5 * gate * (1 + torch.tanh(math.sqrt(2 / math.pi) * (gate + 0.044715 * gate ** 3)))}[act]
    assert nerr(got, f * up) < 1e-2


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
    "mixed": dict(),
    "mha_equal_dims": dict(heads=4, kv_heads=4, dim=16, vdim=16, state=48),
    "one_kv_head": dict(heads=6, kv_heads=1, dim=8, vdim=40, layers=("attention", "attention", "mingru")),
    "recurrent_only": dict(layers=("mingru", "mingru"), mlp_on_mingru=True, state=24),
    "attention_only": dict(layers=("attention",), heads=1, kv_heads=1, every=1, softcap=0.0),
    "odd_sizes": dict(width=50, vocab=37, heads=3, kv_heads=3, dim=20, vdim=12, ff=30, state=33, every=5, coef=1.0,
                      layers=("mingru", "attention", "mingru", "attention"), mlp_on_mingru=True),
}


def build(name, seed=0):
    g = torch.Generator().manual_seed(100 + seed)
    cfg = lo.random_config(g, **VARIANTS[name])
    return cfg, lo.random_weights(cfg, g), g


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(VARIANTS))
def test_whole_prompt_matches_the_plain_model(tmp_path, dtype, name):
    cfg, w, g = build(name)
    toks = torch.randint(0, cfg["vocab"], (83,), generator=g).tolist()
    want, layers = lo.forward(cfg, w, toks, return_layers=True)
    eng = make_engine(tmp_path, cfg, w, dtype)
    out = eng.step_forced([("a", toks, list(range(len(toks))))], want_residual_trace=True)
    for i in range(len(cfg["layers"])):
        assert nerr(out.residual_trace[i], layers[i]) < (5e-6 if dtype == torch.float32 else 2e-2), i
    assert nerr(out.logits, want) < (1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("name", ["mixed", "odd_sizes"])
def test_decoding_token_by_token_equals_the_whole_prompt(tmp_path, name):
    """70 single-token steps on pages of four tokens: every page border, every multiple of the temperature period."""
    cfg, w, g = build(name, 1)
    toks = torch.randint(0, cfg["vocab"], (70,), generator=g).tolist()
    want = lo.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, torch.float32, max_tokens=128, block_size=4)
    got = [eng.step_forced([("a", [t], [0])]).logits.clone() for t in toks]
    assert nerr(torch.cat(got), want) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 2], [40, 2, 17, 1, 1, 2, 64, 5], [1, 130, 1, 1]])
def test_portions_of_any_size_equal_the_whole_prompt(tmp_path, dtype, sizes):
    cfg, w, g = build("mixed", 2)
    n = sum(sizes)
    toks = torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
    want = lo.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, dtype, block_size=16)
    got, at = [], 0
    for s in sizes:
        got.append(eng.step_forced([("a", toks[at:at + s], list(range(s)))]).logits.clone())
        at += s
    assert nerr(torch.cat(got), want) < (1e-5 if dtype == torch.float32 else 3e-2)
    if dtype == torch.bfloat16:      # and how the prompt was cut changes the result by rounding only
        whole = make_engine(tmp_path / "w", cfg, w, dtype).step_forced([("a", toks, list(range(n)))]).logits
        assert nerr(torch.cat(got), whole) < 1.5e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixed_batches_with_reused_pages_and_slots_equal_each_request_alone(tmp_path, dtype):
    """Five requests through two state slots and a pool of 12 pages of 16: requests end, later ones inherit their pages
    and slots (full of the earlier requests' keys and state) and must not see them."""
    cfg, w, g = build("mixed", 3)
    lens = {"a": 70, "b": 9, "c": 55, "d": 33, "e": 60}
    toks = {k: torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for k, n in lens.items()}
    want = {k: lo.forward(cfg, w, t) for k, t in toks.items()}
    eng = make_engine(tmp_path, cfg, w, dtype, max_tokens=12 * 16 - 2 * 16, block_size=16, live=2)
    assert eng.cache.blocks.capacity == 12 and eng.cache.state_slots.capacity == 2
    steps = [
        [("a", 40), ("b", 3)],
        [("a", 2), ("b", 1)],
        [("b", 5), ("a", 27)],           # b ends
        [("a", 1), ("c", 30)],           # a ends; c takes b's slot and pages
        [("c", 1), ("d", 2)],            # d takes a's
        [("d", 31), ("c", 24)],          # both end
        [("e", 59)],
        [("e", 1)],
    ]
    at = {k: 0 for k in lens}
    got = {k: [] for k in lens}
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
        assert nerr(torch.cat(got[k]), want[k]) < (1e-5 if dtype == torch.float32 else 3e-2), k


def test_greedy_generation_through_the_scheduler(tmp_path):
    """Engine.generate (scheduler, chunked prefill with a small token budget, two live requests for four prompts) against a
    greedy loop over the plain model; tokens are compared while the plain model's choice is clear-cut."""
    cfg, w, g = build("mixed", 4)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (19, 3, 41, 1)]
    eng = make_engine(tmp_path, cfg, w, torch.float32, max_tokens=256, block_size=8, live=2, budget=16)
    got = eng.generate(prompts, max_new_tokens=6)
    assert eng.cache.live == 0 and eng.cache.blocks.num_free == eng.cache.blocks.capacity
    for p, out in zip(prompts, got):
        assert len(out) == 6
        t = list(p)
        for tok in out:
            lg = lo.forward(cfg, w, t)[-1]
            top = torch.topk(lg, 2).values
            if float(top[0] - top[1]) < 1e-3:
                break
            assert int(lg.argmax()) == tok
            t.append(tok)


def test_command_line_generates_through_the_registry(tmp_path, capsys):
    from atoma_infer_b200 import checkpoint
    from atoma_infer_b200.__main__ import main
    cfg, w, g = build("mixed", 5)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    checkpoint.write_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    assert main(["generate", "--model", str(tmp_path), "--prompt-ids", "3,4,5,6", "--prompt-ids", "9", "--max-new-tokens", "3",
                 "--dtype", "float32", "--max-tokens", "128", "--max-live", "2"]) == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines() if x.startswith("{")]
    assert [x["prompt"] for x in lines] == [[3, 4, 5, 6], [9]] and all(len(x["generated"]) == 3 for x in lines)
    t = [3, 4, 5, 6]
    lg = lo.forward(cfg, w, t)[-1]
    if float(torch.topk(lg, 2).values[0] - torch.topk(lg, 2).values[1]) > 1e-3:
        assert lines[0]["generated"][0] == int(lg.argmax())
