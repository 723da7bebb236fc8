"""bench.py --design patadra: prefill and decode throughput of the Patadra design (random weights) at sizes that
resemble real models' layers, beside the framework's closest existing model — Llama — at equal width, head count,
layer count and ACTIVATED feed-forward size, and the design's hot kernels against the measured peaks beside
their Llama counterparts.  Not the headline (config 2 is); ONE JSON line in the same format.

Per size: a model of a few layer runs (one layer looped twice) is served through the engine's executor: `prefill` =
one 4096-token prompt in one step; `decode` = one step of 32 sequences at context 4096 (built by prefilling them),
timed with CUDA events around K executor steps after W warm-up steps, inputs shipped from pinned memory every step,
sampled tokens read back; the same step replayed from a CUDA graph is the device-only figure.
Kernel rows: achieved FLOP/s or bytes/s over the measured peaks of MEASURED_PEAKS.json (fallback figures when absent);
L2 is flushed between their iterations."""
from __future__ import annotations

import json
import math
import os

from bench_hybrid import BATCH, CTX, PROMPT, _llama_decode, _peaks, _time

SIZES = {
    # window 1024 at the small size, the whole context at the large one
    "2k-wide": dict(width=2048, heads=16, dim=128, vdim=128, q_rank=768, kv_rank=512, window=1024, experts=32, top=4, ff=1024,
                    shared_ff=2048, groups=2, side=256, vocab=32000, layers=3, loop=(1, 2, 2)),
    "4k-wide": dict(width=4096, heads=32, dim=128, vdim=128, q_rank=1536, kv_rank=512, window=4096, experts=64, top=6, ff=1408,
                    shared_ff=2816, groups=4, side=256, vocab=32000, layers=2, loop=(0, 1, 2)),
}


def _spec(s):
    from atoma_infer_b200.hybrid import HybridSpec, LatentAttentionSpec, LayerSpec, MoeSpec
    att = LatentAttentionSpec(s["heads"], s["dim"], s["vdim"], s["q_rank"], s["kv_rank"], 1.0 / math.sqrt(s["dim"]), s["window"], True)
    moe = MoeSpec(s["experts"], s["top"], s["ff"], 7.0, s["shared_ff"], 7.0, True)
    per_layer = [LayerSpec("latent_attention", latent=att, moe=moe, gated_residual=True, side_part=i, source=i) for i in range(s["layers"])]
    a, b, times = s["loop"]
    order = list(range(a)) + list(range(a, b)) * times + list(range(b, s["layers"]))
    return HybridSpec(s["width"], s["vocab"], 1e-6, 1.0, tuple(per_layer[i] for i in order), norm_offset=0.0, block_style="prenorm",
                      norm_groups=s["groups"], position="learned", max_positions=CTX + 64, logit_softcap=30.0, side_dim=s["side"])


def _weights(torch, spec, s, dev):
    g = torch.Generator(device=dev).manual_seed(13)

    def r(*shape, scale=1.0, mean=0.0):
        return (mean + torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * scale).to(torch.bfloat16)

    W = spec.width
    out = {"embed": r(spec.vocab, W), "pos": r(spec.max_positions, W, scale=0.3), "head": r(spec.vocab, W, scale=W ** -0.5),
           "final_norm": r(W, scale=0.1, mean=1.0), "side_table": r(spec.vocab, s["layers"] * s["side"]), "layers": []}
    a, e = spec.layers[0].latent, spec.layers[0].moe
    for _ in range(s["layers"]):
        out["layers"].append({
            "norm1": r(W, scale=0.1, mean=1.0), "norm2": r(W, scale=0.1, mean=1.0),
            "w_down_in": r(a.q_rank + a.kv_rank + W, W, scale=W ** -0.5), "gate1_bias": r(W, scale=0.3), "gate2_bias": r(W, scale=0.3),
            "dq_norm": r(a.q_rank, scale=0.1, mean=1.0), "dkv_norm": r(a.kv_rank, scale=0.1, mean=1.0),
            "w_uq": r(a.heads * a.dim, a.q_rank, scale=a.q_rank ** -0.5), "w_uk": r(a.heads * a.dim, a.kv_rank, scale=a.kv_rank ** -0.5),
            "w_uv": r(a.heads * a.vdim, a.kv_rank, scale=a.kv_rank ** -0.5), "sink": r(a.heads), "w_o": r(W, a.heads * a.vdim, scale=(a.heads * a.vdim) ** -0.5),
            "w_router": r(e.experts, W, scale=W ** -0.5), "w_shared_gate": r(W, scale=W ** -0.5),
            "w_expert_gate_up": r(e.experts, 2 * e.ff, W, scale=W ** -0.5), "w_expert_down": r(e.experts, W, e.ff, scale=e.ff ** -0.5),
            "w_ff_in": r(2 * e.shared_ff + W, W, scale=W ** -0.5), "w_down": r(W, e.shared_ff, scale=e.shared_ff ** -0.5),
            "side_gate": r(s["side"], W, scale=W ** -0.5), "side_proj": r(W, s["side"], scale=s["side"] ** -0.5), "side_norm": r(W, scale=0.1, mean=0.5)})
    return out


def _row(ms, flops=None, nbytes=None, hbm=None, tf=None):
    d = {"ms": round(ms, 4)}
    if flops is not None:
        d.update(tflops=round(flops / ms / 1e9, 1), frac_of_bf16_peak=round(flops / ms / 1e9 / tf, 3))
    if nbytes is not None:
        d.update(gbs=round(nbytes / ms / 1e6, 1), frac_of_hbm_peak=round(nbytes / ms / 1e6 / hbm, 3))
    return d


def _kernel_rows(torch, s, dev, steps, warmup, hbm, tf):
    """The design's kernels beside Llama's like kernels at the same shapes."""
    from atoma_infer_b200 import hybrid_ops as ho, ops
    H, R, D, W = s["heads"], s["kv_rank"], s["dim"], s["width"]
    bf, page, S = torch.bfloat16, 16, PROMPT
    rows = {}
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    win = s["window"]
    # ---- prompt attention: one prompt of S tokens under the window ----
    nb = S // page
    cache = torch.randn((nb * page, R), device=dev, dtype=bf)
    q = torch.randn((S, H, R), device=dev) * (R ** -0.5)
    pos = torch.arange(S, device=dev, dtype=torch.int64)
    tseq = torch.zeros(S, device=dev, dtype=torch.int32)
    bt = torch.arange(nb, device=dev, dtype=torch.int32).reshape(1, nb)
    qs = torch.tensor([0, S], device=dev, dtype=torch.int32)
    sink = torch.zeros(H, device=dev)
    f = lambda: ho.latent_attention_paged(q, cache, pos, tseq, bt, sink, H, R, page, win, 0.1, S, query_start=qs, max_seq_len=S)
    pairs = sum(min(i + 1, win) for i in range(S))
    rows["latent_attention_prefill"] = _row(_time(torch, f, steps, warmup, flush), flops=4.0 * H * R * pairs, tf=tf)
    # the same prompt on expanded keys and values (what portions of 128 tokens and more run): gather + two projections + attention
    wk, wv = torch.randn((H * D, R), device=dev, dtype=bf) * R ** -0.5, torch.randn((H * D, R), device=dev, dtype=bf) * R ** -0.5
    qe = torch.randn((S, H * D), device=dev, dtype=bf)
    ctx0 = torch.zeros(1, device=dev, dtype=torch.int32)
    oe = torch.empty((S, H * D), device=dev, dtype=bf)
    f = lambda: ho.latent_attention_expanded(qe, cache, wk, wv, qs, ctx0, bt, sink, H, D, R, page, win, 1 / math.sqrt(D), 128, S, S, S, out=oe)
    rows["latent_attention_expanded_prefill"] = _row(_time(torch, f, steps, warmup, flush), flops=4.0 * H * D * pairs + 4.0 * S * H * D * R, tf=tf)
    G = 8
    q3 = torch.randn((S, H, D), device=dev, dtype=bf)
    k3, v3 = torch.randn((S, G, D), device=dev, dtype=bf), torch.randn((S, G, D), device=dev, dtype=bf)
    cu = torch.tensor([0, S], device=dev, dtype=torch.int32)
    f = lambda: ops.flash_attn_varlen(q3, k3, v3, cu, cu, S, S, 1 / math.sqrt(D), True)
    rows["llama_attention_prefill"] = _row(_time(torch, f, steps, warmup, flush), flops=4.0 * H * D * S * (S + 1) / 2, tf=tf)
    # ---- decode attention: BATCH sequences at context CTX ----
    mb = (CTX + page) // page
    nb = BATCH * mb
    cache = torch.randn((nb * page, R), device=dev, dtype=bf)
    q = torch.randn((BATCH, H, R), device=dev) * (R ** -0.5)
    pos = torch.full((BATCH,), CTX, device=dev, dtype=torch.int64)
    tseq = torch.arange(BATCH, device=dev, dtype=torch.int32)
    bt = torch.randperm(nb, device=dev).to(torch.int32).reshape(BATCH, mb)
    qs = torch.arange(BATCH + 1, device=dev, dtype=torch.int32)
    f = lambda: ho.latent_attention_paged(q, cache, pos, tseq, bt, sink, H, R, page, win, 0.1, 1, query_start=qs, max_seq_len=CTX + 1)
    rows["latent_attention_decode"] = _row(_time(torch, f, steps, warmup, flush), nbytes=BATCH * min(CTX + 1, win) * R * 2, hbm=hbm)
    kc, vc = torch.randn((nb, page, G, D), device=dev, dtype=bf), torch.randn((nb, page, G, D), device=dev, dtype=bf)
    q4 = torch.randn((BATCH, 1, H, D), device=dev, dtype=bf)
    sl = torch.full((BATCH,), CTX + 1, device=dev, dtype=torch.int32)
    f = lambda: ops.flash_attn_kv_cache_full(q4, kc, vc, None, 1 / math.sqrt(D), bt, sl, True)
    rows["llama_attention_decode"] = _row(_time(torch, f, steps, warmup, flush), nbytes=BATCH * (CTX + 1) * G * 2 * D * 2, hbm=hbm)
    del kc, vc, cache
    # ---- per-head projections into and out of the latent space (prompt) ----
    wk = torch.randn((H * D, R), device=dev, dtype=bf)
    qh = torch.randn((S, H * D), device=dev, dtype=bf)
    ol = torch.randn((S, H, R), device=dev)
    f = lambda: ho.head_project(qh, wk, H, D, R, True)
    rows["head_project_absorb_prefill"] = _row(_time(torch, f, steps, warmup, flush), flops=2.0 * S * H * D * R, tf=tf)
    f = lambda: ho.head_project(ol, wk, H, D, R, False)
    rows["head_project_expand_prefill"] = _row(_time(torch, f, steps, warmup, flush), flops=2.0 * S * H * D * R, tf=tf)
    # ---- routed experts: prompt (compute bound) and decode step (weight stream) beside a dense feed-forward of the activated size ----
    E, top, ff = s["experts"], s["top"], s["ff"]
    wgu = torch.randn((E, 2 * ff, W), device=dev, dtype=bf) * W ** -0.5
    wd = torch.randn((E, W, ff), device=dev, dtype=bf) * ff ** -0.5
    wr = torch.randn((E, W), device=dev) * W ** -0.5
    for name, T in (("prefill", S), ("decode", BATCH)):
        h = torch.randn((T, W), device=dev, dtype=bf)
        idx, wgt, _ = ho.moe_route(h, wr, None, top)
        used = int(torch.unique(idx).numel())
        f = lambda: ho.moe_experts(h, idx, wgt, wgu, wd, 7.0, 1.702, 1.0)
        ms = _time(torch, f, steps, warmup, flush)
        rows[f"experts_{name}"] = _row(ms, flops=6.0 * T * top * ff * W, nbytes=used * 3 * ff * W * 2, hbm=hbm, tf=tf)
        rows[f"experts_{name}"]["experts_used"] = used
        f = lambda: ho.moe_route(h, wr, None, top)
        rows[f"router_{name}"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * W * 2 + E * W * 4, hbm=hbm)
        F = top * ff
        wgu_d, wd_d = torch.randn((2 * F, W), device=dev, dtype=bf), torch.randn((W, F), device=dev, dtype=bf)
        f = lambda: ho.linear(ho.glu(ho.linear(h, wgu_d), 0), wd_d)
        rows[f"llama_mlp_{name}"] = _row(_time(torch, f, steps, warmup, flush), flops=6.0 * T * F * W, nbytes=3 * F * W * 2, hbm=hbm, tf=tf)
        del wgu_d, wd_d
    del wgu, wd
    # ---- residual update with gate + next norm, beside Llama's add + RMS norm ----
    T = 8192
    y = torch.randn((T, W), device=dev, dtype=bf)
    gate = torch.randn((T, W), device=dev, dtype=bf)
    x = torch.randn((T, W), device=dev)
    b1 = torch.zeros(W, device=dev)
    w1 = torch.ones(W, device=dev)
    f = lambda: ho.gated_residual_norm(x, y=y, gate=gate, gate_bias=b1, w_next=w1, groups=s["groups"], eps=1e-6)
    rows["gated_residual_norm"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * W * (2 + 2 + 4 + 4 + 2), hbm=hbm)
    if hasattr(ops, "add_rmsnorm"):
        res, wbf = torch.randn((T, W), device=dev, dtype=bf), torch.ones(W, device=dev, dtype=bf)
        f = lambda: ops.add_rmsnorm(y, res, wbf, 1e-5)
        rows["llama_add_rmsnorm"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * W * 2 * 4, hbm=hbm)
    return rows


def run(args, torch, dev, json_fd):
    import numpy as np
    from atoma_infer_b200 import _lib
    from atoma_infer_b200.cache import CacheManager
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.hybrid import HybridExecutor, relaunch_last_step
    if args.impl != "ours":
        os.write(json_fd, (json.dumps({"impl": "reference", "unavailable": "the reference has no model of this design"}) + "\n").encode())
        return
    _lib.lib()
    hbm, tf, src = _peaks()
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    page = 16
    out_sizes, headline = {}, None
    for name, s in SIZES.items():
        spec = _spec(s)
        weights = _weights(torch, spec, s, dev)
        nblocks = BATCH * ((CTX + 64) // page + 1) + PROMPT // page + 8
        ex = HybridExecutor(spec, weights, torch.bfloat16, dev, nblocks, page, 0)
        del weights
        eng = Engine(ex, CacheManager(nblocks, page, 0), max_num_batched_tokens=PROMPT, max_num_seqs=BATCH + 1)
        rng = np.random.default_rng(0)
        prompt = rng.integers(0, s["vocab"], size=PROMPT).tolist()

        def prefill():
            eng.step_forced([("p", prompt, [PROMPT - 1])], end=["p"]).next_tokens.cpu()
        ms_prefill = _time(torch, prefill, min(steps, 10), warmup)
        prefill_launches = ex.launches_last_step
        for b in range(BATCH):
            eng.step_forced([(f"d{b}", rng.integers(0, s["vocab"], size=CTX).tolist(), [])])
        tok = [int(t) for t in rng.integers(0, s["vocab"], size=BATCH)]

        def decode():
            eng.step_forced([(f"d{b}", [tok[b]], [0]) for b in range(BATCH)]).next_tokens.cpu()
        ms_decode = _time(torch, decode, min(steps, 40), warmup)
        launches = ex.launches_last_step
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            relaunch_last_step(ex)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            relaunch_last_step(ex)
        ms_decode_graph = _time(torch, graph.replay, steps, warmup)
        del graph
        h2d = BATCH * (4 + 8 + 8 + 4 + 4 + 4 + 4) + BATCH * ((CTX + 64) // page + 1) * 4
        for b in range(BATCH):
            eng.finish_request(f"d{b}")
        del eng, ex
        torch.cuda.empty_cache()
        runs = len(spec.layers)
        llama = dict(width=s["width"], heads=s["heads"], kv_heads=8, dim=s["dim"], ff=s["top"] * s["ff"] + s["shared_ff"], vocab=s["vocab"],
                     layers=runs)
        ms_llama = _llama_decode(torch, llama, dev, steps, warmup)
        rows = _kernel_rows(torch, s, dev, max(3, steps // 2), 3, hbm, tf)
        torch.cuda.empty_cache()
        out_sizes[name] = {
            "sizes": s, "layer_runs": runs, "prefill_tokens_per_s": round(PROMPT / ms_prefill * 1e3, 1), "prefill_ms": round(ms_prefill, 3),
            "prefill_launches": prefill_launches,
            "decode_tokens_per_s": round(BATCH / ms_decode * 1e3, 1), "decode_ms_per_step": round(ms_decode, 4),
            "decode_graph_tokens_per_s": round(BATCH / ms_decode_graph * 1e3, 1), "decode_graph_ms_per_step": round(ms_decode_graph, 4),
            "llama_equal_size": llama, "llama_decode_tokens_per_s": round(BATCH / ms_llama * 1e3, 1) if ms_llama else None,
            "llama_decode_ms_per_step": round(ms_llama, 4) if ms_llama else None,
            "decode_launches_per_step": launches, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": BATCH * 4, "kernels": rows,
        }
        headline = out_sizes[name]
    line = {
        "metric": "Patadra decode tokens/s, batch 32, context 4096, 4k-wide layer sizes (2 layer runs), through the engine's executor",
        "value": headline["decode_graph_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": headline["decode_graph_ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, random tokens)", "impl": "ours",
        "gpu_launches": headline["decode_launches_per_step"],
        "e2e": {"value": headline["decode_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": headline["h2d_bytes_per_step"],
                "d2h_bytes_per_step": headline["d2h_bytes_per_step"]},
        "config": {"design": "Patadra", "batch": BATCH, "ctx": CTX, "prompt": PROMPT, "peaks": src, "hbm_gbs": hbm, "bf16_tflops": tf,
                   "l2": "kernel rows flush L2 between iterations; model steps stream more than L2", "sizes": out_sizes},
    }
    os.write(json_fd, (json.dumps(line) + "\n").encode())
