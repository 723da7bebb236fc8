"""bench.py --design lilovik: prefill and decode throughput of the Lilovik design (random weights) at sizes that
resemble real models' layers, beside the framework's closest existing model — Llama — at equal sizes, and the
design's hot kernels against the measured peaks beside their Llama counterparts.  Not the headline (config 2 is);
ONE JSON line in the same format.

Per size: a model of a few layers (one minGRU layer among attention layers, each with its feed-forward) is served
through the engine's executor: `prefill` = one 4096-token prompt in one step; `decode` = one step of 32 sequences at
context 4096 (built by prefilling them), timed with CUDA events around K executor steps after W warm-up steps, inputs
shipped from pinned memory every step, sampled tokens read back.  `llama_decode` = the Llama decode-step executor
(CUDA graph) with the same width, heads, head size, feed-forward size and layer count at the same batch and context.
Kernel rows: achieved FLOP/s or bytes/s over the measured peaks of MEASURED_PEAKS.json (fallback figures when absent).
Every timed loop works on more than L2 (126 MB) of cache + weights, or flushes L2 between iterations."""
from __future__ import annotations

import json
import os
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

SIZES = {
    # name: width, heads, kv heads, head size, ff, state width, vocab, layers
    "1b-like": dict(width=2048, heads=32, kv_heads=8, dim=64, ff=8192, state=2048, vocab=32000, layers=4),
    "8b-like": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, state=4096, vocab=32000, layers=3),
}
BATCH, CTX, PROMPT = 32, 4096, 4096


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def _time(torch, fn, steps, warmup, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(steps):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / steps


def _spec(torch, s):
    import math
    from atoma_infer_b200.hybrid import AttentionSpec, HybridSpec, LayerSpec, MinGruSpec, MlpSpec, slopes_power_of_two
    att = AttentionSpec(s["heads"], s["kv_heads"], s["dim"], s["dim"], 1.0 / math.sqrt(s["dim"]), 30.0, 0.25, 64,
                        tuple(slopes_power_of_two(s["heads"])))
    layers = []
    for i in range(s["layers"]):
        if i == 1:
            layers.append(LayerSpec("mingru", mingru=MinGruSpec(s["state"]), mlp=MlpSpec(s["ff"], "relu")))
        else:
            layers.append(LayerSpec("attention", attention=att, mlp=MlpSpec(s["ff"], "relu")))
    return HybridSpec(s["width"], s["vocab"], 1e-6, 1.0, tuple(layers))


def _weights(torch, spec, dev):
    g = torch.Generator(device=dev).manual_seed(11)
    bf = torch.bfloat16

    def r(*shape, scale=1.0):
        return (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * scale).to(bf)

    W = spec.width
    out = {"embed": r(spec.vocab, W), "head": r(spec.vocab, W, scale=W ** -0.5), "final_norm": r(W, scale=0.1), "layers": []}
    for ls in spec.layers:
        w = {"norm1": r(W, scale=0.1), "norm1b": r(W, scale=0.1), "norm2": r(W, scale=0.1), "norm2b": r(W, scale=0.1)}
        if ls.mixer == "attention":
            a = ls.attention
            n = (a.heads + a.kv_heads) * a.dim + a.kv_heads * a.vdim
            w.update(w_qkv=r(n, W, scale=W ** -0.5), b_qkv=r(n, scale=0.1), q_norm=1 + r(a.heads * a.dim, scale=0.1),
                     k_norm=1 + r(a.kv_heads * a.dim, scale=0.1),
                     talk=torch.eye(a.heads, device=dev) + 0.1 * r(a.heads, a.heads).float(), head_bias=r(a.heads, scale=0.5) - 1,
                     w_o=r(W, a.heads * a.vdim, scale=(a.heads * a.vdim) ** -0.5))
        else:
            S = ls.mingru.width
            w.update(w_zxg=r(3 * S, W, scale=W ** -0.5), b_zxg=r(3 * S, scale=0.3), w_o=r(W, S, scale=S ** -0.5))
        w.update(w_gate_up=r(2 * ls.mlp.ff, W, scale=W ** -0.5), w_down=r(W, ls.mlp.ff, scale=ls.mlp.ff ** -0.5))
        out["layers"].append(w)
    return out


def _llama_decode(torch, s, dev, steps, warmup):
    from atoma_infer_b200 import ops
    from atoma_infer_b200.llama import DecodeStep, LlamaConfig, LlamaShard
    page = 16
    cfg = LlamaConfig(hidden_size=s["width"], intermediate_size=s["ff"], vocab_size=s["vocab"], num_hidden_layers=s["layers"],
                      num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"], max_position_embeddings=CTX + 16)
    if cfg.head_dim != s["dim"]:
        return None
    shard = LlamaShard.random_init(cfg, device=dev, seed=5)
    mb = (CTX + page) // page
    nb = BATCH * mb + 1
    kv = [torch.randn((2, nb, page, s["kv_heads"], s["dim"]), device=dev, dtype=torch.bfloat16) for _ in range(s["layers"])]
    bt = torch.randperm(nb, device=dev)[: BATCH * mb].to(torch.int32).reshape(BATCH, mb)
    lens = torch.full((BATCH,), CTX + 1, dtype=torch.int32, device=dev)
    pos = lens.long() - 1
    slots = bt[torch.arange(BATCH, device=dev), (pos // page)].long() * page + pos % page
    tokens = torch.randint(0, cfg.vocab_size, (BATCH,), dtype=torch.int32, device=dev)
    ops.set_launch_mode(pdl=True, const_weights=True)
    try:
        step = DecodeStep(shard, kv, max_batch=BATCH)
        step.bind(tokens, pos, slots, bt, lens)
        step.capture()
        ms = _time(torch, step.run, steps, warmup)
        step.check()
        launches = None
    finally:
        ops.set_launch_mode()
    del step, kv, shard
    torch.cuda.empty_cache()
    return ms


def _kernel_rows(torch, s, dev, steps, warmup, hbm, tf):
    """The design's attention kernels beside Llama's at the same shapes."""
    import math
    import numpy as np
    from atoma_infer_b200 import hybrid_ops as ho, ops
    H, G, D = s["heads"], s["kv_heads"], s["dim"]
    bf = torch.bfloat16
    page, S = 16, PROMPT
    rows = {}
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    # ---- prompt attention, one causal prompt of S tokens ----
    nb = S // page
    kc = torch.randn((nb * page, G, D), device=dev, dtype=bf)
    vc = torch.randn((nb * page, G, D), device=dev, dtype=bf)
    q = torch.randn((S, H * D), device=dev, dtype=bf)
    pos = torch.arange(S, device=dev, dtype=torch.int64)
    tseq = torch.zeros(S, device=dev, dtype=torch.int32)
    bt = torch.arange(nb, device=dev, dtype=torch.int32).reshape(1, nb)
    qs = torch.tensor([0, S], device=dev, dtype=torch.int32)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
    pb = torch.zeros(H, device=dev) - 1
    talk = torch.eye(H, device=dev) + 0.05
    f = lambda: ho.sigmoid_attention_paged(q, kc, vc, pos, tseq, bt, slopes, pb, talk, H, G, D, D, page, 1 / math.sqrt(D), 30.0, S,
                                           query_start=qs, max_seq_len=S)
    ms = _time(torch, f, steps, warmup, flush)
    flops = 4.0 * H * D * S * (S + 1) / 2
    rows["attention_prefill"] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "frac_of_bf16_peak": round(flops / ms / 1e9 / tf, 3)}
    q3, k3, v3 = q.view(S, H, D), kc.view(S, G, D), vc.view(S, G, D)
    cu = torch.tensor([0, S], device=dev, dtype=torch.int32)
    f = lambda: ops.flash_attn_varlen(q3, k3, v3, cu, cu, S, S, 1 / math.sqrt(D), True)
    ms = _time(torch, f, steps, warmup, flush)
    rows["llama_attention_prefill"] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "frac_of_bf16_peak": round(flops / ms / 1e9 / tf, 3)}
    # ---- decode attention, BATCH sequences at context CTX ----
    mb = (CTX + page) // page
    nb = BATCH * mb
    kc = torch.randn((nb * page, G, D), device=dev, dtype=bf)
    vc = torch.randn((nb * page, G, D), device=dev, dtype=bf)
    q = torch.randn((BATCH, H * D), device=dev, dtype=bf)
    pos = torch.full((BATCH,), CTX, device=dev, dtype=torch.int64)
    tseq = torch.arange(BATCH, device=dev, dtype=torch.int32)
    bt = torch.randperm(nb, device=dev).to(torch.int32).reshape(BATCH, mb)
    qs = torch.arange(BATCH + 1, device=dev, dtype=torch.int32)
    f = lambda: ho.sigmoid_attention_paged(q, kc, vc, pos, tseq, bt, slopes, pb, talk, H, G, D, D, page, 1 / math.sqrt(D), 30.0, 1,
                                           query_start=qs, max_seq_len=CTX + 1)
    ms = _time(torch, f, steps, warmup, flush)
    nbytes = BATCH * (CTX + 1) * G * 2 * D * 2
    rows["attention_decode"] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms / 1e6 / hbm, 3)}
    kv = torch.stack([kc.view(nb, page, G, D), vc.view(nb, page, G, D)])
    q4 = q.view(BATCH, 1, H, D)
    sl = torch.full((BATCH,), CTX + 1, device=dev, dtype=torch.int32)
    f = lambda: ops.flash_attn_kv_cache_full(q4, kv[0], kv[1], None, 1 / math.sqrt(D), bt, sl, True)
    ms = _time(torch, f, steps, warmup, flush)
    rows["llama_attention_decode"] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms / 1e6 / hbm, 3)}
    # ---- minGRU scan over one prompt, and the fused sandwich norm (both stream their rows once) ----
    Sw = s["state"]
    zxg = torch.randn((S, 3 * Sw), device=dev, dtype=bf)
    state = torch.zeros((1, Sw), device=dev)
    z32 = torch.zeros(1, device=dev, dtype=torch.int32)
    f = lambda: ho.mingru_scan(zxg, None, state, z32, cu, z32, S)
    ms = _time(torch, f, steps, warmup, flush)
    nbytes = S * 4 * Sw * 2
    rows["mingru_scan_prefill"] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms / 1e6 / hbm, 3)}
    W = s["width"]
    T = 8192
    y = torch.randn((T, W), device=dev, dtype=bf)
    x = torch.randn((T, W), device=dev)
    w1 = torch.zeros(W, device=dev)
    f = lambda: ho.postnorm_add_prenorm(y, x, w1, w1, 1e-5, 1.0)
    ms = _time(torch, f, steps, warmup, flush)
    nbytes = T * W * (2 + 4 + 4 + 2)
    rows["postnorm_add_prenorm"] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms / 1e6 / hbm, 3)}
    res = torch.randn((T, W), device=dev, dtype=bf)
    wbf = torch.ones(W, device=dev, dtype=bf)
    f = lambda: ops.add_rmsnorm(y, res, wbf, 1e-5) if hasattr(ops, "add_rmsnorm") else None
    if hasattr(ops, "add_rmsnorm"):
        ms = _time(torch, f, steps, warmup, flush)
        nbytes = T * W * 2 * 4
        rows["llama_add_rmsnorm"] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms / 1e6 / hbm, 3)}
    return rows


def run(args, torch, dev, json_fd):
    import numpy as np
    from atoma_infer_b200 import _lib
    from atoma_infer_b200.cache import CacheManager
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.hybrid import HybridExecutor
    if args.impl != "ours":
        os.write(json_fd, (json.dumps({"impl": "reference", "unavailable": "the reference has no model of this design"}) + "\n").encode())
        return
    _lib.lib()
    hbm, tf, src = _peaks()
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    page = 16
    out_sizes = {}
    headline = None
    for name, s in SIZES.items():
        spec = _spec(torch, s)
        weights = _weights(torch, spec, dev)
        nblocks = BATCH * ((CTX + 64) // page + 1) + PROMPT // page + 8
        ex = HybridExecutor(spec, weights, torch.bfloat16, dev, nblocks, page, BATCH + 1)
        del weights
        eng = Engine(ex, CacheManager(nblocks, page, BATCH + 1), max_num_batched_tokens=PROMPT, max_num_seqs=BATCH + 1)
        rng = np.random.default_rng(0)
        prompt = rng.integers(0, s["vocab"], size=PROMPT).tolist()
        # prefill: one whole prompt per step (admit, run, end: pages and the state slot are reused every iteration)
        def prefill():
            eng.step_forced([("p", prompt, [PROMPT - 1])], end=["p"]).next_tokens.cpu()
        ms_prefill = _time(torch, prefill, steps, warmup)
        # decode: BATCH live sequences at context CTX
        for b in range(BATCH):
            eng.step_forced([(f"d{b}", rng.integers(0, s["vocab"], size=CTX).tolist(), [])])
        tok = [int(t) for t in rng.integers(0, s["vocab"], size=BATCH)]
        n_dec = [0]

        def decode():
            n_dec[0] += 1
            eng.step_forced([(f"d{b}", [tok[b]], [0]) for b in range(BATCH)]).next_tokens.cpu()
        ms_decode = _time(torch, decode, min(steps, 48), warmup)
        launches = ex.launches_last_step
        # the same step's kernels alone: inputs already on the device, replayed from a CUDA graph (as the Llama step is)
        from atoma_infer_b200.hybrid import relaunch_last_step
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
        ms_llama = _llama_decode(torch, s, dev, steps, warmup)
        rows = _kernel_rows(torch, s, dev, max(3, steps // 2), 3, hbm, tf)
        torch.cuda.empty_cache()
        out_sizes[name] = {
            "sizes": s, "prefill_tokens_per_s": round(PROMPT / ms_prefill * 1e3, 1), "prefill_ms": round(ms_prefill, 3),
            "decode_tokens_per_s": round(BATCH / ms_decode * 1e3, 1), "decode_ms_per_step": round(ms_decode, 4),
            "decode_graph_tokens_per_s": round(BATCH / ms_decode_graph * 1e3, 1), "decode_graph_ms_per_step": round(ms_decode_graph, 4),
            "llama_decode_tokens_per_s": round(BATCH / ms_llama * 1e3, 1) if ms_llama else None,
            "llama_decode_ms_per_step": round(ms_llama, 4) if ms_llama else None,
            "decode_launches_per_step": launches, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": BATCH * 4, "kernels": rows,
        }
        if name == "8b-like":
            headline = out_sizes[name]
    line = {
        "metric": "Lilovik decode tokens/s, batch 32, context 4096, 8b-like layer sizes (3 layers), through the engine's executor",
        "value": headline["decode_graph_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": headline["decode_graph_ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, random tokens)", "impl": "ours",
        "gpu_launches": headline["decode_launches_per_step"],
        "e2e": {"value": headline["decode_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": headline["h2d_bytes_per_step"],
                "d2h_bytes_per_step": headline["d2h_bytes_per_step"]},
        "config": {"design": "Lilovik", "batch": BATCH, "ctx": CTX, "prompt": PROMPT, "peaks": src, "hbm_gbs": hbm, "bf16_tflops": tf,
                   "l2": "kernel rows flush L2 between iterations; model steps stream more than L2", "sizes": out_sizes},
    }
    os.write(json_fd, (json.dumps(line) + "\n").encode())
