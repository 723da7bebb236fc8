"""Plain float64 restatement of the Patadra design: one function per mechanism, Python loops, whole sequences,
no paging, no batching.  It shares no code with the package; the GPU tests compare the framework against it.

Notation: x is the residual stream [T, W]; h a normed sublayer input; W_* matrices are stored [out, in] and applied
as `h @ W.T`; sigma is the logistic function.
"""
import math

import torch

F64 = torch.float64


def sigma(z):
    return 1.0 / (1.0 + torch.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ---- norms ----
def unit_rms(v, eps):
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def group_norm(v, weight, groups, eps):
    """The row is cut into `groups` equal consecutive parts, each brought to unit RMS on its own; then the weight."""
    parts = v.reshape(*v.shape[:-1], groups, v.shape[-1] // groups)
    return unit_rms(parts, eps).reshape(v.shape) * weight


# ---- embedding ----
def embed(tokens, positions, table, pos_table):
    return table[torch.as_tensor(tokens)] + pos_table[torch.as_tensor(positions)]


# ---- gated residual ----
def residual_gate(h, w_gate, b_gate):
    return sigma(h @ w_gate.T + b_gate)


# ---- latent attention ----
def latents(h, w_dq, n_dq, w_dkv, n_dkv, eps):
    """(query latent, key/value latent), each an RMS norm with a plain weight of a down projection of h."""
    return unit_rms(h @ w_dq.T, eps) * n_dq, unit_rms(h @ w_dkv.T, eps) * n_dkv


def windowed_sink_softmax(scores, sink):
    """scores [n] of the visible keys of one head; the denominator has one more term exp(sink)."""
    m = max(float(scores.max()), float(sink))
    e = torch.exp(scores - m)
    return e / (e.sum() + math.exp(float(sink) - m))


def latent_attention_heads(c_q, c, w_uq, w_uk, w_uv, sink, heads, dim, vdim, scale, window, first_query=0):
    """c_q [Tq, q_rank] are the queries of positions first_query .. first_query + Tq - 1; c [Tk, kv_rank] the latents of positions
    0 .. Tk - 1.  Returns the concatenated heads [Tq, heads vdim].  Position i sees j with 0 <= i - j < window (window 0: all j <= i)."""
    Tq = c_q.shape[0]
    q = (c_q @ w_uq.T).reshape(Tq, heads, dim)
    k = (c @ w_uk.T).reshape(-1, heads, dim)
    v = (c @ w_uv.T).reshape(-1, heads, vdim)
    out = torch.zeros(Tq, heads, vdim, dtype=F64)
    for t in range(Tq):
        i = first_query + t
        lo = max(0, i - window + 1) if window > 0 else 0
        for hd in range(heads):
            s = (k[lo:i + 1, hd] @ q[t, hd]) * scale
            out[t, hd] = windowed_sink_softmax(s, sink[hd]) @ v[lo:i + 1, hd]
    return out.reshape(Tq, heads * vdim)


# ---- experts ----
def expert(h, w_gate, w_up, w_down, limit, alpha=1.702, shift=1.0):
    g, u = h @ w_gate.T, h @ w_up.T
    if limit > 0:
        g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
    return (g * sigma(alpha * g) * (u + shift)) @ w_down.T


def route(h, w_router, top):
    """(chosen experts [T, top], their sigmoid scores [T, top]); the scores are used as they are."""
    s = sigma(h @ w_router.T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val


def mixture(h, w, prefix, mlp):
    """sum over the chosen experts of expert(score * h), plus the shared expert times sigma(w_sg . h)."""
    idx, val = route(h, w[prefix + "router"], mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), val[t]):
            p = f"{prefix}e{e}."
            out[t] += expert(s * h[t], w[p + "gate"], w[p + "up"], w[p + "down"], mlp["expert"]["limit"])
    if mlp.get("shared"):
        p = prefix + "shared."
        out = out + expert(h, w[p + "gate"], w[p + "up"], w[p + "down"], mlp["shared"]["limit"]) * sigma(h @ w[p + "sg"].T)
    return out


# ---- token side input ----
def side_input(x, tokens, side_table, part, dim, w_gate, w_proj, w_norm, eps):
    e = side_table[torch.as_tensor(tokens)][:, part * dim:(part + 1) * dim]
    y = (gelu_tanh(x @ w_gate.T) * e) @ w_proj.T
    return unit_rms(y, eps) * w_norm


# ---- the model ----
def run_order(cfg):
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return list(range(n))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence from position 0 (and the residual stream after every layer run)."""
    w = {k: v.to(F64) for k, v in w.items()}
    T, eps, groups = len(tokens), cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = embed(tokens, list(range(T)), w["embed"], w["pos"])
    side = (cfg.get("token_side") or {}).get("dim", 0)
    trace = []
    for i in run_order(cfg):
        l, p = cfg["layers"][i], f"l{i}."
        m = l["mixer"]
        h = group_norm(x, w[p + "norm1"], groups, eps)
        c_q, c = latents(h, w[p + "mix.dq"], w[p + "mix.dq.norm"], w[p + "mix.dkv"], w[p + "mix.dkv.norm"], eps)
        a = latent_attention_heads(c_q, c, w[p + "mix.uq"], w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.sink"], m["heads"], m["dim"],
                                   m["vdim"], m["scale"], (m.get("mask") or {}).get("size", 0))
        x = x + (a @ w[p + "mix.o"].T) * residual_gate(h, w[p + "rg1"], w[p + "rg1.b"])
        if l["mlp"] is not None:
            h = group_norm(x, w[p + "norm2"], groups, eps)
            x = x + mixture(h, w, p + "mlp.", l["mlp"]) * residual_gate(h, w[p + "rg2"], w[p + "rg2.b"])
        if side:
            x = x + side_input(x, tokens, w["side.embed"], i, side, w[p + "side.gate"], w[p + "side.proj"], w[p + "side.norm"], eps)
        trace.append(x.clone())
    lg = group_norm(x, w["final.norm"], groups, eps) @ w["head"].T
    cap = cfg.get("logit_softcap") or 0.0
    if cap > 0:
        lg = cap * torch.tanh(lg / cap)
    return (lg, trace) if return_layers else lg


# ---- random models for the tests ----
def random_config(width=48, vocab=61, heads=3, dim=8, vdim=12, q_rank=24, kv_rank=16, window=20, experts=5, top=2, ff=24, shared_ff=40,
                  limit=1.5, shared_limit=2.5, groups=3, layers=3, loop=(1, 2, 2), side=6, softcap=9.0, max_positions=256,
                  no_mlp_layers=(), eps=1e-5, scale=None):
    def layer(i):
        mlp = None
        if i not in no_mlp_layers:
            mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
                   "shared": {"ff": shared_ff, "limit": shared_limit} if shared_ff else None}
        return {"type": "latent_attention",
                "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                          "scale": scale if scale is not None else dim ** -0.5, "mask": {"size": window}}, "mlp": mlp}
    cfg = {"architecture": "Patadra", "vocab": vocab, "width": width, "max_positions": max_positions,
           "norm": {"eps": eps, "groups": groups}, "layers": [layer(i) for i in range(layers)]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if side:
        cfg["token_side"] = {"dim": side}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


def random_weights(cfg, g):
    """bfloat16-representable float32 tensors under the checkpoint's names."""
    W, V = cfg["width"], cfg["vocab"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(torch.bfloat16).float()

    def vec(n, mean=0.0, s=1.0):
        return (mean + s * torch.randn(n, generator=g)).to(torch.bfloat16).float()

    side = (cfg.get("token_side") or {}).get("dim", 0)
    w = {"embed": mat(V, W, math.sqrt(W)), "pos": mat(cfg["max_positions"], W, 0.5 * math.sqrt(W)), "head": mat(V, W, 2.0),
         "final.norm": vec(W, 1.0, 0.2)}
    if side:
        w["side.embed"] = mat(V, side * len(cfg["layers"]), math.sqrt(side * len(cfg["layers"])))
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        w[p + "norm1"], w[p + "norm2"] = vec(W, 1.0, 0.2), vec(W, 1.0, 0.2)
        w[p + "rg1"], w[p + "rg1.b"], w[p + "rg2"], w[p + "rg2.b"] = mat(W, W), vec(W, 0.5, 0.5), mat(W, W), vec(W, 0.5, 0.5)
        w[p + "mix.dq"], w[p + "mix.dq.norm"] = mat(m["q_rank"], W), vec(m["q_rank"], 1.0, 0.2)
        w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(m["kv_rank"], W), vec(m["kv_rank"], 1.0, 0.2)
        w[p + "mix.uq"] = mat(m["heads"] * m["dim"], m["q_rank"], 2.0)
        w[p + "mix.uk"] = mat(m["heads"] * m["dim"], m["kv_rank"], 2.0)
        w[p + "mix.uv"] = mat(m["heads"] * m["vdim"], m["kv_rank"])
        w[p + "mix.sink"] = vec(m["heads"], 0.0, 1.0)
        w[p + "mix.o"] = mat(W, m["heads"] * m["vdim"])
        if l["mlp"] is not None:
            f = l["mlp"]
            w[p + "mlp.router"] = mat(f["router"]["experts"], W, 2.0)
            for e in range(f["router"]["experts"]):
                q = f"{p}mlp.e{e}."
                w[q + "gate"], w[q + "up"], w[q + "down"] = mat(f["expert"]["ff"], W, 2.0), mat(f["expert"]["ff"], W, 2.0), mat(W, f["expert"]["ff"])
            if f.get("shared"):
                q, n = p + "mlp.shared.", f["shared"]["ff"]
                w[q + "gate"], w[q + "up"], w[q + "down"], w[q + "sg"] = mat(n, W, 2.0), mat(n, W, 2.0), mat(W, n), mat(1, W)
        if side:
            w[p + "side.gate"], w[p + "side.proj"], w[p + "side.norm"] = mat(side, W), mat(W, side), vec(W, 0.5, 0.2)
    return w
