"""A plain, slow restatement of the Lilovik design, one function per mechanism, for the tests.

Lilovik is a decoder-only model whose layers are either a sigmoid ("softmax-free") attention with a
talking-heads mix of the attention weights, or a minGRU recurrence; sublayers are wrapped in RMS norms
on both sides and the residual stream carries a sinusoidal position signal added to the embedding.

Everything here runs on whole sequences in the dtype it is given (float64 in the tests) with Python
loops over heads and tokens.  Nothing is shared with the product: no paging, no batching, no kernels.
Weights are a dict name -> torch tensor, the names of a checkpoint's tensors.
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms(x, eps) * (1.0 + w)


def sinusoid(positions, width, dtype):
    """Row p: entry 2i = sin(p / 10000^(2i/width)), entry 2i+1 = cos of the same angle."""
    out = torch.zeros((len(positions), width), dtype=dtype)
    for r, p in enumerate(positions):
        for c in range(width):
            i = c // 2
            ang = float(p) * 10000.0 ** (-2.0 * i / width)
            out[r, c] = math.sin(ang) if c % 2 == 0 else math.cos(ang)
    return out


def embed(weights, tokens, first_position=0):
    e = weights["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    pos = list(range(first_position, first_position + len(tokens)))
    return e + sinusoid(pos, e.shape[-1], e.dtype)


def distance_slopes(heads):
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def query_temperature(p, coef, every):
    return 1.0 + coef * math.log(math.floor((p + 1) / every) + 1.0)


def attention_core(q, k, v, m, head_bias, talk, first_position=0):
    """q [n, H, D] (already normed and tempered) against keys / values [t, G, D] / [t, G, Dv] of positions 0 .. t-1;
    query r sits at position first_position + r.  Returns [n, H, Dv]."""
    H, G, Dv = m["heads"], m["kv_heads"], v.shape[-1]
    n, t = q.shape[0], k.shape[0]
    slopes = distance_slopes(H)
    cap = m.get("softcap") or 0.0
    weight = torch.zeros((H, n, t), dtype=q.dtype)
    i = first_position + torch.arange(n)[:, None]
    j = torch.arange(t)[None, :]
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        s = s - slopes[h] * (i - j).to(q.dtype)
        a = torch.sigmoid(s + head_bias[h])
        weight[h] = torch.where(j <= i, a, torch.zeros_like(a))
    mixed = torch.einsum("hg,gij->hij", talk, weight)
    out = torch.zeros((n, H, Dv), dtype=q.dtype)
    for h in range(H):
        out[:, h] = mixed[h] @ v[:, h // (H // G)]
    return out


def qkv_normed(w, pre, x, m, eps, first_position=0):
    """Projections with biases, the whole-projection q / k norms and the query temperature."""
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = x.shape[0]
    q = x @ w[pre + "q"].T + w[pre + "q.b"]
    k = x @ w[pre + "k"].T + w[pre + "k.b"]
    v = x @ w[pre + "v"].T + w[pre + "v.b"]
    q = rms(q, eps) * w[pre + "q.norm"]          # over the whole projection, all heads at once
    k = rms(k, eps) * w[pre + "k.norm"]
    temp = torch.tensor([query_temperature(first_position + r, m["q_temp"]["coef"], m["q_temp"]["every"]) for r in range(n)],
                        dtype=x.dtype)
    q = q * temp[:, None]
    return q.reshape(n, H, D), k.reshape(n, G, D), v.reshape(n, G, Dv)


def sigmoid_attention(w, pre, x, m, eps):
    """x [n, width] -> [n, width].  m: the layer's mixer sizes and constants."""
    q, k, v = qkv_normed(w, pre, x, m, eps)
    out = attention_core(q, k, v, m, w[pre + "pb"], w[pre + "talk"])
    return out.reshape(x.shape[0], -1) @ w[pre + "o"].T


def mingru(w, pre, x, state=None):
    """x [n, width] -> ([n, width], final state).  The state has the mixer's own width and starts at zero."""
    z = torch.sigmoid(x @ w[pre + "z"].T + w[pre + "z.b"])
    u = x @ w[pre + "x"].T + w[pre + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = x @ w[pre + "g"].T
    gate = gate * torch.sigmoid(gate)
    s = torch.zeros(z.shape[-1], dtype=x.dtype) if state is None else state
    rows = []
    for t in range(x.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        rows.append(s * gate[t])
    return torch.stack(rows) @ w[pre + "o"].T, s


def dense_ff(w, pre, x):
    return (torch.relu(x @ w[pre + "gate"].T) * (x @ w[pre + "up"].T)) @ w[pre + "down"].T


def forward(cfg, weights, tokens, return_layers=False):
    """Logits [n, vocab] of one whole sequence (and the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = embed(weights, tokens)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = norm_one_plus(x, weights[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = sigmoid_attention(weights, p + "mix.", h, layer["mixer"], eps)
        elif layer["type"] == "mingru":
            y, _ = mingru(weights, p + "mix.", h)
        else:
            raise ValueError(layer["type"])
        x = x + norm_one_plus(y, weights[p + "norm1b"], eps)
        if layer["mlp"] is not None:
            h = norm_one_plus(x, weights[p + "norm2"], eps)
            x = x + norm_one_plus(dense_ff(weights, p + "mlp.", h), weights[p + "norm2b"], eps)
        after.append(x)
    logits = norm_one_plus(x, weights["final.norm"], eps) @ weights["head"].T * cfg["logit_scale"]
    return (logits, torch.stack(after)) if return_layers else logits


def random_config(gen, width=48, vocab=61, layers=("attention", "mingru", "attention"), heads=4, kv_heads=2, dim=16, vdim=24,
                  ff=40, state=56, softcap=30.0, coef=0.25, every=8, logit_scale=0.7, eps=1e-5, mlp_on_mingru=False):
    """A small configuration in the checkpoint's config.json form."""
    out = []
    for t in layers:
        if t == "attention":
            out.append({"type": t, "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                             "scale": 1.0 / math.sqrt(dim), "softcap": softcap,
                                             "q_temp": {"coef": coef, "every": every}},
                        "mlp": {"kind": "dense", "ff": ff}})
        else:
            out.append({"type": t, "mixer": {"width": state},
                        "mlp": {"kind": "dense", "ff": ff} if mlp_on_mingru else None})
    return {"architecture": "Lilovik", "layers": out, "logit_scale": logit_scale, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


def random_weights(cfg, gen, dtype=torch.float64, round_to=torch.bfloat16):
    """Random weights with the checkpoint's names; values are representable in `round_to`."""
    W = cfg["width"]

    def r(*shape, scale=1.0):
        t = torch.randn(*shape, generator=gen, dtype=torch.float32) * scale
        return t.to(round_to).to(dtype)

    w = {"embed": r(cfg["vocab"], W), "final.norm": r(W, scale=0.1), "head": r(cfg["vocab"], W, scale=W ** -0.5)}
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer["mlp"] is not None else [])
        for nme in names:
            w[p + nme] = r(W, scale=0.1)
        m = layer["mixer"]
        if layer["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for nme, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                w[p + "mix." + nme] = r(rows, W, scale=W ** -0.5)
                w[p + "mix." + nme + ".b"] = r(rows, scale=0.1)
            w[p + "mix.q.norm"] = (1.0 + r(H * D, scale=0.1)).to(round_to).to(dtype)
            w[p + "mix.k.norm"] = (1.0 + r(G * D, scale=0.1)).to(round_to).to(dtype)
            w[p + "mix.talk"] = (torch.eye(H) + 0.3 * torch.randn(H, H, generator=gen)).to(round_to).to(dtype)
            w[p + "mix.pb"] = (r(H, scale=0.5) - 1.0).to(round_to).to(dtype)
            w[p + "mix.o"] = r(W, H * Dv, scale=(H * Dv) ** -0.5)
        else:
            S = m["width"]
            for nme in ("z", "x", "g"):
                w[p + "mix." + nme] = r(S, W, scale=W ** -0.5)
            w[p + "mix.z.b"] = r(S, scale=0.5)
            w[p + "mix.x.b"] = r(S, scale=0.5)
            w[p + "mix.o"] = r(W, S, scale=S ** -0.5)
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            w[p + "mlp.gate"] = r(F, W, scale=W ** -0.5)
            w[p + "mlp.up"] = r(F, W, scale=W ** -0.5)
            w[p + "mlp.down"] = r(W, F, scale=F ** -0.5)
    return w
