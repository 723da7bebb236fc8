"""Patadra: a pre-norm decoder of latent-attention layers with mixture-of-experts feed-forwards.

config.json gives every size and every constant that can differ between checkpoints:
  architecture "Patadra", vocab, width, max_positions, norm {eps, groups}, logit_softcap, token_side {dim},
  loop {start, stop, times}, and `layers`: per layer its `type` ("latent_attention"), the mixer's sizes
  (`mixer`: heads, dim, vdim, q_rank, kv_rank, scale, mask {size}) and its feed-forward (`mlp`: null, or
  {kind "moe", router {experts, top}, expert {ff, limit}, shared {ff, limit} or null}).
Fixed by the design (and therefore constants here): a learned position table added to the embedding; RMS
norms with plain weights over `groups` equal parts of the row; every sublayer's result times
sigmoid(W h + b) of the sublayer's input; the softmax sink; router scores are sigmoids, not renormalized,
and scale the expert's input; the expert activation g sigmoid(1.702 g) (u + 1) on clamped g and u; the shared
expert's per-token sigmoid gate; the token side input gelu_tanh(W x) * e projected back and added at unit RMS
after the feed-forward; layers `start .. stop - 1` run `times` times in a row with the same weights and a cache
per run; a tanh cap on the logits.

Checkpoint tensors: embed, pos, head, final.norm, side.embed, and per layer i `l<i>.norm1 / norm2`,
`l<i>.rg1 / rg2` (+ `.b`), `l<i>.mix.{dq, dkv, uq, uk, uv, o}`, `l<i>.mix.{dq, dkv}.norm`, `l<i>.mix.sink`,
`l<i>.mlp.router`, `l<i>.mlp.e<k>.{gate, up, down}`, `l<i>.mlp.shared.{gate, up, down, sg}`,
`l<i>.side.{gate, proj, norm}`.
This module turns that into the generic hybrid description (hybrid.py); it has no compute of its own.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .hybrid import HybridSpec, LatentAttentionSpec, LayerSpec, MoeSpec
from .ops import AtomaError

ARCHITECTURE = "Patadra"
ACT_ALPHA = 1.702
ACT_UP_SHIFT = 1.0


def layer_runs(cfg: dict) -> List[int]:
    """The order in which the configured layers run: the looped span repeated in place."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop.get("times", 1))
    if not 0 <= start <= stop <= n or times < 1:
        raise AtomaError(f"loop {loop} does not fit {n} layers")
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def _layer_spec(i: int, l: dict, side: bool) -> LayerSpec:
    if l.get("type") != "latent_attention":
        raise AtomaError(f"layer {i}: mixer type {l.get('type')!r} is not part of the Patadra design")
    m = l["mixer"]
    mask = m.get("mask") or {}
    att = LatentAttentionSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), q_rank=int(m["q_rank"]),
                              kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), window=int(mask.get("size") or 0), sink=True)
    moe = None
    if l.get("mlp") is not None:
        f = l["mlp"]
        if f.get("kind", "moe") != "moe":
            raise AtomaError(f"layer {i}: feed-forward kind {f.get('kind')!r} is not part of the Patadra design")
        sh = f.get("shared") or None
        moe = MoeSpec(experts=int(f["router"]["experts"]), top=int(f["router"]["top"]), ff=int(f["expert"]["ff"]),
                      limit=float(f["expert"].get("limit") or 0.0), shared_ff=int(sh["ff"]) if sh else 0,
                      shared_limit=float(sh.get("limit") or 0.0) if sh else 0.0, shared_gate=bool(sh), alpha=ACT_ALPHA,
                      up_shift=ACT_UP_SHIFT, renormalize=False)
    return LayerSpec("latent_attention", latent=att, moe=moe, gated_residual=True, side_part=i if side else None, source=i)


def spec_from_config(cfg: dict) -> HybridSpec:
    side_dim = int((cfg.get("token_side") or {}).get("dim") or 0)
    per_layer = [_layer_spec(i, l, side_dim > 0) for i, l in enumerate(cfg["layers"])]
    runs = tuple(per_layer[i] for i in layer_runs(cfg))
    norm = cfg.get("norm") or {}
    return HybridSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), eps=float(norm.get("eps", 1e-6)), logit_scale=1.0, layers=runs,
                      norm_offset=0.0, block_style="prenorm", norm_groups=int(norm.get("groups") or 1), position="learned",
                      max_positions=int(cfg["max_positions"]), logit_softcap=float(cfg.get("logit_softcap") or 0.0), side_dim=side_dim)


def weights_from_checkpoint(spec: HybridSpec, cfg: dict, ckpt: Dict[str, torch.Tensor]) -> dict:
    """Checkpoint names -> the generic hybrid layout: one entry per configured layer (runs share it), the projections that
    read the same input stacked for one product, the experts stacked into [experts, ., .] tensors."""
    W = spec.width

    def get(name, shape):
        if name not in ckpt:
            raise AtomaError(f"tensor {name} is missing from the checkpoint")
        t = ckpt[name]
        if tuple(t.shape) != tuple(shape):
            raise AtomaError(f"tensor {name} has shape {tuple(t.shape)}, the configuration needs {tuple(shape)}")
        return t

    def at_least(name, rows, cols):
        """A table that may hold more rows / columns than the configuration uses."""
        if name not in ckpt:
            raise AtomaError(f"tensor {name} is missing from the checkpoint")
        t = ckpt[name]
        if t.dim() != 2 or t.shape[0] < rows or t.shape[1] < cols:
            raise AtomaError(f"tensor {name} has shape {tuple(t.shape)}, the configuration needs at least {(rows, cols)}")
        return t

    n_layers = len(cfg["layers"])
    out = {"embed": get("embed", (spec.vocab, W)), "head": get("head", (spec.vocab, W)), "final_norm": get("final.norm", (W,)),
           "pos": at_least("pos", spec.max_positions, W)[:, :W], "layers": []}
    if spec.side_dim > 0:
        out["side_table"] = at_least("side.embed", spec.vocab, n_layers * spec.side_dim)
    by_source = {ls.source: ls for ls in spec.layers}
    for i in range(n_layers):
        ls = by_source.get(i)
        if ls is None:          # a layer no run uses (an empty loop span cannot produce this; kept for safety)
            out["layers"].append({})
            continue
        a, p = ls.latent, f"l{i}."
        w = {"norm1": get(p + "norm1", (W,)),
             "w_down_in": torch.cat([get(p + "mix.dq", (a.q_rank, W)), get(p + "mix.dkv", (a.kv_rank, W)), get(p + "rg1", (W, W))], 0),
             "gate1_bias": get(p + "rg1.b", (W,)),
             "dq_norm": get(p + "mix.dq.norm", (a.q_rank,)), "dkv_norm": get(p + "mix.dkv.norm", (a.kv_rank,)),
             "w_uq": get(p + "mix.uq", (a.heads * a.dim, a.q_rank)), "w_uk": get(p + "mix.uk", (a.heads * a.dim, a.kv_rank)),
             "w_uv": get(p + "mix.uv", (a.heads * a.vdim, a.kv_rank)), "sink": get(p + "mix.sink", (a.heads,)),
             "w_o": get(p + "mix.o", (W, a.heads * a.vdim))}
        if ls.moe is not None:
            e, q = ls.moe, p + "mlp."
            w["norm2"], w["gate2_bias"] = get(p + "norm2", (W,)), get(p + "rg2.b", (W,))
            w["w_router"] = get(q + "router", (e.experts, W))
            w["w_expert_gate_up"] = torch.stack([torch.cat([get(f"{q}e{k}.gate", (e.ff, W)), get(f"{q}e{k}.up", (e.ff, W))], 0)
                                                 for k in range(e.experts)], 0)
            w["w_expert_down"] = torch.stack([get(f"{q}e{k}.down", (W, e.ff)) for k in range(e.experts)], 0)
            ff_in = []
            if e.shared_ff > 0:
                ff_in += [get(q + "shared.gate", (e.shared_ff, W)), get(q + "shared.up", (e.shared_ff, W))]
                w["w_down"] = get(q + "shared.down", (W, e.shared_ff))
                w["w_shared_gate"] = get(q + "shared.sg", (1, W)).reshape(W)
            w["w_ff_in"] = torch.cat(ff_in + [get(p + "rg2", (W, W))], 0)
        if ls.side_part is not None:
            D = spec.side_dim
            w["side_gate"], w["side_proj"] = get(p + "side.gate", (D, W)), get(p + "side.proj", (W, D))
            w["side_norm"] = get(p + "side.norm", (W,))
        out["layers"].append(w)
    return out
