"""Lilovik: a decoder-only design of sigmoid-attention and minGRU layers between sandwich RMS norms.

config.json gives every size and every constant that can differ between checkpoints:
  architecture "Lilovik", vocab, width, logit_scale, norm.eps, and `layers`: per layer its `type`
  ("attention" | "mingru"), the mixer's sizes (`mixer`) and its feed-forward (`mlp`: {kind "dense", ff} or null).
Fixed by the design (and therefore constants here): norm weights are offsets from one; the position
signal is a sinusoid of base 10000 added to the embedding; attention heads get distance slopes
2^(-8 (h+1) / heads); the feed-forward is ReLU-gated; minGRU's candidate is u + 1/2 for u >= 0, sigmoid(u)
below; the final norm precedes the head and the logits are scaled by logit_scale.

Checkpoint tensors: embed, head, final.norm, and per layer i `l<i>.norm1 / norm1b / norm2 / norm2b`,
`l<i>.mix.{q,k,v}` (+ `.b` biases), `l<i>.mix.{q,k}.norm`, `l<i>.mix.talk`, `l<i>.mix.pb`, `l<i>.mix.o` for
attention; `l<i>.mix.{z,x,g,o}` (+ `z.b`, `x.b`) for minGRU; `l<i>.mlp.{gate,up,down}`.
This module turns that into the generic hybrid description (hybrid.py); it has no compute of its own.
"""
from __future__ import annotations

from typing import Dict

import torch

from .hybrid import AttentionSpec, HybridSpec, LayerSpec, MinGruSpec, MlpSpec, slopes_power_of_two
from .ops import AtomaError

ARCHITECTURE = "Lilovik"


def spec_from_config(cfg: dict) -> HybridSpec:
    layers = []
    for i, l in enumerate(cfg["layers"]):
        mlp = None
        if l.get("mlp") is not None:
            kind = l["mlp"].get("kind", "dense")
            if kind != "dense":
                raise AtomaError(f"layer {i}: feed-forward kind {kind!r} is not part of the Lilovik design")
            mlp = MlpSpec(ff=int(l["mlp"]["ff"]), act="relu")
        m = l["mixer"]
        if l["type"] == "attention":
            qt = m.get("q_temp") or {}
            att = AttentionSpec(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
                                temp_coef=float(qt.get("coef", 0.0)), temp_every=int(qt.get("every", 0)),
                                slopes=tuple(slopes_power_of_two(int(m["heads"]))))
            layers.append(LayerSpec("attention", attention=att, mlp=mlp))
        elif l["type"] == "mingru":
            layers.append(LayerSpec("mingru", mingru=MinGruSpec(width=int(m["width"])), mlp=mlp))
        else:
            raise AtomaError(f"layer {i}: mixer type {l['type']!r} is not part of the Lilovik design")
    return HybridSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), eps=float(cfg["norm"]["eps"]),
                      logit_scale=float(cfg["logit_scale"]), layers=tuple(layers), norm_offset=1.0, position_base=10000.0)


def _expect(t: torch.Tensor, name: str, shape) -> torch.Tensor:
    if tuple(t.shape) != tuple(shape):
        raise AtomaError(f"tensor {name} has shape {tuple(t.shape)}, the configuration needs {tuple(shape)}")
    return t


def weights_from_checkpoint(spec: HybridSpec, ckpt: Dict[str, torch.Tensor]) -> dict:
    """Checkpoint names -> the generic hybrid layout (projections of a sublayer stacked for one GEMM)."""
    W = spec.width

    def get(name, shape):
        if name not in ckpt:
            raise AtomaError(f"tensor {name} is missing from the checkpoint")
        return _expect(ckpt[name], name, shape)

    out = {"embed": get("embed", (spec.vocab, W)), "head": get("head", (spec.vocab, W)),
           "final_norm": get("final.norm", (W,)), "layers": []}
    for i, ls in enumerate(spec.layers):
        p = f"l{i}."
        w = {"norm1": get(p + "norm1", (W,)), "norm1b": get(p + "norm1b", (W,))}
        if ls.mixer == "attention":
            a = ls.attention
            nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            w["w_qkv"] = torch.cat([get(p + "mix.q", (nq, W)), get(p + "mix.k", (nk, W)), get(p + "mix.v", (nv, W))], 0)
            w["b_qkv"] = torch.cat([get(p + "mix.q.b", (nq,)), get(p + "mix.k.b", (nk,)), get(p + "mix.v.b", (nv,))], 0).float()
            w["q_norm"], w["k_norm"] = get(p + "mix.q.norm", (nq,)), get(p + "mix.k.norm", (nk,))
            w["talk"], w["head_bias"] = get(p + "mix.talk", (a.heads, a.heads)), get(p + "mix.pb", (a.heads,))
            w["w_o"] = get(p + "mix.o", (W, a.heads * a.vdim))
        else:
            S = ls.mingru.width
            w["w_zxg"] = torch.cat([get(p + "mix.z", (S, W)), get(p + "mix.x", (S, W)), get(p + "mix.g", (S, W))], 0)
            w["b_zxg"] = torch.cat([get(p + "mix.z.b", (S,)).float(), get(p + "mix.x.b", (S,)).float(), torch.zeros(S)], 0)
            w["w_o"] = get(p + "mix.o", (W, S))
        if ls.mlp is not None:
            F = ls.mlp.ff
            w["norm2"], w["norm2b"] = get(p + "norm2", (W,)), get(p + "norm2b", (W,))
            w["w_gate_up"] = torch.cat([get(p + "mlp.gate", (F, W)), get(p + "mlp.up", (F, W))], 0)
            w["w_down"] = get(p + "mlp.down", (W, F))
        out["layers"].append(w)
    return out
