"""Patadra's configuration and checkpoint reading (host only): layer runs of a looped span, optional parts, the
stacked weight layout, errors for what the design does not have."""
import pytest
import torch

import patadra_oracle as po
from atoma_infer_b200 import models, patadra
from atoma_infer_b200.ops import AtomaError


def test_layer_runs_repeat_the_looped_span_in_place():
    cfg = po.random_config(layers=5, loop=(1, 3, 3))
    assert patadra.layer_runs(cfg) == [0, 1, 2, 1, 2, 1, 2, 3, 4] == po.run_order(cfg)
    assert patadra.layer_runs(po.random_config(layers=3, loop=None)) == [0, 1, 2]
    assert patadra.layer_runs(po.random_config(layers=3, loop=(0, 3, 2))) == [0, 1, 2, 0, 1, 2]
    assert patadra.layer_runs(po.random_config(layers=3, loop=(2, 2, 4))) == [0, 1, 2]
    with pytest.raises(AtomaError):
        patadra.layer_runs(po.random_config(layers=3, loop=(2, 5, 2)))


def test_spec_reads_every_size_and_constant_from_the_configuration():
    cfg = po.random_config(width=50, heads=5, dim=6, vdim=10, q_rank=14, kv_rank=22, window=33, experts=7, top=3, ff=11, shared_ff=13,
                           groups=5, layers=4, loop=(1, 3, 2), side=3, softcap=7.5, no_mlp_layers=(2,), limit=1.25, shared_limit=3.0)
    spec = patadra.spec_from_config(cfg)
    assert [l.source for l in spec.layers] == [0, 1, 2, 1, 2, 3]
    assert spec.block_style == "prenorm" and spec.norm_groups == 5 and spec.norm_offset == 0.0 and spec.position == "learned"
    assert spec.logit_softcap == 7.5 and spec.side_dim == 3 and spec.max_positions == cfg["max_positions"]
    a, e = spec.layers[0].latent, spec.layers[0].moe
    assert (a.heads, a.dim, a.vdim, a.q_rank, a.kv_rank, a.window, a.sink) == (5, 6, 10, 14, 22, 33, True)
    assert (e.experts, e.top, e.ff, e.limit, e.shared_ff, e.shared_limit, e.shared_gate, e.renormalize) == (7, 3, 11, 1.25, 13, 3.0, True, False)
    assert spec.layers[2].moe is None and spec.layers[4].moe is None and spec.layers[2].side_part == 2
    assert spec.cache_bytes_per_token(torch.bfloat16) == 6 * 22 * 2
    plain = patadra.spec_from_config(po.random_config(loop=None, side=0, softcap=0.0, groups=1, shared_ff=0))
    assert plain.side_dim == 0 and plain.logit_softcap == 0.0 and plain.layers[0].side_part is None and plain.layers[0].moe.shared_ff == 0
    assert models.resolve(cfg).name == "Patadra" and not models.resolve(cfg).needs_state(cfg)


def test_weights_are_stacked_per_configured_layer():
    cfg = po.random_config(layers=3, loop=(1, 2, 3))
    w = po.random_weights(cfg, torch.Generator().manual_seed(0))
    spec = patadra.spec_from_config(cfg)
    out = patadra.weights_from_checkpoint(spec, cfg, w)
    assert len(out["layers"]) == 3 and len(spec.layers) == 5
    W, m, f = cfg["width"], cfg["layers"][0]["mixer"], cfg["layers"][0]["mlp"]
    l0 = out["layers"][0]
    assert l0["w_down_in"].shape == (m["q_rank"] + m["kv_rank"] + W, W)
    assert torch.equal(l0["w_down_in"][m["q_rank"]:m["q_rank"] + m["kv_rank"]], w["l0.mix.dkv"])
    assert l0["w_expert_gate_up"].shape == (f["router"]["experts"], 2 * f["expert"]["ff"], W)
    assert torch.equal(l0["w_expert_gate_up"][2, f["expert"]["ff"]:], w["l0.mlp.e2.up"])
    assert l0["w_ff_in"].shape == (2 * f["shared"]["ff"] + W, W) and torch.equal(l0["w_ff_in"][-W:], w["l0.rg2"])
    assert out["side_table"].shape == (cfg["vocab"], 3 * cfg["token_side"]["dim"])
    del w["l1.mix.sink"]
    with pytest.raises(AtomaError, match="l1.mix.sink"):
        patadra.weights_from_checkpoint(spec, cfg, w)


def test_what_the_design_does_not_have_is_refused():
    cfg = po.random_config()
    cfg["layers"][1]["type"] = "attention"
    with pytest.raises(AtomaError):
        patadra.spec_from_config(cfg)
    cfg = po.random_config()
    cfg["layers"][0]["mlp"]["kind"] = "dense"
    with pytest.raises(AtomaError):
        patadra.spec_from_config(cfg)
