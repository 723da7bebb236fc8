"""Llama behind the serving engine: the executor that runs a scheduled MIXED batch (portions of prompts beside
decoded tokens) through the library's Llama operators.

`Llama::forward` in the reference (models/src/llama.rs:456-478) is one code path for prompts and decoded tokens:
wte gather, per block RMSNorm -> q/k/v -> RoPE -> cache write -> attention (FlashAttention::forward,
models/src/flash_attention.rs:322-469) -> o_proj -> residual -> RMSNorm -> SwiGLU MLP -> residual, then ln_f, the
selected rows, lm_head.  Here the same sequence is composed from the operators of include/atoma_llama.h — fused
qkv + RoPE + cache write (`atoma_qkv_rope_cache`), residual add + RMSNorm, fused gate/up + SwiGLU, the tcgen05 GEMMs —
with ONE attention call per layer for the whole batch: a varlen call through the block tables, so that a portion sees
the keys of its earlier portions in the paged cache (csrc/src/lib.rs:1392-1420, flash_attn_varlen_with_block_table).
Decode-only batches of at most 128 sequences can instead be replayed as one CUDA graph with `llama.DecodeStep`.

Checkpoints use the Hugging Face names (model.embed_tokens.weight, model.layers.N.self_attn.q_proj.weight, ...).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch

from . import ops
from .hybrid import StepOutput
from .llama import Llama3RopeScaling, LlamaConfig, LlamaShard, rope_tables
from .ops import AtomaError
from .scheduler import StepPlan
from .worker import InputStager, SequenceInput


def config_from_hf(cfg: dict) -> LlamaConfig:
    rs = cfg.get("rope_scaling")
    scaling = None
    if rs and rs.get("rope_type", rs.get("type")) == "llama3":
        scaling = Llama3RopeScaling(float(rs["factor"]), float(rs["low_freq_factor"]), float(rs["high_freq_factor"]),
                                    int(rs["original_max_position_embeddings"]))
    return LlamaConfig(hidden_size=int(cfg["hidden_size"]), intermediate_size=int(cfg["intermediate_size"]),
                       vocab_size=int(cfg["vocab_size"]), num_hidden_layers=int(cfg["num_hidden_layers"]),
                       num_attention_heads=int(cfg["num_attention_heads"]),
                       num_key_value_heads=int(cfg.get("num_key_value_heads", cfg["num_attention_heads"])),
                       rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-5)), rope_theta=float(cfg.get("rope_theta", 10000.0)),
                       max_position_embeddings=int(cfg.get("max_position_embeddings", 8192)), rope_scaling=scaling,
                       tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)))


def shard_from_checkpoint(cfg: LlamaConfig, ckpt: Dict[str, torch.Tensor], dtype, device, max_pos: Optional[int] = None) -> LlamaShard:
    """The tp = 1 shard in the layout the kernels stream (llama.py: wqkv = [Wq; Wk; Wv], w_gate_up = [Wgate; Wup])."""
    sh = LlamaShard(cfg, 0, 1, dtype, device)

    def get(name):
        if name not in ckpt:
            raise AtomaError(f"tensor {name} is missing from the checkpoint")
        return ckpt[name].to(dtype)

    dev = sh.device
    sh.embed = get("model.embed_tokens.weight").contiguous().to(dev)
    sh.lm_head = sh.embed if cfg.tie_word_embeddings or "lm_head.weight" not in ckpt else get("lm_head.weight").contiguous().to(dev)
    sh.norm_f = get("model.norm.weight").to(dev)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        sh.layers.append({
            "wqkv": torch.cat([get(p + "self_attn.q_proj.weight"), get(p + "self_attn.k_proj.weight"),
                               get(p + "self_attn.v_proj.weight")], 0).contiguous().to(dev),
            "wo": get(p + "self_attn.o_proj.weight").contiguous().to(dev),
            "w_gate_up": torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], 0).contiguous().to(dev),
            "w_down": get(p + "mlp.down_proj.weight").contiguous().to(dev),
            "rms_attn": get(p + "input_layernorm.weight").to(dev),
            "rms_mlp": get(p + "post_attention_layernorm.weight").to(dev),
        })
    sh.cos, sh.sin = rope_tables(cfg, dtype, dev, max_pos)
    return sh


class LlamaExecutor:
    """`execute(plan) -> StepOutput` for the engine; owns the paged caches ([2, num_blocks, block_size, Hkv, D] per
    layer, the reference's layout, flash_attention.rs:239-246)."""

    def __init__(self, shard: LlamaShard, num_blocks: int, block_size: int = 16):
        if shard.world != 1:
            raise AtomaError("the engine executor runs tensor-parallel degree 1; sharded decode steps use llama.DecodeStep")
        if shard.embed is None or shard.lm_head is None:
            raise AtomaError("the executor needs the embedding and the lm_head")
        self.shard, self.cfg = shard, shard.cfg
        self.device, self.dtype = shard.device, shard.dtype
        self.block_size, self.num_blocks = int(block_size), int(num_blocks)
        c = self.cfg
        self.kv_caches = [torch.zeros((2, num_blocks, block_size, c.num_key_value_heads, c.head_dim), dtype=self.dtype,
                                      device=self.device) for _ in shard.layers]
        self._stager = InputStager(device=self.device, block_size=self.block_size, enable_chunked_prefill=True)
        self._sel_host = None

    @classmethod
    def from_checkpoint(cls, cfg: dict, ckpt, dtype, device, cache) -> "LlamaExecutor":
        if dtype not in (torch.bfloat16, torch.float16):
            raise AtomaError("Llama runs in bfloat16 or float16")
        c = config_from_hf(cfg)
        return cls(shard_from_checkpoint(c, ckpt, dtype, device), cache.num_blocks, cache.block_size)

    def execute(self, plan: StepPlan, **_unused) -> StepOutput:
        chunks = plan.chunks
        if not chunks:
            return StepOutput(None, None)
        c = self.cfg
        H, Hk, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        seqs, selected, rows, t0 = [], [], [], 0
        for ch in chunks:
            end = ch.start + ch.count
            ids = np.zeros(end, dtype=np.uint32)
            ids[ch.start:end] = ch.seq.tokens[ch.start:end]
            seqs.append(SequenceInput(ids, num_computed_tokens=ch.start, token_chunk_size=ch.count,
                                      block_table=np.asarray(ch.block_table, dtype=np.uint32), is_prompt=True))
            for w in ch.want:
                selected.append(t0 + w)
                rows.append((ch.seq.seq_id, w))
            t0 += ch.count
        lay, v = self._stager.prepare_raw(seqs)
        T = t0
        max_q, max_k = max(ch.count for ch in chunks), max(ch.start + ch.count for ch in chunks)
        sh = self.shard
        x = ops.embedding(v["tokens"], sh.embed)
        residual = None
        for ly, kv in zip(sh.layers, self.kv_caches):
            residual, h = ops.add_rmsnorm(x, residual, ly["rms_attn"], c.rms_norm_eps)
            qkv = ops.qkv_rope_cache(h, ly["wqkv"], H, Hk, D, v["positions"], sh.cos, sh.sin, kv[0], kv[1], v["slot_mapping"])
            q = qkv[:, :H * D].view(T, H, D)
            att = ops.flash_attn_varlen_with_block_table(q, kv[0], kv[1], None, v["query_start"], v["sequence_start"], max_q, max_k,
                                                         1.0 / math.sqrt(D), None, 0, v["block_tables"])
            o = ops.gemm_tn(att.reshape(T, H * D), ly["wo"])
            residual, h = ops.add_rmsnorm(o, residual, ly["rms_mlp"], c.rms_norm_eps)
            x = ops.gemm_tn(ops.gate_up_silu(h, ly["w_gate_up"]), ly["w_down"])
        _, hn = ops.add_rmsnorm(x, residual, sh.norm_f, c.rms_norm_eps)
        if not selected:
            return StepOutput(None, None, rows)
        sel = torch.tensor(selected, dtype=torch.long, device=self.device)
        logits = ops.gemm_tn(hn.index_select(0, sel).contiguous(), sh.lm_head)
        tok, _, f32 = ops.sample_greedy(logits, want_f32=True)
        return StepOutput(f32, tok, rows)
