"""Python face of the hybrid-model operators (include/atoma_hybrid.h): thin ctypes shims over torch tensors,
one function per operator, used by tests and by callers that compose the operators themselves.
`dtype` follows the activations: torch.bfloat16 or torch.float32.  No fallback path."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import SigmoidAttnArgs
from .ops import AtomaError

_CODES = {torch.bfloat16: 1, torch.float32: 2}


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _s():
    return torch.cuda.current_stream().cuda_stream


def _check():
    L = _lib.lib()
    if L.atoma_last_status() != 0:
        raise AtomaError(L.atoma_last_error().decode())


def debug_flags(flags: int) -> None:
    """bit 0: plain float32 GEMM everywhere; bit 1: general attention kernel only; bit 2: sequential minGRU scan."""
    _lib.lib().atoma_debug_hybrid(int(flags))


def embed_sinusoid(tokens, positions, table, inv_freq):
    T, W = tokens.numel(), table.shape[1]
    out = torch.empty((T, W), dtype=torch.float32, device=table.device)
    _lib.lib().atoma_embed_sinusoid(_p(tokens), _p(positions), _p(table), _p(inv_freq), _p(out), T, W, table.shape[0],
                                    _CODES[table.dtype], _s())
    _check()
    return out


def rmsnorm_rows(x, weight, offset, eps, dtype, rows=None):
    R = x.shape[0] if rows is None else rows.numel()
    out = torch.empty((R, x.shape[1]), dtype=dtype, device=x.device)
    _lib.lib().atoma_rmsnorm_rows(_p(x), _p(rows), _p(weight), offset, _p(out), R, x.shape[1], eps, _CODES[dtype], _s())
    _check()
    return out


def postnorm_add_prenorm(y, x, w_post, w_pre, eps, offset):
    """x is updated in place; returns the next sublayer's normed input (None without w_pre)."""
    h = torch.empty_like(y) if w_pre is not None else None
    _lib.lib().atoma_postnorm_add_prenorm(_p(y), _p(x), _p(w_post), _p(w_pre), _p(h), y.shape[0], y.shape[1], eps, offset,
                                          _CODES[y.dtype], _s())
    _check()
    return h


def qk_norm_cache(qkv, bias, q_w, k_w, positions, slots, k_cache, v_cache, H, G, dim, vdim, eps, temp_coef, temp_every):
    T = qkv.shape[0]
    q = torch.empty((T, H * dim), dtype=qkv.dtype, device=qkv.device)
    _lib.lib().atoma_qk_norm_cache(_p(qkv), _p(bias), _p(q_w), _p(k_w), _p(positions), _p(slots), _p(q), _p(k_cache), _p(v_cache),
                                   T, H, G, dim, vdim, eps, temp_coef, temp_every, _CODES[qkv.dtype], _s())
    _check()
    return q


def sigmoid_attention_paged(q, k_cache, v_cache, positions, token_seq, block_tables, slopes, head_bias, talk, H, G, dim, vdim,
                            block_size, scale, softcap, max_query_len, query_start=None, max_seq_len=None):
    T = q.shape[0]
    if query_start is None:
        counts = torch.bincount(token_seq.long(), minlength=block_tables.shape[0])
        query_start = torch.cat([counts.new_zeros(1), counts.cumsum(0)]).to(torch.int32)
    if max_seq_len is None:
        max_seq_len = int(positions.max()) + 1
    out = torch.empty((T, H * vdim), dtype=q.dtype, device=q.device)
    a = SigmoidAttnArgs()
    a.q, a.k_cache, a.v_cache, a.out = _p(q), _p(k_cache), _p(v_cache), _p(out)
    a.positions, a.token_seq, a.block_tables = _p(positions), _p(token_seq), _p(block_tables)
    a.query_start, a.max_seq_len = _p(query_start), int(max_seq_len)
    a.slopes, a.head_bias, a.talk = _p(slopes), _p(head_bias), _p(talk)
    a.T, a.B, a.max_blocks = T, block_tables.shape[0], block_tables.shape[1]
    a.H, a.G, a.dim, a.vdim, a.block_size = H, G, dim, vdim, block_size
    a.scale, a.softcap, a.dtype, a.max_query_len = scale, softcap, _CODES[q.dtype], max_query_len
    _lib.lib().atoma_sigmoid_attention_paged(C.byref(a), _s())
    _check()
    return out


def mingru_scan(zxg, bias, state, state_slots, query_start, context_lens, max_query_len):
    T, S = zxg.shape[0], zxg.shape[1] // 3
    out = torch.empty((T, S), dtype=zxg.dtype, device=zxg.device)
    _lib.lib().atoma_mingru_scan(_p(zxg), _p(bias), _p(state), _p(state_slots), _p(query_start), _p(context_lens), _p(out), T,
                                 state_slots.numel(), S, max_query_len, _CODES[zxg.dtype], _s())
    _check()
    return out


def glu(gu, act: int):
    T, ff = gu.shape[0], gu.shape[1] // 2
    out = torch.empty((T, ff), dtype=gu.dtype, device=gu.device)
    _lib.lib().atoma_glu(_p(gu), _p(out), T, ff, act, _CODES[gu.dtype], _s())
    _check()
    return out


def linear(x, w):
    y = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
    _lib.lib().atoma_linear(_p(x), _p(w), _p(y), x.shape[0], w.shape[0], x.shape[1], _CODES[x.dtype], _s())
    _check()
    return y


def scale_logits_greedy(logits, scale):
    R, V = logits.shape
    out = torch.empty((R, V), dtype=torch.float32, device=logits.device)
    tok = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _lib.lib().atoma_scale_logits_greedy(_p(logits), _p(out), _p(tok), R, V, scale, _CODES[logits.dtype], _s())
    _check()
    return out, tok


def gate_up_act(x, w_gate_up, act: int):
    """act(x Wg^T) * (x Wu^T) with the activation in the projection's epilogue (bfloat16, T <= 128, K % 64 == 0)."""
    T, ff = x.shape[0], w_gate_up.shape[0] // 2
    out = torch.empty((T, ff), dtype=x.dtype, device=x.device)
    _lib.lib().atoma_gate_up_act(_p(x), _p(w_gate_up), _p(out), T, ff, x.shape[1], x.shape[1], x.shape[1], ff, act, 1, _s())
    _check()
    return out
