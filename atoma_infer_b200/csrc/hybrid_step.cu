// Step executor for hybrid (attention + recurrent) models on a mixed batch — include/atoma_hybrid.h.
//
// One call enqueues the whole forward pass of the step's tokens on one stream, without host
// synchronisation: embedding + position signal, then per layer
//   attention: fused q/k/v projection -> q/k norm + temperature + cache write -> paged sigmoid attention -> o
//   minGRU:    fused z/x/g projection -> scan over each sequence's tokens from its state slot -> o
//   x += norm(mixer out) fused with the next sublayer's input norm; the gated feed-forward likewise;
// and at the end the wanted rows only: final norm, head, logit scale and the greedy choice.
// Keys, values and recurrent state left by earlier steps are read from / written to the paged caches and
// the state slots the batch names; nothing else survives the call.
#include "common.cuh"

#include "atoma_hybrid.h"

#include <algorithm>
#include <nvtx3/nvToolsExt.h>

namespace atoma {

bool hyb_embed_sinusoid(const uint32_t *, const int64_t *, const void *, const double *, float *, int64_t, int64_t, int64_t, uint32_t,
                        cudaStream_t);
bool hyb_rmsnorm_rows(const float *, const int32_t *, const float *, float, void *, int64_t, int64_t, float, uint32_t, cudaStream_t);
bool hyb_postnorm_add_prenorm(const void *, float *, const float *, const float *, void *, int64_t, int64_t, float, float, uint32_t,
                              cudaStream_t);
bool hyb_qk_norm_cache(const void *, const float *, const float *, const float *, const int64_t *, const int64_t *, void *, void *,
                       void *, int64_t, int64_t, int64_t, int64_t, int64_t, float, float, int64_t, uint32_t, cudaStream_t);
bool hyb_attention(const atoma_sigmoid_attn_args &, cudaStream_t);
bool hyb_mingru_scan(const void *, const float *, float *, const int32_t *, const int32_t *, const int32_t *, void *, int64_t, int64_t,
                     int64_t, int32_t, uint32_t, cudaStream_t);
bool hyb_glu(const void *, void *, int64_t, int64_t, int32_t, uint32_t, cudaStream_t);
bool hyb_gate_up_act(const void *, const void *, void *, void *, int64_t, int64_t, int64_t, int32_t, uint32_t, cudaStream_t);
bool hyb_linear(const void *, const void *, void *, int64_t, int64_t, int64_t, uint32_t, cudaStream_t);
bool hyb_scale_greedy(const void *, float *, uint32_t *, int64_t, int64_t, float, uint32_t, cudaStream_t);

namespace {

inline int64_t up256(int64_t x) { return (x + 255) / 256 * 256; }

struct Widths {
    int64_t proj = 0, q = 0, act = 0;   // widest projection output, query row, mixer / feed-forward activation row
};

Widths widths(const atoma_hybrid_model &m) {
    Widths w;
    for (int64_t i = 0; i < m.num_layers; ++i) {
        const atoma_hybrid_layer &l = m.layers[i];
        if (l.mixer == ATOMA_MIXER_SIGMOID_ATTENTION) {
            w.proj = std::max(w.proj, (l.heads + l.kv_heads) * l.dim + l.kv_heads * l.vdim);
            w.q = std::max(w.q, l.heads * l.dim);
            w.act = std::max(w.act, l.heads * l.vdim);
        } else {
            w.proj = std::max(w.proj, 3 * l.state_width);
            w.act = std::max(w.act, l.state_width);
        }
        if (l.has_mlp) {
            w.proj = std::max(w.proj, 2 * l.ff);
            w.act = std::max(w.act, l.ff);
        }
    }
    return w;
}

struct Scratch {
    float *x;
    char *h, *proj, *q, *act, *y, *hs, *lg;
    int64_t total;
};

Scratch carve(const atoma_hybrid_model &m, int64_t T, int64_t S, void *base) {
    const int64_t es = m.dtype == ATOMA_DTYPE_F32 ? 4 : 2;
    const Widths w = widths(m);
    Scratch s{};
    int64_t off = 0;
    char *b = static_cast<char *>(base);
    auto take = [&](int64_t bytes) {
        char *p = b ? b + off : nullptr;
        off += up256(bytes);
        return p;
    };
    s.x = reinterpret_cast<float *>(take(T * m.width * 4));
    s.h = take(T * m.width * es);
    s.proj = take(T * w.proj * es);
    s.q = take(T * w.q * es);
    s.act = take(T * w.act * es);
    s.y = take(T * m.width * es);
    s.hs = take(S * m.width * es);
    s.lg = take(S * m.vocab * es);
    s.total = off;
    return s;
}

}  // namespace
}  // namespace atoma

using namespace atoma;

extern "C" int64_t atoma_hybrid_abi_sizeof(int which) {
    switch (which) {
        case 0: return sizeof(atoma_hybrid_layer);
        case 1: return sizeof(atoma_hybrid_model);
        case 2: return sizeof(atoma_hybrid_batch);
        case 3: return sizeof(atoma_sigmoid_attn_args);
        default: return -1;
    }
}

extern "C" int64_t atoma_hybrid_scratch_bytes(const atoma_hybrid_model *model, int64_t num_tokens, int64_t num_selected) {
    if (!model || !model->layers || num_tokens < 0 || num_selected < 0) return -1;
    return carve(*model, num_tokens, num_selected, nullptr).total;
}

extern "C" void atoma_hybrid_step(const atoma_hybrid_model *model, const atoma_hybrid_batch *batch, atoma_stream_t stream_) {
    clear_status();
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!model || !batch || !model->layers) {
        set_status(kErrInvalidArg, "atoma_hybrid_step: model / batch is NULL");
        return;
    }
    const atoma_hybrid_model &m = *model;
    const atoma_hybrid_batch &b = *batch;
    const int64_t T = b.num_tokens, B = b.num_seqs, S = b.num_selected;
    if (T <= 0 || B <= 0) return;
    if (!b.tokens || !b.positions || !b.slot_mapping || !b.token_seq || !b.query_start || !b.context_lens || !b.block_tables ||
        !b.state_slots || !b.scratch || (S > 0 && (!b.selected || !b.logits)) || !m.embed || !m.inv_freq || !m.final_norm ||
        !m.head || m.width <= 0 || m.vocab <= 0 || m.num_layers <= 0) {
        set_status(kErrInvalidArg, "atoma_hybrid_step: a required tensor is NULL");
        return;
    }
    const Scratch s = carve(m, T, S, b.scratch);
    if (s.total > b.scratch_bytes) {
        set_status(kErrInvalidArg, "atoma_hybrid_step: scratch of %lld bytes, %lld needed", static_cast<long long>(b.scratch_bytes),
                   static_cast<long long>(s.total));
        return;
    }
    nvtxRangePushA("atoma_hybrid_step");
    struct Pop {
        ~Pop() { nvtxRangePop(); }
    } pop;
    const uint32_t dt = m.dtype;
    const int64_t W = m.width;
    const float off = m.norm_offset;
    if (!hyb_embed_sinusoid(b.tokens, b.positions, m.embed, m.inv_freq, s.x, T, W, m.vocab, dt, stream)) return;
    if (!hyb_rmsnorm_rows(s.x, nullptr, m.layers[0].norm1, off, s.h, T, W, m.eps, dt, stream)) return;
    for (int64_t i = 0; i < m.num_layers; ++i) {
        const atoma_hybrid_layer &l = m.layers[i];
        const float *next_norm = i + 1 < m.num_layers ? m.layers[i + 1].norm1 : nullptr;
        if (l.mixer == ATOMA_MIXER_SIGMOID_ATTENTION) {
            const int64_t nqkv = (l.heads + l.kv_heads) * l.dim + l.kv_heads * l.vdim;
            if (!hyb_linear(s.h, l.w_qkv, s.proj, T, nqkv, W, dt, stream)) return;
            if (!hyb_qk_norm_cache(s.proj, l.b_qkv, l.q_norm, l.k_norm, b.positions, b.slot_mapping, s.q, l.k_cache, l.v_cache, T,
                                   l.heads, l.kv_heads, l.dim, l.vdim, m.eps, l.temp_coef, l.temp_every, dt, stream))
                return;
            atoma_sigmoid_attn_args a{};
            a.q = s.q;
            a.k_cache = l.k_cache;
            a.v_cache = l.v_cache;
            a.out = s.act;
            a.positions = b.positions;
            a.token_seq = b.token_seq;
            a.query_start = b.query_start;
            a.max_seq_len = b.max_seq_len;
            a.block_tables = b.block_tables;
            a.slopes = l.slopes;
            a.head_bias = l.head_bias;
            a.talk = l.talk;
            a.T = T;
            a.B = B;
            a.max_blocks = b.max_blocks;
            a.H = l.heads;
            a.G = l.kv_heads;
            a.dim = l.dim;
            a.vdim = l.vdim;
            a.block_size = m.block_size;
            a.scale = l.scale;
            a.softcap = l.softcap;
            a.dtype = dt;
            a.max_query_len = b.max_query_len;
            if (!hyb_attention(a, stream)) return;
            if (!hyb_linear(s.act, l.w_o, s.y, T, W, l.heads * l.vdim, dt, stream)) return;
        } else if (l.mixer == ATOMA_MIXER_MINGRU) {
            const int64_t Sw = l.state_width;
            if (!hyb_linear(s.h, l.w_zxg, s.proj, T, 3 * Sw, W, dt, stream)) return;
            if (!hyb_mingru_scan(s.proj, l.b_zxg, l.state, b.state_slots, b.query_start, b.context_lens, s.act, T, B, Sw,
                                 b.max_query_len, dt, stream))
                return;
            if (!hyb_linear(s.act, l.w_o, s.y, T, W, Sw, dt, stream)) return;
        } else {
            set_status(kErrInvalidArg, "atoma_hybrid_step: layer %lld has unknown mixer %d", static_cast<long long>(i), l.mixer);
            return;
        }
        if (!hyb_postnorm_add_prenorm(s.y, s.x, l.norm1b, l.has_mlp ? l.norm2 : next_norm, s.h, T, W, m.eps, off, dt, stream)) return;
        if (l.has_mlp) {
            if (!hyb_gate_up_act(s.h, l.w_gate_up, s.proj, s.act, T, l.ff, W, l.act, dt, stream)) return;
            if (!hyb_linear(s.act, l.w_down, s.y, T, W, l.ff, dt, stream)) return;
            if (!hyb_postnorm_add_prenorm(s.y, s.x, l.norm2b, next_norm, s.h, T, W, m.eps, off, dt, stream)) return;
        }
        if (b.residual_trace) {
            cudaMemcpyAsync(b.residual_trace + i * T * W, s.x, static_cast<size_t>(T) * W * 4, cudaMemcpyDeviceToDevice, stream);
        }
    }
    if (S > 0) {
        if (!hyb_rmsnorm_rows(s.x, b.selected, m.final_norm, off, s.hs, S, W, m.eps, dt, stream)) return;
        if (!hyb_linear(s.hs, m.head, s.lg, S, m.vocab, W, dt, stream)) return;
        if (!hyb_scale_greedy(s.lg, b.logits, b.next_tokens, S, m.vocab, m.logit_scale, dt, stream)) return;
    }
}
