/*
 * atoma_hybrid.h — operators and the step executor for models whose layers mix attention with
 * recurrent (state-carrying) mixers, run on MIXED batches: portions of prompts beside single decoded
 * tokens, keys and values in a paged cache, recurrent state in per-sequence slots.
 *
 * The first design served through it is Lilovik: sandwich RMS norms (weights stored as offsets from
 * one), a sinusoidal position signal on the embedding, sigmoid attention (no softmax) with a
 * whole-projection q/k norm, a position-dependent query temperature, a tanh soft cap, a linear
 * distance bias and a talking-heads mix of the attention weights, minGRU layers, and a ReLU-gated
 * feed-forward.  Every constant of those mechanisms is an argument, so that another design can use
 * the operator with other values.
 *
 * Conventions: row-major; `dtype` is the number format of activations, large weights and the caches:
 * 1 = bfloat16, 2 = float32 (true 32-bit arithmetic: no reduced-precision matrix mode).  Whatever the
 * dtype, the residual stream, norm statistics, attention scores and weights, recurrent state and all
 * small per-channel parameters (norm weights, biases, per-head tables) are float32.  Everything is
 * stream-ordered and allocates nothing (library workspaces excepted).  Errors: atoma_last_status()
 * / atoma_last_error() (atoma_flash.h).
 */
#ifndef ATOMA_HYBRID_H_
#define ATOMA_HYBRID_H_

#include <stdint.h>

#include "atoma_flash.h"

#ifdef __cplusplus
extern "C" {
#endif

#define ATOMA_DTYPE_BF16 1u
#define ATOMA_DTYPE_F32 2u

/* out[t, 2i] = table[tokens[t], 2i] + sin(positions[t] * inv_freq[i]), out[t, 2i+1] = ... + cos(same); the angle is
 * formed and reduced in double precision (inv_freq [ceil(width/2)] is a device table of doubles). */
void atoma_embed_sinusoid(const uint32_t *tokens, const int64_t *positions, const void *table, const double *inv_freq,
                          float *out, int64_t T, int64_t width, int64_t vocab, uint32_t dtype, atoma_stream_t stream);

/* out[r, :] = x[rows ? rows[r] : r, :] / sqrt(mean(x^2) + eps) * (weight_offset + weight); x float32, out `dtype`. */
void atoma_rmsnorm_rows(const float *x, const int32_t *rows, const float *weight, float weight_offset, void *out,
                        int64_t R, int64_t width, float eps, uint32_t dtype, atoma_stream_t stream);

/* Sandwich-norm residual update and the next sublayer's input norm in ONE kernel:
 *   x[t, :] += rms(y[t, :]) * (weight_offset + w_post);   h[t, :] = rms(x[t, :]) * (weight_offset + w_pre)
 * y, h in `dtype`, x float32 in place; w_pre / h may be NULL (no following norm). */
void atoma_postnorm_add_prenorm(const void *y, float *x, const float *w_post, const float *w_pre, void *h, int64_t T,
                                int64_t width, float eps, float weight_offset, uint32_t dtype, atoma_stream_t stream);

/* After the fused q/k/v projection qkv [T, H dim + G dim + G vdim] (+ bias, float32, may be NULL):
 *   q <- rms over the WHOLE q part * q_weight * (1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)) -> q_out [T, H dim]
 *   k <- rms over the WHOLE k part * k_weight -> key cache row slot_mapping[t];   v -> value cache row
 * caches: [num_blocks * block_size, G, dim] and [.., G, vdim] in `dtype`; slot < 0 is skipped. */
void atoma_qk_norm_cache(const void *qkv, const float *bias, const float *q_weight, const float *k_weight,
                         const int64_t *positions, const int64_t *slot_mapping, void *q_out, void *k_cache, void *v_cache,
                         int64_t T, int64_t H, int64_t G, int64_t dim, int64_t vdim, float eps, float temp_coef,
                         int64_t temp_every, uint32_t dtype, atoma_stream_t stream);

/*
 * Sigmoid attention over a paged cache for a mixed batch.  For query token t of sequence b at position p and every
 * cached key j <= p of that sequence:
 *   s = (q_g . k_j) * scale;  s = softcap * tanh(s / softcap) (softcap > 0);  s -= slopes[g] * (p - j)
 *   a_g = sigmoid(s + head_bias[g]);   a'_h = sum_g talk[h, g] a_g  (talk NULL = identity)
 *   out[t, h, :] = sum_j a'_h(j) v_j[kv head of h, :]
 * Scores, weights and the sums are float32; keys are visited in position order whatever the batch looks like.
 */
typedef struct atoma_sigmoid_attn_args {
    const void *q;                /* [T, H dim] */
    const void *k_cache, *v_cache;
    void *out;                    /* [T, H vdim] */
    const int64_t *positions;     /* [T] */
    const int32_t *token_seq;     /* [T] batch row of every token */
    const int32_t *query_start;   /* [B + 1] first token of every batch row (rows are contiguous, positions ascending) */
    const int32_t *block_tables;  /* [B, max_blocks] */
    const float *slopes, *head_bias, *talk; /* [H], [H], [H, H] */
    int64_t T, B, max_blocks, H, G, dim, vdim, block_size;
    float scale, softcap;
    uint32_t dtype;
    int32_t max_query_len;        /* longest portion of the batch (1 = decode only): selects the kernel */
    int32_t max_seq_len;          /* longest sequence (context + portion) of the batch; 0 = unknown (keys are not split) */
} atoma_sigmoid_attn_args;
void atoma_sigmoid_attention_paged(const atoma_sigmoid_attn_args *args, atoma_stream_t stream);

/*
 * minGRU over a mixed batch.  zxg [T, 3 S] = the fused projections (rows: update gate, candidate, output gate) with
 * bias [3 S] (may be NULL) added here.  Per sequence b (tokens query_start[b] .. query_start[b+1]) and channel c:
 *   z = sigmoid(zpre), cand = u >= 0 ? u + 1/2 : sigmoid(u),  s <- (1 - z) s + z cand,  out = s * silu(g)
 * s starts from state[state_slots[b], c] — from zero when context_lens[b] == 0 — and is stored back.  float32 state.
 */
void atoma_mingru_scan(const void *zxg, const float *bias, float *state, const int32_t *state_slots,
                       const int32_t *query_start, const int32_t *context_lens, void *out, int64_t T, int64_t B, int64_t S,
                       int32_t max_query_len, uint32_t dtype, atoma_stream_t stream);

/* out[t, j] = act(gu[t, j]) * gu[t, ff + j]; act: 0 = silu, 1 = relu, 2 = gelu (tanh form). */
void atoma_glu(const void *gu, void *out, int64_t T, int64_t ff, int32_t act, uint32_t dtype, atoma_stream_t stream);

/* y[T, N] = x[T, K] w[N, K]^T.  bfloat16 with 16-byte aligned rows runs the tcgen05 kernels of atoma_gemm_tn;
 * float32 (and whatever those kernels do not take) runs a plain float32-FMA tile kernel. */
void atoma_linear(const void *x, const void *w, void *y, int64_t T, int64_t N, int64_t K, uint32_t dtype,
                  atoma_stream_t stream);

/* logits_f32[r, :] = logits[r, :] * scale and token_out[r] = the last index of the row's maximum. */
void atoma_scale_logits_greedy(const void *logits, float *logits_f32, uint32_t *token_out, int64_t R, int64_t vocab,
                               float scale, uint32_t dtype, atoma_stream_t stream);

/* ------------------------------------------------------------------------------------------ */
/* Step executor                                                                                */
/* ------------------------------------------------------------------------------------------ */
enum { ATOMA_MIXER_SIGMOID_ATTENTION = 0, ATOMA_MIXER_MINGRU = 1 };
enum { ATOMA_ACT_SILU = 0, ATOMA_ACT_RELU = 1, ATOMA_ACT_GELU_TANH = 2 };

typedef struct atoma_hybrid_layer {
    int32_t mixer, has_mlp;
    const float *norm1, *norm1b, *norm2, *norm2b; /* [width] offsets from one */
    /* attention */
    int64_t heads, kv_heads, dim, vdim, temp_every;
    float scale, softcap, temp_coef;
    const void *w_qkv;      /* [H dim + G dim + G vdim, width] */
    const float *b_qkv;
    const float *q_norm, *k_norm, *talk, *head_bias, *slopes;
    void *k_cache, *v_cache;
    /* minGRU */
    int64_t state_width;
    const void *w_zxg;      /* [3 S, width] */
    const float *b_zxg;
    float *state;           /* [slots, S] */
    /* both mixers */
    const void *w_o;        /* [width, H vdim] or [width, S] */
    /* feed-forward */
    int64_t ff;
    int32_t act;
    const void *w_gate_up;  /* [2 ff, width] */
    const void *w_down;     /* [width, ff] */
} atoma_hybrid_layer;

typedef struct atoma_hybrid_model {
    int64_t width, vocab, num_layers, block_size;
    float eps, logit_scale, norm_offset;
    uint32_t dtype;
    const void *embed;      /* [vocab, width] */
    const double *inv_freq; /* [ceil(width / 2)] */
    const float *final_norm;
    const void *head;       /* [vocab, width] */
    const atoma_hybrid_layer *layers; /* host array */
} atoma_hybrid_model;

typedef struct atoma_hybrid_batch {
    int64_t num_tokens, num_seqs, num_selected, max_blocks;
    int32_t max_query_len, max_seq_len;
    const uint32_t *tokens;       /* [T] */
    const int64_t *positions;     /* [T] */
    const int64_t *slot_mapping;  /* [T] */
    const int32_t *token_seq;     /* [T] */
    const int32_t *query_start;   /* [B + 1] */
    const int32_t *context_lens;  /* [B] tokens already in the cache / state */
    const int32_t *block_tables;  /* [B, max_blocks] */
    const int32_t *state_slots;   /* [B] */
    const int32_t *selected;      /* [num_selected] token rows whose logits are wanted */
    void *scratch;
    int64_t scratch_bytes;
    float *logits;                /* out [num_selected, vocab] */
    uint32_t *next_tokens;        /* out [num_selected] greedy */
    float *residual_trace;        /* optional out [num_layers, T, width]: the residual stream after every layer */
} atoma_hybrid_batch;

int64_t atoma_hybrid_abi_sizeof(int which); /* 0 layer, 1 model, 2 batch, 3 attention args */
int64_t atoma_hybrid_scratch_bytes(const atoma_hybrid_model *model, int64_t num_tokens, int64_t num_selected);
void atoma_hybrid_step(const atoma_hybrid_model *model, const atoma_hybrid_batch *batch, atoma_stream_t stream);

/* Diagnostics: bit 0 = every projection through the plain float32-FMA kernel; bit 1 = the general attention kernel
 * for every batch (no tensor-core prefill / split decode kernels); bit 2 = the sequential minGRU scan. */
void atoma_debug_hybrid(int flags);

#ifdef __cplusplus
}
#endif
#endif /* ATOMA_HYBRID_H_ */
