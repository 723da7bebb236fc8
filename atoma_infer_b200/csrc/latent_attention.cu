// Latent attention over a paged cache of ONE shared latent per token — include/atoma_hybrid.h.
//
// Keys and values of every head are linear images of a cached latent c_j: k_h = Wk_h c_j, v_h = Wv_h c_j.  Nothing
// is expanded per key here: the query is moved into the latent space once (q_lat_h = Wk_h^T q_h, atoma_head_project),
// scores are q_lat_h . c_j, the weighted sum of latents is taken per head, and a head's values come from that sum
// (Wv_h sum_j w_j c_j, atoma_head_project again).  The cache is read once per token for all heads.
//
// Softmax with a sink: the running maximum starts at the sink and the running denominator at one (exp(sink - sink)),
// so the sink is one more term of the denominator that has no key and no value.  Sliding window: keys
// [max(0, p - window + 1), p].  Scores, weights and sums are float32; keys are visited in position order in
// tiles that start at the window's first key, so a query's result does not depend on the batch around it.
#include "common.cuh"
#include "hybrid_common.cuh"

#include "atoma_hybrid.h"

#include <algorithm>

namespace atoma {

extern int g_hybrid_debug;

namespace {

using namespace hybrid;

// ---------------------------------------------------------------------------------------------
// RMS norms of the two latents + cache write
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kRowThreads) latent_norm_cache_kernel(const T *__restrict__ proj, int64_t ld,
                                                                        const float *__restrict__ q_w, const float *__restrict__ kv_w,
                                                                        const int64_t *__restrict__ slots, T *__restrict__ cq_out,
                                                                        T *__restrict__ cache, int q_rank, int kv_rank, float eps) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const T *r = proj + t * ld;
    if (q_rank > 0) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
            const float v = to_f(r[c]);
            ss = fmaf(v, v, ss);
        }
        const float inv = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(q_rank) + eps);
        for (int c = threadIdx.x; c < q_rank; c += blockDim.x) cq_out[t * q_rank + c] = from_f<T>(to_f(r[c]) * inv * q_w[c]);
    }
    const int64_t slot = slots ? slots[t] : -1;
    if (slot < 0) return;
    float ss = 0.f;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
        const float v = to_f(r[q_rank + c]);
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(kv_rank) + eps);
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) cache[slot * kv_rank + c] = from_f<T>(to_f(r[q_rank + c]) * inv * kv_w[c]);
}

// ---------------------------------------------------------------------------------------------
// Per-head projection: out[t, h, n] = sum_k in[t, h, k] w(h, k, n); float32 FMA tiles, k ascending.
// ---------------------------------------------------------------------------------------------
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256) head_project_kernel(const TA *__restrict__ in, int64_t ld_in, int64_t in_hs,
                                                           const TW *__restrict__ w, int64_t w_hs, int64_t w_ks, int64_t w_ns,
                                                           TO *__restrict__ out, int64_t ld_out, int64_t out_hs, int M, int N, int K) {
    __shared__ float xs[16][65], ws[16][65];
    pdl_launch_dependents();
    pdl_wait();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int64_t h = blockIdx.z;
    in += h * in_hs;
    w += h * w_hs;
    out += h * out_hs;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i / 16, k = i % 16;
            xs[k][r] = (m0 + r < M && k0 + k < K) ? to_f(in[static_cast<int64_t>(m0 + r) * ld_in + k0 + k]) : 0.f;
        }
        if (w_ns == 1) {   // n contiguous: read along n
            for (int i = threadIdx.x; i < 64 * 16; i += 256) {
                const int k = i / 64, r = i % 64;
                ws[k][r] = (n0 + r < N && k0 + k < K) ? to_f(w[static_cast<int64_t>(k0 + k) * w_ks + (n0 + r)]) : 0.f;
            }
        } else {
            for (int i = threadIdx.x; i < 64 * 16; i += 256) {
                const int r = i / 16, k = i % 16;
                ws[k][r] = (n0 + r < N && k0 + k < K) ? to_f(w[static_cast<int64_t>(k0 + k) * w_ks + static_cast<int64_t>(n0 + r) * w_ns]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                xv[i] = xs[k][ty * 4 + i];
                wv[i] = ws[k][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) out[static_cast<int64_t>(m) * ld_out + n] = from_f<TO>(acc[i][j]);
        }
}

// ---------------------------------------------------------------------------------------------
// Attention, general kernel: one CTA per (query token, key split).
// ---------------------------------------------------------------------------------------------
constexpr int kLatThreads = 256;
constexpr int kLatKeys = 32;
constexpr int kLatMaxOut = 32;   // outputs per thread: H * R <= 8192

template <typename T>
__global__ void __launch_bounds__(kLatThreads) latent_attn_general_kernel(const atoma_latent_attn_args a, int splits,
                                                                          float *__restrict__ partial, float *__restrict__ partial_ml) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int H = static_cast<int>(a.H), R = static_cast<int>(a.R);
    const int cs = R + 1;                  // padded row of the staged latents
    float *q_s = sm;                       // [H][R]
    float *c_s = q_s + H * R;              // [kLatKeys][R + 1]
    float *w_s = c_s + kLatKeys * cs;      // [H][kLatKeys]
    float *m_s = w_s + H * kLatKeys;       // [H] running maximum
    float *l_s = m_s + H;                  // [H] running denominator
    float *f_s = l_s + H;                  // [H] rescale factor of the tile
    const int t = blockIdx.x;
    const int b = a.token_seq[t];
    const int p = static_cast<int>(a.positions[t]);
    const int32_t *bt = a.block_tables + static_cast<int64_t>(b) * a.max_blocks;
    const T *cache = static_cast<const T *>(a.latent_cache);
    const int bs = static_cast<int>(a.block_size);
    const int lo = a.window > 0 ? max(0, p - static_cast<int>(a.window) + 1) : 0;
    int k_lo = lo, k_hi = p + 1;
    if (splits > 1) {
        const int n = p + 1 - lo;
        const int per = ((n + splits - 1) / splits + kLatKeys - 1) / kLatKeys * kLatKeys;
        k_lo = min(p + 1, lo + static_cast<int>(blockIdx.y) * per);
        k_hi = min(p + 1, k_lo + per);
    }
    const float *q = a.q_lat + static_cast<int64_t>(t) * H * R;
    for (int i = threadIdx.x; i < H * R; i += kLatThreads) q_s[i] = q[i];
    const bool first = blockIdx.y == 0;
    for (int h = threadIdx.x; h < H; h += kLatThreads) {
        const bool snk = first && a.sink != nullptr;
        m_s[h] = snk ? a.sink[h] : -INFINITY;
        l_s[h] = snk ? 1.f : 0.f;
    }
    float acc[kLatMaxOut];
#pragma unroll
    for (int r = 0; r < kLatMaxOut; ++r) acc[r] = 0.f;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int j0 = k_lo; j0 < k_hi; j0 += kLatKeys) {
        for (int i = threadIdx.x; i < kLatKeys * R; i += kLatThreads) {
            const int jj = i / R, r = i % R, j = j0 + jj;
            float v = 0.f;
            if (j < k_hi) v = to_f(cache[(static_cast<int64_t>(bt[j / bs]) * bs + j % bs) * R + r]);
            c_s[jj * cs + r] = v;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < H * kLatKeys; idx += kLatThreads) {
            const int h = idx / kLatKeys, jj = idx % kLatKeys;
            float s = -INFINITY;
            if (j0 + jj < k_hi) {
                const float *qh = q_s + h * R, *cr = c_s + jj * cs;
                float dot = 0.f;
                for (int r = 0; r < R; ++r) dot = fmaf(qh[r], cr[r], dot);
                s = dot * a.scale;
            }
            w_s[idx] = s;
        }
        __syncthreads();
        for (int h = warp; h < H; h += kLatThreads / 32) {
            const float s = w_s[h * kLatKeys + lane];
            float mx = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, mx);    // finite: the tile holds at least one key
            const float e = s == -INFINITY ? 0.f : expf(s - m_new);
            float sum = e;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const float f = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
            w_s[h * kLatKeys + lane] = e;
            __syncwarp();
            if (lane == 0) {
                m_s[h] = m_new;
                l_s[h] = l_s[h] * f + sum;
                f_s[h] = f;
            }
        }
        __syncthreads();
        const int nj = min(kLatKeys, k_hi - j0);
#pragma unroll
        for (int r = 0; r < kLatMaxOut; ++r) {
            const int od = threadIdx.x + r * kLatThreads;
            if (od < H * R) {
                const int h = od / R, d = od % R;
                float s = acc[r] * f_s[h];
                for (int jj = 0; jj < nj; ++jj) s = fmaf(w_s[h * kLatKeys + jj], c_s[jj * cs + d], s);
                acc[r] = s;
            }
        }
        __syncthreads();
    }
    if (partial) {
        float *o = partial + (static_cast<int64_t>(t) * splits + blockIdx.y) * H * R;
#pragma unroll
        for (int r = 0; r < kLatMaxOut; ++r) {
            const int od = threadIdx.x + r * kLatThreads;
            if (od < H * R) o[od] = acc[r];
        }
        float *ml = partial_ml + (static_cast<int64_t>(t) * splits + blockIdx.y) * H * 2;
        for (int h = threadIdx.x; h < H; h += kLatThreads) {
            ml[2 * h] = m_s[h];
            ml[2 * h + 1] = l_s[h];
        }
        return;
    }
    float *o = a.out + static_cast<int64_t>(t) * H * R;
#pragma unroll
    for (int r = 0; r < kLatMaxOut; ++r) {
        const int od = threadIdx.x + r * kLatThreads;
        if (od < H * R) {
            const float l = l_s[od / R];
            o[od] = l > 0.f ? acc[r] / l : 0.f;
        }
    }
}

// Splits of one query are merged in split order: M = max m_k, out = sum_k acc_k e^(m_k - M) / sum_k l_k e^(m_k - M).
__global__ void __launch_bounds__(256) latent_split_reduce_kernel(const float *__restrict__ partial, const float *__restrict__ partial_ml,
                                                                  float *__restrict__ out, int splits, int H, int R) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H * R; i += blockDim.x) {
        const int h = i / R;
        float M = -INFINITY;
        for (int k = 0; k < splits; ++k) M = fmaxf(M, partial_ml[((t * splits + k) * H + h) * 2]);
        float num = 0.f, den = 0.f;
        for (int k = 0; k < splits; ++k) {
            const float m = partial_ml[((t * splits + k) * H + h) * 2];
            if (m == -INFINITY) continue;
            const float f = expf(m - M);
            num = fmaf(partial[(t * splits + k) * H * R + i], f, num);
            den = fmaf(partial_ml[((t * splits + k) * H + h) * 2 + 1], f, den);
        }
        out[t * H * R + i] = den > 0.f ? num / den : 0.f;
    }
}

}  // namespace

#define HYB_DISPATCH(dtype, CALL) ((dtype) == ATOMA_DTYPE_BF16 ? CALL(__nv_bfloat16) : CALL(float))

bool hyb_latent_norm_cache(const void *proj, int64_t ld, const float *q_w, const float *kv_w, const int64_t *slots, void *cq_out,
                           void *cache, int64_t T, int64_t q_rank, int64_t kv_rank, float eps, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_latent_norm_cache")) return false;
    if (!proj || kv_rank <= 0 || q_rank < 0 || ld < q_rank + kv_rank || !kv_w || (q_rank > 0 && (!q_w || !cq_out)) || (slots && !cache)) {
        set_status(kErrInvalidArg, "atoma_latent_norm_cache: null argument or a row stride below q_rank + kv_rank");
        return false;
    }
#define CALL(TT) launch_ex(latent_norm_cache_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(kRowThreads), 0, stream, \
                           static_cast<const TT *>(proj), ld, q_w, kv_w, slots, static_cast<TT *>(cq_out), static_cast<TT *>(cache), \
                           static_cast<int>(q_rank), static_cast<int>(kv_rank), eps)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "latent_norm_cache_kernel");
#undef CALL
}

bool hyb_head_project(const void *in, const void *w, void *out, int64_t T, int64_t H, int64_t n, int64_t R, int32_t absorb, uint32_t dtype,
                      cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_head_project")) return false;
    if (!in || !w || !out || H <= 0 || n <= 0 || R <= 0) {
        set_status(kErrInvalidArg, "atoma_head_project: null argument or empty head");
        return false;
    }
    const int M = static_cast<int>(T);
    cudaError_t e;
    if (absorb) {
        const dim3 grid(static_cast<unsigned>((R + 63) / 64), static_cast<unsigned>((T + 63) / 64), static_cast<unsigned>(H));
#define CALL(TT) launch_ex(head_project_kernel<TT, TT, float>, grid, dim3(256), 0, stream, static_cast<const TT *>(in), H * n, n, \
                           static_cast<const TT *>(w), n * R, R, static_cast<int64_t>(1), static_cast<float *>(out), H * R, R, M, \
                           static_cast<int>(R), static_cast<int>(n))
        e = HYB_DISPATCH(dtype, CALL);
#undef CALL
    } else {
        const dim3 grid(static_cast<unsigned>((n + 63) / 64), static_cast<unsigned>((T + 63) / 64), static_cast<unsigned>(H));
#define CALL(TT) launch_ex(head_project_kernel<float, TT, TT>, grid, dim3(256), 0, stream, static_cast<const float *>(in), H * R, R, \
                           static_cast<const TT *>(w), n * R, static_cast<int64_t>(1), R, static_cast<TT *>(out), H * n, n, M, \
                           static_cast<int>(n), static_cast<int>(R))
        e = HYB_DISPATCH(dtype, CALL);
#undef CALL
    }
    return hybrid::launched(e, "head_project_kernel");
}

bool hyb_latent_attention(const atoma_latent_attn_args &a, cudaStream_t stream) {
    if (a.T <= 0) return true;
    if (!hybrid::known_dtype(a.dtype, "atoma_latent_attention_paged")) return false;
    if (!a.q_lat || !a.latent_cache || !a.out || !a.positions || !a.token_seq || !a.block_tables || a.H <= 0 || a.R <= 0 ||
        a.block_size <= 0 || a.max_blocks <= 0) {
        set_status(kErrInvalidArg, "atoma_latent_attention_paged: null argument or empty shape");
        return false;
    }
    if (a.H * a.R > kLatThreads * kLatMaxOut) {
        set_status(kErrUnsupported, "atoma_latent_attention_paged: heads * latent size = %lld exceeds %d", static_cast<long long>(a.H * a.R),
                   kLatThreads * kLatMaxOut);
        return false;
    }
    const size_t smem = static_cast<size_t>(a.H * a.R + kLatKeys * (a.R + 1) + a.H * kLatKeys + 3 * a.H) * 4;
    if (smem > 200 * 1024) {
        set_status(kErrUnsupported, "atoma_latent_attention_paged: %zu bytes of shared memory", smem);
        return false;
    }
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(latent_attn_general_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(latent_attn_general_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
    // few query tokens over many keys (decode steps): split the keys so that the device is filled
    int64_t span = a.max_seq_len > 0 ? a.max_seq_len : 0;
    if (a.window > 0) span = std::min<int64_t>(span, a.window);
    int splits = 1;
    if (span >= 4 * kLatKeys && !(g_hybrid_debug & 2)) {
        const int64_t want = (2 * current_device_info().sm_count + a.T - 1) / a.T;
        splits = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>({want, (span + 2 * kLatKeys - 1) / (2 * kLatKeys), 64})));
    }
    float *partial = nullptr, *partial_ml = nullptr;
    if (splits > 1) {
        const size_t n_acc = static_cast<size_t>(a.T) * splits * a.H * a.R, n_ml = static_cast<size_t>(a.T) * splits * a.H * 2;
        partial = static_cast<float *>(get_workspace(stream, (n_acc + n_ml) * 4, kWorkspaceHybridAttn));
        if (!partial) return false;
        partial_ml = partial + n_acc;
    }
    const dim3 grid(static_cast<unsigned>(a.T), static_cast<unsigned>(splits));
#define CALL(TT) launch_ex(latent_attn_general_kernel<TT>, grid, dim3(kLatThreads), smem, stream, a, splits, partial, partial_ml)
    if (!hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "latent_attn_general_kernel")) return false;
#undef CALL
    if (splits == 1) return true;
    return hybrid::launched(launch_ex(latent_split_reduce_kernel, dim3(static_cast<unsigned>(a.T)), dim3(256), 0, stream,
                                      static_cast<const float *>(partial), static_cast<const float *>(partial_ml), a.out, splits,
                                      static_cast<int>(a.H), static_cast<int>(a.R)),
                            "latent_split_reduce_kernel");
}

}  // namespace atoma

using namespace atoma;

extern "C" void atoma_latent_norm_cache(const void *proj, int64_t ld, const float *q_weight, const float *kv_weight,
                                        const int64_t *slot_mapping, void *cq_out, void *latent_cache, int64_t T, int64_t q_rank,
                                        int64_t kv_rank, float eps, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_latent_norm_cache(proj, ld, q_weight, kv_weight, slot_mapping, cq_out, latent_cache, T, q_rank, kv_rank, eps, dtype,
                          static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_head_project(const void *in, const void *w, void *out, int64_t T, int64_t H, int64_t n, int64_t R, int32_t absorb,
                                   uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_head_project(in, w, out, T, H, n, R, absorb, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_latent_attention_paged(const atoma_latent_attn_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_latent_attention_paged: args is NULL");
        return;
    }
    hyb_latent_attention(*args, static_cast<cudaStream_t>(stream));
}
