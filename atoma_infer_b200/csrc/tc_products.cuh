// Batched and grouped bfloat16 products on the warp-level tensor-core path (mma.sync m16n8k16, float32 accumulators),
// shared by the per-head latent projections and the routed experts:
//   O(z)[m, n] = sum_k A(z)[m, k] B(z)[n, k]
// A is read as float32 or bfloat16 (converted while it is staged), B is bfloat16 with arbitrary element strides (so a
// weight stored [k][n] needs no transposed copy), O is float32 or bfloat16.  In grouped mode the row tiles belong to
// experts (tile_expert) and B(z) is the tile's expert; with GLU the tile computes the gate and the up product of the same
// rows and stores the clamped gated activation.
// 64 x 64 x 32 tiles, four warps of 32 x 32.  bfloat16 operands with contiguous, 16-byte aligned k runs (the experts' case) go
// through a three-stage cp.async ring, so that a CTA keeps two tiles of weights in flight while it multiplies a third — at
// decode sizes the product is a pure weight stream; otherwise the next tile's operands are fetched into registers
// (converted / transposed there) while the current one is multiplied.  Why not tcgen05 here: the experts' row segments are known on the device only (no host read), a segment
// is often a handful of rows, and the per-head products have K or N of one head (tens to a few hundred) — tiles of 64 rows
// with operands staged by plain loads fit both; a 128-row tensor-memory tile would be mostly padding.
#pragma once

#include "common.cuh"
#include "hybrid_common.cuh"

namespace atoma {
namespace tc {

struct GemmArgs {
    const void *a;
    int64_t lda, a_zs;
    const __nv_bfloat16 *b;
    int64_t b_zs, b_ks, b_ns;
    void *o;
    int64_t ldo, o_zs;
    int M, N, K;
    // grouped mode (tile_expert != nullptr): row tile -> expert, meta[0] = tiles in use
    const int32_t *tile_expert, *meta, *row_pair;
    const float *out_weight;   // per pair, applied to the output row (nullptr: none)
    float limit, alpha, shift; // GLU epilogue
};

constexpr int kTM = 64, kTN = 64, kTK = 32, kLd = kTK + 8, kStages = 3;

__device__ __forceinline__ void cp_async_wait_two() { asm volatile("cp.async.wait_group 2;" ::: "memory"); }

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    uint4 r;
    r.x = pack2<__nv_bfloat16>(v[0], v[1]);
    r.y = pack2<__nv_bfloat16>(v[2], v[3]);
    r.z = pack2<__nv_bfloat16>(v[4], v[5]);
    r.w = pack2<__nv_bfloat16>(v[6], v[7]);
    return r;
}

// Eight elements p[0], p[stride], ... as bfloat16; elements at index >= nvalid are zero.
template <typename TS>
__device__ __forceinline__ uint4 fetch8(const TS *p, int64_t stride, int nvalid, bool vec) {
    if (nvalid <= 0) return make_uint4(0, 0, 0, 0);
    if (vec && nvalid >= 8 && stride == 1) {
        if constexpr (sizeof(TS) == 2) {
            return *reinterpret_cast<const uint4 *>(p);
        } else {
            const float4 lo = *reinterpret_cast<const float4 *>(p), hi = *reinterpret_cast<const float4 *>(p + 4);
            const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            return pack8(v);
        }
    }
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = i < nvalid ? hybrid::to_f(p[i * stride]) : 0.f;
    return pack8(v);
}

template <typename TA, typename TO, bool GLU>
__global__ void __launch_bounds__(128) gemm_kernel(const GemmArgs p) {
    __shared__ __align__(16) __nv_bfloat16 As[kStages][kTM][kLd], Bs[kStages][kTN][kLd], Us[GLU ? kStages : 1][GLU ? kTN : 1][kLd];
    pdl_launch_dependents();
    pdl_wait();
    const int tile_m = blockIdx.y;
    int64_t z = blockIdx.z;
    if (p.tile_expert) {
        if (tile_m >= p.meta[0]) return;
        z = p.tile_expert[tile_m];
    }
    const int m0 = tile_m * kTM, n0 = blockIdx.x * kTN;
    const TA *A = static_cast<const TA *>(p.a) + (p.tile_expert ? 0 : z * p.a_zs);
    const __nv_bfloat16 *B = p.b + z * p.b_zs;
    const __nv_bfloat16 *U = B + static_cast<int64_t>(p.N) * (p.b_ns == 1 ? 1 : p.b_ns);   // GLU: the up rows follow the N gate rows
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 1, wn = warp & 1;
    const bool a_vec = (p.lda % 8 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && (p.a_zs % 8 == 0);
    const bool b_k_contig = p.b_ks == 1;
    const bool b_vec = ((reinterpret_cast<uintptr_t>(B) & 15) == 0) && (p.b_zs % 8 == 0) &&
                       (b_k_contig ? p.b_ns % 8 == 0 : (p.b_ks % 8 == 0 && p.b_ns == 1)) && (!GLU || (static_cast<int64_t>(p.N) * p.b_ns) % 8 == 0);
    // chunk c of a 64 x 32 tile = (row c / 4, k offset (c % 4) * 8); two chunks per thread
    uint4 ra[2], rb[2], ru[2];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int c = tid + s * 128;
            {
                const int r = c >> 2, k = k0 + (c & 3) * 8;
                const int m = m0 + r;
                ra[s] = fetch8<TA>(A + static_cast<int64_t>(m) * p.lda + k, 1, m < p.M ? p.K - k : 0, a_vec);
            }
            if (b_k_contig) {
                const int r = c >> 2, k = k0 + (c & 3) * 8;
                const int n = n0 + r;
                rb[s] = fetch8<__nv_bfloat16>(B + static_cast<int64_t>(n) * p.b_ns + k, 1, n < p.N ? p.K - k : 0, b_vec);
                if constexpr (GLU) ru[s] = fetch8<__nv_bfloat16>(U + static_cast<int64_t>(n) * p.b_ns + k, 1, n < p.N ? p.K - k : 0, b_vec);
            } else {   // chunk = (k row c / 8, eight consecutive n at (c % 8) * 8)
                const int k = k0 + (c >> 3), n = n0 + (c & 7) * 8;
                rb[s] = fetch8<__nv_bfloat16>(B + static_cast<int64_t>(k) * p.b_ks + static_cast<int64_t>(n) * p.b_ns, p.b_ns, k < p.K ? p.N - n : 0,
                                              b_vec);
            }
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int c = tid + s * 128;
            *reinterpret_cast<uint4 *>(&As[0][c >> 2][(c & 3) * 8]) = ra[s];
            if (b_k_contig) {
                *reinterpret_cast<uint4 *>(&Bs[0][c >> 2][(c & 3) * 8]) = rb[s];
                if constexpr (GLU) *reinterpret_cast<uint4 *>(&Us[0][c >> 2][(c & 3) * 8]) = ru[s];
            } else {
                const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&rb[s]);
#pragma unroll
                for (int i = 0; i < 8; ++i) Bs[0][(c & 7) * 8 + i][c >> 3] = e[i];
            }
        }
    };
    float acc[2][4][4] = {}, acu[GLU ? 2 : 1][4][4] = {};
    auto multiply = [&](int st) {
#pragma unroll
        for (int kk = 0; kk < kTK; kk += 16) {
            uint32_t af[2][4];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) ldmatrix_x4(af[mi], smem_u32(&As[st][wm * 32 + mi * 16 + (lane & 15)][kk + (lane >> 4) * 8]));
#pragma unroll
            for (int nj = 0; nj < 2; ++nj) {
                uint32_t bf[4];
                ldmatrix_x4(bf, smem_u32(&Bs[st][wn * 32 + nj * 16 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]));
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
                    Mma16816<__nv_bfloat16>::run(acc[mi][2 * nj], af[mi], bf[0], bf[1]);
                    Mma16816<__nv_bfloat16>::run(acc[mi][2 * nj + 1], af[mi], bf[2], bf[3]);
                }
                if constexpr (GLU) {
                    uint32_t uf[4];
                    ldmatrix_x4(uf, smem_u32(&Us[st][wn * 32 + nj * 16 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]));
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi) {
                        Mma16816<__nv_bfloat16>::run(acu[mi][2 * nj], af[mi], uf[0], uf[1]);
                        Mma16816<__nv_bfloat16>::run(acu[mi][2 * nj + 1], af[mi], uf[2], uf[3]);
                    }
                }
            }
        }
    };
    const bool ring = sizeof(TA) == 2 && a_vec && b_vec && b_k_contig && p.K % kTK == 0;
    if (ring) {
        const __nv_bfloat16 *Ab = reinterpret_cast<const __nv_bfloat16 *>(A);
        auto issue = [&](int kt, int st) {
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                const int c = tid + s * 128, r = c >> 2, kc = (c & 3) * 8, k = kt * kTK + kc;
                const bool min_ = m0 + r < p.M, nin = n0 + r < p.N;
                cp_async_16(smem_u32(&As[st][r][kc]), min_ ? Ab + static_cast<int64_t>(m0 + r) * p.lda + k : Ab, min_ ? 16 : 0);
                cp_async_16(smem_u32(&Bs[st][r][kc]), nin ? B + static_cast<int64_t>(n0 + r) * p.b_ns + k : B, nin ? 16 : 0);
                if constexpr (GLU) cp_async_16(smem_u32(&Us[st][r][kc]), nin ? U + static_cast<int64_t>(n0 + r) * p.b_ns + k : B, nin ? 16 : 0);
            }
        };
        const int nk = p.K / kTK;
        issue(0, 0);
        cp_async_commit();
        if (nk > 1) issue(1, 1);
        cp_async_commit();
        for (int kt = 0; kt < nk; ++kt) {
            if (kt + 2 < nk) issue(kt + 2, (kt + 2) % kStages);
            cp_async_commit();          // one group per iteration, empty at the tail, so that "all but two" means tile kt
            cp_async_wait_two();
            __syncthreads();
            multiply(kt % kStages);
            __syncthreads();
        }
    } else {
        fetch(0);
        for (int k0 = 0; k0 < p.K; k0 += kTK) {
            stash();
            __syncthreads();
            if (k0 + kTK < p.K) fetch(k0 + kTK);
            multiply(0);
            __syncthreads();
        }
    }
    TO *O = static_cast<TO *>(p.o) + (p.tile_expert ? 0 : z * p.o_zs);
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = m0 + wm * 32 + mi * 16 + g + half * 8;
            if (m >= p.M) continue;
            float ow = 1.f;
            if (p.out_weight) {
                const int pair = p.row_pair[m];
                ow = pair >= 0 ? p.out_weight[pair] : 0.f;
            }
#pragma unroll
            for (int ni = 0; ni < 4; ++ni)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int n = n0 + wn * 32 + ni * 8 + 2 * t4 + e;
                    if (n >= p.N) continue;
                    float v = acc[mi][ni][half * 2 + e];
                    if constexpr (GLU) v = hybrid::glu_clamped(v, acu[mi][ni][half * 2 + e], p.limit, p.alpha, p.shift);
                    else v *= ow;
                    O[static_cast<int64_t>(m) * p.ldo + n] = hybrid::from_f<TO>(v);
                }
        }
}

}  // namespace tc
}  // namespace atoma
