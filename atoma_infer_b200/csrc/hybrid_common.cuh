// Device helpers shared by the hybrid-model kernels (hybrid_ops.cu, hybrid_attention.cu): number-format
// conversion, a fixed-order block reduction, and the scalar formulas of the mechanisms — written once so
// that the general, the tensor-core and the split-decode kernels evaluate the same expressions.
#pragma once

#include "common.cuh"

namespace atoma {
namespace hybrid {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Sum over the CTA in a fixed order (lanes by xor tree, then warps in index order); every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float *red /* [32] shared */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    __syncthreads();   // red may still be read from the previous call
    if ((threadIdx.x & 31) == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nwarp; ++i) s += red[i];
    return s;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu(float x) { return x * sigmoidf_(x); }

// Weight of one visible key: dot = q . k (float32), dist = query position - key position >= 0.
__device__ __forceinline__ float sigmoid_weight(float dot, float scale, float softcap, float slope, float dist, float head_bias) {
    float s = dot * scale;
    if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    s -= slope * dist;
    return sigmoidf_(s + head_bias);
}

// minGRU: update gate and candidate from their pre-activations.
__device__ __forceinline__ void mingru_gates(float zpre, float u, float &z, float &cand) {
    z = sigmoidf_(zpre);
    cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
}

__device__ __forceinline__ float glu_act(float g, int act) {
    if (act == 1) return fmaxf(g, 0.f);
    if (act == 2) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return silu(g);
}

// Clamped gated activation: g = min(g, limit), u = clamp(u, -limit, limit) (limit <= 0: no clamp); g sigmoid(alpha g) (u + shift).
__device__ __forceinline__ float glu_clamped(float g, float u, float limit, float alpha, float shift) {
    if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    return g * sigmoidf_(alpha * g) * (u + shift);
}

__device__ __forceinline__ float gelu_tanh(float z) { return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

// Host side: what every operator does after a launch, and the number-format check.
inline bool launched(cudaError_t e, const char *what) {
    note_launch();
    if (e != cudaSuccess) {
        set_status(static_cast<int>(e), "%s: %s", what, cudaGetErrorString(e));
        return false;
    }
    return check_launch(what);
}
inline bool known_dtype(uint32_t dtype, const char *what) {
    if (dtype == 1u || dtype == 2u) return true;
    set_status(kErrInvalidArg, "%s: dtype must be 1 (bfloat16) or 2 (float32), got %u", what, dtype);
    return false;
}

}  // namespace hybrid
}  // namespace atoma
