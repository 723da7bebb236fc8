// Grouped expert products on the 5th-generation tensor cores, for prompt-sized expert segments:
//   out[row, n] = sum_k x[row, k] w[expert(row tile)][n, k]        (x: the gathered, sorted rows; 128-row tiles per expert)
// A CTA owns one (row tile, 128-column tile; 64 gate + 64 up columns with GLU); two CTAs share an SM, so that one's
// epilogue overlaps the other's main loop.  Warp 0 streams the operands with TMA (128-byte swizzle, a three-stage mbarrier
// ring; the weight tile's row coordinate is the expert's offset in the stacked weight tensor, read from the device-side
// tile map), warp 1 issues tcgen05.mma kind::f16 M = 128 with the accumulator in tensor memory, warps 2-5 read it back
// (tcgen05.ld, thread = row) and apply the epilogue.  With GLU the gate rows and the up rows of the same 128 columns are
// loaded into one 128-row operand, one MMA of N = 128 makes both products, and the epilogue stores the clamped gated
// activation.  Every wait is bounded: on a timeout the role sets the error word and the CTA still frees its tensor memory.
#include "common.cuh"
#include "hybrid_common.cuh"

#include "atoma_hybrid.h"

namespace atoma {
namespace {

using namespace hybrid;

constexpr int kUM = 128, kUK = 64, kUStages = 3, kUThreads = 192;
constexpr int kBRows = 128;          // rows of the weight operand per stage = accumulator columns
constexpr uint32_t kWaitLimit = 1u << 22;   // try_wait calls (each may block for a hardware time slice) before a role gives up

struct UmmaArgs {
    __nv_bfloat16 *out;
    int64_t ldo;
    int N, K;
    int rows_per_expert;              // rows of the stacked weight tensor per expert (2 N with GLU, N otherwise)
    const int32_t *tile_expert, *meta, *row_pair;
    const float *out_weight;
    float limit, alpha, shift;
    int *error;                       // set to 1 when a wait ran out
};

__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity, int *error) {
    for (uint32_t i = 0; i < kWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    *error = 1;
    return false;
}

template <bool GLU>
__global__ void __launch_bounds__(kUThreads, 2)
grouped_umma_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const UmmaArgs p) {
    constexpr int kUN = GLU ? kBRows / 2 : kBRows;     // output columns of the CTA
    constexpr int BROWS = kBRows;
    constexpr uint32_t kABytes = kUM * kUK * 2, kBBytes = BROWS * kUK * 2, kStageBytes = kABytes + kBBytes;
    constexpr uint32_t kTmemCols = kBRows;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char *tiles = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    __shared__ __align__(8) uint64_t full[kUStages], empty[kUStages], acc_full;
    __shared__ uint32_t tmem_base_smem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < kUStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        mbar_init(&acc_full, 1);
        fence_mbar_init();
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) tmem_alloc(&tmem_base_smem, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_smem;
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.y;
    const bool active = tile < p.meta[0];
    const int nkb = (p.K + kUK - 1) / kUK;
    const int n0 = blockIdx.x * kUN;
    if (active) {
        if (warp == 0) {
            // ---------------- producer ----------------
            const int w_row = p.tile_expert[tile] * p.rows_per_expert + n0;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % kUStages;
                if (kb >= kUStages && !wait_bounded(&empty[s], ((kb / kUStages) - 1) & 1, p.error)) break;
                if (elect_one_sync()) {
                    unsigned char *st = tiles + s * kStageBytes;
                    mbar_arrive_expect_tx(&full[s], kStageBytes);
                    tma_load_2d(st, &map_x, &full[s], kb * kUK, tile * kUM, kL2EvictFirst);
                    tma_load_2d(st + kABytes, &map_w, &full[s], kb * kUK, w_row, kL2EvictNormal);
                    if constexpr (GLU) tma_load_2d(st + kABytes + kUN * kUK * 2, &map_w, &full[s], kb * kUK, w_row + p.N, kL2EvictNormal);
                }
                __syncwarp();
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            const uint32_t idesc = umma_idesc_f16(kUM, BROWS, true, false);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % kUStages;
                ok = wait_bounded(&full[s], (kb / kUStages) & 1, p.error);
                if (!ok) break;
                tc_fence_after_sync();
                if (elect_one_sync()) {
                    const uint32_t a_addr = smem_u32(tiles + s * kStageBytes), b_addr = a_addr + kABytes;
#pragma unroll
                    for (int kk = 0; kk < kUK / 16; ++kk)
                        umma_f16_ss(tmem_base, umma_desc_k_sw128(a_addr + kk * 32), umma_desc_k_sw128(b_addr + kk * 32), idesc,
                                    (kb | kk) != 0 ? 1u : 0u);
                    umma_commit(&empty[s]);                       // the stage is free once these MMAs have read it
                    if (kb == nkb - 1) umma_commit(&acc_full);    // ... and the accumulator is complete after the last
                }
                __syncwarp();
            }
        } else {
            // ---------------- epilogue: thread = row of the tile ----------------
            const int quad = warp & 3;
            const int row = quad * 32 + lane;
            const int64_t m = static_cast<int64_t>(tile) * kUM + row;
            if (wait_bounded(&acc_full, 0, p.error)) {
                tc_fence_after_sync();
                float ow = 1.f;
                if (!GLU && p.out_weight) {
                    const int pair = p.row_pair[m];
                    ow = pair >= 0 ? p.out_weight[pair] : 0.f;
                }
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
                __nv_bfloat16 *orow = p.out + m * p.ldo;
                for (int c = 0; c < kUN / 32; ++c) {
                    uint32_t gv[32], uv[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, gv);
                    if constexpr (GLU) tmem_ld_32x32b_x32(taddr + kUN + c * 32, uv);
                    tmem_ld_wait();
                    const int nb = n0 + c * 32;
                    if (nb >= p.N) break;
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float g = __uint_as_float(gv[i]);
                        if constexpr (GLU) v[i] = glu_clamped(g, __uint_as_float(uv[i]), p.limit, p.alpha, p.shift);
                        else v[i] = g * ow;
                    }
                    if (nb + 32 <= p.N && (p.ldo % 8) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 && (nb % 8) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 w;
                            w.x = pack2<__nv_bfloat16>(v[i], v[i + 1]);
                            w.y = pack2<__nv_bfloat16>(v[i + 2], v[i + 3]);
                            w.z = pack2<__nv_bfloat16>(v[i + 4], v[i + 5]);
                            w.w = pack2<__nv_bfloat16>(v[i + 6], v[i + 7]);
                            *reinterpret_cast<uint4 *>(orow + nb + i) = w;
                        }
                    } else {
                        for (int i = 0; i < 32 && nb + i < p.N; ++i) orow[nb + i] = __float2bfloat16_rn(v[i]);
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

bool encode_2d(CUtensorMap *out, const void *ptr, int64_t rows, int64_t cols, int box_rows) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) {
        set_status(kErrDriver, "grouped experts: cuTensorMapEncodeTiled is not available");
        return false;
    }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kUK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_status(kErrDriver, "grouped experts: cuTensorMapEncodeTiled failed (CUresult %d)", static_cast<int>(r));
        return false;
    }
    return true;
}

}  // namespace

// Tile rows of this path (the caller pads the experts' segments to it).
int hyb_moe_umma_tile_rows() { return kUM; }

// Shapes this path takes: 16-byte rows for TMA (K % 8 == 0), 16-byte aligned bases, sm_100.
bool hyb_moe_umma_ok(const void *x, const void *w, const void *out, int64_t K, int64_t ldo) {
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return current_device_info().cc_major == 10 && K % 8 == 0 && K >= kUK && ldo > 0 && al(x) && al(w) && al(out);
}

// One grouped product over `max_tiles` row tiles of 128: x [max_tiles * 128, K], w [experts * rows_per_expert, K].
bool hyb_moe_grouped_umma(const void *x, const void *w, void *out, int64_t max_tiles, int64_t experts, int64_t N, int64_t K, bool glu,
                          const int32_t *tile_expert, const int32_t *meta, const int32_t *row_pair, const float *out_weight, float limit,
                          float alpha, float shift, int *error, cudaStream_t stream) {
    CUtensorMap map_x, map_w;
    const int64_t rpe = glu ? 2 * N : N;
    if (!encode_2d(&map_x, x, max_tiles * kUM, K, kUM) || !encode_2d(&map_w, w, experts * rpe, K, glu ? kBRows / 2 : kBRows)) return false;
    UmmaArgs a{};
    a.out = static_cast<__nv_bfloat16 *>(out);
    a.ldo = N;
    a.N = static_cast<int>(N);
    a.K = static_cast<int>(K);
    a.rows_per_expert = static_cast<int>(rpe);
    a.tile_expert = tile_expert;
    a.meta = meta;
    a.row_pair = row_pair;
    a.out_weight = out_weight;
    a.limit = limit;
    a.alpha = alpha;
    a.shift = shift;
    a.error = error;
    const int un = glu ? kBRows / 2 : kBRows;
    const dim3 grid(static_cast<unsigned>((N + un - 1) / un), static_cast<unsigned>(max_tiles));
    const size_t smem = kUStages * (kUM * kUK * 2 + kBRows * kUK * 2) + 1024;
    cudaError_t e;
    if (glu) {
        cudaFuncSetAttribute(grouped_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        e = launch_ex(grouped_umma_kernel<true>, grid, dim3(kUThreads), smem, stream, map_x, map_w, a);
    } else {
        cudaFuncSetAttribute(grouped_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        e = launch_ex(grouped_umma_kernel<false>, grid, dim3(kUThreads), smem, stream, map_x, map_w, a);
    }
    return hybrid::launched(e, "grouped_umma_kernel");
}

}  // namespace atoma
