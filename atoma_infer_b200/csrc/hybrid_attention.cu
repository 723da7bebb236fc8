// Sigmoid attention over a paged cache: the tensor-core kernel for portions of prompts and the split
// kernel for single decoded tokens (include/atoma_hybrid.h).
#include "common.cuh"
#include "hybrid_common.cuh"

#include "atoma_hybrid.h"

namespace atoma {

bool hyb_attention_fast(const atoma_sigmoid_attn_args &a, cudaStream_t stream, bool *taken) {
    (void)a;
    (void)stream;
    *taken = false;
    return true;
}

}  // namespace atoma
