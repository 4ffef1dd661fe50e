// Tensor-core packed causal prefill (placeholder until the tcgen05 kernel lands).
#include "common.cuh"

namespace attn {
bool prefill_tc_supported(int, int) { return false; }
int prefill_tc_launch(const void*, const void*, const void*, const int32_t*, void*, int, int64_t, int, int, int,
                      float, int, int, int32_t*, cudaStream_t) {
    return ATTN_B200_ESHAPE;
}
}  // namespace attn
