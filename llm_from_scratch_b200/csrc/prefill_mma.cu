// Tensor-core path of the ragged causal prefill attention (bf16).
#include "common.cuh"

namespace b200 {

int prefill_mma_launch(const void*, const void*, const void*, void*, int64_t, int64_t, int64_t,
                       const int32_t*, const int32_t*, int, int, int, int, int, int, float,
                       const void*, const void*, const int32_t*, int64_t, int, int64_t, int32_t*,
                       cudaStream_t) {
  return B200_ERR_UNSUPPORTED;
}

}  // namespace b200
