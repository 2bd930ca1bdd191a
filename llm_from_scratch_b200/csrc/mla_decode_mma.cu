// Tensor-core path of the MLA latent-cache decode (bf16).
#include "common.cuh"

namespace b200 {

size_t mla_decode_mma_workspace(int, int, int, int) { return 256; }

int mla_decode_mma_launch(const void*, const void*, const void*, void*, const int32_t*, int64_t,
                          const int64_t*, int, int, int, int, int, int64_t, float, void*, size_t,
                          int32_t*, cudaStream_t) {
  return B200_ERR_UNSUPPORTED;
}

}  // namespace b200
