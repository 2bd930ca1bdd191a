// Token sampling in one launch (reference: Sampler.forward, utils/sampler.py:35-52, and the greedy
// argmax of generate.py:62).
//
// The reference draws  argmax_i softmax(logits / T)_i / E_i  with E_i ~ Exp(1): an exponential race,
// i.e. a sample of the categorical distribution softmax(logits / T).  Taking logarithms,
//   argmax_i  logits_i / T - log(E_i),
// so neither the softmax nor its normaliser has to be materialised: one pass over the row, one
// uniform per element, one block-wide argmax.  A row with T <= 0 (the reference forbids it; the
// benchmark configurations need it) is decoded greedily: argmax of the raw logits, lowest index
// among equal maxima, as torch.argmax.
//
// Random numbers are counter based: element i of row r of call `offset` under `seed` always gets
// the same uniform, whatever the launch shape, so a step can be replayed; the stream is not
// torch's (the reference's draws cannot be reproduced bit for bit by any other generator).
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ uint64_t mix64(uint64_t z) {     // splitmix64 finaliser
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

// uniform in (0, 1]: never 0, so that -log(u) is finite
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t offset, uint32_t row, uint32_t i) {
  const uint64_t h = mix64(mix64(seed ^ (offset * 0x9e3779b97f4a7c15ull)) ^ (static_cast<uint64_t>(row) << 32 | i));
  return (static_cast<float>(h >> 40) + 1.0f) * (1.0f / 16777216.0f);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
sample_kernel(const T* __restrict__ logits, int64_t row_stride, const float* __restrict__ temperatures, int vocab,
              uint64_t seed, uint64_t offset, int64_t* __restrict__ out) {
  __shared__ float s_val[kThreads / 32];
  __shared__ int s_idx[kThreads / 32];
  const int row = blockIdx.x;
  const T* lr = logits + static_cast<int64_t>(row) * row_stride;
  const float t = temperatures ? temperatures[row] : 0.f;
  const bool greedy = !(t > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / t;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += kThreads) {
    float v = to_float<T>(lr[i]);
    if (!greedy) {
      const float e = -__logf(uniform01(seed, offset, row, i));     // Exp(1), > 0 unless u == 1
      v = v * inv_t - __logf(fmaxf(e, 1e-10f));                     // the reference clamps E at 1e-10
    }
    // indices grow within a thread, so a strict comparison keeps the first of equal maxima; NaN never wins
    if (v == v && (v > best || best_i == 0x7fffffff)) {
      best = v;
      best_i = i;
    }
  }
  // argmax across the block; ties go to the lowest index
  auto better = [](float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (better(ov, oi, best, best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kThreads / 32; ++w)
      if (better(s_val[w], s_idx[w], best, best_i)) {
        best = s_val[w];
        best_i = s_idx[w];
      }
    out[row] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_sample(const void* logits, int64_t row_stride, const float* temperatures, int64_t num_rows,
                           int32_t vocab_size, uint64_t seed, uint64_t offset, int64_t* out_tokens,
                           int32_t dtype, void* stream) {
  using namespace b200;
  if (num_rows < 0 || vocab_size <= 0 || row_stride < vocab_size) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (num_rows == 0) return B200_OK;
  if (!logits || !out_tokens) return B200_ERR_ARG;
  if (num_rows > 2147483647) return B200_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = static_cast<int>(num_rows);
  if (dtype == B200_DTYPE_F32)
    sample_kernel<float><<<grid, kThreads, 0, s>>>(static_cast<const float*>(logits), row_stride, temperatures,
                                                   vocab_size, seed, offset, out_tokens);
  else
    sample_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), row_stride,
                                                           temperatures, vocab_size, seed, offset, out_tokens);
  return launch_result();
}
