// MoE routing for inference in one launch: gate scores -> top-k experts per token -> renormalised
// weights -> rows grouped by expert for a grouped GEMM, plus the inverse permutation for the combine.
//
// Arithmetic is Gate.forward of the reference (model/architecture/moe.py:45-90) with the roundings of
// its dtype: scores = sigmoid(logits); selection by top-k of logits + expert_bias (bias cast to the
// dtype first); weights = scores of the selected experts divided by (their sum + 1e-10).  Ties in
// the biased logits go to the lower expert index.
//
// Output rows are ordered by (expert, token, expert rank within the token): a stable counting sort.
// A single CTA does the whole batch (up to 65,536 (token, expert) rows): every thread ranks a
// contiguous chunk of rows with a private per-expert histogram, one warp per expert scans the
// histograms across threads, and each thread then scatters its rows to their final positions.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 1024;
constexpr int kMaxE = 32;   // 32 x 1024 int32 histogram = 128 KiB of shared memory
constexpr int kMaxK = 8;

template <typename T>
__device__ __forceinline__ float round_to(float v) {
  return to_float<T>(from_float<T>(v));
}

struct RouteArgs {
  const void* logits;       // [T, E] dtype
  const float* bias;        // [E]
  int T, E, K;
  int32_t* sorted_token;    // [T*K]  token of sorted row i
  int32_t* sorted_expert;   // [T*K]  expert of sorted row i
  void* sorted_weight;      // [T*K]  dtype, routing weight of sorted row i
  int32_t* offsets;         // [E]    end (exclusive) of each expert's rows
  int32_t* slot_to_row;     // [T, K] sorted-row index of token t's j-th expert in ascending expert order
};

template <typename T>
__global__ void __launch_bounds__(kThreads) moe_route_kernel(const RouteArgs a) {
  extern __shared__ uint8_t smem[];
  // hist[e][thread]: rows of expert e owned by `thread`, later their exclusive prefix over threads
  int32_t* hist = reinterpret_cast<int32_t*>(smem);                 // [E][kThreads]
  int32_t* expert_base = hist + a.E * kThreads;                     // [E + 1]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NT = a.T, E = a.E, K = a.K;
  const int per_thread = (NT + kThreads - 1) / kThreads;
  const int t0 = tid * per_thread, t1 = min(NT, t0 + per_thread);

  for (int e = 0; e < E; ++e) hist[e * kThreads + tid] = 0;
  // pass 1: count.  The top-k is recomputed in pass 2 (cheap: E <= 32) instead of being stored.
  auto select = [&](int t, int (&sel)[kMaxK], float (&wsel)[kMaxK]) {
    const T* row = static_cast<const T*>(a.logits) + static_cast<int64_t>(t) * E;
    float biased[kMaxE];
    for (int e = 0; e < E; ++e) {
      const float lg = to_float<T>(row[e]);
      biased[e] = round_to<T>(lg + round_to<T>(a.bias[e]));
    }
    unsigned long long taken = 0ull;
    for (int k = 0; k < K; ++k) {            // k maxima, lower index first among equals
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e)
        if (!((taken >> e) & 1ull) && (best < 0 || biased[e] > bv)) {
          best = e;
          bv = biased[e];
        }
      taken |= 1ull << best;
    }
    float sum = 0.f;
    int n = 0;
    for (int e = 0; e < E; ++e)               // ascending expert order
      if ((taken >> e) & 1ull) {
        sel[n] = e;
        wsel[n] = round_to<T>(1.f / (1.f + expf(-to_float<T>(row[e]))));
        sum += wsel[n];
        ++n;
      }
    if (K > 1) {
      const float denom = round_to<T>(round_to<T>(sum) + 1e-10f);
      for (int k = 0; k < K; ++k) wsel[k] = round_to<T>(wsel[k] / denom);
    }
  };

  for (int t = t0; t < t1; ++t) {
    int sel[kMaxK];
    float wsel[kMaxK];
    select(t, sel, wsel);
    for (int k = 0; k < K; ++k) hist[sel[k] * kThreads + tid] += 1;
  }
  __syncthreads();
  // exclusive scan over threads, one warp per expert (round-robin), 32 threads' counts per trip
  for (int e = warp; e < E; e += kThreads / 32) {
    int carry = 0;
    for (int base = 0; base < kThreads; base += 32) {
      const int v = hist[e * kThreads + base + lane];
      int x = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      hist[e * kThreads + base + lane] = carry + x - v;
      carry += __shfl_sync(0xffffffffu, x, 31);
    }
    if (lane == 0) expert_base[e + 1] = carry;   // rows of expert e
  }
  __syncthreads();
  if (tid == 0) {
    expert_base[0] = 0;
    for (int e = 0; e < E; ++e) {
      expert_base[e + 1] += expert_base[e];
      a.offsets[e] = expert_base[e + 1];
    }
  }
  __syncthreads();
  // pass 2: scatter rows to expert_base[e] + (rows of e in earlier threads) + (earlier rows of this thread)
  int local[kMaxE];
  for (int e = 0; e < E; ++e) local[e] = 0;
  T* wout = static_cast<T*>(a.sorted_weight);
  for (int t = t0; t < t1; ++t) {
    int sel[kMaxK];
    float wsel[kMaxK];
    select(t, sel, wsel);
    for (int k = 0; k < K; ++k) {
      const int e = sel[k];
      const int pos = expert_base[e] + hist[e * kThreads + tid] + local[e]++;
      a.sorted_token[pos] = t;
      a.sorted_expert[pos] = e;
      wout[pos] = from_float<T>(wsel[k]);
      a.slot_to_row[t * K + k] = pos;
    }
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_moe_route(const void* gate_logits, const float* expert_bias, int32_t num_tokens,
                              int32_t num_experts, int32_t top_k, int32_t* sorted_token,
                              int32_t* sorted_expert, void* sorted_weight, int32_t* expert_offsets,
                              int32_t* slot_to_row, int32_t dtype, void* stream) {
  using namespace b200;
  if (num_tokens < 0 || num_experts <= 0 || top_k <= 0 || top_k > num_experts) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (num_experts > kMaxE || top_k > kMaxK || static_cast<int64_t>(num_tokens) * top_k > 65536)
    return B200_ERR_UNSUPPORTED;
  if (!expert_offsets) return B200_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (num_tokens > 0 &&
      (!gate_logits || !expert_bias || !sorted_token || !sorted_expert || !sorted_weight || !slot_to_row))
    return B200_ERR_ARG;
  RouteArgs a{};
  a.logits = gate_logits;
  a.bias = expert_bias;
  a.T = num_tokens;
  a.E = num_experts;
  a.K = top_k;
  a.sorted_token = sorted_token;
  a.sorted_expert = sorted_expert;
  a.sorted_weight = sorted_weight;
  a.offsets = expert_offsets;
  a.slot_to_row = slot_to_row;
  const size_t smem = (static_cast<size_t>(num_experts) * kThreads + num_experts + 1) * sizeof(int32_t);
  static bool configured[64][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int di = dtype == B200_DTYPE_F32 ? 0 : 1;
  auto kern = di == 0 ? moe_route_kernel<float> : moe_route_kernel<__nv_bfloat16>;
  if (dev >= 0 && dev < 64 && !configured[dev][di]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (kMaxE * kThreads + kMaxE + 1) * 4) != cudaSuccess)
      return B200_ERR_LAUNCH;
    configured[dev][di] = true;
  }
  kern<<<1, kThreads, smem, s>>>(a);
  return launch_result();
}
