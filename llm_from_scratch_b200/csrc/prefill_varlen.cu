// Ragged (varlen) causal prefill attention over cu_seqlens-packed sequences.
//
// Generic path: one warp per (sequence, query token, query head); a lane owns the head-dim
// elements lane, lane+32, ...; keys are visited in order with an fp32 online softmax.  Keys and
// values come either from the packed k/v tensors of the step or, when a cached prefix exists,
// from the paged pool through block_tables (bottom-right aligned causal mask).
#include "common.cuh"

namespace b200 {
namespace {

struct PrefillArgs {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  int64_t q_stride, k_stride, v_stride;  // token strides, elements
  const int32_t* cu_q;
  const int32_t* cu_k;
  int num_seqs, Hq, Hkv, Dqk, Dv;
  float scale_log2;
  const void* kc;
  const void* vc;
  const int32_t* bt;
  int64_t bt_stride;
  int bs;
  int64_t num_blocks;
  int32_t* status;
};

constexpr int kWarps = 4;
constexpr int kMaxPerLane = 8;  // head dims <= 256

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) prefill_simple_kernel(const PrefillArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.z, head = blockIdx.y;
  const int qi = blockIdx.x * kWarps + warp;
  const int q0 = a.cu_q[s], q_len = a.cu_q[s + 1] - q0;
  const int k0 = a.cu_k[s], k_len = a.cu_k[s + 1] - k0;
  if (qi >= q_len) return;
  const int G = a.Hq / a.Hkv, kvh = head / G;
  const int nkeys = k_len - q_len + qi + 1;  // causal, bottom-right aligned
  const T* qp = static_cast<const T*>(a.q) + static_cast<int64_t>(q0 + qi) * a.q_stride +
                static_cast<int64_t>(head) * a.Dqk;
  float qv[kMaxPerLane], acc[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < a.Dqk ? to_float<T>(qp[d]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int j = 0; j < nkeys; ++j) {
    const T* kp;
    const T* vp;
    if (a.bt == nullptr) {
      kp = static_cast<const T*>(a.k) + static_cast<int64_t>(k0 + j) * a.k_stride +
           static_cast<int64_t>(kvh) * a.Dqk;
      vp = static_cast<const T*>(a.v) + static_cast<int64_t>(k0 + j) * a.v_stride +
           static_cast<int64_t>(kvh) * a.Dv;
    } else {
      const int blk = j / a.bs;
      if (blk >= a.bt_stride) {
        report(a.status, B200_ERR_BOUNDS);
        break;
      }
      const int id = a.bt[static_cast<int64_t>(s) * a.bt_stride + blk];
      if (static_cast<uint64_t>(static_cast<int64_t>(id)) >= static_cast<uint64_t>(a.num_blocks)) {
        report(a.status, B200_ERR_BOUNDS);
        continue;
      }
      const int64_t row = (static_cast<int64_t>(id) * a.bs + j % a.bs) * a.Hkv + kvh;
      kp = static_cast<const T*>(a.kc) + row * a.Dqk;
      vp = static_cast<const T*>(a.vc) + row * a.Dv;
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < a.Dqk) dot += qv[i] * to_float<T>(kp[d]);
    }
    dot = warp_sum(dot) * a.scale_log2;
    const float mn = fmaxf(m, dot);
    const float al = exp2f(m - mn), pw = exp2f(dot - mn);
    l = l * al + pw;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < a.Dv) acc[i] = acc[i] * al + pw * to_float<T>(vp[d]);
    }
    m = mn;
  }
  T* op = static_cast<T*>(a.out) + (static_cast<int64_t>(q0 + qi) * a.Hq + head) * a.Dv;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < a.Dv) op[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace

// fast bf16 tensor-core path, defined in prefill_mma.cu; returns B200_ERR_UNSUPPORTED when the
// shape is outside what it implements
int prefill_mma_launch(const void* q, const void* k, const void* v, void* out, int64_t q_stride,
                       int64_t k_stride, int64_t v_stride, const int32_t* cu_q,
                       const int32_t* cu_k, int num_seqs, int max_seqlen_q, int Hq, int Hkv,
                       int Dqk, int Dv, float scale, const void* kc, const void* vc,
                       const int32_t* bt, int64_t bt_stride, int bs, int64_t num_blocks,
                       const int32_t* plan, int plan_tile_rows, int plan_capacity, int32_t* status,
                       cudaStream_t s, const void* k_tail = nullptr, int64_t k_tail_stride = 0, int tail = 0);

// tcgen05 path for packed keys/values (prefill_umma2.cu): head dims 128/128 and 192/128, 256 query rows of one head per CTA
int prefill_umma2_tile_rows(int Hq, int Hkv, int Dqk, int Dv);
int prefill_umma4_tile_rows(int Hq, int Hkv, int Dqk, int Dv);
int prefill_umma4_launch(const void* q, const void* k, const void* v, void* out, int64_t q_stride, int64_t k_stride,
                         int64_t v_stride, int64_t total_q, int64_t total_k, const int32_t* cu_q,
                         const int32_t* cu_k, int num_seqs, int max_seqlen_q, int Hq, int Hkv, int Dqk, int Dv,
                         float scale, const int32_t* plan, int plan_tile_rows, int plan_capacity, int32_t* status,
                         cudaStream_t s);
int prefill_umma2_launch(const void* q, const void* k, const void* v, void* out, int64_t q_stride, int64_t k_stride,
                         int64_t v_stride, int64_t total_q, int64_t total_k, const int32_t* cu_q,
                         const int32_t* cu_k, int num_seqs, int max_seqlen_q, int Hq, int Hkv, int Dqk, int Dv,
                         float scale, const int32_t* plan, int plan_tile_rows, int plan_capacity, int32_t* status,
                         cudaStream_t s, const void* k_tail, int64_t k_tail_stride, int tail);

// tcgen05 path for a paged prefix (prefill_umma.cu): head_dim 128, even group size, two heads per CTA
int prefill_umma_launch(const void* q, const void* k, const void* v, void* out, int64_t q_stride,
                        int64_t k_stride, int64_t v_stride, int64_t total_q, int64_t total_k,
                        const int32_t* cu_q, const int32_t* cu_k,
                        int num_seqs, int max_seqlen_q, int Hq, int Hkv, int Dqk, int Dv, float scale,
                        const void* kc, const void* vc, const int32_t* bt, int64_t bt_stride, int bs,
                        int64_t num_blocks, const int32_t* plan, int plan_tile_rows, int plan_capacity,
                        int32_t* status, cudaStream_t s);

namespace {

// ---------------------------------------------------------------------------------------------
// Tile list for the tiled prefill kernels: every (sequence, query tile) pair once, tiles with the
// highest index (most keys under the causal mask) first, so that the long tiles start early and the
// grid holds no CTA without work.  One CTA: cnt(r) = number of sequences with more than r tiles comes
// from a difference array (+1 at 0, -1 at n_s) and a prefix sum; tiles of rank r then occupy the
// positions [sum_{r' > r} cnt(r'), ...) in arbitrary order (an atomic cursor per rank).
constexpr int kPlanThreads = 1024;
constexpr int kPlanRanks = 4096;     // most tiles one sequence may have

__device__ __forceinline__ void plan_block_scan(int32_t* v, int32_t* warp_tot) {
  // inclusive prefix sum of v[0..kPlanRanks) in place; 4 consecutive entries per thread
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int x[4];
  int sum = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    sum += v[tid * 4 + i];
    x[i] = sum;
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += y;
    }
    warp_tot[lane] = w;
  }
  __syncthreads();
  const int base = incl - sum + (warp ? warp_tot[warp - 1] : 0);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[tid * 4 + i] = base + x[i];
  __syncthreads();
}

__global__ void __launch_bounds__(kPlanThreads)
prefill_plan_kernel(const int32_t* __restrict__ cu_q, int num_seqs, int tile_rows, int32_t* __restrict__ plan,
                    int capacity, int32_t* status) {
  __shared__ int32_t first[kPlanRanks];    // difference array -> cnt(r) -> tiles of rank <= r
  __shared__ int32_t cursor[kPlanRanks];
  __shared__ int32_t warp_tot[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < kPlanRanks; i += kPlanThreads) first[i] = cursor[i] = 0;
  __syncthreads();
  auto tiles_of = [&](int s) {
    const int len = cu_q[s + 1] - cu_q[s];
    int n = len > 0 ? (len + tile_rows - 1) / tile_rows : 0;
    if (n > kPlanRanks) {                  // the host bounds this with max_seqlen_q; a longer row is an error
      report(status, B200_ERR_BOUNDS);
      n = kPlanRanks;
    }
    return n;
  };
  for (int s = tid; s < num_seqs; s += kPlanThreads) {
    const int n = tiles_of(s);
    if (n > 0) {
      atomicAdd(&first[0], 1);
      if (n < kPlanRanks) atomicAdd(&first[n], -1);
    }
  }
  __syncthreads();
  plan_block_scan(first, warp_tot);        // cnt(r)
  plan_block_scan(first, warp_tot);        // tiles of rank <= r
  const int total = first[kPlanRanks - 1];
  if (tid == 0) {
    plan[0] = min(total, capacity);
    plan[1] = tile_rows;
    plan[2] = capacity;
    plan[3] = 0;
    if (total > capacity) report(status, B200_ERR_WORKSPACE);
  }
  for (int s = warp; s < num_seqs; s += kPlanThreads / 32) {
    const int n = tiles_of(s);
    for (int r = lane; r < n; r += 32) {
      const int pos = total - first[r] + atomicAdd(&cursor[r], 1);   // ranks above r come first
      if (pos < capacity) plan[kPlanHeader + pos] = static_cast<int32_t>((static_cast<uint32_t>(s) << 16) | r);
    }
  }
}

}  // namespace
}  // namespace b200

extern "C" int32_t b200_prefill_tile_rows(int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim_qk,
                                          int32_t head_dim_v, int32_t dtype) {
  if (dtype != B200_DTYPE_BF16 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return 0;
  // packed keys: the row-pair tcgen05 kernel serves 128/128 and 192/128 (the two-head kernel, 128 rows per
  // tile, only takes over for a paged prefix and then ignores a 256-row tile list)
  if (const int r = b200::prefill_umma2_tile_rows(num_q_heads, num_kv_heads, head_dim_qk, head_dim_v)) return r;
  // head_dim 64 with query heads in groups of four per KV head: the four-heads-per-CTA tcgen05 kernel, 128 rows
  if (const int r = b200::prefill_umma4_tile_rows(num_q_heads, num_kv_heads, head_dim_qk, head_dim_v)) return r;
  const bool mma = (head_dim_qk == head_dim_v && (head_dim_qk == 32 || head_dim_qk == 64 || head_dim_qk == 128)) ||
                   (head_dim_qk == 192 && head_dim_v == 128);
  return mma ? 64 : 0;
}

extern "C" size_t b200_prefill_plan_bytes(int64_t total_q_tokens, int32_t num_seqs, int32_t tile_rows) {
  if (total_q_tokens < 0 || num_seqs < 0 || tile_rows <= 0) return 0;
  const int64_t capacity = (total_q_tokens + tile_rows - 1) / tile_rows + num_seqs;
  return static_cast<size_t>(b200::kPlanHeader + capacity) * sizeof(int32_t);
}

extern "C" int b200_prefill_plan(const int32_t* cu_seqlens_q, int32_t num_seqs, int32_t max_seqlen_q,
                                 int32_t tile_rows, int32_t* plan, size_t plan_bytes, int32_t* status,
                                 void* stream) {
  using namespace b200;
  if (num_seqs < 0 || tile_rows <= 0 || max_seqlen_q < 0 || !plan) return B200_ERR_ARG;
  if (plan_bytes < (kPlanHeader + 1) * sizeof(int32_t)) return B200_ERR_WORKSPACE;
  if (num_seqs > 65535 || (max_seqlen_q + tile_rows - 1) / tile_rows > kPlanRanks) return B200_ERR_UNSUPPORTED;
  if (num_seqs > 0 && !cu_seqlens_q) return B200_ERR_ARG;
  const int64_t capacity = static_cast<int64_t>(plan_bytes / sizeof(int32_t)) - kPlanHeader;
  prefill_plan_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      cu_seqlens_q, num_seqs, tile_rows, plan, static_cast<int>(capacity > 2147483647 ? 2147483647 : capacity),
      status);
  return launch_result();
}

extern "C" int b200_prefill_varlen(const void* q, const void* k, const void* v, void* out,
                                   int64_t q_token_stride, int64_t k_token_stride,
                                   int64_t v_token_stride, int64_t total_q_tokens,
                                   int64_t total_k_tokens, const int32_t* cu_seqlens_q,
                                   const int32_t* cu_seqlens_k, int32_t num_seqs,
                                   int32_t max_seqlen_q, int32_t max_seqlen_k,
                                   int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim_qk,
                                   int32_t head_dim_v, float scale, const void* k_cache,
                                   const void* v_cache, const int32_t* block_tables,
                                   int64_t bt_stride, int32_t block_size, int64_t num_blocks,
                                   const int64_t* slot_mapping, const int32_t* plan, int32_t plan_tile_rows,
                                   int32_t plan_capacity, int32_t dtype, int32_t* status, void* stream) {
  using namespace b200;
  if (num_seqs < 0 || max_seqlen_q < 0 || max_seqlen_k < 0 || num_q_heads <= 0 ||
      num_kv_heads <= 0 || head_dim_qk <= 0 || head_dim_v <= 0)
    return B200_ERR_ARG;
  if (num_q_heads % num_kv_heads != 0) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (total_q_tokens < 0 || total_k_tokens < 0) return B200_ERR_ARG;
  if (num_seqs == 0 || max_seqlen_q == 0 || total_q_tokens == 0) return B200_OK;
  if (!q || !out || !cu_seqlens_q || !cu_seqlens_k) return B200_ERR_ARG;
  if (block_tables == nullptr) {
    if (!k || !v) return B200_ERR_ARG;
  } else {
    if (!k_cache || !v_cache || block_size <= 0 || bt_stride <= 0 || num_blocks <= 0)
      return B200_ERR_ARG;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  if (slot_mapping != nullptr) {
    // the step's store_kvcache scatter rides in this call: the new tokens' rows go into the pool first (its
    // own launch, ahead of the attention grid in the stream), so a paged prefix read sees them
    if (!k || !v || !k_cache || !v_cache || block_size <= 0 || num_blocks <= 0) return B200_ERR_ARG;
    if (head_dim_qk != head_dim_v) return B200_ERR_UNSUPPORTED;
    const int64_t rows = block_tables == nullptr && total_k_tokens < total_q_tokens ? total_k_tokens : total_q_tokens;
    if (rows > 2147483647LL) return B200_ERR_TOO_LARGE;
    const int rc = b200_store_kvcache(k, v, k_token_stride, v_token_stride, const_cast<void*>(k_cache),
                                      const_cast<void*>(v_cache), slot_mapping, static_cast<int32_t>(rows),
                                      num_kv_heads, head_dim_qk, num_blocks * block_size, dtype, status, stream);
    if (rc != B200_OK) return rc;
  }

  if (dtype == B200_DTYPE_BF16) {
    if (block_tables == nullptr) {
      // packed keys: 256 query rows of one head per CTA (measured 967 against 865 TFLOP/s for the two-head
      // kernel on 262,144 ragged tokens at head_dim 128)
      const int rc2 = prefill_umma2_launch(q, k, v, out, q_token_stride, k_token_stride, v_token_stride,
                                           total_q_tokens, total_k_tokens, cu_seqlens_q, cu_seqlens_k, num_seqs,
                                           max_seqlen_q, num_q_heads, num_kv_heads, head_dim_qk, head_dim_v, scale,
                                           plan, plan_tile_rows, plan_capacity, status, s, nullptr, 0, 0);
      if (rc2 != B200_ERR_UNSUPPORTED) return rc2;
      // head_dim 64, four query heads of a KV head per CTA
      const int rc4 = prefill_umma4_launch(q, k, v, out, q_token_stride, k_token_stride, v_token_stride,
                                           total_q_tokens, total_k_tokens, cu_seqlens_q, cu_seqlens_k, num_seqs,
                                           max_seqlen_q, num_q_heads, num_kv_heads, head_dim_qk, head_dim_v, scale,
                                           plan, plan_tile_rows, plan_capacity, status, s);
      if (rc4 != B200_ERR_UNSUPPORTED) return rc4;
    }
    const int rcu = prefill_umma_launch(q, k, v, out, q_token_stride, k_token_stride, v_token_stride,
                                        total_q_tokens, total_k_tokens, cu_seqlens_q, cu_seqlens_k, num_seqs, max_seqlen_q, num_q_heads,
                                        num_kv_heads, head_dim_qk, head_dim_v, scale, k_cache, v_cache,
                                        block_tables, bt_stride, block_size, num_blocks, plan, plan_tile_rows,
                                        plan_capacity, status, s);
    if (rcu != B200_ERR_UNSUPPORTED) return rcu;
    const int rc = prefill_mma_launch(q, k, v, out, q_token_stride, k_token_stride,
                                      v_token_stride, cu_seqlens_q, cu_seqlens_k, num_seqs,
                                      max_seqlen_q, num_q_heads, num_kv_heads, head_dim_qk,
                                      head_dim_v, scale, k_cache, v_cache, block_tables, bt_stride,
                                      block_size, num_blocks, plan, plan_tile_rows, plan_capacity, status, s);
    if (rc != B200_ERR_UNSUPPORTED) return rc;
  }

  if (head_dim_qk > kMaxPerLane * 32 || head_dim_v > kMaxPerLane * 32) return B200_ERR_UNSUPPORTED;
  if (num_seqs > 65535 || num_q_heads > 65535) return B200_ERR_UNSUPPORTED;
  PrefillArgs a{};
  a.q = q;
  a.k = k;
  a.v = v;
  a.out = out;
  a.q_stride = q_token_stride;
  a.k_stride = k_token_stride;
  a.v_stride = v_token_stride;
  a.cu_q = cu_seqlens_q;
  a.cu_k = cu_seqlens_k;
  a.num_seqs = num_seqs;
  a.Hq = num_q_heads;
  a.Hkv = num_kv_heads;
  a.Dqk = head_dim_qk;
  a.Dv = head_dim_v;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.kc = k_cache;
  a.vc = v_cache;
  a.bt = block_tables;
  a.bt_stride = bt_stride;
  a.bs = block_size;
  a.num_blocks = num_blocks;
  a.status = status;
  dim3 grid((max_seqlen_q + kWarps - 1) / kWarps, num_q_heads, num_seqs);
  if (dtype == B200_DTYPE_F32)
    prefill_simple_kernel<float><<<grid, kWarps * 32, 0, s>>>(a);
  else
    prefill_simple_kernel<__nv_bfloat16><<<grid, kWarps * 32, 0, s>>>(a);
  return launch_result();
}

extern "C" int b200_prefill_varlen_shared_tail(const void* q, const void* k_head, const void* k_tail, const void* v,
                                               void* out, int64_t q_token_stride, int64_t k_head_token_stride,
                                               int64_t k_tail_token_stride, int64_t v_token_stride,
                                               int64_t total_q_tokens, int64_t total_k_tokens,
                                               const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                               int32_t num_seqs, int32_t max_seqlen_q, int32_t num_heads,
                                               int32_t head_dim_qk, int32_t tail_dim, int32_t head_dim_v,
                                               float scale, const int32_t* plan, int32_t plan_tile_rows,
                                               int32_t plan_capacity, int32_t dtype, int32_t* status,
                                               void* stream) {
  using namespace b200;
  if (num_seqs < 0 || max_seqlen_q < 0 || num_heads <= 0 || head_dim_qk <= 0 || head_dim_v <= 0 ||
      tail_dim <= 0 || tail_dim >= head_dim_qk)
    return B200_ERR_ARG;
  if (dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (num_seqs == 0 || max_seqlen_q == 0) return B200_OK;
  if (!q || !k_head || !k_tail || !v || !out || !cu_seqlens_q || !cu_seqlens_k) return B200_ERR_ARG;
  if (total_q_tokens <= 0 || total_k_tokens <= 0) return B200_ERR_ARG;
  const int rc2 = prefill_umma2_launch(q, k_head, v, out, q_token_stride, k_head_token_stride, v_token_stride,
                                       total_q_tokens, total_k_tokens, cu_seqlens_q, cu_seqlens_k, num_seqs,
                                       max_seqlen_q, num_heads, num_heads, head_dim_qk, head_dim_v, scale, plan,
                                       plan_tile_rows, plan_capacity, status, static_cast<cudaStream_t>(stream),
                                       k_tail, k_tail_token_stride, tail_dim);
  if (rc2 != B200_ERR_UNSUPPORTED) return rc2;
  return prefill_mma_launch(q, k_head, v, out, q_token_stride, k_head_token_stride, v_token_stride, cu_seqlens_q,
                            cu_seqlens_k, num_seqs, max_seqlen_q, num_heads, num_heads, head_dim_qk, head_dim_v,
                            scale, nullptr, nullptr, nullptr, 0, 0, 0, plan, plan_tile_rows, plan_capacity, status,
                            static_cast<cudaStream_t>(stream), k_tail, k_tail_token_stride, tail_dim);
}
