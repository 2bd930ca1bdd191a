// MLA latent-cache decode attention (absorbed form): for every sequence and head
//   score[t] = (q_abs . c_t + q_rope . pe_t) * scale,  P = softmax(score),  out = sum_t P[t] c_t
// where the latent pool row of token t is [c_t (kv_lora_rank) | pe_t (rope_dim)].
//
// Generic path: one CTA per (sequence, head), 4 warps striding over the tokens, a lane owning the
// row elements lane, lane+32, ...; fp32 online softmax, warps merged through shared memory.
#include "common.cuh"

namespace b200 {
namespace {

struct MlaArgs {
  const void* q_abs;
  const void* q_rope;
  const void* lat;
  void* out;
  const int32_t* bt;
  int64_t bt_stride;
  const int64_t* lens;
  int batch, H, r, dr, bs;
  int64_t num_blocks;
  float scale_log2;
  int32_t* status;
};

constexpr int kWarps = 4;
constexpr int kMaxQ = 18;  // (r + dr) <= 576
constexpr int kMaxV = 16;  // r <= 512

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) mla_decode_simple_kernel(const MlaArgs a) {
  __shared__ float s_m[kWarps], s_l[kWarps];
  __shared__ float s_acc[kWarps][kMaxV * 32];
  const int seq = blockIdx.x, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = a.r, dr = a.dr, row_len = r + dr;
  T* op = static_cast<T*>(a.out) + (static_cast<int64_t>(seq) * a.H + head) * r;
  int64_t len64 = a.lens[seq];
  if (len64 <= 0) {
    for (int d = threadIdx.x; d < r; d += blockDim.x) op[d] = from_float<T>(0.f);
    return;
  }
  const int64_t cap = a.bt_stride * a.bs;
  if (len64 > cap) {
    report(a.status, B200_ERR_BOUNDS);
    len64 = cap;
  }
  const int len = static_cast<int>(len64);
  const T* qa = static_cast<const T*>(a.q_abs) + (static_cast<int64_t>(seq) * a.H + head) * r;
  const T* qr = static_cast<const T*>(a.q_rope) + (static_cast<int64_t>(seq) * a.H + head) * dr;
  float qv[kMaxQ], acc[kMaxV];
#pragma unroll
  for (int i = 0; i < kMaxQ; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < r ? to_float<T>(qa[d]) : (d < row_len ? to_float<T>(qr[d - r]) : 0.f);
  }
#pragma unroll
  for (int i = 0; i < kMaxV; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const T* lat = static_cast<const T*>(a.lat);
  for (int t = warp; t < len; t += kWarps) {
    const int id = a.bt[static_cast<int64_t>(seq) * a.bt_stride + t / a.bs];
    if (static_cast<uint64_t>(static_cast<int64_t>(id)) >= static_cast<uint64_t>(a.num_blocks)) {
      report(a.status, B200_ERR_BOUNDS);
      continue;
    }
    const T* row = lat + (static_cast<int64_t>(id) * a.bs + t % a.bs) * row_len;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxQ; ++i) {
      const int d = lane + 32 * i;
      if (d < row_len) dot += qv[i] * to_float<T>(row[d]);
    }
    dot = warp_sum(dot) * a.scale_log2;
    const float mn = fmaxf(m, dot);
    const float al = exp2f(m - mn), pw = exp2f(dot - mn);
    l = l * al + pw;
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int d = lane + 32 * i;
      if (d < r) acc[i] = acc[i] * al + pw * to_float<T>(row[d]);
    }
    m = mn;
  }
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
#pragma unroll
  for (int i = 0; i < kMaxV; ++i) s_acc[warp][lane + 32 * i] = acc[i];
  __syncthreads();
  float M = -INFINITY;
  for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w]);
  float wgt[kWarps], Lsum = 0.f;
  for (int w = 0; w < kWarps; ++w) {
    wgt[w] = s_m[w] == -INFINITY ? 0.f : exp2f(s_m[w] - M);
    Lsum += wgt[w] * s_l[w];
  }
  for (int d = threadIdx.x; d < r; d += blockDim.x) {
    float v = 0.f;
    for (int w = 0; w < kWarps; ++w) v += wgt[w] * s_acc[w][d];
    op[d] = from_float<T>(Lsum > 0.f ? v / Lsum : 0.f);
  }
}

}  // namespace

// tensor-core path (mla_decode_mma.cu); B200_ERR_UNSUPPORTED when the shape is outside it
int mla_decode_mma_launch(const void* q_abs, const void* q_rope, const void* lat, void* out,
                          const int32_t* bt, int64_t bt_stride, const int64_t* lens, int batch,
                          int H, int r, int dr, int bs, int64_t num_blocks, float scale,
                          void* workspace, size_t workspace_bytes, int32_t* status,
                          cudaStream_t s);
size_t mla_decode_mma_workspace(int batch, int H, int r, int dr);
}  // namespace b200

extern "C" size_t b200_mla_decode_workspace_bytes(int32_t batch, int32_t num_heads,
                                                  int32_t kv_lora_rank, int32_t rope_dim,
                                                  int32_t dtype) {
  if (batch <= 0 || num_heads <= 0 || kv_lora_rank <= 0 || rope_dim < 0) return 0;
  if (dtype != B200_DTYPE_BF16) return 256;
  const size_t w = b200::mla_decode_mma_workspace(batch, num_heads, kv_lora_rank, rope_dim);
  return w > 256 ? w : 256;
}

extern "C" int b200_mla_decode(const void* q_abs, const void* q_rope, const void* latent_cache,
                               void* out_latent, const int32_t* block_tables, int64_t bt_stride,
                               const int64_t* context_lens, int32_t batch, int32_t num_heads,
                               int32_t kv_lora_rank, int32_t rope_dim, int32_t block_size,
                               int64_t num_blocks, float scale, void* workspace,
                               size_t workspace_bytes, int32_t dtype, int32_t* status,
                               void* stream) {
  using namespace b200;
  if (batch < 0 || num_heads <= 0 || kv_lora_rank <= 0 || rope_dim < 0 || block_size <= 0 ||
      num_blocks < 0 || bt_stride <= 0)
    return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (batch == 0) return B200_OK;
  if (!q_abs || (rope_dim > 0 && !q_rope) || !out_latent || !block_tables || !context_lens)
    return B200_ERR_ARG;
  if (num_blocks > 0 && !latent_cache) return B200_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == B200_DTYPE_BF16) {
    const int rc = mla_decode_mma_launch(q_abs, q_rope, latent_cache, out_latent, block_tables,
                                         bt_stride, context_lens, batch, num_heads, kv_lora_rank,
                                         rope_dim, block_size, num_blocks, scale, workspace,
                                         workspace_bytes, status, s);
    if (rc != B200_ERR_UNSUPPORTED) return rc;
  }
  if (kv_lora_rank + rope_dim > kMaxQ * 32 || kv_lora_rank > kMaxV * 32 ||
      batch > 2147483647 / 1 || num_heads > 65535)
    return B200_ERR_UNSUPPORTED;
  MlaArgs a{};
  a.q_abs = q_abs;
  a.q_rope = q_rope;
  a.lat = latent_cache;
  a.out = out_latent;
  a.bt = block_tables;
  a.bt_stride = bt_stride;
  a.lens = context_lens;
  a.batch = batch;
  a.H = num_heads;
  a.r = kv_lora_rank;
  a.dr = rope_dim;
  a.bs = block_size;
  a.num_blocks = num_blocks;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  dim3 grid(batch, num_heads);
  if (dtype == B200_DTYPE_F32)
    mla_decode_simple_kernel<float><<<grid, kWarps * 32, 0, s>>>(a);
  else
    mla_decode_simple_kernel<__nv_bfloat16><<<grid, kWarps * 32, 0, s>>>(a);
  return launch_result();
}
