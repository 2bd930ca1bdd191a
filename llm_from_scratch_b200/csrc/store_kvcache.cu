// store_kvcache: scatter the new tokens' K/V rows into the paged pool through slot_mapping.
//
// Pure HBM traffic: every row (Hkv*D elements, 2 KiB for 8 heads x 128 x bf16) is read once and
// written once.  One "unit" is a 16-byte chunk of one row; a thread moves UNROLL chunks of K and
// UNROLL chunks of V per loop trip, issuing all loads before the first store so that 2*UNROLL*16
// bytes per thread are in flight.  Consecutive lanes take consecutive chunks of the same row, so
// every warp-level access is a contiguous 512-byte segment.  The grid is a multiple of the SM
// count; a grid-stride loop covers any number of tokens.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kCtasPerSm = 8;

// rows are `cpr` 16-byte chunks long; strides are in 16-byte chunks
__global__ void __launch_bounds__(kThreads)
store_kvcache_vec16(const uint4* __restrict__ k, const uint4* __restrict__ v, int64_t k_stride,
                    int64_t v_stride, uint4* __restrict__ kc, uint4* __restrict__ vc,
                    const int64_t* __restrict__ slots, int64_t total, int cpr, int64_t num_slots,
                    int32_t* status) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; base < total;
       base += step * kUnroll) {
    uint4 kr[kUnroll], vr[kUnroll];
    int64_t dst[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + u * step;
      dst[u] = -1;
      if (i < total) {
        const int64_t t = i / cpr;
        const int c = static_cast<int>(i - t * cpr);
        const int64_t slot = __ldg(slots + t);
        if (slot >= 0) {
          if (slot < num_slots) {
            dst[u] = slot * cpr + c;
            kr[u] = __ldcs(k + t * k_stride + c);
            if (v != nullptr) vr[u] = __ldcs(v + t * v_stride + c);
          } else {
            report(status, B200_ERR_BOUNDS);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (dst[u] >= 0) {
        kc[dst[u]] = kr[u];
        if (v != nullptr) vc[dst[u]] = vr[u];
      }
    }
  }
}

// element-granular fallback for rows that are not a multiple of 16 bytes or are misaligned
template <typename T>
__global__ void __launch_bounds__(kThreads)
store_kvcache_scalar(const T* __restrict__ k, const T* __restrict__ v, int64_t k_stride,
                     int64_t v_stride, T* __restrict__ kc, T* __restrict__ vc,
                     const int64_t* __restrict__ slots, int64_t total, int row, int64_t num_slots,
                     int32_t* status) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += step) {
    const int64_t t = i / row;
    const int c = static_cast<int>(i - t * row);
    const int64_t slot = slots[t];
    if (slot < 0) continue;
    if (slot >= num_slots) {
      report(status, B200_ERR_BOUNDS);
      continue;
    }
    kc[slot * row + c] = k[t * k_stride + c];
    if (v != nullptr) vc[slot * row + c] = v[t * v_stride + c];
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_store_kvcache(const void* k, const void* v, int64_t k_token_stride,
                                  int64_t v_token_stride, void* k_cache, void* v_cache,
                                  const int64_t* slot_mapping, int32_t num_tokens,
                                  int32_t num_kv_heads, int32_t head_dim, int64_t num_slots,
                                  int32_t dtype, int32_t* status, void* stream) {
  using namespace b200;
  if (num_tokens < 0 || num_kv_heads <= 0 || head_dim <= 0 || num_slots < 0) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (num_tokens == 0) return B200_OK;
  if (!k || !k_cache || !slot_mapping) return B200_ERR_ARG;
  if ((v == nullptr) != (v_cache == nullptr)) return B200_ERR_ARG;  // both or neither
  if (v == nullptr) v_token_stride = k_token_stride;
  const int esize = dtype == B200_DTYPE_F32 ? 4 : 2;
  const int64_t row = static_cast<int64_t>(num_kv_heads) * head_dim;
  if (k_token_stride < row || v_token_stride < row) return B200_ERR_ARG;
  const int sms = sm_count_cached();
  if (sms <= 0) return B200_ERR_NO_DEVICE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t row_bytes = row * esize;
  const bool vec = (row_bytes % 16 == 0) && (k_token_stride * esize % 16 == 0) &&
                   (v_token_stride * esize % 16 == 0) && aligned16(k) && aligned16(v) &&
                   aligned16(k_cache) && aligned16(v_cache);  // a null v is "aligned"
  if (vec) {
    const int cpr = static_cast<int>(row_bytes / 16);
    const int64_t total = static_cast<int64_t>(num_tokens) * cpr;
    int64_t want = (total + int64_t(kThreads) * kUnroll - 1) / (int64_t(kThreads) * kUnroll);
    int64_t cap = int64_t(sms) * kCtasPerSm;
    int grid = static_cast<int>(want < cap ? want : cap);
    if (grid < 1) grid = 1;
    store_kvcache_vec16<<<grid, kThreads, 0, s>>>(
        static_cast<const uint4*>(k), static_cast<const uint4*>(v), k_token_stride * esize / 16,
        v_token_stride * esize / 16, static_cast<uint4*>(k_cache), static_cast<uint4*>(v_cache),
        slot_mapping, total, cpr, num_slots, status);
  } else {
    const int64_t total = static_cast<int64_t>(num_tokens) * row;
    int64_t want = (total + kThreads - 1) / kThreads;
    int64_t cap = int64_t(sms) * kCtasPerSm;
    int grid = static_cast<int>(want < cap ? want : cap);
    if (grid < 1) grid = 1;
    if (dtype == B200_DTYPE_F32) {
      store_kvcache_scalar<float><<<grid, kThreads, 0, s>>>(
          static_cast<const float*>(k), static_cast<const float*>(v), k_token_stride,
          v_token_stride, static_cast<float*>(k_cache), static_cast<float*>(v_cache), slot_mapping,
          total, static_cast<int>(row), num_slots, status);
    } else {
      store_kvcache_scalar<__nv_bfloat16><<<grid, kThreads, 0, s>>>(
          static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
          k_token_stride, v_token_stride, static_cast<__nv_bfloat16*>(k_cache),
          static_cast<__nv_bfloat16*>(v_cache), slot_mapping, total, static_cast<int>(row),
          num_slots, status);
    }
  }
  return launch_result();
}
