// Pieces shared by the two decode kernels (paged GQA, MLA latent): the on-device cut of the flat
// KV-block list into equal per-CTA ranges, and the launch of the kernel that merges the partial
// results of sequences cut across CTAs.
#pragma once

#include "common.cuh"

namespace b200 {

// Blocks of a context of `len` tokens, never more than the block-table row holds.
__device__ __forceinline__ int num_kv_blocks(int64_t len, int64_t bt_stride, int bs) {
  if (len <= 0) return 0;
  int64_t n = (len + bs - 1) / bs;
  return static_cast<int>(n < bt_stride ? n : bt_stride);
}

// Inclusive scan over the CTA; `scratch` holds one int per warp.  Every thread must call it.
__device__ __forceinline__ int block_inclusive_scan(int v, int* scratch, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) scratch[warp] = x;
  __syncthreads();
  int add = 0, tot = 0;
  for (int w = 0; w < nw; ++w) {
    int s = scratch[w];
    if (w < warp) add += s;
    tot += s;
  }
  __syncthreads();
  *total = tot;
  return x + add;
}

// This CTA's share of the flat (sequence, block) list: `cnt` blocks starting at block `start_off`
// of sequence `start_seq`; `per_cta` is the common range length (the last CTAs may get less or
// nothing: cnt == 0).  `scratch` is 34 ints of shared memory.  Every thread must call it.
struct CtaRange {
  int start, cnt, per_cta, start_seq, start_off;
};
__device__ __forceinline__ CtaRange plan_cta_range(const int64_t* lens, int batch,
                                                   int64_t bt_stride, int bs, int* scratch) {
  int local = 0;
  for (int i = threadIdx.x; i < batch; i += blockDim.x)
    local += num_kv_blocks(lens[i], bt_stride, bs);
  int T;
  block_inclusive_scan(local, scratch, &T);
  CtaRange r;
  const int P = gridDim.x, p = blockIdx.x;
  r.per_cta = (T + P - 1) / P;
  r.start = p * r.per_cta;
  r.cnt = (r.per_cta == 0 || r.start >= T) ? 0 : min(r.per_cta, T - r.start);
  r.start_seq = r.start_off = 0;
  if (r.cnt == 0) return r;   // uniform over the CTA
  int carry = 0;
  for (int base = 0; base < batch; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int v = i < batch ? num_kv_blocks(lens[i], bt_stride, bs) : 0;
    int tot;
    const int incl = block_inclusive_scan(v, scratch, &tot) + carry;
    const int excl = incl - v;
    if (v > 0 && excl <= r.start && r.start < incl) {
      scratch[32] = i;
      scratch[33] = r.start - excl;
    }
    carry += tot;
  }
  __syncthreads();
  r.start_seq = scratch[32];
  r.start_off = scratch[33];
  return r;
}

// Workspace layout shared by both decode kernels:
//   part_o  [grid][2][H][D] fp32   unnormalised partial outputs (slot 1: the sequence starts in
//                                   this CTA and continues past it; slot 0: it started earlier)
//   part_ml [grid][2][H][2] fp32   running max (log2 domain) and sum
//   seq_info[batch][2]      int32  first / last CTA of a cut sequence, or -1 / -1
struct CombineArgs {
  void* out;               // [batch][H][D] bf16
  const int64_t* lens;
  const float* part_o;
  const float* part_ml;
  const int32_t* seq_info;
  int batch, H, D;
};
int decode_combine_launch(const CombineArgs& c, cudaStream_t s);

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }
inline size_t decode_workspace_bytes(size_t grid, int batch, int H, int D) {
  return align256(grid * 2 * H * D * sizeof(float)) + align256(grid * 2 * H * 2 * sizeof(float)) +
         align256(static_cast<size_t>(batch) * 2 * sizeof(int32_t));
}

}  // namespace b200
