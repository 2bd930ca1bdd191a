// Paged GQA decode attention.
//
// Fast path (bf16, block_size 16, head_dim 32/64/128, group size <= 16, Hkv <= 16)
// ---------------------------------------------------------------------------------------------
// The work is the flat list of all KV blocks of all sequences, in (sequence, block) order.  It is
// cut into gridDim.x equal contiguous ranges, one per persistent CTA, so every CTA streams the
// same number of bytes whatever the mix of context lengths ("split-K" falls out of the cut).  Each
// CTA recomputes the cut from context_lens itself, so the launch needs no host-side knowledge of
// the lengths and can be captured in a CUDA graph.
//
// A sequence that crosses a cut is finished inside the same launch: every warp that completes a
// piece writes its unnormalised (max, sum, O) partials, fences, and bumps an arrival counter of
// its (sequence, KV head); the warp whose arrival completes the count merges the pieces in fixed
// CTA order (so the result does not depend on which warp came last), writes the output rows and
// returns the counter to zero.  The counters occupy the first kDecodeCounterBytes of the workspace,
// which must be zero when the buffer is first used; every launch leaves them zero.  That form serves
// small batches (a decode step is then a chain of short dependent kernels, and this removes one);
// larger batches use a separate merge kernel launched as a programmatic dependent, which merges all
// sequences in parallel instead of lengthening the tails of the streaming CTAs.
//
// A CTA has one warp per KV head; the warps of a CTA walk the same blocks, so between them they
// read each 16-token block of the pool as one contiguous Hkv*D*16*2-byte segment of K and one of
// V.  Every warp owns a private 3-stage ring of (K tile, V tile) in shared memory that it fills
// with 16-byte cp.async.cg copies (coalesced 256-byte rows, XOR-swizzled so ldmatrix is free of
// bank conflicts) and drains with no CTA-wide barrier.  The G query heads that share the KV head
// are the N dimension of mma.sync m16n8k16: S^T[token, head] = K . Q^T and O^T[d, head] =
// V^T . P^T, so each K/V byte is read from HBM exactly once and used for all G heads.  Softmax is
// the online form in fp32 in the log2 domain; column statistics are reduced with warp shuffles.
//
// Generic path (any dtype / head_dim <= 256 / block size): one CTA per (sequence, query head),
// fp32 FMA arithmetic.  It is the path the fp32 engine configuration uses.
#include <limits.h>

#include "decode_common.cuh"

namespace b200 {
namespace {

constexpr int kTok = 16;    // tokens per KV block on the fast path
constexpr size_t kDecodeCounterBytes = 256 * 1024;  // arrival counters at the head of the workspace
constexpr int64_t kDecodeCounters = kDecodeCounterBytes / sizeof(int32_t);
constexpr int kFusedMergeMaxBatch = 32;  // batches up to this size merge split contexts inside the launch
constexpr int kStages = 3;  // (K,V) tiles in flight per warp
constexpr int kMinBlocksPerCta = 4;  // small problems use fewer CTAs instead of more pieces to merge
constexpr int kMaxFastThreads = 512;

struct DecodeArgs {
  const void* q;
  const void* kc;
  const void* vc;
  void* out;
  const int32_t* bt;
  int64_t bt_stride;
  const int64_t* lens;
  int batch, Hq, Hkv, D, bs;
  int64_t num_blocks;
  float scale_log2;  // softmax scale * log2(e)
  float* part_o;     // [grid][2][Hq][D]   unnormalised partial outputs
  float* part_ml;    // [grid][2][Hq][2]   running max (log2 domain) and sum
  int32_t* seq_info; // [batch][2]         first / last CTA of a split sequence, or -1 (separate merge kernel)
  int32_t* counters; // [batch][Hkv]       arrivals per (sequence, KV head), zero between launches; null = separate merge
  int32_t* status;
};

struct Cursor {
  int seq, blk, nblk, len;
};

template <int D>
__device__ __forceinline__ int swizzle_chunk(int c, int t) {
  constexpr int CPR = D / 8;
  if (CPR >= 8) return c ^ (t & 7);
  return c ^ ((t >> 1) & (CPR - 1));  // CPR == 4: two rows share a 128-byte line
}

// Merge of the `np` pieces of (sequence `seq`, KV head `h`) by one warp: pieces live in the partial slots of
// CTAs first .. first + np - 1 (slot 1 in the CTA where the sequence starts, slot 0 in the others).  Four
// fp32 columns per lane, 32 / (D / 4) heads per pass; the lanes of a head share the search for its maximum,
// and the weighted sum takes four pieces per trip so that their loads are in flight together.  Loads bypass
// L1: other SMs wrote the data.
template <int D>
__device__ __forceinline__ void merge_split_sequence(const DecodeArgs& a, int seq, int h, int G, int first,
                                                     int np, int lane) {
  constexpr int LPH = D / 4;    // lanes per head
  constexpr int HPP = 32 / LPH; // heads per pass
  const int64_t n = static_cast<int64_t>(a.Hq) * D;
  const int sub = lane % LPH;
  const int col = sub * 4;
  auto slot_of = [&](int p) -> int64_t { return static_cast<int64_t>(first + p) * 2 + (p == 0 ? 1 : 0); };
  for (int hb = 0; hb < G; hb += HPP) {
    const int hl = hb + lane / LPH;
    const bool active = hl < G;
    const int head = h * G + (active ? hl : 0);
    float M = -INFINITY;
    for (int p = sub; p < np; p += LPH) M = fmaxf(M, __ldcg(a.part_ml + (slot_of(p) * a.Hq + head) * 2));
#pragma unroll
    for (int off = 1; off < LPH; off <<= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p0 = 0; p0 < np; p0 += 4) {
      float2 ml[4];
      float4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const bool in = p0 + u < np;
        const int64_t slot = slot_of(in ? p0 + u : 0);
        ml[u] = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (slot * a.Hq + head) * 2));
        x[u] = __ldcg(reinterpret_cast<const float4*>(a.part_o + slot * n + head * D + col));
        if (!in) ml[u] = make_float2(-INFINITY, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float w = exp2f(ml[u].x - M);   // 0 for the padding of the last trip
        L += w * ml[u].y;
        acc.x += w * x[u].x;
        acc.y += w * x[u].y;
        acc.z += w * x[u].z;
        acc.w += w * x[u].w;
      }
    }
    if (active) {
      const float inv = 1.f / L;
      uint2 packed;
      packed.x = pack_bf16x2(acc.x * inv, acc.y * inv);
      packed.y = pack_bf16x2(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(a.out) + (static_cast<int64_t>(seq) * a.Hq + head) * D +
                                col) = packed;
    }
  }
}

template <int D, int NT>
__global__ void __launch_bounds__(kMaxFastThreads)
paged_decode_bf16_kernel(const DecodeArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_scan[32];
  __shared__ int s_start_seq, s_start_off;

  constexpr int ROWB = D * 2;         // bytes per token row of one head
  constexpr int TILEB = kTok * ROWB;  // one K (or V) tile
  constexpr int CPR = D / 8;          // 16-byte chunks per row
  constexpr int KS = D / 16;          // k-steps of QK^T == m-tiles of PV
  constexpr int LOADS = (kTok * CPR) / 32;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int B = a.batch;
  const int G = a.Hq / a.Hkv;
  const int p = blockIdx.x, P = gridDim.x;

  // ---- plan: total block count, then the (sequence, block) where this CTA's range starts ----
  int local = 0;
  for (int i = threadIdx.x; i < B; i += blockDim.x)
    local += num_kv_blocks(a.lens[i], a.bt_stride, kTok);
  int T;
  block_inclusive_scan(local, s_scan, &T);
  if (a.counters == nullptr) {
    // the merge kernel is launched as a programmatic dependent: let its CTAs be placed while this grid
    // runs (they wait for this grid's completion before they read anything)
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  } else {
    // rows of empty contexts are zero (no piece of them exists to write anything)
    for (int i = p; i < B; i += P) {
      if (a.lens[i] > 0) continue;
      uint32_t* row = reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(a.out) +
                                                  static_cast<int64_t>(i) * a.Hq * D);
      for (int e = threadIdx.x; e < a.Hq * D / 2; e += blockDim.x) row[e] = 0u;
    }
  }
  const int Q = T == 0 ? 0 : max((T + P - 1) / P, kMinBlocksPerCta);
  const int start = p * Q;
  if (Q == 0 || start >= T) return;
  const int cnt = min(Q, T - start);
  {
    int carry = 0;
    for (int base = 0; base < B; base += blockDim.x) {
      const int i = base + threadIdx.x;
      const int v = i < B ? num_kv_blocks(a.lens[i], a.bt_stride, kTok) : 0;
      int tot;
      const int incl = block_inclusive_scan(v, s_scan, &tot) + carry;
      const int excl = incl - v;
      if (v > 0 && excl <= start && start < incl) {
        s_start_seq = i;
        s_start_off = start - excl;
      }
      carry += tot;
    }
    __syncthreads();
  }

  auto load_seq = [&](Cursor& c) {
    const int64_t len = a.lens[c.seq];
    c.nblk = num_kv_blocks(len, a.bt_stride, kTok);
    const int64_t cap = static_cast<int64_t>(c.nblk) * kTok;
    if (len > cap) report(a.status, B200_ERR_BOUNDS);  // table row too short for the context
    c.len = static_cast<int>(len < cap ? len : cap);
  };
  auto advance = [&](Cursor& c) {
    if (++c.blk < c.nblk) return;
    c.blk = 0;
    do {
      if (++c.seq >= B) {
        c.nblk = INT_MAX;
        c.len = 0;
        c.seq = B - 1;
        return;
      }
      load_seq(c);
    } while (c.nblk == 0);
  };

  Cursor L, C;
  L.seq = C.seq = s_start_seq;
  L.blk = C.blk = s_start_off;
  load_seq(L);
  C.nblk = L.nblk;
  C.len = L.len;
  int next_id = a.bt[static_cast<int64_t>(L.seq) * a.bt_stride + L.blk];

  const int h = warp;  // KV head of this warp
  const uint32_t ring = smem_u32(smem) + warp * (kStages * 2 * TILEB);
  const int64_t row_stride = static_cast<int64_t>(a.Hkv) * ROWB;  // bytes between tokens
  const uint8_t* kbase = static_cast<const uint8_t*>(a.kc) + static_cast<int64_t>(h) * ROWB;
  const uint8_t* vbase = static_cast<const uint8_t*>(a.vc) + static_cast<int64_t>(h) * ROWB;

  auto issue = [&](int stage) {
    const int id = next_id;
    const int valid = L.len - L.blk * kTok;  // tokens of this block inside the context
    const bool ok = static_cast<uint64_t>(static_cast<int64_t>(id)) <
                    static_cast<uint64_t>(a.num_blocks);
    if (!ok) report(a.status, B200_ERR_BOUNDS);
    const int64_t blk_off = ok ? static_cast<int64_t>(id) * kTok * row_stride : 0;
    const uint32_t kdst = ring + stage * (2 * TILEB), vdst = kdst + TILEB;
#pragma unroll
    for (int j = 0; j < LOADS; ++j) {
      const int idx = lane + 32 * j;
      const int t = idx / CPR, c = idx % CPR;
      const int bytes = (ok && t < valid) ? 16 : 0;
      const int64_t off = blk_off + (bytes ? t * row_stride + c * 16 : 0);
      const uint32_t d = t * ROWB + swizzle_chunk<D>(c, t) * 16;
      cp_async16(kdst + d, kbase + off, bytes);
      cp_async16(vdst + d, vbase + off, bytes);
    }
  };

  float o[NT][KS][4];
  float mrow[NT][2], lrow[NT][2];
  uint32_t qf[NT][KS][2];
  int seg_first = 0;
  bool fresh = true;

  int issued = 0;
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (issued < cnt) {
      issue(s);
      if (++issued < cnt) {
        advance(L);
        next_id = a.bt[static_cast<int64_t>(L.seq) * a.bt_stride + L.blk];
      }
    }
    cp_async_commit();
  }

  for (int j = 0; j < cnt; ++j) {
    if (issued < cnt) {
      issue((j + kStages - 1) % kStages);
      if (++issued < cnt) {
        advance(L);
        next_id = a.bt[static_cast<int64_t>(L.seq) * a.bt_stride + L.blk];
      }
    }
    cp_async_commit();

    if (fresh) {
      fresh = false;
      seg_first = C.blk;
      const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(a.q) +
                                (static_cast<int64_t>(C.seq) * a.Hq + h * G) * D;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int head = nt * 8 + g;
        mrow[nt][0] = mrow[nt][1] = -INFINITY;
        lrow[nt][0] = lrow[nt][1] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          o[nt][ks][0] = o[nt][ks][1] = o[nt][ks][2] = o[nt][ks][3] = 0.f;
          uint32_t b0 = 0, b1 = 0;
          if (head < G) {
            const uint32_t* src =
                reinterpret_cast<const uint32_t*>(qp + head * D + ks * 16 + tq * 2);
            b0 = __ldg(src);
            b1 = __ldg(src + 4);
          }
          qf[nt][ks][0] = b0;
          qf[nt][ks][1] = b1;
        }
      }
    }

    cp_async_wait<kStages - 1>();
    __syncwarp();

    const uint32_t kt = ring + (j % kStages) * (2 * TILEB), vt = kt + TILEB;
    const int valid = C.len - C.blk * kTok;

    // ---- S^T[token, head] = K . Q^T ----
    float s[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    {
      const int t = (lane & 7) + ((lane >> 3) & 1) * 8;  // matrices 0,2: tokens 0-7; 1,3: 8-15
      const int chalf = lane >> 4;                       // matrices 2,3: upper 8 of the k-step
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t af[4];
        ldmatrix_x4(af, kt + t * ROWB + swizzle_chunk<D>(2 * ks + chalf, t) * 16);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(s[nt], af, qf[nt][ks]);
      }
    }

    // ---- online softmax over the token axis (rows g and g+8 of the tile) ----
    uint32_t pb[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float x0 = s[nt][0] * a.scale_log2, x1 = s[nt][1] * a.scale_log2;
      float x2 = s[nt][2] * a.scale_log2, x3 = s[nt][3] * a.scale_log2;
      if (g >= valid) x0 = x1 = -INFINITY;
      if (g + 8 >= valid) x2 = x3 = -INFINITY;
      float mx0 = fmaxf(x0, x2), mx1 = fmaxf(x1, x3);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
      }
      const float mn0 = fmaxf(mrow[nt][0], mx0), mn1 = fmaxf(mrow[nt][1], mx1);
      const float al0 = fast_exp2(mrow[nt][0] - mn0), al1 = fast_exp2(mrow[nt][1] - mn1);
      mrow[nt][0] = mn0;
      mrow[nt][1] = mn1;
      const float p0 = fast_exp2(x0 - mn0), p1 = fast_exp2(x1 - mn1);
      const float p2 = fast_exp2(x2 - mn0), p3 = fast_exp2(x3 - mn1);
      lrow[nt][0] = lrow[nt][0] * al0 + p0 + p2;
      lrow[nt][1] = lrow[nt][1] * al1 + p1 + p3;
      pb[nt][0] = movmatrix_trans(pack_bf16x2(p0, p1));
      pb[nt][1] = movmatrix_trans(pack_bf16x2(p2, p3));
#pragma unroll
      for (int mt = 0; mt < KS; ++mt) {
        o[nt][mt][0] *= al0;
        o[nt][mt][1] *= al1;
        o[nt][mt][2] *= al0;
        o[nt][mt][3] *= al1;
      }
    }

    // ---- O^T[d, head] += V^T . P^T ----
    {
      const int t = (lane & 7) + (lane >> 4) * 8;  // matrices 0,1: tokens 0-7; 2,3: tokens 8-15
      const int chalf = (lane >> 3) & 1;           // matrices 1,3: upper 8 of the 16 d values
#pragma unroll
      for (int mt = 0; mt < KS; ++mt) {
        uint32_t af[4];
        ldmatrix_x4_trans(af, vt + t * ROWB + swizzle_chunk<D>(2 * mt + chalf, t) * 16);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(o[nt][mt], af, pb[nt]);
      }
    }
    __syncwarp();  // the stage may be refilled by the next trip

    const bool seq_end = (C.blk == C.nblk - 1);
    if (seq_end || j == cnt - 1) {
      fresh = true;
      const bool whole = seq_end && seg_first == 0;
      const int slot = seg_first > 0 ? 0 : 1;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float l0 = lrow[nt][0], l1 = lrow[nt][1];
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          l0 += __shfl_xor_sync(0xffffffffu, l0, off);
          l1 += __shfl_xor_sync(0xffffffffu, l1, off);
        }
        const int head0 = nt * 8 + tq * 2;
        if (whole) {
          const float i0 = 1.f / l0, i1 = 1.f / l1;
          __nv_bfloat16* op = static_cast<__nv_bfloat16*>(a.out) +
                              (static_cast<int64_t>(C.seq) * a.Hq + h * G) * D;
#pragma unroll
          for (int mt = 0; mt < KS; ++mt) {
            const int d = mt * 16 + g;
            if (head0 < G) {
              op[head0 * D + d] = __float2bfloat16_rn(o[nt][mt][0] * i0);
              op[head0 * D + d + 8] = __float2bfloat16_rn(o[nt][mt][2] * i0);
            }
            if (head0 + 1 < G) {
              op[(head0 + 1) * D + d] = __float2bfloat16_rn(o[nt][mt][1] * i1);
              op[(head0 + 1) * D + d + 8] = __float2bfloat16_rn(o[nt][mt][3] * i1);
            }
          }
        } else {
          const int64_t pslot = static_cast<int64_t>(p) * 2 + slot;
          float* po = a.part_o + (pslot * a.Hq + h * G) * D;
          float* pml = a.part_ml + (pslot * a.Hq + h * G) * 2;
#pragma unroll
          for (int mt = 0; mt < KS; ++mt) {
            const int d = mt * 16 + g;
            if (head0 < G) {
              po[head0 * D + d] = o[nt][mt][0];
              po[head0 * D + d + 8] = o[nt][mt][2];
            }
            if (head0 + 1 < G) {
              po[(head0 + 1) * D + d] = o[nt][mt][1];
              po[(head0 + 1) * D + d + 8] = o[nt][mt][3];
            }
          }
          if (g == 0) {
            if (head0 < G) {
              pml[head0 * 2] = mrow[nt][0];
              pml[head0 * 2 + 1] = l0;
            }
            if (head0 + 1 < G) {
              pml[(head0 + 1) * 2] = mrow[nt][1];
              pml[(head0 + 1) * 2 + 1] = l1;
            }
          }
        }
      }
      if (a.counters == nullptr) {
        if (seq_end && warp == 0 && lane == 0) {
          const int seq_start_flat = start + j - C.blk;
          a.seq_info[2 * C.seq] = whole ? -1 : seq_start_flat / Q;
          a.seq_info[2 * C.seq + 1] = whole ? -1 : p;
        }
      } else if (!whole) {
        // this warp's piece of (sequence, KV head) is in the workspace: publish it, count the arrival, and
        // merge if every other piece has arrived already
        const int seq_start_flat = start + j - C.blk;
        const int first = seq_start_flat / Q;
        const int np = (seq_start_flat + C.nblk - 1) / Q - first + 1;
        __threadfence();
        __syncwarp();
        int32_t* cnt = a.counters + static_cast<int64_t>(C.seq) * a.Hkv + h;
        int arrived = 0;
        if (lane == 0) arrived = atomicAdd(cnt, 1);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived == np - 1) {
          __threadfence();
          merge_split_sequence<D>(a, C.seq, h, G, first, np, lane);
          if (lane == 0) *cnt = 0;   // ready for the next launch
        }
      }
    }
    if (j + 1 < cnt) advance(C);
  }
  cp_async_wait<0>();
}

// Merges the partial results of sequences that were cut across CTAs; zero-fills rows whose
// context is empty.  One CTA per sequence.  Most sequences are not cut and leave at once; for the
// others the per-head weights 2^(m_p - M) / L are computed once into shared memory, then every
// thread sums its float4 columns over the parts with all loads of a trip independent.
constexpr int kCombineThreads = 256;
constexpr int kCombineMaxParts = 8;  // parts whose weights are kept in shared memory per trip

__global__ void __launch_bounds__(kCombineThreads)
paged_decode_combine_kernel(const DecodeArgs a) {
  extern __shared__ float s_w[];  // [kCombineMaxParts][Hq]
  // launched early (programmatic dependent of the attention kernel): everything below reads its results
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const int i = blockIdx.x;
  const int n = a.Hq * a.D;
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(a.out) + static_cast<int64_t>(i) * n;
  const int64_t len = a.lens[i];
  const int first = a.seq_info[2 * i], last = a.seq_info[2 * i + 1];
  if (len <= 0) {
    for (int e = threadIdx.x; e < n; e += kCombineThreads) op[e] = __float2bfloat16_rn(0.f);
    return;
  }
  if (first < 0) return;
  const int np = last - first + 1;
  auto slot_of = [&](int p) -> int64_t {
    return static_cast<int64_t>(first + p) * 2 + (p == 0 ? 1 : 0);
  };
  // per-head maximum and normaliser over all parts (np is small: a sequence of L tokens spans
  // about L / (tokens per CTA) + 1 CTAs)
  float* s_M = s_w + kCombineMaxParts * a.Hq;  // [Hq]
  float* s_inv = s_M + a.Hq;                   // [Hq]
  for (int h = threadIdx.x; h < a.Hq; h += kCombineThreads) {
    float M = -INFINITY;
    for (int p = 0; p < np; ++p) M = fmaxf(M, a.part_ml[(slot_of(p) * a.Hq + h) * 2]);
    float L = 0.f;
    for (int p = 0; p < np; ++p) {
      const float2 ml = *reinterpret_cast<const float2*>(a.part_ml + (slot_of(p) * a.Hq + h) * 2);
      L += exp2f(ml.x - M) * ml.y;
    }
    s_M[h] = M;
    s_inv[h] = 1.f / L;
  }
  __syncthreads();
  constexpr int kVec = 4;
  const int nvec = n / kVec;  // D is a multiple of 16 on this path
  float4 acc[4];
  // every thread owns up to 4 float4 columns (n <= 16 * 256 * 4 covers Hq*D <= 16384)
  for (int base = 0; base < nvec; base += kCombineThreads * 4) {
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p0 = 0; p0 < np; p0 += kCombineMaxParts) {
      const int pc = min(kCombineMaxParts, np - p0);
      __syncthreads();
      for (int t = threadIdx.x; t < pc * a.Hq; t += kCombineThreads) {
        const int p = p0 + t / a.Hq, h = t % a.Hq;
        s_w[t] = exp2f(a.part_ml[(slot_of(p) * a.Hq + h) * 2] - s_M[h]) * s_inv[h];
      }
      __syncthreads();
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int vi = base + u * kCombineThreads + threadIdx.x;
        if (vi < nvec) {
          const int head = (vi * kVec) / a.D;
          for (int p = 0; p < pc; ++p) {
            const float4 x =
                *reinterpret_cast<const float4*>(a.part_o + slot_of(p0 + p) * n + vi * kVec);
            const float w = s_w[p * a.Hq + head];
            acc[u].x += w * x.x;
            acc[u].y += w * x.y;
            acc[u].z += w * x.z;
            acc[u].w += w * x.w;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int vi = base + u * kCombineThreads + threadIdx.x;
      if (vi < nvec) {
        uint2 packed;
        packed.x = pack_bf16x2(acc[u].x, acc[u].y);
        packed.y = pack_bf16x2(acc[u].z, acc[u].w);
        *reinterpret_cast<uint2*>(op + vi * kVec) = packed;
      }
    }
  }
}

// The combine follows the attention kernel in the stream and reads only what that kernel wrote: as a
// programmatic dependent its launch and CTA placement overlap the attention kernel's tail.
int launch_combine(const DecodeArgs& a, int batch, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(batch);
  cfg.blockDim = dim3(kCombineThreads);
  cfg.dynamicSmemBytes = (kCombineMaxParts + 2) * a.Hq * sizeof(float);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, paged_decode_combine_kernel, a) != cudaSuccess) {
    cudaGetLastError();
    return B200_ERR_LAUNCH;
  }
  return launch_result();
}

}  // namespace

int decode_combine_launch(const CombineArgs& c, cudaStream_t s) {
  DecodeArgs a{};
  a.out = c.out;
  a.lens = c.lens;
  a.part_o = const_cast<float*>(c.part_o);
  a.part_ml = const_cast<float*>(c.part_ml);
  a.seq_info = const_cast<int32_t*>(c.seq_info);
  a.batch = c.batch;
  a.Hq = c.H;
  a.D = c.D;
  return launch_combine(a, c.batch, s);
}

namespace {

// ---------------------------------------------------------------------------------------------
// Generic path: grid (batch, Hq), 4 warps; warp w takes tokens w, w+4, ...; a lane owns the
// head-dim elements lane, lane+32, ...
// ---------------------------------------------------------------------------------------------
constexpr int kSimpleWarps = 4;
constexpr int kSimpleMaxPerLane = 8;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(kSimpleWarps * 32) paged_decode_simple_kernel(const DecodeArgs a) {
  __shared__ float s_m[kSimpleWarps], s_l[kSimpleWarps];
  __shared__ float s_acc[kSimpleWarps][kSimpleMaxPerLane * 32];
  const int seq = blockIdx.x, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = a.D, G = a.Hq / a.Hkv, kvh = head / G;
  T* op = static_cast<T*>(a.out) + (static_cast<int64_t>(seq) * a.Hq + head) * D;
  int64_t len64 = a.lens[seq];
  if (len64 <= 0) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) op[d] = from_float<T>(0.f);
    return;
  }
  const int64_t cap = a.bt_stride * a.bs;
  if (len64 > cap) {
    report(a.status, B200_ERR_BOUNDS);
    len64 = cap;
  }
  const int len = static_cast<int>(len64);
  const T* qp = static_cast<const T*>(a.q) + (static_cast<int64_t>(seq) * a.Hq + head) * D;
  float qv[kSimpleMaxPerLane], acc[kSimpleMaxPerLane];
#pragma unroll
  for (int k = 0; k < kSimpleMaxPerLane; ++k) {
    const int d = lane + 32 * k;
    qv[k] = d < D ? to_float<T>(qp[d]) : 0.f;
    acc[k] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const T* kc = static_cast<const T*>(a.kc);
  const T* vc = static_cast<const T*>(a.vc);
  for (int t = warp; t < len; t += kSimpleWarps) {
    const int id = a.bt[static_cast<int64_t>(seq) * a.bt_stride + t / a.bs];
    if (static_cast<uint64_t>(static_cast<int64_t>(id)) >= static_cast<uint64_t>(a.num_blocks)) {
      report(a.status, B200_ERR_BOUNDS);
      continue;
    }
    const int64_t row = ((static_cast<int64_t>(id) * a.bs + t % a.bs) * a.Hkv + kvh) * D;
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < kSimpleMaxPerLane; ++k) {
      const int d = lane + 32 * k;
      if (d < D) dot += qv[k] * to_float<T>(kc[row + d]);
    }
    dot = warp_sum(dot) * a.scale_log2;
    const float mn = fmaxf(m, dot);
    const float al = exp2f(m - mn), pw = exp2f(dot - mn);
    l = l * al + pw;
#pragma unroll
    for (int k = 0; k < kSimpleMaxPerLane; ++k) {
      const int d = lane + 32 * k;
      if (d < D) acc[k] = acc[k] * al + pw * to_float<T>(vc[row + d]);
    }
    m = mn;
  }
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
#pragma unroll
  for (int k = 0; k < kSimpleMaxPerLane; ++k) s_acc[warp][lane + 32 * k] = acc[k];
  __syncthreads();
  float M = -INFINITY;
  for (int w = 0; w < kSimpleWarps; ++w) M = fmaxf(M, s_m[w]);
  float Lsum = 0.f;
  float wgt[kSimpleWarps];
  for (int w = 0; w < kSimpleWarps; ++w) {
    wgt[w] = s_m[w] == -INFINITY ? 0.f : exp2f(s_m[w] - M);
    Lsum += wgt[w] * s_l[w];
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = 0.f;
    for (int w = 0; w < kSimpleWarps; ++w) v += wgt[w] * s_acc[w][d];
    op[d] = from_float<T>(Lsum > 0.f ? v / Lsum : 0.f);
  }
}

struct FastPlan {
  bool ok;
  int nt;
  int threads;
  size_t smem;
  int ctas_per_sm;
};

FastPlan fast_plan(int Hq, int Hkv, int D, int bs, int dtype) {
  FastPlan pl{};
  pl.ok = false;
  if (dtype != B200_DTYPE_BF16 || bs != kTok) return pl;
  if (D != 32 && D != 64 && D != 128) return pl;
  if (Hkv <= 0 || Hkv > kMaxFastThreads / 32 || Hq % Hkv != 0) return pl;
  const int G = Hq / Hkv;
  if (G > 16) return pl;
  pl.nt = G > 8 ? 2 : 1;
  pl.threads = Hkv * 32;
  pl.smem = static_cast<size_t>(Hkv) * kStages * 2 * kTok * D * 2;
  const size_t budget = 220 * 1024;
  if (pl.smem > budget) return pl;
  int c = static_cast<int>(budget / (pl.smem + 1024));
  const int by_threads = 2048 / pl.threads;
  if (c > by_threads) c = by_threads;
  if (c > 8) c = 8;
  if (c < 1) c = 1;
  pl.ctas_per_sm = c;
  pl.ok = true;
  return pl;
}

template <int D, int NT>
int launch_fast(const DecodeArgs& a, const FastPlan& pl, int grid, cudaStream_t s) {
  // per-device "shared-memory limit raised" flags: written without a lock; two host threads racing here both
  // make the same idempotent cudaFuncSetAttribute call and both store true
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(paged_decode_bf16_kernel<D, NT>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             220 * 1024) != cudaSuccess)
      return B200_ERR_LAUNCH;
    configured[dev] = true;
  }
  paged_decode_bf16_kernel<D, NT><<<grid, pl.threads, pl.smem, s>>>(a);
  return launch_result();
}

}  // namespace
}  // namespace b200

extern "C" size_t b200_paged_decode_gqa_workspace_bytes(int32_t batch, int32_t num_q_heads,
                                                        int32_t num_kv_heads, int32_t head_dim,
                                                        int32_t dtype) {
  using namespace b200;
  if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0) return 0;
  const FastPlan pl = fast_plan(num_q_heads, num_kv_heads, head_dim, kTok, dtype);
  if (!pl.ok) return 256;
  int sms = sm_count_cached();
  if (sms <= 0) sms = 148;
  const size_t grid = static_cast<size_t>(sms) * pl.ctas_per_sm;
  size_t bytes = kDecodeCounterBytes;
  bytes += align256(grid * 2 * num_q_heads * head_dim * sizeof(float));
  bytes += align256(grid * 2 * num_q_heads * 2 * sizeof(float));
  bytes += align256(static_cast<size_t>(batch) * 2 * sizeof(int32_t));
  return bytes;
}

extern "C" int b200_paged_decode_gqa(const void* q, const void* k_cache, const void* v_cache,
                                     void* out, const int32_t* block_tables, int64_t bt_stride,
                                     const int64_t* context_lens, int32_t batch,
                                     int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                     int32_t block_size, int64_t num_blocks, float scale,
                                     void* workspace, size_t workspace_bytes, int32_t dtype,
                                     int32_t* status, void* stream) {
  using namespace b200;
  if (batch < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || block_size <= 0 ||
      num_blocks < 0 || bt_stride <= 0)
    return B200_ERR_ARG;
  if (num_q_heads % num_kv_heads != 0) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (batch == 0) return B200_OK;
  if (!q || !out || !block_tables || !context_lens) return B200_ERR_ARG;
  if (num_blocks > 0 && (!k_cache || !v_cache)) return B200_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  DecodeArgs a{};
  a.q = q;
  a.kc = k_cache;
  a.vc = v_cache;
  a.out = out;
  a.bt = block_tables;
  a.bt_stride = bt_stride;
  a.lens = context_lens;
  a.batch = batch;
  a.Hq = num_q_heads;
  a.Hkv = num_kv_heads;
  a.D = head_dim;
  a.bs = block_size;
  a.num_blocks = num_blocks;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;

  const FastPlan pl = fast_plan(num_q_heads, num_kv_heads, head_dim, block_size, dtype);
  const bool fast = pl.ok && aligned16(q) && aligned16(k_cache) && aligned16(v_cache);
  if (fast) {
    const int sms = sm_count_cached();
    if (sms <= 0) return B200_ERR_NO_DEVICE;
    const size_t need = b200_paged_decode_gqa_workspace_bytes(batch, num_q_heads, num_kv_heads,
                                                              head_dim, dtype);
    if (!workspace || workspace_bytes < need) return B200_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return B200_ERR_ALIGN;
    const size_t grid = static_cast<size_t>(sms) * pl.ctas_per_sm;
    uint8_t* w = static_cast<uint8_t*>(workspace);
    // Which merge: inside the launch for small batches, where a step is a chain of short kernels and one launch
    // fewer shortens it (one 700-token sequence at 16/4 heads x 64: 9.1 against 10.2 us per call); a separate
    // kernel, launched as a programmatic dependent, for large ones, where its 256 threads per sequence merge in
    // parallel while the in-launch merges would lengthen the tail of the streaming CTAs (256 sequences of
    // 200-1300 tokens: 41.1 against 43.6 us per call).
#if defined(B200_DECODE_SEPARATE_MERGE)     // build-time switches for A/B timing of the two forms
    const bool fused_merge = false;
#elif defined(B200_DECODE_FUSED_MERGE)
    const bool fused_merge = static_cast<int64_t>(batch) * num_kv_heads <= kDecodeCounters;
#else
    const bool fused_merge = batch <= kFusedMergeMaxBatch;
#endif
    a.counters = fused_merge ? reinterpret_cast<int32_t*>(w) : nullptr;
    w += kDecodeCounterBytes;
    a.part_o = reinterpret_cast<float*>(w);
    w += align256(grid * 2 * num_q_heads * head_dim * sizeof(float));
    a.part_ml = reinterpret_cast<float*>(w);
    w += align256(grid * 2 * num_q_heads * 2 * sizeof(float));
    a.seq_info = reinterpret_cast<int32_t*>(w);
    int rc;
    const int gi = static_cast<int>(grid);
    if (head_dim == 128)
      rc = pl.nt == 1 ? launch_fast<128, 1>(a, pl, gi, s) : launch_fast<128, 2>(a, pl, gi, s);
    else if (head_dim == 64)
      rc = pl.nt == 1 ? launch_fast<64, 1>(a, pl, gi, s) : launch_fast<64, 2>(a, pl, gi, s);
    else
      rc = pl.nt == 1 ? launch_fast<32, 1>(a, pl, gi, s) : launch_fast<32, 2>(a, pl, gi, s);
    if (rc != B200_OK || fused_merge) return rc;
    return launch_combine(a, batch, s);
  }

  if (head_dim > kSimpleMaxPerLane * 32) return B200_ERR_UNSUPPORTED;
  dim3 grid(batch, num_q_heads);
  if (dtype == B200_DTYPE_F32)
    paged_decode_simple_kernel<float><<<grid, kSimpleWarps * 32, 0, s>>>(a);
  else
    paged_decode_simple_kernel<__nv_bfloat16><<<grid, kSimpleWarps * 32, 0, s>>>(a);
  return launch_result();
}

// ---------------------------------------------------------------------------------------------
// Paged GQA decode for callers that cannot allocate device memory.
//
// Some hosts of this library hold no allocator they may call on the decode path: an engine that
// has handed the whole GPU to its KV pool and keeps nothing back for scratch, a plugin loaded into
// a server whose memory is budgeted by someone else, or a step replayed from a pre-recorded
// command list where a cudaMalloc would serialise the device.  For them the split-context scratch
// lives in a fixed device array that is part of the library image: every GPU that loads the
// library holds kStaticScratchBytes of it until the process exits, and problems whose scratch
// would not fit are refused instead of allocated for.
//
// The array's name is only a device address inside device code.  On the host it is a stand-in
// symbol, so the device address is looked up once per device with cudaGetSymbolAddress (with that
// device current) and cached; that first call per device does the lookup and should therefore be
// made before any stream capture starts.  All calls share the one array and it keeps whatever the
// previous call left in it.  Only its first 256 KiB (the arrival counters of split sequences) must be zero
// when a call starts: the array is zero when the library is loaded and every call returns the counters it
// touched to zero, so nothing has to be cleared between calls; the partial results behind them are written
// before they are read within one call.  Two calls that overlap on the GPU (different streams, or different
// host threads) would corrupt each other's counters and partial results.
// ---------------------------------------------------------------------------------------------
namespace b200 {
namespace {

constexpr size_t kStaticScratchBytes = B200_STATIC_SCRATCH_BYTES;  // 8 MiB per GPU
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

int static_scratch_address(void** out) {
  // per-device cache of the symbol's address: written without a lock; racing host threads look up and
  // store the same value
  static void* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200_ERR_NO_DEVICE;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_decode_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return B200_ERR_LAUNCH;
    }
    cached[dev] = p;
  }
  *out = cached[dev];
  return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" int b200_paged_decode_gqa_static(const void* q, const void* k_cache,
                                            const void* v_cache, void* out,
                                            const int32_t* block_tables, int64_t bt_stride,
                                            const int64_t* context_lens, int32_t batch,
                                            int32_t num_q_heads, int32_t num_kv_heads,
                                            int32_t head_dim, int32_t block_size,
                                            int64_t num_blocks, float scale, int32_t dtype,
                                            int32_t* status, void* stream) {
  using namespace b200;
  if (batch > 0 && num_q_heads > 0 && num_kv_heads > 0 && head_dim > 0 && block_size > 0) {
    // refuse only what would really use more scratch than the array holds: the same test the callee makes
    // before it takes the split-context path (other shapes run the one-CTA-per-head kernel, which needs none)
    const FastPlan pl = fast_plan(num_q_heads, num_kv_heads, head_dim, block_size, dtype);
    const bool fast = pl.ok && aligned16(q) && aligned16(k_cache) && aligned16(v_cache);
    if (fast && b200_paged_decode_gqa_workspace_bytes(batch, num_q_heads, num_kv_heads, head_dim, dtype) >
                    kStaticScratchBytes)
      return B200_ERR_TOO_LARGE;
  }
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != B200_OK) return rc;
  return b200_paged_decode_gqa(q, k_cache, v_cache, out, block_tables, bt_stride, context_lens,
                               batch, num_q_heads, num_kv_heads, head_dim, block_size, num_blocks,
                               scale, scratch, kStaticScratchBytes, dtype, status, stream);
}
