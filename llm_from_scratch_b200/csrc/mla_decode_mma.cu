// MLA latent-cache decode, bf16, tensor-core path (kv_lora_rank 512, rope_dim 64, <= 16 heads,
// block size 16).
//
// Every cached token is one 1152-byte latent row [c (512) | pe (64)] shared by all heads, so a
// 16-token block is one contiguous 18 KiB segment.  The heads of a sequence are the M = 16 rows
// of mma.sync m16n8k16:  S[head, token] = Q[head, 576] . row^T  and  O[head, 512] += P . c.
// At 16 heads that is 30 flop per byte read — HBM-bound, but far more arithmetic than FMA units
// sustain, which is the only reason the contractions sit on the tensor cores.
//
// Work split: as in the GQA decode kernel the flat list of all KV blocks is cut into equal
// contiguous ranges, one per persistent CTA (one CTA per SM); sequences cut across CTAs are merged
// by the shared combine kernel.  A CTA consumes its range in groups of four blocks (64 tokens) held in
// a two-group shared-memory ring (72 KiB per group), so one group is in flight while the previous one
// is being used.  The ring is filled by a 17th warp with TMA: a block is ONE box of a rank-3 view of the
// pool (64 columns x 16 tokens x 9 slabs, strides 2 B / 1152 B / 128 B), written slab by slab with the
// 128-byte swizzle that ldmatrix wants and counted on an mbarrier per ring half; named barriers hand a
// half back to the producer.  (With 16-byte cp.async copies issued by the compute warps themselves, 1200
// of the 4300 clocks of a group went into pushing 4608 copies through the load/store unit.)
// The 16 compute warps then run, per group:
//   phase 1  warp w: tokens 16*(w&3)..+15, quarter (w>>2) of the 576-wide contraction -> partial S
//            (its Q fragments stay in registers for the whole sequence segment)
//   phase 2  warp h: sums the quarters of head h, scale, mask, online softmax (fp32, log2 domain), P -> smem
//   phase 3  warp w: O[:, 32w..32w+31] += P . c
#include <cuda.h>

#include "decode_common.cuh"
#include "umma.cuh"

namespace b200 {
namespace {

constexpr int kTok = 16;
constexpr int R = 512, DR = 64, ROW = R + DR;     // latent row, elements
constexpr int ROWB = ROW * 2;                     // 1152 bytes
constexpr int CPR = ROWB / 16;                    // 72 chunks per row
constexpr int BLKB = kTok * ROWB;                 // 18432 bytes per block
constexpr int GROUP = 4;                          // blocks per group (64 tokens)
constexpr int GT = GROUP * kTok;                  // 64
constexpr int kCompute = 512;                     // 16 compute warps: 4 token blocks x 4 k-quarters
constexpr int kProducers = 32;                    // one warp that only fills the ring (TMA)
constexpr int kThreads = kCompute + kProducers;
constexpr int KSTEPS = ROW / 16;                  // 36
constexpr int QUART_K = KSTEPS / 4;               // 9 k-steps per warp in phase 1
constexpr int SP_STRIDE = GT + 8;                 // padded row of the partial-S buffer (floats)
constexpr int SLABS = ROW / 64;                   // 9 slabs of 64 columns (128 bytes) per block

// shared memory map (bytes)
constexpr int OFF_RING = 0;                                   // 2 groups x 4 blocks
constexpr int OFF_Q = OFF_RING + 2 * GROUP * BLKB;            // 16 x 1152
constexpr int OFF_SPART = OFF_Q + 16 * ROWB;                  // [4][16][72] fp32
constexpr int OFF_P = OFF_SPART + 4 * 16 * SP_STRIDE * 4;     // [16][64] bf16
constexpr int OFF_STAT = OFF_P + 16 * GT * 2;                 // alpha[16], m[16], l[16] fp32
constexpr int OFF_SCAN = OFF_STAT + 3 * 16 * 4;               // 34 ints
constexpr int OFF_BAR = (OFF_SCAN + 34 * 4 + 15) & ~15;        // full[2] mbarriers
constexpr int SMEM_BYTES = OFF_BAR + 2 * 8 + 8 + 1024;       // + slack to align the ring to 1024 bytes

struct MlaArgs {
  const __nv_bfloat16* q_abs;   // [B, H, 512]
  const __nv_bfloat16* q_rope;  // [B, H, 64]
  const uint8_t* lat;           // [num_blocks, 16, 576] bf16
  __nv_bfloat16* out;           // [B, H, 512]
  const int32_t* bt;
  int64_t bt_stride;
  const int64_t* lens;
  int batch, H;
  int64_t num_blocks;
  float scale_log2;
  float* part_o;
  float* part_ml;
  int32_t* seq_info;
  int32_t* status;
};

struct Cursor {
  int seq, blk, nblk, len, remaining;
};
struct Group {
  int seq, blk0, n, len, nblk;
  int ids[4];   // physical block ids, fetched when the group is formed (well before they are used)
};

__device__ __forceinline__ int swz72(int c, int row) { return c ^ (row & 7); }

// byte offset of 16-byte chunk c (0..71) of token row r (0..15) inside a block of the ring: 9 slabs of
// [16 rows x 128 B], chunks XOR-swizzled with the row as TMA's 128-byte swizzle writes them
__device__ __forceinline__ int lat_off(int r, int c) {
  return (c >> 3) * (kTok * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}

// Named barriers: 1 = the compute warps among themselves; 2 + half = "ring half filled" (producers arrive,
// compute warps wait); 4 + half = "ring half free" (compute warps arrive, producers wait).
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kCompute) : "memory"); }
__device__ __forceinline__ void named_sync(int id) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "n"(kThreads) : "memory");
}
__device__ __forceinline__ void named_arrive(int id) {
  asm volatile("bar.arrive %0, %1;\n" ::"r"(id), "n"(kThreads) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
mla_decode_mma_kernel(const MlaArgs a, const __grid_constant__ CUtensorMap tm_lat) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  float* s_part = reinterpret_cast<float*>(smem + OFF_SPART);
  float* s_alpha = reinterpret_cast<float*>(smem + OFF_STAT);
  float* s_m = s_alpha + 16;
  float* s_l = s_alpha + 32;
  int* s_scan = reinterpret_cast<int*>(smem + OFF_SCAN);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int B = a.batch, H = a.H, p = blockIdx.x;
  // the combine kernel is a programmatic dependent: its CTAs may be placed while this grid runs
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

  const CtaRange rg = plan_cta_range(a.lens, B, a.bt_stride, kTok, s_scan);
  if (rg.cnt == 0) return;
  auto full_bar = [&](int half) -> uint32_t { return sbase + OFF_BAR + half * 8; };
  // Ring rows that no copy has written (blocks past the end of a group, at first) are read by phase 3
  // with weight 0: they must hold finite numbers, so the ring starts as zeros.
  for (int i = tid; i < 2 * GROUP * BLKB / 16; i += kThreads)
    reinterpret_cast<uint4*>(smem + OFF_RING)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (tid == 0) {
    umma::mbar_init(full_bar(0), GROUP);        // one arrival (with its byte count) per block of the group
    umma::mbar_init(full_bar(1), GROUP);
    umma::mbar_init_fence();
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tm_lat)) : "memory");
  }
  umma::fence_async_proxy();
  __syncthreads();

  auto load_seq = [&](Cursor& c) {
    const int64_t len = a.lens[c.seq];
    c.nblk = num_kv_blocks(len, a.bt_stride, kTok);
    const int64_t cap = static_cast<int64_t>(c.nblk) * kTok;
    if (len > cap) report(a.status, B200_ERR_BOUNDS);
    c.len = static_cast<int>(len < cap ? len : cap);
  };
  // next group of up to four consecutive blocks of one sequence inside this CTA's range
  auto next_group = [&](Cursor& c, bool with_ids) -> Group {
    Group gr;
    gr.seq = c.seq;
    gr.blk0 = c.blk;
    gr.len = c.len;
    gr.nblk = c.nblk;
    gr.n = min(GROUP, min(c.nblk - c.blk, c.remaining));
#pragma unroll
    for (int b = 0; b < GROUP; ++b)
      gr.ids[b] = (with_ids && b < gr.n)
                      ? __ldg(a.bt + static_cast<int64_t>(gr.seq) * a.bt_stride + gr.blk0 + b)
                      : -1;
    c.blk += gr.n;
    c.remaining -= gr.n;
    if (c.blk >= c.nblk && c.remaining > 0) {
      c.blk = 0;
      do {
        ++c.seq;
        load_seq(c);
      } while (c.nblk == 0 && c.seq + 1 < B);
    }
    return gr;
  };

  Cursor L, C;
  L.seq = rg.start_seq;
  L.blk = rg.start_off;
  L.remaining = rg.cnt;
  load_seq(L);
  C = L;

  // fills ring half `half` with the blocks of a group: one rank-3 TMA box per block (64 columns x 16
  // tokens x 9 slabs), each counted on the half's barrier; a missing or out-of-pool block only arrives
  auto issue_group = [&](const Group& gr, int half) {
    const uint32_t bar = full_bar(half);
#pragma unroll
    for (int b = 0; b < GROUP; ++b) {
      bool load = false;
      int id = 0;
      if (b < gr.n) {
        id = gr.ids[b];
        load = static_cast<uint64_t>(static_cast<int64_t>(id)) < static_cast<uint64_t>(a.num_blocks);
        if (!load) report(a.status, B200_ERR_BOUNDS);
      }
      if (load) {
        umma::mbar_expect_tx(bar, BLKB);
        umma::tma_load_3d(sbase + OFF_RING + (half * GROUP + b) * BLKB, &tm_lat, 0, id * kTok, 0, bar);
      } else {
        umma::mbar_arrive(bar);
      }
    }
  };
  int groups_total = 0;
  {
    // number of groups in the range (walk a copy of the cursor; a few iterations)
    Cursor t = L;
    while (t.remaining > 0) {
      next_group(t, false);
      ++groups_total;
    }
  }
  if (warp >= kCompute / 32) {
    // =============================== producer ===============================
    // One warp does nothing but fill the ring; the compute warps used to spend ~1200 clocks per group
    // pushing 4608 16-byte cp.async copies through the load/store unit.
    for (int g = 0; g < groups_total; ++g) {
      const int half = g & 1;
      if (g >= 2) named_sync(4 + half);          // the compute warps are done with group g - 2
      const Group gr = next_group(L, true);
      if (lane == 0) issue_group(gr, half);
      __syncwarp();
    }
    return;
  }

  float o[4][4];
  uint32_t qf[QUART_K][4];
  bool fresh = true, load_q = false;
  int seg_first = 0;
  int flat = rg.start;   // flat index of the first block of the current group

  for (int gi = 0; gi < groups_total; ++gi) {
    const Group gr = next_group(C, false);
    const int half = gi & 1;
    const uint32_t ring = sbase + OFF_RING + half * GROUP * BLKB;
    // ---- new segment: stage Q = [q_abs | q_rope] (rows >= H are zero), reset the running state
    if (fresh) {
      fresh = false;
      seg_first = gr.blk0;
      for (int idx = tid; idx < 16 * CPR; idx += kCompute) {
        const int r = idx / CPR, c = idx - r * CPR;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (r < H) {
          const int64_t row = static_cast<int64_t>(gr.seq) * H + r;
          val = c < R / 8 ? __ldg(reinterpret_cast<const uint4*>(a.q_abs + row * R) + c)
                          : __ldg(reinterpret_cast<const uint4*>(a.q_rope + row * DR) + (c - R / 8));
        }
        *reinterpret_cast<uint4*>(smem + OFF_Q + r * ROWB + swz72(c, r) * 16) = val;
      }
#pragma unroll
      for (int n = 0; n < 4; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
      load_q = true;
      if (tid < 16) {
        s_m[tid] = -INFINITY;
        s_l[tid] = 0.f;
      }
    }
    {
      // the group has landed (one lane per warp polls, bounded); the barrier makes the verdict uniform and
      // orders the Q staging above among the compute warps
      int never = 0, ok = 1;
      if (lane == 0) ok = umma::mbar_wait(full_bar(half), (gi >> 1) & 1, &never);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      {
        // rows of the group's last block past the end of the context hold whatever the pool has there:
        // zero them (their softmax weight is 0, but 0 * NaN is not)
        const int valid = min(gr.len - gr.blk0 * kTok, gr.n * kTok);
        const int extra = gr.n * kTok - valid;               // 0..15 rows, all in block gr.n - 1
        for (int idx = tid; idx < extra * CPR; idx += kCompute) {
          const int r = valid % kTok + idx / CPR, c = idx % CPR;
          *reinterpret_cast<uint4*>(smem + OFF_RING + (half * GROUP + gr.n - 1) * BLKB + lat_off(r, c)) =
              make_uint4(0u, 0u, 0u, 0u);
        }
        if (extra > 0) umma::fence_async_proxy();            // before the copy that refills this half
      }
      int bad;
      asm volatile("{\n.reg .pred p, q;\nsetp.eq.s32 p, %1, 0;\nbar.red.or.pred q, 1, %2, p;\nselp.s32 %0, 1, 0, q;\n}\n"
                   : "=r"(bad) : "r"(ok), "n"(kCompute) : "memory");
      // a timeout is reported and the group is computed on whatever is there: leaving the loop would
      // strand the producer warps at their barrier
      if (bad && tid == 0) report(a.status, B200_ERR_TIMEOUT);
    }

    // ---- phase 1: partial S[head, token] over this warp's 16 tokens and a quarter of the 576 columns
    {
      const int t4 = warp & 3, kq = warp >> 2;
      if (load_q) {
        load_q = false;
        const uint32_t sQ = sbase + OFF_Q;
        const int rq = (lane & 7) + ((lane >> 3) & 1) * 8, chq = lane >> 4;   // A operand: Q rows
#pragma unroll
        for (int i = 0; i < QUART_K; ++i)
          ldmatrix_x4(qf[i], sQ + rq * ROWB + swz72(2 * (kq * QUART_K + i) + chq, rq) * 16);
      }
      float sacc[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
      const uint32_t blk = ring + t4 * BLKB;
      const int rb = (lane & 7) + (lane >> 4) * 8, chb = (lane >> 3) & 1;   // B operand: token rows
#pragma unroll
      for (int i = 0; i < QUART_K; ++i) {
        uint32_t bf[4];
        ldmatrix_x4(bf, blk + lat_off(rb, 2 * (kq * QUART_K + i) + chb));
        const uint32_t b0[2] = {bf[0], bf[1]}, b1[2] = {bf[2], bf[3]};
        mma_bf16_16816(sacc[0], qf[i], b0);
        mma_bf16_16816(sacc[1], qf[i], b1);
      }
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int token = t4 * 16 + n * 8 + tq * 2;
        *reinterpret_cast<float2*>(s_part + (kq * 16 + g) * SP_STRIDE + token) = make_float2(sacc[n][0], sacc[n][1]);
        *reinterpret_cast<float2*>(s_part + (kq * 16 + g + 8) * SP_STRIDE + token) = make_float2(sacc[n][2], sacc[n][3]);
      }
    }
    compute_sync();

    // ---- phase 2: online softmax over the 64 tokens of the group; warp = head, lane = 2 tokens
    {
      const int h = warp, t0 = lane * 2;
      const int valid = min(gr.len - gr.blk0 * kTok, gr.n * kTok);
      float x[2] = {0.f, 0.f};
#pragma unroll
      for (int kq = 0; kq < 4; ++kq) {
        const float2 v = *reinterpret_cast<const float2*>(s_part + (kq * 16 + h) * SP_STRIDE + t0);
        x[0] += v.x;
        x[1] += v.y;
      }
      x[0] = t0 < valid ? x[0] * a.scale_log2 : -INFINITY;
      x[1] = t0 + 1 < valid ? x[1] * a.scale_log2 : -INFINITY;
      const float mx = warp_max(fmaxf(x[0], x[1]));
      const float m_old = s_m[h], l_old = s_l[h];
      const float m_new = fmaxf(m_old, mx);   // finite: token 0 of every group is valid
      const float alpha = fast_exp2(m_old - m_new);
      const float p0 = fast_exp2(x[0] - m_new), p1 = fast_exp2(x[1] - m_new);
      const float sum = warp_sum(p0 + p1);
      __syncwarp();
      if (lane == 0) {
        s_m[h] = m_new;
        s_l[h] = l_old * alpha + sum;
        s_alpha[h] = alpha;
      }
      *reinterpret_cast<uint32_t*>(smem + OFF_P + h * 128 + (((lane >> 2) ^ (h & 7)) * 16) + (lane & 3) * 4) =
          pack_bf16x2(p0, p1);
    }
    compute_sync();

    // ---- phase 3: O[:, 32*warp .. +31] = alpha * O + P . c
    {
      const float al0 = s_alpha[g], al1 = s_alpha[g + 8];
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        o[n][0] *= al0;
        o[n][1] *= al0;
        o[n][2] *= al1;
        o[n][3] *= al1;
      }
      const uint32_t sP = sbase + OFF_P;
      const int rp = (lane & 7) + ((lane >> 3) & 1) * 8, chp = lane >> 4;   // A: P rows; B: token rows
#pragma unroll
      for (int kk = 0; kk < GROUP; ++kk) {
        uint32_t pf[4];
        ldmatrix_x4(pf, sP + rp * 128 + (((2 * kk + chp) ^ (rp & 7)) * 16));
#pragma unroll
        for (int pr2 = 0; pr2 < 2; ++pr2) {
          uint32_t bf[4];
          const int chunk = 4 * warp + 2 * pr2 + chp;
          ldmatrix_x4_trans(bf, ring + kk * BLKB + lat_off(rp, chunk));
          const uint32_t b0[2] = {bf[0], bf[1]}, b1[2] = {bf[2], bf[3]};
          mma_bf16_16816(o[2 * pr2], pf, b0);
          mma_bf16_16816(o[2 * pr2 + 1], pf, b1);
        }
      }
    }
    compute_sync();   // P and the partial-S buffer are free again
    if (gi + 2 < groups_total) named_arrive(4 + half);   // ... and so is this ring half: the producers refill it

    const bool seq_end = gr.blk0 + gr.n == gr.nblk;
    if (seq_end || gi == groups_total - 1) {
      fresh = true;
      const bool whole = seq_end && seg_first == 0;
      const int h0 = g, h1 = g + 8;
      if (whole) {
        const float i0 = 1.f / s_l[h0], i1 = 1.f / s_l[h1];
        __nv_bfloat16* ob = a.out + static_cast<int64_t>(gr.seq) * H * R;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const int d = 32 * warp + n * 8 + tq * 2;
          if (h0 < H) *reinterpret_cast<uint32_t*>(ob + h0 * R + d) = pack_bf16x2(o[n][0] * i0, o[n][1] * i0);
          if (h1 < H) *reinterpret_cast<uint32_t*>(ob + h1 * R + d) = pack_bf16x2(o[n][2] * i1, o[n][3] * i1);
        }
      } else {
        const int64_t pslot = static_cast<int64_t>(p) * 2 + (seg_first > 0 ? 0 : 1);
        float* po = a.part_o + pslot * H * R;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const int d = 32 * warp + n * 8 + tq * 2;
          if (h0 < H) *reinterpret_cast<float2*>(po + h0 * R + d) = make_float2(o[n][0], o[n][1]);
          if (h1 < H) *reinterpret_cast<float2*>(po + h1 * R + d) = make_float2(o[n][2], o[n][3]);
        }
        if (tid < H)
          *reinterpret_cast<float2*>(a.part_ml + (pslot * H + tid) * 2) = make_float2(s_m[tid], s_l[tid]);
      }
      if (seq_end && tid == 0) {
        const int seq_start_flat = flat - gr.blk0;
        a.seq_info[2 * gr.seq] = whole ? -1 : seq_start_flat / rg.per_cta;
        a.seq_info[2 * gr.seq + 1] = whole ? -1 : p;
      }
      compute_sync();   // the running state is re-initialised by the next segment
    }
    flat += gr.n;
  }
}

bool mla_fast_shape(int H, int r, int dr, int bs) {
  return r == R && dr == DR && bs == kTok && H >= 1 && H <= 16;
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn tensor_map_encoder() {
  static EncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

}  // namespace

size_t mla_decode_mma_workspace(int batch, int H, int r, int dr) {
  if (!mla_fast_shape(H, r, dr, kTok)) return 256;
  int sms = sm_count_cached();
  if (sms <= 0) sms = 148;
  return decode_workspace_bytes(static_cast<size_t>(sms), batch, H, R);
}

int mla_decode_mma_launch(const void* q_abs, const void* q_rope, const void* lat, void* out,
                          const int32_t* bt, int64_t bt_stride, const int64_t* lens, int batch,
                          int H, int r, int dr, int bs, int64_t num_blocks, float scale,
                          void* workspace, size_t workspace_bytes, int32_t* status,
                          cudaStream_t s) {
  if (!mla_fast_shape(H, r, dr, bs)) return B200_ERR_UNSUPPORTED;
  if (!aligned16(q_abs) || !aligned16(q_rope) || !aligned16(lat) || !aligned16(out))
    return B200_ERR_UNSUPPORTED;
  if (num_blocks <= 0 || num_blocks * kTok > 2147483647LL) return B200_ERR_UNSUPPORTED;
  EncodeFn enc = tensor_map_encoder();
  if (enc == nullptr) return B200_ERR_UNSUPPORTED;
  const int sms = sm_count_cached();
  if (sms <= 0) return B200_ERR_NO_DEVICE;
  const size_t grid = static_cast<size_t>(sms);
  const size_t need = decode_workspace_bytes(grid, batch, H, R);
  if (!workspace || workspace_bytes < need) return B200_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return B200_ERR_ALIGN;
  // The pool seen as (column within a slab: 64, token row: num_blocks * 16, slab: 9) with strides
  // (2 B, 1152 B, 128 B): one box = one KV block, written slab by slab — [9][16 tokens][128 B] — which is
  // the layout lat_off() addresses, so a block is a single copy instruction.
  CUtensorMap tm;
  {
    const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(num_blocks) * kTok, static_cast<cuuint64_t>(SLABS)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ROWB), 128};
    const cuuint32_t box[3] = {64, kTok, static_cast<cuuint32_t>(SLABS)};
    const cuuint32_t estr[3] = {1, 1, 1};
    if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(lat), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return B200_ERR_UNSUPPORTED;
  }
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(mla_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES) != cudaSuccess)
      return B200_ERR_LAUNCH;
    configured[dev] = true;
  }
  MlaArgs a{};
  a.q_abs = static_cast<const __nv_bfloat16*>(q_abs);
  a.q_rope = static_cast<const __nv_bfloat16*>(q_rope);
  a.lat = static_cast<const uint8_t*>(lat);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.bt = bt;
  a.bt_stride = bt_stride;
  a.lens = lens;
  a.batch = batch;
  a.H = H;
  a.num_blocks = num_blocks;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  uint8_t* w = static_cast<uint8_t*>(workspace);
  a.part_o = reinterpret_cast<float*>(w);
  w += align256(grid * 2 * H * R * sizeof(float));
  a.part_ml = reinterpret_cast<float*>(w);
  w += align256(grid * 2 * H * 2 * sizeof(float));
  a.seq_info = reinterpret_cast<int32_t*>(w);
  mla_decode_mma_kernel<<<static_cast<int>(grid), kThreads, SMEM_BYTES, s>>>(a, tm);
  const int rc = launch_result();
  if (rc != B200_OK) return rc;
  CombineArgs c{};
  c.out = out;
  c.lens = lens;
  c.part_o = a.part_o;
  c.part_ml = a.part_ml;
  c.seq_info = a.seq_info;
  c.batch = batch;
  c.H = H;
  c.D = R;
  return decode_combine_launch(c, s);
}

}  // namespace b200
