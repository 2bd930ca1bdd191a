// MLA latent-cache decode on the sm_100a tensor cores (tcgen05): the absorbed branch of
// MultiHeadLatentAttention.forward (model/attention/MLA.py:136-178) over a paged latent pool.
//
//   score[h, t] = (q_abs[h] . c[t] + q_rope[h] . pe[t]) * scale      (MLA.py:153-156)
//   out[h]      = softmax_t(score[h, :]) . c                          (MLA.py:177)
//
// Why tcgen05 here: the contraction is only 30 flop per byte, so the kernel is bound by moving the
// latent rows, and what limits an mma.sync version is not the tensor pipe but the shared-memory pipe
// (every row is written once by the copy and read twice through ldmatrix, plus the exchange of
// partial scores).  With tcgen05 the tensor core reads its operands from shared memory itself:
// no ldmatrix, no fragments in registers, and the two contractions need no CTA-wide barrier.
//
// Both contractions put the 128 TOKENS of a tile where the tensor core wants its long dimension:
//   S^T [128 tokens x 16 heads]  = C [128 x 576] . Q^T        A = latent tile, K-major (rows = tokens)
//   O^T [128 dims   x 16 heads] += C^T [128 x 128 tokens] . P^T   A = the SAME bytes read MN-major
// so one staged copy of the tile serves both, in the 128-byte-swizzled layout TMA writes.
//
// CTA = one SM, 192 threads.  Warp 0: producer (lanes 0-7 own the 8 KV blocks of a tile and issue
// their TMA boxes), warp 1: MMA issuer (one lane) and tensor-memory owner, warps 2-5: softmax and
// output (thread = tensor-memory lane = token for S^T, = latent column for O^T).  The flat list of
// KV blocks of all sequences is cut into equal contiguous ranges, one per CTA (as in the GQA decode
// kernel); a sequence cut across CTAs leaves partial (O, max, sum) in the workspace and the shared
// combine kernel merges them.
//
// Shared memory: 5 slots of 32 KB hold pairs of 64-column slabs [128 tokens x 128 B] of the latent
// part (a tile needs 4), 2 slots of 16 KB the rope slab, so one pair and one rope slab of the next
// tile are in flight while a tile is being used; Q^T (18 KB) and P^T (4 KB) are the B operands.
// Every wait is bounded; a timeout sets the status word to B200_ERR_TIMEOUT and all roles leave.
#include <cuda.h>

#include "common.cuh"
#include "decode_common.cuh"
#include "umma.cuh"

namespace b200 {
namespace {

constexpr int kTok = 16;               // tokens per KV block
constexpr int R = 512, DR = 64, W = R + DR;
constexpr int kThreads = 192;
constexpr int TILE_BLOCKS = 8, TILE_TOK = TILE_BLOCKS * kTok;   // 128 tokens
constexpr int SLAB_BYTES = TILE_TOK * 128;                      // [128 tokens x 64 columns] bf16
constexpr int PAIR_BYTES = 2 * SLAB_BYTES;
constexpr int PAIRS = 5, ROPES = 2;
constexpr int QSLAB_BYTES = 16 * 128;                           // [16 heads x 64 columns] bf16
constexpr int OFF_PAIR = 0;
constexpr int OFF_ROPE = OFF_PAIR + PAIRS * PAIR_BYTES;         // 163840
constexpr int OFF_Q = OFF_ROPE + ROPES * SLAB_BYTES;            // 196608
constexpr int OFF_P = OFF_Q + (W / 64) * QSLAB_BYTES;           // 215040
constexpr int OFF_RED = OFF_P + 2 * QSLAB_BYTES;                // 219136: float [2][4][16]
constexpr int OFF_BAR = OFF_RED + 2 * 4 * 16 * 4;               // 219648
// barriers
constexpr int PAIR_FULL = 0, PAIR_FREE = PAIRS, ROPE_FULL = 2 * PAIRS, ROPE_FREE = 2 * PAIRS + ROPES;
constexpr int S_FULL = 2 * PAIRS + 2 * ROPES, P_READY = S_FULL + 1, PV_DONE = S_FULL + 2, Q_READY = S_FULL + 3;
constexpr int NUM_BARS = S_FULL + 4;                            // 18
constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;                // tmem pointer, abort, go, scan scratch
constexpr int SMEM_BYTES = OFF_MISC + 64 + 36 * 4 + 1024;       // + alignment slack
constexpr int TMEM_COLS = 128;                                  // S at 0, O tiles at 32 + 16 j
constexpr float kRescaleThreshold = 8.f;                        // log2 units

struct UArgs {
  const __nv_bfloat16* q_abs;   // [B, H, 512]
  const __nv_bfloat16* q_rope;  // [B, H, 64]
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

// The tiles of this CTA's block range, in order: up to 8 consecutive blocks of one sequence.
struct Tile {
  int seq, blk0, n, nblk, len;   // sequence, first block, blocks, blocks / tokens of the sequence
  int seg_first;                 // first block of the sequence inside this CTA (0: it starts here)
  bool first, last, seq_end;     // first / last tile of the segment; the sequence ends with this tile
  int flat;                      // flat index of blk0 in the global block list
};
struct TileIter {
  const UArgs& a;
  int seq, blk, nblk, len, remaining, flat, seg_first;
  bool fresh;
  __device__ TileIter(const UArgs& a_, const CtaRange& rg) : a(a_) {
    seq = rg.start_seq;
    blk = rg.start_off;
    remaining = rg.cnt;
    flat = rg.start;
    fresh = true;
    seg_first = 0;
    load();
  }
  __device__ void load() {
    const int64_t l = a.lens[seq];
    nblk = num_kv_blocks(l, a.bt_stride, kTok);
    const int64_t cap = static_cast<int64_t>(nblk) * kTok;
    len = static_cast<int>(l < cap ? l : cap);
  }
  __device__ bool done() const { return remaining <= 0; }
  __device__ Tile next() {
    Tile t;
    t.seq = seq;
    t.blk0 = blk;
    t.nblk = nblk;
    t.len = len;
    t.n = min(TILE_BLOCKS, min(nblk - blk, remaining));
    t.first = fresh;
    if (fresh) seg_first = blk;
    t.seg_first = seg_first;
    t.flat = flat;
    blk += t.n;
    remaining -= t.n;
    flat += t.n;
    t.seq_end = blk >= nblk;
    t.last = t.seq_end || remaining <= 0;
    fresh = t.last;
    if (t.seq_end && remaining > 0) {
      blk = 0;
      do {
        ++seq;
        load();
      } while (nblk == 0 && seq + 1 < a.batch);
    }
    return t;
  }
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tensor_map, int c0, int c1,
                                            uint32_t mbar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
          "r"(dst_smem),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(c0), "r"(c1), "r"(mbar)
      : "memory");
}
__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kThreads, 1)
mla_decode_umma_kernel(const UArgs a, const __grid_constant__ CUtensorMap tm_lat) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(smem);
  float* red = reinterpret_cast<float*>(smem + OFF_RED);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + OFF_MISC + 4);
  volatile int* s_go = reinterpret_cast<volatile int*>(smem + OFF_MISC + 8);
  int* s_scan = reinterpret_cast<int*>(smem + OFF_MISC + 16);
  auto bar = [&](int i) -> uint32_t { return sb + OFF_BAR + i * 8; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const CtaRange rg = plan_cta_range(a.lens, a.batch, a.bt_stride, kTok, s_scan);
  if (rg.cnt == 0) return;                        // uniform, before any barrier / allocation

  // Rows of a slab that no copy has written yet are read by the second contraction with weight 0:
  // they must hold finite numbers, so the rings start as zeros.
  for (int i = tid; i < OFF_Q / 16; i += kThreads) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (tid == 0) {
    for (int i = 0; i < PAIRS; ++i) {
      umma::mbar_init(bar(PAIR_FULL + i), 1);
      umma::mbar_init(bar(PAIR_FREE + i), 1);
    }
    for (int i = 0; i < ROPES; ++i) {
      umma::mbar_init(bar(ROPE_FULL + i), 1);
      umma::mbar_init(bar(ROPE_FREE + i), 1);
    }
    umma::mbar_init(bar(S_FULL), 1);
    umma::mbar_init(bar(P_READY), 128);
    umma::mbar_init(bar(PV_DONE), 1);
    umma::mbar_init(bar(Q_READY), 128);
    *s_abort = 0;
    *s_go = 1;
    umma::mbar_init_fence();
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tm_lat)) : "memory");
  }
  if (warp == 1) umma::tmem_alloc(sb + OFF_MISC, TMEM_COLS);
  umma::fence_async_proxy();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;

  auto give_up = [&]() {
    *s_abort = 1;
    report(a.status, B200_ERR_TIMEOUT);
  };

  if (warp == 0) {
    // =============================== producer ===============================
    TileIter it(a, rg);
    int pair_n = 0, rope_n = 0;
    bool ok = true;
    while (!it.done() && ok) {
      const Tile t = it.next();
      int id = -1;
      if (lane < t.n) {
        id = __ldg(a.bt + static_cast<int64_t>(t.seq) * a.bt_stride + t.blk0 + lane);
        if (static_cast<uint64_t>(static_cast<int64_t>(id)) >= static_cast<uint64_t>(a.num_blocks)) {
          report(a.status, B200_ERR_BOUNDS);       // the block is skipped: its rows keep finite stale values
          id = -1;
        }
      }
      const uint32_t bytes = __popc(__ballot_sync(0xffffffffu, id >= 0)) * (kTok * 128);
      for (int j = 0; j <= 4 && ok; ++j) {          // four slab pairs of the latent part, then the rope slab
        const bool rope = j == 4;
        const int n = rope ? rope_n : pair_n, ring = rope ? ROPES : PAIRS;
        const int slot = n % ring, use = n / ring;
        if (use > 0) {
          int good = 1;
          if (lane == 0) good = umma::mbar_wait(bar((rope ? ROPE_FREE : PAIR_FREE) + slot), (use - 1) & 1, s_abort);
          good = __shfl_sync(0xffffffffu, good, 0);
          if (!good) {
            if (lane == 0) give_up();
            ok = false;
            break;
          }
        }
        const uint32_t full = bar((rope ? ROPE_FULL : PAIR_FULL) + slot);
        if (lane == 0) umma::mbar_expect_tx(full, rope ? bytes : 2 * bytes);
        __syncwarp();
        if (id >= 0) {
          if (rope) {
            tma_load_2d(sb + OFF_ROPE + slot * SLAB_BYTES + lane * (kTok * 128), &tm_lat, R, id * kTok, full);
          } else {
            const uint32_t dst = sb + OFF_PAIR + slot * PAIR_BYTES + lane * (kTok * 128);
            tma_load_2d(dst, &tm_lat, (2 * j) * 64, id * kTok, full);
            tma_load_2d(dst + SLAB_BYTES, &tm_lat, (2 * j + 1) * 64, id * kTok, full);
          }
        }
        if (rope) ++rope_n; else ++pair_n;
      }
    }
    if (*s_abort && lane == 0) {
      // copies still in flight must land before the CTA gives its shared memory back
      int never = 0;
      for (int x = max(0, pair_n - PAIRS); x < pair_n; ++x)
        umma::mbar_wait(bar(PAIR_FULL + x % PAIRS), (x / PAIRS) & 1, &never, 1 << 16);
      for (int x = max(0, rope_n - ROPES); x < rope_n; ++x)
        umma::mbar_wait(bar(ROPE_FULL + x % ROPES), (x / ROPES) & 1, &never, 1 << 16);
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      TileIter it(a, rg);
      const uint32_t idesc_qk = umma::instr_desc_bf16(TILE_TOK, 16, false, false);
      const uint32_t idesc_pv = umma::instr_desc_bf16(128, 16, true, false);
      const uint32_t qbase = sb + OFF_Q, pbase = sb + OFF_P;
      int pair_n = 0, rope_n = 0, tile_n = 0, seg_n = 0;
      bool ok = true;
#define MMA_WAIT(idx, parity)                                \
  if (!umma::mbar_wait(bar(idx), (parity), s_abort)) {       \
    give_up();                                               \
    ok = false;                                              \
    break;                                                   \
  }
      while (!it.done() && ok) {
        const Tile t = it.next();
        do {
          if (t.first) {
            MMA_WAIT(Q_READY, seg_n & 1)
            ++seg_n;
          }
          // ---- S^T = C . Q^T : 9 slabs of 64 columns, 4 k-steps of 16 each
          for (int j = 0; j < 4 && ok; ++j) {
            const int n = pair_n + j, slot = n % PAIRS;
            MMA_WAIT(PAIR_FULL + slot, (n / PAIRS) & 1)
            umma::fence_after_sync();
            const uint32_t base = sb + OFF_PAIR + slot * PAIR_BYTES;
#pragma unroll
            for (int s = 0; s < 2; ++s)
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                umma::mma_ss(tmem, umma::smem_desc(base + s * SLAB_BYTES + kk * 32, 0, 1024),
                             umma::smem_desc(qbase + (2 * j + s) * QSLAB_BYTES + kk * 32, 0, 1024), idesc_qk,
                             (j | s | kk) != 0);
          }
          if (!ok) break;
          {
            const int slot = rope_n % ROPES;
            MMA_WAIT(ROPE_FULL + slot, (rope_n / ROPES) & 1)
            umma::fence_after_sync();
            const uint32_t base = sb + OFF_ROPE + slot * SLAB_BYTES;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma::mma_ss(tmem, umma::smem_desc(base + kk * 32, 0, 1024),
                           umma::smem_desc(qbase + 8 * QSLAB_BYTES + kk * 32, 0, 1024), idesc_qk, 1);
            umma::commit(bar(ROPE_FREE + slot));
            ++rope_n;
          }
          umma::commit(bar(S_FULL));
          // ---- O^T += C^T . P^T : one k-step per KV block of the tile, four tiles of 128 latent columns
          MMA_WAIT(P_READY, tile_n & 1)
          umma::fence_after_sync();
          for (int j = 0; j < 4; ++j) {
            const int slot = (pair_n + j) % PAIRS;
            const uint32_t base = sb + OFF_PAIR + slot * PAIR_BYTES;
            for (int ks = 0; ks < t.n; ++ks)
              umma::mma_ss(tmem + 32 + 16 * j, umma::smem_desc(base + ks * (kTok * 128), SLAB_BYTES, 1024),
                                  umma::smem_desc(pbase + (ks >> 2) * QSLAB_BYTES + (ks & 3) * 32, 0, 1024),
                                  idesc_pv, !t.first || ks > 0);
            umma::commit(bar(PAIR_FREE + slot));
          }
          pair_n += 4;
          umma::commit(bar(PV_DONE));
          ++tile_n;
        } while (false);
      }
#undef MMA_WAIT
    }
  } else {
    // =============================== softmax / output (4 warps) ===============================
    const int q = warp & 3;                       // tensor-memory lane quarter of this warp
    const int i = q * 32 + lane;                  // token of the tile (S^T) / latent column of a 128-wide tile (O^T)
    const int et = tid - 64;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const int H = a.H;
    TileIter it(a, rg);
    int tile_n = 0, pair_n = 0;
    float m_run[16], l[16];
    while (!it.done()) {
      const Tile t = it.next();
      if (t.first) {
        // stage Q^T = [q_abs | q_rope] of the sequence as 9 swizzled slabs [16 heads x 64 columns]; rows >= H are zero
        for (int idx = et; idx < 16 * (W / 8); idx += 128) {
          const int h = idx / (W / 8), c = idx - h * (W / 8);      // 16-byte chunk c of head h
          uint4 val = make_uint4(0u, 0u, 0u, 0u);
          if (h < H) {
            const int64_t row = static_cast<int64_t>(t.seq) * H + h;
            val = c < R / 8 ? __ldg(reinterpret_cast<const uint4*>(a.q_abs + row * R) + c)
                            : __ldg(reinterpret_cast<const uint4*>(a.q_rope + row * DR) + (c - R / 8));
          }
          *reinterpret_cast<uint4*>(smem + OFF_Q + (c >> 3) * QSLAB_BYTES + h * 128 + (((c & 7) ^ (h & 7)) << 4)) = val;
        }
#pragma unroll
        for (int h = 0; h < 16; ++h) {
          m_run[h] = -INFINITY;
          l[h] = 0.f;
        }
        umma::fence_async_proxy();
        umma::mbar_arrive(bar(Q_READY));
      }
      if (!umma::mbar_wait(bar(S_FULL), tile_n & 1, s_abort)) give_up();
      umma::fence_after_sync();
      const int par = tile_n & 1;
      const int ntok = min(t.n * kTok, t.len - t.blk0 * kTok);
      const bool valid = i < ntok;
      float sc[16];
      {
        uint32_t r[16];
        umma::tmem_ld16(tmem + lane_sel, r);
#pragma unroll
        for (int h = 0; h < 16; ++h) sc[h] = valid ? __uint_as_float(r[h]) * a.scale_log2 : -INFINITY;
      }
      // per-head maximum over the 128 tokens: butterfly inside the warp, then across the four warps
#pragma unroll
      for (int h = 0; h < 16; ++h) {
        float v = sc[h];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
        if (lane == 0) red[par * 64 + q * 16 + h] = v;
      }
      if (et == 0) *s_go = !*s_abort;
      softmax_sync();
      if (!*s_go) break;                          // uniform: written once before the barrier
      float alpha[16];
      bool any = false;
#pragma unroll
      for (int h = 0; h < 16; ++h) {
        const float* rp = red + par * 64 + h;
        const float mt = fmaxf(fmaxf(rp[0], rp[16]), fmaxf(rp[32], rp[48]));
        // lazy rescale: the reference maximum moves only when it grows by more than the threshold
        if (mt > m_run[h] + kRescaleThreshold || (m_run[h] == -INFINITY && mt > -INFINITY)) {
          alpha[h] = m_run[h] == -INFINITY ? 0.f : ex2(m_run[h] - mt);
          m_run[h] = mt;
          l[h] *= alpha[h];
          any = true;
        } else {
          alpha[h] = 1.f;
        }
      }
      if (any && !t.first) {
        // the previous tile's second contraction is complete (S_FULL follows it in the MMA queue)
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
          uint32_t o[16];
          umma::tmem_ld16(tmem + lane_sel + 32 + 16 * j, o);
#pragma unroll
          for (int h = 0; h < 16; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * alpha[h]);
          umma::tmem_st16(tmem + lane_sel + 32 + 16 * j, o);
        }
        umma::tmem_wait_st();
      }
      // P^T[head][token] as bf16 into the swizzled B operand; row sums stay per thread until the flush
      {
        uint8_t* prow = smem + OFF_P + (i >> 6) * QSLAB_BYTES + (i & 7) * 2;
        const int chunk = (i & 63) >> 3;
#pragma unroll
        for (int h = 0; h < 16; ++h) {
          const float p = valid ? ex2(sc[h] - m_run[h]) : 0.f;
          l[h] += p;
          *reinterpret_cast<__nv_bfloat16*>(prow + h * 128 + ((chunk ^ (h & 7)) << 4)) = __float2bfloat16(p);
        }
      }
      // rows of the tile's last block past the end of the context hold whatever the pool has there:
      // zero them before the second contraction reads them (their weight is 0, but 0 * NaN is not)
      if (!valid && i < t.n * kTok) {
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
          uint4* row = reinterpret_cast<uint4*>(smem + OFF_PAIR + ((pair_n + j) % PAIRS) * PAIR_BYTES + i * 128);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            row[c] = make_uint4(0u, 0u, 0u, 0u);
            row[c + SLAB_BYTES / 16] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
      pair_n += 4;
      umma::fence_async_proxy();
      umma::fence_before_sync();
      umma::mbar_arrive(bar(P_READY));

      if (t.last) {
        // ---- end of the sequence's segment in this CTA: total row sums, then O^T out of tensor memory
        if (!umma::mbar_wait(bar(PV_DONE), tile_n & 1, s_abort)) give_up();
        umma::fence_after_sync();
        float* rs = red + (par ^ 1) * 64;
#pragma unroll
        for (int h = 0; h < 16; ++h) {
          float v = l[h];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0) rs[q * 16 + h] = v;
        }
        if (et == 0) *s_go = !*s_abort;
        softmax_sync();
        if (!*s_go) break;
        float L[16];
#pragma unroll
        for (int h = 0; h < 16; ++h) L[h] = rs[h] + rs[16 + h] + rs[32 + h] + rs[48 + h];
        const bool whole = t.seq_end && t.seg_first == 0;
        const int64_t pslot = static_cast<int64_t>(blockIdx.x) * 2 + (t.seg_first > 0 ? 0 : 1);
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
          uint32_t o[16];
          umma::tmem_ld16(tmem + lane_sel + 32 + 16 * j, o);
          const int d = 128 * j + i;
          if (whole) {
            __nv_bfloat16* ob = a.out + static_cast<int64_t>(t.seq) * H * R + d;
#pragma unroll
            for (int h = 0; h < 16; ++h)
              if (h < H) ob[h * R] = __float2bfloat16(__uint_as_float(o[h]) / L[h]);
          } else {
            float* po = a.part_o + pslot * H * R + d;
#pragma unroll
            for (int h = 0; h < 16; ++h)
              if (h < H) po[h * R] = __uint_as_float(o[h]);
          }
        }
        if (!whole) {
#pragma unroll
          for (int h = 0; h < 16; ++h)
            if (et == h && h < H)
              *reinterpret_cast<float2*>(a.part_ml + (pslot * H + h) * 2) = make_float2(m_run[h], L[h]);
        }
        if (t.seq_end && et == 0) {
          a.seq_info[2 * t.seq] = whole ? -1 : (t.flat - t.blk0) / rg.per_cta;
          a.seq_info[2 * t.seq + 1] = whole ? -1 : static_cast<int>(blockIdx.x);
        }
        softmax_sync();                            // the sums buffer is the next tile's maxima buffer
      }
      ++tile_n;
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 1) umma::tmem_dealloc(tmem, TMEM_COLS);
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

// Same contract as mla_decode_mma_launch (mla_decode_mma.cu); B200_ERR_UNSUPPORTED = try the next kernel.
int mla_decode_umma_launch(const void* q_abs, const void* q_rope, const void* lat, void* out,
                           const int32_t* bt, int64_t bt_stride, const int64_t* lens, int batch, int H,
                           int r, int dr, int bs, int64_t num_blocks, float scale, void* workspace,
                           size_t workspace_bytes, int32_t* status, cudaStream_t s) {
  if (r != R || dr != DR || bs != kTok || H < 1 || H > 16) return B200_ERR_UNSUPPORTED;
  if (!aligned16(q_abs) || !aligned16(q_rope) || !aligned16(lat) || !aligned16(out)) return B200_ERR_UNSUPPORTED;
  if (num_blocks <= 0 || num_blocks * kTok > 2147483647LL) return B200_ERR_UNSUPPORTED;
  EncodeFn enc = tensor_map_encoder();
  if (enc == nullptr) return B200_ERR_UNSUPPORTED;
  const int sms = sm_count_cached();
  if (sms <= 0) return B200_ERR_NO_DEVICE;
  const size_t grid = static_cast<size_t>(sms);
  const size_t need = decode_workspace_bytes(grid, batch, H, R);
  if (!workspace || workspace_bytes < need) return B200_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return B200_ERR_ALIGN;
  // the pool as [num_blocks * 16 rows, 576 columns]; one box = 64 columns of one KV block
  CUtensorMap tm;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(num_blocks) * kTok};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(W) * 2};
  const cuuint32_t box[2] = {64, kTok};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(lat), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return B200_ERR_UNSUPPORTED;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return B200_ERR_UNSUPPORTED;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(mla_decode_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return B200_ERR_LAUNCH;
    configured[dev] = true;
  }
  UArgs a{};
  a.q_abs = static_cast<const __nv_bfloat16*>(q_abs);
  a.q_rope = static_cast<const __nv_bfloat16*>(q_rope);
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
  mla_decode_umma_kernel<<<static_cast<int>(grid), kThreads, SMEM_BYTES, s>>>(a, tm);
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
