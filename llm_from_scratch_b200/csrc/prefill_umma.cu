// Ragged causal prefill attention, bf16, head_dim 128, on the Blackwell tensor cores (tcgen05).
// Packed keys are served faster by prefill_umma2.cu (see the dispatch in prefill_varlen.cu); this kernel
// runs when part of the context comes from the paged pool.
//
// One CTA owns a 128-row query tile of TWO query heads that share a KV head (grouped-query
// attention), so every K/V tile staged in shared memory feeds two independent attention problems
// A and B.  Tensor memory (512 columns) holds, for each of them, the 128x128 fp32 score tile S and
// the 128x128 fp32 output accumulator O; the bf16 probabilities P overwrite the first 64 columns
// of S and are consumed from tensor memory as the A operand of O += P.V.
//
//   warp 0      K producer (+ both Q tiles): one thread issuing TMA tile copies (cp.async.bulk.tensor,
//               128-byte swizzle, completion counted on an mbarrier) for packed k/v; for the paged
//               pool the whole warp stages rows with 16-byte cp.async instead, because rows past the
//               end of a context must be zero-filled rather than read
//   warp 1      V producer, likewise
//   warp 2      tensor-memory allocation; lane 0 issues every tcgen05.mma
//   warps 4-7   softmax of problem A: one thread per query row, so row max / row sum need no shuffles
//   warps 8-11  softmax of problem B
//
// Per KV tile j the issuing thread runs  S_A = Q_A.K_j^T | O_B += P_B(j-1).V_(j-1) | S_B = Q_B.K_j^T |
// O_A += P_A(j).V_j : the tensor core works on one problem while the softmax warps of the other
// turn their S into P.  Rescaling of O by 2^(m_old - m_new) is done lazily — only when a row maximum
// grows by more than 2^8 — which leaves the result exact because P and the row sum use the same
// reference maximum.  All synchronisation is by mbarriers (tcgen05.commit for MMA completion,
// thread arrivals otherwise); every wait is bounded and a timeout aborts the CTA cleanly.
//
// Keys/values come from the packed k/v tensors or, with a cached prefix, from the paged pool through
// the block table (mask bottom-right aligned).  Tiles above the causal diagonal are never loaded.
#include <cuda.h>
#include <string.h>

#include "umma.cuh"

namespace b200 {
namespace {

constexpr int BM = 128, BN = 128, D = 128;
constexpr int kThreads = 384;
constexpr int TILE_BYTES = BM * D * 2;        // 32 KiB: two 16 KiB halves of 64 columns
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int OFF_QA = 0, OFF_QB = TILE_BYTES;
constexpr int OFF_K = 2 * TILE_BYTES;         // 2 stages
constexpr int OFF_V = 4 * TILE_BYTES;         // 2 stages
constexpr int OFF_BAR = 6 * TILE_BYTES;       // barriers, tensor-memory pointer, abort flag
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;   // + slack to align the base to 1024 bytes
constexpr float kRescaleThreshold = 8.f;      // log2 units
// Every kPolyEvery-th pair of exponentials can be evaluated by a polynomial on the FMA pipe instead of
// the special-function unit.  Measured on the 262K-token stress batch: 855 TFLOP/s with 0 (off),
// 789 TFLOP/s with 4 — the softmax warps are issue-bound, not SFU-bound — so it is off.
constexpr int kPolyEvery = 0;
// Also measured and not kept: two threads per query row (640-thread CTA, one named-barrier exchange
// of the row statistics per KV tile): 802 TFLOP/s against 861 with one thread per row.

enum Bar { Q_FULL = 0, K_FULL = 1, V_FULL = 3, K_EMPTY = 5, V_EMPTY = 7, S_FULL = 9, P_READY = 11, O_FINAL = 13, NUM_BARS = 14 };

struct UmmaArgs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  __nv_bfloat16* out;
  int64_t q_stride, k_stride, v_stride;
  const int32_t* cu_q;
  const int32_t* cu_k;
  int Hq, Hkv, ntiles_max;
  const int32_t* plan;   // tile list (see b200_prefill_plan) or null: grid (head pair, seq, tile rank)
  float scale_log2;
  const __nv_bfloat16* kc;
  const __nv_bfloat16* vc;
  const int32_t* bt;
  int64_t bt_stride;
  int bs;
  int64_t num_blocks;
  int32_t* status;
};

// byte offset of 16-byte chunk c16 (0..15) of row r inside a 128x128 bf16 tile
__device__ __forceinline__ uint32_t tile_off(int r, int c16) {
  return (c16 >> 3) * HALF_BYTES + r * 128 + (((c16 & 7) ^ (r & 7)) << 4);
}

template <bool PAGED>
__global__ void __launch_bounds__(kThreads, 1)
prefill_umma_kernel(const UmmaArgs a, const __grid_constant__ CUtensorMap tm_q,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NUM_BARS * 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + OFF_BAR + NUM_BARS * 8 + 8);
  auto bar = [&](int i) -> uint32_t { return sb + OFF_BAR + i * 8; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pair = blockIdx.x;
  int seq, tile;
  if (a.plan) {                                  // grid (head pair, tile-list slot)
    if (static_cast<int>(blockIdx.y) >= a.plan[0]) return;
    const uint32_t entry = static_cast<uint32_t>(a.plan[kPlanHeader + blockIdx.y]);
    seq = entry >> 16;
    tile = entry & 0xffffu;
  } else {
    seq = blockIdx.y;
    tile = a.ntiles_max - 1 - blockIdx.z;
  }
  const int q0 = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q0;
  const int k0 = a.cu_k[seq], k_len = a.cu_k[seq + 1] - k0;
  const int m0 = tile * BM;
  if (m0 >= q_len) return;                       // uniform over the CTA, before any barrier / allocation
  const int off = k_len - q_len;
  const int head_a = 2 * pair, head_b = head_a + 1;
  const int kvh = head_a / (a.Hq / a.Hkv);
  const int rows_q = min(BM, q_len - m0);
  int kmax = off + m0 + rows_q;
  if (kmax > k_len) kmax = k_len;
  if (kmax < 1) kmax = 1;
  const int n = (kmax + BN - 1) / BN;            // KV tiles; >= 1

  if (tid == 0) {
    // paged: every lane of a producer warp arrives; TMA: one arrival + the transferred byte count
    umma::mbar_init(bar(Q_FULL), PAGED ? 64 : 1);
    for (int s = 0; s < 2; ++s) {
      umma::mbar_init(bar(K_FULL + s), PAGED ? 32 : 1);
      umma::mbar_init(bar(V_FULL + s), PAGED ? 32 : 1);
      umma::mbar_init(bar(K_EMPTY + s), 1);
      umma::mbar_init(bar(V_EMPTY + s), 1);
      umma::mbar_init(bar(S_FULL + s), 1);
      umma::mbar_init(bar(P_READY + s), 128);
    }
    umma::mbar_init(bar(O_FINAL), 1);
    *s_abort = 0;
    umma::mbar_init_fence();
  }
  if (warp == 2) umma::tmem_alloc(sb + OFF_BAR + NUM_BARS * 8, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;
  const uint32_t tS[2] = {tmem, tmem + 256}, tO[2] = {tmem + 128, tmem + 384};

  auto give_up = [&]() {
    *s_abort = 1;
    report(a.status, B200_ERR_TIMEOUT);
  };
#define WAIT_OR_ABORT(idx, parity)                                   \
  if (!umma::mbar_wait(bar(idx), (parity), s_abort)) {               \
    give_up();                                                       \
    break;                                                           \
  }

  if (!PAGED && warp < 2) {
    // =============================== TMA producers ===============================
    if (lane == 0) {
      const bool is_k = warp == 0;
      if (is_k) {
        umma::mbar_expect_tx(bar(Q_FULL), 2 * TILE_BYTES);
        for (int x = 0; x < 2; ++x)
          for (int h = 0; h < 2; ++h)
            umma::tma_load_3d(sb + (x ? OFF_QB : OFF_QA) + h * HALF_BYTES, &tm_q, h * 64, x ? head_b : head_a,
                              q0 + m0, bar(Q_FULL));
      }
      const int full0 = is_k ? K_FULL : V_FULL, empty0 = is_k ? K_EMPTY : V_EMPTY;
      const uint32_t stage0 = sb + (is_k ? OFF_K : OFF_V);
      const CUtensorMap* tm = is_k ? &tm_k : &tm_v;
      for (int j = 0; j < n; ++j) {
        const int st = j & 1;
        if (j >= 2) WAIT_OR_ABORT(empty0 + st, ((j >> 1) - 1) & 1)
        umma::mbar_expect_tx(bar(full0 + st), TILE_BYTES);
        for (int h = 0; h < 2; ++h)
          umma::tma_load_3d(stage0 + st * TILE_BYTES + h * HALF_BYTES, tm, h * 64, kvh, k0 + j * BN,
                            bar(full0 + st));
      }
    }
  } else if (warp < 2) {
    // =============================== cp.async producers (paged pool) ===============================
    const bool is_k = warp == 0;
    const int head = is_k ? head_a : head_b;
    // Q tile of this warp's head
    for (int i = 0; i < (BM * 16) / 32; ++i) {
      const int idx = lane + 32 * i, r = idx >> 4, c16 = idx & 15;
      const bool ok = r < rows_q;
      const __nv_bfloat16* src = a.q + static_cast<int64_t>(q0 + m0 + (ok ? r : 0)) * a.q_stride +
                                 static_cast<int64_t>(head) * D + c16 * 8;
      cp_async16(sb + (is_k ? OFF_QA : OFF_QB) + tile_off(r, c16), src, ok ? 16 : 0);
    }
    cp_async_commit();
    auto row_ptr = [&](int key) -> const __nv_bfloat16* {
      if (PAGED) {
        const int id = __ldg(a.bt + static_cast<int64_t>(seq) * a.bt_stride + key / a.bs);
        if (static_cast<uint64_t>(static_cast<int64_t>(id)) >= static_cast<uint64_t>(a.num_blocks)) {
          report(a.status, B200_ERR_BOUNDS);
          return nullptr;
        }
        const __nv_bfloat16* base = is_k ? a.kc : a.vc;
        return base + ((static_cast<int64_t>(id) * a.bs + key % a.bs) * a.Hkv + kvh) * D;
      }
      return (is_k ? a.k + static_cast<int64_t>(k0 + key) * a.k_stride
                   : a.v + static_cast<int64_t>(k0 + key) * a.v_stride) + static_cast<int64_t>(kvh) * D;
    };
    const int full0 = is_k ? K_FULL : V_FULL, empty0 = is_k ? K_EMPTY : V_EMPTY;
    const uint32_t stage0 = sb + (is_k ? OFF_K : OFF_V);
    for (int j = 0; j < n; ++j) {
      const int st = j & 1;
      if (j >= 2) WAIT_OR_ABORT(empty0 + st, ((j >> 1) - 1) & 1)
      const int n0 = j * BN, valid = min(BN, kmax - n0);
      // lane owns 16-byte column (lane & 15) of rows (lane >> 4) + 2*i
      const int c16 = lane & 15;
      for (int i = 0; i < BN / 2; ++i) {
        const int r = (lane >> 4) + 2 * i;
        const __nv_bfloat16* src = r < valid ? row_ptr(n0 + r) : nullptr;
        cp_async16(stage0 + st * TILE_BYTES + tile_off(r, c16), src ? src + c16 * 8 : a.q, src ? 16 : 0);
      }
      cp_async_commit();
      // everything older than the tile just issued has landed: publish it
      cp_async_wait<1>();
      umma::fence_async_proxy();
      if (j == 0) umma::mbar_arrive(bar(Q_FULL));
      else umma::mbar_arrive(bar(full0 + ((j - 1) & 1)));
    }
    cp_async_wait<0>();
    umma::fence_async_proxy();
    if (!*s_abort) umma::mbar_arrive(bar(full0 + ((n - 1) & 1)));
  } else if (warp == 2) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      const uint32_t idesc_qk = umma::instr_desc_bf16(BM, BN, false, false);
      const uint32_t idesc_pv = umma::instr_desc_bf16(BM, D, false, true);
      auto qk = [&](int x, int st) {     // S_x = Q_x . K^T : contraction over d, 8 steps of 16
        const uint32_t qbase = sb + (x ? OFF_QB : OFF_QA), kbase = sb + OFF_K + st * TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t o = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
          umma::mma_ss(tS[x], umma::smem_desc(qbase + o, 0, 1024), umma::smem_desc(kbase + o, 0, 1024),
                       idesc_qk, ks > 0);
        }
      };
      auto pv = [&](int x, int st, bool first) {   // O_x += P_x . V : contraction over 128 keys
        const uint32_t vbase = sb + OFF_V + st * TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_ts(tO[x], tS[x] + ks * 8, umma::smem_desc(vbase + ks * 2048, HALF_BYTES, 1024), idesc_pv,
                       !(first && ks == 0));
      };
      bool ok = umma::mbar_wait(bar(Q_FULL), 0, s_abort);
      if (!ok) give_up();
      for (int j = 0; ok && j < n; ++j) {
        const int st = j & 1, ph = (j >> 1) & 1;
        WAIT_OR_ABORT(K_FULL + st, ph)
        umma::fence_async_proxy();
        umma::fence_after_sync();
        qk(0, st);
        umma::commit(bar(S_FULL + 0));
        if (j > 0) {
          WAIT_OR_ABORT(P_READY + 1, (j - 1) & 1)
          WAIT_OR_ABORT(V_FULL + ((j - 1) & 1), ((j - 1) >> 1) & 1)
          umma::fence_async_proxy();
          umma::fence_after_sync();
          pv(1, (j - 1) & 1, j - 1 == 0);
          umma::commit(bar(V_EMPTY + ((j - 1) & 1)));
        }
        qk(1, st);
        umma::commit(bar(S_FULL + 1));
        umma::commit(bar(K_EMPTY + st));
        WAIT_OR_ABORT(P_READY + 0, j & 1)
        WAIT_OR_ABORT(V_FULL + st, ph)
        umma::fence_async_proxy();
        umma::fence_after_sync();
        pv(0, st, j == 0);
      }
      if (!*s_abort) {
        do {
          WAIT_OR_ABORT(P_READY + 1, (n - 1) & 1)
          WAIT_OR_ABORT(V_FULL + ((n - 1) & 1), ((n - 1) >> 1) & 1)
          umma::fence_async_proxy();
          umma::fence_after_sync();
          pv(1, (n - 1) & 1, n - 1 == 0);
          umma::commit(bar(O_FINAL));
        } while (false);
      }
    }
  } else if (warp >= 4) {
    // =============================== softmax / epilogue ===============================
    const int x = warp >= 8 ? 1 : 0;                        // problem A or B
    const int row = (warp & 3) * 32 + lane;                 // query row of the tile == tensor-memory lane
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tSx = tS[x] + lane_sel, tOx = tO[x] + lane_sel;
    const int qrow = m0 + row;                              // index of the query inside its sequence
    const int lim = min(off + qrow, kmax - 1);              // last visible key
    float m_ref = -INFINITY, l = 0.f;
    bool alive = true;
    for (int j = 0; j < n; ++j) {
      // tensor-memory loads / stores are warp-collective: the whole warp continues or stops together
      if (!__all_sync(0xffffffffu, umma::mbar_wait(bar(S_FULL + x), j & 1, s_abort))) {
        give_up();
        alive = false;
        break;
      }
      umma::fence_after_sync();
      const int n0 = j * BN;
      const bool masked = n0 + BN - 1 > lim;
      // tensor-memory loads are warp-collective, so the masked / unmasked variants are chosen per warp
      const bool warp_masked = __any_sync(0xffffffffu, masked);
      // pass 1: row maximum of the raw scores (the scale is positive, so it commutes with max).
      // Chunks of 32 columns are double-buffered: the next load is in flight while one is reduced.
      float mx;
      {
        float mx0 = -INFINITY, mx1 = -INFINITY;
        auto reduce = [&](const uint32_t (&r)[32], int c) {
          if (warp_masked) {
            const int kb = n0 + c * 32;
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              mx0 = fmaxf(mx0, kb + e > lim ? -INFINITY : __uint_as_float(r[e]));
              mx1 = fmaxf(mx1, kb + e + 1 > lim ? -INFINITY : __uint_as_float(r[e + 1]));
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              mx0 = fmaxf(mx0, __uint_as_float(r[e]));
              mx1 = fmaxf(mx1, __uint_as_float(r[e + 1]));
            }
          }
        };
        uint32_t ra[32], rb[32];
        umma::tmem_ld32(tSx, ra);
        umma::tmem_ld32_issue(tSx + 32, rb);
        reduce(ra, 0);
        umma::tmem_ld32_wait(rb);
        umma::tmem_ld32_issue(tSx + 64, ra);
        reduce(rb, 1);
        umma::tmem_ld32_wait(ra);
        umma::tmem_ld32_issue(tSx + 96, rb);
        reduce(ra, 2);
        umma::tmem_ld32_wait(rb);
        reduce(rb, 3);
        mx = fmaxf(mx0, mx1) * a.scale_log2;
      }
      // lazy rescale: move the reference maximum only when it grows by more than the threshold
      const bool need = mx > m_ref + kRescaleThreshold || (m_ref == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = need ? mx : m_ref;
        const float alpha = (m_ref == -INFINITY) ? (need ? 0.f : 1.f) : fast_exp2(m_ref - m_new);
        l *= alpha;
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            umma::tmem_ld32(tOx + c * 32, r);
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            umma::tmem_st32(tOx + c * 32, r);
          }
          umma::tmem_wait_st();
        }
        m_ref = m_new;
      }
      // pass 2: P = 2^(s * scale - m_ref) as bf16 into the first 64 columns of S, row sum in fp32;
      // the multiply-subtract and the row sum run two elements per instruction
      const float sub = m_ref == -INFINITY ? 0.f : m_ref;
      const uint64_t scale2 = umma::pack_f32x2(a.scale_log2, a.scale_log2);
      const uint64_t nsub2 = umma::pack_f32x2(-sub, -sub);
      uint64_t lsum2 = umma::pack_f32x2(0.f, 0.f);
      auto emit = [&](const uint32_t (&r)[32], int c) {
        uint32_t pk[16];
        const int kb = n0 + c * 32;
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float s0, s1;
          umma::unpack_f32x2(
              umma::fma_f32x2(umma::pack_f32x2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), scale2, nsub2),
              s0, s1);
          if (warp_masked) {
            if (kb + e > lim) s0 = -INFINITY;
            if (kb + e + 1 > lim) s1 = -INFINITY;
          }
          // every kPolyEvery-th pair takes the polynomial route to unload the special-function unit
          const bool poly = kPolyEvery > 0 && ((e >> 1) % (kPolyEvery > 0 ? kPolyEvery : 1)) == 0;
          const float p0 = poly ? umma::exp2_poly(s0) : fast_exp2(s0);
          const float p1 = poly ? umma::exp2_poly(s1) : fast_exp2(s1);
          lsum2 = umma::add_f32x2(lsum2, umma::pack_f32x2(p0, p1));
          pk[e >> 1] = pack_bf16x2(p0, p1);
        }
        umma::tmem_st16(tSx + c * 16, pk);
      };
      {
        uint32_t ra[32], rb[32];
        umma::tmem_ld32(tSx, ra);
        umma::tmem_ld32_issue(tSx + 32, rb);
        emit(ra, 0);
        umma::tmem_ld32_wait(rb);
        umma::tmem_ld32_issue(tSx + 64, ra);
        emit(rb, 1);
        umma::tmem_ld32_wait(ra);
        umma::tmem_ld32_issue(tSx + 96, rb);
        emit(ra, 2);
        umma::tmem_ld32_wait(rb);
        emit(rb, 3);
      }
      {
        float la, lb;
        umma::unpack_f32x2(lsum2, la, lb);
        l += la + lb;
      }
      umma::tmem_wait_st();
      umma::fence_before_sync();
      umma::mbar_arrive(bar(P_READY + x));
    }
    if (alive && __all_sync(0xffffffffu, umma::mbar_wait(bar(O_FINAL), 0, s_abort))) {
      umma::fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* op = a.out + (static_cast<int64_t>(q0 + qrow) * a.Hq + (x ? head_b : head_a)) * D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        umma::tmem_ld32(tOx + c * 32, r);     // warp-collective: every lane loads, valid rows store
        if (row < rows_q) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(r[e + 4]) * inv, __uint_as_float(r[e + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(r[e + 6]) * inv, __uint_as_float(r[e + 7]) * inv);
            *reinterpret_cast<uint4*>(op + c * 32 + e) = v;
          }
        }
      }
    } else if (alive) {
      give_up();
    }
  }
#undef WAIT_OR_ABORT
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 2) umma::tmem_dealloc(tmem, 512);
}


}  // namespace

namespace {

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

// [tokens, heads, 128] bf16 with a free token stride, seen as (d, head, token); one box is 64 columns
// of one head for 128 consecutive tokens, written to shared memory with the 128-byte swizzle.
bool make_map(CUtensorMap* m, const void* base, int64_t tokens, int heads, int64_t token_stride) {
  EncodeFn enc = tensor_map_encoder();
  if (enc == nullptr || tokens <= 0) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(heads),
                              static_cast<cuuint64_t>(tokens)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(token_stride) * 2};
  const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(BN)};
  const cuuint32_t estr[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int prefill_umma_launch(const void* q, const void* k, const void* v, void* out, int64_t q_stride,
                        int64_t k_stride, int64_t v_stride, int64_t total_q, int64_t total_k,
                        const int32_t* cu_q, const int32_t* cu_k, int num_seqs, int max_seqlen_q, int Hq, int Hkv, int Dqk, int Dv, float scale,
                        const void* kc, const void* vc, const int32_t* bt, int64_t bt_stride, int bs,
                        int64_t num_blocks, const int32_t* plan, int plan_tile_rows, int plan_capacity,
                        int32_t* status, cudaStream_t s) {
  const bool paged = bt != nullptr;
  if (Dqk != D || Dv != D || Hkv <= 0 || Hq % Hkv != 0 || ((Hq / Hkv) & 1)) return B200_ERR_UNSUPPORTED;
  if (!(scale > 0.f)) return B200_ERR_UNSUPPORTED;   // the row maximum is taken before scaling
  const int ntiles = (max_seqlen_q + BM - 1) / BM;
  if (num_seqs > 65535 || ntiles > 65535) return B200_ERR_UNSUPPORTED;
  auto al = [](const void* p, int64_t stride) { return aligned16(p) && (stride * 2) % 16 == 0; };
  if (!al(q, q_stride) || !aligned16(out)) return B200_ERR_UNSUPPORTED;
  if (paged ? !(aligned16(kc) && aligned16(vc)) : !(al(k, k_stride) && al(v, v_stride)))
    return B200_ERR_UNSUPPORTED;
  UmmaArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.q_stride = q_stride;
  a.k_stride = k_stride;
  a.v_stride = v_stride;
  a.cu_q = cu_q;
  a.cu_k = cu_k;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.ntiles_max = ntiles;
  a.plan = (plan != nullptr && plan_tile_rows == BM && plan_capacity > 0 && plan_capacity <= 65535) ? plan : nullptr;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.kc = static_cast<const __nv_bfloat16*>(kc);
  a.vc = static_cast<const __nv_bfloat16*>(vc);
  a.bt = bt;
  a.bt_stride = bt_stride;
  a.bs = bs;
  a.num_blocks = num_blocks;
  a.status = status;
  static bool configured[64][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = paged ? prefill_umma_kernel<true> : prefill_umma_kernel<false>;
  if (dev >= 0 && dev < 64 && !configured[dev][paged]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return B200_ERR_LAUNCH;
    configured[dev][paged] = true;
  }
  CUtensorMap tm_q, tm_k, tm_v;
  memset(&tm_q, 0, sizeof(tm_q));
  memset(&tm_k, 0, sizeof(tm_k));
  memset(&tm_v, 0, sizeof(tm_v));
  if (!paged) {
    // the token stride must be a multiple of 16 bytes for TMA (checked above)
    if (!make_map(&tm_q, q, total_q, Hq, q_stride) || !make_map(&tm_k, k, total_k, Hkv, k_stride) ||
        !make_map(&tm_v, v, total_k, Hkv, v_stride))
      return B200_ERR_UNSUPPORTED;   // falls back to the mma.sync kernel
  }
  dim3 grid(Hq / 2, num_seqs, ntiles);
  if (a.plan) grid = dim3(Hq / 2, plan_capacity, 1);
  kern<<<grid, kThreads, SMEM_BYTES, s>>>(a, tm_q, tm_k, tm_v);
  return launch_result();
}


}  // namespace b200
