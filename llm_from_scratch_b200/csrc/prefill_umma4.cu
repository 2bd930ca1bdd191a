// Ragged causal prefill attention on the Blackwell tensor cores (tcgen05) for head_dim 64 over packed
// keys/values, written for the regime of a serving engine's prefill steps: many short sequences (a few
// hundred tokens), grouped-query heads.
//
// One CTA owns 128 consecutive query rows of the FOUR query heads that share one KV head: four
// 128 x 64 problems that walk the same K/V tiles of 64 keys.  A tile staged in shared memory is used four
// times, and a CTA has four times the work of a one-head tile, which is what short sequences lack: with
// ~540-token prompts a (head, 256-row) tile meets at most nine key tiles, and the fixed cost of a CTA
// (tensor-memory allocation, barrier set-up, first TMA round trip) would dominate.
//
//   warp 0        K producer (+ the four Q tiles): one thread issuing TMA tile copies (128-byte swizzle)
//   warp 1        V producer
//   warps 2-5     lane 0 of warp 2 + x issues the tcgen05.mma of problem x; warp 2 owns the tensor memory
//   warps 6-9     softmax of problems 0 and 1, alternating: one thread per query row
//   warps 10-13   softmax of problems 2 and 3
//
// Tensor memory (512 columns): per problem a score buffer S 128 x 64 fp32 (bf16 P overwrites its first 32
// columns and is the A operand of O += P.V) and O 128 x 64 fp32.  With one score buffer per problem the
// order on a problem's issuing thread is S(j) -> wait for P(j) -> P(j).V(j) -> S(j+1); the tensor pipe is
// kept busy by the other three problems, and a softmax group works on one of its problems while the
// products of the other are in the pipe.  A commit covers every earlier tcgen05 operation of its thread, so
// when S(j) is announced P(j-1).V(j-1) has completed and O may be rescaled without a further wait.
// K/V tiles go through a ring of NST stages that all four problems release.  Every wait is bounded; a
// timeout aborts the CTA (status word B200_ERR_TIMEOUT) and the CTA still frees its tensor memory.
//
// Arithmetic: scaled_dot_product_attention of the reference (model/attention/utils.py:51-63) per sequence
// with the causal mask of model/transformer.py:174-176, KV heads shared as GQA.py:118-125.
#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace b200 {
namespace {

constexpr int BM = 128, BN = 64, D = 64, NP = 4;
constexpr int kThreads = (2 + NP + 8) * 32;     // 448
constexpr int Q_BYTES = BM * 128;               // one head: 128 rows x 64 columns
constexpr int K_BYTES = BN * 128, V_BYTES = BN * 128, STAGE = K_BYTES + V_BYTES;
constexpr int NST = 4;
constexpr float kRescaleThreshold = 8.f;        // log2 units

constexpr int OFF_Q = 0, OFF_KV = NP * Q_BYTES, OFF_BAR = OFF_KV + NST * STAGE;
// barriers: Q_FULL, per stage K_FULL, V_FULL, K_EMPTY, V_EMPTY (NP arrivals each), per problem S_FULL, P_READY,
// O_FINAL
constexpr int Q_FULL = 0, K_FULL = 1, V_FULL = 1 + NST, K_EMPTY = 1 + 2 * NST, V_EMPTY = 1 + 3 * NST,
              S_FULL = 1 + 4 * NST, P_READY = S_FULL + NP, O_FINAL = S_FULL + 2 * NP, TURN = S_FULL + 3 * NP,
              NUM_BARS = TURN + 8;   // TURN[softmax group][scheduler]: whose exponentials run next
constexpr int SMEM = OFF_BAR + NUM_BARS * 8 + 32 + 1024;   // + slack to align the base to 1024 bytes
constexpr int TCOLS = 512;

struct Args4 {
  __nv_bfloat16* out;
  const int32_t* cu_q;
  const int32_t* cu_k;
  int Hq, Hkv, ntiles_max;
  const int32_t* plan;   // tile list for 128-row tiles (see b200_prefill_plan) or null: grid (head group, seq, tile rank)
  float scale_log2;
  int32_t* status;
};

__global__ void __launch_bounds__(kThreads, 1)
prefill_umma4_kernel(const Args4 a, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(smem);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NUM_BARS * 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + OFF_BAR + NUM_BARS * 8 + 8);
  auto bar = [&](int i) -> uint32_t { return sb + OFF_BAR + i * 8; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = a.Hq / a.Hkv;
  const int head0 = blockIdx.x * NP;             // first of the four query heads; all share one KV head
  const int kvh = head0 / G;
  int seq, tile;
  if (a.plan) {                                  // grid (head group, tile-list slot)
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
  const int rows = min(BM, q_len - m0);
  int kmax = off + m0 + rows;                    // keys visible to the last row of the tile
  if (kmax > k_len) kmax = k_len;
  if (kmax < 1) kmax = 1;
  const int n = (kmax + BN - 1) / BN;            // KV tiles walked by the CTA; >= 1

  if (tid == 0) {
    umma::mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < NST; ++s) {
      umma::mbar_init(bar(K_FULL + s), 1);
      umma::mbar_init(bar(V_FULL + s), 1);
      umma::mbar_init(bar(K_EMPTY + s), NP);
      umma::mbar_init(bar(V_EMPTY + s), NP);
    }
    for (int x = 0; x < NP; ++x) {
      umma::mbar_init(bar(S_FULL + x), 1);
      umma::mbar_init(bar(P_READY + x), 128);
      umma::mbar_init(bar(O_FINAL + x), 1);
    }
    for (int i = 0; i < 8; ++i) umma::mbar_init(bar(TURN + i), 32);
    *s_abort = 0;
    umma::mbar_init_fence();
  }
  if (warp == 2) umma::tmem_alloc(sb + OFF_BAR + NUM_BARS * 8, TCOLS);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;

  auto give_up = [&]() {
    *s_abort = 1;
    report(a.status, B200_ERR_TIMEOUT);
  };
#define WAIT_OR_ABORT(idx, parity)                                   \
  if (!umma::mbar_wait(bar(idx), (parity), s_abort)) {               \
    give_up();                                                       \
    break;                                                           \
  }

  if (warp < 2) {
    // =============================== TMA producers ===============================
    if (lane == 0) {
      const bool is_k = warp == 0;
      if (is_k) {
        umma::mbar_expect_tx(bar(Q_FULL), NP * Q_BYTES);
        for (int x = 0; x < NP; ++x)
          umma::tma_load_3d(sb + OFF_Q + x * Q_BYTES, &tm_q, 0, head0 + x, q0 + m0, bar(Q_FULL));
      }
      const int full0 = is_k ? K_FULL : V_FULL, empty0 = is_k ? K_EMPTY : V_EMPTY;
      int j = 0;
      for (; j < n; ++j) {
        const int st = j % NST;
        if (j >= NST) WAIT_OR_ABORT(empty0 + st, ((j / NST) - 1) & 1)   // all four problems released the stage
        const uint32_t dst = sb + OFF_KV + st * STAGE + (is_k ? 0 : K_BYTES);
        umma::mbar_expect_tx(bar(full0 + st), is_k ? K_BYTES : V_BYTES);
        umma::tma_load_3d(dst, is_k ? &tm_k : &tm_v, 0, kvh, k0 + j * BN, bar(full0 + st));
      }
      if (*s_abort) {
        // copies still in flight must land before the CTA gives its shared memory back
        int never = 0;
        if (is_k) umma::mbar_wait(bar(Q_FULL), 0, &never, 1 << 16);
        for (int x = max(0, j - NST); x < j; ++x)
          umma::mbar_wait(bar(full0 + x % NST), (x / NST) & 1, &never, 1 << 16);
      }
    }
  } else if (warp < 2 + NP) {
    // =============================== MMA issuers ===============================
    const int x = warp - 2;                      // problem = query head head0 + x
    if (lane == 0) {
      const uint32_t idesc_qk = umma::instr_desc_bf16(BM, BN, false, false);
      const uint32_t idesc_pv = umma::instr_desc_bf16(BM, D, false, true);
      const uint32_t qbase = sb + OFF_Q + x * Q_BYTES;
      const uint32_t tS = tmem + x * 128, tO = tS + 64;
      bool ok = umma::mbar_wait(bar(Q_FULL), 0, s_abort);
      if (!ok) give_up();
      for (int j = 0; ok && j < n; ++j) {
        const int st = j % NST, ph = (j / NST) & 1;
        WAIT_OR_ABORT(K_FULL + st, ph)
        umma::fence_after_sync();
        const uint32_t kbase = sb + OFF_KV + st * STAGE, vbase = kbase + K_BYTES;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)        // S = Q . K_j^T : contraction over d in steps of 16
          umma::mma_ss(tS, umma::smem_desc(qbase + ks * 32, 0, 1024), umma::smem_desc(kbase + ks * 32, 0, 1024),
                       idesc_qk, ks > 0);
        umma::commit(bar(S_FULL + x));
        umma::commit(bar(K_EMPTY + st));
        WAIT_OR_ABORT(P_READY + x, j & 1)
        WAIT_OR_ABORT(V_FULL + st, ph)
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks)       // O += P . V_j : contraction over the 64 keys
          umma::mma_ts(tO, tS + ks * 8, umma::smem_desc(vbase + ks * 2048, K_BYTES, 1024), idesc_pv,
                       !(j == 0 && ks == 0));
        umma::commit(bar(V_EMPTY + st));
        if (j == n - 1) umma::commit(bar(O_FINAL + x));
      }
    }
  } else {
    // =============================== softmax / epilogue ===============================
    const int grp = (warp - (2 + NP)) >> 2;                 // 0: problems 0, 1;  1: problems 2, 3
    const int row = (warp & 3) * 32 + lane;                 // query row of the tile == tensor-memory lane
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int qrow = m0 + row;                              // index of the query inside its sequence
    const int lim = min(off + qrow, kmax - 1);              // last visible key
    float m_ref[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    bool alive = true;
    for (int j = 0; j < n && alive; ++j) {
      const int n0 = j * BN;
      const bool warp_masked = __any_sync(0xffffffffu, n0 + BN - 1 > lim);
#pragma unroll
      for (int pp = 0; pp < 2; ++pp) {
        const int x = grp * 2 + pp;
        const uint32_t tSx = tmem + x * 128 + lane_sel, tOx = tSx + 64;
        // tensor-memory loads / stores are warp-collective: the whole warp continues or stops together
        if (!__all_sync(0xffffffffu, umma::mbar_wait(bar(S_FULL + x), j & 1, s_abort))) {
          give_up();
          alive = false;
          break;
        }
        umma::fence_after_sync();
        // the 64 raw scores of the row stay in registers for both passes
        uint32_t ra[32], rb[32];
        umma::tmem_ld32(tSx, ra);
        umma::tmem_ld32_issue(tSx + 32, rb);
        float mx0 = -INFINITY, mx1 = -INFINITY;
        if (warp_masked) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (n0 + e > lim) ra[e] = 0xff800000u;          // -inf
        }
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          mx0 = fmaxf(mx0, __uint_as_float(ra[e]));
          mx1 = fmaxf(mx1, __uint_as_float(ra[e + 1]));
        }
        umma::tmem_ld32_wait(rb);
        if (warp_masked) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (n0 + 32 + e > lim) rb[e] = 0xff800000u;
        }
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          mx0 = fmaxf(mx0, __uint_as_float(rb[e]));
          mx1 = fmaxf(mx1, __uint_as_float(rb[e + 1]));
        }
        const float mx = fmaxf(mx0, mx1) * a.scale_log2;    // the scale is positive: it commutes with max
        // lazy rescale: move the reference maximum only when it grows by more than the threshold
        const bool need = mx > m_ref[pp] + kRescaleThreshold || (m_ref[pp] == -INFINITY && mx > -INFINITY);
        if (__any_sync(0xffffffffu, need)) {
          const float m_new = need ? mx : m_ref[pp];
          const float alpha = (m_ref[pp] == -INFINITY) ? (need ? 0.f : 1.f) : fast_exp2(m_ref[pp] - m_new);
          l[pp] *= alpha;
          if (j > 0) {     // P(j-1).V(j-1) has completed: it was issued before the scores just announced
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
              uint32_t r[32];
              umma::tmem_ld32(tOx + c * 32, r);
#pragma unroll
              for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
              umma::tmem_st32(tOx + c * 32, r);
            }
            umma::tmem_wait_st();
          }
          m_ref[pp] = m_new;
        }
        // The exponentials of the two softmax warps of a scheduler (this row quarter of either group) take turns:
        // group 0's k-th tile, group 1's k-th, group 0's (k + 1)-th, ...  Left alone the two warps run in step,
        // share the special-function unit during their exponentials (64 per row and tile: 512 clocks per warp,
        // more than the tensor pipe needs for the tile at this head dimension) and leave it idle during their
        // loads and maxima; in turns one warp's loads, maxima and waits run under the other's exponentials.
        {
          const int k = 2 * j + pp;
          if (grp == 0 ? k >= 1 : true) {
            if (!__all_sync(0xffffffffu, umma::mbar_wait(bar(TURN + grp * 4 + (warp & 3)), (grp == 0 ? k - 1 : k) & 1,
                                                         s_abort))) {
              give_up();
              alive = false;
              break;
            }
          }
        }
        // P = 2^(s * scale - m_ref) as bf16 into the first 32 columns of S, row sum in fp32
        const float sub = m_ref[pp] == -INFINITY ? 0.f : m_ref[pp];
        const uint64_t scale2 = umma::pack_f32x2(a.scale_log2, a.scale_log2);
        const uint64_t nsub2 = umma::pack_f32x2(-sub, -sub);
        uint64_t lsum2 = umma::pack_f32x2(0.f, 0.f);
        auto emit = [&](const uint32_t (&r)[32], int c) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float s0, s1;
            umma::unpack_f32x2(
                umma::fma_f32x2(umma::pack_f32x2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), scale2, nsub2),
                s0, s1);
            const float p0 = fast_exp2(s0), p1 = fast_exp2(s1);   // 2^-inf = 0 for masked keys
            lsum2 = umma::add_f32x2(lsum2, umma::pack_f32x2(p0, p1));
            pk[e >> 1] = pack_bf16x2(p0, p1);
          }
          umma::tmem_st16(tSx + c * 16, pk);
        };
        emit(ra, 0);
        emit(rb, 1);
        umma::mbar_arrive(bar(TURN + (grp ^ 1) * 4 + (warp & 3)));   // the other group's turn
        {
          float la, lb;
          umma::unpack_f32x2(lsum2, la, lb);
          l[pp] += la + lb;
        }
        umma::tmem_wait_st();
        umma::fence_before_sync();
        umma::mbar_arrive(bar(P_READY + x));
      }
    }
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
      const int x = grp * 2 + pp;
      const uint32_t tOx = tmem + x * 128 + 64 + lane_sel;
      if (alive && __all_sync(0xffffffffu, umma::mbar_wait(bar(O_FINAL + x), 0, s_abort))) {
        umma::fence_after_sync();
        const float inv = l[pp] > 0.f ? 1.f / l[pp] : 0.f;
        __nv_bfloat16* op = a.out + (static_cast<int64_t>(q0 + qrow) * a.Hq + head0 + x) * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          umma::tmem_ld32(tOx + c * 32, r);     // warp-collective: every lane loads, valid rows store
          if (row < rows) {
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
        alive = false;
      }
    }
  }
#undef WAIT_OR_ABORT
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 2) umma::tmem_dealloc(tmem, TCOLS);
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn tensor_map_encoder4() {
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

// [tokens, heads, 64] bf16 with a free token stride, seen as (d, head, token); one box is the 64 columns of
// one head for `box_rows` consecutive tokens, written to shared memory with the 128-byte swizzle.
bool make_map4(CUtensorMap* m, const void* base, int64_t tokens, int heads, int64_t token_stride, int box_rows) {
  EncodeFn enc = tensor_map_encoder4();
  if (enc == nullptr || tokens <= 0) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(heads),
                              static_cast<cuuint64_t>(tokens)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(token_stride) * 2};
  const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Query rows per CTA of this kernel for a shape it serves, else 0: head_dim 64 with the query heads of a KV
// head in whole groups of four.
int prefill_umma4_tile_rows(int Hq, int Hkv, int Dqk, int Dv) {
  if (Hkv <= 0 || Hq % Hkv != 0) return 0;
  const int G = Hq / Hkv;
  return (Dqk == D && Dv == D && G % NP == 0) ? BM : 0;
}

// Packed keys/values only.  Returns B200_ERR_UNSUPPORTED for anything it does not implement (the caller then
// uses the mma.sync kernel).
int prefill_umma4_launch(const void* q, const void* k, const void* v, void* out, int64_t q_stride, int64_t k_stride,
                         int64_t v_stride, int64_t total_q, int64_t total_k, const int32_t* cu_q,
                         const int32_t* cu_k, int num_seqs, int max_seqlen_q, int Hq, int Hkv, int Dqk, int Dv,
                         float scale, const int32_t* plan, int plan_tile_rows, int plan_capacity, int32_t* status,
                         cudaStream_t s) {
  if (prefill_umma4_tile_rows(Hq, Hkv, Dqk, Dv) == 0) return B200_ERR_UNSUPPORTED;
  if (!(scale > 0.f)) return B200_ERR_UNSUPPORTED;   // the row maximum is taken before scaling
  const int ntiles = (max_seqlen_q + BM - 1) / BM;
  if (num_seqs > 65535 || ntiles > 65535 || Hq > 65535) return B200_ERR_UNSUPPORTED;
  auto al = [](const void* p, int64_t stride) { return p != nullptr && aligned16(p) && (stride * 2) % 16 == 0; };
  if (!al(q, q_stride) || !al(k, k_stride) || !al(v, v_stride) || !aligned16(out)) return B200_ERR_UNSUPPORTED;
  Args4 a{};
  a.out = static_cast<__nv_bfloat16*>(out);
  a.cu_q = cu_q;
  a.cu_k = cu_k;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.ntiles_max = ntiles;
  a.plan = (plan != nullptr && plan_tile_rows == BM && plan_capacity > 0 && plan_capacity <= 65535) ? plan : nullptr;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  CUtensorMap tq, tk, tv;
  memset(&tq, 0, sizeof(tq));
  memset(&tk, 0, sizeof(tk));
  memset(&tv, 0, sizeof(tv));
  if (!make_map4(&tq, q, total_q, Hq, q_stride, BM) || !make_map4(&tk, k, total_k, Hkv, k_stride, BN) ||
      !make_map4(&tv, v, total_k, Hkv, v_stride, BN))
    return B200_ERR_UNSUPPORTED;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
  static bool configured[64] = {};    // per-device flag, written without a lock (idempotent)
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return B200_ERR_UNSUPPORTED;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(prefill_umma4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return B200_ERR_LAUNCH;
    configured[dev] = true;
  }
  dim3 grid(Hq / NP, num_seqs, ntiles);
  if (a.plan) grid = dim3(Hq / NP, plan_capacity, 1);
  prefill_umma4_kernel<<<grid, kThreads, SMEM, s>>>(a, tq, tk, tv);
  return launch_result();
}

}  // namespace b200
