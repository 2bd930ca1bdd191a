// Ragged causal prefill attention on the Blackwell tensor cores (tcgen05) over packed keys/values, head
// dims 128/128 (any group size) and 192/128 (the expanded form of multi-head latent attention, MLA.py:131,
// with the rotary key part read from a tensor shared by all heads or from the key tensor itself).
//
// One CTA owns 256 consecutive query rows of ONE head: two 128-row problems A (rows 0-127) and B
// (rows 128-255) that walk the same K/V tiles of 64 keys, so a tile staged in shared memory is used
// twice and the tensor core works on one problem while the softmax warps of the other turn S into P.
// Problem B sees up to two more key tiles than A (causal mask); A simply stops earlier.
//
//   warp 0      K producer (+ both Q tiles): one thread issuing TMA tile copies (128-byte swizzle)
//   warp 1      V producer
//   warp 2      tensor-memory allocation; lane 0 issues the tcgen05.mma of problem A
//   warp 3      lane 0 issues the tcgen05.mma of problem B
//   warps 4-7   softmax of A: one thread per query row, the 64 scores of a tile held in registers
//   warps 8-11  softmax of B
//
// Tensor memory per problem (256 columns): two score buffers S 128 x 64 fp32 (bf16 P overwrites the first
// 32 columns of its buffer and is the A operand of O += P.V) and O 128 x DV fp32.  Each issuing thread puts
// the scores of tile j + 1 into the other buffer before it waits for the probabilities of tile j, so the
// softmax warps find their next tile ready, and one problem's waits never hold up the other's instructions.
// K/V tiles go through a ring of NST stages that both problems release.  Rescaling of O is lazy as in
// prefill_umma.cu and waits for the P.V product before it.  Every wait is bounded; a timeout aborts the CTA
// and is reported.
//
// What sets the pace, measured with clock counters in the warps: (1) the special-function unit — the 64
// exponentials of a row tile occupy it for 512 clocks per warp, and the A and B warps of a scheduler, left
// alone, run in step, share it during their exponentials (1,200 clocks each) and leave it idle during their
// loads and maxima; their exponential phases therefore take turns (A(j), B(j), A(j + 1), ...; 650 clocks each),
// and one warp's loads, maxima and waits run under the other's exponentials; (2) the issuing threads' own
// instruction streams (each shares its scheduler with two softmax warps): descriptors are formed once and only
// their address field advanced, and one tcgen05.commit per product serves every waiter (the barrier that frees a
// K stage also announces the scores computed from it, the barrier that frees a V stage also announces the
// product into O).
#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace b200 {
namespace {

constexpr int BM = 128, BN = 64, ROWS = 2 * BM;
constexpr int kThreads = 384;
constexpr int Q_SLAB = BM * 128;   // 64 columns of 128 rows
constexpr int K_SLAB = BN * 128;   // 64 columns of 64 rows
constexpr float kRescaleThreshold = 8.f;   // log2 units

template <int DQK, int DV>
struct Lay {
  static constexpr int QS = DQK / 64, VS = DV / 64;
  static constexpr int Q_BYTES = QS * Q_SLAB, K_BYTES = QS * K_SLAB, V_BYTES = VS * K_SLAB;
  static constexpr int STAGE = K_BYTES + V_BYTES;
  static constexpr int NST = DQK >= 192 ? 3 : 4;
  static constexpr int OFF_QA = 0, OFF_QB = Q_BYTES, OFF_KV = 2 * Q_BYTES;
  static constexpr int OFF_BAR = OFF_KV + NST * STAGE;
  // barriers: Q_FULL; per stage K_FULL, V_FULL; per stage and problem QK_DONE (the scores of the tile in this
  // stage are in tensor memory, and the K stage is free for this problem) and PV_DONE (the product of the tile
  // in this stage is in O, and the V stage is free for this problem); per problem and score buffer P_READY;
  // per scheduler TURN_A, TURN_B (whose exponentials run next).
  // P_READY is per buffer because the softmax warps may finish tile j + 1 before the issuing thread has looked at
  // tile j (the scores of both were issued ahead); a single barrier would then have completed two phases and a
  // wait by parity could not tell tile j from tile j + 2.  No other barrier can run two phases ahead of a waiter.
  static constexpr int Q_FULL = 0, K_FULL = 1, V_FULL = 1 + NST, QK_DONE = 1 + 2 * NST, PV_DONE = 1 + 4 * NST,
                       P_READY = 1 + 6 * NST, TURN = P_READY + 4, NUM_BARS = TURN + 8;
  static constexpr int SMEM = OFF_BAR + NUM_BARS * 8 + 32 + 1024;   // + slack to align the base to 1024 bytes
  static constexpr int TCOLS_USED = 2 * (128 + DV);   // per problem: two score buffers of 64 columns + O
  static constexpr int TCOLS = TCOLS_USED > 256 ? 512 : 256;
};

struct Args2 {
  __nv_bfloat16* out;
  const int32_t* cu_q;
  const int32_t* cu_k;
  int Hq, Hkv, ntiles_max;
  const int32_t* plan;   // tile list for 256-row tiles (see b200_prefill_plan) or null: grid (head, seq, tile rank)
  float scale_log2;
  int32_t* status;
};

template <int DQK, int DV, bool TAIL>
__global__ void __launch_bounds__(kThreads, 1)
prefill_umma2_kernel(const Args2 a, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_kt, const __grid_constant__ CUtensorMap tm_v) {
  using L = Lay<DQK, DV>;
  constexpr int NST = L::NST;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(smem);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + L::OFF_BAR + L::NUM_BARS * 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + L::OFF_BAR + L::NUM_BARS * 8 + 8);
  auto bar = [&](int i) -> uint32_t { return sb + L::OFF_BAR + i * 8; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.x;
  int seq, tile;
  if (a.plan) {                                  // grid (head, tile-list slot)
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
  const int m0 = tile * ROWS;
  if (m0 >= q_len) return;                       // uniform over the CTA, before any barrier / allocation
  const int off = k_len - q_len;
  const int kvh = head / (a.Hq / a.Hkv);
  // rows and visible keys of the two problems; B may be empty (the sequence ends inside A)
  int rows[2], kmax[2], nt[2];
  rows[0] = min(BM, q_len - m0);
  rows[1] = max(0, min(BM, q_len - m0 - BM));
  for (int x = 0; x < 2; ++x) {
    int km = off + m0 + x * BM + rows[x];
    if (km > k_len) km = k_len;
    if (km < 1) km = 1;
    kmax[x] = km;
    nt[x] = rows[x] > 0 ? (km + BN - 1) / BN : 0;
  }
  const bool has_b = rows[1] > 0;
  const int n = max(nt[0], nt[1]);               // KV tiles walked by the CTA; >= 1

  if (tid == 0) {
    umma::mbar_init(bar(L::Q_FULL), 1);
    for (int s = 0; s < NST; ++s) {
      umma::mbar_init(bar(L::K_FULL + s), 1);
      umma::mbar_init(bar(L::V_FULL + s), 1);
      for (int x = 0; x < 2; ++x) {
        umma::mbar_init(bar(L::QK_DONE + 2 * s + x), 1);
        umma::mbar_init(bar(L::PV_DONE + 2 * s + x), 1);
      }
    }
    for (int i = 0; i < 4; ++i) umma::mbar_init(bar(L::P_READY + i), 128);
    for (int i = 0; i < 8; ++i) umma::mbar_init(bar(L::TURN + i), 32);
    *s_abort = 0;
    umma::mbar_init_fence();
  }
  if (warp == 2) umma::tmem_alloc(sb + L::OFF_BAR + L::NUM_BARS * 8, L::TCOLS);
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
        umma::mbar_expect_tx(bar(L::Q_FULL), (has_b ? 2 : 1) * L::Q_BYTES);
        for (int x = 0; x < (has_b ? 2 : 1); ++x)
          for (int h = 0; h < L::QS; ++h)
            umma::tma_load_3d(sb + (x ? L::OFF_QB : L::OFF_QA) + h * Q_SLAB, &tm_q, h * 64, head,
                              q0 + m0 + x * BM, bar(L::Q_FULL));
      }
      const int full0 = is_k ? L::K_FULL : L::V_FULL, empty0 = is_k ? L::QK_DONE : L::PV_DONE;
      for (int j = 0; j < n; ++j) {
        const int st = j % NST;
        if (j >= NST) {   // both problems must have released the tile that occupied this stage
          if (j - NST < nt[0]) WAIT_OR_ABORT(empty0 + 2 * st, ((j / NST) - 1) & 1)
          if (j - NST < nt[1]) WAIT_OR_ABORT(empty0 + 2 * st + 1, ((j / NST) - 1) & 1)
        }
        const uint32_t dst = sb + L::OFF_KV + st * L::STAGE + (is_k ? 0 : L::K_BYTES);
        if (is_k) {
          umma::mbar_expect_tx(bar(full0 + st), L::K_BYTES);
          for (int h = 0; h < L::QS; ++h) {
            if (TAIL && h == L::QS - 1)
              umma::tma_load_3d(dst + h * K_SLAB, &tm_kt, 0, 0, k0 + j * BN, bar(full0 + st));
            else
              umma::tma_load_3d(dst + h * K_SLAB, &tm_k, h * 64, kvh, k0 + j * BN, bar(full0 + st));
          }
        } else {
          umma::mbar_expect_tx(bar(full0 + st), L::V_BYTES);
          for (int h = 0; h < L::VS; ++h)
            umma::tma_load_3d(dst + h * K_SLAB, &tm_v, h * 64, kvh, k0 + j * BN, bar(full0 + st));
        }
      }
    }
  } else if (warp < 4) {
    // =============================== MMA issuers ===============================
    const int x = warp - 2;
    if (lane == 0 && nt[x] > 0) {
      const uint32_t idesc_qk = umma::instr_desc_bf16(BM, BN, false, false);
      const uint32_t idesc_pv = umma::instr_desc_bf16(BM, DV, false, true);
      const int nx = nt[x];
      const uint64_t qd = umma::smem_desc(sb + (x ? L::OFF_QB : L::OFF_QA), 0, 1024);
      const uint64_t kd = umma::smem_desc(sb + L::OFF_KV, 0, 1024);
      const uint64_t vd = umma::smem_desc(sb + L::OFF_KV + L::K_BYTES, K_SLAB, 1024);
      const uint32_t tSx = tmem + x * (128 + DV), tOx = tSx + 128;
      auto qk = [&](int st, int buf) {       // S[buf] = Q . K^T of the tile in stage st, contraction in steps of 16
        const uint32_t so = st * (L::STAGE >> 4);
#pragma unroll
        for (int ks = 0; ks < DQK / 16; ++ks)
          umma::mma_ss(tSx + buf * 64, umma::desc_advance(qd, ((ks >> 2) * Q_SLAB + (ks & 3) * 32) >> 4),
                       umma::desc_advance(kd, so + (((ks >> 2) * K_SLAB + (ks & 3) * 32) >> 4)), idesc_qk, ks > 0);
        umma::commit(bar(L::QK_DONE + x) + st * 16);
      };
      bool ok = umma::mbar_wait(bar(L::Q_FULL), 0, s_abort) && umma::mbar_wait(bar(L::K_FULL + 0), 0, s_abort);
      if (!ok) give_up();
      if (ok) {
        umma::fence_after_sync();
        qk(0, 0);
      }
      int st = 0, ph = 0;                      // stage and phase of tile j
      for (int j = 0; ok && j < nx; ++j) {
        int st1 = st + 1, ph1 = ph;
        if (st1 == NST) {
          st1 = 0;
          ph1 ^= 1;
        }
        if (j + 1 < nx) {
          WAIT_OR_ABORT(L::K_FULL + st1, ph1)
          umma::fence_after_sync();
          qk(st1, (j + 1) & 1);
        }
        WAIT_OR_ABORT(L::P_READY + 2 * x + (j & 1), (j >> 1) & 1)
        WAIT_OR_ABORT(L::V_FULL + st, ph)
        umma::fence_after_sync();
        const uint32_t so = st * (L::STAGE >> 4);
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks)        // O += P[j & 1] . V_j : contraction over the 64 keys
          umma::mma_ts(tOx, tSx + (j & 1) * 64 + ks * 8, umma::desc_advance(vd, so + ks * (2048 >> 4)), idesc_pv,
                       !(j == 0 && ks == 0));
        umma::commit(bar(L::PV_DONE + x) + st * 16);
        st = st1;
        ph = ph1;
      }
    }
  } else {
    // =============================== softmax / epilogue ===============================
    const int x = warp >= 8 ? 1 : 0;                        // problem A or B
    const int row = (warp & 3) * 32 + lane;                 // query row of the problem == tensor-memory lane
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS0 = tmem + x * (128 + DV) + lane_sel, tOx = tS0 + 128;
    const int qrow = m0 + x * BM + row;                     // index of the query inside its sequence
    const int lim = min(off + qrow, kmax[x] - 1);           // last visible key
    const int nx = nt[x];
    const uint32_t qk_done = bar(L::QK_DONE + x), pv_done = bar(L::PV_DONE + x);
    const uint32_t my_turn = bar(L::TURN + (x == 0 ? 0 : 4) + (warp & 3));
    const uint32_t their_turn = bar(L::TURN + (x == 0 ? 4 : 0) + (warp & 3));
    float m_ref = -INFINITY, l = 0.f;
    bool alive = true;
    int st = 0, ph = 0, stp = 0, php = 0;                   // stage and phase of tile j and of tile j - 1
    for (int j = 0; j < nx; ++j) {
      // tensor-memory loads / stores are warp-collective: the whole warp continues or stops together
      const uint32_t tSx = tS0 + (j & 1) * 64;                // score buffer of this tile
      if (!__all_sync(0xffffffffu, umma::mbar_wait(qk_done + st * 16, ph, s_abort))) {
        give_up();
        alive = false;
        break;
      }
      umma::fence_after_sync();
      const int n0 = j * BN;
      const bool warp_masked = __any_sync(0xffffffffu, n0 + BN - 1 > lim);
      // the 64 raw scores of the row stay in registers for both passes
      uint32_t ra[32], rb[32];
      umma::tmem_ld32(tSx, ra);
      umma::tmem_ld32_issue(tSx + 32, rb);
      float mx0 = -INFINITY, mx1 = -INFINITY;
      if (warp_masked) {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (n0 + e > lim) ra[e] = 0xff800000u;            // -inf
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
      const float mx = fmaxf(mx0, mx1) * a.scale_log2;      // the scale is positive: it commutes with max
      // lazy rescale: move the reference maximum only when it grows by more than the threshold
      const bool need = mx > m_ref + kRescaleThreshold || (m_ref == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = need ? mx : m_ref;
        const float alpha = (m_ref == -INFINITY) ? (need ? 0.f : 1.f) : fast_exp2(m_ref - m_new);
        l *= alpha;
        if (j > 0) {
          // O still receives P(j-1).V(j-1): the scores of this tile were issued ahead of that product
          if (!__all_sync(0xffffffffu, umma::mbar_wait(pv_done + stp * 16, php, s_abort))) {
            give_up();
            alive = false;
            break;
          }
          umma::fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < DV / 32; ++c) {
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
      // whose exponentials run now: A(j) follows B(j - 1), B(j) follows A(j) while A has tiles left
      if (x == 0 ? (has_b && j >= 1) : (j < nt[0])) {
        if (!__all_sync(0xffffffffu, umma::mbar_wait(my_turn, (x == 0 ? j - 1 : j) & 1, s_abort))) {
          give_up();
          alive = false;
          break;
        }
      }
      // P = 2^(s * scale - m_ref) as bf16 into the first 32 columns of S, row sum in fp32
      const float sub = m_ref == -INFINITY ? 0.f : m_ref;
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
      umma::mbar_arrive(their_turn);
      {
        float la, lb;
        umma::unpack_f32x2(lsum2, la, lb);
        l += la + lb;
      }
      umma::tmem_wait_st();
      umma::fence_before_sync();
      umma::mbar_arrive(bar(L::P_READY + 2 * x + (j & 1)));
      stp = st;
      php = ph;
      if (++st == NST) {
        st = 0;
        ph ^= 1;
      }
    }
    if (nx > 0) {
      // the last product: stp / php are the stage and phase of tile nx - 1
      if (alive && __all_sync(0xffffffffu, umma::mbar_wait(pv_done + stp * 16, php, s_abort))) {
        umma::fence_after_sync();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* op = a.out + (static_cast<int64_t>(q0 + qrow) * a.Hq + head) * DV;
#pragma unroll 1
        for (int c = 0; c < DV / 32; ++c) {
          uint32_t r[32];
          umma::tmem_ld32(tOx + c * 32, r);     // warp-collective: every lane loads, valid rows store
          if (row < rows[x]) {
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
  }
#undef WAIT_OR_ABORT
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 2) umma::tmem_dealloc(tmem, L::TCOLS);
}

}  // namespace

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn tensor_map_encoder2() {
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

// [tokens, heads, width] bf16 with a free token stride, seen as (d, head, token); one box is 64 columns of
// one head for `box_rows` consecutive tokens, written to shared memory with the 128-byte swizzle.
bool make_map2(CUtensorMap* m, const void* base, int64_t tokens, int heads, int width, int64_t token_stride,
               int box_rows) {
  EncodeFn enc = tensor_map_encoder2();
  if (enc == nullptr || tokens <= 0) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(heads),
                              static_cast<cuuint64_t>(tokens)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(width) * 2, static_cast<cuuint64_t>(token_stride) * 2};
  const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int DQK, int DV, bool TAIL>
int launch2(const Args2& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tkt,
            const CUtensorMap& tv, dim3 grid, cudaStream_t s) {
  using L = Lay<DQK, DV>;
  static_assert(L::SMEM <= 227 * 1024, "shared memory budget");
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return B200_ERR_UNSUPPORTED;
  auto kern = prefill_umma2_kernel<DQK, DV, TAIL>;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM) != cudaSuccess)
      return B200_ERR_LAUNCH;
    configured[dev] = true;
  }
  kern<<<grid, kThreads, L::SMEM, s>>>(a, tq, tk, tkt, tv);
  return launch_result();
}

}  // namespace

// Query rows per CTA of this kernel for a shape it serves, else 0.
int prefill_umma2_tile_rows(int Hq, int Hkv, int Dqk, int Dv) {
  if (Hkv <= 0 || Hq % Hkv != 0) return 0;
  // head_dim 64 has a kernel of its own (prefill_umma4.cu, four heads of a KV head per CTA): one head per CTA
  // leaves a CTA too little work on short sequences (76 us per layer here on 7,300-token batches of ~540-token
  // sequences against 36 us there)
  const bool ok = (Dqk == 192 && Dv == 128) || (Dqk == 128 && Dv == 128);
  return ok ? ROWS : 0;
}

// Packed keys/values only.  k_tail != null: the last `tail` (= 64) columns of every head's key come from
// k_tail [total_k, tail] and k holds Dqk - tail columns per head.  Returns B200_ERR_UNSUPPORTED for
// anything it does not implement (the caller then uses the mma.sync kernel).
int prefill_umma2_launch(const void* q, const void* k, const void* v, void* out, int64_t q_stride, int64_t k_stride,
                         int64_t v_stride, int64_t total_q, int64_t total_k, const int32_t* cu_q,
                         const int32_t* cu_k, int num_seqs, int max_seqlen_q, int Hq, int Hkv, int Dqk, int Dv,
                         float scale, const int32_t* plan, int plan_tile_rows, int plan_capacity, int32_t* status,
                         cudaStream_t s, const void* k_tail, int64_t k_tail_stride, int tail) {
  if (prefill_umma2_tile_rows(Hq, Hkv, Dqk, Dv) == 0) return B200_ERR_UNSUPPORTED;
  if (tail != 0 && (tail != 64 || Dqk != 192 || k_tail == nullptr)) return B200_ERR_UNSUPPORTED;
  if (!(scale > 0.f)) return B200_ERR_UNSUPPORTED;   // the row maximum is taken before scaling
  const int ntiles = (max_seqlen_q + ROWS - 1) / ROWS;
  if (num_seqs > 65535 || ntiles > 65535 || Hq > 65535) return B200_ERR_UNSUPPORTED;
  auto al = [](const void* p, int64_t stride) { return p != nullptr && aligned16(p) && (stride * 2) % 16 == 0; };
  if (!al(q, q_stride) || !al(k, k_stride) || !al(v, v_stride) || !aligned16(out)) return B200_ERR_UNSUPPORTED;
  if (tail && !al(k_tail, k_tail_stride)) return B200_ERR_UNSUPPORTED;
  Args2 a{};
  a.out = static_cast<__nv_bfloat16*>(out);
  a.cu_q = cu_q;
  a.cu_k = cu_k;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.ntiles_max = ntiles;
  a.plan = (plan != nullptr && plan_tile_rows == ROWS && plan_capacity > 0 && plan_capacity <= 65535) ? plan : nullptr;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  CUtensorMap tq, tk, tkt, tv;
  memset(&tq, 0, sizeof(tq));
  memset(&tk, 0, sizeof(tk));
  memset(&tkt, 0, sizeof(tkt));
  memset(&tv, 0, sizeof(tv));
  if (!make_map2(&tq, q, total_q, Hq, Dqk, q_stride, BM) || !make_map2(&tk, k, total_k, Hkv, Dqk - tail, k_stride, BN) ||
      !make_map2(&tv, v, total_k, Hkv, Dv, v_stride, BN))
    return B200_ERR_UNSUPPORTED;
  if (tail && !make_map2(&tkt, k_tail, total_k, 1, tail, k_tail_stride, BN)) return B200_ERR_UNSUPPORTED;
  dim3 grid(Hq, num_seqs, ntiles);
  if (a.plan) grid = dim3(Hq, plan_capacity, 1);
  if (Dqk == 192) {
    return tail ? launch2<192, 128, true>(a, tq, tk, tkt, tv, grid, s)
                : launch2<192, 128, false>(a, tq, tk, tkt, tv, grid, s);
  }
  return launch2<128, 128, false>(a, tq, tk, tkt, tv, grid, s);
}

}  // namespace b200
