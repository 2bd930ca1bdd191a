// Ragged causal prefill attention, bf16, mma.sync path.
//
// One CTA (4 warps) owns a 64-row query tile of one (sequence, query head) and streams the
// sequence's keys/values in 64-row tiles through a 2-stage cp.async ring; tiles above the causal
// diagonal are never loaded.  S = Q.K^T and O += P.V run on mma.sync m16n8k16 with fp32
// accumulators, softmax is the online form in the log2 domain with quad shuffles for the row
// statistics.  Keys/values come from the packed k/v tensors of the step or, when part of the
// context is already cached, from the paged pool through the block table (the mask is then
// bottom-right aligned: query i of a sequence sees keys 0 .. k_len - q_len + i).
//
// The grid is (query heads, sequences, query tiles) with the tile index reversed, so that the
// tiles with the most keys are scheduled first and the short tail of a ragged batch fills the
// gaps; CTAs whose tile lies past the end of their sequence return at once.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int BM = 64;   // query rows per CTA
constexpr int BN = 64;   // key rows per tile
constexpr int kThreads = 128;

struct MmaArgs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  __nv_bfloat16* out;
  int64_t q_stride, k_stride, v_stride;  // elements between tokens
  // keys in two parts (packed K only): columns [0, DQK - tail) per kv head from `k`, the last `tail`
  // columns from `k_tail`, one row per token shared by every head (MLA's rotary key part)
  const __nv_bfloat16* k_tail;
  int64_t k_tail_stride;
  const int32_t* cu_q;
  const int32_t* cu_k;
  int Hq, Hkv, ntiles_max;
  const int32_t* plan;   // tile list (see b200_prefill_plan) or null: grid (head, seq, tile rank)
  float scale_log2;
  const __nv_bfloat16* kc;
  const __nv_bfloat16* vc;
  const int32_t* bt;
  int64_t bt_stride;
  int bs;
  int64_t num_blocks;
  int32_t* status;
};

template <int D>
__device__ __forceinline__ int swz(int c, int row) {
  constexpr int CPR = D / 8;
  if (CPR >= 8) return c ^ (row & 7);
  return c ^ ((row >> 1) & (CPR - 1));
}

template <int DQK, int DV, bool PAGED, int TAIL = 0>
__global__ void __launch_bounds__(kThreads, 2) prefill_mma_kernel(const MmaArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int KQ = DQK / 16;   // k-steps of S
  constexpr int NV = DV / 8;     // n-tiles of O
  constexpr int QB = BM * DQK * 2, KB = BN * DQK * 2, VB = BN * DV * 2;

  const int head = blockIdx.x;
  int seq, tile;
  if (a.plan) {                                   // grid (head, tile-list slot)
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
  if (m0 >= q_len) return;
  const int off = k_len - q_len;                 // keys every new token sees besides its own prefix
  const int kvh = head / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int rows_q = min(BM, q_len - m0);
  int kmax = off + m0 + rows_q;                  // keys visible to the last row of the tile
  if (kmax > k_len) kmax = k_len;
  if (kmax < 0) kmax = 0;
  const int ntiles = (kmax + BN - 1) / BN;

  const uint32_t sQ = smem_u32(smem), sK = sQ + QB, sV = sK + 2 * KB;

  auto k_row = [&](int n) -> const __nv_bfloat16* {
    if (PAGED) {
      const int id = __ldg(a.bt + static_cast<int64_t>(seq) * a.bt_stride + n / a.bs);
      if (static_cast<uint64_t>(static_cast<int64_t>(id)) >= static_cast<uint64_t>(a.num_blocks)) {
        report(a.status, B200_ERR_BOUNDS);
        return nullptr;
      }
      return a.kc + ((static_cast<int64_t>(id) * a.bs + n % a.bs) * a.Hkv + kvh) * DQK;
    }
    return a.k + static_cast<int64_t>(k0 + n) * a.k_stride + static_cast<int64_t>(kvh) * (DQK - TAIL);
  };
  auto v_row = [&](int n) -> const __nv_bfloat16* {
    if (PAGED) {
      const int id = __ldg(a.bt + static_cast<int64_t>(seq) * a.bt_stride + n / a.bs);
      if (static_cast<uint64_t>(static_cast<int64_t>(id)) >= static_cast<uint64_t>(a.num_blocks))
        return nullptr;
      return a.vc + ((static_cast<int64_t>(id) * a.bs + n % a.bs) * a.Hkv + kvh) * DV;
    }
    return a.v + static_cast<int64_t>(k0 + n) * a.v_stride + static_cast<int64_t>(kvh) * DV;
  };
  // safe dummy address for zero-filled chunks
  const __nv_bfloat16* dummy = a.q;
  auto load_kv = [&](int j, int stage) {
    const int n0 = j * BN;
    const int valid = min(BN, kmax - n0);
    constexpr int CPRK = DQK / 8, CPRV = DV / 8;
    if constexpr (TAIL == 0) {
#pragma unroll
      for (int i = 0; i < BN * CPRK / kThreads; ++i) {
        const int idx = threadIdx.x + i * kThreads;
        const int r = idx / CPRK, c = idx % CPRK;
        const __nv_bfloat16* src = r < valid ? k_row(n0 + r) : nullptr;
        cp_async16(sK + stage * KB + r * (DQK * 2) + swz<DQK>(c, r) * 16,
                   src ? src + c * 8 : dummy, src ? 16 : 0);
      }
    } else {
      // per-head columns, then the tail columns every head shares: two loops with power-of-two row widths
      constexpr int CH = (DQK - TAIL) / 8, CT = TAIL / 8;
#pragma unroll
      for (int i = 0; i < BN * CH / kThreads; ++i) {
        const int idx = threadIdx.x + i * kThreads;
        const int r = idx / CH, c = idx % CH;
        const __nv_bfloat16* src = r < valid ? k_row(n0 + r) : nullptr;
        cp_async16(sK + stage * KB + r * (DQK * 2) + swz<DQK>(c, r) * 16,
                   src ? src + c * 8 : dummy, src ? 16 : 0);
      }
#pragma unroll
      for (int i = 0; i < BN * CT / kThreads; ++i) {
        const int idx = threadIdx.x + i * kThreads;
        const int r = idx / CT, c = idx % CT;
        const bool ok = r < valid;
        cp_async16(sK + stage * KB + r * (DQK * 2) + swz<DQK>(CH + c, r) * 16,
                   ok ? a.k_tail + static_cast<int64_t>(k0 + n0 + r) * a.k_tail_stride + c * 8 : dummy, ok ? 16 : 0);
      }
    }
#pragma unroll
    for (int i = 0; i < BN * CPRV / kThreads; ++i) {
      const int idx = threadIdx.x + i * kThreads;
      const int r = idx / CPRV, c = idx % CPRV;
      const __nv_bfloat16* src = r < valid ? v_row(n0 + r) : nullptr;
      cp_async16(sV + stage * VB + r * (DV * 2) + swz<DV>(c, r) * 16, src ? src + c * 8 : dummy,
                 src ? 16 : 0);
    }
  };

  // ---- Q tile -> smem (group 0), first K/V tile (group 1) ----
  {
    constexpr int CPR = DQK / 8;
#pragma unroll
    for (int i = 0; i < BM * CPR / kThreads; ++i) {
      const int idx = threadIdx.x + i * kThreads;
      const int r = idx / CPR, c = idx % CPR;
      const bool ok = r < rows_q;
      const __nv_bfloat16* src =
          a.q + static_cast<int64_t>(q0 + m0 + (ok ? r : 0)) * a.q_stride +
          static_cast<int64_t>(head) * DQK + c * 8;
      cp_async16(sQ + r * (DQK * 2) + swz<DQK>(c, r) * 16, src, ok ? 16 : 0);
    }
  }
  cp_async_commit();
  if (ntiles > 0) load_kv(0, 0);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  // Q fragments of this warp's 16 rows: A operand, row-major
  uint32_t qf[KQ][4];
  {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int chalf = lane >> 4;
#pragma unroll
    for (int ks = 0; ks < KQ; ++ks)
      ldmatrix_x4(qf[ks], sQ + r * (DQK * 2) + swz<DQK>(2 * ks + chalf, r) * 16);
  }

  float o[NV][4];
#pragma unroll
  for (int n = 0; n < NV; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
  const int row0 = m0 + warp * 16 + g;  // query index (within the sequence) of c0/c1; +8 for c2/c3

  for (int j = 0; j < ntiles; ++j) {
    const int stage = j & 1;
    if (j + 1 < ntiles) load_kv(j + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const uint32_t kt = sK + stage * KB, vt = sV + stage * VB;
    // ---- S = Q K^T : 16 x 64 per warp ----
    float s[BN / 8][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    {
      // ldmatrix.x4: matrices (n-tile 2p, k lo), (2p, k hi), (2p+1, k lo), (2p+1, k hi)
      const int r_in = (lane & 7) + (lane >> 4) * 8;
      const int chalf = (lane >> 3) & 1;
#pragma unroll
      for (int ks = 0; ks < KQ; ++ks) {
#pragma unroll
        for (int p = 0; p < BN / 16; ++p) {
          uint32_t bf[4];
          const int r = p * 16 + r_in;
          ldmatrix_x4(bf, kt + r * (DQK * 2) + swz<DQK>(2 * ks + chalf, r) * 16);
          const uint32_t b0[2] = {bf[0], bf[1]}, b1[2] = {bf[2], bf[3]};
          mma_bf16_16816(s[2 * p], qf[ks], b0);
          mma_bf16_16816(s[2 * p + 1], qf[ks], b1);
        }
      }
    }
    // ---- scale, causal / length mask, online softmax ----
    const int n0 = j * BN;
    const bool need_mask = (n0 + BN - 1 > off + m0 + warp * 16) || (n0 + BN > kmax);
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] *= a.scale_log2;
      if (need_mask) {
        const int key = n0 + n * 8 + tq * 2;
        const int lim0 = min(off + row0, kmax - 1), lim1 = min(off + row0 + 8, kmax - 1);
        if (key > lim0) s[n][0] = -INFINITY;
        if (key + 1 > lim0) s[n][1] = -INFINITY;
        if (key > lim1) s[n][2] = -INFINITY;
        if (key + 1 > lim1) s[n][3] = -INFINITY;
      }
      mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
      mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m_r[0], mx0), mn1 = fmaxf(m_r[1], mx1);
    // a row whose keys are all masked so far keeps m = -inf; use 0 as the subtrahend then
    const float sub0 = mn0 == -INFINITY ? 0.f : mn0, sub1 = mn1 == -INFINITY ? 0.f : mn1;
    const float al0 = fast_exp2(m_r[0] - sub0), al1 = fast_exp2(m_r[1] - sub1);
    m_r[0] = mn0;
    m_r[1] = mn1;
    float ls0 = 0.f, ls1 = 0.f;
    uint32_t pf[BN / 16][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
      const float p0 = fast_exp2(s[n][0] - sub0), p1 = fast_exp2(s[n][1] - sub0);
      const float p2 = fast_exp2(s[n][2] - sub1), p3 = fast_exp2(s[n][3] - sub1);
      ls0 += p0 + p1;
      ls1 += p2 + p3;
      pf[n >> 1][(n & 1) * 2] = pack_bf16x2(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(p2, p3);
    }
    l_r[0] = l_r[0] * al0 + ls0;
    l_r[1] = l_r[1] * al1 + ls1;
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      o[n][0] *= al0;
      o[n][1] *= al0;
      o[n][2] *= al1;
      o[n][3] *= al1;
    }
    // ---- O += P V ----
    {
      // ldmatrix.x4.trans: (keys lo, d-chunk c), (keys hi, c), (keys lo, c+1), (keys hi, c+1)
      const int r_in = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int cadd = lane >> 4;
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
        for (int c = 0; c < NV; c += 2) {
          uint32_t bf[4];
          const int r = kk * 16 + r_in;
          ldmatrix_x4_trans(bf, vt + r * (DV * 2) + swz<DV>(c + cadd, r) * 16);
          const uint32_t b0[2] = {bf[0], bf[1]}, b1[2] = {bf[2], bf[3]};
          mma_bf16_16816(o[c], pf[kk], b0);
          mma_bf16_16816(o[c + 1], pf[kk], b1);
        }
      }
    }
    __syncthreads();  // everyone is done with this stage before it is refilled
  }
  cp_async_wait<0>();

  // ---- epilogue ----
  float l0 = l_r[0], l1 = l_r[1];
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  __nv_bfloat16* ob = a.out + (static_cast<int64_t>(q0 + m0) * a.Hq + head) * DV;
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    const int d = n * 8 + tq * 2;
    if (r0 < rows_q)
      *reinterpret_cast<uint32_t*>(ob + static_cast<int64_t>(r0) * a.Hq * DV + d) =
          pack_bf16x2(o[n][0] * i0, o[n][1] * i0);
    if (r1 < rows_q)
      *reinterpret_cast<uint32_t*>(ob + static_cast<int64_t>(r1) * a.Hq * DV + d) =
          pack_bf16x2(o[n][2] * i1, o[n][3] * i1);
  }
}

template <int DQK, int DV, int TAIL = 0>
int launch(const MmaArgs& a, int num_seqs, int plan_capacity, bool paged, cudaStream_t s) {
  constexpr size_t smem = size_t(BM) * DQK * 2 + 2 * size_t(BN) * DQK * 2 + 2 * size_t(BN) * DV * 2;
  static bool configured[64][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = paged ? prefill_mma_kernel<DQK, DV, true, 0> : prefill_mma_kernel<DQK, DV, false, TAIL>;
  if (dev >= 0 && dev < 64 && !configured[dev][paged]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return B200_ERR_LAUNCH;
    configured[dev][paged] = true;
  }
  dim3 grid(a.Hq, num_seqs, a.ntiles_max);
  if (a.plan) grid = dim3(a.Hq, plan_capacity, 1);
  kern<<<grid, kThreads, smem, s>>>(a);
  return launch_result();
}

}  // namespace

int prefill_mma_launch(const void* q, const void* k, const void* v, void* out, int64_t q_stride,
                       int64_t k_stride, int64_t v_stride, const int32_t* cu_q,
                       const int32_t* cu_k, int num_seqs, int max_seqlen_q, int Hq, int Hkv,
                       int Dqk, int Dv, float scale, const void* kc, const void* vc,
                       const int32_t* bt, int64_t bt_stride, int bs, int64_t num_blocks,
                       const int32_t* plan, int plan_tile_rows, int plan_capacity, int32_t* status,
                       cudaStream_t s, const void* k_tail, int64_t k_tail_stride, int tail) {
  const bool paged = bt != nullptr;
  if (tail < 0 || tail % 8 || tail >= Dqk || (tail > 0 && (paged || !k_tail))) return B200_ERR_ARG;
  const bool shape_ok = (Dqk == Dv && (Dqk == 32 || Dqk == 64 || Dqk == 128)) ||
                        (Dqk == 192 && Dv == 128);
  if (!shape_ok) return B200_ERR_UNSUPPORTED;
  const int ntiles = (max_seqlen_q + BM - 1) / BM;
  if (num_seqs > 65535 || ntiles > 65535) return B200_ERR_UNSUPPORTED;
  // 16-byte rows: pointers and token strides must keep every 8-element chunk aligned
  auto al = [](const void* p, int64_t stride) {
    return p == nullptr || (aligned16(p) && (stride * 2) % 16 == 0);
  };
  if (!al(q, q_stride) || !aligned16(out)) return B200_ERR_UNSUPPORTED;
  if (paged ? !(aligned16(kc) && aligned16(vc)) : !(al(k, k_stride) && al(v, v_stride)))
    return B200_ERR_UNSUPPORTED;
  if (tail > 0 && !al(k_tail, k_tail_stride)) return B200_ERR_UNSUPPORTED;
  MmaArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.q_stride = q_stride;
  a.k_stride = k_stride;
  a.v_stride = v_stride;
  a.k_tail = static_cast<const __nv_bfloat16*>(k_tail);
  a.k_tail_stride = k_tail_stride;
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
  if (tail > 0) {   // compiled for MLA's split: 128 per-head columns + 64 shared
    if (Dqk != 192 || tail != 64) return B200_ERR_UNSUPPORTED;
    return launch<192, 128, 64>(a, num_seqs, plan_capacity, false, s);
  }
  if (Dqk == 192) return launch<192, 128>(a, num_seqs, plan_capacity, paged, s);
  if (Dqk == 128) return launch<128, 128>(a, num_seqs, plan_capacity, paged, s);
  if (Dqk == 64) return launch<64, 64>(a, num_seqs, plan_capacity, paged, s);
  return launch<32, 32>(a, num_seqs, plan_capacity, paged, s);
}

}  // namespace b200
