// Grouped GEMM for MoE inference at PREFILL sizes (hundreds of rows per expert), on the sm_100a tensor cores
// (tcgen05): the compute-bound sibling of moe_gemm.cu, which serves the weight-streaming decode regime.
// Same contract (the per-expert loop of MOE.moe_infer, model/architecture/moe.py:299-339; SwiGLU of
// mlp.py:61-67 in mode 1), conventional orientation: TOKEN rows are the M dimension of the MMA, 256 weight rows
// its N dimension.  A work item is a 256 x 256 tile computed as two M = 128 products on the same weight
// operand (two accumulators of 256 tensor-memory columns): with 128 x 256 tiles every CTA pulls 48 KB from L2
// per 64-wide k-step for 4.2 MFLOP and the kernel was bound by L2-to-SM bandwidth at ~1 us per k-step; the
// square tile moves 64 KB for twice the arithmetic.
//
//   mode 0:  out[r, n0 .. n0+255]  = X[r] . W_e[n0 .. n0+255]^T (+ bias)
//   mode 1:  a tile holds 128 rows of w1 and the matching 128 rows of w3 of the same features, so
//            act[r, f0 .. f0+127] = silu(X[r] . W1^T + b1) * (X[r] . W3^T + b3) is formed in the epilogue and the
//            [rows, 2 * d_ff] intermediate is never written
//
// Persistent CTAs (one per SM) walk the list of (group, 256-row tile, column tile) work items, column tile
// fastest; groups are the experts' row ranges (read from expert_offsets on the device) plus, when
// dense_rows > 0, one more group with weight set E (a shared expert over all tokens in the same launch).
//   warp 0      TMA producer: one thread, ring of 3 stages of (A 32 KB | B 32 KB), 128-byte swizzle
//   warp 1      tensor-memory owner; lane 0 issues tcgen05.mma (M 128, N 256, K 16), one per row half
//   warps 2-9   epilogue: thread = token row; tensor memory -> registers -> bias / rounding / SwiGLU -> global.
// A tile whose group has at most 128 rows left skips its second half (no copy, no MMA).
// Every wait is bounded; a timeout raises the CTA's abort flag, is reported (B200_ERR_TIMEOUT), copies in
// flight are drained and the tensor memory is freed.
#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 320;
constexpr int BM = 256;                 // token rows per tile (two M = 128 halves)
constexpr int BN = 256;                 // weight rows per tile
constexpr int BK = 64;                  // K elements per stage (128 bytes)
constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128, STAGE = A_BYTES + B_BYTES;
constexpr int NST = 3;
constexpr int kMaxGroups = 66;          // 64 experts + a dense tail + sentinel
constexpr int OFF_BAR = NST * STAGE;
constexpr int FULL = 0, EMPTY = NST, ACC_FULL = 2 * NST, ACC_EMPTY = 2 * NST + 1, NUM_BARS = 2 * NST + 2;
constexpr int OFF_TAB = OFF_BAR + NUM_BARS * 8 + 16;             // group table: first row, rows, first m-tile
constexpr int SMEM = OFF_TAB + 3 * kMaxGroups * 4 + 1024;       // + slack to align the base to 1024 bytes

struct RowsArgs {
  const int32_t* offsets;     // [E] exclusive end of every expert's rows
  int num_experts, dense_rows;
  int64_t num_rows;
  int n_out, k_dim, mode;
  __nv_bfloat16* out;         // [R, n_out]
  const __nv_bfloat16* bias;  // mode 0: [sets, n_out]; mode 1: [sets, 2 * n_out]; or null
  int32_t* status;
};

__device__ __forceinline__ void tma_2d(uint32_t dst_smem, const void* tensor_map, int c0, int c1, uint32_t mbar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
          "r"(dst_smem),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(c0), "r"(c1), "r"(mbar)
      : "memory");
}

union Bf16x8r {
  uint4 u;
  __nv_bfloat16 b[8];
};
__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16(v)); }

__global__ void __launch_bounds__(kThreads, 1)
moe_gemm_rows_kernel(const RowsArgs a, const __grid_constant__ CUtensorMap tm_x,
                     const __grid_constant__ CUtensorMap tm_w) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(smem);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NUM_BARS * 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + OFF_BAR + NUM_BARS * 8 + 4);
  int* g_row0 = reinterpret_cast<int*>(smem + OFF_TAB);      // first row of the group
  int* g_rows = g_row0 + kMaxGroups;                         // its row count
  int* g_tile0 = g_rows + kMaxGroups;                        // m-tiles of the groups before it; [groups] = total
  auto bar = [&](int i) -> uint32_t { return sb + OFF_BAR + i * 8; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool swiglu = a.mode == 1;
  const int groups = a.num_experts + (a.dense_rows > 0 ? 1 : 0);
  const int feat_per_tile = swiglu ? BN / 2 : BN;            // output columns an item produces
  const int n_tiles = (a.n_out + feat_per_tile - 1) / feat_per_tile;
  const int num_k = (a.k_dim + BK - 1) / BK;                 // a ragged K tail is zero-filled by TMA
  const int w_rows = swiglu ? 2 * a.n_out : a.n_out;         // weight rows per set

  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tm_x)) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tm_w)) : "memory");
    int tiles = 0, prev = 0;
    for (int e = 0; e < groups; ++e) {
      int r0, rows;
      if (e < a.num_experts) {
        const int end = a.offsets[e];
        r0 = prev;
        rows = end - prev;
        prev = end;
      } else {
        r0 = prev;
        rows = a.dense_rows;
      }
      if (rows < 0) rows = 0;
      g_row0[e] = r0;
      g_rows[e] = rows;
      g_tile0[e] = tiles;
      tiles += (rows + BM - 1) / BM;
    }
    g_tile0[groups] = tiles;
    for (int s = 0; s < NST; ++s) {
      umma::mbar_init(bar(FULL + s), 1);
      umma::mbar_init(bar(EMPTY + s), 1);
    }
    umma::mbar_init(bar(ACC_FULL), 1);
    umma::mbar_init(bar(ACC_EMPTY), 256);
    *s_abort = 0;
    umma::mbar_init_fence();
  }
  if (warp == 1) umma::tmem_alloc(sb + OFF_BAR + NUM_BARS * 8, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;
  const int total_items = g_tile0[groups] * n_tiles;

  // work item w -> (group, row tile within the group, column tile); every role walks the same sequence
  struct Item {
    int e, row0, rows, n0;   // group (= weight set), first row of the tile, valid rows in it, first output column
  };
  auto item_of = [&](int w) -> Item {
    const int nt = w % n_tiles, mt = w / n_tiles;
    int e = 0;
    while (e + 1 < groups && g_tile0[e + 1] <= mt) ++e;
    const int local = mt - g_tile0[e];
    Item it;
    it.e = e;
    it.row0 = g_row0[e] + local * BM;
    it.rows = min(BM, g_rows[e] - local * BM);
    it.n0 = nt * feat_per_tile;
    return it;
  };
  auto give_up = [&]() {
    *s_abort = 1;
    report(a.status, B200_ERR_TIMEOUT);
  };

  if (warp == 0) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      int it = 0;      // stages issued so far
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_items; w += gridDim.x) {
        const Item im = item_of(w);
        const int wrow = im.e * w_rows + im.n0;            // first weight row of the tile (mode 1: of its w1 half)
        for (int ks = 0; ks < num_k; ++ks, ++it) {
          const int st = it % NST;
          if (it >= NST && !umma::mbar_wait(bar(EMPTY + st), ((it / NST) - 1) & 1, s_abort)) {
            give_up();
            ok = false;
            break;
          }
          const uint32_t dst = sb + st * STAGE;
          const bool two = im.rows > 128;                  // the second row half holds rows of this group
          umma::mbar_expect_tx(bar(FULL + st), two ? STAGE : STAGE - A_BYTES / 2);
          tma_2d(dst, &tm_x, ks * BK, im.row0, bar(FULL + st));
          if (two) tma_2d(dst + A_BYTES / 2, &tm_x, ks * BK, im.row0 + 128, bar(FULL + st));
          if (swiglu) {
            tma_2d(dst + A_BYTES, &tm_w, ks * BK, wrow, bar(FULL + st));                          // 128 rows of w1
            tma_2d(dst + A_BYTES + B_BYTES / 2, &tm_w, ks * BK, wrow + a.n_out, bar(FULL + st));   // ... of w3
          } else {
            tma_2d(dst + A_BYTES, &tm_w, ks * BK, wrow, bar(FULL + st));
            tma_2d(dst + A_BYTES + B_BYTES / 2, &tm_w, ks * BK, wrow + BN / 2, bar(FULL + st));
          }
        }
      }
      if (*s_abort) {
        // copies still in flight must land before the CTA gives its shared memory back
        int never = 0;
        for (int x = max(0, it - NST); x < it; ++x)
          umma::mbar_wait(bar(FULL + x % NST), (x / NST) & 1, &never, 1 << 16);
      }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      const uint32_t idesc = umma::instr_desc_bf16(128, BN, false, false);
      int it = 0, n_item = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_items; w += gridDim.x, ++n_item) {
        const Item im = item_of(w);
        const bool two = im.rows > 128;
        if (n_item >= 1 && !umma::mbar_wait(bar(ACC_EMPTY), (n_item - 1) & 1, s_abort)) {
          give_up();
          break;
        }
        umma::fence_after_sync();
        for (int ks = 0; ks < num_k; ++ks, ++it) {
          const int st = it % NST;
          if (!umma::mbar_wait(bar(FULL + st), (it / NST) & 1, s_abort)) {
            give_up();
            ok = false;
            break;
          }
          umma::fence_after_sync();
          const uint32_t sa = sb + st * STAGE;
          const uint64_t adesc0 = umma::smem_desc(sa, 0, 1024);
          const uint64_t adesc1 = umma::smem_desc(sa + A_BYTES / 2, 0, 1024);
          const uint64_t bdesc = umma::smem_desc(sa + A_BYTES, 0, 1024);
#pragma unroll
          for (int j = 0; j < BK / 16; ++j) {
            umma::mma_ss(tmem, adesc0 + 2 * j, bdesc + 2 * j, idesc, (ks | j) != 0);
            if (two) umma::mma_ss(tmem + BN, adesc1 + 2 * j, bdesc + 2 * j, idesc, (ks | j) != 0);
          }
          umma::commit(bar(EMPTY + st));
        }
        if (ok) umma::commit(bar(ACC_FULL));
      }
    }
  } else {
    // =============================== epilogue (8 warps, thread = token row) ===============================
    const int q = warp & 3;                          // tensor-memory lane quarter this warp may read
    const int half = (warp - 2) >> 2;                // row half of the tile = accumulator
    const int row = half * 128 + q * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    int n_item = 0;
    for (int w = blockIdx.x; w < total_items; w += gridDim.x, ++n_item) {
      const Item im = item_of(w);
      // tensor-memory loads are warp-collective: the whole warp continues or stops together
      if (!__all_sync(0xffffffffu, umma::mbar_wait(bar(ACC_FULL), n_item & 1, s_abort))) {
        give_up();
        break;
      }
      umma::fence_after_sync();
      const uint32_t acc = tmem + half * BN + lane_sel;
      const bool valid = row < im.rows;
      __nv_bfloat16* orow = a.out + (static_cast<int64_t>(im.row0) + row) * a.n_out + im.n0;
      if (swiglu) {
        const __nv_bfloat16* bg = a.bias ? a.bias + static_cast<int64_t>(im.e) * 2 * a.n_out + im.n0 : nullptr;
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          uint32_t g[32], u[32];
          umma::tmem_ld32_issue(acc + c, g);
          umma::tmem_ld32(acc + BN / 2 + c, u);
          umma::tmem_ld32_wait(g);
#pragma unroll
          for (int e8 = 0; e8 < 32; e8 += 8) {
            const int f = im.n0 + c + e8;            // feature of the first of these 8 columns
            if (!valid || f >= a.n_out) continue;    // n_out is a multiple of 8: whole groups are in or out
            Bf16x8r o, b1, b3;
            if (bg) {
              b1.u = __ldg(reinterpret_cast<const uint4*>(bg + c + e8));
              b3.u = __ldg(reinterpret_cast<const uint4*>(bg + a.n_out + c + e8));
            }
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              float gv = bf16r(__uint_as_float(g[e8 + x])), uv = bf16r(__uint_as_float(u[e8 + x]));
              if (bg) {
                gv = bf16r(gv + __bfloat162float(b1.b[x]));
                uv = bf16r(uv + __bfloat162float(b3.b[x]));
              }
              // fast exponential and division: their ~1e-6 relative error disappears in the bf16 rounding of silu
              const float sv = bf16r(__fdividef(gv, 1.f + __expf(-gv)));
              o.b[x] = __float2bfloat16(sv * uv);
            }
            *reinterpret_cast<uint4*>(orow + c + e8) = o.u;
          }
          __syncwarp();      // the next tensor-memory load is warp-collective
        }
      } else {
        const __nv_bfloat16* bp = a.bias ? a.bias + static_cast<int64_t>(im.e) * a.n_out + im.n0 : nullptr;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          umma::tmem_ld32(acc + c, r);
#pragma unroll
          for (int e8 = 0; e8 < 32; e8 += 8) {
            const int f = im.n0 + c + e8;
            if (!valid || f >= a.n_out) continue;
            Bf16x8r o, bb;
            if (bp) bb.u = __ldg(reinterpret_cast<const uint4*>(bp + c + e8));
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              float y = bf16r(__uint_as_float(r[e8 + x]));
              if (bp) y += __bfloat162float(bb.b[x]);
              o.b[x] = __float2bfloat16(y);
            }
            *reinterpret_cast<uint4*>(orow + c + e8) = o.u;
          }
          __syncwarp();
        }
      }
      umma::fence_before_sync();
      umma::mbar_arrive(bar(ACC_EMPTY));
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 1) umma::tmem_dealloc(tmem, 512);
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn rows_tensor_map_encoder() {
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

// [rows, k] bf16 row-major seen as (k, row); one box is 64 K-elements (128 bytes) of 128 rows, written to
// shared memory with the 128-byte swizzle; out-of-range elements read as zero.
bool rows_make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t k) {
  EncodeFn enc = rows_tensor_map_encoder();
  if (enc == nullptr || rows <= 0) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), 128};   // halves of the A and B tiles
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Launch for the compute-bound regime; B200_ERR_UNSUPPORTED for shapes it does not take (the caller then uses
// the weight-streaming kernel with several passes).
int moe_gemm_rows_launch(const void* x, const void* w, const void* bias, void* out, const int32_t* expert_offsets,
                         int64_t num_rows, int num_experts, int dense_rows, int n_out, int k_dim, int mode,
                         int32_t* status, cudaStream_t s) {
  if (n_out % 8 != 0 || k_dim % 8 != 0 || num_experts + 1 >= kMaxGroups) return B200_ERR_UNSUPPORTED;
  const int64_t w_sets = num_experts + (dense_rows > 0 ? 1 : 0);
  const int64_t w_rows = w_sets * (mode == 1 ? 2 : 1) * n_out;
  if (w_rows > 2147483647LL || num_rows > 2147483647LL) return B200_ERR_UNSUPPORTED;
  CUtensorMap tx, tw;
  if (!rows_make_map(&tx, x, num_rows, k_dim) || !rows_make_map(&tw, w, w_rows, k_dim)) return B200_ERR_UNSUPPORTED;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
  static bool configured[64] = {};    // per-device flag, written without a lock (idempotent)
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return B200_ERR_UNSUPPORTED;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(moe_gemm_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return B200_ERR_LAUNCH;
    configured[dev] = true;
  }
  const int sms = sm_count_cached();
  if (sms <= 0) return B200_ERR_NO_DEVICE;
  RowsArgs a{};
  a.offsets = expert_offsets;
  a.num_experts = num_experts;
  a.dense_rows = dense_rows;
  a.num_rows = num_rows;
  a.n_out = n_out;
  a.k_dim = k_dim;
  a.mode = mode;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.status = status;
  // upper bound of the work items, so that small problems do not launch idle CTAs
  const int64_t feat = mode == 1 ? BN / 2 : BN;
  const int64_t max_items = ((num_rows + BM - 1) / BM + w_sets) * ((n_out + feat - 1) / feat);
  const int grid = static_cast<int>(max_items < sms ? (max_items > 0 ? max_items : 1) : sms);
  moe_gemm_rows_kernel<<<grid, kThreads, SMEM, s>>>(a, tx, tw);
  return launch_result();
}

}  // namespace b200
