// Grouped GEMM for MoE inference on the sm_100a tensor cores (tcgen05), written for the regime the
// decode step lives in: few rows per expert, so the layer is bound by streaming the expert weights
// from HBM once.  It replaces the per-expert loop of MOE.moe_infer (model/architecture/moe.py:299-339).
//
//   rows of X are grouped by expert (expert e owns rows [offsets[e-1], offsets[e]));
//   mode 0:  out[r, :]  = X[r, :] . W_e^T                      W [E, n_out, K]
//   mode 1:  act[r, :]  = silu(X[r] . W1_e^T + b1_e) * (X[r] . W3_e^T + b3_e)   W [E, 2*d_ff, K] = [w1 | w3]
//            (the SwiGLU of mlp.py:61-67; every intermediate rounded to bf16 like the tensor ops)
//
// The operands are swapped with respect to the usual layout: the 128 rows of a WEIGHT tile are the M
// dimension of the MMA and the (few) token rows are its N dimension (16..NPASS), so a CTA streams
// its weight tile exactly once whatever the row count, and the accumulator D^T [feature, token] sits
// in tensor memory with one output feature per lane.  In mode 1 the tile holds 64 rows of w1 and the
// matching 64 rows of w3, so gate and up projections of a feature meet in one CTA.
//
// One CTA per (weight tile, expert); 192 threads: warp 0 = TMA producer (one lane), warp 1 = MMA
// issuer (one lane) and tensor-memory owner, warps 2-5 = epilogue: tensor memory -> registers ->
// a [16 tokens][128 features] tile in shared memory -> row-wise rounding / bias / SwiGLU with 8
// features per thread -> 16-byte global stores.  A ring of STAGES shared-memory stages (16 KB of weights + NPASS x 128 B of token rows,
// 128-byte swizzle) is filled by TMA and drained by tcgen05.mma; mbarriers carry full/empty; every
// wait is bounded and a timeout aborts the CTA cleanly (status word = B200_ERR_TIMEOUT).
// Experts with more than NPASS rows take several passes over their weight tile (L2 hits).
//
// Mode 2 turns the same kernel into the greedy head of the decoder (lm_head followed by argmax,
// TransformerLM.lm_head model/transformer.py:160,183 and generate.py:62): one weight set [vocab, K], every row of
// X belongs to it, and the epilogue keeps, per token and per 128-row vocabulary tile, only the largest logit
// bf16(acc + bias) and its (lowest) index; a small second kernel reduces the tiles.  The logits are never written.
#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 192;
constexpr int BM = 128;              // weight rows per tile
constexpr int BK = 64;               // K elements per stage (128 bytes)
constexpr int A_BYTES = BM * 128;    // 16 KB
constexpr int XBOX = 32;             // token rows per TMA box
constexpr int XCH_STRIDE = 132;      // floats per token row of the epilogue tile (128 features + pad)

struct GemmArgs {
  const int32_t* offsets;   // [E] exclusive end of every expert's rows
  int n_out;                // output features per expert (mode 1: d_ff)
  int k_dim;
  int mode;
  __nv_bfloat16* out;       // [R, n_out]
  const __nv_bfloat16* bias;  // mode 0: [E, n_out]; mode 1: [E, 2*n_out]; or null
  int32_t* status;
  int num_experts;          // routed experts; groups past them are chunks of the dense tail
  int dense_rows;           // rows after the grouped ones that all use weight set `num_experts`
  int rows_single;          // mode 2: the row count of the single group (offsets is not read)
  unsigned long long* amax_key;   // mode 2: [tiles][rows_single] best (logit, row) key of the tile
};

template <int NPASS, int STAGES>
struct Layout {
  static constexpr int B_BYTES = NPASS * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int OFF_XCH = STAGES * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_XCH + 16 * XCH_STRIDE * 4;
  static constexpr int NUM_BARS = 2 * STAGES + 2;     // full[], empty[], acc_full, acc_empty
  static constexpr int SMEM = OFF_BAR + NUM_BARS * 8 + 16 + 1024;   // + alignment slack
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tensor_map, int c0, int c1,
                                            uint32_t mbar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
          "r"(dst_smem),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(c0), "r"(c1), "r"(mbar)
      : "memory");
}

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

union Bf16x8 {
  uint4 u;
  __nv_bfloat16 b[8];
};

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16(v)); }

template <int NPASS, int STAGES>
__global__ void __launch_bounds__(kThreads)
moe_gemm_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap tm_w,
                const __grid_constant__ CUtensorMap tm_x) {
  using L = Layout<NPASS, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(smem);
  float* xch = reinterpret_cast<float*>(smem + L::OFF_XCH);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + L::OFF_BAR + L::NUM_BARS * 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + L::OFF_BAR + L::NUM_BARS * 8 + 4);
  volatile int* s_go = reinterpret_cast<volatile int*>(smem + L::OFF_BAR + L::NUM_BARS * 8 + 8);
  auto bar = [&](int i) -> uint32_t { return sb + L::OFF_BAR + i * 8; };
  constexpr int FULL = 0, EMPTY = STAGES, ACC_FULL = 2 * STAGES, ACC_EMPTY = 2 * STAGES + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x;
  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tm_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tm_x)) : "memory");
  }
  int e = blockIdx.y, row0, rows;
  if (a.mode == 2) {
    row0 = 0;
    rows = a.rows_single;
  } else if (e < a.num_experts) {
    row0 = e ? a.offsets[e - 1] : 0;
    rows = a.offsets[e] - row0;
  } else {
    // dense tail (a shared expert applied to every token): chunk (e - num_experts) of NPASS rows after the
    // grouped rows, weight set num_experts; one pass per CTA, so these CTAs cost what the others cost
    const int chunk = e - a.num_experts;
    row0 = a.offsets[a.num_experts - 1] + chunk * NPASS;
    rows = min(NPASS, a.dense_rows - chunk * NPASS);
    e = a.num_experts;
  }
  if (rows <= 0) return;                                   // uniform, before any barrier / allocation
  const int npass = (rows + NPASS - 1) / NPASS;
  const int num_k = (a.k_dim + BK - 1) / BK;               // a ragged K tail is zero-filled by TMA
  const bool swiglu = a.mode == 1;
  // first weight row of each 64-row half of the tile, in the [E * rows_per_expert, K] view
  const int w_rows = swiglu ? 2 * a.n_out : a.n_out;
  const int wrow_a = e * w_rows + (swiglu ? tile * 64 : tile * BM);
  const int wrow_b = swiglu ? e * w_rows + a.n_out + tile * 64 : wrow_a + 64;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      umma::mbar_init(bar(FULL + s), 1);
      umma::mbar_init(bar(EMPTY + s), 1);
    }
    umma::mbar_init(bar(ACC_FULL), 1);
    umma::mbar_init(bar(ACC_EMPTY), 128);
    *s_abort = 0;
    *s_go = 1;
    umma::mbar_init_fence();
  }
  if (warp == 1) umma::tmem_alloc(sb + L::OFF_BAR + L::NUM_BARS * 8, NPASS < 32 ? 32 : NPASS);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;

  auto give_up = [&]() {
    *s_abort = 1;
    report(a.status, B200_ERR_TIMEOUT);
  };

  if (warp == 0) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      const int total = npass * num_k;
      auto weights = [&](int i) {           // stage i: arm the barrier for the whole stage, copy the weight tile
        const int pass = i / num_k, ks = i - pass * num_k;
        const int nb = (min(NPASS, rows - pass * NPASS) + XBOX - 1) / XBOX;
        const int st = i % STAGES;
        const uint32_t dst = sb + st * L::STAGE_BYTES;
        umma::mbar_expect_tx(bar(FULL + st), A_BYTES + nb * (XBOX * 128));
        tma_load_2d(dst, &tm_w, ks * BK, wrow_a, bar(FULL + st));
        if (swiglu) tma_load_2d(dst + A_BYTES / 2, &tm_w, ks * BK, wrow_b, bar(FULL + st));
      };
      auto tokens = [&](int i) {            // stage i: the token rows
        const int pass = i / num_k, ks = i - pass * num_k;
        const int nb = (min(NPASS, rows - pass * NPASS) + XBOX - 1) / XBOX;
        const int st = i % STAGES;
        const uint32_t dst = sb + st * L::STAGE_BYTES + A_BYTES;
        const int xrow = row0 + pass * NPASS;
        for (int j = 0; j < nb; ++j)
          tma_load_2d(dst + j * (XBOX * 128), &tm_x, ks * BK, xrow + j * XBOX, bar(FULL + st));
      };
      // The weights do not depend on the kernel before this one in the stream, the token rows do: when
      // this grid was launched early (programmatic dependent launch) the first ring of weight tiles is
      // already streaming while the producer of the rows finishes; griddepcontrol.wait returns at once
      // in an ordinary launch.
      const int pre = min(STAGES, total);
      for (int i = 0; i < pre; ++i) weights(i);
      asm volatile("griddepcontrol.wait;\n" ::: "memory");
      for (int i = 0; i < pre; ++i) tokens(i);
      int it = pre;
      for (; it < total; ++it) {
        const int st = it % STAGES;
        if (!umma::mbar_wait(bar(EMPTY + st), ((it / STAGES) - 1) & 1, s_abort)) {
          give_up();
          break;
        }
        weights(it);
        tokens(it);
      }
      // let the next kernel in the stream start its own prologue while this one drains
      asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
      if (*s_abort) {
        // copies still in flight must land before the CTA gives its shared memory back
        int never = 0;
        for (int x = max(0, it - STAGES); x < it; ++x)
          umma::mbar_wait(bar(FULL + x % STAGES), (x / STAGES) & 1, &never, 1 << 16);
      }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int pass = 0; pass < npass && ok; ++pass) {
        const int n = min(NPASS, rows - pass * NPASS);
        const int N = ((n + 15) / 16) * 16;
        const uint32_t idesc = umma::instr_desc_bf16(BM, N, false, false);
        if (pass > 0 && !umma::mbar_wait(bar(ACC_EMPTY), (pass - 1) & 1, s_abort)) {
          give_up();
          break;
        }
        umma::fence_after_sync();
        for (int ks = 0; ks < num_k; ++ks, ++it) {
          const int st = it % STAGES;
          if (!umma::mbar_wait(bar(FULL + st), (it / STAGES) & 1, s_abort)) {
            give_up();
            ok = false;
            break;
          }
          umma::fence_after_sync();
          const uint32_t sa = sb + st * L::STAGE_BYTES;
          const uint64_t adesc = umma::smem_desc(sa, 0, 1024);
          const uint64_t bdesc = umma::smem_desc(sa + A_BYTES, 0, 1024);
#pragma unroll
          for (int j = 0; j < BK / 16; ++j)
            umma::mma_ss(tmem, adesc + 2 * j, bdesc + 2 * j, idesc, (ks | j) != 0);
          umma::commit(bar(EMPTY + st));
        }
        if (ok) umma::commit(bar(ACC_FULL));
      }
    }
  } else {
    // =============================== epilogue (4 warps) ===============================
    const int q = warp & 3;                    // tensor-memory lane quarter this warp may read
    const int et = tid - 64;                   // 0..127
    for (int pass = 0; pass < npass; ++pass) {
      const int n = min(NPASS, rows - pass * NPASS);
      const int N = ((n + 15) / 16) * 16;
      if (!umma::mbar_wait(bar(ACC_FULL), pass & 1, s_abort)) give_up();
      // agree on abort among the four warps before any of them enters the barriers below
      epilogue_sync();
      if (et == 0) *s_go = !*s_abort;
      epilogue_sync();
      if (!*s_go) break;
      umma::fence_after_sync();
      const int64_t out_row0 = static_cast<int64_t>(row0) + pass * NPASS;
      if (a.mode == 2) {
        // Greedy head: this thread owns vocabulary row f with one accumulator per token.  Every logit becomes a
        // 64-bit key (order-preserving image of the bf16 logit, then the complement of f, so that the largest
        // key is the largest logit at the lowest row).  32 tokens at a time, a butterfly over the warp's 32 rows
        // leaves lane l with the best key of token c0 + l (31 exchanges instead of 32 x 5); the four warps then
        // meet in shared memory.
        const int f = tile * BM + q * 32 + lane;
        const float bias_f = (a.bias && f < a.n_out) ? __bfloat162float(a.bias[f]) : 0.f;
        unsigned long long* keys = reinterpret_cast<unsigned long long*>(xch);   // [4 warps][32 tokens]
        for (int c0 = 0; c0 < N; c0 += 32) {
          uint32_t r[32];
          if (c0 + 32 <= N) {
            umma::tmem_ld32(tmem + (static_cast<uint32_t>(q * 32) << 16) + c0, r);
          } else {      // N is a multiple of 16: a last half chunk
            uint32_t h[16];
            umma::tmem_ld16(tmem + (static_cast<uint32_t>(q * 32) << 16) + c0, h);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              r[j] = h[j];
              r[j + 16] = 0;
            }
          }
          unsigned long long key[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float y = bf16_round(__uint_as_float(r[j]) + bias_f);
            uint32_t u = __float_as_uint(y);
            u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
            key[j] = f < a.n_out ? (static_cast<unsigned long long>(u) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(f))
                                 : 0ull;
          }
#pragma unroll
          for (int sft = 16; sft >= 1; sft >>= 1) {
            const bool upper = (lane & sft) != 0;
#pragma unroll
            for (int j = 0; j < sft; ++j) {
              const unsigned long long keep = upper ? key[j + sft] : key[j];
              const unsigned long long send = upper ? key[j] : key[j + sft];
              const unsigned long long other = __shfl_xor_sync(0xffffffffu, send, sft);
              key[j] = keep > other ? keep : other;
            }
          }
          keys[q * 32 + lane] = key[0];
          epilogue_sync();
          if (q == 0) {
            const int tok = c0 + lane;
            unsigned long long best = keys[lane];
#pragma unroll
            for (int w = 1; w < 4; ++w) {
              const unsigned long long o = keys[w * 32 + lane];
              best = o > best ? o : best;
            }
            if (tok < n) a.amax_key[static_cast<int64_t>(tile) * a.rows_single + out_row0 + tok] = best;
          }
          epilogue_sync();
        }
      } else
      // 16 tokens at a time: every thread parks its feature's 16 accumulators in a [token][feature]
      // tile of shared memory, then the 128 threads walk the tile row-wise, 8 features per thread,
      // so that rounding / SwiGLU work is spread evenly and global stores are 16 bytes wide
      for (int c0 = 0; c0 < N; c0 += 16) {
        uint32_t r[16];
        umma::tmem_ld16(tmem + (static_cast<uint32_t>(q * 32) << 16) + c0, r);
#pragma unroll
        for (int j = 0; j < 16; ++j) xch[j * XCH_STRIDE + q * 32 + lane] = __uint_as_float(r[j]);
        epilogue_sync();
        if (!swiglu) {
          const int f8 = (et & 15) * 8, f = tile * BM + f8;
          const bool vec = (a.n_out & 7) == 0;
          for (int j = et >> 4; j < 16; j += 8) {
            const int tok = c0 + j;
            if (tok >= n || f >= a.n_out) continue;
            const float4 v0 = *reinterpret_cast<const float4*>(xch + j * XCH_STRIDE + f8);
            const float4 v1 = *reinterpret_cast<const float4*>(xch + j * XCH_STRIDE + f8 + 4);
            float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            __nv_bfloat16* dst = a.out + (out_row0 + tok) * a.n_out + f;
            const __nv_bfloat16* bp = a.bias ? a.bias + static_cast<int64_t>(e) * a.n_out + f : nullptr;
            if (vec) {
              Bf16x8 o, bb;
              if (bp) bb.u = *reinterpret_cast<const uint4*>(bp);
#pragma unroll
              for (int x = 0; x < 8; ++x) {
                float y = bf16_round(v[x]);
                if (bp) y += __bfloat162float(bb.b[x]);
                o.b[x] = __float2bfloat16(y);
              }
              *reinterpret_cast<uint4*>(dst) = o.u;
            } else {
              for (int x = 0; x < 8 && f + x < a.n_out; ++x) {
                float y = bf16_round(v[x]);
                if (bp) y += __bfloat162float(bp[x]);
                dst[x] = __float2bfloat16(y);
              }
            }
          }
        } else {
          // tile columns 0..63 = gate (w1 rows), 64..127 = up (w3 rows) of the same 64 features
          const int f8 = (et & 7) * 8, f = tile * 64 + f8;
          const bool vec = (a.n_out & 7) == 0;
          const int j = et >> 3;               // 16 tokens x 8 feature groups = 128 threads
          const int tok = c0 + j;
          if (tok < n && f < a.n_out) {
            const float* gp = xch + j * XCH_STRIDE + f8;
            const float4 g0 = *reinterpret_cast<const float4*>(gp), g1 = *reinterpret_cast<const float4*>(gp + 4);
            const float4 u0 = *reinterpret_cast<const float4*>(gp + 64), u1 = *reinterpret_cast<const float4*>(gp + 68);
            const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
            __nv_bfloat16* dst = a.out + (out_row0 + tok) * a.n_out + f;
            const __nv_bfloat16* bg = a.bias ? a.bias + static_cast<int64_t>(e) * 2 * a.n_out + f : nullptr;
            Bf16x8 o, b1, b3;
            if (bg && vec) {
              b1.u = *reinterpret_cast<const uint4*>(bg);
              b3.u = *reinterpret_cast<const uint4*>(bg + a.n_out);
            }
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              float gv = bf16_round(g[x]), uv = bf16_round(u[x]);
              if (bg && (vec || f + x < a.n_out)) {
                gv = bf16_round(gv + __bfloat162float(vec ? b1.b[x] : bg[x]));
                uv = bf16_round(uv + __bfloat162float(vec ? b3.b[x] : bg[a.n_out + x]));
              }
              const float sv = bf16_round(gv / (1.f + expf(-gv)));
              o.b[x] = __float2bfloat16(sv * uv);
            }
            if (vec) {
              *reinterpret_cast<uint4*>(dst) = o.u;
            } else {
              for (int x = 0; x < 8 && f + x < a.n_out; ++x) dst[x] = o.b[x];
            }
          }
        }
        epilogue_sync();
      }
      umma::fence_before_sync();
      umma::mbar_arrive(bar(ACC_EMPTY));
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 1) umma::tmem_dealloc(tmem, NPASS < 32 ? 32 : NPASS);
}

// Second stage of the greedy head: per token, the largest key over the vocabulary tiles (largest logit, lowest
// row among equals).  One warp per token.
__global__ void __launch_bounds__(256)
lm_head_argmax_finish_kernel(const unsigned long long* __restrict__ keys, int tiles, int rows,
                             int64_t* __restrict__ tokens) {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  unsigned long long best = 0ull;
  for (int t = lane; t < tiles; t += 32) {
    const unsigned long long k = keys[static_cast<int64_t>(t) * rows + row];
    best = k > best ? k : best;
  }
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, off);
    best = o > best ? o : best;
  }
  if (lane == 0) tokens[row] = best == 0ull ? 0 : static_cast<int64_t>(0xFFFFFFFFu - static_cast<uint32_t>(best));
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

// [rows, k] bf16 row-major seen as (k, row); one box is 64 K-elements (128 bytes) of `box_rows` rows,
// written to shared memory with the 128-byte swizzle; out-of-range elements read as zero.
bool make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t k, int box_rows) {
  EncodeFn enc = tensor_map_encoder();
  if (enc == nullptr || rows <= 0) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NPASS, int STAGES>
int launch(const GemmArgs& a, const CUtensorMap& tw, const CUtensorMap& tx, dim3 grid, bool early, cudaStream_t s) {
  using L = Layout<NPASS, STAGES>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return B200_ERR_UNSUPPORTED;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(moe_gemm_kernel<NPASS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::SMEM) != cudaSuccess)
      return B200_ERR_LAUNCH;
    configured[dev] = true;
  }
  // Only the token rows depend on the kernel before this one in the stream when the caller says so
  // (`early`): launched as a programmatic dependent, the prologue and first weight tiles overlap the tail of
  // that kernel (which may be any kernel: one that never triggers releases its dependents as its CTAs exit)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = L::SMEM;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, moe_gemm_kernel<NPASS, STAGES>, a, tw, tx) != cudaSuccess) {
    cudaGetLastError();
    return B200_ERR_LAUNCH;
  }
  return launch_result();
}

}  // namespace

int moe_gemm_rows_launch(const void* x, const void* w, const void* bias, void* out, const int32_t* expert_offsets,
                         int64_t num_rows, int num_experts, int dense_rows, int n_out, int k_dim, int mode,
                         int32_t* status, cudaStream_t s);

}  // namespace b200

extern "C" int b200_moe_grouped_gemm(const void* x, const void* w, const void* bias, void* out,
                                     const int32_t* expert_offsets, int64_t num_rows, int32_t num_experts,
                                     int32_t dense_rows, int32_t n_out, int32_t k_dim, int32_t mode,
                                     int32_t dtype, int32_t* status, void* stream) {
  using namespace b200;
  const bool early = (mode & B200_MOE_GEMM_EARLY_LAUNCH) != 0;
  mode &= ~B200_MOE_GEMM_EARLY_LAUNCH;
  if (num_rows < 0 || num_experts <= 0 || n_out <= 0 || k_dim <= 0 || (mode != 0 && mode != 1) ||
      dense_rows < 0 || dense_rows > num_rows)
    return B200_ERR_ARG;
  if (dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (num_rows == 0) return B200_OK;
  if (!x || !w || !out || !expert_offsets) return B200_ERR_ARG;
  if (k_dim % 8 != 0 || !aligned16(x) || !aligned16(w)) return B200_ERR_ALIGN;   // TMA: 16-byte rows
  if (num_experts > 65535 || num_rows > 2147483647) return B200_ERR_TOO_LARGE;
  const int64_t w_sets = num_experts + (dense_rows > 0 ? 1 : 0);
  const int64_t w_rows = w_sets * (mode == 1 ? 2 : 1) * n_out;
  if (w_rows > 2147483647) return B200_ERR_TOO_LARGE;
  CUtensorMap tw, tx;
  if (!make_map(&tw, w, w_rows, k_dim, mode == 1 ? 64 : BM) || !make_map(&tx, x, num_rows, k_dim, XBOX))
    return B200_ERR_UNSUPPORTED;
  GemmArgs a{};
  a.offsets = expert_offsets;
  a.n_out = n_out;
  a.k_dim = k_dim;
  a.mode = mode;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.status = status;
  a.num_experts = num_experts;
  a.dense_rows = dense_rows;
  const int tiles = mode == 1 ? (n_out + 63) / 64 : (n_out + BM - 1) / BM;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // few rows per expert: deep ring of small stages, two CTAs per SM; otherwise 256 rows per pass
  const int64_t grouped = num_rows - dense_rows;
  if (grouped <= 64LL * num_experts) {
    const dim3 grid(tiles, num_experts + (dense_rows + 63) / 64);
    return launch<64, 4>(a, tw, tx, grid, early, s);
  }
  // many rows per expert: the compute-bound kernel (token rows as the MMA M side, persistent CTAs)
  const int rc = moe_gemm_rows_launch(x, w, bias, out, expert_offsets, num_rows, num_experts, dense_rows, n_out, k_dim,
                                      mode, status, s);
  if (rc != B200_ERR_UNSUPPORTED) return rc;
  const dim3 grid(tiles, num_experts + (dense_rows + 255) / 256);
  return launch<256, 4>(a, tw, tx, grid, early, s);
}

/* Greedy head: tokens[r] = argmax_v bf16(hidden[r] . W[v] + bias[v]), lowest v among equal maxima. */
extern "C" size_t b200_lm_head_argmax_workspace_bytes(int32_t num_rows, int32_t vocab_size) {
  if (num_rows <= 0 || vocab_size <= 0) return 0;
  const size_t tiles = (static_cast<size_t>(vocab_size) + b200::BM - 1) / b200::BM;
  return tiles * num_rows * sizeof(unsigned long long) + 256;
}

extern "C" int b200_lm_head_argmax(const void* hidden, const void* w, const void* bias, int64_t* tokens,
                                   int32_t num_rows, int32_t vocab_size, int32_t k_dim, void* workspace,
                                   size_t workspace_bytes, int32_t dtype, int32_t* status, void* stream) {
  using namespace b200;
  if (num_rows < 0 || vocab_size <= 0 || k_dim <= 0) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (num_rows == 0) return B200_OK;
  if (!hidden || !w || !tokens) return B200_ERR_ARG;
  if (k_dim % 8 != 0 || !aligned16(hidden) || !aligned16(w)) return B200_ERR_ALIGN;
  if (!workspace || workspace_bytes < b200_lm_head_argmax_workspace_bytes(num_rows, vocab_size)) return B200_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return B200_ERR_ALIGN;
  CUtensorMap tw, tx;
  if (!make_map(&tw, w, vocab_size, k_dim, BM) || !make_map(&tx, hidden, num_rows, k_dim, XBOX)) return B200_ERR_UNSUPPORTED;
  const int tiles = (vocab_size + BM - 1) / BM;
  GemmArgs a{};
  a.n_out = vocab_size;
  a.k_dim = k_dim;
  a.mode = 2;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.status = status;
  a.num_experts = 1;
  a.rows_single = num_rows;
  a.amax_key = static_cast<unsigned long long*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(tiles, 1);
  const int rc = num_rows <= 64 ? launch<64, 4>(a, tw, tx, grid, false, s) : launch<256, 4>(a, tw, tx, grid, false, s);
  if (rc != B200_OK) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((num_rows + 7) / 8);
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, lm_head_argmax_finish_kernel, static_cast<const unsigned long long*>(a.amax_key),
                         tiles, static_cast<int>(num_rows), tokens) != cudaSuccess) {
    cudaGetLastError();
    return B200_ERR_LAUNCH;
  }
  return launch_result();
}
