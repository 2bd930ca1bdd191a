// MoE routing for inference: gate scores -> top-k experts per token -> renormalised weights -> rows
// grouped by expert for a grouped GEMM, plus the inverse permutation for the combine.
//
// Arithmetic is Gate.forward of the reference (model/architecture/moe.py:45-90) with the roundings of
// its dtype: scores = sigmoid(logits); selection by top-k of logits + expert_bias (bias cast to the
// dtype first); weights = scores of the selected experts divided by (their sum + 1e-10).  Ties in
// the biased logits go to the lower expert index.
//
// Output rows are ordered by (expert, token): a stable counting sort.  One thread owns one token and
// a CTA owns 256 consecutive tokens.  A token selects an expert at most once, so "my token uses
// expert e" is one bit per thread: a warp ballot per expert gives both the warp's count and the
// thread's rank inside the warp.  With more than one CTA a first launch writes every CTA's
// per-expert counts to the workspace; the scatter launch sums them (all CTAs -> expert totals,
// earlier CTAs -> this CTA's first row of every expert) and writes the rows.  A batch that fits one
// CTA (decode) needs the scatter launch only.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kTok = 256;     // tokens (= threads) per CTA
constexpr int kWarps = kTok / 32;
constexpr int kMaxE = 64;
constexpr int kMaxK = 8;
constexpr int kMaxTokens = 65536;

template <typename T>
__device__ __forceinline__ float round_to(float v) {
  return to_float<T>(from_float<T>(v));
}

struct RouteArgs {
  const void* logits;       // [T, E] dtype
  const float* bias;        // [E]
  int T, E, K;
  int32_t* sorted_token;    // [T*K]  token of sorted row i
  int32_t* sorted_expert;   // [T*K]  expert of sorted row i
  void* sorted_weight;      // [T*K]  dtype, routing weight of sorted row i
  int32_t* offsets;         // [E]    end (exclusive) of each expert's rows
  int32_t* slot_to_row;     // [T, K] sorted-row index of token t's j-th expert in ascending expert order
  int32_t* cta_counts;      // [gridDim.x, E] workspace (unused with one CTA)
  int identity_tail;        // also write sorted_token[T*K + t] = t (rows of a shared expert after the grouped ones)
};

// 32-bit expert masks up to 32 experts, 64-bit above: the selection loops are all shifts and tests
template <int EMAX>
struct MaskOf {
  using type = uint32_t;
};
template <>
struct MaskOf<64> {
  using type = unsigned long long;
};
__device__ __forceinline__ int lowest_bit(uint32_t m) { return __ffs(static_cast<int>(m)) - 1; }
__device__ __forceinline__ int lowest_bit(unsigned long long m) { return __ffsll(static_cast<long long>(m)) - 1; }

// bit e set: the token routes to expert e; `biased` holds logits + bias of the E experts (-inf beyond E).
template <int EMAX>
__device__ __forceinline__ typename MaskOf<EMAX>::type top_k_mask(const float (&biased)[EMAX], int E, int K) {
  using M = typename MaskOf<EMAX>::type;
  M taken = 0;
  for (int k = 0; k < K; ++k) {            // k maxima, lower index first among equals
    int best = -1;
    float bv = -INFINITY;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
      const bool open = e < E && !((taken >> e) & M(1));
      if (open && (best < 0 || biased[e] > bv)) {
        best = e;
        bv = biased[e];
      }
    }
    taken |= M(1) << best;
  }
  return taken;
}

// bit e set: token t routes to expert e.  EMAX (>= E) is a compile-time bound so that the biased
// logits live in registers.
template <typename T, int EMAX>
__device__ __forceinline__ typename MaskOf<EMAX>::type select_mask(const RouteArgs& a, int t) {
  using M = typename MaskOf<EMAX>::type;
  const T* row = static_cast<const T*>(a.logits) + static_cast<int64_t>(t) * a.E;
  float biased[EMAX];
#pragma unroll
  for (int e = 0; e < EMAX; ++e)
    biased[e] = e < a.E ? round_to<T>(to_float<T>(row[e]) + round_to<T>(a.bias[e])) : -INFINITY;
  M taken = 0;
  for (int k = 0; k < a.K; ++k) {            // k maxima, lower index first among equals
    int best = -1;
    float bv = -INFINITY;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
      const bool open = e < a.E && !((taken >> e) & M(1));
      if (open && (best < 0 || biased[e] > bv)) {
        best = e;
        bv = biased[e];
      }
    }
    taken |= M(1) << best;
  }
  return taken;
}

// per-warp counts of every expert into warp_cnt[warp][e]; ranks[n] = number of lower lanes of the warp
// that also use the n-th (ascending) expert of this thread's token
template <typename M>
__device__ __forceinline__ void warp_counts(M taken, int E, int32_t (*warp_cnt)[kMaxE], int* ranks) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned lt = (1u << lane) - 1u;
  int n = 0;
  for (int e = 0; e < E; ++e) {
    const bool mine = (taken >> e) & M(1);
    const unsigned b = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) warp_cnt[warp][e] = __popc(b);
    if (mine && n < kMaxK) ranks[n++] = __popc(b & lt);
  }
}

template <typename T, int EMAX>
__global__ void __launch_bounds__(kTok) moe_count_kernel(const RouteArgs a) {
  __shared__ int32_t warp_cnt[kWarps][kMaxE];
  const int t = blockIdx.x * kTok + threadIdx.x;
  using M = typename MaskOf<EMAX>::type;
  const M taken = t < a.T ? select_mask<T, EMAX>(a, t) : M(0);
  int ranks[kMaxK];
  warp_counts(taken, a.E, warp_cnt, ranks);
  __syncthreads();
  if (threadIdx.x < a.E) {
    int s = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) s += warp_cnt[w][threadIdx.x];
    a.cta_counts[blockIdx.x * a.E + threadIdx.x] = s;
  }
}

// Shared memory of the scatter step.
struct ScatterSmem {
  int32_t warp_cnt[kWarps][kMaxE];   // rows of expert e owned by warp w
  int32_t warp_pre[kWarps][kMaxE];   // ... by the warps before w
  int32_t tot_s[kMaxE], bef_s[kMaxE];
  int32_t base[kMaxE];               // first output row of this CTA's rows of expert e
};

// routing weights of the selected experts of one token (ascending expert order): sigmoid scores of the
// logits, renormalised over the selection when K > 1, with the roundings of the dtype
template <typename T, typename M, typename LogitOf>
__device__ __forceinline__ void routing_weights(M taken, int K, LogitOf logit_of, int* sel, float* wsel) {
  float sum = 0.f;
  int n = 0;
  for (M rest = taken; rest != 0 && n < kMaxK; rest &= rest - 1, ++n) {   // set bits, ascending
    const int e = lowest_bit(rest);
    sel[n] = e;
    wsel[n] = round_to<T>(1.f / (1.f + expf(-logit_of(e))));
    sum += wsel[n];
  }
  if (K > 1) {
    const float denom = round_to<T>(round_to<T>(sum) + 1e-10f);
    for (int k = 0; k < K; ++k) wsel[k] = round_to<T>(wsel[k] / denom);
  }
}

// The counting sort of one CTA's 256 tokens: thread `threadIdx.x` owns token t with expert mask `taken`,
// experts sel[] and weights wsel[]; cta / num_ctas place the CTA among those that share the sort (their
// per-expert counts are in a.cta_counts when num_ctas > 1).  Every thread of the CTA must call it.
template <typename T, typename M>
__device__ __forceinline__ void scatter_rows(const RouteArgs& a, ScatterSmem& sm, int t, M taken, const int* sel,
                                             const float* wsel, int cta, int num_ctas) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int E = a.E, K = a.K;
  int ranks[kMaxK];
  warp_counts(taken, E, sm.warp_cnt, ranks);
  __syncthreads();
  // rows of every expert in all CTAs (tot) and in the CTAs before this one (bef); prefix over warps
  for (int i = tid; i < kWarps * E; i += kTok) {
    const int w = i / E, e = i - w * E;
    int pre = 0;
    for (int x = 0; x < w; ++x) pre += sm.warp_cnt[x][e];
    sm.warp_pre[w][e] = pre;
  }
  if (tid < E) {
    int tot = 0, bef = 0;
    if (num_ctas > 1) {
      for (int c = 0; c < num_ctas; ++c) {
        const int v = a.cta_counts[c * E + tid];
        tot += v;
        if (c < cta) bef += v;
      }
    } else {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) tot += sm.warp_cnt[w][tid];
    }
    sm.tot_s[tid] = tot;
    sm.bef_s[tid] = bef;
  }
  __syncthreads();
  if (warp == 0) {       // exclusive scan of the expert totals, 32 experts per trip
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int v = e < E ? sm.tot_s[e] : 0;
      int x = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      if (e < E) {
        sm.base[e] = carry + x - v + sm.bef_s[e];
        if (cta == 0) a.offsets[e] = carry + x;
      }
      carry += __shfl_sync(0xffffffffu, x, 31);
    }
  }
  __syncthreads();
  if (t >= a.T) return;
  if (a.identity_tail) a.sorted_token[a.T * K + t] = t;
  T* wout = static_cast<T*>(a.sorted_weight);
  for (int k = 0; k < K; ++k) {
    const int e = sel[k];
    const int pos = sm.base[e] + sm.warp_pre[warp][e] + ranks[k];
    a.sorted_token[pos] = t;
    a.sorted_expert[pos] = e;
    wout[pos] = from_float<T>(wsel[k]);
    a.slot_to_row[t * K + k] = pos;
  }
}

template <typename T, int EMAX>
__global__ void __launch_bounds__(kTok) moe_scatter_kernel(const RouteArgs a) {
  __shared__ ScatterSmem sm;
  const int t = blockIdx.x * kTok + threadIdx.x;
  using M = typename MaskOf<EMAX>::type;
  const M taken = t < a.T ? select_mask<T, EMAX>(a, t) : M(0);
  int sel[kMaxK];
  float wsel[kMaxK];
  if (t < a.T) {
    const T* row = static_cast<const T*>(a.logits) + static_cast<int64_t>(t) * a.E;
    routing_weights<T>(taken, a.K, [&](int e) { return to_float<T>(row[e]); }, sel, wsel);
  }
  scatter_rows<T>(a, sm, t, taken, sel, wsel, blockIdx.x, gridDim.x);
}

// ---------------------------------------------------------------------------------------------
// Gate projection + routing (+ row gather) in one launch, for batches of at most 256 tokens (decode):
//   logits[t, e] = bf16( x[t] . gate_w[e] )        Gate.forward, moe.py:49-52 (a bias-free matmul)
// followed by exactly the selection, weights and counting sort of the kernels above.  Phase 1: a warp per
// token computes the E dot products (x row in registers, gate rows through L1), selects the experts and
// leaves (mask, weights) in the workspace; CTAs take a ticket when they are done.  Phase 2: the CTA that
// takes the last ticket sorts all tokens (one thread per token), and when `gathered` is given copies the
// rows of x into sorted order (+ the identity tail) — worth doing here only for small batches, where one
// SM copies the few rows faster than another launch would start.
struct GateRouteArgs {
  RouteArgs r;                      // logits unused
  const __nv_bfloat16* x;           // [T, d]
  const __nv_bfloat16* gate_w;      // [E, d]
  int d;
  int32_t* ticket;                  // zero between launches
  unsigned long long* masks;        // [T]
  float* weights;                   // [T][kMaxK]
  __nv_bfloat16* gathered;          // [T*K (+ T), d] or null
};

constexpr int kGateWarps = 8;       // tokens per CTA in phase 1
constexpr size_t kGateSmemMax = 160 * 1024;   // largest gate matrix staged in shared memory

template <int EMAX>
__global__ void __launch_bounds__(kTok) moe_gate_route_kernel(const GateRouteArgs g) {
  using T = __nv_bfloat16;
  using M = typename MaskOf<EMAX>::type;
  __shared__ ScatterSmem sm;
  __shared__ int s_last;
  const RouteArgs& a = g.r;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int E = a.E, d = g.d;
  extern __shared__ uint4 s_gate[];            // the gate matrix [E, d] bf16: every warp of the CTA reads all of it
  {
    // this warp's token row first (up to 8 pieces per lane in flight), then the gate matrix, eight independent
    // loads per thread per trip: everything the phase reads from global memory is requested before anything
    // waits for it
    constexpr int kXPieces = 8;                  // d <= 2048 keeps the row in registers
    const int t = blockIdx.x * kGateWarps + warp;
    const bool live = t < a.T;
    uint4 xrow[kXPieces];
    const uint4* xr = reinterpret_cast<const uint4*>(g.x + static_cast<int64_t>(live ? t : 0) * d);
#pragma unroll
    for (int j = 0; j < kXPieces; ++j) {
      const int c = lane + 32 * j;               // 16-byte piece index within the row
      xrow[j] = (live && c * 8 < d) ? xr[c] : make_uint4(0u, 0u, 0u, 0u);
    }
    const uint4* src = reinterpret_cast<const uint4*>(g.gate_w);
    const int pieces = E * d / 8;
    for (int base = 0; base < pieces; base += kTok * 8) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = base + u * kTok + tid;
        v[u] = i < pieces ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = base + u * kTok + tid;
        if (i < pieces) s_gate[i] = v[u];
      }
    }
    __syncthreads();
    if (live) {
      float acc[EMAX];
#pragma unroll
      for (int e = 0; e < EMAX; ++e) acc[e] = 0.f;
#pragma unroll
      for (int j = 0; j < kXPieces; ++j) {
        const int c = (lane + 32 * j) * 8;
        if (c < d) {
          union { uint4 u; T b[8]; } xv;
          xv.u = xrow[j];
          float xf[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) xf[i] = __bfloat162float(xv.b[i]);
#pragma unroll
          for (int e = 0; e < EMAX; ++e) {
            if (e < E) {
              union { uint4 u; T b[8]; } wv;
              wv.u = s_gate[(e * d + c) / 8];
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[e] = fmaf(xf[i], __bfloat162float(wv.b[i]), acc[e]);
            }
          }
        }
      }
      float biased[EMAX];
#pragma unroll
      for (int e = 0; e < EMAX; ++e) {
        acc[e] = round_to<T>(warp_sum(acc[e]));     // every lane holds the logit
        biased[e] = e < E ? round_to<T>(acc[e] + round_to<T>(a.bias[e])) : -INFINITY;
      }
      const M taken = top_k_mask<EMAX>(biased, E, a.K);
      int sel[kMaxK];
      float wsel[kMaxK];
      routing_weights<T>(taken, a.K, [&](int e) {
        float v = 0.f;
#pragma unroll
        for (int x = 0; x < EMAX; ++x) v = x == e ? acc[x] : v;
        return v; }, sel, wsel);
      if (lane == 0) {
        g.masks[t] = static_cast<unsigned long long>(taken);
        for (int k = 0; k < a.K; ++k) g.weights[t * kMaxK + k] = wsel[k];
      }
    }
  }
  if (gridDim.x > 1) {
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(g.ticket, 1) == static_cast<int>(gridDim.x) - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) *g.ticket = 0;     // ready for the next launch
  } else {
    __syncthreads();                 // a single CTA: its own writes are visible to it after the barrier
  }
  const int t = tid;
  M taken = 0;
  int sel[kMaxK];
  float wsel[kMaxK];
  if (t < a.T) {
    taken = static_cast<M>(__ldcg(g.masks + t));
    int n = 0;
    for (M rest = taken; rest != 0 && n < kMaxK; rest &= rest - 1, ++n) {
      sel[n] = lowest_bit(rest);
      wsel[n] = __ldcg(g.weights + t * kMaxK + n);
    }
  }
  scatter_rows<T>(a, sm, t, taken, sel, wsel, 0, 1);
  if (g.gathered == nullptr) return;
  __syncthreads();                   // sorted_token is complete (written by this CTA)
  const int rows = a.T * a.K + (a.identity_tail ? a.T : 0);
  const int per_row = d / 8;         // 16-byte pieces per row
  for (int i = tid; i < rows * per_row; i += kTok) {
    const int r = i / per_row, c = i - r * per_row;
    const int src = a.sorted_token[r];
    reinterpret_cast<uint4*>(g.gathered + static_cast<int64_t>(r) * d)[c] =
        *reinterpret_cast<const uint4*>(g.x + static_cast<int64_t>(src) * d + c * 8);
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU over fused up-projection rows: act[r, j] = silu(h[r, j] + b[e_r, j]) * (h[r, F + j] + b[e_r, F + j])
// with every intermediate rounded to the dtype (bias add, silu, product), as the tensor-op sequence
// add -> silu -> mul on dtype tensors rounds.
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_kernel(const T* __restrict__ h, const T* __restrict__ bias, const int32_t* __restrict__ row_expert,
              T* __restrict__ act, int64_t rows, int F) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * F) return;
  const int64_t r = i / F;
  const int j = static_cast<int>(i - r * F);
  float g = to_float<T>(h[r * 2 * F + j]), u = to_float<T>(h[r * 2 * F + F + j]);
  if (bias) {
    const T* b = bias + static_cast<int64_t>(row_expert ? row_expert[r] : 0) * 2 * F;
    g = round_to<T>(g + to_float<T>(b[j]));
    u = round_to<T>(u + to_float<T>(b[F + j]));
  }
  const float s = round_to<T>(g / (1.f + expf(-g)));
  act[r * F + j] = from_float<T>(s * u);
}

// bf16, F % 8 == 0: eight outputs per thread with 16-byte loads
__global__ void __launch_bounds__(256)
swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ bias,
                     const int32_t* __restrict__ row_expert, __nv_bfloat16* __restrict__ act, int64_t rows,
                     int F) {
  const int F8 = F >> 3;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * F8) return;
  const int64_t r = i / F8;
  const int j = static_cast<int>(i - r * F8) << 3;
  union V {
    uint4 u;
    __nv_bfloat16 b[8];
  };
  V g, u, bg, bu, o;
  g.u = *reinterpret_cast<const uint4*>(h + r * 2 * F + j);
  u.u = *reinterpret_cast<const uint4*>(h + r * 2 * F + F + j);
  if (bias) {
    const __nv_bfloat16* b = bias + static_cast<int64_t>(row_expert ? row_expert[r] : 0) * 2 * F;
    bg.u = *reinterpret_cast<const uint4*>(b + j);
    bu.u = *reinterpret_cast<const uint4*>(b + F + j);
  }
#pragma unroll
  for (int x = 0; x < 8; ++x) {
    float gv = __bfloat162float(g.b[x]), uv = __bfloat162float(u.b[x]);
    if (bias) {
      gv = round_to<__nv_bfloat16>(gv + __bfloat162float(bg.b[x]));
      uv = round_to<__nv_bfloat16>(uv + __bfloat162float(bu.b[x]));
    }
    const float s = round_to<__nv_bfloat16>(gv / (1.f + expf(-gv)));
    o.b[x] = __float2bfloat16(s * uv);
  }
  *reinterpret_cast<uint4*>(act + r * F + j) = o.u;
}

// ---------------------------------------------------------------------------------------------
// Combine: out[t] = sum over the token's K expert rows in ascending expert order of
// round(round(y[row] + b2[e]) * w[row]), every partial sum rounded to the dtype (the reference
// accumulates with scatter_add_ in the activation dtype, moe.py:312-339), then + shared[t].
template <typename T>
__global__ void __launch_bounds__(256)
combine_kernel(const T* __restrict__ y, const T* __restrict__ bias, const int32_t* __restrict__ row_expert,
               const T* __restrict__ row_weight, const int32_t* __restrict__ slot_to_row,
               const T* __restrict__ shared, T* __restrict__ out, int64_t tokens, int K, int d) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= tokens * d) return;
  const int64_t t = i / d;
  const int j = static_cast<int>(i - t * d);
  float acc = 0.f;
  for (int k = 0; k < K; ++k) {
    const int row = slot_to_row[t * K + k];
    float v = to_float<T>(y[static_cast<int64_t>(row) * d + j]);
    if (bias) v = round_to<T>(v + to_float<T>(bias[static_cast<int64_t>(row_expert[row]) * d + j]));
    v = round_to<T>(v * to_float<T>(row_weight[row]));
    acc = k == 0 ? v : round_to<T>(acc + v);
  }
  if (shared) acc = round_to<T>(acc + to_float<T>(shared[i]));
  out[i] = from_float<T>(acc);
}

__global__ void __launch_bounds__(256)
combine_bf16x8_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ bias,
                      const int32_t* __restrict__ row_expert, const __nv_bfloat16* __restrict__ row_weight,
                      const int32_t* __restrict__ slot_to_row, const __nv_bfloat16* __restrict__ shared,
                      __nv_bfloat16* __restrict__ out, int64_t tokens, int K, int d) {
  const int d8 = d >> 3;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= tokens * d8) return;
  const int64_t t = i / d8;
  const int j = static_cast<int>(i - t * d8) << 3;
  union V {
    uint4 u;
    __nv_bfloat16 b[8];
  };
  float acc[8];
  for (int k = 0; k < K; ++k) {
    const int row = slot_to_row[t * K + k];
    V v, b;
    v.u = *reinterpret_cast<const uint4*>(y + static_cast<int64_t>(row) * d + j);
    if (bias) b.u = *reinterpret_cast<const uint4*>(bias + static_cast<int64_t>(row_expert[row]) * d + j);
    const float w = __bfloat162float(row_weight[row]);
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      float f = __bfloat162float(v.b[x]);
      if (bias) f = round_to<__nv_bfloat16>(f + __bfloat162float(b.b[x]));
      f = round_to<__nv_bfloat16>(f * w);
      acc[x] = k == 0 ? f : round_to<__nv_bfloat16>(acc[x] + f);
    }
  }
  V o;
  if (shared) {
    V s;
    s.u = *reinterpret_cast<const uint4*>(shared + t * d + j);
#pragma unroll
    for (int x = 0; x < 8; ++x) acc[x] = acc[x] + __bfloat162float(s.b[x]);
  }
#pragma unroll
  for (int x = 0; x < 8; ++x) o.b[x] = __float2bfloat16(acc[x]);
  *reinterpret_cast<uint4*>(out + t * d + j) = o.u;
}

}  // namespace
}  // namespace b200

extern "C" size_t b200_moe_route_workspace_bytes(int32_t num_tokens, int32_t num_experts) {
  if (num_tokens <= b200::kTok || num_experts <= 0) return 0;
  const size_t ctas = (static_cast<size_t>(num_tokens) + b200::kTok - 1) / b200::kTok;
  return ctas * static_cast<size_t>(num_experts) * sizeof(int32_t);
}

extern "C" int b200_moe_route(const void* gate_logits, const float* expert_bias, int32_t num_tokens,
                              int32_t num_experts, int32_t top_k, int32_t* sorted_token,
                              int32_t* sorted_expert, void* sorted_weight, int32_t* expert_offsets,
                              int32_t* slot_to_row, int32_t identity_tail, void* workspace,
                              size_t workspace_bytes, int32_t dtype, void* stream) {
  using namespace b200;
  if (num_tokens < 0 || num_experts <= 0 || top_k <= 0 || top_k > num_experts) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (num_experts > kMaxE || top_k > kMaxK || num_tokens > kMaxTokens) return B200_ERR_UNSUPPORTED;
  if (!expert_offsets) return B200_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (num_tokens > 0 &&
      (!gate_logits || !expert_bias || !sorted_token || !sorted_expert || !sorted_weight || !slot_to_row))
    return B200_ERR_ARG;
  const size_t need = b200_moe_route_workspace_bytes(num_tokens, num_experts);
  if (need > 0 && (!workspace || workspace_bytes < need)) return B200_ERR_WORKSPACE;
  RouteArgs a{};
  a.logits = gate_logits;
  a.bias = expert_bias;
  a.T = num_tokens;
  a.E = num_experts;
  a.K = top_k;
  a.sorted_token = sorted_token;
  a.sorted_expert = sorted_expert;
  a.sorted_weight = sorted_weight;
  a.offsets = expert_offsets;
  a.slot_to_row = slot_to_row;
  a.cta_counts = static_cast<int32_t*>(workspace);
  a.identity_tail = identity_tail != 0;
  const int grid = num_tokens == 0 ? 1 : (num_tokens + kTok - 1) / kTok;   // 0 tokens: offsets = 0
#define ROUTE_LAUNCH(T, EMAX)                                                       \
  do {                                                                              \
    if (grid > 1) moe_count_kernel<T, EMAX><<<grid, kTok, 0, s>>>(a);               \
    moe_scatter_kernel<T, EMAX><<<grid, kTok, 0, s>>>(a);                           \
  } while (0)
  if (dtype == B200_DTYPE_F32) {
    if (num_experts <= 16) ROUTE_LAUNCH(float, 16);
    else if (num_experts <= 32) ROUTE_LAUNCH(float, 32);
    else ROUTE_LAUNCH(float, 64);
  } else {
    if (num_experts <= 16) ROUTE_LAUNCH(__nv_bfloat16, 16);
    else if (num_experts <= 32) ROUTE_LAUNCH(__nv_bfloat16, 32);
    else ROUTE_LAUNCH(__nv_bfloat16, 64);
  }
#undef ROUTE_LAUNCH
  return launch_result();
}

extern "C" size_t b200_moe_gate_route_workspace_bytes(void) {
  return 256 + b200::kTok * sizeof(unsigned long long) + b200::kTok * b200::kMaxK * sizeof(float);
}

extern "C" int b200_moe_gate_route(const void* x, const void* gate_weight, const float* expert_bias,
                                   int32_t num_tokens, int32_t num_experts, int32_t top_k, int32_t d_model,
                                   int32_t* sorted_token, int32_t* sorted_expert, void* sorted_weight,
                                   int32_t* expert_offsets, int32_t* slot_to_row, int32_t identity_tail,
                                   void* gathered, void* workspace, size_t workspace_bytes, int32_t dtype,
                                   void* stream) {
  using namespace b200;
  if (num_tokens < 0 || num_experts <= 0 || top_k <= 0 || top_k > num_experts || d_model <= 0) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_BF16 || num_experts > kMaxE || top_k > kMaxK || num_tokens > kTok || d_model % 8 != 0 ||
      d_model > 2048)
    return B200_ERR_UNSUPPORTED;
  if (num_tokens == 0) return B200_ERR_UNSUPPORTED;   // the plain routing entry point writes the empty offsets
  if (!x || !gate_weight || !expert_bias || !sorted_token || !sorted_expert || !sorted_weight || !expert_offsets ||
      !slot_to_row)
    return B200_ERR_ARG;
  if (!aligned16(x) || !aligned16(gate_weight) || (gathered && !aligned16(gathered))) return B200_ERR_ALIGN;
  if (!workspace || workspace_bytes < b200_moe_gate_route_workspace_bytes()) return B200_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return B200_ERR_ALIGN;
  GateRouteArgs g{};
  g.r.bias = expert_bias;
  g.r.T = num_tokens;
  g.r.E = num_experts;
  g.r.K = top_k;
  g.r.sorted_token = sorted_token;
  g.r.sorted_expert = sorted_expert;
  g.r.sorted_weight = sorted_weight;
  g.r.offsets = expert_offsets;
  g.r.slot_to_row = slot_to_row;
  g.r.identity_tail = identity_tail != 0;
  g.x = static_cast<const __nv_bfloat16*>(x);
  g.gate_w = static_cast<const __nv_bfloat16*>(gate_weight);
  g.d = d_model;
  uint8_t* w = static_cast<uint8_t*>(workspace);
  g.ticket = reinterpret_cast<int32_t*>(w);
  g.masks = reinterpret_cast<unsigned long long*>(w + 256);
  g.weights = reinterpret_cast<float*>(w + 256 + kTok * sizeof(unsigned long long));
  g.gathered = static_cast<__nv_bfloat16*>(gathered);
  const int grid = (num_tokens + kGateWarps - 1) / kGateWarps;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = static_cast<size_t>(num_experts) * d_model * sizeof(__nv_bfloat16);   // the gate matrix
  if (smem > kGateSmemMax) return B200_ERR_UNSUPPORTED;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return B200_ERR_UNSUPPORTED;
#define GATE_LAUNCH(EMAX)                                                                                          \
  do {                                                                                                             \
    static bool configured[64] = {};   /* per-device flag, idempotent (see the note on statics in the header) */   \
    if (!configured[dev]) {                                                                                        \
      if (cudaFuncSetAttribute(moe_gate_route_kernel<EMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                               static_cast<int>(kGateSmemMax)) != cudaSuccess)                                     \
        return B200_ERR_LAUNCH;                                                                                    \
      configured[dev] = true;                                                                                      \
    }                                                                                                              \
    moe_gate_route_kernel<EMAX><<<grid, kTok, smem, s>>>(g);                                                       \
  } while (0)
  if (num_experts <= 16) GATE_LAUNCH(16);
  else if (num_experts <= 32) GATE_LAUNCH(32);
  else GATE_LAUNCH(64);
#undef GATE_LAUNCH
  return launch_result();
}

extern "C" int b200_swiglu(const void* h, const void* bias, const int32_t* row_expert, void* act,
                           int64_t num_rows, int32_t d_ff, int32_t dtype, void* stream) {
  using namespace b200;
  if (num_rows < 0 || d_ff <= 0) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (num_rows == 0) return B200_OK;
  if (!h || !act) return B200_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = dtype == B200_DTYPE_BF16 && d_ff % 8 == 0 && aligned16(h) && aligned16(act) &&
                   (!bias || aligned16(bias));
  const int64_t work = vec ? num_rows * (d_ff / 8) : num_rows * d_ff;
  const int64_t grid = (work + 255) / 256;
  if (grid > 2147483647) return B200_ERR_TOO_LARGE;
  if (vec)
    swiglu_bf16x8_kernel<<<static_cast<int>(grid), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(bias), row_expert,
        static_cast<__nv_bfloat16*>(act), num_rows, d_ff);
  else if (dtype == B200_DTYPE_BF16)
    swiglu_kernel<__nv_bfloat16><<<static_cast<int>(grid), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(bias), row_expert,
        static_cast<__nv_bfloat16*>(act), num_rows, d_ff);
  else
    swiglu_kernel<float><<<static_cast<int>(grid), 256, 0, s>>>(
        static_cast<const float*>(h), static_cast<const float*>(bias), row_expert, static_cast<float*>(act),
        num_rows, d_ff);
  return launch_result();
}

extern "C" int b200_moe_combine(const void* expert_out, const void* bias, const int32_t* row_expert,
                                const void* row_weight, const int32_t* slot_to_row, const void* shared,
                                void* out, int64_t num_tokens, int32_t top_k, int32_t d_model,
                                int32_t dtype, void* stream) {
  using namespace b200;
  if (num_tokens < 0 || top_k <= 0 || d_model <= 0) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (num_tokens == 0) return B200_OK;
  if (!expert_out || !row_weight || !slot_to_row || !out || (bias && !row_expert)) return B200_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = dtype == B200_DTYPE_BF16 && d_model % 8 == 0 && aligned16(expert_out) &&
                   aligned16(out) && (!bias || aligned16(bias)) && (!shared || aligned16(shared));
  const int64_t work = vec ? num_tokens * (d_model / 8) : num_tokens * d_model;
  const int64_t grid = (work + 255) / 256;
  if (grid > 2147483647) return B200_ERR_TOO_LARGE;
  if (vec)
    combine_bf16x8_kernel<<<static_cast<int>(grid), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(expert_out), static_cast<const __nv_bfloat16*>(bias), row_expert,
        static_cast<const __nv_bfloat16*>(row_weight), slot_to_row,
        static_cast<const __nv_bfloat16*>(shared), static_cast<__nv_bfloat16*>(out), num_tokens, top_k,
        d_model);
  else if (dtype == B200_DTYPE_BF16)
    combine_kernel<__nv_bfloat16><<<static_cast<int>(grid), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(expert_out), static_cast<const __nv_bfloat16*>(bias), row_expert,
        static_cast<const __nv_bfloat16*>(row_weight), slot_to_row,
        static_cast<const __nv_bfloat16*>(shared), static_cast<__nv_bfloat16*>(out), num_tokens, top_k,
        d_model);
  else
    combine_kernel<float><<<static_cast<int>(grid), 256, 0, s>>>(
        static_cast<const float*>(expert_out), static_cast<const float*>(bias), row_expert,
        static_cast<const float*>(row_weight), slot_to_row, static_cast<const float*>(shared),
        static_cast<float*>(out), num_tokens, top_k, d_model);
  return launch_result();
}
