// Fused element-wise stages around attention (one launch each instead of ~10 / ~25 tensor ops):
//
//  add_rmsnorm          residual-stream RMSNorm with the optional fused residual add of the reference
//                       (model/utils.py:54-67): xf = float(x) [+ float(residual)];
//                       y = (w * xf * rsqrt(mean(xf^2) + eps)) -> dtype of x; new residual = xf -> dtype of x.
//  qk_norm_rope_store   what GroupedQueryAttention.forward does between the projections and the
//                       attention call (model/attention/GQA.py:81-102): RMSNorm over the WHOLE projected
//                       q vector and the whole k vector (eps = machine epsilon of the dtype, result
//                       rounded to the dtype), half-split RoPE in fp32 at the token's position, result
//                       rounded to the dtype; K (after norm + RoPE) and V (raw) are also scattered into
//                       the paged cache through slot_mapping.
//
// General kernels: one CTA per token row, reduced with warp shuffles + one shared-memory exchange.
// bf16 rows whose widths are multiples of 256 take the fast kernels: one warp per row, 16-byte
// loads and stores, warp shuffles only.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();   // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) t += scratch[w];
  return t;
}

template <typename T, typename R>
__global__ void __launch_bounds__(kThreads)
add_rmsnorm_kernel(const T* __restrict__ x, const R* __restrict__ residual, const float* __restrict__ w,
                   T* __restrict__ y, T* __restrict__ res_out, int d, float eps) {
  __shared__ float scratch[kThreads / 32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * d;
  const R* rr = residual ? residual + row * d : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += kThreads) {
    float v = to_float<T>(xr[i]);
    if (rr) v += to_float<R>(rr[i]);
    ss += v * v;
  }
  const float inv = rsqrtf(block_sum(ss, scratch) / static_cast<float>(d) + eps);
  for (int i = threadIdx.x; i < d; i += kThreads) {
    float v = to_float<T>(xr[i]);
    if (rr) v += to_float<R>(rr[i]);
    y[row * d + i] = from_float<T>(w[i] * v * inv);
    if (res_out) res_out[row * d + i] = from_float<T>(v);
  }
}

struct QkArgs {
  const void* qkv;       // [T, qkv_stride]: q (Hq*D) | k (Hkv*D) | v (Hkv*D)
  int64_t qkv_stride;
  const float* q_norm_w; // [Hq*D]
  const float* k_norm_w; // [Hkv*D]
  const float* rope;     // [max_pos, D]: cos (D/2) | sin (D/2)
  const int64_t* positions;
  int64_t max_pos;
  void* q_out;           // [T, Hq, D]
  void* k_out;           // [T, Hkv, D]
  void* k_cache;         // [num_slots, Hkv, D] or null
  void* v_cache;
  const int64_t* slots;
  int64_t num_slots;
  int Hq, Hkv, D;
  float eps;
  int32_t* status;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) qk_norm_rope_store_kernel(const QkArgs a) {
  __shared__ float scratch[kThreads / 32];
  const int64_t t = blockIdx.x;
  const int Wq = a.Hq * a.D, Wk = a.Hkv * a.D, half = a.D / 2;
  const T* row = static_cast<const T*>(a.qkv) + t * a.qkv_stride;
  const T* qr = row;
  const T* kr = row + Wq;
  const T* vr = row + Wq + Wk;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < Wq; i += kThreads) {
    const float v = to_float<T>(qr[i]);
    sq += v * v;
  }
  for (int i = threadIdx.x; i < Wk; i += kThreads) {
    const float v = to_float<T>(kr[i]);
    sk += v * v;
  }
  const float iq = rsqrtf(block_sum(sq, scratch) / static_cast<float>(Wq) + a.eps);
  const float ik = rsqrtf(block_sum(sk, scratch) / static_cast<float>(Wk) + a.eps);
  int64_t pos = a.positions[t];
  if (pos < 0 || pos >= a.max_pos) {
    report(a.status, B200_ERR_BOUNDS);
    pos = pos < 0 ? 0 : a.max_pos - 1;
  }
  const float* cs = a.rope + pos * a.D;
  int64_t slot = a.k_cache ? a.slots[t] : -1;
  if (slot >= a.num_slots) {
    report(a.status, B200_ERR_BOUNDS);
    slot = -1;
  }
  T* qo = static_cast<T*>(a.q_out) + t * Wq;
  T* ko = static_cast<T*>(a.k_out) + t * Wk;
  T* kc = slot >= 0 ? static_cast<T*>(a.k_cache) + slot * Wk : nullptr;
  T* vc = slot >= 0 ? static_cast<T*>(a.v_cache) + slot * Wk : nullptr;
  // normalised values are rounded to the dtype before the rotation, as nn.RMSNorm returns its input dtype
  for (int i = threadIdx.x; i < a.Hq * half; i += kThreads) {
    const int h = i / half, j = i - h * half;
    const int i1 = h * a.D + j, i2 = i1 + half;
    const float x1 = to_float<T>(from_float<T>(to_float<T>(qr[i1]) * iq * a.q_norm_w[i1]));
    const float x2 = to_float<T>(from_float<T>(to_float<T>(qr[i2]) * iq * a.q_norm_w[i2]));
    const float c = cs[j], s = cs[half + j];
    qo[i1] = from_float<T>(x1 * c - x2 * s);
    qo[i2] = from_float<T>(x2 * c + x1 * s);
  }
  for (int i = threadIdx.x; i < a.Hkv * half; i += kThreads) {
    const int h = i / half, j = i - h * half;
    const int i1 = h * a.D + j, i2 = i1 + half;
    const float x1 = to_float<T>(from_float<T>(to_float<T>(kr[i1]) * ik * a.k_norm_w[i1]));
    const float x2 = to_float<T>(from_float<T>(to_float<T>(kr[i2]) * ik * a.k_norm_w[i2]));
    const float c = cs[j], s = cs[half + j];
    const T y1 = from_float<T>(x1 * c - x2 * s), y2 = from_float<T>(x2 * c + x1 * s);
    ko[i1] = y1;
    ko[i2] = y2;
    if (kc) {
      kc[i1] = y1;
      kc[i2] = y2;
    }
  }
  if (vc)
    for (int i = threadIdx.x; i < Wk; i += kThreads) vc[i] = vr[i];
}


// ---- bf16 fast paths: one warp per token row, 16-byte loads, no shared memory -------------------
union Bf16x8 {
  uint4 u;
  __nv_bfloat16 b[8];
};

constexpr int kWarpRows = 4;   // rows (warps) per CTA

// d % 256 == 0, d <= 2048: the row stays in registers between the reduction and the scaling
template <int CHUNKS>
__global__ void __launch_bounds__(kWarpRows * 32)
add_rmsnorm_bf16_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                             const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                             __nv_bfloat16* __restrict__ res_out, int64_t rows, float eps) {
  constexpr int d = CHUNKS * 256;
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpRows + (threadIdx.x >> 5);
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * d;
  float v[CHUNKS][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    Bf16x8 a, r;
    a.u = *reinterpret_cast<const uint4*>(xr + c * 256 + lane * 8);
    if (residual) r.u = *reinterpret_cast<const uint4*>(residual + row * d + c * 256 + lane * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float f = __bfloat162float(a.b[i]);
      if (residual) f += __bfloat162float(r.b[i]);
      v[c][i] = f;
      ss += f * f;
    }
  }
  const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(d) + eps);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const float4 w0 = *reinterpret_cast<const float4*>(w + c * 256 + lane * 8);
    const float4 w1 = *reinterpret_cast<const float4*>(w + c * 256 + lane * 8 + 4);
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    Bf16x8 o, ro;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o.b[i] = __float2bfloat16(ww[i] * v[c][i] * inv);
      ro.b[i] = __float2bfloat16(v[c][i]);
    }
    *reinterpret_cast<uint4*>(y + row * d + c * 256 + lane * 8) = o.u;
    if (res_out) *reinterpret_cast<uint4*>(res_out + row * d + c * 256 + lane * 8) = ro.u;
  }
}

// Hq*D and Hkv*D multiples of 256, D in {32, 64, 128, 256}: a lane's 8 elements and their RoPE
// partners (half a head away) sit in the same 256-element chunk, (D/2)/8 lanes apart.
// NQ / NK = number of 256-element chunks of the q / k row (compile-time, so that the whole row sits in
// registers and every global load of the token is in flight before the first one is waited for).
template <int NQ, int NK>
__global__ void __launch_bounds__(kWarpRows * 32)
qk_norm_rope_store_bf16_warp_kernel(const QkArgs a, int64_t num_tokens) {
  using T = __nv_bfloat16;
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarpRows + (threadIdx.x >> 5);
  if (t >= num_tokens) return;
  constexpr int Wq = NQ * 256, Wk = NK * 256;
  const int half = a.D / 2, partner = half / 8;
  const T* qr = static_cast<const T*>(a.qkv) + t * a.qkv_stride;
  const T* kr = qr + Wq;
  const T* vr = kr + Wk;
  // position and slot first, then the row: the rotation coefficients (a second round trip behind the
  // position) are fetched while the row's loads are still in flight
  int64_t pos = a.positions[t];
  int64_t slot = a.k_cache ? a.slots[t] : -1;
  Bf16x8 qv[NQ], kv[NK];
  uint4 vv[NK];
#pragma unroll
  for (int j = 0; j < NQ; ++j) qv[j].u = *reinterpret_cast<const uint4*>(qr + j * 256 + lane * 8);
#pragma unroll
  for (int j = 0; j < NK; ++j) kv[j].u = *reinterpret_cast<const uint4*>(kr + j * 256 + lane * 8);
  const bool store = slot >= 0 && slot < a.num_slots;
  if (a.k_cache && slot >= a.num_slots && lane == 0) report(a.status, B200_ERR_BOUNDS);
  if (store) {
#pragma unroll
    for (int j = 0; j < NK; ++j) vv[j] = *reinterpret_cast<const uint4*>(vr + j * 256 + lane * 8);
  }
  if (pos < 0 || pos >= a.max_pos) {
    if (lane == 0) report(a.status, B200_ERR_BOUNDS);
    pos = pos < 0 ? 0 : a.max_pos - 1;
  }
  // a lane's eight elements sit at the same offset of their head in every chunk (256 is a multiple of D): one
  // set of eight cosines and sines serves all chunks of q and k
  const float* cs = a.rope + pos * a.D;
  const int j0 = (lane * 8) % a.D;
  const bool first = j0 < half;
  const int jj = first ? j0 : j0 - half;
  const float4 c0 = *reinterpret_cast<const float4*>(cs + jj), c1 = *reinterpret_cast<const float4*>(cs + jj + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(cs + half + jj);
  const float4 s1 = *reinterpret_cast<const float4*>(cs + half + jj + 4);
  const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  float sq = 0.f, sk = 0.f;
#pragma unroll
  for (int j = 0; j < NQ; ++j) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float f = __bfloat162float(qv[j].b[i]);
      sq += f * f;
    }
  }
#pragma unroll
  for (int j = 0; j < NK; ++j) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float f = __bfloat162float(kv[j].b[i]);
      sk += f * f;
    }
  }
  const float iq = rsqrtf(warp_sum(sq) / static_cast<float>(Wq) + a.eps);
  const float ik = rsqrtf(warp_sum(sk) / static_cast<float>(Wk) + a.eps);
  // one 256-element chunk of q or k: normalise, round, rotate, round
  auto rotate = [&](const Bf16x8& u, const float* nw, float inv, int c) -> uint4 {
    Bf16x8 o;
    const float4 w0 = *reinterpret_cast<const float4*>(nw + c), w1 = *reinterpret_cast<const float4*>(nw + c + 4);
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float xv = __bfloat162float(__float2bfloat16(__bfloat162float(u.b[i]) * inv * ww[i]));
      const float pv = __shfl_xor_sync(0xffffffffu, xv, partner);
      o.b[i] = __float2bfloat16(first ? xv * cc[i] - pv * sn[i] : xv * cc[i] + pv * sn[i]);
    }
    return o.u;
  };
  T* qo = static_cast<T*>(a.q_out) + t * Wq;
#pragma unroll
  for (int j = 0; j < NQ; ++j)
    *reinterpret_cast<uint4*>(qo + j * 256 + lane * 8) = rotate(qv[j], a.q_norm_w, iq, j * 256 + lane * 8);
  T* ko = static_cast<T*>(a.k_out) + t * Wk;
  T* kc = store ? static_cast<T*>(a.k_cache) + slot * Wk : nullptr;
  T* vc = store ? static_cast<T*>(a.v_cache) + slot * Wk : nullptr;
#pragma unroll
  for (int j = 0; j < NK; ++j) {
    const int c = j * 256 + lane * 8;
    const uint4 o = rotate(kv[j], a.k_norm_w, ik, c);
    *reinterpret_cast<uint4*>(ko + c) = o;
    if (store) {
      *reinterpret_cast<uint4*>(kc + c) = o;
      *reinterpret_cast<uint4*>(vc + c) = vv[j];
    }
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_add_rmsnorm(const void* x, const void* residual, const float* weight, void* y,
                                void* residual_out, int64_t num_rows, int32_t dim, float eps,
                                int32_t dtype, int32_t residual_dtype, void* stream) {
  using namespace b200;
  if (num_rows < 0 || dim <= 0) return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (residual && residual_dtype != B200_DTYPE_F32 && residual_dtype != B200_DTYPE_BF16)
    return B200_ERR_UNSUPPORTED;
  if (num_rows == 0) return B200_OK;
  if (!x || !weight || !y) return B200_ERR_ARG;
  if (num_rows > 2147483647) return B200_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = static_cast<int>(num_rows);
  if (dtype == B200_DTYPE_BF16 && (!residual || residual_dtype == B200_DTYPE_BF16) && dim % 256 == 0 &&
      dim <= 2048 && aligned16(x) && aligned16(y) && aligned16(weight) && (!residual || aligned16(residual)) &&
      (!residual_out || aligned16(residual_out))) {
    const int wgrid = static_cast<int>((num_rows + kWarpRows - 1) / kWarpRows);
#define WARP_LAUNCH(C)                                                                               \
  case C:                                                                                            \
    add_rmsnorm_bf16_warp_kernel<C><<<wgrid, kWarpRows * 32, 0, s>>>(                                \
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual), weight,   \
        static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(residual_out), num_rows, eps);   \
    break
    switch (dim / 256) {
      WARP_LAUNCH(1); WARP_LAUNCH(2); WARP_LAUNCH(3); WARP_LAUNCH(4);
      WARP_LAUNCH(5); WARP_LAUNCH(6); WARP_LAUNCH(7); WARP_LAUNCH(8);
    }
#undef WARP_LAUNCH
    return launch_result();
  }
  const bool rf32 = !residual || residual_dtype == B200_DTYPE_F32;
#define LAUNCH(T, R)                                                                               \
  add_rmsnorm_kernel<T, R><<<grid, kThreads, 0, s>>>(static_cast<const T*>(x),                     \
                                                     static_cast<const R*>(residual), weight,      \
                                                     static_cast<T*>(y),                           \
                                                     static_cast<T*>(residual_out), dim, eps)
  if (dtype == B200_DTYPE_F32) {
    if (rf32) LAUNCH(float, float); else LAUNCH(float, __nv_bfloat16);
  } else {
    if (rf32) LAUNCH(__nv_bfloat16, float); else LAUNCH(__nv_bfloat16, __nv_bfloat16);
  }
#undef LAUNCH
  return launch_result();
}

extern "C" int b200_qk_norm_rope_store(const void* qkv, int64_t qkv_token_stride,
                                       const float* q_norm_weight, const float* k_norm_weight,
                                       const float* rope_table, int64_t rope_positions,
                                       const int64_t* positions, void* q_out, void* k_out,
                                       void* k_cache, void* v_cache, const int64_t* slot_mapping,
                                       int64_t num_slots, int64_t num_tokens, int32_t num_q_heads,
                                       int32_t num_kv_heads, int32_t head_dim, float eps, int32_t dtype,
                                       int32_t* status, void* stream) {
  using namespace b200;
  if (num_tokens < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || (head_dim & 1) ||
      rope_positions <= 0)
    return B200_ERR_ARG;
  if (dtype != B200_DTYPE_F32 && dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  if (num_tokens == 0) return B200_OK;
  if (!qkv || !q_norm_weight || !k_norm_weight || !rope_table || !positions || !q_out || !k_out)
    return B200_ERR_ARG;
  if ((k_cache == nullptr) != (v_cache == nullptr)) return B200_ERR_ARG;
  if (k_cache && !slot_mapping) return B200_ERR_ARG;
  const int64_t width = static_cast<int64_t>(num_q_heads + 2 * num_kv_heads) * head_dim;
  if (qkv_token_stride < width || num_tokens > 2147483647) return B200_ERR_ARG;
  QkArgs a{};
  a.qkv = qkv;
  a.qkv_stride = qkv_token_stride;
  a.q_norm_w = q_norm_weight;
  a.k_norm_w = k_norm_weight;
  a.rope = rope_table;
  a.positions = positions;
  a.max_pos = rope_positions;
  a.q_out = q_out;
  a.k_out = k_out;
  a.k_cache = k_cache;
  a.v_cache = v_cache;
  a.slots = slot_mapping;
  a.num_slots = num_slots;
  a.Hq = num_q_heads;
  a.Hkv = num_kv_heads;
  a.D = head_dim;
  a.eps = eps;
  a.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = static_cast<int>(num_tokens);
  const int Wq = num_q_heads * head_dim, Wk = num_kv_heads * head_dim;
  const bool d_ok = head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256;
  if (dtype == B200_DTYPE_BF16 && d_ok && Wq % 256 == 0 && Wk % 256 == 0 && qkv_token_stride % 8 == 0 &&
      aligned16(qkv) && aligned16(q_norm_weight) && aligned16(k_norm_weight) && aligned16(rope_table) &&
      aligned16(q_out) && aligned16(k_out) && (!k_cache || (aligned16(k_cache) && aligned16(v_cache)))) {
    const int wgrid = static_cast<int>((num_tokens + kWarpRows - 1) / kWarpRows);
    const int nq = Wq / 256, nk = Wk / 256;
#define QK_LAUNCH(NQ, NK)                                                                       \
  if (nq == NQ && nk == NK) {                                                                   \
    qk_norm_rope_store_bf16_warp_kernel<NQ, NK><<<wgrid, kWarpRows * 32, 0, s>>>(a, num_tokens); \
    return launch_result();                                                                     \
  }
    // (q chunks, k chunks) of the row widths in use: 16/4 heads x 64, 32/8 x 128, 8/2 x 128, 16/16 x 64, 4/2 x 64 ...
    QK_LAUNCH(4, 1) QK_LAUNCH(16, 4) QK_LAUNCH(4, 4) QK_LAUNCH(8, 2) QK_LAUNCH(8, 8) QK_LAUNCH(2, 1) QK_LAUNCH(1, 1)
    QK_LAUNCH(2, 2) QK_LAUNCH(8, 1) QK_LAUNCH(8, 4) QK_LAUNCH(16, 2) QK_LAUNCH(16, 8)
#undef QK_LAUNCH
  }
  if (dtype == B200_DTYPE_F32)
    qk_norm_rope_store_kernel<float><<<grid, kThreads, 0, s>>>(a);
  else
    qk_norm_rope_store_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(a);
  return launch_result();
}

// ---------------------------------------------------------------------------------------------
// MLA pre-attention stage (MultiHeadLatentAttention.forward between the projections and the attention,
// model/attention/MLA.py:114-131,137-138), one warp per token:
//   q_out[t, h]   = [ q_nope[t, h] (copied) | rope(q_rope[t, h]) ]           from the q up-projection row
//   rows_out[t]   = [ kv_norm(c[t]) | rope(k_rope[t]) ]                       from the kv down-projection row
//   latent_cache[slot_mapping[t]] = rows_out[t]                               (slot < 0 skipped)
// kv_norm is RMSNorm over the kv_lora_rank columns in fp32, rounded to the dtype.  RoPE is the
// reference's half-split rotation in fp32 with the table sliced to the first rope_dim columns of a row:
// cos = row[0 : rope_dim/2], sin = row[rope_dim/2 : rope_dim] — for a table wider than rope_dim that
// "sin" is not a sine (model/attention/utils.py:38); the slice is reproduced as it is.
namespace b200 {
namespace {

struct MlaProArgs {
  const __nv_bfloat16* qf;      // [T, >= H*hd + H*dr]: q_nope of all heads, then q_rope of all heads
  int64_t qf_stride;
  const __nv_bfloat16* kvp;     // [T, >= r + dr]: latent c, then k_rope
  int64_t kvp_stride;
  const float* kv_norm_w;       // [r]
  const float* rope;            // [max_pos, rope_width]
  int64_t rope_width, max_pos;
  const int64_t* positions;
  __nv_bfloat16* q_out;         // [T, H, hd + dr]
  __nv_bfloat16* rows_out;      // [T, r + dr] or null
  __nv_bfloat16* cache;         // [num_slots, r + dr] or null
  const int64_t* slots;
  int64_t num_slots;
  int H, hd, dr, r;
  float eps;
  int32_t* status;
};

// rotate 8 consecutive elements of a half-split pair: x = own chunk, the partner chunk (half a vector
// away) comes from the lane `partner_lanes` away; j0 = index of the chunk's first element within its half
__device__ __forceinline__ uint4 rope8(uint4 raw, bool first_half, const float* cs, int j0, int half, int partner_lanes) {
  Bf16x8 u, o;
  u.u = raw;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float xv = __bfloat162float(u.b[i]);
    const float pv = __shfl_xor_sync(0xffffffffu, xv, partner_lanes);
    const float c = cs[j0 + i], s = cs[half + j0 + i];
    o.b[i] = __float2bfloat16(first_half ? xv * c - pv * s : xv * c + pv * s);
  }
  return o.u;
}

__global__ void __launch_bounds__(kWarpRows * 32) mla_prologue_kernel(const MlaProArgs a, int64_t num_tokens) {
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kWarpRows + (threadIdx.x >> 5);
  if (t >= num_tokens) return;
  const int H = a.H, hd = a.hd, dr = a.dr, r = a.r, half = dr / 2, W = hd + dr;
  int64_t pos = a.positions[t];
  if (pos < 0 || pos >= a.max_pos) {
    if (lane == 0) report(a.status, B200_ERR_BOUNDS);
    pos = pos < 0 ? 0 : a.max_pos - 1;
  }
  const float* cs = a.rope + pos * a.rope_width;
  const __nv_bfloat16* qrow = a.qf + t * a.qf_stride;
  __nv_bfloat16* qo = a.q_out + t * H * W;
  // ---- q_nope: straight copy, 16 bytes per lane and trip
  const int nope_chunks = H * hd / 8, cph = hd / 8;
  for (int c = lane; c < nope_chunks; c += 32) {
    const int h = c / cph, j = c - h * cph;
    *reinterpret_cast<uint4*>(qo + h * W + j * 8) = *reinterpret_cast<const uint4*>(qrow + c * 8);
  }
  // ---- q_rope: dr/8 chunks per head, partner chunk half a head away = (dr/16) lanes away
  const int rpc = dr / 8, partner = rpc / 2;
  const __nv_bfloat16* qr = qrow + H * hd;
  for (int c0 = 0; c0 < H * rpc; c0 += 32) {      // H * rpc is a multiple of 32 or the tail lanes idle in pairs
    const int c = c0 + lane;
    const bool live = c < H * rpc;
    const int h = live ? c / rpc : 0, j = live ? c - h * rpc : 0;
    const uint4 raw = live ? *reinterpret_cast<const uint4*>(qr + c * 8) : make_uint4(0u, 0u, 0u, 0u);
    const bool first = j < partner;
    const uint4 rot = rope8(raw, first, cs, (first ? j : j - partner) * 8, half, partner);
    if (live) *reinterpret_cast<uint4*>(qo + h * W + hd + j * 8) = rot;
  }
  // ---- latent row: RMSNorm of c, RoPE of k_rope
  const __nv_bfloat16* krow = a.kvp + t * a.kvp_stride;
  float ss = 0.f;
  for (int c = lane; c < r / 8; c += 32) {
    Bf16x8 u;
    u.u = *reinterpret_cast<const uint4*>(krow + c * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float f = __bfloat162float(u.b[i]);
      ss += f * f;
    }
  }
  const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(r) + a.eps);
  int64_t slot = a.cache ? a.slots[t] : -1;
  if (slot >= a.num_slots) {
    if (lane == 0) report(a.status, B200_ERR_BOUNDS);
    slot = -1;
  }
  __nv_bfloat16* ro = a.rows_out ? a.rows_out + t * (r + dr) : nullptr;
  __nv_bfloat16* co = slot >= 0 ? a.cache + slot * (r + dr) : nullptr;
  for (int c = lane; c < r / 8; c += 32) {
    Bf16x8 u, o;
    u.u = *reinterpret_cast<const uint4*>(krow + c * 8);
    const float4 w0 = *reinterpret_cast<const float4*>(a.kv_norm_w + c * 8);
    const float4 w1 = *reinterpret_cast<const float4*>(a.kv_norm_w + c * 8 + 4);
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) o.b[i] = __float2bfloat16(__bfloat162float(u.b[i]) * inv * ww[i]);
    if (ro) *reinterpret_cast<uint4*>(ro + c * 8) = o.u;
    if (co) *reinterpret_cast<uint4*>(co + c * 8) = o.u;
  }
  {
    const bool live = lane < rpc;
    const uint4 raw = live ? *reinterpret_cast<const uint4*>(krow + r + lane * 8) : make_uint4(0u, 0u, 0u, 0u);
    const bool first = lane < partner;
    const uint4 rot = rope8(raw, first, cs, (first ? lane : lane - partner) * 8, half, partner);
    if (live) {
      if (ro) *reinterpret_cast<uint4*>(ro + r + lane * 8) = rot;
      if (co) *reinterpret_cast<uint4*>(co + r + lane * 8) = rot;
    }
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_mla_prologue(const void* q_up, int64_t q_up_stride, const void* kv_down, int64_t kv_down_stride,
                                 const float* kv_norm_weight, const float* rope_table, int64_t rope_width,
                                 int64_t rope_positions, const int64_t* positions, void* q_out, void* rows_out,
                                 void* latent_cache, const int64_t* slot_mapping, int64_t num_slots,
                                 int64_t num_tokens, int32_t num_heads, int32_t head_dim, int32_t rope_dim,
                                 int32_t kv_lora_rank, float eps, int32_t dtype, int32_t* status, void* stream) {
  using namespace b200;
  if (num_tokens < 0 || num_heads <= 0 || head_dim <= 0 || rope_dim <= 0 || kv_lora_rank <= 0 || rope_positions <= 0)
    return B200_ERR_ARG;
  if (dtype != B200_DTYPE_BF16) return B200_ERR_UNSUPPORTED;
  // 16-byte chunks everywhere, and a rotation partner that is a whole number of lanes away
  const int rpc = rope_dim / 8;
  if (head_dim % 8 || rope_dim % 16 || kv_lora_rank % 8 || (rpc & (rpc - 1)) || rpc > 32 || rope_width < rope_dim)
    return B200_ERR_UNSUPPORTED;
  if (num_tokens == 0) return B200_OK;
  if (!q_up || !kv_down || !kv_norm_weight || !rope_table || !positions || !q_out) return B200_ERR_ARG;
  if (latent_cache && !slot_mapping) return B200_ERR_ARG;
  const int64_t q_w = static_cast<int64_t>(num_heads) * (head_dim + rope_dim);
  if (q_up_stride < q_w || kv_down_stride < kv_lora_rank + rope_dim || q_up_stride % 8 || kv_down_stride % 8)
    return B200_ERR_ARG;
  if (!aligned16(q_up) || !aligned16(kv_down) || !aligned16(kv_norm_weight) || !aligned16(q_out) ||
      (rows_out && !aligned16(rows_out)) || (latent_cache && !aligned16(latent_cache)))
    return B200_ERR_ALIGN;
  if (num_tokens > 2147483647LL * kWarpRows) return B200_ERR_TOO_LARGE;
  MlaProArgs a{};
  a.qf = static_cast<const __nv_bfloat16*>(q_up);
  a.qf_stride = q_up_stride;
  a.kvp = static_cast<const __nv_bfloat16*>(kv_down);
  a.kvp_stride = kv_down_stride;
  a.kv_norm_w = kv_norm_weight;
  a.rope = rope_table;
  a.rope_width = rope_width;
  a.max_pos = rope_positions;
  a.positions = positions;
  a.q_out = static_cast<__nv_bfloat16*>(q_out);
  a.rows_out = static_cast<__nv_bfloat16*>(rows_out);
  a.cache = static_cast<__nv_bfloat16*>(latent_cache);
  a.slots = slot_mapping;
  a.num_slots = num_slots;
  a.H = num_heads;
  a.hd = head_dim;
  a.dr = rope_dim;
  a.r = kv_lora_rank;
  a.eps = eps;
  a.status = status;
  const int grid = static_cast<int>((num_tokens + kWarpRows - 1) / kWarpRows);
  mla_prologue_kernel<<<grid, kWarpRows * 32, 0, static_cast<cudaStream_t>(stream)>>>(a, num_tokens);
  return launch_result();
}
