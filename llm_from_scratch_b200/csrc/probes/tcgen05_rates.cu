// Microbenchmarks behind the figures quoted for the tcgen05 kernels: throughput of a chain of
// tcgen05.mma (cta_group::1, M = 128, bf16, K = 16) for several N with operands in shared memory (SS) or A
// in tensor memory (TS), and the latency of tcgen05.ld / tcgen05.st with the tensor pipe idle.
// Not part of the library; build and run on a B200:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -Iinclude \
//        -o tcgen05_rates llm_from_scratch_b200/csrc/probes/tcgen05_rates.cu && ./tcgen05_rates
// Every wait is bounded (umma::mbar_wait); nothing here can spin forever.
#include <cstdio>
#include <cuda.h>
#include "../common.cuh"
#include "../umma.cuh"
using namespace b200;

template <int N, bool TS, int ACCS>
__global__ void __launch_bounds__(128, 1) rate_kernel(long long* out, int iters) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(smem);
  __shared__ uint64_t bar_mem;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&bar_mem);
  for (int i = threadIdx.x; i < (64 + 64) * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) {
    umma::mbar_init(bar, 1);
    abort_flag = 0;
    umma::mbar_init_fence();
  }
  if (threadIdx.x < 32) umma::tmem_alloc(smem_u32(&tmem_slot), 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = umma::instr_desc_bf16(128, N, false, false);
    const uint32_t abase = sb, bbase = sb + 64 * 1024;   // A: 128 rows x 64 cols slabs; B: N rows x 64 cols slabs
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint32_t acc = tmem + ((it * 4 + ks) % ACCS) * (N < 128 ? 128 : N > 128 ? 256 : 128) % 512;
        if (TS)
          umma::mma_ts(acc, tmem + 448 + ks * 8, umma::smem_desc(bbase + ks * 32, 0, 1024), idesc, 1);
        else
          umma::mma_ss(acc, umma::smem_desc(abase + ks * 32, 0, 1024), umma::smem_desc(bbase + ks * 32, 0, 1024), idesc, 1);
      }
    }
    umma::commit(bar);
    volatile int* ab = &abort_flag;
    const bool ok = umma::mbar_wait(bar, 0, ab);
    const long long t1 = clock64();
    if (blockIdx.x == 0) out[0] = ok ? (t1 - t0) : -1;
  }
  umma::fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) umma::tmem_dealloc(tmem, 512);
}

template <int N, bool TS, int ACCS>
void run(const char* name, long long* d_out) {
  const int iters = 2000;
  auto k = rate_kernel<N, TS, ACCS>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 130 * 1024);
  for (int grid : {1, 148}) {
    k<<<grid, 128, 130 * 1024>>>(d_out, iters);
    cudaError_t e = cudaDeviceSynchronize();
    long long h = 0;
    cudaMemcpy(&h, d_out, 8, cudaMemcpyDeviceToHost);
    printf("%-28s grid %3d: %s  %.1f clocks per MMA (math at peak: %.0f)\n", name, grid, cudaGetErrorString(e),
           double(h) / (iters * 4), 128.0 * N * 16 * 2 / 8192.0);
  }
}

__global__ void __launch_bounds__(128, 1) lat_kernel(long long* out, int iters) {
  __shared__ uint32_t tmem_slot;
  if (threadIdx.x < 32) umma::tmem_alloc(smem_u32(&tmem_slot), 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot + ((threadIdx.x >> 5) * 32 << 16);
  uint32_t r[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = i;
  umma::tmem_st32(tmem, r);
  umma::tmem_wait_st();
  __syncwarp();
  long long t0 = clock64();
  uint32_t acc = 0;
  for (int it = 0; it < iters; ++it) {
    umma::tmem_ld32(tmem + (acc & 32), r);       // address depends on the previous load: a dependent chain
    acc += r[0] & 32;
  }
  long long t1 = clock64();
  for (int it = 0; it < iters; ++it) {
    r[0] = acc + it;
    umma::tmem_st32(tmem, r);
    umma::tmem_wait_st();
  }
  long long t2 = clock64();
  // 16-column store as the softmax does it, then ld
  uint32_t q[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) q[i] = r[i];
  for (int it = 0; it < iters; ++it) {
    umma::tmem_st16(tmem, q);
    umma::tmem_wait_st();
    umma::tmem_ld32(tmem, r);
    q[0] = r[1];
  }
  long long t3 = clock64();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    out[0] = (t1 - t0) / iters;
    out[1] = (t2 - t1) / iters;
    out[2] = (t3 - t2) / iters;
    out[3] = acc + q[0];
  }
  umma::fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) umma::tmem_dealloc(tmem_slot, 512);
}

int main() {
  long long* d_out;
  cudaMalloc(&d_out, 64);
  run<64, false, 1>("N=64 SS, one accumulator", d_out);
  run<64, false, 2>("N=64 SS, two accumulators", d_out);
  run<128, false, 1>("N=128 SS, one accumulator", d_out);
  run<128, false, 2>("N=128 SS, two accumulators", d_out);
  run<256, false, 1>("N=256 SS, one accumulator", d_out);
  run<128, true, 1>("N=128 TS, one accumulator", d_out);
  run<128, true, 2>("N=128 TS, two accumulators", d_out);
  run<16, false, 1>("N=16 SS, one accumulator", d_out);
  for (int grid : {1, 148}) {
    lat_kernel<<<grid, 128>>>(d_out, 2000);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[4];
    cudaMemcpy(h, d_out, 32, cudaMemcpyDeviceToHost);
    printf("grid %3d %s: ld.x32+wait %lld clk, st.x32+wait::st %lld clk, st.x16+wait+ld.x32+wait %lld clk\n", grid,
           cudaGetErrorString(e), h[0], h[1], h[2]);
  }
  return 0;
}
