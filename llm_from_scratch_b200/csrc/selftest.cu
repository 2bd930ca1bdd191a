// Diagnostic launch that drives the bounded-wait give-up path of the tcgen05 / TMA kernels on purpose.
//
// Every mbarrier wait in those kernels is bounded (umma::mbar_wait): a wait that runs out raises a CTA-wide
// abort flag, reports B200_ERR_TIMEOUT in the status word, every other wait of the CTA leaves when it sees
// the flag, and the CTA still frees its tensor memory before it exits.  In a healthy run no wait ever runs
// out, so this path would never execute under test.  The kernel below makes it execute without any fault
// or unbounded loop: one CTA allocates tensor memory, arms an mbarrier that expects two arrivals, arrives
// once, and lets two threads wait on it — one with a short poll limit (it times out and raises the flag),
// one with the kernels' default limit (it must leave through the flag long before that).  Then the tensor
// memory is freed and the CTA exits normally.
#include "umma.cuh"

namespace b200 {
namespace {

constexpr int kCols = 32;  // tensor-memory columns held across the failed wait

__global__ void __launch_bounds__(128) bounded_wait_selftest_kernel(int short_limit, int32_t* result,
                                                                   int32_t* status) {
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar = smem_u32(&s_bar);
  if (threadIdx.x == 0) {
    s_abort = 0;
    umma::mbar_init(bar, 2);  // two arrivals complete the phase; only one will ever come
    umma::mbar_init_fence();
  }
  __syncthreads();
  if (warp == 0) umma::tmem_alloc(smem_u32(&s_tmem), kCols);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = s_tmem;
  if (threadIdx.x == 0) umma::mbar_arrive(bar);

  if (warp == 1 && lane == 0) {
    // the waiter that gives up: the kernels' reaction to a wait that ran out
    int polls = 0;
    const bool ok = umma::mbar_wait(bar, 0, &s_abort, short_limit, &polls);
    if (!ok) {
      s_abort = 1;
      report(status, B200_ERR_TIMEOUT);
    }
    result[0] = ok ? 1 : 0;
    result[1] = polls;
  } else if (warp == 2 && lane == 0) {
    // a waiter of another role with the default limit: leaves when it sees the flag
    int polls = 0;
    const bool ok = umma::mbar_wait(bar, 0, &s_abort, 1 << 22, &polls);
    result[2] = ok ? 1 : 0;
    result[3] = polls;
  }
  __syncthreads();
  umma::fence_before_sync();
  if (warp == 0) umma::tmem_dealloc(tmem, kCols);
  if (threadIdx.x == 0) result[4] = static_cast<int32_t>(tmem >> 16) == 0 ? 1 : 0;  // lane field of the base is 0
}

}  // namespace
}  // namespace b200

extern "C" int b200_selftest_bounded_wait(int32_t poll_limit, int32_t* result, int32_t* status,
                                          void* stream) {
  using namespace b200;
  if (poll_limit < 1 || poll_limit > (1 << 16) || result == nullptr) return B200_ERR_ARG;
  bounded_wait_selftest_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(poll_limit, result, status);
  return launch_result();
}
