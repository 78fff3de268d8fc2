// Self-test of the bounded-wait path the tensor-core GEMMs rely on.
//
// The reference has no failure detection: a kernel that never finishes hangs
// the process (its runtime's error path is exception -> print -> abort,
// lib/ExecutionEngine/LEVELZERORUNTIME/LevelZeroRuntimeWrappers.cpp:41-53).
// Here every device-side wait gives up after a limit, records a status code
// in the stream's host-visible status word and lets the kernel return, and
// gpuWait turns that word into the reference's error convention.  This kernel
// exercises exactly that chain without touching anything else: one thread
// waits on an mbarrier that nothing ever arrives at, with a limit of about a
// millisecond, then reports kStatusSelfTestTimeout and exits normally.
#include "tcgen05_ptx.cuh"

namespace imex {
namespace {

__global__ void wait_selftest_kernel(unsigned *status, long long limit_cycles) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t b = tc::smem_u32(&bar);
  if (threadIdx.x == 0) {
    tc::mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!tc::mbar_wait(b, 0, limit_cycles)) tc::report(status, kStatusSelfTestTimeout);
  }
}

} // namespace

cudaError_t launch_wait_selftest(unsigned *status, cudaStream_t stream) {
  wait_selftest_kernel<<<1, 32, 0, stream>>>(status, 2000000LL);  // ~1 ms
  return cudaGetLastError();
}

} // namespace imex
