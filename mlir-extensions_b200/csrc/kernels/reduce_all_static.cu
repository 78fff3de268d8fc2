// Full sum reduction that allocates nothing: imexReduceAllF32Static.
//
// The regular path (gpuLaunchKernel on an IMEX_OP_REDUCE_ALL kernel) keeps its
// block partials in a buffer the stream object obtains from cudaMalloc on
// first use.  Some callers cannot let a library do that: services that carve
// up all device memory at start-up and leave the CUDA allocator nothing,
// latency-critical loops in which cudaMalloc's device-wide synchronisation is
// not acceptable, and code that sits between a framework's own allocator and
// the GPU and must not go around it.  For them this entry point runs the same
// two kernels with the partials in a fixed array that is part of the library
// image: every GPU that loads the library carries these 256 KiB until exit.
//
// The array's name is only a handle on the host.  Its device address is looked
// up once per device with cudaGetSymbolAddress, during the first call made
// while that device is current; that first call should therefore happen before
// any stream capture is begun.  All calls share the one array and it keeps
// whatever the last call left in it: calls that overlap on the GPU (different
// streams, no ordering between them) race on it and must be serialised by the
// caller.  Nothing in it has to start at zero — stage 1 overwrites every
// partial that stage 2 reads — so no clearing launch is needed.
#include "kernels.h"

#include <cstdio>
#include <mutex>

namespace {

constexpr int64_t kMaxPartials = 65536;  // 256 KiB of f32
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_static_partials[kMaxPartials];

std::mutex g_setup_mutex;
float *g_partials_addr[kMaxDevices] = {};

// Device address of the array on the current device; looked up once per device.
cudaError_t partials_for_current_device(float **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_partials_addr[dev]) {
    float *p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_partials);
    if (e != cudaSuccess) return e;
    g_partials_addr[dev] = p;
  }
  *out = g_partials_addr[dev];
  return cudaSuccess;
}

} // namespace

extern "C" int imexReduceAllF32Static(const float *x, float *y, int64_t n, int accumulate,
                                      void *cudaStream) {
  if (n < 0 || (n > 0 && !x) || !y) {
    fprintf(stderr, "imexReduceAllF32Static: invalid argument (x=%p y=%p n=%lld)\n",
            static_cast<const void *>(x), static_cast<void *>(y), static_cast<long long>(n));
    return 1;
  }
  const int64_t partials = imex::reduce_all_partials(n);
  if (partials > kMaxPartials) {
    fprintf(stderr,
            "imexReduceAllF32Static: n=%lld needs %lld block partials, the built-in scratch array "
            "holds %lld (at most %lld elements per call); use the gpuLaunchKernel path for larger "
            "inputs\n",
            static_cast<long long>(n), static_cast<long long>(partials),
            static_cast<long long>(kMaxPartials),
            static_cast<long long>(kMaxPartials * imex::reduce_all_block_elems()));
    return 2;
  }
  float *scratch = nullptr;
  cudaError_t e = partials_for_current_device(&scratch);
  if (e != cudaSuccess) {
    fprintf(stderr, "imexReduceAllF32Static: cudaGetSymbolAddress failed: %s\n",
            cudaGetErrorString(e));
    return 3;
  }
  e = imex::launch_reduce_all_f32(x, y, n, accumulate != 0, scratch,
                                  static_cast<cudaStream_t>(cudaStream));
  if (e != cudaSuccess) {
    fprintf(stderr, "imexReduceAllF32Static: launch failed: %s\n", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
