// Peer memory for the row-sharded ops: one process per GPU, buffers shared over CUDA IPC,
// copies driven by the copy engines over NVLink, and a small stream-ordered barrier.
//
// The reference replicates data between the ranks of a sharded array through its
// distributed runtime (the `_idtr_*` calls behind lib/Dialect/DistRuntime, MPI underneath).
// Here the one exchange of the row-sharded GEMM — every rank needs all of B — is done
// without a single SM: the source rank's B is cut into one slice per other rank, each rank
// pulls its own slice from the source with cudaMemcpyAsync on an IPC mapping (a DMA over
// NVLink), the ranks meet in imexPeerBarrier, and each rank pulls the remaining slices from
// the ranks that hold them.  The data always lands in the puller's own HBM before any GEMM
// reads it (no kernel and no TMA load ever touches a peer's memory on this path; only the
// barrier kernel stores and polls 4-byte flags there).  An NCCL broadcast of the same bytes
// runs 32 CTAs that the GEMM beside it has to leave free; this needs none.
//
// The barrier kernel polls a flag another GPU writes.  Every rank runs it on its own GPU
// (never two ranks on one GPU), and the wait is bounded: when it runs out the kernel
// records kStatusPeerWaitTimeout in the stream's status word and returns, and gpuWait
// reports it through the library's error convention.
#include "../../../include/imex_cuda_runtime.h"
#include "../kernels/kernels.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

namespace {

template <typename F> auto catchAll(F &&func) {
  try {
    return func();
  } catch (const std::exception &e) {
    fprintf(stdout, "An exception was thrown: %s\n", e.what());
    fflush(stdout);
    abort();
  }
}

void check(cudaError_t e, const char *what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(e));
}

constexpr int kMaxRanks = 16;
struct PeerFlags {
  unsigned *flags[kMaxRanks];  // flags[r]: rank r's array of `world` words (r == rank: the local one)
};

// Each of the first `world` threads: tell peer t that this rank has arrived (slot [rank] of
// t's array), then wait until peer t has arrived here (slot [t] of the local array).  Epochs
// only grow, so nothing is ever reset; comparisons are wrap-safe.
__global__ void peer_barrier_kernel(PeerFlags p, int world, int rank, unsigned epoch, unsigned *status,
                                    long long limit_cycles) {
  const int t = threadIdx.x;
  if (t >= world || t == rank) return;
  __threadfence_system();  // everything this stream did before the barrier is visible first
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[t] + rank), "r"(epoch) : "memory");
  const long long t0 = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.flags[rank] + t) : "memory");
    if (static_cast<int>(v - epoch) >= 0) break;
    if (clock64() - t0 > limit_cycles) {
      atomicCAS(status, 0u, static_cast<unsigned>(imex::kStatusPeerWaitTimeout));
      break;
    }
    __nanosleep(200);
  }
}

std::mutex g_mu;
std::map<void *, void *> g_opened;  // mapped pointer handed out -> base returned by cudaIpcOpenMemHandle

} // namespace

extern "C" {

int imexIpcExport(void *devPtr, void *handleOut) {
  return catchAll([&]() {
    if (!devPtr || !handleOut) throw std::runtime_error("imexIpcExport: null argument");
    cudaIpcMemHandle_t h;
    check(cudaIpcGetMemHandle(&h, devPtr), "cudaIpcGetMemHandle (the pointer must be the start of a gpuMemAlloc allocation)");
    static_assert(sizeof h == 64, "IPC handle size");
    memcpy(handleOut, &h, sizeof h);
    return 0;
  });
}

void *imexIpcOpen(const void *handle) {
  return catchAll([&]() -> void * {
    if (!handle) throw std::runtime_error("imexIpcOpen: null handle");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void *p = nullptr;
    check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    std::lock_guard<std::mutex> lock(g_mu);
    g_opened[p] = p;
    return p;
  });
}

void imexIpcClose(void *mapped) {
  catchAll([&]() {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_opened.find(mapped);
    if (it == g_opened.end()) return;
    cudaIpcCloseMemHandle(it->second);
    g_opened.erase(it);
  });
}

void imexMemCopyAsync(void *stream, void *dst, const void *src, size_t bytes) {
  catchAll([&]() {
    if (!stream) throw std::runtime_error("imexMemCopyAsync: null stream");
    if (!bytes) return;
    check(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(imexStreamNative(stream))),
          "cudaMemcpyAsync");
  });
}

void imexPeerBarrier(void *stream, void **peerFlags, int world, int rank, uint32_t epoch) {
  catchAll([&]() {
    if (!stream || !peerFlags) throw std::runtime_error("imexPeerBarrier: null argument");
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
      throw std::runtime_error("imexPeerBarrier: 1..16 ranks");
    if (world == 1) return;
    PeerFlags p{};
    for (int r = 0; r < world; ++r) {
      if (!peerFlags[r]) throw std::runtime_error("imexPeerBarrier: a peer's flag array is not mapped");
      p.flags[r] = static_cast<unsigned *>(peerFlags[r]);
    }
    long long limit = 4000000000LL;  // ~2 s of SM clocks
    if (const char *e = getenv("IMEX_PEER_WAIT_CYCLES")) {
      const long long v = atoll(e);
      if (v > 0) limit = v;
    }
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(imexStreamNative(stream))>>>(
        p, world, rank, epoch, static_cast<unsigned *>(imexStreamStatusWord(stream)), limit);
    check(cudaGetLastError(), "launch of the peer barrier");
  });
}

} // extern "C"
