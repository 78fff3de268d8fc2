/* GPU runtime-wrapper C ABI, served by CUDA on B200 (libimex_cuda_runtime.so).
 *
 * These are the symbols the host code emitted by the reference's
 * convert-gpux-to-llvm pass calls (lib/Conversion/GPUXToLLVM/GPUXToLLVMPass.cpp:120-209)
 * and that its Level Zero / SYCL wrapper libraries export
 * (lib/ExecutionEngine/LEVELZERORUNTIME/LevelZeroRuntimeWrappers.cpp:606-741,
 *  lib/ExecutionEngine/SYCLRUNTIME/SyclRuntimeWrappers.cpp:417-505).
 * Names, argument order and argument meaning are the reference's; a host
 * program linked against either reference library links against this one.
 *
 * Error convention (LevelZeroRuntimeWrappers.cpp:41-53): no status codes.
 * Any failure prints "An exception was thrown: <what>" to stdout, flushes and
 * calls abort().
 */
#ifndef IMEX_CUDA_RUNTIME_H
#define IMEX_CUDA_RUNTIME_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* One kernel argument: `data` points at a slot holding the value (a device
 * pointer for memrefs — aligned base pointer only — or a scalar), `size` is
 * its size in bytes.  Arrays are terminated by {NULL, 0}.
 * (LevelZeroRuntimeWrappers.cpp:80-89; built at GPUXToLLVMPass.cpp:540-623) */
typedef struct ImexParamDesc {
  void *data;
  size_t size;
} ImexParamDesc;

/* One dependency: an event returned by an earlier gpuLaunchKernel.  Arrays
 * are terminated by {NULL}.  (LevelZeroRuntimeWrappers.cpp:91-97) */
typedef struct ImexEventDesc {
  void *event;
} ImexEventDesc;

/* LevelZeroRuntimeWrappers.cpp:606-622.  Both arguments are NULL in all
 * emitted code (GPUXToLLVMPass.cpp:753-755) and select the current CUDA
 * device and a new stream.  Non-NULL values are backend handles, here:
 * `device` -> const int32_t* CUDA device ordinal; `context` -> an existing
 * cudaStream_t to adopt (not destroyed by gpuStreamDestroy). */
void *gpuCreateStream(void *device, void *context);
/* LevelZeroRuntimeWrappers.cpp:624-626 */
void gpuStreamDestroy(void *stream);
/* LevelZeroRuntimeWrappers.cpp:628-632.  isShared: host-visible memory that
 * host code reads and writes directly (gpu.alloc host_shared,
 * lib/Transforms/InsertGPUAllocs.cpp:376-412) -> CUDA managed memory,
 * prefetched to the device at launch.  alignment is always 64 in emitted
 * code (GPUXToLLVMPass.cpp:304); cudaMalloc gives 256. */
void *gpuMemAlloc(void *stream, size_t size, size_t alignment, bool isShared);
/* LevelZeroRuntimeWrappers.cpp:634-637 */
void gpuMemFree(void *stream, void *ptr);
/* LevelZeroRuntimeWrappers.cpp:639-642.  Blocking, like both reference
 * back-ends; direction is inferred from the pointers. */
void gpuMemCopy(void *stream, void *dst, void *src, size_t size);
void gpuMemcpy(void *stream, void *dst, void *src, size_t size); /* alias */
/* LevelZeroRuntimeWrappers.cpp:644-647, 396-432.  `data` is a kernel
 * descriptor blob (imex_b200_blob.h); the parsed module is cached by blob
 * address and lives until process exit. */
void *gpuModuleLoad(void *stream, const void *data, size_t dataSize);
/* LevelZeroRuntimeWrappers.cpp:649-652.  The handle belongs to the module:
 * asking for the same name again returns the same handle. */
void *gpuKernelGet(void *stream, void *module, const char *name);
/* LevelZeroRuntimeWrappers.cpp:654-664, 507-603.  grid/block sizes describe
 * the reference's one-work-item-per-element launch and are NOT used: each
 * recognised op launches its own sm_100a geometry.  sharedMemBytes != 0
 * means the last param is the local-memory placeholder and is dropped
 * (LevelZeroRuntimeWrappers.cpp:462-475).  8-byte params whose value is not
 * device-accessible memory (index scalars of loop bounds) are not operands
 * and are skipped wherever they stand.  Returns an event that later
 * launches may list in depEvents; events come from a ring of 256 per stream
 * (the reference's fixed pool, LevelZeroRuntimeWrappers.cpp:155-168), so a
 * handle is valid for the next 255 launches on that stream.  With IMEX_ENABLE_PROFILING set the launch
 * is repeated and timed first (IMEX_PROFILING_RUNS, IMEX_PROFILING_WARMUPS,
 * IMEX_ENABLE_CACHE_FLUSHING; LevelZeroRuntimeWrappers.cpp:521-597). */
void *gpuLaunchKernel(void *stream, void *kernel, size_t gridX, size_t gridY,
                      size_t gridZ, size_t blockX, size_t blockY, size_t blockZ,
                      size_t sharedMemBytes, void *params, void *depEvents);
/* LevelZeroRuntimeWrappers.cpp:666-671 (no-op there: synchronous queue;
 * SyclRuntimeWrappers.cpp:498-505 waits).  Here: cudaStreamSynchronize, then
 * the device status word is checked. */
void gpuWait(void *stream);
/* declared by the lowering (GPUXToLLVMPass.cpp:129-134) */
void gpuModuleUnload(void *module);

/* Upstream-style wrappers the Level Zero library also exports for
 * gpu-to-llvm (LevelZeroRuntimeWrappers.cpp:673-741). */
void *mgpuStreamCreate(void);
void mgpuStreamSynchronize(void *stream);
void mgpuStreamDestroy(void *stream);
void *mgpuMemAlloc(size_t size, void *stream, bool isShared);
void mgpuMemFree(void *stream, void *ptr);
void *mgpuModuleLoad(const void *data, size_t dataSize);
void *mgpuModuleGetFunction(void *module, const char *name);
void mgpuModuleUnload(void *module);
void mgpuLaunchKernel(void *kernel, size_t gridX, size_t gridY, size_t gridZ,
                      size_t blockX, size_t blockY, size_t blockZ,
                      size_t sharedMemBytes, void *stream, void **params,
                      void **extra, size_t paramsCount);

/* ---- additions of this library (no reference counterpart of the same name) */

/* The cudaStream_t behind a stream handle, for callers that record their own
 * CUDA events around launches. */
void *imexStreamNative(void *stream);
/* Milliseconds between two events returned by gpuLaunchKernel's profiling
 * pair: imexEventRecord returns a new timing event recorded on the stream. */
void *imexEventRecord(void *stream);
float imexEventElapsedMs(void *startEvent, void *stopEvent);
/* Device address of the stream's status word (0 = fine): kernels with bounded waits store a
 * code there when a wait runs out, gpuWait reads it. */
void *imexStreamStatusWord(void *stream);
/* Adds n to the launch counter (for kernels launched outside gpuLaunchKernel). */
void imexNoteLaunches(uint64_t n);

/* ---- peer memory between the processes of one node (one process per GPU).  No reference
 * counterpart: the reference leaves data exchange between ranks to its distributed runtime
 * (the `_idtr_*` calls behind lib/Dialect/DistRuntime).  Used by the row-sharded GEMM to
 * replicate B with the copy engines over NVLink instead of an SM-based collective.
 *
 * imexIpcExport: writes the 64-byte CUDA IPC handle of a gpuMemAlloc allocation (devPtr must
 *   be the pointer gpuMemAlloc returned) to handleOut.  imexIpcOpen: maps an allocation
 *   another process exported and returns its address here; imexIpcClose unmaps it.
 * imexMemCopyAsync: cudaMemcpyAsync on the stream, no wait (gpuMemCopy blocks); with an
 *   IPC-mapped source this is a DMA over NVLink that occupies no SM.
 * imexPeerBarrier: stream-ordered barrier over `world` ranks.  peerFlags[r] is rank r's flag
 *   array (`world` zero-initialised uint32 words, the local one for r == rank, IPC-mapped
 *   otherwise); every rank passes the same, strictly growing `epoch`.  A one-block kernel
 *   stores the epoch into this rank's slot of every peer's array and polls the local array;
 *   the wait is bounded (~2 s; IMEX_PEER_WAIT_CYCLES) and its expiry is reported by gpuWait. */
int imexIpcExport(void *devPtr, void *handleOut);
void *imexIpcOpen(const void *handle);
void imexIpcClose(void *mapped);
void imexMemCopyAsync(void *stream, void *dst, const void *src, size_t bytes);
void imexPeerBarrier(void *stream, void **peerFlags, int world, int rank, uint32_t epoch);

/* Kernels of this library launched since load (all streams). */
uint64_t imexLaunchCount(void);
/* Name of the device kernel family the last gpuLaunchKernel on this stream
 * dispatched to ("gemm_tcgen05", "gemm_f32_simt", ...). */
const char *imexLastKernelName(void *stream);
/* Block partition of `extent` over `numShards` (the reference's sharding rule,
 * lib/Dialect/NDArray/Extensions/MeshShardingExtensions.cpp:74-100: the LAST
 * extent%numShards shards get one extra element).  Both return -1 for
 * numShards <= 0, a shard outside [0, numShards) or a negative extent. */
int64_t imexShardSize(int64_t shard, int64_t numShards, int64_t extent);
int64_t imexShardOffset(int64_t shard, int64_t numShards, int64_t extent);
/* Timing statistics of the profiling loop
 * (lib/ExecutionEngine/ExecutionEngineUtils/ExecutionEngineUtils.cpp:18-150).
 * which: 0 avg, 1 min, 2 max, 3 median, 4 stddev, 5 variance, 6 P95, 7 P5,
 * 8 middle-third average. */
float imexStat(int which, const float *values, size_t n);

/* Failure-path self-test: enqueues a one-thread kernel whose bounded wait (about
 * a millisecond, on a barrier nothing signals) runs out; the kernel records a
 * status code and returns normally, and the next gpuWait on the stream reports
 * "device kernel reported status 99" through the error convention.  No fault,
 * trap or hang is involved; the context stays usable. */
void imexSelfTestWaitTimeout(void *stream);

/* Full sum of n f32 values without any allocation — no counterpart in the
 * reference (its runtime always allocates through the driver).
 *   *y = (accumulate ? *y : 0) + sum x[0..n)       x, y: device pointers
 * Same kernels and result as an IMEX_OP_REDUCE_ALL launch, but the block
 * partials live in a 256 KiB array built into the library instead of a
 * cudaMalloc'ed buffer, for callers that must not let a library allocate:
 * hosts that hand out all device memory themselves, loops that cannot afford
 * cudaMalloc's device-wide synchronisation.  Limit: 65536 partials, i.e.
 * n <= 65536 * 16384 = 1,073,741,824 elements; larger n is refused.
 * cudaStream: a cudaStream_t (NULL = default stream); the launch is
 * asynchronous on it.  The first call made with a given device current looks
 * up the array's device address and should come before any stream capture.
 * The array is shared by all calls and keeps the last call's contents: calls
 * that may overlap on the GPU must be ordered by the caller.
 * Returns 0, or: 1 invalid argument, 2 n beyond the limit, 3 address look-up
 * failed, 4 launch failed (a message goes to stderr; nothing is aborted). */
int imexReduceAllF32Static(const float *x, float *y, int64_t n, int accumulate, void *cudaStream);

#ifdef __cplusplus
}
#endif
#endif
