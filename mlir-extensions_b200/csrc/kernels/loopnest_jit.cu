// Loop-nest kernels (IMEX_OP_LOOPNEST): CUDA C++ text from the kernel blob, compiled for
// sm_100a at first launch and cached by its text.
//
// The text is what the front end writes for a linalg.generic that is none of the
// recognised hot-path ops (csrc/frontend/loopnest.h): one thread per point of the parallel
// iteration space, reduction loops serial per thread — the reference pipeline's own
// lowering of every linalg op (benchmarks/pipelines/linalg-to-gpu.pp:3-47).  This file
// supplies the prelude the text is written against (element-type helpers, the thread
// index) and launches 256-thread blocks over `threads` points.  There is no interpreter
// behind it: without NVRTC a loop-nest kernel cannot run and the launch fails.
#include "jit_common.h"
#include "kernels.h"

#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace imex {
namespace {

const char *kLoopNestPrelude = R"SRC(
typedef unsigned short u16;
typedef unsigned char u8;
typedef long long i64;
typedef unsigned long long u64;
#define IMX_THREAD_INDEX (blockIdx.x * (i64)blockDim.x + threadIdx.x)
__device__ __forceinline__ float imx_f16_to_f32(u16 h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
__device__ __forceinline__ u16 imx_f32_to_f16(float f) { u16 h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
__device__ __forceinline__ float imx_bf16_to_f32(u16 h) { return __uint_as_float(((unsigned)h) << 16); }
__device__ __forceinline__ u16 imx_f32_to_bf16(float f) { u16 h; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
__device__ __forceinline__ float imx_rf16(float f) { return imx_f16_to_f32(imx_f32_to_f16(f)); }
__device__ __forceinline__ float imx_rbf16(float f) { return imx_bf16_to_f32(imx_f32_to_bf16(f)); }
__device__ __forceinline__ float imx_nan32() { return __uint_as_float(0x7fc00000u); }
__device__ __forceinline__ float imx_inf32() { return __uint_as_float(0x7f800000u); }
__device__ __forceinline__ double imx_nan64() { return __longlong_as_double(0x7ff8000000000000LL); }
__device__ __forceinline__ double imx_inf64() { return __longlong_as_double(0x7ff0000000000000LL); }
__device__ __forceinline__ int imx_f32_bits(float f) { return __float_as_int(f); }
__device__ __forceinline__ float imx_bits_f32(int i) { return __int_as_float(i); }
// arith.maximumf / minimumf: NaN if either is NaN; maxnumf / minnumf: the number if one is NaN
__device__ __forceinline__ float imx_maximum(float a, float b) { return a != a ? a : (b != b ? b : fmaxf(a, b)); }
__device__ __forceinline__ float imx_minimum(float a, float b) { return a != a ? a : (b != b ? b : fminf(a, b)); }
__device__ __forceinline__ double imx_maximum(double a, double b) { return a != a ? a : (b != b ? b : fmax(a, b)); }
__device__ __forceinline__ double imx_minimum(double a, double b) { return a != a ? a : (b != b ? b : fmin(a, b)); }
// math.exp on an f16 / bf16 value (the result is rounded to the type by the caller): 2^(x log2 e)
// on the hardware unit with the rounding error of the product fed back.  Rounded to the type
// these equal libm's expf rounded to the type for every one of the 65536 arguments of the type
// (the f16 form leaves out the low part of log2 e; both tested over all arguments on the device).
__device__ __forceinline__ float imx_exp_16(float x, float l2e_lo) {
  const float y = __fmul_rn(x, 1.44269502162933349609375f);
  float r = __fmaf_rn(x, 1.44269502162933349609375f, -y);
  r = __fmaf_rn(x, l2e_lo, r);
  float e;
  asm("ex2.approx.f32 %0, %1;" : "=f"(e) : "f"(y));
  const float c = __fmaf_rn(e, __fmul_rn(r, 0.693147182464599609375f), e);
  return c == c ? c : e;   // infinite x, or 2^y = inf with a negative residual: no correction
}
__device__ __forceinline__ float imx_exp_f16(float x) { return imx_exp_16(x, 0.0f); }
__device__ __forceinline__ float imx_exp_bf16(float x) { return imx_exp_16(x, 1.92596299112661746e-8f); }
__device__ __forceinline__ float imx_maxnum(float a, float b) { return fmaxf(a, b); }
__device__ __forceinline__ float imx_minnum(float a, float b) { return fminf(a, b); }
__device__ __forceinline__ double imx_maxnum(double a, double b) { return fmax(a, b); }
__device__ __forceinline__ double imx_minnum(double a, double b) { return fmin(a, b); }
)SRC";

std::mutex g_mu;
std::map<std::string, jit::Compiled> g_cache;  // keyed by device + kernel text

} // namespace

const char *loopnest_prelude() { return kLoopNestPrelude; }

// cudaErrorNotSupported: the text could not be compiled (no NVRTC, or a compile error: the
// compiler's output goes to *log when given).
cudaError_t launch_loopnest(const char *source, size_t source_bytes, void *const *ptrs, int n_ptrs,
                            int64_t threads, cudaStream_t stream, std::string *log) {
  if (threads <= 0) return cudaSuccess;
  if (!source || !source_bytes || n_ptrs < 1 || n_ptrs > 32) return cudaErrorInvalidValue;
  int device = 0;
  cudaGetDevice(&device);
  std::string key = std::to_string(device) + "|";
  key.append(source, source_bytes);
  jit::Compiled c;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_cache.find(key);
    if (it == g_cache.end()) {
      cudaFree(nullptr);  // the primary context exists before the module is loaded into it
      std::string src(kLoopNestPrelude);
      src.append(source, source_bytes);
      it = g_cache.emplace(key, jit::compile_kernel(src, "imex_loopnest")).first;
    }
    c = it->second;
  }
  if (c.failed || !c.fn) {
    if (log) *log = c.log;
    return cudaErrorNotSupported;
  }
  std::vector<void *> slots(ptrs, ptrs + n_ptrs);
  std::vector<void *> args;
  for (auto &s : slots) args.push_back(&s);
  const int64_t blocks = (threads + 255) / 256;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  const CUresult rc = jit::driver().launchKernel(c.fn, static_cast<unsigned>(blocks), 1, 1, 256, 1, 1, 0, stream,
                                                 args.data(), nullptr);
  return rc == CUDA_SUCCESS ? cudaSuccess : cudaErrorLaunchFailure;
}

} // namespace imex
