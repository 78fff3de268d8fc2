// Standalone relu / silu (benchmarks/relu/relu_gpu.mlir.in,
// benchmarks/silu/silu_gpu.mlir.in) and the seeded input generators that
// stand in for the reference's unseeded std::mt19937 fill
// (lib/ExecutionEngine/ImexRunnerUtils.cpp:38-50).
#include "epilogue.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace imex {
namespace {

// Four 16-byte loads per thread are issued before the first value is used: with one load per
// iteration the silu chain (exp, reciprocal: two trips through the special-function unit)
// left each warp too long between its loads to keep HBM busy (4.9 TB/s against relu's 6.3).
template <int EPI>
__global__ void __launch_bounds__(256)
eltwise_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t n, int vec_ok) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec_ok) {
    const int64_t nvec = n >> 2;
    const float4 *xv = reinterpret_cast<const float4 *>(x);
    float4 *yv = reinterpret_cast<float4 *>(y);
    int64_t i = t0;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = xv[i + u * stride];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        v[u].x = apply_epilogue(v[u].x, EPI);
        v[u].y = apply_epilogue(v[u].y, EPI);
        v[u].z = apply_epilogue(v[u].z, EPI);
        v[u].w = apply_epilogue(v[u].w, EPI);
        yv[i + u * stride] = v[u];
      }
    }
    for (; i < nvec; i += stride) {
      float4 v = xv[i];
      v.x = apply_epilogue(v.x, EPI);
      v.y = apply_epilogue(v.y, EPI);
      v.z = apply_epilogue(v.z, EPI);
      v.w = apply_epilogue(v.w, EPI);
      yv[i] = v;
    }
    for (int64_t j = (nvec << 2) + t0; j < n; j += stride) y[j] = apply_epilogue(x[j], EPI);
  } else {
    for (int64_t i = t0; i < n; i += stride) y[i] = apply_epilogue(x[i], EPI);
  }
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float v) {
  return __float2half_rn(v);
}

template <typename T>
__global__ void __launch_bounds__(256)
fill_uniform_kernel(T *__restrict__ y, int64_t n, uint64_t seed, int64_t first, float lo,
                    float hi) {
  const float span = __fsub_rn(hi, lo);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    uint64_t h = splitmix64(static_cast<uint64_t>(first + i) + seed * 0x9E3779B97F4A7C15ULL);
    float u = __fmul_rn(static_cast<float>(static_cast<uint32_t>(h >> 40)), 1.0f / 16777216.0f);
    y[i] = from_f32<T>(__fadd_rn(lo, __fmul_rn(u, span)));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
fill_normal_kernel(T *__restrict__ y, int64_t n, uint64_t seed, int64_t first, float mean,
                   float stddev) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    uint64_t h = splitmix64(static_cast<uint64_t>(first + i) + seed * 0x9E3779B97F4A7C15ULL);
    float u1 = (static_cast<float>(static_cast<uint32_t>(h >> 40)) + 1.0f) * (1.0f / 16777216.0f);
    float u2 = static_cast<float>(static_cast<uint32_t>(h >> 16) & 0xFFFFFFu) * (1.0f / 16777216.0f);
    float r = sqrtf(-2.0f * logf(u1));
    float z = r * cospif(2.0f * u2);
    y[i] = from_f32<T>(mean + stddev * z);
  }
}

// arith.extf / arith.truncf as a standalone generic (test/PlaidML/CppEdsl.DotF16_AccF32.mlir:22-47):
// 16-bit -> f32 is exact, f32 -> 16-bit rounds to nearest even.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
convert_kernel(const TIn *__restrict__ x, TOut *__restrict__ y, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v;
    if constexpr (sizeof(TIn) == 4) v = x[i];
    else v = static_cast<float>(x[i]);
    y[i] = from_f32<TOut>(v);
  }
}

unsigned grid_for(int64_t n) {
  int64_t b = (n + 255) / 256;
  if (b > 148 * 32) b = 148 * 32;
  return static_cast<unsigned>(b < 1 ? 1 : b);
}

} // namespace

cudaError_t launch_eltwise_f32(const float *x, float *y, int64_t n, int epilogue,
                               cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  int vec_ok = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  const unsigned g = grid_for((n + 3) / 4);
  if (epilogue == kEpiRelu) eltwise_kernel<kEpiRelu><<<g, 256, 0, stream>>>(x, y, n, vec_ok);
  else if (epilogue == kEpiSilu) eltwise_kernel<kEpiSilu><<<g, 256, 0, stream>>>(x, y, n, vec_ok);
  else eltwise_kernel<kEpiNone><<<g, 256, 0, stream>>>(x, y, n, vec_ok);
  return cudaGetLastError();
}

cudaError_t launch_convert(const void *x, void *y, int64_t n, int in_dtype, int out_dtype,
                           cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  const unsigned g = grid_for(n);
#define IMEX_CONVERT(TI, TO) \
  convert_kernel<TI, TO><<<g, 256, 0, stream>>>(static_cast<const TI *>(x), static_cast<TO *>(y), n)
  if (in_dtype == kF32 && out_dtype == kF16) IMEX_CONVERT(float, __half);
  else if (in_dtype == kF32 && out_dtype == kBF16) IMEX_CONVERT(float, __nv_bfloat16);
  else if (in_dtype == kF16 && out_dtype == kF32) IMEX_CONVERT(__half, float);
  else if (in_dtype == kBF16 && out_dtype == kF32) IMEX_CONVERT(__nv_bfloat16, float);
  else return cudaErrorInvalidValue;
#undef IMEX_CONVERT
  return cudaGetLastError();
}

cudaError_t launch_fill_uniform(void *y, int64_t n, int dtype, uint64_t seed, int64_t first,
                                float lo, float hi, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (dtype == kF32)
    fill_uniform_kernel<float><<<grid_for(n), 256, 0, stream>>>(static_cast<float *>(y), n, seed,
                                                                first, lo, hi);
  else if (dtype == kBF16)
    fill_uniform_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, stream>>>(
        static_cast<__nv_bfloat16 *>(y), n, seed, first, lo, hi);
  else if (dtype == kF16)
    fill_uniform_kernel<__half><<<grid_for(n), 256, 0, stream>>>(static_cast<__half *>(y), n, seed,
                                                                 first, lo, hi);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t launch_fill_normal(void *y, int64_t n, int dtype, uint64_t seed, int64_t first,
                               float mean, float stddev, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (dtype == kF32)
    fill_normal_kernel<float><<<grid_for(n), 256, 0, stream>>>(static_cast<float *>(y), n, seed,
                                                               first, mean, stddev);
  else if (dtype == kBF16)
    fill_normal_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, stream>>>(
        static_cast<__nv_bfloat16 *>(y), n, seed, first, mean, stddev);
  else if (dtype == kF16)
    fill_normal_kernel<__half><<<grid_for(n), 256, 0, stream>>>(static_cast<__half *>(y), n, seed,
                                                                first, mean, stddev);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

} // namespace imex
