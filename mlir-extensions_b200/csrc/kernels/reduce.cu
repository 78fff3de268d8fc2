// Sum reductions (f32): y = init + sum x, reference generic `addf out, in`
// with an ascending reduction index.
//   rows    : (d0,d1)->(d0,d1) in, (d0,d1)->(d0) out — the softmax row-sum
//             step (benchmarks/softmax/softmax_gpu.mlir.in:32-37) and the
//             small XeGPU tests (test/Integration/Dialect/XeGPU/VC/block_reduce_dim_1_fp32.mlir:31-35)
//   leading : reduce the leading dim (benchmarks/reduce/reduce_gpu.mlir.in:8-18)
//   all     : full sum to a scalar (test/PlaidML/OpTest.Sum.mlir:16-25)
// The reference's GPU lowering runs a serial loop per output element
// (test/SPIRV/OpTest.Sum_FLOAT32.mlir:39).  Rows: one warp per row, 128-bit
// loads, 8 loads in flight per lane, shuffle tree; HBM traffic = the input once
// + the output.  Leading: one thread per output column, l ascending — same
// order as the loop nest, bit-identical, and coalesced across the warp.
#include "kernels.h"

namespace imex {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float4 ldg_stream(const float4 *p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

constexpr int ROWS_WARPS = 8;

__global__ void __launch_bounds__(ROWS_WARPS * 32)
reduce_rows_warp_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t rows,
                        int64_t cols, int accumulate, int vec_ok) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * ROWS_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * ROWS_WARPS;
  for (int64_t row = warp0; row < rows; row += nwarps) {
    const float *xr = x + row * cols;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (vec_ok) {
      const float4 *xv = reinterpret_cast<const float4 *>(xr);
      const int64_t nvec = cols >> 2;
      int64_t i = lane;
      for (; i + 32 * 7 < nvec; i += 32 * 8) {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = ldg_stream(xv + i + 32 * u);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          s0 += v[u].x; s1 += v[u].y; s2 += v[u].z; s3 += v[u].w;
        }
      }
      for (; i < nvec; i += 32) {
        float4 v = ldg_stream(xv + i);
        s0 += v.x; s1 += v.y; s2 += v.z; s3 += v.w;
      }
    } else {
      for (int64_t c = lane; c < cols; c += 32) s0 += xr[c];
    }
    float s = warp_sum((s0 + s1) + (s2 + s3));
    if (lane == 0) y[row] = accumulate ? y[row] + s : s;
  }
}

// Few long rows: one block per row.
__global__ void __launch_bounds__(256)
reduce_rows_block_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t rows,
                         int64_t cols, int accumulate) {
  __shared__ float red[8];
  const int tid = threadIdx.x;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float *xr = x + row * cols;
    float s = 0.f;
    for (int64_t c = tid; c < cols; c += 256) s += xr[c];
    s = warp_sum(s);
    if ((tid & 31) == 0) red[tid >> 5] = s;
    __syncthreads();
    if (tid == 0) {
      float t = red[0];
      for (int w = 1; w < 8; ++w) t += red[w];
      y[row] = accumulate ? y[row] + t : t;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256)
reduce_leading_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t lead,
                      int64_t inner, int accumulate) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < inner;
       i += stride) {
    float acc = accumulate ? y[i] : 0.0f;
    int64_t l = 0;
    for (; l + 8 <= lead; l += 8) {  // loads hoisted, adds stay in order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldg(x + (l + u) * inner + i);
#pragma unroll
      for (int u = 0; u < 8; ++u) acc = __fadd_rn(acc, v[u]);
    }
    for (; l < lead; ++l) acc = __fadd_rn(acc, __ldg(x + l * inner + i));
    y[i] = acc;
  }
}

constexpr int ALL_BLOCK = 256;
constexpr int64_t ALL_PER_BLOCK = 256 * 4 * 16;  // elements one block sums

__global__ void __launch_bounds__(ALL_BLOCK)
reduce_all_stage1_kernel(const float *__restrict__ x, float *__restrict__ partials, int64_t n) {
  __shared__ float red[ALL_BLOCK / 32];
  const int tid = threadIdx.x;
  const int64_t begin = static_cast<int64_t>(blockIdx.x) * ALL_PER_BLOCK;
  const int64_t end = begin + ALL_PER_BLOCK < n ? begin + ALL_PER_BLOCK : n;
  float s = 0.f;
  for (int64_t i = begin + tid; i < end; i += ALL_BLOCK) s += x[i];
  s = warp_sum(s);
  if ((tid & 31) == 0) red[tid >> 5] = s;
  __syncthreads();
  if (tid == 0) {
    float t = red[0];
    for (int w = 1; w < ALL_BLOCK / 32; ++w) t += red[w];
    partials[blockIdx.x] = t;
  }
}

__global__ void __launch_bounds__(ALL_BLOCK)
reduce_all_stage2_kernel(const float *__restrict__ partials, int64_t count, float *__restrict__ y,
                         int accumulate) {
  __shared__ float red[ALL_BLOCK / 32];
  const int tid = threadIdx.x;
  float s = 0.f;
  for (int64_t i = tid; i < count; i += ALL_BLOCK) s += partials[i];
  s = warp_sum(s);
  if ((tid & 31) == 0) red[tid >> 5] = s;
  __syncthreads();
  if (tid == 0) {
    float t = red[0];
    for (int w = 1; w < ALL_BLOCK / 32; ++w) t += red[w];
    *y = accumulate ? *y + t : t;
  }
}

} // namespace

cudaError_t launch_reduce_rows_f32(const float *x, float *y, int64_t rows, int64_t cols,
                                   bool accumulate, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  const int vec_ok = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  if (rows < 148 * 4 && cols >= 16384) {
    reduce_rows_block_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(x, y, rows, cols,
                                                                              accumulate ? 1 : 0);
    return cudaGetLastError();
  }
  int64_t blocks = (rows + ROWS_WARPS - 1) / ROWS_WARPS;
  const int64_t cap = 148 * 8 * 4;  // 8 resident blocks per SM, a few waves
  if (blocks > cap) blocks = cap;
  reduce_rows_warp_kernel<<<static_cast<unsigned>(blocks), ROWS_WARPS * 32, 0, stream>>>(
      x, y, rows, cols, accumulate ? 1 : 0, vec_ok);
  return cudaGetLastError();
}

cudaError_t launch_reduce_leading_f32(const float *x, float *y, int64_t lead, int64_t inner,
                                      bool accumulate, cudaStream_t stream) {
  if (inner <= 0) return cudaSuccess;
  int64_t blocks = (inner + 255) / 256;
  const int64_t cap = 148 * 8 * 8;
  if (blocks > cap) blocks = cap;
  reduce_leading_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(x, y, lead, inner,
                                                                           accumulate ? 1 : 0);
  return cudaGetLastError();
}

int64_t reduce_all_block_elems() { return ALL_PER_BLOCK; }

int64_t reduce_all_partials(int64_t n) {
  int64_t b = (n + ALL_PER_BLOCK - 1) / ALL_PER_BLOCK;
  return b < 1 ? 1 : b;
}

cudaError_t launch_reduce_all_f32(const float *x, float *y, int64_t n, bool accumulate,
                                  float *partials, cudaStream_t stream) {
  const int64_t blocks = reduce_all_partials(n);
  reduce_all_stage1_kernel<<<static_cast<unsigned>(blocks), ALL_BLOCK, 0, stream>>>(x, partials,
                                                                                     n > 0 ? n : 0);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  reduce_all_stage2_kernel<<<1, ALL_BLOCK, 0, stream>>>(partials, blocks, y, accumulate ? 1 : 0);
  return cudaGetLastError();
}

} // namespace imex
