// One-pass row softmax over the last dim (f32).
//
// The reference lowers softmax to six launches with four full-size
// temporaries (fill, row max, x-max, exp, fill, row sum, divide:
// benchmarks/softmax/softmax_gpu.mlir.in:8-42; one work-item per row or per
// element, test/SPIRV/OpTest.Softmax_FLOAT32.mlir:64-86).  Here a row is read
// from HBM once with 128-bit loads, kept in registers, and written once:
// algorithmic traffic = 2 * rows * cols * 4 bytes.
//
// Arithmetic per element is the reference's: t = x - max (exact max),
// e = exp(t) (see exp_neg: within ~3e-7 of libm's expf), y = e / sum correctly rounded (see div_by).  Only the order of the adds in
// `sum` differs from the sequential loop (per-lane partial sums + shuffle
// tree), which is where the <= 1e-5 relative tolerance goes.
#include "kernels.h"
#include "epilogue.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cfloat>
#include <cstdlib>

namespace imex {
namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// fmaxf drops NaNs where arith.maximumf keeps them; a NaN element still turns
// the whole row into NaN through exp -> sum -> divide, as in the reference.

__device__ __forceinline__ float4 ldg_stream4(const float4 *p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
// e / s by one correctly rounded reciprocal per row (rc = rn(1 / s)) and one residual step per
// element (q = e * rc; q += (e - q * s) * rc): the correctly rounded quotient for every normal
// result (Markstein), at 3 instructions per element instead of the ~10 of a full IEEE
// division sequence.
__device__ __forceinline__ float div_by(float e, float s, float rc) {
  const float q = __fmul_rn(e, rc);
  return __fmaf_rn(__fmaf_rn(-q, s, e), rc, q);
}

// One warp per row, the whole row in registers: cols == 4 * 32 * V exactly or
// ragged (guarded), cols <= 128 * V.
template <int V, bool FULL>
__global__ void __launch_bounds__(256)
softmax_warp_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t rows, int cols,
                    float max_init) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float4 *xr = reinterpret_cast<const float4 *>(x + row * cols);
  float4 *yr = reinterpret_cast<float4 *>(y + row * cols);
  const int nvec = cols >> 2;

  float4 v[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int idx = lane + 32 * i;
    v[i] = (FULL || idx < nvec) ? __ldg(xr + idx) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
  }
  float m = max_init;
#pragma unroll
  for (int i = 0; i < V; ++i) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
  m = warp_max(m);

  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    // a lane past the end of the row holds -inf: exp gives 0, which adds nothing
    v[i].x = exp_neg(v[i].x - m);
    v[i].y = exp_neg(v[i].y - m);
    v[i].z = exp_neg(v[i].z - m);
    v[i].w = exp_neg(v[i].w - m);
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  s = warp_sum(s);
  // division by one correctly rounded reciprocal and a residual step per element (div_by);
  // a sum that is not a finite normal number >= 1 (NaN row, overflow) takes the full division
  if (s >= 1.0f && s < 3.0e38f) {
    const float rc = __frcp_rn(s);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int idx = lane + 32 * i;
      if (FULL || idx < nvec)
        yr[idx] = make_float4(div_by(v[i].x, s, rc), div_by(v[i].y, s, rc), div_by(v[i].z, s, rc),
                              div_by(v[i].w, s, rc));
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int idx = lane + 32 * i;
      if (FULL || idx < nvec)
        yr[idx] = make_float4(__fdiv_rn(v[i].x, s), __fdiv_rn(v[i].y, s), __fdiv_rn(v[i].z, s),
                              __fdiv_rn(v[i].w, s));
    }
  }
}

// The same row-in-registers scheme for problems of only a few rows per SM (config 2 of the
// benchmark set: 4096 x 1024, i.e. 27.7 rows per SM).  With CTAs of eight rows the rows
// land unevenly (four CTAs on some SMs, three on others) and the last CTA to be scheduled
// sets the time.  Here the grid is one CTA per SM and each CTA has as many warps as its
// share of the rows (up to MAXW), so every SM issues all of its loads in the first
// microsecond and owns the same number of rows to within one; with more rows than
// SMs x MAXW a warp walks several rows.  Row r goes to CTA r % gridDim.x.
// FULL: cols == 4 * 32 * V exactly, so no lane is ever past the end of its row and the loop
// bodies carry no predicates (the benchmark's 1024 columns with V = 8).
template <int V, int MAXW, bool FULL>
__global__ void __launch_bounds__(32 * MAXW)
softmax_warp_balanced_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t rows, int cols,
                             float max_init) {
  // Launched with programmatic stream serialisation: this grid may be set up on the SMs while
  // the launch before it in the stream is still running.  Nothing is read or written before
  // the wait, which returns once that launch has completed and its writes are visible; the
  // launch after this one is allowed to be set up from here on.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int nvec = cols >> 2;
  for (int64_t row = blockIdx.x + static_cast<int64_t>(gridDim.x) * warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * nwarps) {
    const float4 *xr = reinterpret_cast<const float4 *>(x + row * cols);
    float4 *yr = reinterpret_cast<float4 *>(y + row * cols);
    float4 v[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int idx = lane + 32 * i;
      v[i] = (FULL || idx < nvec) ? ldg_stream4(xr + idx) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
    float m = max_init;
#pragma unroll
    for (int i = 0; i < V; ++i) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    m = warp_max(m);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      // a lane past the end of the row holds -inf: exp gives 0, which adds nothing
      v[i].x = exp_neg(v[i].x - m);
      v[i].y = exp_neg(v[i].y - m);
      v[i].z = exp_neg(v[i].z - m);
      v[i].w = exp_neg(v[i].w - m);
      s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    s = warp_sum(s);
    // a sum that is not a finite normal number >= 1 (NaN row, overflow) takes the full division
    if (s >= 1.0f && s < 3.0e38f) {
      const float rc = __frcp_rn(s);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const int idx = lane + 32 * i;
        if (FULL || idx < nvec)
          yr[idx] = make_float4(div_by(v[i].x, s, rc), div_by(v[i].y, s, rc), div_by(v[i].z, s, rc),
                                div_by(v[i].w, s, rc));
      }
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const int idx = lane + 32 * i;
        if (FULL || idx < nvec)
          yr[idx] = make_float4(__fdiv_rn(v[i].x, s), __fdiv_rn(v[i].y, s), __fdiv_rn(v[i].z, s),
                                __fdiv_rn(v[i].w, s));
      }
    }
  }
}

// Any cols: one block per row, three sweeps over the row (the 2nd and 3rd hit
// L1/L2).  Used for ragged or very long rows.
__global__ void __launch_bounds__(256)
softmax_block_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t rows,
                     int64_t cols, float max_init) {
  __shared__ float red[8];
  __shared__ float bcast;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float *xr = x + row * cols;
    float *yr = y + row * cols;
    float m = max_init;
    for (int64_t c = tid; c < cols; c += 256) m = fmaxf(m, xr[c]);
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (tid == 0) {
      float t = red[0];
      for (int w = 1; w < 8; ++w) t = fmaxf(t, red[w]);
      bcast = t;
    }
    __syncthreads();
    m = bcast;
    float s = 0.0f;
    for (int64_t c = tid; c < cols; c += 256) s += exp_neg(xr[c] - m);
    s = warp_sum(s);
    __syncthreads();
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (tid == 0) {
      float t = red[0];
      for (int w = 1; w < 8; ++w) t += red[w];
      bcast = t;
    }
    __syncthreads();
    s = bcast;
    for (int64_t c = tid; c < cols; c += 256) yr[c] = __fdiv_rn(exp_neg(xr[c] - m), s);
    __syncthreads();
  }
}

// Rows of at most 64 elements (the reference's golden tests: 10x20): one thread
// per row walking the row in order, so the row sum is the very sequence of
// f32 additions the loop nest performs; exp is evaluated in f64 and rounded
// once, which agrees with glibc's correctly-rounded-in-practice expf.  The
// printed six digits of test/PlaidML/OpTest.Softmax.mlir:98-109 depend on it.
__global__ void __launch_bounds__(128)
softmax_tiny_rows_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t rows, int cols,
                         float max_init) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const float *xr = x + row * cols;
  float *yr = y + row * cols;
  float e[64];
  float m = max_init;
  for (int c = 0; c < cols; ++c) m = fmaxf(m, xr[c]);
  float s = 0.0f;
#pragma unroll 1
  for (int c = 0; c < cols; ++c) {
    e[c] = static_cast<float>(exp(static_cast<double>(__fsub_rn(xr[c], m))));
    s = __fadd_rn(e[c], s);
  }
  for (int c = 0; c < cols; ++c) yr[c] = __fdiv_rn(e[c], s);
}

// How many rows per SM the balanced kernel takes before the plain grid of 8-row CTAs
// (which refills SMs as CTAs finish) streams as well.
constexpr int64_t kBalancedMaxRowsPerSm = 128;

template <int V>
cudaError_t launch_warp(const float *x, float *y, int64_t rows, int cols, float max_init,
                        cudaStream_t stream) {
  static const int sms = [] {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
  }();
  static const int variant = getenv("IMEX_SOFTMAX_VARIANT") ? atoi(getenv("IMEX_SOFTMAX_VARIANT")) : 1;
  if (variant == 1 && rows <= kBalancedMaxRowsPerSm * sms) {
    constexpr int MAXW = V <= 8 ? 32 : 16;
    const int64_t per_sm = (rows + sms - 1) / sms;            // rows of the fullest SM
    const int64_t rounds = (per_sm + MAXW - 1) / MAXW;        // rows a warp walks
    const int warps_cta = static_cast<int>((per_sm + rounds - 1) / rounds);
    const unsigned grid = static_cast<unsigned>(rows < sms ? rows : sms);
    // a launch of a few microseconds: let its set-up overlap the end of the launch before it
    // (IMEX_SOFTMAX_PDL=0: plain stream order)
    static const bool pdl = !(getenv("IMEX_SOFTMAX_PDL") && atoi(getenv("IMEX_SOFTMAX_PDL")) == 0);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(32 * warps_cta);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    if (cols == 4 * 32 * V)
      return cudaLaunchKernelEx(&cfg, softmax_warp_balanced_kernel<V, MAXW, true>, x, y, rows, cols, max_init);
    return cudaLaunchKernelEx(&cfg, softmax_warp_balanced_kernel<V, MAXW, false>, x, y, rows, cols, max_init);
  }
  const int warps = 8;
  unsigned grid = static_cast<unsigned>((rows + warps - 1) / warps);
  if (cols == 4 * 32 * V) softmax_warp_kernel<V, true><<<grid, warps * 32, 0, stream>>>(x, y, rows, cols, max_init);
  else softmax_warp_kernel<V, false><<<grid, warps * 32, 0, stream>>>(x, y, rows, cols, max_init);
  return cudaGetLastError();
}

// 16-bit rows (the f16 / bf16 rows of the reference's benchmark grid,
// benchmarks/softmax/softmax.dtypes.in): the chain's generics run in the element type, so
// every operation rounds to it, and the row sum is a sequential chain of rounded adds whose
// order decides the result.  One block per row: the row is staged in shared memory as f32,
// max / subtract / exp / divide run on all threads, the sum on one thread in index order.
template <bool BF16>
__device__ __forceinline__ float round16(float v) {
  if (BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return __half2float(__float2half_rn(v));
}
template <bool BF16>
__device__ __forceinline__ uint16_t to_bits16(float v) {  // v holds a 16-bit value exactly
  if (BF16) return static_cast<uint16_t>(__float_as_uint(v) >> 16);
  return __half_as_ushort(__float2half_rn(v));
}
template <bool BF16>
__device__ __forceinline__ uint16_t add16(uint16_t a, uint16_t b) {
  uint16_t d;
  if (BF16) asm("add.rn.bf16 %0, %1, %2;" : "=h"(d) : "h"(a), "h"(b));
  else asm("add.rn.f16 %0, %1, %2;" : "=h"(d) : "h"(a), "h"(b));
  return d;
}
template <bool BF16>
__global__ void __launch_bounds__(256)
softmax_rows_x16_kernel(const uint16_t *__restrict__ x, uint16_t *__restrict__ y, int64_t rows,
                        int cols, float max_init) {
  extern __shared__ float row[];
  __shared__ float red[8];
  __shared__ float total;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint16_t *xr = x + r * cols;
    float mx = max_init;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
      const float v = BF16 ? __uint_as_float(static_cast<uint32_t>(xr[i]) << 16)
                           : __half2float(__ushort_as_half(xr[i]));
      row[i] = v;
      mx = fmaxf(mx, v);
    }
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
      const float t = round16<BF16>(__fsub_rn(row[i], mx));
      // the two forms that give libm's expf rounded to the type for every argument of the type
      row[i] = round16<BF16>(BF16 ? exp_neg(t) : exp_f16_arg(t));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      // The chain s <- round16(x_i + s) is the critical path of the kernel.  One native 16-bit
      // add per step (add.rn.f16 / add.rn.bf16, latency of one instruction) gives the same
      // bits as add in f32 and round: the exact sum rounded once to 11 (8) bits equals the sum
      // rounded to f32's 24 bits and then to 11 (8), since 24 >= 2 * 11 + 2.  The values of
      // the row are already 16-bit values held in f32, so converting them is exact and off
      // the chain.
      uint16_t sum = 0;
      int i = 0;
      for (; i + 4 <= cols; i += 4) {
        uint16_t v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = to_bits16<BF16>(row[i + u]);
#pragma unroll
        for (int u = 0; u < 4; ++u) sum = add16<BF16>(v[u], sum);
      }
      for (; i < cols; ++i) sum = add16<BF16>(to_bits16<BF16>(row[i]), sum);
      total = BF16 ? __uint_as_float(static_cast<uint32_t>(sum) << 16) : __half2float(__ushort_as_half(sum));
    }
    __syncthreads();
    const float sum = total;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
      const float q = __fdiv_rn(row[i], sum);
      y[r * cols + i] = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(q)) : __half_as_ushort(__float2half_rn(q));
    }
    __syncthreads();
  }
}

} // namespace

cudaError_t launch_softmax_x16(const void *x, void *y, int64_t rows, int64_t cols, bool neg_inf_init,
                               bool is_bf16, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  if (cols > 12288) return cudaErrorNotSupported;  // the row is staged in 48 KB of shared memory
  // -FLT_MAX is not a 16-bit value: the fill of the IR holds it rounded to the element type
  const float max_init = neg_inf_init ? -INFINITY : (is_bf16 ? -3.3895313892515355e38f : -INFINITY);
  const unsigned grid = static_cast<unsigned>(rows < 148 * 8 ? rows : 148 * 8);
  const size_t smem = static_cast<size_t>(cols) * sizeof(float);
  if (is_bf16)
    softmax_rows_x16_kernel<true><<<grid, 256, smem, stream>>>(static_cast<const uint16_t *>(x),
                                                               static_cast<uint16_t *>(y), rows,
                                                               static_cast<int>(cols), max_init);
  else
    softmax_rows_x16_kernel<false><<<grid, 256, smem, stream>>>(static_cast<const uint16_t *>(x),
                                                                static_cast<uint16_t *>(y), rows,
                                                                static_cast<int>(cols), max_init);
  return cudaGetLastError();
}

cudaError_t launch_softmax_f32(const float *x, float *y, int64_t rows, int64_t cols,
                               bool neg_inf_init, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  const float max_init = neg_inf_init ? -INFINITY : -FLT_MAX;
  if (cols <= 64 && rows <= 65536) {
    softmax_tiny_rows_kernel<<<static_cast<unsigned>((rows + 127) / 128), 128, 0, stream>>>(
        x, y, rows, static_cast<int>(cols), max_init);
    return cudaGetLastError();
  }
  const bool vec_ok = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
  if (vec_ok && cols <= 128) return launch_warp<1>(x, y, rows, (int)cols, max_init, stream);
  if (vec_ok && cols <= 256) return launch_warp<2>(x, y, rows, (int)cols, max_init, stream);
  if (vec_ok && cols <= 512) return launch_warp<4>(x, y, rows, (int)cols, max_init, stream);
  if (vec_ok && cols <= 1024) return launch_warp<8>(x, y, rows, (int)cols, max_init, stream);
  if (vec_ok && cols <= 2048) return launch_warp<16>(x, y, rows, (int)cols, max_init, stream);
  unsigned grid = static_cast<unsigned>(rows < 148 * 16 ? rows : 148 * 16);
  softmax_block_kernel<<<grid, 256, 0, stream>>>(x, y, rows, cols, max_init);
  return cudaGetLastError();
}

} // namespace imex
