// Elementwise epilogues, following the reference's generics op for op.
#pragma once
#include "kernels.h"

namespace imex {

// cmpf ugt x, 0 ; select x, 0   (benchmarks/relu/relu_gpu.mlir.in:6-11):
// unordered-or-greater, so NaN passes through and -0 becomes +0.
__device__ __forceinline__ float relu_ugt(float x) { return !(x <= 0.0f) ? x : 0.0f; }

// negf, exp, addf 1, divf 1/., then mulf s*x
// (benchmarks/silu/silu_gpu.mlir.in:6-18); every step separately rounded.
__device__ __forceinline__ float silu_chain(float x) {
  float e = expf(-x);
  float d = __fadd_rn(e, 1.0f);
  float s = __fdiv_rn(1.0f, d);
  return __fmul_rn(s, x);
}

// Tensor-core path only: the same function with the hardware exp2 / reciprocal
// approximations (relative error ~1e-6, far inside the 1e-3 Frobenius budget of
// the 16-bit GEMM); a quarter of the instructions of silu_chain.
__device__ __forceinline__ float silu_fast(float x) {
  return __fdividef(x, 1.0f + __expf(-x));
}

__device__ __forceinline__ float apply_epilogue_fast(float v, int epilogue) {
  if (epilogue == kEpiRelu) return relu_ugt(v);
  if (epilogue == kEpiSilu) return silu_fast(v);
  return v;
}

__device__ __forceinline__ float apply_epilogue(float v, int epilogue) {
  if (epilogue == kEpiRelu) return relu_ugt(v);
  if (epilogue == kEpiSilu) return silu_chain(v);
  return v;
}

__device__ __forceinline__ float load_as_f32(const float *p, int64_t i) { return p[i]; }

__device__ __forceinline__ float bf16_bits_to_f32(unsigned short b) {
  return __uint_as_float(static_cast<unsigned>(b) << 16);
}

} // namespace imex
