// Elementwise epilogues, following the reference's generics op for op.
#pragma once
#include "kernels.h"

namespace imex {

// cmpf ugt x, 0 ; select x, 0   (benchmarks/relu/relu_gpu.mlir.in:6-11):
// unordered-or-greater, so NaN passes through and -0 becomes +0.
__device__ __forceinline__ float relu_ugt(float x) { return !(x <= 0.0f) ? x : 0.0f; }

// exp(t) in a handful of instructions: 2^(t*log2e) through the
// hardware ex2 unit, with the rounding error of the product t*log2e (which
// alone would cost 1.5e-6 relative at t = -26) fed back as a first-order
// correction.  y + r is t*log2e to ~2^-48 relative (log2e split in hi + lo, the
// product's residual recovered with an FMA); ex2.approx is good to 2 ulp, so the
// result is within ~3e-7 of libm's expf, which the CPU pipeline calls
// (convert-math-to-libm).  libm's expf costs ~25 instructions per element and,
// with every warp of the single wave in the same phase, was a third of the
// 4096x1024 softmax kernel's time.  NaN, -inf (ex2(-inf) = 0) and +inf pass through; results
// below the normal range come out as the hardware's subnormals, overflow as +inf: where the
// correction is not a number (an infinite argument, or 2^y = inf times a negative residual)
// the uncorrected 2^y is the result.
__device__ __forceinline__ float exp_neg(float t) {
  const float L2E_HI = 1.44269502162933349609375f;   // float(log2(e))
  const float L2E_LO = 1.92596299112661746e-8f;      // log2(e) - L2E_HI
  const float LN2 = 0.693147182464599609375f;
  const float y = __fmul_rn(t, L2E_HI);
  float r = __fmaf_rn(t, L2E_HI, -y);                // exact residual of the product
  r = __fmaf_rn(t, L2E_LO, r);
  float e;
  asm("ex2.approx.f32 %0, %1;" : "=f"(e) : "f"(y));
  // 2^(y + r) = 2^y * (1 + r ln2 + ...);  |r| < 2^-18, the next term is below 2^-38
  const float c = __fmaf_rn(e, __fmul_rn(r, LN2), e);
  return c == c ? c : e;
}

// exp of an f16 value, for a result that is rounded to f16: without the low part of log2 e.
// Rounded to f16 it equals libm's expf rounded to f16 for every one of the 65536 f16 arguments,
// as exp_neg does for every bf16 argument (both tested over all arguments on the device).  A result
// below f32's normal range rounds to zero in f16 flushed or not: the flushing form of ex2.
__device__ __forceinline__ float exp_f16_arg(float t) {
  const float L2E_HI = 1.44269502162933349609375f;
  const float y = __fmul_rn(t, L2E_HI);
  const float r = __fmaf_rn(t, L2E_HI, -y);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(y));
  const float c = __fmaf_rn(e, __fmul_rn(r, 0.693147182464599609375f), e);
  return c == c ? c : e;
}

// negf, exp, addf 1, divf 1/., then mulf s*x
// (benchmarks/silu/silu_gpu.mlir.in:6-18); every step separately rounded.
__device__ __forceinline__ float silu_chain(float x) {
  float e = exp_neg(-x);
  float d = __fadd_rn(e, 1.0f);
  float s = __frcp_rn(d);   // 1 / d correctly rounded = the IEEE quotient divf gives
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
