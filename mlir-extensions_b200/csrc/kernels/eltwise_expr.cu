// A chain of elementwise linalg.generic ops fused into one pass over HBM, optionally
// feeding a sum over the leading dimension.
//
// Reference: benchmarks/kLoopFusion/kLoopFusion.mlir.in:4-30 (log, absf, addf, subf over
// two 512x1024 inputs: four generics, three temporaries in the reference's lowering) and
// benchmarks/kInputFusion/kInputFusion.mlir.in:6-41 (the same kind of chain feeding a
// column reduce, maps (d0,d1)->(d1,d0) in, (d0,d1)->(d0) out).  Here the chain arrives as
// a postfix program (ImexExprCode in include/imex_b200_blob.h) and every element is read
// once and written once.
//
// Arithmetic: each operation is evaluated in f32 and rounded to the element type of the
// IR (f32: nothing to do; f16 / bf16: one rounding per operation, which is how 16-bit
// float operations are legalised on a CPU without native support).  add/sub/mul/div are
// separately rounded (no FMA contraction).
#include "epilogue.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace imex {
namespace {

struct ExprParams {
  const void *in[4];
  void *out;
  long long rows, cols;
  unsigned char code[32];
  int ncode;
  float c0, c1;
  int dtype;      // element type of the inputs and of every intermediate
  int out_dtype;  // element type of Y (elementwise form)
  int accumulate;
};

__device__ __forceinline__ float round_to(float v, int dt) {
  if (dt == kF16) return __half2float(__float2half_rn(v));
  if (dt == kBF16) return __bfloat162float(__float2bfloat16_rn(v));
  return v;
}

__device__ __forceinline__ float load_elem(const void *p, long long i, int dt) {
  if (dt == kF32) return static_cast<const float *>(p)[i];
  if (dt == kF16) return __half2float(static_cast<const __half *>(p)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
}

// V consecutive elements starting at index i (a multiple of V; the arrays are 16-byte
// aligned when V == 4): one 16-byte or 8-byte load instead of four scalar ones
template <int V>
__device__ __forceinline__ void load_vec(const void *p, long long i, int dt, float (&out)[V]) {
  if constexpr (V == 4) {
    if (dt == kF32) {
      const float4 q = *reinterpret_cast<const float4 *>(static_cast<const float *>(p) + i);
      out[0] = q.x; out[1] = q.y; out[2] = q.z; out[3] = q.w;
    } else {
      const uint2 q = *reinterpret_cast<const uint2 *>(static_cast<const unsigned short *>(p) + i);
      const unsigned short h[4] = {static_cast<unsigned short>(q.x), static_cast<unsigned short>(q.x >> 16),
                                   static_cast<unsigned short>(q.y), static_cast<unsigned short>(q.y >> 16)};
#pragma unroll
      for (int v = 0; v < 4; ++v)
        out[v] = dt == kF16 ? __half2float(__ushort_as_half(h[v])) : bf16_bits_to_f32(h[v]);
    }
  } else {
#pragma unroll
    for (int v = 0; v < V; ++v) out[v] = load_elem(p, i + v, dt);
  }
}

__device__ __forceinline__ void store_elem(void *p, long long i, float v, int dt) {
  if (dt == kF32) static_cast<float *>(p)[i] = v;
  else if (dt == kF16) static_cast<__half *>(p)[i] = __float2half_rn(v);
  else static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float maximumf(float a, float b) {
  if (a != a) return a;
  if (b != b) return b;
  return fmaxf(a, b);
}
__device__ __forceinline__ float minimumf(float a, float b) {
  if (a != a) return a;
  if (b != b) return b;
  return fminf(a, b);
}

__device__ __forceinline__ float unary(int op, float x, int dt) {
  switch (op) {
  case 32: return -x;
  case 33: return fabsf(x);
  case 34: return logf(x);
  // 16-bit types: the forms that round to libm's 16-bit value for every argument, as in the compiled chains
  case 35: return dt == kF16 ? exp_f16_arg(x) : dt == kBF16 ? exp_neg(x) : expf(x);
  case 36: return __fsqrt_rn(x);
  case 37: return __fdiv_rn(1.0f, __fsqrt_rn(x));
  case 38: return tanhf(x);
  case 39: return relu_ugt(x);
  }
  return x;
}

__device__ __forceinline__ float binary(int op, float a, float b) {
  switch (op) {
  case 64: return __fadd_rn(a, b);
  case 65: return __fsub_rn(a, b);
  case 66: return __fmul_rn(a, b);
  case 67: return __fdiv_rn(a, b);
  case 68: return maximumf(a, b);
  case 69: return minimumf(a, b);
  }
  return a;
}

// Evaluates the program for V consecutive columns of one row.  The top of the stack
// lives in registers; deeper entries in a small per-thread array (program-uniform
// indices, so it stays in L1).
template <int V>
__device__ __forceinline__ void evaluate(const ExprParams &p, long long row, long long col, float (&top)[V]) {
  float deep[7][V];
  int sp = 0;  // values on the stack, top included
#pragma unroll 1
  for (int pc = 0; pc < p.ncode; ++pc) {
    const int op = p.code[pc];
    if (op < 32) {  // push
      if (sp > 0) {
#pragma unroll
        for (int v = 0; v < V; ++v) deep[sp - 1][v] = top[v];
      }
      ++sp;
      if (op >= 1 && op <= 4) {
        load_vec<V>(p.in[op - 1], row * p.cols + col, p.dtype, top);
      } else if (op >= 5 && op <= 8) {
        load_vec<V>(p.in[op - 5], col, p.dtype, top);
      } else if (op >= 9 && op <= 12) {
        const float x = load_elem(p.in[op - 9], row, p.dtype);
#pragma unroll
        for (int v = 0; v < V; ++v) top[v] = x;
      } else {
        const float x = op == 13 ? p.c0 : op == 14 ? p.c1 : op == 16 ? 1.0f : 0.0f;
#pragma unroll
        for (int v = 0; v < V; ++v) top[v] = round_to(x, p.dtype);
      }
    } else if (op < 64) {
#pragma unroll
      for (int v = 0; v < V; ++v) top[v] = round_to(unary(op, top[v], p.dtype), p.dtype);
    } else {
      --sp;
#pragma unroll
      for (int v = 0; v < V; ++v) top[v] = round_to(binary(op, deep[sp - 1][v], top[v]), p.dtype);
    }
  }
}

template <int V>
__global__ void __launch_bounds__(256) expr_elementwise_kernel(const ExprParams p) {
  const long long groups_per_row = p.cols / V;
  const long long total = p.rows * groups_per_row;
  for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < total;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = g / groups_per_row, col = (g % groups_per_row) * V;
    float r[V];
    evaluate<V>(p, row, col, r);
    const long long base = row * p.cols + col;
    if (V == 4 && p.out_dtype == kF32) {
      *reinterpret_cast<float4 *>(static_cast<float *>(p.out) + base) = make_float4(r[0], r[1], r[2], r[3]);
    } else {
#pragma unroll
      for (int v = 0; v < V; ++v) store_elem(p.out, base + v, r[v], p.out_dtype);
    }
  }
}

// Y[col] = (Y[col]) + sum over rows, ascending, of the expression: one thread per column,
// consecutive threads on consecutive columns (coalesced), the order of the loop nest.
__global__ void __launch_bounds__(256) expr_reduce_leading_kernel(const ExprParams p) {
  const long long col = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (col >= p.cols) return;
  float acc = p.accumulate ? load_elem(p.out, col, p.dtype) : 0.0f;
  for (long long row = 0; row < p.rows; ++row) {
    float r[1];
    evaluate<1>(p, row, col, r);
    acc = round_to(__fadd_rn(acc, r[0]), p.dtype);
  }
  store_elem(p.out, col, acc, p.dtype);
}

} // namespace

// Checks a postfix program: known opcodes, inputs < n_inputs, stack never empty or deeper
// than 8, exactly one value left.  Returns the number of code bytes, or -1.
int expr_validate(const unsigned char *code, int max_len, int n_inputs) {
  int sp = 0, n = 0;
  for (; n < max_len && code[n] != 0; ++n) {
    const int op = code[n];
    if (op >= 1 && op <= 12) {
      if ((op - 1) % 4 >= n_inputs) return -1;
      ++sp;
    } else if (op >= 13 && op <= 16) {
      ++sp;
    } else if (op >= 32 && op <= 39) {
      if (sp < 1) return -1;
    } else if (op >= 64 && op <= 69) {
      if (sp < 2) return -1;
      --sp;
    } else {
      return -1;
    }
    if (sp > 8) return -1;
  }
  return sp == 1 ? n : -1;
}

cudaError_t launch_expr(const void *const *inputs, int n_inputs, void *out, int64_t rows, int64_t cols,
                        const unsigned char *code, int ncode, float c0, float c1, int dtype,
                        int out_dtype, bool reduce_leading, bool accumulate, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  if (n_inputs < 0 || n_inputs > 4 || ncode < 1 || ncode > 32) return cudaErrorInvalidValue;
  if (expr_validate(code, ncode, n_inputs) != ncode) return cudaErrorInvalidValue;
  ExprParams p{};
  bool aligned = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  for (int i = 0; i < n_inputs; ++i) {
    p.in[i] = inputs[i];
    aligned = aligned && (reinterpret_cast<uintptr_t>(inputs[i]) & 15) == 0;
  }
  p.out = out;
  p.rows = rows;
  p.cols = cols;
  for (int i = 0; i < ncode; ++i) p.code[i] = code[i];
  p.ncode = ncode;
  p.c0 = c0;
  p.c1 = c1;
  p.dtype = dtype;
  p.out_dtype = out_dtype;
  p.accumulate = accumulate ? 1 : 0;
  if (reduce_leading) {
    const unsigned blocks = static_cast<unsigned>((cols + 255) / 256);
    expr_reduce_leading_kernel<<<blocks, 256, 0, stream>>>(p);
    return cudaGetLastError();
  }
  const bool vec = aligned && cols % 4 == 0;
  const long long groups = vec ? rows * (cols / 4) : rows * cols;
  long long blocks = (groups + 255) / 256;
  const long long cap = 148LL * 16;
  if (blocks > cap) blocks = cap;
  if (vec)
    expr_elementwise_kernel<4><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  else
    expr_elementwise_kernel<1><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

} // namespace imex
