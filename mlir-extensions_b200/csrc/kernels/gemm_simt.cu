// Bit-exact SIMT GEMM: C[i,j] = C0[i,j] + sum_k A[i,k]*B[k,j] with k ascending
// and the multiply and the add rounded separately — the arithmetic of the
// scalar loop nest that convert-linalg-to-loops produces for linalg.matmul
// (reference: test/PlaidML/OpTest.Matmul.mlir:14-20,
//  test/PlaidML/OpTest.GEMM_FLOAT32.mlir:37-42; 16-bit inputs extended to f32
//  first as in test/SPIRV/OpTest.GEMM_BF16_ACC_F32.mlir:126-141).
// Changing the summation order moves some outputs by far more than 1e-4
// relative (cancellation), so this path keeps the order; it is FP32-pipe
// bound, not a tensor-core kernel.
#include "epilogue.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace imex {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename O> __device__ __forceinline__ O from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// trans_a: A is stored [K,M]; trans_b: B is stored [N,K].  O = element type of C
// (f32 accumulation in every case, one rounding when O is 16 bits wide).
template <typename T, typename O>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T *__restrict__ A, const T *__restrict__ B, O *__restrict__ C,
                 const float *__restrict__ bias, int64_t M, int64_t N, int64_t K, int64_t lda,
                 int64_t ldb, int64_t ldc, int epilogue, int accumulate, int trans_a, int trans_b) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int64_t r = m0 + ty * TM + i, c = n0 + tx * TN + j;
      acc[i][j] = (accumulate && r < M && c < N) ? to_f32(C[r * ldc + c]) : 0.0f;
    }

  for (int64_t k0 = 0; k0 < K; k0 += BK) {
    // A tile: BM x BK, stored k-major so the inner loop reads it conflict-free
    for (int e = tid; e < BM * BK; e += 256) {
      // consecutive threads walk the contiguous dimension of the stored array
      int m = trans_a ? e % BM : e / BK, k = trans_a ? e / BM : e % BK;
      int64_t r = m0 + m, kk = k0 + k;
      As[k][m] = (r < M && kk < K) ? to_f32(trans_a ? A[kk * lda + r] : A[r * lda + kk]) : 0.0f;
    }
    for (int e = tid; e < BK * BN; e += 256) {
      int k = trans_b ? e % BK : e / BN, n = trans_b ? e / BK : e % BN;
      int64_t kk = k0 + k, c = n0 + n;
      Bs[k][n] = (kk < K && c < N) ? to_f32(trans_b ? B[c * ldb + kk] : B[kk * ldb + c]) : 0.0f;
    }
    __syncthreads();
    // only real k steps: a padded step would add +0 and could flip a -0 result
    const int kmax = (K - k0 < BK) ? static_cast<int>(K - k0) : BK;
    for (int k = 0; k < kmax; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j)
          acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int64_t r = m0 + ty * TM + i, c = n0 + tx * TN + j;
      if (r < M && c < N) {
        float v = acc[i][j];
        if (bias) v = __fadd_rn(v, bias[c]);
        C[r * ldc + c] = from_f32<O>(apply_epilogue(v, epilogue));
      }
    }
}

} // namespace

namespace {
template <typename T, typename O>
void launch_typed(const GemmProblem &p, dim3 grid, int64_t lda, int64_t ldb, int64_t ldc,
                  cudaStream_t stream) {
  gemm_simt_kernel<T, O><<<grid, 256, 0, stream>>>(
      static_cast<const T *>(p.A), static_cast<const T *>(p.B), reinterpret_cast<O *>(p.C), p.bias,
      p.M, p.N, p.K, lda, ldb, ldc, p.epilogue, p.accumulate ? 1 : 0, p.trans_a ? 1 : 0,
      p.trans_b ? 1 : 0);
}
template <typename T>
bool launch_in(const GemmProblem &p, dim3 grid, int64_t lda, int64_t ldb, int64_t ldc,
               cudaStream_t stream) {
  if (p.out_dtype == kF32) launch_typed<T, float>(p, grid, lda, ldb, ldc, stream);
  else if (p.out_dtype == kBF16) launch_typed<T, __nv_bfloat16>(p, grid, lda, ldb, ldc, stream);
  else if (p.out_dtype == kF16) launch_typed<T, __half>(p, grid, lda, ldb, ldc, stream);
  else return false;
  return true;
}
} // namespace

cudaError_t launch_gemm_simt(const GemmProblem &p, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0) return cudaSuccess;
  const int64_t lda = p.lda > 0 ? p.lda : (p.trans_a ? p.M : p.K),
                ldb = p.ldb > 0 ? p.ldb : (p.trans_b ? p.K : p.N), ldc = p.ldc > 0 ? p.ldc : p.N;
  dim3 grid(static_cast<unsigned>((p.N + BN - 1) / BN), static_cast<unsigned>((p.M + BM - 1) / BM));
  bool ok;
  if (p.in_dtype == kF32) ok = launch_in<float>(p, grid, lda, ldb, ldc, stream);
  else if (p.in_dtype == kBF16) ok = launch_in<__nv_bfloat16>(p, grid, lda, ldb, ldc, stream);
  else if (p.in_dtype == kF16) ok = launch_in<__half>(p, grid, lda, ldb, ldc, stream);
  else ok = false;
  if (!ok) return cudaErrorInvalidValue;
  return cudaGetLastError();
}

} // namespace imex
