// Launchers of the sm_100a kernels behind the GPU runtime-wrapper C ABI.
// Every launcher enqueues on `stream` and returns the launch status; none
// allocates.  `status` is a host-mapped error word kernels with bounded
// waits write to when a wait runs out (0 = fine).
#pragma once

#include <cuda_runtime.h>
#include <cstdint>
#include <string>

namespace imex {

enum DType : int { kF32 = 1, kBF16 = 2, kF16 = 3, kI32 = 4 };
enum Epilogue : int { kEpiNone = 0, kEpiRelu = 1, kEpiSilu = 2 };

// Device status codes written to the status word.
enum Status : unsigned {
  kStatusOk = 0,
  kStatusTmaWaitTimeout = 1,   // producer gave up waiting for a free smem stage
  kStatusMmaWaitTimeout = 2,   // MMA warp gave up waiting for operands / a free accumulator
  kStatusEpiWaitTimeout = 3,   // epilogue gave up waiting for an accumulator
  kStatusPeerWaitTimeout = 4,  // the cross-rank barrier gave up waiting for a peer
  kStatusSelfTestTimeout = 99  // the wait self-test ran out, as it is meant to
};

struct GemmProblem {
  const void *A;      // [M,K] row-major, in_dtype ([K,M] when trans_a)
  const void *B;      // [K,N] row-major, in_dtype ([N,K] when trans_b)
  float *C;           // [M,N] row-major; elements are out_dtype (f32 unless stated)
  const float *bias;  // [N] f32 or nullptr
  int64_t M, N, K;
  // row pitches of the arrays as stored, in elements; 0 = dense
  int64_t lda = 0, ldb = 0, ldc = 0;
  int in_dtype;       // DType
  int out_dtype = kF32;  // kF32, or kBF16 / kF16: f32 accumulation (and f32 C input when
                         // `accumulate`), one rounding to 16 bits after bias + epilogue
  bool trans_a = false;  // C = A^T . B with A stored [K,M]
  bool trans_b = false;  // C = A . B^T with B stored [N,K]
  int epilogue;       // Epilogue
  bool accumulate;    // C is read as the initial value
  int sm_margin = 0;  // SMs the persistent kernels leave unused
  void *workspace = nullptr;   // device scratch for a k-split tail (optional)
  size_t workspace_bytes = 0;
  int *launched = nullptr;     // out (optional): kernels this call enqueued (2 with a k-split tail)
};

// f32 or 16-bit inputs, one thread per 4x4 outputs, k ascending with
// separately rounded multiply and add: bit-identical to the scalar loop nest
// of linalg-to-loops.  Any shape.
cudaError_t launch_gemm_simt(const GemmProblem &p, cudaStream_t stream);

// bf16/f16 -> f32 on the 5th-gen tensor cores (tcgen05.mma, TMEM
// accumulators, TMA-fed 128B-swizzled smem ring, persistent tiles).
// Needs the contiguous extents of A and B (K or M; N or K) to be multiples of
// 8, pitches that keep rows 16-byte aligned and 16-byte aligned A, B, C.
bool gemm_tcgen05_supported(const GemmProblem &p);
cudaError_t launch_gemm_tcgen05(const GemmProblem &p, unsigned *status,
                                cudaStream_t stream);
// CTA pairs (tcgen05.mma.cta_group::2, 256x256 tile per pair); also takes
// transposed operands (trans_a / trans_b) and bf16 / f16 outputs.
bool gemm_tcgen05_2cta_supported(const GemmProblem &p);
bool gemm_tcgen05_2cta_preferred(const GemmProblem &p);
size_t gemm_tcgen05_workspace_bytes();  // scratch the pair kernel can use for a k-split tail
cudaError_t launch_gemm_tcgen05_2cta(const GemmProblem &p, unsigned *status,
                                     cudaStream_t stream);

// O = softmax(sm_scale * Q K^T) V per head; Q, K, V, O are [heads * n_ctx, 64] f16 or bf16
// arrays, heads one after the other (tcgen05 for both products, one pass over K and V).
bool flash_attention_supported(int64_t heads, int64_t n_ctx, int64_t d_head, int dtype, const void *q,
                               const void *k, const void *v, const void *o);
cudaError_t launch_flash_attention_fwd(const void *q, const void *k, const void *v, void *o, int64_t heads,
                                       int64_t n_ctx, int64_t d_head, float sm_scale, int dtype,
                                       unsigned *status, cudaStream_t stream);

// One thread waits (bounded, ~1 ms) on a barrier nothing signals and reports
// kStatusSelfTestTimeout: exercises wait expiry -> status word -> gpuWait error.
cudaError_t launch_wait_selftest(unsigned *status, cudaStream_t stream);

// Row softmax over the last dim (one pass over HBM: read X once, write Y once).
cudaError_t launch_softmax_f32(const float *x, float *y, int64_t rows, int64_t cols,
                               bool neg_inf_init, cudaStream_t stream);

// The same chain on f16 / bf16 rows: every operation rounds to the element type and the row
// sum is the sequential chain of rounded adds that the loop nest performs.  cols <= 12288.
cudaError_t launch_softmax_x16(const void *x, void *y, int64_t rows, int64_t cols, bool neg_inf_init,
                               bool is_bf16, cudaStream_t stream);

// Y[r] = (acc ? Y[r] : 0) + sum_c X[r,c]
cudaError_t launch_reduce_rows_f32(const float *x, float *y, int64_t rows, int64_t cols,
                                   bool accumulate, cudaStream_t stream);
// Y[i] = (acc ? Y[i] : 0) + sum_l X[l,i], l ascending (bit-identical to the loop nest)
cudaError_t launch_reduce_leading_f32(const float *x, float *y, int64_t lead, int64_t inner,
                                      bool accumulate, cudaStream_t stream);
// *Y = (acc ? *Y : 0) + sum X.  `partials` is scratch for reduce_all_partials() floats.
int64_t reduce_all_partials(int64_t n);
int64_t reduce_all_block_elems();  // elements summed into one partial
cudaError_t launch_reduce_all_f32(const float *x, float *y, int64_t n, bool accumulate,
                                  float *partials, cudaStream_t stream);

// Y[j,i] = X[i,j]; elem_bytes 4 or 2.
cudaError_t launch_transpose2d(const void *x, void *y, int64_t rows, int64_t cols,
                               int elem_bytes, cudaStream_t stream);
// rank-3 permutation of 4- or 2-byte elements: Y dims = X dims permuted by perm.
cudaError_t launch_transpose3d(const void *x, void *y, const int64_t dims[3], const int perm[3],
                               int elem_bytes, cudaStream_t stream);

// Y[i] = epilogue(X[i]) (standalone relu / silu)
cudaError_t launch_eltwise_f32(const float *x, float *y, int64_t n, int epilogue,
                               cudaStream_t stream);

// A fused chain of elementwise ops as a postfix program (ImexExprCode): Y[r,c] =
// program(X_k[r,c] | X_k[c] | X_k[r] ...), every operation rounded to `dtype`; with
// reduce_leading Y[c] = (acc ? Y[c] : 0) + sum_r program(...), r ascending.
int expr_validate(const unsigned char *code, int max_len, int n_inputs);
cudaError_t launch_expr(const void *const *inputs, int n_inputs, void *out, int64_t rows, int64_t cols,
                        const unsigned char *code, int ncode, float c0, float c1, int dtype,
                        int out_dtype, bool reduce_leading, bool accumulate, cudaStream_t stream);

// The same call served by a kernel compiled for this program at first use (NVRTC);
// cudaErrorNotSupported when no compiled kernel can be had: use launch_expr then.
cudaError_t launch_expr_jit(const void *const *inputs, int n_inputs, void *out, int64_t rows, int64_t cols,
                            const unsigned char *code, int ncode, float c0, float c1, int dtype,
                            int out_dtype, bool reduce_leading, bool accumulate, cudaStream_t stream);

// A loop-nest kernel given as CUDA C++ text (one `extern "C" __global__ void
// imex_loopnest(pointers...)` written against loopnest_prelude()): compiled for sm_100a at
// first use, cached by text, launched over `threads` points.  cudaErrorNotSupported when it
// cannot be compiled (*log then holds the compiler's output).
const char *loopnest_prelude();
cudaError_t launch_loopnest(const char *source, size_t source_bytes, void *const *ptrs, int n_ptrs,
                            int64_t threads, cudaStream_t stream, std::string *log);

// Y[i] = convert(X[i]): f32 <-> bf16 / f16 (arith.extf / arith.truncf generics)
cudaError_t launch_convert(const void *x, void *y, int64_t n, int in_dtype, int out_dtype,
                           cudaStream_t stream);

// Seeded synthetic inputs.  uniform: lo + (hi-lo)*u24(seed, first+i), the same
// integer hash as the CPU oracle (bit-identical in f32).  normal: Box-Muller.
cudaError_t launch_fill_uniform(void *y, int64_t n, int dtype, uint64_t seed, int64_t first,
                                float lo, float hi, cudaStream_t stream);
cudaError_t launch_fill_normal(void *y, int64_t n, int dtype, uint64_t seed, int64_t first,
                               float mean, float stddev, cudaStream_t stream);

} // namespace imex
