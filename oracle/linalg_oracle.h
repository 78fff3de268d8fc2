/* CPU oracle for the IMEX hot path — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of what the reference's CPU pipeline
 * (imex-runner + test/PlaidML/linalg-to-cpu.pp:2-19 /
 * benchmarks/pipelines/linalg-to-cpu.pp:2-27: linalg -> scf loops -> LLVM)
 * computes for the ops on the hot path.  The lowering itself lives in
 * llvm-project @ a5641e23331a9bfae03a97fba5e4dff1f7c69f63
 * (build_tools/llvm_version.txt:1), which is not vendored in the reference;
 * its published algorithm is: walk the linalg iteration space with d0 as the
 * outermost loop, evaluate the region body once per point in the element
 * type of the IR, load/store the output element around every body
 * evaluation, no reassociation, no FMA contraction, math.exp -> libm expf.
 *
 * Parity pins: tests/golden/reference_vectors.json (values transcribed from
 * the CHECK lines of the reference's own tests) and oracle/_ref (the
 * reference's in-tree CPU GEMM compiled from its own source file).
 * silu and the one-generic-at-a-time functions in 16-bit element types
 * (oracle_unary / oracle_binary / oracle_reduce_leading_as) are pinned through
 * the reference's generated tests (test/Gen/PlaidML templates and the
 * benchmark templates with their printed CHECK values): tests/test_oracle_pins.py
 * runs the same programs through these functions and through the loop-nest
 * checker that reproduces those CHECK lines.
 * PARITY UNPINNED (the reference prints no values for it):
 * oracle_attention_fwd_x16.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
 * load this library.  The product never does.
 */
#ifndef IMEX_B200_LINALG_ORACLE_H
#define IMEX_B200_LINALG_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORACLE_EPI_NONE = 0, ORACLE_EPI_RELU = 1, ORACLE_EPI_SILU = 2 };
enum { ORACLE_SOFTMAX_BENCH = 0, ORACLE_SOFTMAX_PLAIDML = 1 };

/* --- 16-bit float helpers (ImexRunnerUtils.cpp:118-169) ------------------ */
float oracle_bf16_to_f32(uint16_t bits);
float oracle_f16_to_f32(uint16_t bits);
uint16_t oracle_f32_to_bf16(float v); /* round to nearest even */
uint16_t oracle_f32_to_f16(float v);  /* round to nearest even */
void oracle_round_to_bf16(const float *src, uint16_t *dst, int64_t n);
void oracle_round_to_f16(const float *src, uint16_t *dst, int64_t n);

/* --- matmul: C[i,j] = C[i,j] + A[i,k]*B[k,j], k ascending ----------------
 * linalg.matmul (test/PlaidML/OpTest.Matmul.mlir:14-20) and the matmul-shaped
 * generic (test/PlaidML/OpTest.GEMM_FLOAT32.mlir:13-15,37-42).
 * *_loops: literal i,j,k loop nest of convert-linalg-to-loops, one thread
 *          (this is what the CPU baseline times).
 * *_fast : identical per-element arithmetic, i,k,j order, rows split over
 *          OpenMP threads (checker for large shapes; every C[i,j] still sees
 *          the same sequence of roundings). */
void oracle_matmul_f32_loops(const float *A, const float *B, float *C,
                             int64_t M, int64_t N, int64_t K);
void oracle_matmul_f32_fast(const float *A, const float *B, float *C,
                            int64_t M, int64_t N, int64_t K);
/* 16-bit inputs extended to f32 first (arith.extf), f32 accumulate
 * (test/SPIRV/OpTest.GEMM_BF16_ACC_F32.mlir:126-141,
 *  test/PlaidML/CppEdsl.DotF16_AccF32.mlir:19-47). is_bf16: 1 bf16, 0 f16. */
void oracle_matmul_x16_f32_loops(const uint16_t *A, const uint16_t *B,
                                 float *C, int64_t M, int64_t N, int64_t K,
                                 int is_bf16);
void oracle_matmul_x16_f32_fast(const uint16_t *A, const uint16_t *B, float *C,
                                int64_t M, int64_t N, int64_t K, int is_bf16);
/* rows [row0,row0+nrows) of the product only (sampled-row checks of shapes
 * whose full oracle would take hours). C points at the first sampled row. */
void oracle_matmul_x16_f32_rows(const uint16_t *A, const uint16_t *B, float *C,
                                int64_t row0, int64_t nrows, int64_t N,
                                int64_t K, int is_bf16);

/* bias[j] broadcast-added to every row (the reference's fused-epilogue GEMM
 * test, test/Integration/Dialect/XeGPU/WG/gemm_4kx4kx4k_f16_f16_f32_bias.mlir:91-113). */
void oracle_bias_add_f32(float *C, const float *bias, int64_t M, int64_t N);

/* --- elementwise epilogues -------------------------------------------- */
/* relu: cmpf ugt x,0 ; select x,0 (benchmarks/relu/relu_gpu.mlir.in:6-11) */
void oracle_relu_f32(const float *x, float *y, int64_t n);
/* silu: s = 1/(exp(-x)+1) ; y = s*x, two generics
 * (benchmarks/silu/silu_gpu.mlir.in:6-18) */
void oracle_silu_f32(const float *x, float *y, int64_t n);
void oracle_epilogue_f32(float *c, int64_t n, int epilogue);

/* --- one elementwise generic at a time, in the element type of the IR ------
 * The fused-chain benchmarks (benchmarks/kLoopFusion/kLoopFusion.mlir.in:4-30,
 * benchmarks/kInputFusion/kInputFusion.mlir.in:6-41) are chains of these, each
 * with its own full-size result; @dtype@ is f32, f16 or bf16
 * (kLoopFusion.dtypes.in).  Arrays hold the values as f32; `dtype` (ORACLE_DT_*)
 * says which type they stand for: a 16-bit operation is extend, operate in f32,
 * round to nearest even back (how LLVM legalises half / bfloat arithmetic where
 * the CPU has none).  The mnemonics are those of the IR. */
enum { ORACLE_DT_F32 = 1, ORACLE_DT_BF16 = 2, ORACLE_DT_F16 = 3 };
enum {
  ORACLE_OP_NEGF = 32, ORACLE_OP_ABSF = 33, ORACLE_OP_LOG = 34, ORACLE_OP_EXP = 35,
  ORACLE_OP_SQRT = 36, ORACLE_OP_RSQRT = 37, ORACLE_OP_TANH = 38, ORACLE_OP_RELU = 39,
  ORACLE_OP_ADDF = 64, ORACLE_OP_SUBF = 65, ORACLE_OP_MULF = 66, ORACLE_OP_DIVF = 67,
  ORACLE_OP_MAXIMUMF = 68, ORACLE_OP_MINIMUMF = 69
};
float oracle_round_as(float v, int dtype);
int oracle_unary(int op, int dtype, const float *x, float *y, int64_t n);
int oracle_binary(int op, int dtype, const float *a, const float *b, float *y, int64_t n);
/* y[j] = init[j] + sum_i x[i,j], i ascending, every add rounded to dtype: the
 * column reduce of kInputFusion.mlir.in:29-39 (maps (d0,d1)->(d1,d0), (d0,d1)->(d0)) */
void oracle_reduce_leading_as(int dtype, const float *x, float *y, int64_t lead, int64_t inner);

/* --- attention forward ----------------------------------------------------
 * The CPU check of the reference's flash-attention test
 * (test/Integration/Dialect/XeGPU/WG/flash_attention_fwd.mlir:334-432): Q, K, V
 * and O are [heads * n_ctx, d_head] 16-bit arrays, heads laid out one after the
 * other; per head S = sm_scale * (Q . K^T) in f32 (k ascending); row max with
 * maximumf from -inf; exp2((s - max) * log2e); row sum (j ascending); p / sum;
 * O = P . V with p truncated to the 16-bit type first, f32 accumulation (key
 * ascending), result truncated to the 16-bit type.  Rows are independent and are
 * spread over threads. */
void oracle_attention_fwd_x16(const uint16_t *Q, const uint16_t *K, const uint16_t *V, uint16_t *O,
                              int64_t heads, int64_t n_ctx, int64_t d_head, float sm_scale,
                              int is_bf16);

/* --- softmax over the last dim ------------------------------------------
 * BENCH  : fill -FLT_MAX; maximumf; x-max; exp; fill 0; sum (in+out); div
 *          (benchmarks/softmax/softmax_gpu.mlir.in:8-42)
 * PLAIDML: fill -inf; cmpf ogt+select; rest the same
 *          (test/PlaidML/OpTest.Softmax.mlir:34-95) */
void oracle_softmax_f32(const float *x, float *y, int64_t rows, int64_t cols,
                        int flavour);

/* --- reductions (addf out,in; ascending index) ------------------------- */
/* y[r] = y[r] + sum_c x[r,c]  (row form: softmax_gpu.mlir.in:32-37) */
void oracle_reduce_rows_f32(const float *x, float *y, int64_t rows,
                            int64_t cols);
/* y[i] = y[i] + sum_l x[l,i]  (leading-dim form: benchmarks/reduce/reduce_gpu.mlir.in:8-18;
 * iteration order is inner index outer loop, l innermost) */
void oracle_reduce_leading_f32(const float *x, float *y, int64_t lead,
                               int64_t inner);
/* *y = *y + sum of everything, row-major order (test/PlaidML/OpTest.Sum.mlir:16-25) */
void oracle_reduce_all_f32(const float *x, float *y, int64_t n);

/* --- transpose ---------------------------------------------------------- */
/* y[j,i] = x[i,j] (benchmarks/transpose/transpose2d_gpu.mlir.in:1-10) */
void oracle_transpose2d_b32(const uint32_t *x, uint32_t *y, int64_t rows,
                            int64_t cols);
void oracle_transpose2d_b16(const uint16_t *x, uint16_t *y, int64_t rows,
                            int64_t cols);
/* rank-3 permutation: y[idx[perm[0]], idx[perm[1]], idx[perm[2]]] = x[idx]
 * (benchmarks/transpose/transpose3d_gpu.mlir.in:1-10) */
void oracle_transpose3d_b32(const uint32_t *x, uint32_t *y, const int64_t *dims,
                            const int *perm);

/* --- seeded synthetic inputs ------------------------------------------- */
/* v[i] = lo + (hi-lo) * u24(seed, first+i), u24 = top 24 bits of
 * splitmix64(first+i + seed*GOLDEN) / 2^24; f32 mul then f32 add.
 * (stands in for the unseeded std::mt19937 fill, ImexRunnerUtils.cpp:38-50) */
void oracle_fill_uniform_f32(float *v, int64_t n, uint64_t seed, int64_t first,
                             float lo, float hi);

/* --- comparison helpers (ImexRunnerUtils.cpp:185-205,217-255) ----------- */
int oracle_allclose_f32(const float *got, const float *ref, int64_t n); /* atol 1e-4, rtol 1e-3 */
double oracle_max_rel_err_f32(const float *got, const float *ref, int64_t n,
                              double floor_abs);
double oracle_rel_frobenius_f32(const float *got, const float *ref, int64_t n);

#ifdef __cplusplus
}
#endif
#endif
