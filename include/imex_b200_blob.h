/* Kernel-descriptor blob: what gpuModuleLoad receives on the B200 path.
 *
 * In the reference the `gpu.binary` attribute of a gpu.module holds a
 * serialised SPIR-V module (lib/Transforms/SerializeSPIRV.cpp:64-69,
 * include/imex/Utils/GPUSerialize.h:15) that Level Zero JIT-compiles in
 * gpuModuleLoad (lib/ExecutionEngine/LEVELZERORUNTIME/LevelZeroRuntimeWrappers.cpp:396-432).
 * Here the same slot holds a table of descriptors, one per outlined kernel:
 * which hot-path op the kernel is, its element types, its static shape and
 * its fused epilogue.  Kernel arguments are bare pointers with no shape
 * (lib/Conversion/GPUXToLLVM/GPUXToLLVMPass.cpp:571-584), so the shape has to
 * travel here.  The outlined kernel NAME is not semantic (`test_kernel`,
 * `test_kernel_0`, ...): gpuKernelGet only uses it to pick the table row.
 *
 * Layout (little endian, no padding beyond what the structs show):
 *   ImexBlobHeader, then num_kernels * ImexKernelDesc, then an optional payload
 *   (kernel text of IMEX_OP_LOOPNEST descriptors, addressed by offset).
 * The magic can never be mistaken for SPIR-V (0x07230203); a blob without it
 * is rejected through the library's error convention.
 */
#ifndef IMEX_B200_BLOB_H
#define IMEX_B200_BLOB_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IMEX_BLOB_MAGIC 0x0030303242584D49ULL /* "IMXB200\0" */
#define IMEX_BLOB_VERSION 1u
#define IMEX_KERNEL_NAME_MAX 64

/* Hot-path ops.  Argument order of each (all bare device pointers, in the
 * order the launch passes them; trailing scalar params the lowering adds for
 * loop bounds are ignored):
 *   GEMM            A[M,K], B[K,N], C[M,N] (, bias[N] when IMEX_FLAG_BIAS)
 *                   dims = {M, N, K, lda, ldb, ldc}; row pitches in elements, 0 = dense
 *                   (memref strides are static in the IR, so they travel here too);
 *                   C = (C when IMEX_FLAG_ACCUMULATE else 0) + A.B, then + bias,
 *                   then epilogue.  IMEX_FLAG_TRANS_A: A is stored [K,M] (C = A^T.B);
 *                   IMEX_FLAG_TRANS_B: B is stored [N,K] (C = A.B^T); pitches are
 *                   those of the arrays as stored.  out_dtype F32, or BF16 / F16:
 *                   f32 accumulation, one rounding to 16 bits at the end (the
 *                   f16-result GEMMs of test/Integration/Dialect/XeGPU/WG/
 *                   gemm_4kx4kx4k_f16_f16_f16.mlir; operand layouts of
 *                   gemm_4kx4kx4k_transpose_{a,b}.mlir)
 *   SOFTMAX         X[rows,cols], Y[rows,cols]           dims = {rows, cols}
 *   REDUCE_ROWS     X[rows,cols], Y[rows]                dims = {rows, cols}
 *                   Y[r] = (Y[r] when ACCUMULATE else 0) + sum_c X[r,c]
 *   REDUCE_LEADING  X[lead,inner], Y[inner]              dims = {lead, inner}
 *   REDUCE_ALL      X[n], Y[1]                           dims = {n}
 *   TRANSPOSE2D     X[rows,cols], Y[cols,rows]           dims = {rows, cols}
 *   TRANSPOSE3D     X[d0,d1,d2], Y[permuted]             dims = {d0,d1,d2,p0,p1,p2}
 *   ELTWISE         X[n], Y[n] with `epilogue` applied   dims = {n}
 *                   (in_dtype != out_dtype: arith.extf / arith.truncf, no epilogue)
 *   EXPR            X0 .. X(k-1), Y: a chain of elementwise generics fused into one pass
 *                   (benchmarks/kLoopFusion/kLoopFusion.mlir.in:4-30).  dims = {rows, cols,
 *                   p0, p1, p2, p3}: the four p words hold up to 32 bytes of postfix
 *                   program (ImexExprCode, little endian, first byte = lowest byte of p0,
 *                   IMEX_X_END-terminated when shorter).  Inputs are full [rows,cols]
 *                   tensors, row vectors [cols] or column vectors [rows], as the push
 *                   opcode says; all of in_dtype.  Every operation rounds to in_dtype
 *                   (f16/bf16 arithmetic is extend - operate in f32 - truncate, per
 *                   operation, as the reference's CPU lowering of 16-bit float ops does).
 *                   IMEX_FLAG_REDUCE_LEADING: Y[cols] = (Y when ACCUMULATE else 0) +
 *                   sum over rows, ascending, of the expression (the elementwise chain
 *                   feeding a column reduce, benchmarks/kInputFusion/kInputFusion.mlir.in:
 *                   6-41); otherwise Y[rows,cols] of out_dtype.
 *   ATTENTION_FWD   Q, K, V, O: [heads * n_ctx, d_head] f16 or bf16, heads one after the
 *                   other; dims = {heads, n_ctx, d_head}; fparams[0] = sm_scale;
 *                   O = softmax(sm_scale * Q K^T) V per head, f32 accumulation
 *                   (test/Integration/Dialect/XeGPU/WG/flash_attention_fwd.mlir:254-330)
 *   LOOPNEST        any other linalg.generic, lowered the way the reference's pipeline lowers
 *                   every linalg op (benchmarks/pipelines/linalg-to-gpu.pp:3-47): a loop nest
 *                   whose parallel loops are mapped to threads and whose reduction loops run
 *                   serially per thread.  The kernel is CUDA C++ text in the blob's payload
 *                   (one `extern "C" __global__ void imex_loopnest(...)`, see
 *                   csrc/frontend/loopnest.h), compiled for sm_100a at first launch, as the
 *                   reference's runtime compiles SPIR-V when a module is loaded.
 *                   dims = {threads, payload offset from the start of the blob, payload
 *                   bytes (text without NUL), number of pointer arguments}; pointers = the
 *                   tensor inputs in order, then the outputs.
 *   FILL_UNIFORM    Y[n]  dims = {n, seed, first}; fparams = {lo, hi}
 *   FILL_NORMAL     Y[n]  dims = {n, seed, first}; fparams = {mean, stddev}
 */
enum ImexOp {
  IMEX_OP_GEMM = 1,
  IMEX_OP_SOFTMAX = 2,
  IMEX_OP_REDUCE_ROWS = 3,
  IMEX_OP_REDUCE_LEADING = 4,
  IMEX_OP_REDUCE_ALL = 5,
  IMEX_OP_TRANSPOSE2D = 6,
  IMEX_OP_TRANSPOSE3D = 7,
  IMEX_OP_ELTWISE = 8,
  IMEX_OP_FILL_UNIFORM = 9,
  IMEX_OP_FILL_NORMAL = 10,
  IMEX_OP_EXPR = 11,
  IMEX_OP_ATTENTION_FWD = 12,
  IMEX_OP_LOOPNEST = 13
};

/* Postfix code of IMEX_OP_EXPR.  Pushes take the element of input k at the current
 * (row, col); unary operations replace the top of the stack, binary ones pop b then a
 * and push a (op) b.  The stack holds at most IMEX_EXPR_MAX_STACK values. */
enum ImexExprCode {
  IMEX_X_END = 0,
  IMEX_X_IN = 1,    /* +k, k = 0..3: X_k[row, col]                    */
  IMEX_X_ROWV = 5,  /* +k: X_k[col]   (one value per column)          */
  IMEX_X_COLV = 9,  /* +k: X_k[row]   (one value per row)             */
  IMEX_X_C0 = 13,   /* fparams[0] */
  IMEX_X_C1 = 14,   /* fparams[1] */
  IMEX_X_ZERO = 15,
  IMEX_X_ONE = 16,
  IMEX_X_NEG = 32,
  IMEX_X_ABS = 33,
  IMEX_X_LOG = 34,
  IMEX_X_EXP = 35,
  IMEX_X_SQRT = 36,
  IMEX_X_RSQRT = 37,
  IMEX_X_TANH = 38,
  IMEX_X_RELU = 39, /* select(cmpf ugt x, 0 ; x, 0) */
  IMEX_X_ADD = 64,
  IMEX_X_SUB = 65,
  IMEX_X_MUL = 66,
  IMEX_X_DIV = 67,
  IMEX_X_MAX = 68,  /* arith.maximumf: NaN if either is NaN */
  IMEX_X_MIN = 69
};
#define IMEX_EXPR_MAX_CODE 32
#define IMEX_EXPR_MAX_INPUTS 4
#define IMEX_EXPR_MAX_STACK 8

enum ImexDType { IMEX_F32 = 1, IMEX_BF16 = 2, IMEX_F16 = 3, IMEX_I32 = 4 };

/* relu: cmpf ugt x,0 ; select x,0   (benchmarks/relu/relu_gpu.mlir.in:6-11)
 * silu: x * 1/(exp(-x)+1)           (benchmarks/silu/silu_gpu.mlir.in:6-18) */
enum ImexEpilogue { IMEX_EPI_NONE = 0, IMEX_EPI_RELU = 1, IMEX_EPI_SILU = 2 };

enum ImexFlags {
  IMEX_FLAG_ACCUMULATE = 1u << 0, /* output is read as the initial value */
  IMEX_FLAG_BIAS = 1u << 1,       /* GEMM: 4th pointer is bias[N] (f32)   */
  IMEX_FLAG_SOFTMAX_NEG_INF = 1u << 2, /* PlaidML form: max starts at -inf, cmpf ogt */
  IMEX_FLAG_TRANS_A = 1u << 3,    /* GEMM: A stored [K,M]                 */
  IMEX_FLAG_TRANS_B = 1u << 4,    /* GEMM: B stored [N,K]                 */
  IMEX_FLAG_REDUCE_LEADING = 1u << 5 /* EXPR: sum the expression over the rows */
};

typedef struct ImexBlobHeader {
  uint64_t magic;
  uint32_t version;
  uint32_t num_kernels;
} ImexBlobHeader;

typedef struct ImexKernelDesc {
  char name[IMEX_KERNEL_NAME_MAX]; /* NUL-terminated outlined kernel name */
  uint32_t op;                     /* ImexOp */
  uint32_t in_dtype;               /* ImexDType of the inputs */
  uint32_t out_dtype;              /* ImexDType of the output */
  uint32_t epilogue;               /* ImexEpilogue */
  uint32_t flags;                  /* ImexFlags */
  uint32_t sm_margin;              /* GEMM: SMs left free for a collective running beside it */
  int64_t dims[6];
  float fparams[2];
} ImexKernelDesc;

#ifdef __cplusplus
}
#endif
#endif
