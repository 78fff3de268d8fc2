// Recogniser: classifies the linalg ops of a function and groups them into
// the hot-path kernels of the B200 runtime.  It plays the part of the
// reference's GPU pipeline between linalg and the runtime ABI
// (benchmarks/pipelines/linalg-to-gpu.pp:3-47): where that pipeline lowers
// every linalg op to loops, outlines one GPU kernel per loop nest and
// serialises SPIR-V, this one recognises WHICH op (or chain of ops) a piece of
// IR is and emits a kernel descriptor for it.  The numeric contract is the
// IR's: the tensor-core GEMM is chosen only for 16-bit inputs extended to f32
// with an f32 multiply-add; an f16 multiply-add is not (it would round
// differently) and is rejected.  IR that matches nothing is an error — there
// is no CPU fallback.
#pragma once

#include "mlir_text.h"

#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

namespace imex {
namespace fe {

enum class Kind {
  Unknown,
  Matmul,        // C[d0,d1] += A[d0,d2] * B[d2,d1]   (named op or generic; transA / transB:
                 // A indexed [d2,d0] / B indexed [d1,d2], linalg.matmul_transpose_a / _b)
  Add,           // elementwise x + y
  BroadcastRow,  // out[i,j] = v[j]   (the bias broadcast in front of an Add)
  Relu,          // select(cmpf ugt x, 0 ; x, 0)
  Sigmoid,       // 1 / (exp(-x) + 1)
  Mul,           // elementwise x * y
  RowMax,        // running max over the last dim (maxf / maximumf / cmpf ogt + select)
  SubRowBcast,   // x[i,j] - v[i,0]
  Exp,
  RowSum,        // sum over the last dim
  DivRowBcast,   // x[i,j] / v[i,0]
  Transpose,     // pure permutation
  ReduceLeading, // sum over the leading dim
  ReduceAll,     // sum of everything
  ExtF,          // 16-bit -> f32
  TruncF,        // f32 -> 16-bit
  Elementwise,   // any other supported elementwise body (see classifyElementwise)
  Fill
};

const char *kindName(Kind k);

struct Classified {
  Kind kind = Kind::Unknown;
  std::string expr;           // canonical form of the body, for diagnostics
  bool rowMaxOgt = false;     // RowMax written as cmpf ogt + select (init -inf form)
  bool transA = false;        // Matmul: A is stored [K,M]
  bool transB = false;        // Matmul: B is stored [N,K]
  std::vector<int> perm;      // Transpose: output dim i = input dim perm[i]
  std::string why;            // reason when Unknown
};

// Any all-parallel generic whose body is a tree of the operations the fused
// elementwise kernel knows (IMEX_OP_EXPR) and whose operands are read at the loop
// point itself, as a row vector ((d0,d1)->(d1)) or as a column vector
// ((d0,d1)->(d0) / (d0,0)).  Chains of these fuse into one launch
// (benchmarks/kLoopFusion/kLoopFusion.mlir.in:4-30).
struct ExprTree {
  enum { Input, Const, Unary, Binary } kind = Input;
  int index = 0;     // Input: which operand
  double value = 0;  // Const
  int opcode = 0;    // Unary / Binary: ImexExprCode
  std::shared_ptr<ExprTree> a, b;
};
struct ElementwiseInfo {
  std::string expr;            // canonical body expression over in0.. and c(value)
  std::vector<int> inputMode;  // per input: 0 = full tensor, 1 = row vector, 2 = column vector
  std::shared_ptr<ExprTree> tree;
};
// Tree of a canonical body expression; null when it uses anything the fused kernel lacks.
std::shared_ptr<ExprTree> parseElementwiseExpr(const std::string &expr);

// Scalar constants visible to linalg bodies: SSA name -> value.
using ConstantTable = std::map<std::string, double>;

Classified classify(const Op &op, const ConstantTable &constants);
bool classifyElementwise(const Op &op, const ConstantTable &constants, ElementwiseInfo &info);

} // namespace fe
} // namespace imex
