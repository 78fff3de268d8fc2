// A reader for the subset of MLIR's textual form that the reference's
// hot-path programs use (func / arith / math / tensor / linalg / scf, see
// benchmarks/*/*.mlir.in, test/PlaidML/OpTest.{Matmul,GEMM_FLOAT32,Softmax,
// Sum,Transpose,Relu}.mlir).  It stands where imex-opt's parser stands in the
// reference (tools/imex-opt/imex-opt.cpp:35-49): it produces the in-memory
// form the recogniser works on.  Anything outside the subset is a parse
// error naming the line — never a silent skip.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace imex {
namespace fe {

struct ParseError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct Type {
  enum Kind { None, Scalar, Tensor, MemRef } kind = None;
  std::string elt;             // f32, bf16, f16, f64, i1, i8, i32, i64, index
  std::vector<int64_t> shape;  // static dims; -1 = dynamic
  bool unranked = false;       // tensor<*xf32>
  bool isShaped() const { return kind == Tensor || kind == MemRef; }
  int64_t count() const {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
  std::string str() const;
};

// One result of an affine map.  The hot-path kernels only take a loop dimension or a
// constant (`simple`); anything else (d1 + d3, d1 floordiv 3, 2 * d0 ...) keeps its text as
// a C expression over d0, d1, ... for the loop-nest kernels and matches no recognised op
// (value = -1).
struct MapResult {
  bool isConst = false;
  int64_t value = 0;     // dimension index or the constant; -1 when not simple
  bool simple = true;
  std::string expr;      // C expression over d0.. (always set)
  int shiftDim = -1;     // "d<shiftDim> + shift" (a dimension moved by a constant): not simple,
  int64_t shift = 0;     // but still one-to-one
};
struct AffineMap {
  int numDims = 0;
  std::vector<MapResult> results;
  bool isIdentity() const;
  std::string str() const;
};

struct Op;
struct Block {
  std::vector<std::string> args;
  std::vector<Type> argTypes;
  std::vector<std::unique_ptr<Op>> ops;
};

struct Op {
  std::string name;                   // "linalg.generic", "arith.constant", ...
  int line = 0;
  std::vector<std::string> results;   // "%0" (a "%4:2" definition gives %4#0, %4#1)
  std::vector<Type> resultTypes;
  std::vector<std::string> operands;  // generic operand list (order of appearance)
  std::vector<Type> operandTypes;
  // linalg structured ops
  std::vector<std::string> ins, outs;
  std::vector<Type> insTypes, outsTypes;
  std::vector<AffineMap> maps;
  std::vector<std::string> iterators;  // "parallel" / "reduction"
  std::unique_ptr<Block> body;         // region of linalg.generic / scf.for; "then" region of scf.if
  std::unique_ptr<Block> elseBody;     // "else" region of scf.if; "do" region of scf.while (body: "before")
  // arith.constant
  bool hasDense = false;
  bool denseSplat = false;
  std::vector<double> numbers;         // scalar value, splat value or dense payload (row-major)
  std::vector<uint64_t> rawBits;       // hex literals keep their bits (0xFF800000)
  std::vector<bool> isRaw;
  // call / cmpf / misc
  std::string callee;                  // "@printMemrefF32"; gpu.launch_func: "@module::@kernel"
  std::string text;                    // vector.print str "..."
  std::string predicate;               // cmpf / cmpi predicate
  int64_t intAttr = 0;                 // linalg.index dimension
  std::vector<Type> bodyOperandTypes;  // per operand of a scalar op, when the syntax gives them
  std::vector<std::vector<int64_t>> reassociation;  // expand/collapse_shape
  std::vector<std::string> iterArgs, iterInits;     // scf.for iter_args
};

struct Function {
  std::string name;  // "@main"
  bool isDeclaration = false;
  std::vector<std::string> args;
  std::vector<Type> argTypes;
  std::vector<Type> resultTypes;
  Block body;
};

// shard.grid @name(shape = 4): a grid of processes arrays are split over
// (test/Dialect/NDArray/Extensions/sharding_propagation.mlir:4)
struct Grid {
  std::string name;
  std::vector<int64_t> shape;
};

// A gpu.func inside a gpu.module: its signature and the text of its body.  The body is
// device code of another dialect (XeGPU in the reference's integration tests); it is kept as
// text for the kernel recogniser (gpu_kernels.h), not parsed into operations.
struct GpuKernel {
  std::string module, name;  // "@test_kernel", "@test_kernel"
  std::vector<std::string> args;
  std::vector<Type> argTypes;
  std::string body;
  int line = 0;
};

struct Module {
  std::string name;
  std::vector<Function> functions;
  std::vector<Grid> grids;
  std::vector<GpuKernel> gpuKernels;
  const Function *find(const std::string &symbol) const;
};

Module parseModule(const std::string &text);
Type parseTypeString(const std::string &text);

} // namespace fe
} // namespace imex
