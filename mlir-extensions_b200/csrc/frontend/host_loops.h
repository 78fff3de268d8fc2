// Host-side loop nests of scalar code over memrefs, compiled to a small register program.
//
// The reference's GPU-dialect integration tests prepare and post-process their arrays on the
// host with scf.for nests of memref.load / arith / memref.store over every element (zero C,
// add the bias to the CPU reference, build a transposed copy: test/Integration/Dialect/XeGPU/WG/
// gemm_4kx4kx4k_f16_f16_f32_bias.mlir:131-150, 161-170) — tens of millions of iterations that a
// tree-walking interpreter with named values would spend minutes on.  compile() resolves every
// value to a register once and run() executes the nest at a few nanoseconds per operation.
// Arithmetic keeps the IR's types: f32 operations round to f32, 16-bit elements are converted
// on load and store, index / integer arithmetic is exact.  Anything other than scalar arith,
// memref.load / store and nested scf.for without iter_args is left to the interpreter.
#pragma once

#include "mlir_text.h"

#include <cstdint>
#include <functional>
#include <string>
#include <vector>

namespace imex {
namespace fe {

struct HostArray {   // a memref the nest touches: host-visible storage and its static shape
  void *data = nullptr;
  std::string elt;
  std::vector<int64_t> shape;
};

class HostLoopProgram {
public:
  // Looks up a value defined outside the nest: returns true and sets `scalar` for a scalar,
  // or fills `array` (data may be null when nothing is to be run, e.g. when only planning).
  using Lookup = std::function<bool(const std::string &name, double &scalar, HostArray &array, bool &isArray)>;

  // False (with `why`) when the loop contains something this compiler does not take.
  bool compile(const Op &forOp, const Lookup &lookup, std::string &why);
  void run();

private:
  enum Code { Const, Add, Sub, Mul, Div, Neg, Max, Min, AddI, SubI, MulI, DivI, RemI, Copy, ToInt, F32, Load, Store, For, End };
  struct Ins {
    Code code;
    int dst = -1, a = -1, b = -1;
    double imm = 0;
    bool f32 = false;        // round the result to f32
    int array = -1;          // Load / Store
    std::vector<int> idx;    // index registers
    int end = -1;            // For: index of the matching End
    int lb = -1, ub = -1, step = -1;
  };
  std::vector<Ins> code;
  std::vector<double> regs;
  std::vector<HostArray> arrays;
  bool block(const Block &b, std::vector<std::pair<std::string, int>> &env, const Lookup &lookup, std::string &why);
  int reg(const std::string &name, std::vector<std::pair<std::string, int>> &env, const Lookup &lookup, std::string &why);
  int arrayOf(const std::string &name, const Lookup &lookup, std::string &why);
  std::vector<std::pair<std::string, int>> arrayIndex;
};

} // namespace fe
} // namespace imex
