// Loop-nest kernels: any linalg.generic that is none of the recognised hot-path ops.
//
// The reference's GPU pipeline turns every linalg op into a loop nest, maps the parallel
// loops to work-items and outlines one kernel per nest, each work-item running the
// reduction loops serially (benchmarks/pipelines/linalg-to-gpu.pp:3-47; the result for a
// matmul is test/SPIRV/OpTest.GEMM_BF16_ACC_F32.mlir:129-140).  This is the same lowering
// written out as CUDA C++ text: one thread per point of the parallel iteration space, the
// reduction dimensions as ascending serial loops around the region's body, every body
// operation evaluated in the IR's element type (f16 / bf16: operate in f32, round after
// every operation; integers wrap).  Per output element the sequence of operations is
// exactly that of linalg-to-loops on the CPU, so exactly-rounded bodies give bit-identical
// results.  The text travels in the kernel blob (IMEX_OP_LOOPNEST) and the runtime
// compiles it for sm_100a when the module is first launched, as the reference's runtime
// compiles SPIR-V at gpuModuleLoad.
#pragma once

#include "mlir_text.h"
#include "recognise.h"

#include <string>
#include <vector>

namespace imex {
namespace fe {

struct LoopNestKernel {
  std::string source;               // one `extern "C" __global__ void imex_loopnest(...)`
  std::vector<int> pointerInputs;   // indices into op.ins passed as pointers, in argument order
                                    // (scalar ins are written into the text as literals)
  std::vector<bool> readsInit;      // per output: the kernel reads the output's initial contents
  std::vector<std::string> captured;  // tensors of the enclosing function the region reads with
                                      // tensor.extract: pointer arguments after the outputs
  int64_t threads = 1;              // points of the parallel iteration space
  std::string summary;              // for plans and diagnostics
};

// False (with `why`) when the op cannot be written as a loop nest: extents still dynamic in
// the types it is given (`types` carries the actual ones when the IR's are dynamic), an
// operation or element type without a C counterpart, an output indexed by a reduction
// dimension, or a parallel dimension missing from an output's map.
// `types`, when given, replaces the operand types written in the op (ins, then outs): the
// shapes the operands actually have here (one rank's rows of a row-sharded array).
bool buildLoopNest(const Op &op, const ConstantTable &constants, LoopNestKernel &out, std::string &why,
                   const std::vector<Type> *types = nullptr);

// tensor.pad with static amounts and a constant padding value (test/PlaidML/CppEdsl.Convolution.mlir:26-29):
// one thread per element of the result, which is the source element at (position - low) or
// the padding value outside the source.
bool buildPad(const Type &src, const Type &dst, const std::vector<int64_t> &low, double value, LoopNestKernel &out,
              std::string &why);

// tensor.extract_slice with static offsets, sizes and strides
// (test/Jax/janet/jit__get_age_weights_from_tables.8_linalg.mlir:60): one thread per element of the result.
bool buildSlice(const Type &src, const Type &dst, const std::vector<int64_t> &offsets, const std::vector<int64_t> &sizes,
                const std::vector<int64_t> &strides, LoopNestKernel &out, std::string &why);

} // namespace fe
} // namespace imex
