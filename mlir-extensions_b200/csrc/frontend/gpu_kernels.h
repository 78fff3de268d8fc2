// Recognition of hand-written GPU-dialect kernels.
//
// The reference's XeGPU integration tests (test/Integration/Dialect/XeGPU/WG/gemm_*.mlir,
// simple_gemm.mlir) carry their device code as a gpu.func of XeGPU-dialect operations and
// drive it from host code with gpu.alloc / gpu.memcpy / gpu.launch_func.  That device code
// cannot be compiled for sm_100; what CAN be served is the operation it performs.  The
// recogniser reads the gpu.func's signature and follows the data flow of its body text —
// which kernel arguments reach the A, B and accumulator operands of `xegpu.dpas`, which one
// the result is stored to, whether an operand passes a `vector.transpose`, whether a rank-1
// f32 argument is added to the result — and, if that makes a matrix product, describes it as
// a GEMM descriptor of the runtime.  Anything else is refused by name.
#pragma once

#include "mlir_text.h"

#include <string>

namespace imex {
namespace fe {

struct GpuGemm {
  int a = -1, b = -1, c = -1, bias = -1;  // indices into the gpu.func's arguments
  bool transA = false, transB = false;    // A is stored [K,M] / B is stored [N,K]
  bool readsC = false;                    // the accumulator starts from C's contents
  int64_t M = 0, N = 0, K = 0;
};

bool recogniseGpuGemm(const GpuKernel &k, GpuGemm &out, std::string &why);

} // namespace fe
} // namespace imex
