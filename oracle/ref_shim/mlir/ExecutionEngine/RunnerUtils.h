/* Stand-in for the upstream MLIR header of the same name (not part of the
 * reference tree).  TEST INFRASTRUCTURE ONLY.  The reference source only
 * needs impl::printMemRef to exist; oracle/_ref is used for its GEMM and
 * comparison helpers, so the printer here is a plain row-major dump. */
#ifndef IMEX_B200_SHIM_RUNNERUTILS_H
#define IMEX_B200_SHIM_RUNNERUTILS_H

#include "mlir/ExecutionEngine/CRunnerUtils.h"
#include "mlir/ExecutionEngine/Float16bits.h"
#include <iostream>

namespace impl {
inline float shimToFloat(float v) { return v; }
inline float shimToFloat(bf16 v) { return oracle_bf16_to_f32(v.bits); }
inline float shimToFloat(f16 v) { return oracle_f16_to_f32(v.bits); }

template <typename T> void printMemRef(UnrankedMemRefType<T> &m) {
  DynamicMemRefType<T> d(m);
  std::cout << "Unranked Memref rank = " << d.rank << " data = [";
  bool first = true;
  for (auto it = d.begin(); it != d.end(); ++it) {
    std::cout << (first ? "" : ", ") << shimToFloat(*it);
    first = false;
  }
  std::cout << "]\n";
}
} // namespace impl

#endif
