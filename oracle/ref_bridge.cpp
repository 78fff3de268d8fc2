// TEST INFRASTRUCTURE ONLY.  C-callable doors into the reference's own code
// compiled into oracle/_ref/libimex_ref_utils.so: its timing statistics
// (lib/ExecutionEngine/ExecutionEngineUtils/ExecutionEngineUtils.cpp:18-150,
// C++-mangled there) and its CPU GEMM / allclose, which take unranked-memref
// descriptors (lib/ExecutionEngine/ImexRunnerUtils.cpp:185-205,257-338).
#include "imex/ExecutionEngine/ExecutionEngineUtils.h"
#include "imex/ExecutionEngine/ImexRunnerUtils.h"
#include <cstdint>
#include <vector>

namespace {
template <typename T> struct Desc2D {
  T *allocated;
  T *aligned;
  int64_t offset;
  int64_t sizes[2];
  int64_t strides[2];
};
template <typename T> Desc2D<T> rowMajor(T *p, int64_t r, int64_t c) {
  return Desc2D<T>{p, p, 0, {r, c}, {c, 1}};
}
} // namespace

extern "C" {

// which: 0 avg, 1 min, 2 max, 3 median, 4 stddev, 5 variance, 6 P95, 7 P5,
// 8 middle-third average
float ref_stat(int which, const float *v, int64_t n) {
  std::vector<float> x(v, v + n);
  switch (which) {
  case 0: return calculateAverage(x);
  case 1: return calculateMin(x);
  case 2: return calculateMax(x);
  case 3: return calculateMedian(x);
  case 4: return calculateStdDev(x);
  case 5: return calculateVariance(x);
  case 6: return calculateP95(x);
  case 7: return calculateP5(x);
  case 8: return calculateMiddleThirdAverage(x);
  }
  return -1.0f;
}

// C (f32, row-major, M x N) += A (M x K) * B (K x N); kind: 0 bf16, 1 f16
void ref_gemm_x16_f32(const uint16_t *A, const uint16_t *B, float *C,
                      int64_t M, int64_t N, int64_t K, int kind) {
  auto dc = rowMajor<float>(C, M, N);
  UnrankedMemRefType<float> uc{2, &dc};
  if (kind == 0) {
    auto da = rowMajor<bf16>((bf16 *)A, M, K);
    auto db = rowMajor<bf16>((bf16 *)B, K, N);
    UnrankedMemRefType<bf16> ua{2, &da}, ub{2, &db};
    _mlir_ciface_gemmBF16BF16F32(&ua, &ub, &uc);
  } else {
    auto da = rowMajor<f16>((f16 *)A, M, K);
    auto db = rowMajor<f16>((f16 *)B, K, N);
    UnrankedMemRefType<f16> ua{2, &da}, ub{2, &db};
    _mlir_ciface_gemmF16F16F32(&ua, &ub, &uc);
  }
}

int ref_allclose_f32(const float *got, const float *ref, int64_t n) {
  auto dg = rowMajor<float>((float *)got, 1, n);
  auto dr = rowMajor<float>((float *)ref, 1, n);
  UnrankedMemRefType<float> ug{2, &dg}, ur{2, &dr};
  return _mlir_ciface_allcloseF32(&ug, &ur) ? 1 : 0;
}
}
