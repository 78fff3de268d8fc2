/* Host runner utilities (libimex_runner_utils.so).
 *
 * The functions MLIR test programs call from their entry function: the ones
 * the reference's libimex_runner_utils.so exports
 * (include/imex/ExecutionEngine/ImexRunnerUtils.h:66-134,
 *  lib/ExecutionEngine/ImexRunnerUtils.cpp) plus the upstream
 * mlir_runner_utils / mlir_c_runner_utils symbols its tests use
 * (printMemrefF32, printMemrefI32, rtclock, printF64, printCString,
 * printNewline: benchmarks/softmax/softmax_cpu.mlir.in:5-8,
 * test/PlaidML/OpTest.Matmul.mlir:23).  Same names, same argument meaning.
 *
 * Memrefs arrive as "unranked memref" pairs {rank, descriptor*}; the
 * descriptor is { T *allocated; T *aligned; int64_t offset;
 * int64_t sizes[rank]; int64_t strides[rank]; }
 * (ImexRunnerUtils.h:36-42).  16-bit floats are passed as their bit patterns.
 */
#ifndef IMEX_RUNNER_UTILS_H
#define IMEX_RUNNER_UTILS_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ImexUnrankedMemRef {
  int64_t rank;
  void *descriptor;
} ImexUnrankedMemRef;

/* ImexRunnerUtils.cpp:27-36, 56-76: fill with a constant */
void _mlir_ciface_fillResource1DBF16(ImexUnrankedMemRef *m, float value);
void _mlir_ciface_fillResource1DF16(ImexUnrankedMemRef *m, float value);
void _mlir_ciface_fillResource1DF32(ImexUnrankedMemRef *m, float value);
/* ImexRunnerUtils.cpp:38-50, 78-101: uniform [lower, upper), truncated to an
 * integer when genInt.  The reference seeds from std::random_device; here the
 * environment variable IMEX_FILL_SEED makes the stream reproducible. */
void _mlir_ciface_fillResource1DRandomBF16(ImexUnrankedMemRef *m, float lower, float upper, bool genInt);
void _mlir_ciface_fillResource1DRandomF16(ImexUnrankedMemRef *m, float lower, float upper, bool genInt);
void _mlir_ciface_fillResource1DRandomF32(ImexUnrankedMemRef *m, float lower, float upper, bool genInt);
/* ImexRunnerUtils.cpp:103-119 */
void _mlir_ciface_printMemrefBF16(ImexUnrankedMemRef *m);
void _mlir_ciface_printMemrefF16(ImexUnrankedMemRef *m);
void printMemrefBF16(int64_t rank, void *descriptor);
void printMemrefF16(int64_t rank, void *descriptor);
/* ImexRunnerUtils.cpp:185-215, 340-376: |a-b| <= 1e-4 + 1e-3*|b| elementwise */
bool _mlir_ciface_allcloseBF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *ref);
bool _mlir_ciface_allcloseF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *ref);
bool _mlir_ciface_allcloseF32(ImexUnrankedMemRef *m, ImexUnrankedMemRef *ref);
void _mlir_ciface_printAllcloseBF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *ref);
void _mlir_ciface_printAllcloseF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *ref);
void _mlir_ciface_printAllcloseF32(ImexUnrankedMemRef *m, ImexUnrankedMemRef *ref);
/* ImexRunnerUtils.cpp:217-255, 340-353 */
void _mlir_ciface_printMaxErrorBF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *n);
void _mlir_ciface_printMaxErrorF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *n);
void _mlir_ciface_printMaxErrorF32(ImexUnrankedMemRef *m, ImexUnrankedMemRef *n);
/* ImexRunnerUtils.cpp:257-338, 378-400: host GEMM the reference's tests compare
 * their device result with: C(f32) += A.B with inputs widened to f32, loops
 * i,k,j; the F16F16F16 flavour rounds the result through f16. */
void _mlir_ciface_gemmF16F16F16(ImexUnrankedMemRef *a, ImexUnrankedMemRef *b, ImexUnrankedMemRef *c);
void _mlir_ciface_gemmF16F16F32(ImexUnrankedMemRef *a, ImexUnrankedMemRef *b, ImexUnrankedMemRef *c);
void _mlir_ciface_gemmBF16BF16F32(ImexUnrankedMemRef *a, ImexUnrankedMemRef *b, ImexUnrankedMemRef *c);

/* Upstream runner-utils symbols used by the reference's tests and benchmarks. */
void _mlir_ciface_printMemrefF32(ImexUnrankedMemRef *m);
void _mlir_ciface_printMemrefF64(ImexUnrankedMemRef *m);
void _mlir_ciface_printMemrefI8(ImexUnrankedMemRef *m);
void _mlir_ciface_printMemrefI16(ImexUnrankedMemRef *m);
void _mlir_ciface_printMemrefI32(ImexUnrankedMemRef *m);
void _mlir_ciface_printMemrefI64(ImexUnrankedMemRef *m);
void printMemrefF32(int64_t rank, void *descriptor);
void printMemrefF64(int64_t rank, void *descriptor);
void printMemrefI8(int64_t rank, void *descriptor);
void printMemrefI16(int64_t rank, void *descriptor);
void printMemrefI32(int64_t rank, void *descriptor);
void printMemrefI64(int64_t rank, void *descriptor);
double rtclock(void);
void printF32(float v);
void printF64(double v);
void printI64(int64_t v);
void printU64(uint64_t v);
void printCString(char *s);
void printOpen(void);
void printClose(void);
void printComma(void);
void printNewline(void);

#ifdef __cplusplus
}
#endif
#endif
