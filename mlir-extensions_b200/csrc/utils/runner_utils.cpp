// Host runner utilities: see include/imex_runner_utils.h for the reference
// files each function follows.  Pure host code, no CUDA.
#include "../../../include/imex_runner_utils.h"

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <limits>
#include <random>
#include <vector>

namespace {

// ---- 16-bit floats ----------------------------------------------------------
float bf16ToF32(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
uint16_t f32ToBf16(float v) {
  uint32_t u;
  std::memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
float f16ToF32(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      u = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
uint16_t f32ToF16(float v) {
  uint32_t u;
  std::memcpy(&u, &v, 4);
  const uint16_t sign = static_cast<uint16_t>((u >> 16) & 0x8000u);
  const uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return sign | 0x7e00u;
  if (a >= 0x47800000u) return sign | 0x7c00u;
  if (a < 0x33000000u) return sign;
  const int32_t e = static_cast<int32_t>(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u, base = 0;
  int shift = 13;
  if (e < -14) {
    shift += -14 - e;
  } else {
    base = static_cast<uint32_t>(e + 15) << 10;
    m &= 0x7fffffu;
  }
  uint32_t q = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  uint32_t r = base + q;
  if (r > 0x7c00u) r = 0x7c00u;
  return sign | static_cast<uint16_t>(r);
}

struct BF16 { uint16_t bits; };
struct F16 { uint16_t bits; };
template <typename T> float toFloat(T v) { return static_cast<float>(v); }
template <> float toFloat<BF16>(BF16 v) { return bf16ToF32(v.bits); }
template <> float toFloat<F16>(F16 v) { return f16ToF32(v.bits); }
template <typename T> T fromFloat(float v) { return static_cast<T>(v); }
template <> BF16 fromFloat<BF16>(float v) { return BF16{f32ToBf16(v)}; }
template <> F16 fromFloat<F16>(float v) { return F16{f32ToF16(v)}; }

// ---- strided view of an unranked memref -----------------------------------
template <typename T> struct View {
  int64_t rank;
  T *data;
  int64_t offset;
  const int64_t *sizes;
  const int64_t *strides;

  explicit View(const ImexUnrankedMemRef &u) : rank(u.rank) {
    auto **ptrs = static_cast<T **>(u.descriptor);
    data = ptrs[1];
    const auto *ints = reinterpret_cast<const int64_t *>(ptrs + 2);
    offset = ints[0];
    sizes = ints + 1;
    strides = ints + 1 + rank;
  }
  int64_t count() const {
    int64_t n = 1;
    for (int64_t d = 0; d < rank; ++d) n *= sizes[d];
    return n;
  }
  // element at row-major linear position i
  T &at(int64_t i) const {
    int64_t pos = offset;
    for (int64_t d = rank - 1; d >= 0; --d) {
      pos += (i % sizes[d]) * strides[d];
      i /= sizes[d];
    }
    return data[pos];
  }
};

// ---- printing (format of the upstream runner-utils memref printer, as pinned
//      by the CHECK lines of the reference's tests) --------------------------
template <typename T> void printValue(T v) {
  if constexpr (sizeof(T) == 1)
    std::cout << static_cast<int>(v);
  else
    std::cout << v;
}
template <> void printValue<BF16>(BF16 v) { std::cout << toFloat(v); }
template <> void printValue<F16>(F16 v) { std::cout << toFloat(v); }

template <typename T>
void printRec(const View<T> &v, int64_t dim, int64_t pos) {
  if (dim == v.rank) {
    printValue(v.data[pos]);
    return;
  }
  std::cout << "[";
  for (int64_t i = 0; i < v.sizes[dim]; ++i) {
    if (i) {
      if (dim == v.rank - 1) {
        std::cout << ",   ";
      } else {
        std::cout << ", \n";
        for (int64_t s = 0; s <= dim; ++s) std::cout << " ";
      }
    }
    printRec(v, dim + 1, pos + i * v.strides[dim]);
  }
  std::cout << "]";
}

template <typename T> void printMemref(ImexUnrankedMemRef *m) {
  View<T> v(*m);
  std::cout << "Unranked Memref base@ = " << static_cast<const void *>(v.data) << " rank = " << v.rank
            << " offset = " << v.offset << " sizes = [";
  for (int64_t d = 0; d < v.rank; ++d) std::cout << (d ? ", " : "") << v.sizes[d];
  std::cout << "] strides = [";
  for (int64_t d = 0; d < v.rank; ++d) std::cout << (d ? ", " : "") << v.strides[d];
  std::cout << "] data = \n";
  if (v.rank == 0) {
    std::cout << "[";
    printValue(v.data[v.offset]);
    std::cout << "]";
  } else {
    printRec(v, 0, v.offset);
  }
  std::cout << "\n";
  std::cout.flush();
}

// ---- fills --------------------------------------------------------------
template <typename T> void fill(ImexUnrankedMemRef *m, float value) {
  View<T> v(*m);
  const T x = fromFloat<T>(value);
  for (int64_t i = 0, n = v.count(); i < n; ++i) v.at(i) = x;
}

std::mt19937 &generator() {
  static std::mt19937 gen = [] {
    if (const char *s = std::getenv("IMEX_FILL_SEED"))
      return std::mt19937(static_cast<uint32_t>(std::strtoul(s, nullptr, 10)));
    std::random_device rd;
    return std::mt19937(rd());
  }();
  return gen;
}

template <typename T> void fillRandom(ImexUnrankedMemRef *m, float lower, float upper, bool genInt) {
  View<T> v(*m);
  std::uniform_real_distribution<> dist(lower, upper);
  auto &gen = generator();
  for (int64_t i = 0, n = v.count(); i < n; ++i) {
    const double x = dist(gen);
    v.at(i) = fromFloat<T>(static_cast<float>(genInt ? static_cast<double>(static_cast<int>(x)) : x));
  }
}

// ---- comparisons ------------------------------------------------------------
template <typename T> bool allclose(ImexUnrankedMemRef *m, ImexUnrankedMemRef *ref) {
  const float atol = 1e-04f, rtol = 1e-03f;
  View<T> a(*m);
  View<float> b(*ref);
  const int64_t n = std::min(a.count(), b.count());
  for (int64_t i = 0; i < n; ++i) {
    const float lhs = toFloat(a.at(i)), rhs = b.at(i);
    if (std::fabs(lhs - rhs) > atol + rtol * std::fabs(rhs)) return false;
  }
  return true;
}

template <typename T> void printAllclose(ImexUnrankedMemRef *m, ImexUnrankedMemRef *ref) {
  std::cout << (allclose<T>(m, ref) ? "[ALLCLOSE: TRUE]\n" : "[ALLCLOSE: FALSE]\n");
  std::cout.flush();
}

template <typename T> void printMaxError(ImexUnrankedMemRef *m, ImexUnrankedMemRef *n) {
  View<T> a(*m), b(*n);
  const int64_t cnt = std::min(a.count(), b.count());
  const double inf = std::numeric_limits<double>::infinity();
  double maxAbs = 0.0, maxRel = 0.0, absI = inf, absJ = inf, relI = inf, relJ = inf;
  int64_t absAt = 0, relAt = 0;
  for (int64_t i = 0; i < cnt; ++i) {
    const double x = toFloat(a.at(i)), y = toFloat(b.at(i));
    const double delta = std::fabs(x - y);
    const double rel = delta / std::fmax(std::fabs(x), std::fabs(y));
    if (delta > maxAbs) { maxAbs = delta; absAt = i; absI = x; absJ = y; }
    if (rel > maxRel) { maxRel = rel; relAt = i; relI = x; relJ = y; }
  }
  std::cout << "Max absolute error " << maxAbs << " at idx=" << absAt << " (i=" << absI
            << ", j=" << absJ << ")\n";
  std::cout << "Max relative error " << maxRel << " at idx=" << relAt << " (i=" << relI
            << ", j=" << relJ << ")\n";
  std::cout.flush();
}

// ---- host GEMM ------------------------------------------------------------
template <typename AB, typename COut>
void gemm(ImexUnrankedMemRef *A, ImexUnrankedMemRef *B, ImexUnrankedMemRef *C) {
  View<AB> a(*A), b(*B);
  View<float> c(*C);
  if (a.rank != 2 || b.rank != 2 || c.rank != 2) {
    std::cout << "Expecting 2D memrefs, got A rank: " << a.rank << ", B rank: " << b.rank
              << ", C rank: " << c.rank << '\n';
    return;
  }
  if (a.sizes[1] != b.sizes[0] || a.sizes[0] != c.sizes[0] || b.sizes[1] != c.sizes[1]) {
    std::cout << "Incompatible matrix dimensions: A: [" << a.sizes[0] << ", " << a.sizes[1]
              << "], B: [" << b.sizes[0] << ", " << b.sizes[1] << "], C: [" << c.sizes[0] << ", "
              << c.sizes[1] << "]\n";
    return;
  }
  const int64_t M = a.sizes[0], K = a.sizes[1], N = b.sizes[1];
  std::vector<float> fa(static_cast<size_t>(M * K)), fb(static_cast<size_t>(K * N)),
      fc(static_cast<size_t>(M * N));
  for (int64_t i = 0; i < M * K; ++i) fa[i] = toFloat(a.at(i));
  for (int64_t i = 0; i < K * N; ++i) fb[i] = toFloat(b.at(i));
  for (int64_t i = 0; i < M * N; ++i) fc[i] = c.at(i);
  for (int64_t i = 0; i < M; ++i)
    for (int64_t k = 0; k < K; ++k) {
      const float x = fa[i * K + k];
      for (int64_t j = 0; j < N; ++j) {
        const float p = x * fb[k * N + j];
        fc[i * N + j] = fc[i * N + j] + p;
      }
    }
  for (int64_t i = 0; i < M * N; ++i) {
    float r = fc[i];
    if constexpr (!std::is_same_v<COut, float>) r = toFloat(fromFloat<COut>(r));
    c.at(i) = r;
  }
}

template <typename T> void printRanked(int64_t rank, void *descriptor) {
  ImexUnrankedMemRef u{rank, descriptor};
  printMemref<T>(&u);
}

} // namespace

extern "C" {

void _mlir_ciface_fillResource1DBF16(ImexUnrankedMemRef *m, float v) { fill<BF16>(m, v); }
void _mlir_ciface_fillResource1DF16(ImexUnrankedMemRef *m, float v) { fill<F16>(m, v); }
void _mlir_ciface_fillResource1DF32(ImexUnrankedMemRef *m, float v) { fill<float>(m, v); }
void _mlir_ciface_fillResource1DRandomBF16(ImexUnrankedMemRef *m, float lo, float hi, bool gi) {
  fillRandom<BF16>(m, lo, hi, gi);
}
void _mlir_ciface_fillResource1DRandomF16(ImexUnrankedMemRef *m, float lo, float hi, bool gi) {
  fillRandom<F16>(m, lo, hi, gi);
}
void _mlir_ciface_fillResource1DRandomF32(ImexUnrankedMemRef *m, float lo, float hi, bool gi) {
  fillRandom<float>(m, lo, hi, gi);
}
void _mlir_ciface_printMemrefBF16(ImexUnrankedMemRef *m) { printMemref<BF16>(m); }
void _mlir_ciface_printMemrefF16(ImexUnrankedMemRef *m) { printMemref<F16>(m); }
void printMemrefBF16(int64_t rank, void *d) { printRanked<BF16>(rank, d); }
void printMemrefF16(int64_t rank, void *d) { printRanked<F16>(rank, d); }
bool _mlir_ciface_allcloseBF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *r) { return allclose<BF16>(m, r); }
bool _mlir_ciface_allcloseF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *r) { return allclose<F16>(m, r); }
bool _mlir_ciface_allcloseF32(ImexUnrankedMemRef *m, ImexUnrankedMemRef *r) { return allclose<float>(m, r); }
void _mlir_ciface_printAllcloseBF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *r) { printAllclose<BF16>(m, r); }
void _mlir_ciface_printAllcloseF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *r) { printAllclose<F16>(m, r); }
void _mlir_ciface_printAllcloseF32(ImexUnrankedMemRef *m, ImexUnrankedMemRef *r) { printAllclose<float>(m, r); }
void _mlir_ciface_printMaxErrorBF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *n) { printMaxError<BF16>(m, n); }
void _mlir_ciface_printMaxErrorF16(ImexUnrankedMemRef *m, ImexUnrankedMemRef *n) { printMaxError<F16>(m, n); }
void _mlir_ciface_printMaxErrorF32(ImexUnrankedMemRef *m, ImexUnrankedMemRef *n) { printMaxError<float>(m, n); }
void _mlir_ciface_gemmF16F16F16(ImexUnrankedMemRef *a, ImexUnrankedMemRef *b, ImexUnrankedMemRef *c) { gemm<F16, F16>(a, b, c); }
void _mlir_ciface_gemmF16F16F32(ImexUnrankedMemRef *a, ImexUnrankedMemRef *b, ImexUnrankedMemRef *c) { gemm<F16, float>(a, b, c); }
void _mlir_ciface_gemmBF16BF16F32(ImexUnrankedMemRef *a, ImexUnrankedMemRef *b, ImexUnrankedMemRef *c) { gemm<BF16, float>(a, b, c); }

void _mlir_ciface_printMemrefF32(ImexUnrankedMemRef *m) { printMemref<float>(m); }
void _mlir_ciface_printMemrefF64(ImexUnrankedMemRef *m) { printMemref<double>(m); }
void _mlir_ciface_printMemrefI8(ImexUnrankedMemRef *m) { printMemref<int8_t>(m); }
void _mlir_ciface_printMemrefI16(ImexUnrankedMemRef *m) { printMemref<int16_t>(m); }
void _mlir_ciface_printMemrefI32(ImexUnrankedMemRef *m) { printMemref<int32_t>(m); }
void _mlir_ciface_printMemrefI64(ImexUnrankedMemRef *m) { printMemref<int64_t>(m); }
void printMemrefF32(int64_t rank, void *d) { printRanked<float>(rank, d); }
void printMemrefF64(int64_t rank, void *d) { printRanked<double>(rank, d); }
void printMemrefI8(int64_t rank, void *d) { printRanked<int8_t>(rank, d); }
void printMemrefI16(int64_t rank, void *d) { printRanked<int16_t>(rank, d); }
void printMemrefI32(int64_t rank, void *d) { printRanked<int32_t>(rank, d); }
void printMemrefI64(int64_t rank, void *d) { printRanked<int64_t>(rank, d); }

double rtclock(void) {
  using namespace std::chrono;
  return duration<double>(steady_clock::now().time_since_epoch()).count();
}
void printF32(float v) { std::cout << v; std::cout.flush(); }
void printF64(double v) { std::cout << v; std::cout.flush(); }
void printI64(int64_t v) { std::cout << v; std::cout.flush(); }
void printU64(uint64_t v) { std::cout << v; std::cout.flush(); }
void printCString(char *s) { std::cout << s; std::cout.flush(); }
void printOpen(void) { std::cout << "( "; std::cout.flush(); }
void printClose(void) { std::cout << " )"; std::cout.flush(); }
void printComma(void) { std::cout << ", "; std::cout.flush(); }
void printNewline(void) { std::cout << "\n"; std::cout.flush(); }

} // extern "C"
