// Fused elementwise chains compiled at first use.
//
// The reference compiles its kernels when a module is first loaded (SPIR-V handed to
// the driver's JIT, lib/ExecutionEngine/LEVELZERORUNTIME/LevelZeroRuntimeWrappers.cpp:
// 402-431).  The expression programs of IMEX_OP_EXPR get the same treatment: the postfix
// code is turned into straight-line CUDA C++ inside a fixed, hand-written kernel frame
// (128-bit loads and stores, four or eight elements per thread), compiled for sm_100a
// with NVRTC, loaded through the driver API and cached per (device, program, types).
// NVRTC and the driver entry points are looked up at run time; when either is missing
// or a compilation fails, the caller uses the interpreting kernel in eltwise_expr.cu
// instead (same arithmetic, same results, slower).
//
// Arithmetic is that of eltwise_expr.cu: every operation in f32, rounded to the element
// type after every operation, no contraction.
#include "jit_common.h"
#include "kernels.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

namespace imex {
namespace {

// ---- source generation -----------------------------------------------------------------
const char *kPrelude = R"SRC(
typedef unsigned short u16;
__device__ __forceinline__ float h2f(u16 h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
__device__ __forceinline__ u16 f2h(float f) { u16 h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
__device__ __forceinline__ float b2f(u16 h) { return __uint_as_float(((unsigned)h) << 16); }
__device__ __forceinline__ u16 f2b(float f) { u16 h; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
__device__ __forceinline__ float maximumf(float a, float b) { return a != a ? a : (b != b ? b : fmaxf(a, b)); }
__device__ __forceinline__ float minimumf(float a, float b) { return a != a ? a : (b != b ? b : fminf(a, b)); }
__device__ __forceinline__ float relu_ugt(float x) { return !(x <= 0.0f) ? x : 0.0f; }
// exp for results that are rounded to 16 bits: 2^(t log2 e) on the hardware unit with the rounding
// error of the product fed back (within 3e-7 of libm's expf, a thousandth of a 16-bit half-ulp)
__device__ __forceinline__ float exp_c(float t) {
  const float y = __fmul_rn(t, 1.44269502162933349609375f);
  float r = __fmaf_rn(t, 1.44269502162933349609375f, -y);
  r = __fmaf_rn(t, 1.92596299112661746e-8f, r);
  float e;
  asm("ex2.approx.f32 %0, %1;" : "=f"(e) : "f"(y));
  const float c = __fmaf_rn(e, __fmul_rn(r, 0.693147182464599609375f), e);
  return c == c ? c : e;   // infinite t, or 2^y = inf with a negative residual: no correction
}
// The form for f16 chains: without the low part of log2 e.  Rounded to f16 it equals libm's expf
// rounded to f16 for every one of the 65536 f16 arguments (tested on the device), as exp_c does
// for every bf16 argument.  Results below f32's normal range round to zero in f16 whether they are
// flushed or not, so the flushing form of ex2 is used.
__device__ __forceinline__ float exp_s(float t) {
  const float y = __fmul_rn(t, 1.44269502162933349609375f);
  const float r = __fmaf_rn(t, 1.44269502162933349609375f, -y);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(y));
  const float c = __fmaf_rn(e, __fmul_rn(r, 0.693147182464599609375f), e);
  return c == c ? c : e;
}
// 1 / x for an f16 x whose quotient is rounded to f16: the hardware approximation, at most one
// f32 ulp (2^-23 relative) off, rounds to the same f16 value as the exact quotient, because for
// every finite f16 x the quotient lies more than 2^-22.5 (relative) away from the nearest f16
// rounding boundary, denormal results included (all 31743 positive values checked on the host;
// tests compare all 65536 bit patterns on the device).  An f16 value extended to f32 is never
// an f32 denormal, nor is its reciprocal, so the flushing form loses nothing.
__device__ __forceinline__ float rcp_h(float x) { float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
// The same for bf16, whose range is that of f32: the form that keeps denormal arguments and
// results.  A bf16 quotient is at least 2^-17 (relative; 2^-9 of a denormal step) from a rounding
// boundary, far more than the approximation's one f32 ulp.
__device__ __forceinline__ float rcp_b(float x) { float r; asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
// two 16-bit values in one register (element 0 in the low half)
__device__ __forceinline__ unsigned pack_h(float lo, float hi) { unsigned d; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo)); return d; }
__device__ __forceinline__ unsigned pack_b(float lo, float hi) { unsigned d; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo)); return d; }
__device__ __forceinline__ float lo_h(unsigned x) { float f; asm("{.reg .b16 l, h; mov.b32 {l, h}, %1; cvt.f32.f16 %0, l;}" : "=f"(f) : "r"(x)); return f; }
__device__ __forceinline__ float hi_h(unsigned x) { float f; asm("{.reg .b16 l, h; mov.b32 {l, h}, %1; cvt.f32.f16 %0, h;}" : "=f"(f) : "r"(x)); return f; }
__device__ __forceinline__ float lo_b(unsigned x) { return __uint_as_float(x << 16); }
__device__ __forceinline__ float hi_b(unsigned x) { return __uint_as_float(x & 0xffff0000u); }
__device__ __forceinline__ unsigned add_h(unsigned a, unsigned b) { unsigned d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ unsigned sub_h(unsigned a, unsigned b) { unsigned d; asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ unsigned mul_h(unsigned a, unsigned b) { unsigned d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
// relu as the reference writes it (x > 0 or unordered ? x : 0) on both halves: the halves that
// compare <= 0 (never a NaN) are cleared, which also turns -0 into +0
__device__ __forceinline__ unsigned relu_h(unsigned x) { unsigned m; asm("set.le.u32.f16x2 %0, %1, %2;" : "=r"(m) : "r"(x), "r"(0u)); return x & ~m; }
__device__ __forceinline__ unsigned relu_b(unsigned x) { unsigned m; asm("set.le.u32.bf16x2 %0, %1, %2;" : "=r"(m) : "r"(x), "r"(0u)); return x & ~m; }
// arith.maximumf / minimumf: NaN if either operand is one
__device__ __forceinline__ unsigned max_h(unsigned a, unsigned b) { unsigned d; asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ unsigned min_h(unsigned a, unsigned b) { unsigned d; asm("min.NaN.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ unsigned max_b(unsigned a, unsigned b) { unsigned d; asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ unsigned min_b(unsigned a, unsigned b) { unsigned d; asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ unsigned add_b(unsigned a, unsigned b) { unsigned d; asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ unsigned sub_b(unsigned a, unsigned b) { unsigned d; asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ unsigned mul_b(unsigned a, unsigned b) { unsigned d; asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
)SRC";

struct TypeInfo {
  const char *ctype;   // storage type
  const char *load;    // storage -> f32
  const char *round;   // f32 -> f32 rounded to the type
  const char *store;   // f32 -> storage
};
TypeInfo type_info(int dt) {
  if (dt == kF16) return {"u16", "h2f", "RH", "f2h"};
  if (dt == kBF16) return {"u16", "b2f", "RB", "f2b"};
  return {"float", "", "", ""};
}

// Straight-line code of the program: statements defining t0, t1, ...; returns the name
// of the result.  Input k at the current element is `x<k>`.
std::string emit_body(const unsigned char *code, int ncode, const std::string &round,
                      std::ostringstream &os) {
  std::vector<std::string> st;
  int t = 0;
  auto def = [&](const std::string &rhs, bool rounded) {
    const std::string name = "t" + std::to_string(t++);
    os << "    const float " << name << " = " << (rounded && !round.empty() ? round + "(" + rhs + ")" : rhs)
       << ";\n";
    return name;
  };
  for (int i = 0; i < ncode; ++i) {
    const int op = code[i];
    if (op >= 1 && op <= 12) {
      st.push_back("x" + std::to_string((op - 1) % 4));
    } else if (op == 13 || op == 14) {
      st.push_back(def(op == 13 ? "c0" : "c1", true));
    } else if (op == 15) {
      st.push_back("0.0f");
    } else if (op == 16) {
      st.push_back("1.0f");
    } else if (op < 64) {
      const std::string a = st.back();
      st.pop_back();
      const char *f = op == 32 ? "-" : op == 33 ? "fabsf" : op == 34 ? "logf" : op == 35 ? "expf"
                      : op == 36 ? "__fsqrt_rn" : op == 38 ? "tanhf" : op == 39 ? "relu_ugt" : "";
      st.push_back(def(op == 37 ? "__fdiv_rn(1.0f, __fsqrt_rn(" + a + "))" : std::string(f) + "(" + a + ")", true));
    } else {
      const std::string b = st.back();
      st.pop_back();
      const std::string a = st.back();
      st.pop_back();
      const char *f = op == 64 ? "__fadd_rn" : op == 65 ? "__fsub_rn" : op == 66 ? "__fmul_rn"
                      : op == 67 ? "__fdiv_rn" : op == 68 ? "maximumf" : "minimumf";
      // 1 / b: the correctly rounded reciprocal is the IEEE quotient, in half the instructions
      if (op == 67 && a == "1.0f") st.push_back(def("__frcp_rn(" + b + ")", true));
      else st.push_back(def(std::string(f) + "(" + a + ", " + b + ")", true));
    }
  }
  return st.back();
}

// The same program on PAIRS of 16-bit values held in one 32-bit register (f16 / bf16
// elementwise kernels).  add / sub / mul run as one packed instruction on both values:
// rounding the exact result once to an 11-bit (8-bit) significand equals rounding it to
// f32's 24 bits first and then to 16 bits (24 >= 2 * 11 + 2, so the double rounding is
// innocuous), i.e. the result is bit for bit that of extend - operate in f32 - round.  neg
// and abs are sign-bit operations, relu clears the halves that compare <= 0, maximumf / minimumf
// are the packed NaN-propagating instructions.  Everything else unpacks to f32, applies the f32
// function and packs with one rounding conversion for both values.
std::string emit_body_packed(const unsigned char *code, int ncode, bool bf16, std::ostringstream &os) {
  const std::string sfx = bf16 ? "_b" : "_h";
  std::vector<std::string> st;
  int t = 0;
  auto def = [&](const std::string &rhs) {
    const std::string name = "t" + std::to_string(t++);
    os << "    const unsigned " << name << " = " << rhs << ";\n";
    return name;
  };
  auto via_f32 = [&](const std::string &fn_lo, const std::string &fn_hi) {
    return "pack" + sfx + "(" + fn_lo + ", " + fn_hi + ")";
  };
  for (int i = 0; i < ncode; ++i) {
    const int op = code[i];
    if (op >= 1 && op <= 12) {
      st.push_back("x" + std::to_string((op - 1) % 4));
    } else if (op == 13 || op == 14) {
      st.push_back(op == 13 ? "pc0" : "pc1");
    } else if (op == 15) {
      st.push_back("0u");
    } else if (op == 16) {
      st.push_back(bf16 ? "0x3f803f80u" : "0x3c003c00u");
    } else if (op < 64) {
      const std::string a = st.back();
      st.pop_back();
      if (op == 32) { st.push_back(def("(" + a + " ^ 0x80008000u)")); continue; }
      if (op == 33) { st.push_back(def("(" + a + " & 0x7fff7fffu)")); continue; }
      if (op == 39) { st.push_back(def("relu" + sfx + "(" + a + ")")); continue; }
      const std::string lo = "lo" + sfx + "(" + a + ")", hi = "hi" + sfx + "(" + a + ")";
      auto f = [&](const std::string &x) -> std::string {
        switch (op) {
        case 34: return "logf(" + x + ")";
        case 35: return (bf16 ? "exp_c(" : "exp_s(") + x + ")";
        case 36: return "__fsqrt_rn(" + x + ")";
        case 37: return "__fdiv_rn(1.0f, __fsqrt_rn(" + x + "))";
        case 38: return "tanhf(" + x + ")";
        default: return "relu_ugt(" + x + ")";
        }
      };
      st.push_back(def(via_f32(f(lo), f(hi))));
    } else {
      const std::string b = st.back();
      st.pop_back();
      const std::string a = st.back();
      st.pop_back();
      if (op == 64) { st.push_back(def("add" + sfx + "(" + a + ", " + b + ")")); continue; }
      if (op == 65) { st.push_back(def("sub" + sfx + "(" + a + ", " + b + ")")); continue; }
      if (op == 66) { st.push_back(def("mul" + sfx + "(" + a + ", " + b + ")")); continue; }
      if (op == 68) { st.push_back(def("max" + sfx + "(" + a + ", " + b + ")")); continue; }
      if (op == 69) { st.push_back(def("min" + sfx + "(" + a + ", " + b + ")")); continue; }
      // what is left is the division: 1 / b through the hardware reciprocal (rcp_h, rcp_b: the
      // same 16-bit value as the quotient for every b), a / b as the IEEE quotient in f32
      const char *fn = "__fdiv_rn";
      if (a == "0x3f803f80u" || a == "0x3c003c00u") {
        const std::string rcp = bf16 ? "rcp_b" : "rcp_h";
        st.push_back(def(via_f32(rcp + "(lo" + sfx + "(" + b + "))", rcp + "(hi" + sfx + "(" + b + "))")));
        continue;
      }
      st.push_back(def(via_f32(std::string(fn) + "(lo" + sfx + "(" + a + "), lo" + sfx + "(" + b + "))",
                               std::string(fn) + "(hi" + sfx + "(" + a + "), hi" + sfx + "(" + b + "))")));
    }
  }
  return st.back();
}

struct Shape {
  int mode[4];  // per input: 0 full, 1 row vector, 2 column vector, -1 unused
  int n_inputs;
};

Shape input_shape(const unsigned char *code, int ncode, int n_inputs) {
  Shape s;
  s.n_inputs = n_inputs;
  for (int k = 0; k < 4; ++k) s.mode[k] = -1;
  for (int i = 0; i < ncode; ++i)
    if (code[i] >= 1 && code[i] <= 12) s.mode[(code[i] - 1) % 4] = (code[i] - 1) / 4;
  return s;
}

// One input may be pushed in one mode only (the front end never mixes them).
bool single_mode(const unsigned char *code, int ncode) {
  int seen[4] = {-1, -1, -1, -1};
  for (int i = 0; i < ncode; ++i)
    if (code[i] >= 1 && code[i] <= 12) {
      const int k = (code[i] - 1) % 4, m = (code[i] - 1) / 4;
      if (seen[k] >= 0 && seen[k] != m) return false;
      seen[k] = m;
    }
  return true;
}

// reduce with vec == -1: the "tall" form of the leading-dim reduce (many rows, few columns)
std::string generate(const unsigned char *code, int ncode, int n_inputs, int dtype, int out_dtype,
                     bool reduce, int vec) {
  const TypeInfo in = type_info(dtype), out = type_info(reduce ? dtype : out_dtype);
  const Shape sh = input_shape(code, ncode, n_inputs);
  std::ostringstream os;
  os << kPrelude;
  os << "#define RH(x) h2f(f2h(x))\n#define RB(x) b2f(f2b(x))\n";
  os << "extern \"C\" __global__ void __launch_bounds__(256) expr_kernel(";
  for (int k = 0; k < n_inputs; ++k) os << "const " << in.ctype << " *__restrict__ p" << k << ", ";
  os << out.ctype << " *__restrict__ y, long long rows, long long cols, float c0, float c1, int accumulate) {\n";
  auto load = [&](int k, const std::string &idx) {
    return std::string(in.load) + "(p" + std::to_string(k) + "[" + idx + "])";
  };
  if (reduce && vec == -1) {
    // Few columns, many rows (the reference's kInputFusion: 512 x 1024): one thread per column
    // would walk the rows alone, evaluating the chain's transcendental functions one after the
    // other.  Here a CTA takes 16 columns; all 256 threads evaluate the chain for a tile of 128
    // rows into shared memory, then one thread per column adds the tile's values in row
    // order: the rounded adds keep the loop nest's order, the rest runs in parallel.
    os << "  __shared__ float vals[128][17];\n"
       << "  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;\n"
       << "  const long long col = blockIdx.x * 16LL + tx;\n"
       << "  const bool live = col < cols;\n"
       << "  float acc = (live && ty == 0 && accumulate) ? " << in.load << "(y[col]) : 0.0f;\n"
       << "  for (long long r0 = 0; r0 < rows; r0 += 128) {\n"
       << "#pragma unroll\n"   // all eight passes at once: their loads are in flight together
       << "    for (int i = 0; i < 8; ++i) {\n"
       << "      const long long row = r0 + ty + 16 * i;\n"
       << "      if (live && row < rows) {\n";
    for (int k = 0; k < n_inputs; ++k)
      if (sh.mode[k] >= 0)
        os << "    const float x" << k << " = "
           << load(k, sh.mode[k] == 0 ? "row * cols + col" : sh.mode[k] == 1 ? "col" : "row") << ";\n";
    const std::string r = emit_body(code, ncode, in.round, os);
    os << "        vals[ty + 16 * i][tx] = " << r << ";\n      }\n    }\n"
       << "    __syncthreads();\n"
       << "    if (live && ty == 0) {\n"
       << "      const int n = rows - r0 < 128 ? (int)(rows - r0) : 128;\n"
       << "#pragma unroll 8\n"
       << "      for (int k = 0; k < n; ++k) acc = "
       << (in.round[0] ? std::string(in.round) + "(__fadd_rn(acc, vals[k][tx]))" : "__fadd_rn(acc, vals[k][tx])") << ";\n"
       << "    }\n    __syncthreads();\n  }\n"
       << "  if (live && ty == 0) y[col] = " << out.store << "(acc);\n}\n";
    return os.str();
  }
  auto vec_type = [](int bytes) { return bytes == 16 ? "uint4" : bytes == 8 ? "uint2" : bytes == 4 ? "unsigned" : "u16"; };
  if (reduce && vec >= 2) {
    // Many columns: `vec` adjacent columns per thread (16-byte loads), one running sum per
    // column, each added to in row order.
    const int in_bytes = dtype == kF32 ? 4 : 2;
    const std::string vt = vec_type(vec * in_bytes);
    os << "  const long long col = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * " << vec << ";\n"
       << "  if (col >= cols) return;\n"
       << "  float acc[" << vec << "];\n"
       << "  __align__(16) " << in.ctype << " yv[" << vec << "];\n"
       << "  if (accumulate) *reinterpret_cast<" << vt << " *>(yv) = *reinterpret_cast<const " << vt << " *>(y + col);\n"
       << "#pragma unroll\n  for (int e = 0; e < " << vec << "; ++e) acc[e] = accumulate ? " << in.load << "(yv[e]) : 0.0f;\n"
       << "#pragma unroll 4\n  for (long long row = 0; row < rows; ++row) {\n";
    for (int k = 0; k < n_inputs; ++k) {
      if (sh.mode[k] < 0) continue;
      if (sh.mode[k] == 2) {
        os << "    const float s" << k << " = " << load(k, "row") << ";\n";
        continue;
      }
      os << "    __align__(16) " << in.ctype << " v" << k << "[" << vec << "];\n"
         << "    *reinterpret_cast<" << vt << " *>(v" << k << ") = *reinterpret_cast<const " << vt << " *>(p" << k
         << " + " << (sh.mode[k] == 0 ? "row * cols + col" : "col") << ");\n";
    }
    os << "#pragma unroll\n    for (int e = 0; e < " << vec << "; ++e) {\n";
    for (int k = 0; k < n_inputs; ++k) {
      if (sh.mode[k] < 0) continue;
      if (sh.mode[k] == 2) os << "    const float x" << k << " = s" << k << ";\n";
      else os << "    const float x" << k << " = " << in.load << "(v" << k << "[e]);\n";
    }
    const std::string r = emit_body(code, ncode, in.round, os);
    os << "      acc[e] = "
       << (in.round[0] ? std::string(in.round) + "(__fadd_rn(acc[e], " + r + "))" : "__fadd_rn(acc[e], " + r + ")")
       << ";\n    }\n  }\n"
       << "#pragma unroll\n  for (int e = 0; e < " << vec << "; ++e) yv[e] = " << out.store << "(acc[e]);\n"
       << "  *reinterpret_cast<" << vt << " *>(y + col) = *reinterpret_cast<const " << vt << " *>(yv);\n}\n";
    return os.str();
  }
  if (reduce) {
    os << "  const long long col = blockIdx.x * (long long)blockDim.x + threadIdx.x;\n"
       << "  if (col >= cols) return;\n"
       << "  float acc = accumulate ? " << in.load << "(y[col]) : 0.0f;\n"
       << "  for (long long row = 0; row < rows; ++row) {\n";
    for (int k = 0; k < n_inputs; ++k)
      if (sh.mode[k] >= 0)
        os << "    const float x" << k << " = "
           << load(k, sh.mode[k] == 0 ? "row * cols + col" : sh.mode[k] == 1 ? "col" : "row") << ";\n";
    const std::string r = emit_body(code, ncode, in.round, os);
    os << "    acc = " << (in.round[0] ? std::string(in.round) + "(__fadd_rn(acc, " + r + "))" : "__fadd_rn(acc, " + r + ")")
       << ";\n  }\n"
       << "  y[col] = " << out.store << "(acc);\n}\n";
    return os.str();
  }
  // elementwise: `vec` consecutive columns of one row per thread and group.  A thread loads the
  // inputs of several groups before it computes the first: with one group in flight per thread a
  // chain with transcendental functions keeps a warp too long between its loads to saturate
  // HBM.  Four groups in f32; two in the 16-bit types, whose chains are bound by instruction
  // issue (8 values per 16 bytes) and lose occupancy to the extra registers (measured on the
  // log chain: 4739 / 4911 / 4574 GB/s with 1 / 2 / 4 groups).
  const int U = dtype == kF32 ? 4 : 2;
  const int in_bytes = dtype == kF32 ? 4 : 2, out_bytes = (out_dtype == kF32 ? 4 : 2);
  os << "  const long long groups_per_row = cols / " << vec << ", total = rows * groups_per_row;\n"
     << "  const long long stride = (long long)gridDim.x * blockDim.x;\n"
     << "  struct Grp {\n    long long base;\n";
  for (int k = 0; k < n_inputs; ++k) {
    if (sh.mode[k] < 0) continue;
    if (sh.mode[k] == 2) os << "    float s" << k << ";\n";
    else os << "    __align__(16) " << in.ctype << " v" << k << "[" << vec << "];\n";
  }
  os << "  };\n"
     << "  auto load_grp = [&](long long g, Grp &q) {\n"
     << "    const long long row = g / groups_per_row, col = (g % groups_per_row) * " << vec << ";\n"
     << "    q.base = row * cols + col;\n";
  for (int k = 0; k < n_inputs; ++k) {
    if (sh.mode[k] < 0) continue;
    if (sh.mode[k] == 2) {
      os << "    q.s" << k << " = " << load(k, "row") << ";\n";
      continue;
    }
    const std::string at = sh.mode[k] == 0 ? "q.base" : "col";
    if (vec == 1) os << "    q.v" << k << "[0] = p" << k << "[" << at << "];\n";
    else
      os << "    *reinterpret_cast<" << vec_type(vec * in_bytes) << " *>(q.v" << k << ") = *reinterpret_cast<const "
         << vec_type(vec * in_bytes) << " *>(p" << k << " + " << at << ");\n";
  }
  os << "  };\n"
     << "  auto run_grp = [&](const Grp &q) {\n"
     << "    const long long base = q.base;\n";
  if (dtype != kF32 && vec >= 2) {
    // 16-bit arithmetic on pairs: see emit_body_packed
    const bool bf = dtype == kBF16;
    const std::string sfx = bf ? "_b" : "_h";
    os << "    const unsigned pc0 = pack" << sfx << "(c0, c0), pc1 = pack" << sfx << "(c1, c1);\n";
    os << "    __align__(16) " << out.ctype << " r[" << vec << "];\n"
       << "#pragma unroll\n    for (int e = 0; e < " << vec / 2 << "; ++e) {\n";
    for (int k = 0; k < n_inputs; ++k) {
      if (sh.mode[k] < 0) continue;
      if (sh.mode[k] == 2) os << "    const unsigned x" << k << " = pack" << sfx << "(q.s" << k << ", q.s" << k << ");\n";
      else os << "    const unsigned x" << k << " = reinterpret_cast<const unsigned *>(q.v" << k << ")[e];\n";
    }
    const std::string r = emit_body_packed(code, ncode, bf, os);
    if (out_dtype == kF32) os << "    r[2 * e] = lo" << sfx << "(" << r << ");\n    r[2 * e + 1] = hi" << sfx << "(" << r << ");\n    }\n";
    else os << "    reinterpret_cast<unsigned *>(r)[e] = " << r << ";\n    }\n";
    os << "    *reinterpret_cast<" << vec_type(vec * out_bytes) << " *>(y + base) = *reinterpret_cast<const "
       << vec_type(vec * out_bytes) << " *>(r);\n";
  } else {
    os << "    __align__(16) " << out.ctype << " r[" << vec << "];\n"
       << "#pragma unroll\n    for (int e = 0; e < " << vec << "; ++e) {\n";
    for (int k = 0; k < n_inputs; ++k) {
      if (sh.mode[k] < 0) continue;
      if (sh.mode[k] == 2) os << "    const float x" << k << " = q.s" << k << ";\n";
      else os << "    const float x" << k << " = " << in.load << "(q.v" << k << "[e]);\n";
    }
    const std::string r = emit_body(code, ncode, in.round, os);
    os << "    r[e] = " << out.store << "(" << r << ");\n    }\n";
    if (vec == 1) os << "    y[base] = r[0];\n";
    else
      os << "    *reinterpret_cast<" << vec_type(vec * out_bytes) << " *>(y + base) = *reinterpret_cast<const "
         << vec_type(vec * out_bytes) << " *>(r);\n";
  }
  os << "  };\n"
     << "  long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x;\n"
     << "  for (; g + " << U - 1 << " * stride < total; g += " << U << " * stride) {\n"
     << "    Grp q[" << U << "];\n"
     << "#pragma unroll\n    for (int u = 0; u < " << U << "; ++u) load_grp(g + u * stride, q[u]);\n"
     << "#pragma unroll\n    for (int u = 0; u < " << U << "; ++u) run_grp(q[u]);\n"
     << "  }\n"
     << "  for (; g < total; g += stride) {\n    Grp q;\n    load_grp(g, q);\n    run_grp(q);\n  }\n}\n";
  return os.str();
}

using jit::Compiled;
using jit::driver;
using jit::nvrtc;

std::mutex g_mu;
std::map<std::string, Compiled> g_cache;

Compiled compile(const std::string &src) { return jit::compile_kernel(src, "expr_kernel"); }

} // namespace

// cudaErrorNotSupported: no compiled kernel for this call (NVRTC or the driver entry
// points are missing, the compilation failed, or IMEX_B200_NO_JIT is set); the caller
// then runs the interpreting kernel.
cudaError_t launch_expr_jit(const void *const *inputs, int n_inputs, void *out, int64_t rows, int64_t cols,
                            const unsigned char *code, int ncode, float c0, float c1, int dtype,
                            int out_dtype, bool reduce_leading, bool accumulate, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  if (getenv("IMEX_B200_NO_JIT") || !nvrtc().ok || !driver().ok) return cudaErrorNotSupported;
  if (n_inputs < 0 || n_inputs > 4 || ncode < 1 || ncode > 32) return cudaErrorInvalidValue;
  if (expr_validate(code, ncode, n_inputs) != ncode || !single_mode(code, ncode)) return cudaErrorNotSupported;
  // elements per thread: 16 bytes of the narrower of input and output type, when the
  // row length and the alignment allow it
  int vec = 1;
  // too few columns to fill the GPU with one thread each, and enough rows to share out
  if (reduce_leading && rows >= 64 && cols < 148LL * 256) vec = -1;
  if (reduce_leading && vec == 1) {
    // enough columns to fill the GPU with several per thread, and 16-byte alignment throughout
    const int want = dtype == kF32 ? 4 : 8;
    bool aligned = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && cols % want == 0;
    for (int i = 0; i < n_inputs; ++i) aligned = aligned && (reinterpret_cast<uintptr_t>(inputs[i]) & 15) == 0;
    if (aligned && cols / want >= 148LL * 512) vec = want;
  }
  if (!reduce_leading) {
    bool aligned = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    for (int i = 0; i < n_inputs; ++i) aligned = aligned && (reinterpret_cast<uintptr_t>(inputs[i]) & 15) == 0;
    const int want = (dtype == kF32 || out_dtype == kF32) ? 4 : 8;
    if (aligned && cols % want == 0) vec = want;
    else if (aligned && cols % 4 == 0) vec = 4;
  }
  int device = 0;
  cudaGetDevice(&device);
  std::string key(reinterpret_cast<const char *>(code), static_cast<size_t>(ncode));
  key += "|" + std::to_string(device) + "|" + std::to_string(dtype) + "|" + std::to_string(out_dtype) + "|" +
         std::to_string(reduce_leading) + "|" + std::to_string(vec) + "|" + std::to_string(n_inputs);
  Compiled c;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_cache.find(key);
    if (it == g_cache.end()) {
      cudaFree(nullptr);  // the primary context exists before the module is loaded into it
      it = g_cache.emplace(key, compile(generate(code, ncode, n_inputs, dtype, out_dtype, reduce_leading, vec))).first;
    }
    c = it->second;
  }
  if (c.failed || !c.fn) return cudaErrorNotSupported;
  const void *in[4] = {nullptr, nullptr, nullptr, nullptr};
  for (int i = 0; i < n_inputs; ++i) in[i] = inputs[i];
  long long r = rows, cl = cols;
  int acc = accumulate ? 1 : 0;
  std::vector<void *> args;
  for (int i = 0; i < n_inputs; ++i) args.push_back(&in[i]);
  args.push_back(&out);
  args.push_back(&r);
  args.push_back(&cl);
  args.push_back(&c0);
  args.push_back(&c1);
  args.push_back(&acc);
  unsigned blocks;
  if (reduce_leading) {
    blocks = static_cast<unsigned>(vec == -1 ? (cols + 15) / 16 : vec > 1 ? (cols / vec + 255) / 256 : (cols + 255) / 256);
  } else {
    const long long groups = rows * (cols / vec);
    long long b = (groups + 255) / 256;
    const long long cap = 148LL * 32;
    blocks = static_cast<unsigned>(b > cap ? cap : b);
  }
  const CUresult rc = driver().launchKernel(c.fn, blocks, 1, 1, 256, 1, 1, 0, stream, args.data(), nullptr);
  return rc == CUDA_SUCCESS ? cudaSuccess : cudaErrorLaunchFailure;
}

} // namespace imex
