// CPU stand-in for the GPU runtime-wrapper C ABI — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// Linked with the front end's sources into oracle/_cpu/imex-oracle-runner (see the
// Makefile), it lets the reference's own .mlir tests run on the host through the same
// parser: the runner is started with --all-loopnests, so every linalg op arrives here as
// the loop nest that the reference's CPU pipeline makes of it (test/PlaidML/linalg-to-cpu.pp:
// convert-linalg-to-loops, then LLVM), written as C++ text.  The text is compiled with the
// host compiler (-O2 -ffp-contract=off -fno-fast-math: separately rounded multiply and
// add, glibc's expf / logf, exactly what mlir-runner's JIT-compiled loops call) and run
// once per point of the parallel iteration space, in order.  What it prints is checked
// against the CHECK lines the reference's tests carry; the GPU kernels are then checked
// against it.  Nothing under mlir-extensions_b200/ links or loads this file.
#include "../include/imex_b200_blob.h"
#include "../include/imex_cuda_runtime.h"

#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

[[noreturn]] void fail(const std::string &what) {
  fprintf(stdout, "An exception was thrown: %s\n", what.c_str());
  fflush(stdout);
  abort();
}

struct Module {
  std::vector<ImexKernelDesc> kernels;
  std::vector<std::string> sources;
};
struct Kernel {
  ImexKernelDesc desc;
  std::string source;
};
using RunFn = void (*)(void **, long long);

std::map<const void *, std::unique_ptr<Module>> g_modules;
std::vector<std::unique_ptr<Kernel>> g_kernels;
std::map<std::string, RunFn> g_compiled;

// What the kernel text is written against, for the host; and a driver that walks the
// parallel iteration space in order.
const char *kHostPrelude = R"SRC(
#include <cmath>
#include <cstring>
#include <utility>
typedef unsigned short u16;
typedef unsigned char u8;
typedef long long i64;
typedef unsigned long long u64;
#define __global__
#define __restrict__ __restrict
static i64 imx_host_index;
#define IMX_THREAD_INDEX imx_host_index
static inline float imx_f16_to_f32(u16 h) { _Float16 x; std::memcpy(&x, &h, 2); return (float)x; }
static inline u16 imx_f32_to_f16(float f) { _Float16 x = (_Float16)f; u16 h; std::memcpy(&h, &x, 2); return h; }
static inline float imx_bf16_to_f32(u16 h) { unsigned u = ((unsigned)h) << 16; float f; std::memcpy(&f, &u, 4); return f; }
static inline u16 imx_f32_to_bf16(float f) {
  unsigned u; std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (u16)((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (u16)(u >> 16);
}
static inline float imx_rf16(float f) { return imx_f16_to_f32(imx_f32_to_f16(f)); }
static inline float imx_rbf16(float f) { return imx_bf16_to_f32(imx_f32_to_bf16(f)); }
static inline float imx_nan32() { return std::nanf(""); }
static inline float imx_inf32() { return INFINITY; }
static inline double imx_nan64() { return std::nan(""); }
static inline double imx_inf64() { return (double)INFINITY; }
static inline int imx_f32_bits(float f) { int i; std::memcpy(&i, &f, 4); return i; }
static inline float imx_bits_f32(int i) { float f; std::memcpy(&f, &i, 4); return f; }
static inline float imx_maximum(float a, float b) { return a != a ? a : (b != b ? b : fmaxf(a, b)); }
static inline float imx_minimum(float a, float b) { return a != a ? a : (b != b ? b : fminf(a, b)); }
static inline double imx_maximum(double a, double b) { return a != a ? a : (b != b ? b : fmax(a, b)); }
static inline double imx_minimum(double a, double b) { return a != a ? a : (b != b ? b : fmin(a, b)); }
static inline float imx_exp_f16(float x) { return expf(x); }   // the device side has forms of its own for 16-bit arguments
static inline float imx_exp_bf16(float x) { return expf(x); }
static inline float imx_maxnum(float a, float b) { return fmaxf(a, b); }
static inline float imx_minnum(float a, float b) { return fminf(a, b); }
static inline double imx_maxnum(double a, double b) { return fmax(a, b); }
static inline double imx_minnum(double a, double b) { return fmin(a, b); }
)SRC";

const char *kHostDriver = R"SRC(
template <typename... A, std::size_t... I>
static void imx_call(void (*f)(A...), void **p, std::index_sequence<I...>) { f((A)p[I]...); }
template <typename... A>
static void imx_run(void (*f)(A...), void **p, i64 n) {
  for (i64 i = 0; i < n; ++i) { imx_host_index = i; imx_call(f, p, std::index_sequence_for<A...>{}); }
}
extern "C" void imex_loopnest_run(void **p, long long n) { imx_run(&imex_loopnest, p, n); }
)SRC";

unsigned long long hashOf(const std::string &s) {
  unsigned long long h = 1469598103934665603ULL;
  for (unsigned char c : s) h = (h ^ c) * 1099511628211ULL;
  return h;
}

RunFn compile(const std::string &source) {
  auto it = g_compiled.find(source);
  if (it != g_compiled.end()) return it->second;
  const char *tmp = getenv("TMPDIR");
  const std::string dir = std::string(tmp && *tmp ? tmp : "/tmp") + "/imex_oracle_loopnests_" + std::to_string(getuid());
  mkdir(dir.c_str(), 0700);
  char name[64];
  snprintf(name, sizeof name, "%016llx", hashOf(source));
  const std::string base = dir + "/" + name, so = base + ".so";
  if (access(so.c_str(), R_OK) != 0) {
    const std::string cpp = base + "." + std::to_string(getpid()) + ".cpp", part = base + "." + std::to_string(getpid()) + ".so";
    {
      std::ofstream f(cpp);
      f << kHostPrelude << source << kHostDriver;
    }
    const std::string cmd = "g++ -std=c++17 -O2 -ffp-contract=off -fno-fast-math -fwrapv -fPIC -shared -w -o " + part +
                            " " + cpp + " 2> " + base + ".log";
    if (system(cmd.c_str()) != 0) fail("the host compiler refused a loop-nest kernel; see " + base + ".log\n" + source);
    rename(part.c_str(), so.c_str());
    unlink(cpp.c_str());
  }
  void *h = dlopen(so.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!h) fail(std::string("dlopen of a compiled loop nest failed: ") + dlerror());
  auto fn = reinterpret_cast<RunFn>(dlsym(h, "imex_loopnest_run"));
  if (!fn) fail("compiled loop nest has no entry point");
  g_compiled[source] = fn;
  return fn;
}

// IMEX_OP_GEMM on the host, the way the reference's CPU pipeline computes a matmul: per output
// element, k ascending, multiply then add in f32 with separate roundings (16-bit inputs
// extended first), then + bias, then one rounding to a 16-bit result type.  Reached by the
// gpu.func kernels the front end recognises as GEMMs (no epilogue there).
float elt_to_f32(const void *p, int64_t i, uint32_t dt) {
  if (dt == IMEX_F32) return static_cast<const float *>(p)[i];
  const uint16_t h = static_cast<const uint16_t *>(p)[i];
  if (dt == IMEX_BF16) { uint32_t u = static_cast<uint32_t>(h) << 16; float f; memcpy(&f, &u, 4); return f; }
  _Float16 x; memcpy(&x, &h, 2); return static_cast<float>(x);
}
void host_gemm(const ImexKernelDesc &d, const std::vector<void *> &ptrs) {
  const bool bias = d.flags & IMEX_FLAG_BIAS, acc = d.flags & IMEX_FLAG_ACCUMULATE;
  const bool ta = d.flags & IMEX_FLAG_TRANS_A, tb = d.flags & IMEX_FLAG_TRANS_B;
  if (ptrs.size() < (bias ? 4u : 3u)) fail("gpuLaunchKernel: gemm needs A, B, C (and bias)");
  if (d.epilogue != IMEX_EPI_NONE || d.dims[3] || d.dims[4] || d.dims[5]) fail("host gemm: epilogues and pitches are not served here");
  const int64_t M = d.dims[0], N = d.dims[1], K = d.dims[2];
  const void *A = ptrs[0], *B = ptrs[1];
  const float *bv = bias ? static_cast<const float *>(ptrs[3]) : nullptr;
  std::vector<float> row(static_cast<size_t>(N));
  for (int64_t i = 0; i < M; ++i) {
    for (int64_t j = 0; j < N; ++j) row[j] = acc ? elt_to_f32(ptrs[2], i * N + j, d.out_dtype) : 0.0f;
    for (int64_t k = 0; k < K; ++k) {
      const float a = elt_to_f32(A, ta ? k * M + i : i * K + k, d.in_dtype);
      for (int64_t j = 0; j < N; ++j) {
        const float p = a * elt_to_f32(B, tb ? j * K + k : k * N + j, d.in_dtype);
        row[j] = row[j] + p;
      }
    }
    for (int64_t j = 0; j < N; ++j) {
      float v = row[j];
      if (bv) v = v + bv[j];
      if (d.out_dtype == IMEX_F32) static_cast<float *>(ptrs[2])[i * N + j] = v;
      else if (d.out_dtype == IMEX_F16) { _Float16 x = static_cast<_Float16>(v); memcpy(static_cast<uint16_t *>(ptrs[2]) + i * N + j, &x, 2); }
      else {
        uint32_t u; memcpy(&u, &v, 4);
        u += 0x7fffu + ((u >> 16) & 1u);
        static_cast<uint16_t *>(ptrs[2])[i * N + j] = static_cast<uint16_t>(u >> 16);
      }
    }
  }
}

} // namespace

extern "C" {

void *gpuCreateStream(void *, void *) { return new int(0); }
void gpuStreamDestroy(void *stream) { delete static_cast<int *>(stream); }
void *gpuMemAlloc(void *, size_t size, size_t, bool) {
  void *p = nullptr;
  if (posix_memalign(&p, 64, size ? size : 64) != 0) fail("gpuMemAlloc: out of host memory");
  return p;
}
void gpuMemFree(void *, void *ptr) { free(ptr); }
void gpuMemCopy(void *, void *dst, void *src, size_t size) { memmove(dst, src, size); }
void gpuMemcpy(void *s, void *dst, void *src, size_t size) { gpuMemCopy(s, dst, src, size); }

void *gpuModuleLoad(void *, const void *data, size_t size) {
  auto it = g_modules.find(data);
  if (it != g_modules.end()) return it->second.get();
  ImexBlobHeader h;
  if (size < sizeof h) fail("gpuModuleLoad: blob too small");
  memcpy(&h, data, sizeof h);
  if (h.magic != IMEX_BLOB_MAGIC) fail("gpuModuleLoad: bad blob magic");
  auto m = std::make_unique<Module>();
  m->kernels.resize(h.num_kernels);
  m->sources.resize(h.num_kernels);
  memcpy(m->kernels.data(), static_cast<const char *>(data) + sizeof h, h.num_kernels * sizeof(ImexKernelDesc));
  for (size_t i = 0; i < m->kernels.size(); ++i) {
    const ImexKernelDesc &k = m->kernels[i];
    if (k.op == IMEX_OP_GEMM) continue;  // served by host_gemm below (GPU-dialect kernels recognised as GEMMs)
    if (k.op != IMEX_OP_LOOPNEST)
      fail("the CPU checker runs loop nests only (start the runner with --all-loopnests); got op " + std::to_string(k.op));
    if (k.dims[1] < 0 || k.dims[2] <= 0 || static_cast<size_t>(k.dims[1] + k.dims[2]) > size)
      fail("gpuModuleLoad: kernel text outside the blob");
    m->sources[i].assign(static_cast<const char *>(data) + k.dims[1], static_cast<size_t>(k.dims[2]));
  }
  Module *raw = m.get();
  g_modules[data] = std::move(m);
  return raw;
}

void *gpuKernelGet(void *, void *module, const char *name) {
  auto *m = static_cast<Module *>(module);
  for (size_t i = 0; i < m->kernels.size(); ++i)
    if (strncmp(m->kernels[i].name, name, IMEX_KERNEL_NAME_MAX) == 0) {
      g_kernels.push_back(std::make_unique<Kernel>());
      g_kernels.back()->desc = m->kernels[i];
      g_kernels.back()->source = m->sources[i];
      return g_kernels.back().get();
    }
  fail(std::string("gpuKernelGet: no kernel named ") + name);
}

void *gpuLaunchKernel(void *, void *kernel, size_t, size_t, size_t, size_t, size_t, size_t, size_t, void *params,
                      void *) {
  auto *k = static_cast<Kernel *>(kernel);
  auto *p = static_cast<ImexParamDesc *>(params);
  std::vector<void *> ptrs;
  for (size_t i = 0; p && !(p[i].data == nullptr && p[i].size == 0); ++i) {
    void *v;
    memcpy(&v, p[i].data, sizeof v);
    ptrs.push_back(v);
  }
  if (k->desc.op == IMEX_OP_GEMM) {
    host_gemm(k->desc, ptrs);
    return nullptr;
  }
  if (static_cast<int64_t>(ptrs.size()) < k->desc.dims[3]) fail("gpuLaunchKernel: too few pointer arguments");
  compile(k->source)(ptrs.data(), k->desc.dims[0]);
  return nullptr;
}

// Block partition of the reference (lib/Dialect/NDArray/Extensions/MeshShardingExtensions.cpp:
// 74-100): shards are extent / n long and the last extent % n of them one longer.
int64_t imexShardSize(int64_t shard, int64_t numShards, int64_t extent) {
  const int64_t longer_from = numShards - extent % numShards;
  return extent / numShards + (shard >= longer_from ? 1 : 0);
}
int64_t imexShardOffset(int64_t shard, int64_t numShards, int64_t extent) {
  const int64_t longer_from = numShards - extent % numShards;
  return shard * (extent / numShards) + (shard > longer_from ? shard - longer_from : 0);
}

void gpuWait(void *) {}
void gpuModuleUnload(void *) {}

} // extern "C"
