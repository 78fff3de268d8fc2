// Run-time compilation shared by the kernels that are compiled at first use (the fused
// elementwise chains of expr_jit.cu and the loop nests of loopnest_jit.cu): NVRTC is
// looked up with dlopen, the three driver entry points needed to run a cubin through
// cudaGetDriverEntryPoint, and compile_kernel() turns CUDA C++ text into a CUfunction for
// sm_100a.  The reference does the same job when a module is loaded: it hands SPIR-V to
// the driver's JIT (lib/ExecutionEngine/LEVELZERORUNTIME/LevelZeroRuntimeWrappers.cpp:402-431).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

namespace imex {
namespace jit {

// ---- NVRTC, through dlopen ------------------------------------------------------
struct Nvrtc {
  using Program = void *;
  int (*createProgram)(Program *, const char *, const char *, int, const char *const *,
                       const char *const *) = nullptr;
  int (*compileProgram)(Program, int, const char *const *) = nullptr;
  int (*getCUBINSize)(Program, size_t *) = nullptr;
  int (*getCUBIN)(Program, char *) = nullptr;
  int (*getProgramLogSize)(Program, size_t *) = nullptr;
  int (*getProgramLog)(Program, char *) = nullptr;
  int (*destroyProgram)(Program *) = nullptr;
  bool ok = false;
};

inline const Nvrtc &nvrtc() {
  static Nvrtc n = [] {
    Nvrtc r;
    void *h = nullptr;
    for (const char *name : {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                             "/usr/local/cuda/lib64/libnvrtc.so"}) {
      h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
      if (h) break;
    }
    if (!h) return r;
    auto sym = [&](const char *s) { return dlsym(h, s); };
    r.createProgram = reinterpret_cast<decltype(r.createProgram)>(sym("nvrtcCreateProgram"));
    r.compileProgram = reinterpret_cast<decltype(r.compileProgram)>(sym("nvrtcCompileProgram"));
    r.getCUBINSize = reinterpret_cast<decltype(r.getCUBINSize)>(sym("nvrtcGetCUBINSize"));
    r.getCUBIN = reinterpret_cast<decltype(r.getCUBIN)>(sym("nvrtcGetCUBIN"));
    r.getProgramLogSize = reinterpret_cast<decltype(r.getProgramLogSize)>(sym("nvrtcGetProgramLogSize"));
    r.getProgramLog = reinterpret_cast<decltype(r.getProgramLog)>(sym("nvrtcGetProgramLog"));
    r.destroyProgram = reinterpret_cast<decltype(r.destroyProgram)>(sym("nvrtcDestroyProgram"));
    r.ok = r.createProgram && r.compileProgram && r.getCUBINSize && r.getCUBIN && r.destroyProgram;
    return r;
  }();
  return n;
}

// ---- the three driver calls needed to run a cubin -------------------------------------
struct Driver {
  CUresult (*moduleLoadData)(CUmodule *, const void *) = nullptr;
  CUresult (*moduleGetFunction)(CUfunction *, CUmodule, const char *) = nullptr;
  CUresult (*launchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                           unsigned, CUstream, void **, void **) = nullptr;
  bool ok = false;
};

inline const Driver &driver() {
  static Driver d = [] {
    Driver r;
    auto get = [](const char *name) -> void * {
      void *p = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
          q != cudaDriverEntryPointSuccess)
        return nullptr;
      return p;
    };
    r.moduleLoadData = reinterpret_cast<decltype(r.moduleLoadData)>(get("cuModuleLoadData"));
    r.moduleGetFunction = reinterpret_cast<decltype(r.moduleGetFunction)>(get("cuModuleGetFunction"));
    r.launchKernel = reinterpret_cast<decltype(r.launchKernel)>(get("cuLaunchKernel"));
    r.ok = r.moduleLoadData && r.moduleGetFunction && r.launchKernel;
    return r;
  }();
  return d;
}

struct Compiled {
  CUfunction fn = nullptr;
  bool failed = false;
  std::string log;  // compiler output when the compilation failed
};

// Compiles `src` for sm_100a (no FMA contraction) and returns the entry `name`.
inline Compiled compile_kernel(const std::string &src, const char *name) {
  Compiled c;
  const Nvrtc &n = nvrtc();
  const Driver &d = driver();
  if (!n.ok || !d.ok) {
    c.failed = true;
    c.log = "NVRTC or the CUDA driver entry points are not available";
    return c;
  }
  Nvrtc::Program prog = nullptr;
  if (n.createProgram(&prog, src.c_str(), "imex_jit.cu", 0, nullptr, nullptr) != 0) {
    c.failed = true;
    c.log = "nvrtcCreateProgram failed";
    return c;
  }
  const char *opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device", "--fmad=false"};
  const int rc = n.compileProgram(prog, 4, opts);
  if (rc != 0) {
    if (n.getProgramLogSize && n.getProgramLog) {
      size_t sz = 0;
      n.getProgramLogSize(prog, &sz);
      c.log.assign(sz, '\0');
      if (sz) n.getProgramLog(prog, &c.log[0]);
    }
    if (getenv("IMEX_B200_JIT_VERBOSE"))
      fprintf(stderr, "[imex jit] compilation failed:\n%s\n%s\n", c.log.c_str(), src.c_str());
    n.destroyProgram(&prog);
    c.failed = true;
    return c;
  }
  size_t size = 0;
  std::vector<char> cubin;
  if (n.getCUBINSize(prog, &size) == 0 && size > 0) {
    cubin.resize(size);
    if (n.getCUBIN(prog, cubin.data()) != 0) cubin.clear();
  }
  n.destroyProgram(&prog);
  CUmodule mod = nullptr;
  if (cubin.empty() || d.moduleLoadData(&mod, cubin.data()) != CUDA_SUCCESS ||
      d.moduleGetFunction(&c.fn, mod, name) != CUDA_SUCCESS) {
    c.fn = nullptr;
    c.failed = true;
    c.log = "the compiled module could not be loaded";
  }
  return c;
}

} // namespace jit
} // namespace imex
