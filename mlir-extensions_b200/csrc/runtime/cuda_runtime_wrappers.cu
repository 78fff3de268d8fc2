// CUDA implementation of the reference's GPU runtime-wrapper C ABI
// (libimex_cuda_runtime.so).  It takes the place of the Level Zero and SYCL
// wrapper libraries (lib/ExecutionEngine/LEVELZERORUNTIME/LevelZeroRuntimeWrappers.cpp,
// lib/ExecutionEngine/SYCLRUNTIME/SyclRuntimeWrappers.cpp): same symbols, same
// argument meaning, same error convention.  Where those libraries hand a
// SPIR-V module to the driver's JIT, this one reads a kernel-descriptor blob
// (include/imex_b200_blob.h) and dispatches each recognised op to a
// hand-written sm_100a kernel.  There is no CPU fallback: an op or blob it
// does not know is an error.
#include "../../../include/imex_b200_blob.h"
#include "../../../include/imex_cuda_runtime.h"
#include "../kernels/kernels.h"
#include "stats.h"

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

// Error convention of the reference (LevelZeroRuntimeWrappers.cpp:41-53).
template <typename F> auto catchAll(F &&func) {
  try {
    return func();
  } catch (const std::exception &e) {
    fprintf(stdout, "An exception was thrown: %s\n", e.what());
    fflush(stdout);
    abort();
  } catch (...) {
    fprintf(stdout, "An unknown exception was thrown\n");
    fflush(stdout);
    abort();
  }
}

void check(cudaError_t e, const char *what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(e));
}
#define CHECK_CUDA(expr) check((expr), #expr)

struct Allocation {
  size_t size;
  bool managed;
  int device;
};

struct Stream;
struct Event {
  cudaEvent_t ev = nullptr;
  // Set instead of recording `ev` when the launch was issued while its stream was being
  // captured into a CUDA graph: an event record would become a graph node of its own between
  // the kernel nodes (about a microsecond each, and it cuts the programmatic edge that lets
  // consecutive launches overlap).  Such a handle orders only work on the same stream, which
  // stream order gives anyway.
  Stream *ordered_on = nullptr;
};

// Launch-completion events come from a ring of kEventSlots per stream, created on first
// use and re-recorded when the ring wraps: the reference hands out events from one fixed
// pool of 256 slots as well (LevelZeroRuntimeWrappers.cpp:155-168) and nobody ever releases
// them.  A handle therefore stays meaningful for the next 255 launches on its stream.
constexpr size_t kEventSlots = 256;

struct Stream {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool owned = true;
  unsigned *status_host = nullptr;  // mapped, written by kernels whose bounded waits run out
  unsigned *status_dev = nullptr;
  float *scratch = nullptr;  // reduce-all partials
  size_t scratch_bytes = 0;
  const char *last_kernel = "";
  Event events[kEventSlots];
  size_t next_event = 0;
  std::unordered_set<const void *> device_ptrs;  // parameter values already seen to be device memory
};

struct Kernel {
  ImexKernelDesc desc;
  const std::string *source = nullptr;  // IMEX_OP_LOOPNEST: kernel text, owned by the module
};

struct Module {
  std::vector<ImexKernelDesc> kernels;
  std::vector<std::string> sources;  // per kernel: the text of an IMEX_OP_LOOPNEST kernel, else empty
  std::vector<std::unique_ptr<Kernel>> handles;  // one per table row, made on first gpuKernelGet
};

std::mutex g_mutex;
std::map<const void *, std::unique_ptr<Module>> g_modules;  // keyed by blob address, lives to exit
std::unordered_map<void *, Allocation> g_allocs;
std::atomic<uint64_t> g_launches{0};

const char *op_name(uint32_t op) {
  switch (op) {
  case IMEX_OP_GEMM: return "gemm";
  case IMEX_OP_SOFTMAX: return "softmax";
  case IMEX_OP_REDUCE_ROWS: return "reduce_rows";
  case IMEX_OP_REDUCE_LEADING: return "reduce_leading";
  case IMEX_OP_REDUCE_ALL: return "reduce_all";
  case IMEX_OP_TRANSPOSE2D: return "transpose2d";
  case IMEX_OP_TRANSPOSE3D: return "transpose3d";
  case IMEX_OP_ELTWISE: return "eltwise";
  case IMEX_OP_FILL_UNIFORM: return "fill_uniform";
  case IMEX_OP_FILL_NORMAL: return "fill_normal";
  case IMEX_OP_EXPR: return "expr";
  case IMEX_OP_ATTENTION_FWD: return "attention_fwd";
  case IMEX_OP_LOOPNEST: return "loopnest";
  }
  return nullptr;
}

size_t dtype_bytes(uint32_t dt) {
  switch (dt) {
  case IMEX_F32: case IMEX_I32: return 4;
  case IMEX_BF16: case IMEX_F16: return 2;
  }
  throw std::runtime_error("unknown element type " + std::to_string(dt));
}

Stream *make_stream(const int32_t *device, cudaStream_t adopt) {
  auto s = std::make_unique<Stream>();
  if (device) {
    s->device = *device;
    CHECK_CUDA(cudaSetDevice(s->device));
  } else {
    CHECK_CUDA(cudaGetDevice(&s->device));
  }
  if (adopt) {
    s->stream = adopt;
    s->owned = false;
  } else {
    CHECK_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
  }
  CHECK_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&s->status_host), sizeof(unsigned),
                           cudaHostAllocMapped));
  *s->status_host = 0;
  CHECK_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&s->status_dev), s->status_host, 0));
  return s.release();
}

void destroy_stream(Stream *s) {
  if (!s) return;
  if (s->scratch) cudaFree(s->scratch);
  for (auto &e : s->events)
    if (e.ev) cudaEventDestroy(e.ev);
  if (s->status_host) cudaFreeHost(s->status_host);
  if (s->owned && s->stream) CHECK_CUDA(cudaStreamDestroy(s->stream));
  delete s;
}

void *alloc_memory(Stream *s, size_t size, size_t /*alignment*/, bool shared) {
  void *p = nullptr;
  const size_t bytes = size ? size : 1;
  if (s) CHECK_CUDA(cudaSetDevice(s->device));
  if (getenv("IMEX_B200_FAIL_ALLOC"))  // host-side fault injection for tests
    throw std::runtime_error("gpuMemAlloc failed: injected allocation failure");
  if (shared)
    CHECK_CUDA(cudaMallocManaged(&p, bytes));
  else
    CHECK_CUDA(cudaMalloc(&p, bytes));
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  g_allocs[p] = Allocation{size, shared, dev};
  return p;
}

void free_memory(void *p) {
  if (!p) return;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_allocs.erase(p);
  }
  CHECK_CUDA(cudaFree(p));
}

Module *load_module(const void *data, size_t size) {
  if (!data) throw std::runtime_error("gpuModuleLoad: null blob");
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_modules.find(data);
    if (it != g_modules.end()) return it->second.get();
  }
  if (size < sizeof(ImexBlobHeader)) throw std::runtime_error("gpuModuleLoad: blob too small");
  ImexBlobHeader h;
  memcpy(&h, data, sizeof h);
  if (h.magic != IMEX_BLOB_MAGIC) {
    uint32_t w;
    memcpy(&w, data, 4);
    if (w == 0x07230203u)
      throw std::runtime_error("gpuModuleLoad: blob is a SPIR-V module; this runtime loads "
                               "IMEX B200 kernel-descriptor blobs only");
    throw std::runtime_error("gpuModuleLoad: bad blob magic");
  }
  if (h.version != IMEX_BLOB_VERSION)
    throw std::runtime_error("gpuModuleLoad: unsupported blob version " + std::to_string(h.version));
  if (size < sizeof h + static_cast<size_t>(h.num_kernels) * sizeof(ImexKernelDesc))
    throw std::runtime_error("gpuModuleLoad: blob truncated");
  auto m = std::make_unique<Module>();
  m->kernels.resize(h.num_kernels);
  memcpy(m->kernels.data(), static_cast<const char *>(data) + sizeof h,
         h.num_kernels * sizeof(ImexKernelDesc));
  m->sources.resize(h.num_kernels);
  for (size_t i = 0; i < m->kernels.size(); ++i) {
    auto &k = m->kernels[i];
    k.name[IMEX_KERNEL_NAME_MAX - 1] = 0;
    if (!op_name(k.op))
      throw std::runtime_error(std::string("gpuModuleLoad: kernel '") + k.name +
                               "' names an unknown op " + std::to_string(k.op));
    if (k.op == IMEX_OP_LOOPNEST) {  // the kernel's text lies in the payload behind the table
      const int64_t off = k.dims[1], len = k.dims[2];
      if (off < 0 || len <= 0 || static_cast<uint64_t>(off) + static_cast<uint64_t>(len) > size)
        throw std::runtime_error(std::string("gpuModuleLoad: kernel '") + k.name + "' points outside the blob");
      m->sources[i].assign(static_cast<const char *>(data) + off, static_cast<size_t>(len));
    }
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  auto &slot = g_modules[data];
  if (!slot) slot = std::move(m);
  return slot.get();
}

Kernel *get_kernel(Module *m, const char *name) {
  if (!m || !name) throw std::runtime_error("gpuKernelGet: null module or name");
  for (size_t i = 0; i < m->kernels.size(); ++i)
    if (strncmp(m->kernels[i].name, name, IMEX_KERNEL_NAME_MAX) == 0) {
      // the handle belongs to the module (which lives to exit): asking twice gives the same one
      std::lock_guard<std::mutex> lock(g_mutex);
      if (m->handles.size() < m->kernels.size()) m->handles.resize(m->kernels.size());
      if (!m->handles[i]) {
        m->handles[i] = std::make_unique<Kernel>();
        m->handles[i]->desc = m->kernels[i];
        m->handles[i]->source = &m->sources[i];
      }
      return m->handles[i].get();
    }
  throw std::runtime_error(std::string("gpuKernelGet: no kernel named '") + name + "' in module");
}

template <typename T> size_t countUntilNull(T *p, bool (*isEnd)(const T &)) {
  size_t n = 0;
  while (!isEnd(p[n])) ++n;
  return n;
}

void prefetch_managed(Stream *s, void *ptr) {
  Allocation a;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_allocs.find(ptr);
    if (it == g_allocs.end() || !it->second.managed) return;
    a = it->second;
  }
  // host code filled this buffer; move it before the kernel touches it so the
  // launch does not run at page-fault speed
#if CUDART_VERSION >= 13000
  cudaMemLocation loc;
  loc.type = cudaMemLocationTypeDevice;
  loc.id = s->device;
  cudaMemPrefetchAsync(ptr, a.size, loc, 0, s->stream);
#else
  cudaMemPrefetchAsync(ptr, a.size, s->device, s->stream);
#endif
}

void ensure_scratch(Stream *s, size_t bytes) {
  if (s->scratch_bytes >= bytes) return;
  if (s->scratch) {
    CHECK_CUDA(cudaStreamSynchronize(s->stream));
    CHECK_CUDA(cudaFree(s->scratch));
  }
  size_t cap = bytes < (1u << 20) ? (1u << 20) : bytes;
  CHECK_CUDA(cudaMalloc(reinterpret_cast<void **>(&s->scratch), cap));
  s->scratch_bytes = cap;
}

// One enqueue of the op a kernel handle stands for.
void enqueue(Stream *s, const ImexKernelDesc &d, void **ptrs, size_t nptrs, const std::string *source = nullptr) {
  auto need = [&](size_t n) {
    if (nptrs < n)
      throw std::runtime_error(std::string("gpuLaunchKernel: '") + d.name + "' (" + op_name(d.op) +
                               ") needs " + std::to_string(n) + " pointer arguments, got " +
                               std::to_string(nptrs));
  };
  const bool acc = d.flags & IMEX_FLAG_ACCUMULATE;
  cudaError_t err = cudaSuccess;
  int launches = 1;
  switch (d.op) {
  case IMEX_OP_GEMM: {
    const bool has_bias = d.flags & IMEX_FLAG_BIAS;
    need(has_bias ? 4 : 3);
    if (d.out_dtype != IMEX_F32 && d.out_dtype != IMEX_BF16 && d.out_dtype != IMEX_F16)
      throw std::runtime_error("gpuLaunchKernel: gemm output must be f32, bf16 or f16");
    imex::GemmProblem g;
    g.A = ptrs[0];
    g.B = ptrs[1];
    g.C = static_cast<float *>(ptrs[2]);
    g.bias = has_bias ? static_cast<const float *>(ptrs[3]) : nullptr;
    g.M = d.dims[0];
    g.N = d.dims[1];
    g.K = d.dims[2];
    g.lda = d.dims[3];
    g.ldb = d.dims[4];
    g.ldc = d.dims[5];
    g.in_dtype = static_cast<int>(d.in_dtype);
    g.out_dtype = static_cast<int>(d.out_dtype);
    g.trans_a = d.flags & IMEX_FLAG_TRANS_A;
    g.trans_b = d.flags & IMEX_FLAG_TRANS_B;
    g.epilogue = static_cast<int>(d.epilogue);
    g.accumulate = acc;
    g.sm_margin = static_cast<int>(d.sm_margin);
    g.launched = &launches;
    if (g.M < 0 || g.N < 0 || g.K < 0) throw std::runtime_error("gpuLaunchKernel: negative gemm dims");
    if ((g.lda && g.lda < (g.trans_a ? g.M : g.K)) || (g.ldb && g.ldb < (g.trans_b ? g.K : g.N)) ||
        (g.ldc && g.ldc < g.N))
      throw std::runtime_error("gpuLaunchKernel: gemm row pitch smaller than the row");
    const bool force_simt = getenv("IMEX_B200_FORCE_SIMT_GEMM") != nullptr;
    bool done = false;
    if (!force_simt && imex::gemm_tcgen05_2cta_preferred(g)) {
      ensure_scratch(s, imex::gemm_tcgen05_workspace_bytes());
      g.workspace = s->scratch;
      g.workspace_bytes = s->scratch_bytes;
      s->last_kernel = "gemm_tcgen05_2cta";
      err = imex::launch_gemm_tcgen05_2cta(g, s->status_dev, s->stream);
      done = err != cudaErrorNotSupported;
    } else if (!force_simt && imex::gemm_tcgen05_supported(g)) {
      s->last_kernel = "gemm_tcgen05";
      err = imex::launch_gemm_tcgen05(g, s->status_dev, s->stream);
      done = err != cudaErrorNotSupported;
    }
    if (done) {
    } else if (d.in_dtype == IMEX_F32 || d.in_dtype == IMEX_BF16 || d.in_dtype == IMEX_F16) {
      s->last_kernel = "gemm_simt";
      err = imex::launch_gemm_simt(g, s->stream);
    } else {
      throw std::runtime_error("gpuLaunchKernel: gemm input type not supported");
    }
    break;
  }
  case IMEX_OP_SOFTMAX:
    need(2);
    if (d.in_dtype != d.out_dtype) throw std::runtime_error("gpuLaunchKernel: softmax keeps its element type");
    if (d.in_dtype == IMEX_F16 || d.in_dtype == IMEX_BF16) {
      s->last_kernel = "softmax_x16";
      err = imex::launch_softmax_x16(ptrs[0], ptrs[1], d.dims[0], d.dims[1], d.flags & IMEX_FLAG_SOFTMAX_NEG_INF,
                                     d.in_dtype == IMEX_BF16, s->stream);
      if (err == cudaErrorNotSupported)
        throw std::runtime_error("gpuLaunchKernel: 16-bit softmax rows hold at most 12288 values");
      break;
    }
    if (d.in_dtype != IMEX_F32) throw std::runtime_error("gpuLaunchKernel: softmax is f32, f16 or bf16");
    s->last_kernel = "softmax";
    err = imex::launch_softmax_f32(static_cast<const float *>(ptrs[0]), static_cast<float *>(ptrs[1]),
                                   d.dims[0], d.dims[1], d.flags & IMEX_FLAG_SOFTMAX_NEG_INF,
                                   s->stream);
    break;
  case IMEX_OP_REDUCE_ROWS:
    need(2);
    if (d.in_dtype != IMEX_F32) throw std::runtime_error("gpuLaunchKernel: reduce is f32 only");
    s->last_kernel = "reduce_rows";
    err = imex::launch_reduce_rows_f32(static_cast<const float *>(ptrs[0]),
                                       static_cast<float *>(ptrs[1]), d.dims[0], d.dims[1], acc,
                                       s->stream);
    break;
  case IMEX_OP_REDUCE_LEADING:
    need(2);
    if (d.in_dtype != IMEX_F32) throw std::runtime_error("gpuLaunchKernel: reduce is f32 only");
    s->last_kernel = "reduce_leading";
    err = imex::launch_reduce_leading_f32(static_cast<const float *>(ptrs[0]),
                                          static_cast<float *>(ptrs[1]), d.dims[0], d.dims[1], acc,
                                          s->stream);
    break;
  case IMEX_OP_REDUCE_ALL: {
    need(2);
    if (d.in_dtype != IMEX_F32) throw std::runtime_error("gpuLaunchKernel: reduce is f32 only");
    ensure_scratch(s, static_cast<size_t>(imex::reduce_all_partials(d.dims[0])) * sizeof(float));
    s->last_kernel = "reduce_all";
    launches = 2;
    err = imex::launch_reduce_all_f32(static_cast<const float *>(ptrs[0]),
                                      static_cast<float *>(ptrs[1]), d.dims[0], acc, s->scratch,
                                      s->stream);
    break;
  }
  case IMEX_OP_TRANSPOSE2D:
    need(2);
    s->last_kernel = "transpose2d";
    err = imex::launch_transpose2d(ptrs[0], ptrs[1], d.dims[0], d.dims[1],
                                   static_cast<int>(dtype_bytes(d.in_dtype)), s->stream);
    break;
  case IMEX_OP_TRANSPOSE3D: {
    need(2);
    if (d.in_dtype != d.out_dtype) throw std::runtime_error("gpuLaunchKernel: a transpose keeps its element type");
    const int64_t dims[3] = {d.dims[0], d.dims[1], d.dims[2]};
    const int perm[3] = {static_cast<int>(d.dims[3]), static_cast<int>(d.dims[4]),
                         static_cast<int>(d.dims[5])};
    int seen = 0;
    for (int q : perm) {
      if (q < 0 || q > 2) throw std::runtime_error("gpuLaunchKernel: bad transpose3d permutation");
      seen |= 1 << q;
    }
    if (seen != 7) throw std::runtime_error("gpuLaunchKernel: bad transpose3d permutation");
    s->last_kernel = "transpose3d";
    err = imex::launch_transpose3d(ptrs[0], ptrs[1], dims, perm, static_cast<int>(dtype_bytes(d.in_dtype)), s->stream);
    break;
  }
  case IMEX_OP_ELTWISE:
    need(2);
    if (d.in_dtype != d.out_dtype) {  // extf / truncf
      if (d.epilogue != IMEX_EPI_NONE)
        throw std::runtime_error("gpuLaunchKernel: a converting eltwise kernel takes no epilogue");
      s->last_kernel = "convert";
      err = imex::launch_convert(ptrs[0], ptrs[1], d.dims[0], static_cast<int>(d.in_dtype),
                                 static_cast<int>(d.out_dtype), s->stream);
      break;
    }
    if (d.in_dtype != IMEX_F32) throw std::runtime_error("gpuLaunchKernel: eltwise is f32 only");
    s->last_kernel = "eltwise";
    err = imex::launch_eltwise_f32(static_cast<const float *>(ptrs[0]), static_cast<float *>(ptrs[1]),
                                   d.dims[0], static_cast<int>(d.epilogue), s->stream);
    break;
  case IMEX_OP_EXPR: {
    // dims = {rows, cols, 32 bytes of postfix code}; pointers = inputs in order, then Y
    unsigned char code[IMEX_EXPR_MAX_CODE];
    std::memcpy(code, &d.dims[2], sizeof code);
    int n_inputs = 0;
    for (int i = 0; i < IMEX_EXPR_MAX_CODE && code[i] != IMEX_X_END; ++i)
      if (code[i] >= IMEX_X_IN && code[i] < IMEX_X_C0) n_inputs = std::max(n_inputs, (code[i] - 1) % 4 + 1);
    const int ncode = imex::expr_validate(code, IMEX_EXPR_MAX_CODE, n_inputs);
    if (ncode < 1) throw std::runtime_error("gpuLaunchKernel: malformed expression program");
    need(static_cast<size_t>(n_inputs) + 1);
    const bool reduce = d.flags & IMEX_FLAG_REDUCE_LEADING;
    if (reduce && d.out_dtype != d.in_dtype)
      throw std::runtime_error("gpuLaunchKernel: a reducing expression keeps its element type");
    // compiled for this program when NVRTC is there, interpreted otherwise
    s->last_kernel = reduce ? "expr_reduce_leading_jit" : "expr_jit";
    err = imex::launch_expr_jit(ptrs, n_inputs, ptrs[n_inputs], d.dims[0], d.dims[1], code, ncode,
                                d.fparams[0], d.fparams[1], static_cast<int>(d.in_dtype),
                                static_cast<int>(d.out_dtype), reduce, acc, s->stream);
    if (err == cudaErrorNotSupported) {
      s->last_kernel = reduce ? "expr_reduce_leading" : "expr";
      err = imex::launch_expr(ptrs, n_inputs, ptrs[n_inputs], d.dims[0], d.dims[1], code, ncode,
                              d.fparams[0], d.fparams[1], static_cast<int>(d.in_dtype),
                              static_cast<int>(d.out_dtype), reduce, acc, s->stream);
    }
    break;
  }
  case IMEX_OP_ATTENTION_FWD:
    need(4);
    if (d.in_dtype != d.out_dtype) throw std::runtime_error("gpuLaunchKernel: attention keeps its element type");
    if (!imex::flash_attention_supported(d.dims[0], d.dims[1], d.dims[2], static_cast<int>(d.in_dtype), ptrs[0],
                                         ptrs[1], ptrs[2], ptrs[3]))
      throw std::runtime_error("gpuLaunchKernel: attention needs f16/bf16, d_head 64 and 16-byte aligned arrays");
    s->last_kernel = "flash_attention_fwd";
    err = imex::launch_flash_attention_fwd(ptrs[0], ptrs[1], ptrs[2], ptrs[3], d.dims[0], d.dims[1], d.dims[2],
                                           d.fparams[0], static_cast<int>(d.in_dtype), s->status_dev, s->stream);
    break;
  case IMEX_OP_LOOPNEST: {
    const size_t want = static_cast<size_t>(d.dims[3]);
    if (want < 1 || want > 32) throw std::runtime_error("gpuLaunchKernel: loop-nest kernels take 1..32 pointers");
    need(want);
    if (!source || source->empty()) throw std::runtime_error("gpuLaunchKernel: loop-nest kernel without text");
    std::string log;
    s->last_kernel = "loopnest_jit";
    err = imex::launch_loopnest(source->data(), source->size(), ptrs, static_cast<int>(want), d.dims[0],
                                s->stream, &log);
    if (err == cudaErrorNotSupported)
      throw std::runtime_error(std::string("gpuLaunchKernel: the loop-nest kernel '") + d.name +
                               "' could not be compiled for sm_100a (there is no interpreter behind it): " + log);
    break;
  }
  case IMEX_OP_FILL_UNIFORM:
    need(1);
    s->last_kernel = "fill_uniform";
    err = imex::launch_fill_uniform(ptrs[0], d.dims[0], static_cast<int>(d.out_dtype),
                                    static_cast<uint64_t>(d.dims[1]), d.dims[2], d.fparams[0],
                                    d.fparams[1], s->stream);
    break;
  case IMEX_OP_FILL_NORMAL:
    need(1);
    s->last_kernel = "fill_normal";
    err = imex::launch_fill_normal(ptrs[0], d.dims[0], static_cast<int>(d.out_dtype),
                                   static_cast<uint64_t>(d.dims[1]), d.dims[2], d.fparams[0],
                                   d.fparams[1], s->stream);
    break;
  default:
    throw std::runtime_error("gpuLaunchKernel: unknown op");
  }
  check(err, (std::string("launch of ") + op_name(d.op)).c_str());
  g_launches.fetch_add(launches, std::memory_order_relaxed);
}

void check_status(Stream *s) {
  unsigned st = *reinterpret_cast<volatile unsigned *>(s->status_host);
  if (st != 0) {
    *s->status_host = 0;
    throw std::runtime_error("device kernel reported status " + std::to_string(st) +
                             " (a bounded wait ran out)");
  }
}

// The reference's profiling loop (LevelZeroRuntimeWrappers.cpp:521-597): warm-ups,
// then `rounds` timed launches, optionally flushing the last-level cache before
// each by writing a buffer twice its size; one statistics line on stdout.
void profile(Stream *s, const ImexKernelDesc &d, void **ptrs, size_t nptrs, const std::string *source) {
  long rounds = 1000, warmups = 3;
  if (const char *e = getenv("IMEX_PROFILING_RUNS")) {
    long v = strtol(e, nullptr, 10);
    if (v) rounds = v;
  }
  if (const char *e = getenv("IMEX_PROFILING_WARMUPS")) {
    long v = strtol(e, nullptr, 10);
    if (v >= 0) warmups = v;
  }
  const bool flush = getenv("IMEX_ENABLE_CACHE_FLUSHING") != nullptr;
  void *cache = nullptr;
  size_t cache_bytes = 0;
  if (flush) {
    int l2 = 0;
    CHECK_CUDA(cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, s->device));
    cache_bytes = 2 * static_cast<size_t>(l2);
    CHECK_CUDA(cudaMalloc(&cache, cache_bytes));
  }
  for (long r = 0; r < warmups; ++r) enqueue(s, d, ptrs, nptrs, source);
  cudaEvent_t e0, e1;
  CHECK_CUDA(cudaEventCreate(&e0));
  CHECK_CUDA(cudaEventCreate(&e1));
  std::vector<float> ms(static_cast<size_t>(rounds), 0.0f);
  for (long r = 0; r < rounds; ++r) {
    if (flush) CHECK_CUDA(cudaMemsetAsync(cache, 0, cache_bytes, s->stream));
    CHECK_CUDA(cudaEventRecord(e0, s->stream));
    enqueue(s, d, ptrs, nptrs, source);
    CHECK_CUDA(cudaEventRecord(e1, s->stream));
    CHECK_CUDA(cudaEventSynchronize(e1));
    CHECK_CUDA(cudaEventElapsedTime(&ms[static_cast<size_t>(r)], e0, e1));
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (cache) CHECK_CUDA(cudaFree(cache));
  fprintf(stdout,
          "the kernel execution time is (ms, on CUDA runtime):"
          "avg: %.4f, min: %.4f, max: %.4f, median: %4f, std_deviation: %4f, "
          "variance: %4f, P95: %4f, P5: %4f, median_one_third_avg: %4f (over "
          "%ld runs)\n",
          imex::calculateAverage(ms), imex::calculateMin(ms), imex::calculateMax(ms),
          imex::calculateMedian(ms), imex::calculateStdDev(ms), imex::calculateVariance(ms),
          imex::calculateP95(ms), imex::calculateP5(ms), imex::calculateMiddleThirdAverage(ms),
          rounds);
  fflush(stdout);
}

// Is this 8-byte parameter value the address of memory a kernel can read?  Allocations of
// this library are known; anything else is asked of the driver once and remembered.
bool is_device_pointer(Stream *s, void *v) {
  if (!v) return false;
  if (s->device_ptrs.count(v)) return true;
  bool yes = false;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    yes = g_allocs.count(v) != 0;
  }
  if (!yes) {
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, v) != cudaSuccess) {
      cudaGetLastError();  // an ordinary integer: not an error of the launch
      return false;
    }
    yes = a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged ||
          (a.type == cudaMemoryTypeHost && a.devicePointer != nullptr);
  }
  if (yes) {
    if (s->device_ptrs.size() > 4096) s->device_ptrs.clear();
    s->device_ptrs.insert(v);
  }
  return yes;
}

Event *launch(Stream *s, Kernel *k, size_t sharedMemBytes, ImexParamDesc *params,
              ImexEventDesc *deps) {
  if (!s || !k) throw std::runtime_error("gpuLaunchKernel: null stream or kernel");
  CHECK_CUDA(cudaSetDevice(s->device));
  size_t nparams = 0;
  if (params)
    while (!(params[nparams].data == nullptr && params[nparams].size == 0)) ++nparams;
  // the caller passes an i32; the last param is the local-memory placeholder then
  if ((sharedMemBytes & 0xFFFFFFFFu) != 0 && nparams > 0) --nparams;
  // The lowering passes memrefs as bare pointers and index scalars (loop bounds) by value,
  // both 8 bytes wide (GPUXToLLVMPass.cpp:571-584).  Only values that ARE device-accessible
  // memory count as the op's operands; an index that sits between two memrefs is skipped
  // instead of shifting the operands behind it.
  std::vector<void *> ptrs;
  for (size_t i = 0; i < nparams; ++i) {
    if (params[i].size == sizeof(void *) && params[i].data) {
      void *v;
      memcpy(&v, params[i].data, sizeof v);
      if (is_device_pointer(s, v)) ptrs.push_back(v);
    }
  }
  if (deps)
    for (size_t i = 0; deps[i].event; ++i) {
      auto *dep = static_cast<Event *>(deps[i].event);
      if (dep->ordered_on) {
        if (dep->ordered_on != s)
          throw std::runtime_error("gpuLaunchKernel: a launch captured into a CUDA graph cannot be waited for from "
                                   "another stream");
        continue;   // same stream: already ordered
      }
      CHECK_CUDA(cudaStreamWaitEvent(s->stream, dep->ev, 0));
    }
  for (void *p : ptrs) prefetch_managed(s, p);
  if (getenv("IMEX_ENABLE_PROFILING")) profile(s, k->desc, ptrs.data(), ptrs.size(), k->source);
  enqueue(s, k->desc, ptrs.data(), ptrs.size(), k->source);
  Event *ev = &s->events[s->next_event++ % kEventSlots];
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  CHECK_CUDA(cudaStreamIsCapturing(s->stream, &capturing));
  if (capturing == cudaStreamCaptureStatusActive) {
    ev->ordered_on = s;
    return ev;
  }
  ev->ordered_on = nullptr;
  if (!ev->ev) CHECK_CUDA(cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming));
  CHECK_CUDA(cudaEventRecord(ev->ev, s->stream));
  return ev;
}

thread_local Stream *t_default_stream = nullptr;
Stream *default_stream() {
  if (!t_default_stream) t_default_stream = make_stream(nullptr, nullptr);
  return t_default_stream;
}

} // namespace

extern "C" {

void *gpuCreateStream(void *device, void *context) {
  return catchAll([&]() -> void * {
    return make_stream(static_cast<const int32_t *>(device), static_cast<cudaStream_t>(context));
  });
}

void gpuStreamDestroy(void *stream) {
  catchAll([&]() { destroy_stream(static_cast<Stream *>(stream)); });
}

void *gpuMemAlloc(void *stream, size_t size, size_t alignment, bool isShared) {
  return catchAll(
      [&]() { return alloc_memory(static_cast<Stream *>(stream), size, alignment, isShared); });
}

void gpuMemFree(void *stream, void *ptr) {
  (void)stream;
  catchAll([&]() { free_memory(ptr); });
}

void gpuMemCopy(void *stream, void *dst, void *src, size_t size) {
  catchAll([&]() {
    auto *s = static_cast<Stream *>(stream);
    if (!size) return;
    if (s) {
      CHECK_CUDA(cudaSetDevice(s->device));
      CHECK_CUDA(cudaMemcpyAsync(dst, src, size, cudaMemcpyDefault, s->stream));
      CHECK_CUDA(cudaStreamSynchronize(s->stream));
    } else {
      CHECK_CUDA(cudaMemcpy(dst, src, size, cudaMemcpyDefault));
    }
  });
}

void gpuMemcpy(void *stream, void *dst, void *src, size_t size) {
  gpuMemCopy(stream, dst, src, size);
}

void *gpuModuleLoad(void *stream, const void *data, size_t dataSize) {
  (void)stream;
  return catchAll([&]() -> void * { return load_module(data, dataSize); });
}

void *gpuKernelGet(void *stream, void *module, const char *name) {
  (void)stream;
  return catchAll([&]() -> void * { return get_kernel(static_cast<Module *>(module), name); });
}

void *gpuLaunchKernel(void *stream, void *kernel, size_t gridX, size_t gridY, size_t gridZ,
                      size_t blockX, size_t blockY, size_t blockZ, size_t sharedMemBytes,
                      void *params, void *depEvents) {
  (void)gridX; (void)gridY; (void)gridZ; (void)blockX; (void)blockY; (void)blockZ;
  return catchAll([&]() -> void * {
    return launch(static_cast<Stream *>(stream), static_cast<Kernel *>(kernel), sharedMemBytes,
                  static_cast<ImexParamDesc *>(params), static_cast<ImexEventDesc *>(depEvents));
  });
}

void gpuWait(void *stream) {
  catchAll([&]() {
    auto *s = static_cast<Stream *>(stream);
    if (!s) throw std::runtime_error("gpuWait: null stream");
    CHECK_CUDA(cudaStreamSynchronize(s->stream));
    check_status(s);
  });
}

void gpuModuleUnload(void *module) { (void)module; /* modules are cached until exit */ }

// ---- upstream-style wrappers (LevelZeroRuntimeWrappers.cpp:673-741) --------
void *mgpuStreamCreate(void) {
  return catchAll([&]() -> void * { return make_stream(nullptr, nullptr); });
}
void mgpuStreamSynchronize(void *stream) { gpuWait(stream); }
void mgpuStreamDestroy(void *stream) { gpuStreamDestroy(stream); }
void *mgpuMemAlloc(size_t size, void *stream, bool isShared) {
  return catchAll([&]() {
    Stream *s = stream ? static_cast<Stream *>(stream) : default_stream();
    return alloc_memory(s, size, 64, isShared);
  });
}
void mgpuMemFree(void *stream, void *ptr) { gpuMemFree(stream, ptr); }
void *mgpuModuleLoad(const void *data, size_t dataSize) {
  return gpuModuleLoad(nullptr, data, dataSize);
}
void *mgpuModuleGetFunction(void *module, const char *name) {
  return gpuKernelGet(nullptr, module, name);
}
void mgpuModuleUnload(void *module) { (void)module; }
void mgpuLaunchKernel(void *kernel, size_t gridX, size_t gridY, size_t gridZ, size_t blockX,
                      size_t blockY, size_t blockZ, size_t sharedMemBytes, void *stream,
                      void **params, void **extra, size_t paramsCount) {
  (void)gridX; (void)gridY; (void)gridZ; (void)blockX; (void)blockY; (void)blockZ; (void)extra;
  catchAll([&]() {
    // every param is a pointer to a pointer-sized slot (LevelZeroRuntimeWrappers.cpp:697-699)
    std::vector<ImexParamDesc> descs(paramsCount + 1);
    for (size_t i = 0; i < paramsCount; ++i) descs[i] = ImexParamDesc{params[i], sizeof(void *)};
    descs[paramsCount] = ImexParamDesc{nullptr, 0};
    Stream *s = stream ? static_cast<Stream *>(stream) : default_stream();
    launch(s, static_cast<Kernel *>(kernel), sharedMemBytes, descs.data(), nullptr);
  });
}

// ---- additions ---------------------------------------------------------------
void *imexStreamNative(void *stream) {
  return stream ? static_cast<void *>(static_cast<Stream *>(stream)->stream) : nullptr;
}

void *imexStreamStatusWord(void *stream) {
  return stream ? static_cast<void *>(static_cast<Stream *>(stream)->status_dev) : nullptr;
}

void imexNoteLaunches(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void *imexEventRecord(void *stream) {
  return catchAll([&]() -> void * {
    auto *s = static_cast<Stream *>(stream);
    if (!s) throw std::runtime_error("imexEventRecord: null stream");
    auto *ev = new Event;
    CHECK_CUDA(cudaEventCreate(&ev->ev));
    CHECK_CUDA(cudaEventRecord(ev->ev, s->stream));
    return ev;
  });
}

float imexEventElapsedMs(void *startEvent, void *stopEvent) {
  return catchAll([&]() {
    auto *a = static_cast<Event *>(startEvent);
    auto *b = static_cast<Event *>(stopEvent);
    CHECK_CUDA(cudaEventSynchronize(b->ev));
    float ms = 0.f;
    CHECK_CUDA(cudaEventElapsedTime(&ms, a->ev, b->ev));
    return ms;
  });
}

uint64_t imexLaunchCount(void) { return g_launches.load(); }

const char *imexLastKernelName(void *stream) {
  return stream ? static_cast<Stream *>(stream)->last_kernel : "";
}

int64_t imexShardSize(int64_t shard, int64_t numShards, int64_t extent) {
  if (numShards <= 0 || shard < 0 || shard >= numShards || extent < 0) return -1;
  return extent / numShards + (shard >= numShards - (extent % numShards) ? 1 : 0);
}

int64_t imexShardOffset(int64_t shard, int64_t numShards, int64_t extent) {
  if (numShards <= 0 || shard < 0 || shard >= numShards || extent < 0) return -1;
  int64_t extra = shard - (numShards - (extent % numShards));
  return shard * (extent / numShards) + (extra > 0 ? extra : 0);
}

void imexSelfTestWaitTimeout(void *stream) {
  catchAll([&]() {
    auto *s = static_cast<Stream *>(stream);
    if (!s) throw std::runtime_error("imexSelfTestWaitTimeout: null stream");
    CHECK_CUDA(cudaSetDevice(s->device));
    check(imex::launch_wait_selftest(s->status_dev, s->stream), "launch of wait self-test");
    g_launches.fetch_add(1, std::memory_order_relaxed);
  });
}

float imexStat(int which, const float *values, size_t n) {
  std::vector<float> v(values, values + n);
  switch (which) {
  case 0: return imex::calculateAverage(v);
  case 1: return imex::calculateMin(v);
  case 2: return imex::calculateMax(v);
  case 3: return imex::calculateMedian(v);
  case 4: return imex::calculateStdDev(v);
  case 5: return imex::calculateVariance(v);
  case 6: return imex::calculateP95(v);
  case 7: return imex::calculateP5(v);
  case 8: return imex::calculateMiddleThirdAverage(v);
  }
  return -1.0f;
}

} // extern "C"
