// imex-b200-runner: runs a func/linalg MLIR program on the B200 runtime.
//
// It takes the place of the `imex-opt | mlir-runner` pair that the reference's
// imex-runner.py drives (tools/imex-runner/imex-runner.py.in:141-216): the
// entry function is interpreted on the host for its scaffolding (constants,
// tensor.empty, calls, casts, prints, timing loops) and every linalg op — or
// recognised chain of linalg ops — becomes one kernel-descriptor module that
// is executed with exactly the call sequence the reference's lowered host code
// uses (lib/Conversion/GPUXToLLVM/GPUXToLLVMPass.cpp:456-713):
//   gpuModuleLoad(blob) -> gpuKernelGet(name) -> gpuLaunchKernel(bare pointers)
//   -> gpuWait,  with gpuCreateStream once per function
//   (lib/Conversion/GPUToGPUX/GPUToGPUX.cpp:36-59) and gpuMemAlloc / gpuMemCopy
//   for every buffer (lib/Transforms/InsertGPUAllocs.cpp:376-469).
// Fusions: softmax chain -> one kernel; sigmoid+mul -> silu; matmul + relu/silu
// -> fused GEMM epilogue; extf producers of a matmul -> 16-bit GEMM inputs.
// IR that matches nothing is an error (exit 1): there is no CPU fallback.
//
//   imex-b200-runner FILE.mlir [-e main] [--entry-point-result=void]
//                    [--shared-libs=...] [--emit-plan] [--trace] [--all-loopnests]
//                    [--shard-rank R --shard-count N]
// --shard-rank / --shard-count: this process is rank R of the N ranks of the program's
//              shard.grid; tensors annotated `shard.shard ... split_axes = [[0]]` are held
//              and computed by rows, rank R owning its block of the partition rule.
// --emit-plan: recognise and print the kernels and ABI calls without touching
//              a GPU.   --trace (or IMEX_B200_TRACE=1): log ABI calls to stderr.
#include "../../../include/imex_b200_blob.h"
#include "../../../include/imex_cuda_runtime.h"
#include "../../../include/imex_runner_utils.h"
#include "gpu_kernels.h"
#include "host_loops.h"
#include "loopnest.h"
#include "mlir_text.h"
#include "recognise.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <memory>
#include <set>
#include <sstream>

using namespace imex::fe;

namespace {

bool g_plan = false;   // --emit-plan: no GPU calls
bool g_trace = false;  // log ABI calls
// --all-loopnests: recognise nothing; every linalg op becomes the loop nest that the
// reference's linalg-to-loops lowering makes of it (a self-check of the hot-path kernels
// against the plain lowering, and the mode the CPU checker under oracle/ runs in)
bool g_allLoopNests = false;
// --shard-rank R --shard-count N: this process is rank R of the N ranks of a shard.grid;
// values annotated `split_axes = [[0]]` hold only this rank's block of rows
int g_shardRank = 0, g_shardCount = 1;

[[noreturn]] void die(const std::string &msg) {
  std::cout.flush();
  std::cerr << "imex-b200-runner: error: " << msg << "\n";
  std::exit(1);
}

void trace(const std::string &line) {
  if (g_plan)
    std::cout << line << "\n";
  else if (g_trace)
    std::cerr << "[abi] " << line << "\n";
}

size_t eltBytes(const std::string &e) {
  if (e == "f32" || e == "i32") return 4;
  if (e == "f16" || e == "bf16" || e == "i16") return 2;
  if (e == "f64" || e == "i64" || e == "index") return 8;
  if (e == "i8" || e == "i1") return 1;
  die("element type " + e + " is not supported");
}

uint32_t dtypeCode(const std::string &e) {
  if (e == "f32") return IMEX_F32;
  if (e == "bf16") return IMEX_BF16;
  if (e == "f16") return IMEX_F16;
  if (e == "i32") return IMEX_I32;
  die("element type " + e + " has no kernel");
}

uint16_t f32ToBf16(float v) {
  uint32_t u;
  std::memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
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

float f16BitsToF32(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0x1f) u = sign | 0x7f800000u | (man << 13);
  else if (exp != 0) u = sign | ((exp + 112u) << 23) | (man << 13);
  else if (man == 0) u = sign;
  else {  // subnormal: normalise
    int e = -1;
    uint32_t m = man;
    do { ++e; m <<= 1; } while (!(m & 0x400u));
    u = sign | ((112u - e) << 23) | ((m & 0x3ffu) << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// ---- runtime values ---------------------------------------------------------
struct Buffer {  // a device allocation, freed with the last reference
  void *stream = nullptr;
  void *ptr = nullptr;
  size_t bytes = 0;
  bool hostVisible = false;  // memref.alloc / gpu.alloc host_shared: managed memory the host code reads and writes
  ~Buffer() {
    if (ptr && !g_plan) {
      trace("gpuMemFree");
      gpuMemFree(stream, ptr);
    }
  }
};

// A fused elementwise chain that has not been launched yet: leaves are device buffers.
struct XNode {
  enum { Leaf, Const, Unary, Binary } kind = Leaf;
  int opcode = 0;               // ImexExprCode of a Unary / Binary node
  double value = 0;             // Const
  std::shared_ptr<Buffer> buf;  // Leaf
  int mode = 0;                 // Leaf: 0 full tensor, 1 row vector, 2 column vector
  std::shared_ptr<XNode> a, b;
};
using XNodeP = std::shared_ptr<XNode>;

struct Value {
  enum { Empty, Scalar, Tensor } kind = Empty;
  Type type;
  double scalar = 0;
  std::shared_ptr<Buffer> buf;
  XNodeP lazy;  // set instead of buf while the chain producing this tensor is still open
  // what is known about the contents without reading them back
  bool isFill = false;
  double fillValue = 0;
  // >= 0: the tensor is split by rows over the ranks of a shard.grid; this is the extent of
  // dim 0 of the whole array, type.shape[0] the rows this rank holds
  int64_t globalRows = -1;
};

struct Sharding {  // a shard.sharding value
  std::string grid;
  std::vector<std::vector<int64_t>> splitAxes;
};

struct Frame {
  std::map<std::string, Value> vals;
  ConstantTable constants;
  std::map<std::string, Sharding> shardings;
};

class Runner {
public:
  Runner(const Module &m) : mod(m) {}

  void runEntry(const std::string &entry) {
    const Function *f = mod.find("@" + entry);
    if (!f) die("entry function @" + entry + " not found");
    if (f->isDeclaration) die("entry function has no body");
    if (!f->args.empty()) die("the entry function must take no arguments");
    call(*f, {});
  }

private:
  struct SoftmaxPlan {
    std::string x;
    const Op *sum = nullptr;
    bool negInf = false;
  };
  const Module &mod;
  std::map<const Op *, SoftmaxPlan> pendingSoftmax;  // keyed by the chain's final divide
  int kernelCounter = 0;
  void *curStream = nullptr;  // stream of the function being interpreted
  const std::map<std::string, int> *curUses = nullptr;  // use counts of that function (nested bodies included)
  std::vector<std::unique_ptr<std::vector<char>>> blobs;  // modules are cached by blob address

  // ---- device helpers ---------------------------------------------------
  // While a linalg op with a row-sharded operand runs: extent of the split dimension in the
  // whole array (G), rows of this rank (L) and their offset.  Results whose leading extent is
  // G are allocated with L rows and are row-sharded themselves.
  struct ShardCtx {
    bool active = false;
    int64_t G = 0, L = 0, r0 = 0;
  } curShard;

  Type localType(Type t) const {
    if (curShard.active && !t.shape.empty() && t.shape[0] == curShard.G) t.shape[0] = curShard.L;
    return t;
  }

  Value makeTensor(void *stream, const Type &declared) {
    const Type t = localType(declared);
    Value made = makeTensorExact(stream, t);
    // every tensor an op on a row-sharded operand makes is split the same way
    if (curShard.active && !declared.shape.empty() &&
        (declared.shape[0] == curShard.G || declared.shape[0] == curShard.L))
      made.globalRows = curShard.G;
    return made;
  }

  Value makeTensorExact(void *stream, const Type &t, bool hostVisible = false) {
    if (t.unranked) die("cannot allocate an unranked tensor");
    for (auto d : t.shape)
      if (d < 0) die("an array with an extent that is still unknown cannot be allocated (" + t.str() + ")");
    Value v;
    v.kind = Value::Tensor;
    v.type = t;
    v.buf = std::make_shared<Buffer>();
    v.buf->stream = stream;
    v.buf->bytes = static_cast<size_t>(t.count()) * eltBytes(t.elt);
    v.buf->hostVisible = hostVisible;
    trace("gpuMemAlloc(" + std::to_string(v.buf->bytes) + " bytes, align 64, " + (hostVisible ? "host_shared" : "device") +
          ")  // " + t.str());
    if (!g_plan) v.buf->ptr = gpuMemAlloc(stream, v.buf->bytes, 64, hostVisible);
    return v;
  }

  std::vector<char> encode(const Type &t, const std::vector<double> &vals, const Op *src) {
    const size_t n = static_cast<size_t>(t.count());
    std::vector<char> out(n * eltBytes(t.elt));
    for (size_t i = 0; i < n; ++i) {
      const size_t k = vals.size() == 1 ? 0 : i;
      double d = vals[k];
      const bool raw = src && src->isRaw.size() > k && src->isRaw[k];
      const uint64_t bits = raw ? src->rawBits[k] : 0;
      char *p = out.data() + i * eltBytes(t.elt);
      if (t.elt == "f32") {
        float f = static_cast<float>(d);
        if (raw) {
          uint32_t u = static_cast<uint32_t>(bits);
          std::memcpy(&f, &u, 4);
        }
        std::memcpy(p, &f, 4);
      } else if (t.elt == "bf16" || t.elt == "f16") {
        uint16_t h = raw ? static_cast<uint16_t>(bits)
                         : (t.elt == "bf16" ? f32ToBf16(static_cast<float>(d)) : f32ToF16(static_cast<float>(d)));
        std::memcpy(p, &h, 2);
      } else if (t.elt == "f64") {
        std::memcpy(p, &d, 8);
      } else if (t.elt == "i32") {
        int32_t x = static_cast<int32_t>(d);
        std::memcpy(p, &x, 4);
      } else if (t.elt == "i64" || t.elt == "index") {
        int64_t x = static_cast<int64_t>(d);
        std::memcpy(p, &x, 8);
      } else if (t.elt == "i16") {
        int16_t x = static_cast<int16_t>(d);
        std::memcpy(p, &x, 2);
      } else if (t.elt == "i8" || t.elt == "i1") {
        int8_t x = static_cast<int8_t>(d);
        std::memcpy(p, &x, 1);
      } else {
        die("constant of type " + t.elt + " is not supported");
      }
    }
    return out;
  }

  void upload(void *stream, Value &v, const std::vector<char> &host) {
    trace("gpuMemCopy(host -> device, " + std::to_string(host.size()) + " bytes)");
    if (!g_plan && !host.empty()) gpuMemCopy(stream, v.buf->ptr, const_cast<char *>(host.data()), host.size());
  }

  // One kernel: module with one descriptor, loaded, looked up, launched, waited for.
  void launch(void *stream, ImexKernelDesc d, const std::vector<void *> &ptrs, const std::string &what,
              const std::string &payload = std::string(), bool wait = true) {
    std::snprintf(d.name, sizeof d.name, "imex_b200_kernel_%d", kernelCounter++);
    auto blob = std::make_unique<std::vector<char>>(sizeof(ImexBlobHeader) + sizeof(ImexKernelDesc) + payload.size());
    ImexBlobHeader h{IMEX_BLOB_MAGIC, IMEX_BLOB_VERSION, 1};
    if (!payload.empty()) {  // kernel text behind the descriptor table
      d.dims[1] = static_cast<int64_t>(sizeof h + sizeof d);
      d.dims[2] = static_cast<int64_t>(payload.size());
      std::memcpy(blob->data() + sizeof h + sizeof d, payload.data(), payload.size());
    }
    std::memcpy(blob->data(), &h, sizeof h);
    std::memcpy(blob->data() + sizeof h, &d, sizeof d);
    std::ostringstream os;
    os << "kernel " << d.name << " = " << what << " dims=[" << d.dims[0] << "," << d.dims[1] << ","
       << d.dims[2] << "] epilogue=" << d.epilogue << " flags=" << d.flags;
    trace(os.str());
    trace(std::string("gpuModuleLoad(blob, ") + std::to_string(blob->size()) + " bytes)");
    trace(std::string("gpuKernelGet(\"") + d.name + "\")");
    trace("gpuLaunchKernel(" + std::to_string(ptrs.size()) + " pointer params)");
    if (wait) trace("gpuWait");
    if (!g_plan) {
      void *m = gpuModuleLoad(stream, blob->data(), blob->size());
      void *k = gpuKernelGet(stream, m, d.name);
      std::vector<void *> slots(ptrs);
      std::vector<ImexParamDesc> params;
      for (auto &s : slots) params.push_back(ImexParamDesc{&s, sizeof(void *)});
      params.push_back(ImexParamDesc{nullptr, 0});
      ImexEventDesc none[1] = {{nullptr}};
      gpuLaunchKernel(stream, k, 1, 1, 1, 1, 1, 1, 0, params.data(), none);
      if (wait) gpuWait(stream);  // a linalg op's launch is synchronous; gpu.launch_func has its own gpu.wait
    }
    blobs.push_back(std::move(blob));
  }

  ImexKernelDesc desc(uint32_t op, uint32_t in, uint32_t out) {
    ImexKernelDesc d;
    std::memset(&d, 0, sizeof d);
    d.op = op;
    d.in_dtype = in;
    d.out_dtype = out;
    return d;
  }

  // ---- function interpretation --------------------------------------------
  std::vector<Value> call(const Function &f, const std::vector<Value> &args) {
    Frame fr;
    for (size_t i = 0; i < f.args.size(); ++i) fr.vals[f.args[i]] = args[i];
    trace("gpuCreateStream(null, null)  // function " + f.name);
    void *stream = g_plan ? nullptr : gpuCreateStream(nullptr, nullptr);
    std::set<const Op *> absorbed;
    std::map<std::string, const Op *> defs;
    std::map<std::string, int> uses;
    index(f.body, defs, uses);
    void *outerStream = curStream;
    const std::map<std::string, int> *outerUses = curUses;
    curStream = stream;
    curUses = &uses;
    std::vector<Value> results = runBlock(f.body, fr, stream, absorbed, defs, uses);
    curStream = outerStream;
    curUses = outerUses;
    fr.vals.clear();  // frees this function's buffers (results hold their own references)
    if (!g_plan) {
      // results must outlive the stream handle they were allocated with
      for (auto &r : results)
        if (r.buf) r.buf->stream = nullptr;
    }
    trace("gpuStreamDestroy");
    if (!g_plan) gpuStreamDestroy(stream);
    return results;
  }

  // scf.while on the host: the "before" region decides (scf.condition) and forwards values, the
  // "do" region computes the next ones.  Each region is run as a block of its own; the values
  // that cross a region boundary are in device memory (no elementwise chain stays open across it).
  void whileOp(const Op &op, Frame &fr, void *stream) {
    const std::string where = "line " + std::to_string(op.line) + ": ";
    if (!op.body || !op.elseBody || op.elseBody->args.size() != op.resultTypes.size())
      die(where + "scf.while without its two regions");
    std::vector<Value> carried;
    for (auto &i : op.iterInits) carried.push_back(get(fr, i, op));
    std::map<std::string, const Op *> defsBefore, defsAfter;
    std::map<std::string, int> usesBefore, usesAfter;
    index(*op.body, defsBefore, usesBefore);
    index(*op.elseBody, defsAfter, usesAfter);
    const std::map<std::string, int> *outerUses = curUses;
    std::vector<Value> forwarded;
    for (int64_t it = 0;; ++it) {
      if (carried.size() != op.body->args.size()) die(where + "scf.while carries a different number of values than it declares");
      for (size_t k = 0; k < carried.size(); ++k) fr.vals[op.body->args[k]] = carried[k];
      std::set<const Op *> none;
      curUses = &usesBefore;
      std::vector<Value> c = runBlock(*op.body, fr, stream, none, defsBefore, usesBefore);
      if (c.empty() || c[0].kind != Value::Scalar) die(where + "the first region of scf.while must end in scf.condition");
      forwarded.assign(c.begin() + 1, c.end());
      if (forwarded.size() != op.elseBody->args.size()) die(where + "scf.condition forwards a different number of values");
      // a plan lists the launches of the loop once
      const bool again = g_plan ? it == 0 : c[0].scalar != 0;
      if (!again) break;
      for (size_t k = 0; k < forwarded.size(); ++k) fr.vals[op.elseBody->args[k]] = forwarded[k];
      none.clear();
      curUses = &usesAfter;
      carried = runBlock(*op.elseBody, fr, stream, none, defsAfter, usesAfter);
    }
    curUses = outerUses;
    for (size_t k = 0; k < op.results.size() && k < forwarded.size(); ++k) fr.vals[op.results[k]] = forwarded[k];
  }

  // tensors of the enclosing function that the region of a linalg.generic reads with
  // tensor.extract: uses that no operand list shows
  static void countCaptured(const Block &b, std::map<std::string, int> &uses) {
    for (auto &o : b.ops) {
      if (o->name == "tensor.extract" && !o->operands.empty()) uses[o->operands[0]]++;
      if (o->body) countCaptured(*o->body, uses);
      if (o->elseBody) countCaptured(*o->elseBody, uses);
    }
  }

  static void index(const Block &b, std::map<std::string, const Op *> &defs, std::map<std::string, int> &uses) {
    for (auto &o : b.ops) {
      for (auto &r : o->results) defs[r] = o.get();
      for (auto &v : o->operands) uses[v]++;
      for (auto &v : o->ins) uses[v]++;
      for (auto &v : o->outs) uses[v]++;
      for (auto &v : o->iterInits) uses[v]++;
      if (o->body && o->name == "scf.for") index(*o->body, defs, uses);
      if (o->body && o->name == "linalg.generic") countCaptured(*o->body, uses);
      if (o->name == "scf.while" && o->body && o->elseBody) {
        // uses only: a value of this block that a region of the loop reads has a use that is not
        // visible at this level (no fusion across it); the regions' own definitions are indexed
        // when they run
        std::map<std::string, const Op *> regionDefs;
        index(*o->body, regionDefs, uses);
        index(*o->elseBody, regionDefs, uses);
      }
    }
  }

  // The value with its contents in device memory (an open elementwise chain is launched).
  Value &get(Frame &fr, const std::string &name, const Op &at) {
    Value &v = peek(fr, name, at);
    if (v.lazy) materialise(v);
    return v;
  }
  // The value as it is: possibly an open elementwise chain (v.lazy) without a buffer.
  Value &peek(Frame &fr, const std::string &name, const Op &at) {
    auto it = fr.vals.find(name);
    if (it == fr.vals.end()) die("line " + std::to_string(at.line) + ": use of undefined value " + name);
    return it->second;
  }

  // ---- fused elementwise chains ---------------------------------------------------
  struct ExprProgram {
    std::vector<unsigned char> code;
    std::vector<std::shared_ptr<Buffer>> inputs;
    float consts[2] = {0, 0};
    int nconsts = 0;
  };
  // Postfix code of a tree; false when it needs more than the kernel has (4 inputs, two
  // free constants, 32 operations, 8 stack slots).
  bool emit(const XNodeP &n, ExprProgram &p, int &sp, int &maxsp) {
    switch (n->kind) {
    case XNode::Leaf: {
      size_t k = 0;
      for (; k < p.inputs.size(); ++k)
        if (p.inputs[k] == n->buf) break;
      if (k == p.inputs.size()) {
        if (k == IMEX_EXPR_MAX_INPUTS) return false;
        p.inputs.push_back(n->buf);
      }
      p.code.push_back(static_cast<unsigned char>((n->mode == 0 ? IMEX_X_IN : n->mode == 1 ? IMEX_X_ROWV : IMEX_X_COLV) + k));
      maxsp = std::max(maxsp, ++sp);
      break;
    }
    case XNode::Const: {
      const float f = static_cast<float>(n->value);
      if (f == 0.0f && !std::signbit(f)) p.code.push_back(IMEX_X_ZERO);
      else if (f == 1.0f) p.code.push_back(IMEX_X_ONE);
      else {
        int k = 0;
        for (; k < p.nconsts; ++k)
          if (std::memcmp(&p.consts[k], &f, 4) == 0) break;
        if (k == p.nconsts) {
          if (k == 2) return false;
          p.consts[p.nconsts++] = f;
        }
        p.code.push_back(static_cast<unsigned char>(IMEX_X_C0 + k));
      }
      maxsp = std::max(maxsp, ++sp);
      break;
    }
    case XNode::Unary:
      if (!emit(n->a, p, sp, maxsp)) return false;
      p.code.push_back(static_cast<unsigned char>(n->opcode));
      break;
    case XNode::Binary:
      if (!emit(n->a, p, sp, maxsp) || !emit(n->b, p, sp, maxsp)) return false;
      p.code.push_back(static_cast<unsigned char>(n->opcode));
      --sp;
      break;
    }
    return p.code.size() <= IMEX_EXPR_MAX_CODE && maxsp <= IMEX_EXPR_MAX_STACK;
  }
  bool compile(const XNodeP &tree, ExprProgram &p) {
    int sp = 0, maxsp = 0;
    return emit(tree, p, sp, maxsp);
  }
  static bool hasVectorLeaf(const XNodeP &n) {
    if (!n) return false;
    if (n->kind == XNode::Leaf) return n->mode != 0;
    return hasVectorLeaf(n->a) || hasVectorLeaf(n->b);
  }
  // Rows x columns the kernel walks: the tensor's own last dimension when a row or column
  // vector is broadcast along it, otherwise one long row (any rank, best vector width).
  static void shape2d(const Type &t, const XNodeP &tree, int64_t &rows, int64_t &cols) {
    if (hasVectorLeaf(tree)) {
      cols = t.shape.empty() ? 1 : t.shape.back();
      rows = cols ? t.count() / cols : 0;
    } else {
      rows = 1;
      cols = t.count();
    }
  }
  ImexKernelDesc exprDesc(const ExprProgram &p, const Type &in, uint32_t outDtype, int64_t rows, int64_t cols) {
    ImexKernelDesc d = desc(IMEX_OP_EXPR, dtypeCode(in.elt), outDtype);
    d.dims[0] = rows;
    d.dims[1] = cols;
    unsigned char code[IMEX_EXPR_MAX_CODE] = {0};
    std::memcpy(code, p.code.data(), p.code.size());
    std::memcpy(&d.dims[2], code, sizeof code);
    d.fparams[0] = p.consts[0];
    d.fparams[1] = p.consts[1];
    return d;
  }
  std::string exprText(const ExprProgram &p) {
    std::ostringstream os;
    os << "expr[" << p.code.size() << " ops, " << p.inputs.size() << " inputs]";
    return os.str();
  }
  // Launches the open chain of `v` into a fresh buffer.
  void materialise(Value &v) {
    ExprProgram p;
    if (!compile(v.lazy, p)) die("internal: an elementwise chain outgrew the fused kernel");
    Value out = makeTensorExact(curStream, v.type);
    int64_t rows, cols;
    shape2d(v.type, v.lazy, rows, cols);
    std::vector<void *> ptrs;
    for (auto &b : p.inputs) ptrs.push_back(b->ptr);
    ptrs.push_back(out.buf->ptr);
    launch(curStream, exprDesc(p, v.type, dtypeCode(v.type.elt), rows, cols), ptrs, exprText(p) + " " + v.type.elt);
    v.buf = out.buf;
    v.lazy.reset();
  }
  XNodeP substitute(const std::shared_ptr<ExprTree> &t, const std::vector<XNodeP> &operands) {
    auto n = std::make_shared<XNode>();
    switch (t->kind) {
    case ExprTree::Input:
      if (t->index < 0 || static_cast<size_t>(t->index) >= operands.size()) die("internal: operand index");
      return operands[t->index];
    case ExprTree::Const:
      n->kind = XNode::Const;
      n->value = t->value;
      return n;
    case ExprTree::Unary:
      n->kind = XNode::Unary;
      n->opcode = t->opcode;
      n->a = substitute(t->a, operands);
      return n;
    case ExprTree::Binary:
      n->kind = XNode::Binary;
      n->opcode = t->opcode;
      n->a = substitute(t->a, operands);
      n->b = substitute(t->b, operands);
      return n;
    }
    return n;
  }
  static XNodeP leaf(const Value &v, int mode) {
    auto n = std::make_shared<XNode>();
    n->kind = XNode::Leaf;
    n->buf = v.buf;
    n->mode = mode;
    return n;
  }
  // An elementwise generic outside the named chains: joins the chain of its operands; is
  // launched at once unless every user can take it over (another elementwise generic reading
  // it at the loop point, or the column reduce of kInputFusion.mlir.in:29-39).
  void elementwiseOp(const Op &op, const Block &b, Frame &fr, const std::string &where) {
    ElementwiseInfo info;
    const Type declaredT = op.resultTypes.empty() ? op.outsTypes[0] : op.resultTypes[0];
    const Type outT = localType(declaredT);
    bool fusable = classifyElementwise(op, fr.constants, info) &&
                   (outT.elt == "f32" || outT.elt == "f16" || outT.elt == "bf16");
    bool broadcast = false;
    for (int m : info.inputMode) broadcast = broadcast || m != 0;
    fusable = fusable && !(broadcast && outT.shape.size() != 2);
    for (size_t i = 0; fusable && i < op.ins.size(); ++i) {
      Value &v = peek(fr, op.ins[i], op);
      fusable = v.kind == Value::Tensor && v.type.elt == outT.elt;
    }
    if (!fusable) {  // outside what the fused elementwise kernel takes: a loop nest of its own
      loopNestOp(op, fr, curStream, where, "an elementwise body, operand type or broadcast the fused kernel lacks");
      return;
    }
    auto build = [&](bool inlineLazy) {
      std::vector<XNodeP> operands;
      for (size_t i = 0; i < op.ins.size(); ++i) {
        Value &v = peek(fr, op.ins[i], op);
        if (v.kind != Value::Tensor) die(where + "elementwise operand that is not a tensor");
        if (v.type.elt != outT.elt) die(where + "elementwise op mixing " + v.type.elt + " and " + outT.elt);
        int mode = info.inputMode[i];
        if (mode == 0 && v.type.count() != outT.count()) {
          // a row broadcast that was kept as its vector (see BroadcastRow) and is read here
          if (!v.lazy && v.type.shape.size() == 1 && outT.shape.size() == 2 && v.type.shape[0] == outT.shape[1])
            mode = 1;
          else
            die(where + "elementwise operand of another size than the result");
        }
        if (v.lazy && inlineLazy && mode == 0)
          operands.push_back(v.lazy);
        else
          operands.push_back(leaf(get(fr, op.ins[i], op), mode));
      }
      return substitute(info.tree, operands);
    };
    XNodeP tree = build(true);
    ExprProgram probe;
    if (!compile(tree, probe)) {
      tree = build(false);  // the operands' chains are launched on their own
      ExprProgram alone;
      if (!compile(tree, alone)) die(where + "elementwise body too large for one fused kernel");
    }
    Value out;
    out.kind = Value::Tensor;
    out.type = outT;
    out.lazy = tree;
    if (curShard.active && !declaredT.shape.empty() && declaredT.shape[0] == curShard.G) out.globalRows = curShard.G;
    const std::string res = op.results.empty() ? "" : op.results[0];
    bool defer = !res.empty() && (!curUses || allUsesVisible(res, b, *curUses));
    auto us = usersOf(res, b);
    defer = defer && !us.empty();
    for (auto *u : us) {
      bool ok = false;
      ElementwiseInfo ui;
      const Classified uc = classOf(u, fr);
      if (uc.kind == Kind::Elementwise || uc.kind == Kind::Add || uc.kind == Kind::Mul || uc.kind == Kind::Exp) {
        ok = classifyElementwise(*u, fr.constants, ui);
        for (size_t i = 0; ok && i < u->ins.size(); ++i)
          if (u->ins[i] == res) ok = ui.inputMode[i] == 0;
        for (auto &o : u->outs) ok = ok && o != res;
      } else if (uc.kind == Kind::ReduceLeading) {
        ok = u->ins.size() == 1 && u->ins[0] == res && outT.shape.size() == 2;
      }
      defer = defer && ok;
    }
    if (!defer) materialise(out);
    else trace("deferred: " + info.expr + "  // joins the next elementwise kernel");
    fr.vals[res] = out;
  }

  // linalg.matmul / matmul_transpose_a / _b / transpose written out as the linalg.generic they
  // stand for (multiply, then add to the output element; operands of another element type
  // are converted to the output's first, as the named ops define).
  std::unique_ptr<Op> namedOpAsGeneric(const Op &op, const std::string &where) {
    auto g = std::make_unique<Op>();
    g->name = "linalg.generic";
    g->line = op.line;
    g->results = op.results;
    g->resultTypes = op.resultTypes;
    g->ins = op.ins;
    g->insTypes = op.insTypes;
    g->outs = op.outs;
    g->outsTypes = op.outsTypes;
    g->body = std::make_unique<Block>();
    auto dimMap = [](int nd, std::vector<int> dims) {
      AffineMap m;
      m.numDims = nd;
      for (int d : dims) {
        MapResult r;
        r.value = d;
        r.expr = "d" + std::to_string(d);
        m.results.push_back(r);
      }
      return m;
    };
    auto scalarOp = [&](const std::string &name, const std::string &res, std::vector<std::string> operands,
                        const std::string &elt, const std::string &fromElt = "") {
      auto o = std::make_unique<Op>();
      o->name = name;
      o->results = {res};
      o->operands = std::move(operands);
      Type t;
      t.kind = Type::Scalar;
      t.elt = elt;
      o->resultTypes = {t};
      Type f = t;
      if (!fromElt.empty()) f.elt = fromElt;
      o->operandTypes = {f};
      g->body->ops.push_back(std::move(o));
    };
    auto yield = [&](const std::string &v) {
      auto o = std::make_unique<Op>();
      o->name = "linalg.yield";
      o->operands = {v};
      g->body->ops.push_back(std::move(o));
    };
    if (op.name == "linalg.matmul" || op.name == "linalg.matmul_transpose_a" || op.name == "linalg.matmul_transpose_b") {
      if (op.ins.size() != 2 || op.outs.size() != 1) die(where + "malformed " + op.name);
      const bool ta = op.name == "linalg.matmul_transpose_a", tb = op.name == "linalg.matmul_transpose_b";
      g->maps = {dimMap(3, ta ? std::vector<int>{2, 0} : std::vector<int>{0, 2}),
                 dimMap(3, tb ? std::vector<int>{1, 2} : std::vector<int>{2, 1}), dimMap(3, {0, 1})};
      g->iterators = {"parallel", "parallel", "reduction"};
      g->body->args = {"%a", "%b", "%c"};
      const std::string e = op.outsTypes[0].elt;
      const bool fl = e[0] == 'f' || e[0] == 'b';
      std::string a = "%a", bv = "%b";
      auto convert = [&](const std::string &v, const std::string &from) {
        if (from == e) return v;
        const bool ffrom = from[0] == 'f' || from[0] == 'b';
        const std::string name = ffrom && fl ? "arith.extf" : !ffrom && fl ? "arith.sitofp" : !ffrom ? "arith.extsi" : "";
        if (name.empty()) die(where + op.name + " converting " + from + " to " + e);
        scalarOp(name, v + "x", {v}, e, from);
        return v + "x";
      };
      a = convert(a, op.insTypes[0].elt);
      bv = convert(bv, op.insTypes[1].elt);
      scalarOp(fl ? "arith.mulf" : "arith.muli", "%m", {a, bv}, e);
      scalarOp(fl ? "arith.addf" : "arith.addi", "%s", {"%c", "%m"}, e);
      yield("%s");
    } else if (op.name == "linalg.transpose") {
      const int nd = static_cast<int>(op.reassociation.size());
      std::vector<int> ident, outDims(nd);
      for (int i = 0; i < nd; ++i) ident.push_back(i);
      // result dim i = input dim perm[i]: iterate over the input's dims, the output is indexed by them permuted
      std::vector<int> perm;
      for (auto &grp : op.reassociation) perm.push_back(static_cast<int>(grp[0]));
      g->maps = {dimMap(nd, ident), dimMap(nd, perm)};
      g->iterators.assign(nd, "parallel");
      g->body->args = {"%a", "%c"};
      yield("%a");
    } else if (op.name == "linalg.copy") {
      const int nd = static_cast<int>(op.outsTypes[0].shape.size());
      std::vector<int> ident;
      for (int i = 0; i < nd; ++i) ident.push_back(i);
      g->maps = {dimMap(nd, ident), dimMap(nd, ident)};
      g->iterators.assign(nd, "parallel");
      g->body->args = {"%a", "%c"};
      yield("%a");
    } else {
      die(where + op.name + " has no loop-nest form here");
    }
    return g;
  }

  // Any linalg.generic that is none of the recognised ops: the reference pipeline's own
  // lowering, a loop nest with its parallel loops on threads (loopnest.h).
  static bool hasDynamicExtent(const Op &op) {
    for (auto *types : {&op.insTypes, &op.outsTypes})
      for (auto &t : *types)
        for (auto d : t.shape)
          if (d < 0) return true;
    return false;
  }

  void loopNestOp(const Op &op, Frame &fr, void *stream, const std::string &where, const std::string &because) {
    LoopNestKernel k;
    std::string why;
    if (op.results.empty())
      die(where + "linalg ops on buffers (no results) are not supported: the runner works on tensors");
    // operand types as they are here: this rank's rows of a row-sharded array; the extents that
    // the IR leaves dynamic (tensor<?x?xf32>), taken from the values
    std::vector<Type> actual;
    const bool dynamic = hasDynamicExtent(op);
    if (curShard.active || dynamic) {
      for (size_t i = 0; i < op.ins.size(); ++i) {
        auto it = fr.vals.find(op.ins[i]);
        actual.push_back(it != fr.vals.end() && it->second.kind == Value::Tensor ? it->second.type : op.insTypes[i]);
      }
      for (size_t r = 0; r < op.outs.size(); ++r) {
        auto it = fr.vals.find(op.outs[r]);
        if (dynamic && it != fr.vals.end() && it->second.kind == Value::Tensor) actual.push_back(it->second.type);
        else actual.push_back(localType(op.outsTypes[r]));
      }
    }
    if (!buildLoopNest(op, fr.constants, k, why, actual.empty() ? nullptr : &actual))
      die(where + op.name + " is not a recognised hot-path op (" + because + ") and cannot be written as a loop nest (" +
          why + "); no CPU fallback");
    std::vector<void *> ptrs;
    for (int i : k.pointerInputs) ptrs.push_back(get(fr, op.ins[i], op).buf->ptr);
    std::vector<Value> outs;
    for (size_t r = 0; r < op.outs.size(); ++r) {
      const Type t = dynamic ? actual[op.ins.size() + r] : r < op.resultTypes.size() ? op.resultTypes[r] : op.outsTypes[r];
      Value out = makeTensor(stream, t);
      if (k.readsInit[r]) {
        Value &init = get(fr, op.outs[r], op);
        trace("gpuMemCopy(device -> device, " + std::to_string(out.buf->bytes) + " bytes)  // initial value of the result");
        if (!g_plan && out.buf->bytes) gpuMemCopy(stream, out.buf->ptr, init.buf->ptr, out.buf->bytes);
      }
      ptrs.push_back(out.buf->ptr);
      outs.push_back(out);
    }
    for (auto &name : k.captured) {  // tensors the region reads with tensor.extract
      Value &v = get(fr, name, op);
      if (v.kind != Value::Tensor) die(where + "tensor.extract from " + name + ", which is no tensor here");
      if (v.globalRows >= 0) die(where + "tensor.extract inside a region from " + name + ", which is split by rows over ranks");
      ptrs.push_back(v.buf->ptr);
    }
    ImexKernelDesc d = desc(IMEX_OP_LOOPNEST, 0, 0);
    d.dims[0] = k.threads;
    d.dims[3] = static_cast<int64_t>(ptrs.size());
    launch(stream, d, ptrs, k.summary, k.source);
    for (size_t r = 0; r < op.results.size() && r < outs.size(); ++r) fr.vals[op.results[r]] = outs[r];
  }

  // tensor.pad with static amounts and a constant padding value: one launch of a loop-nest kernel.
  void padOp(const Op &op, Frame &fr, void *stream) {
    const std::string where = "line " + std::to_string(op.line) + ": ";
    // the region yields the padding value: a constant of the enclosing function or of the region
    double value = 0.0;
    bool known = false;
    if (op.body && !op.body->ops.empty()) {
      std::map<std::string, double> local;
      for (auto &o : op.body->ops) {
        if (o->name == "arith.constant" && !o->numbers.empty() && !o->results.empty()) local[o->results[0]] = o->numbers[0];
        if (o->name == "tensor.yield" && o->operands.size() == 1) {
          auto it = local.find(o->operands[0]);
          if (it != local.end()) { value = it->second; known = true; }
          auto jt = fr.constants.find(o->operands[0]);
          if (!known && jt != fr.constants.end()) { value = jt->second; known = true; }
        }
      }
    }
    if (!known) die(where + "tensor.pad whose padding value is not a constant is not supported");
    if (op.reassociation.size() != 2) die(where + "tensor.pad without low / high amounts");
    Value &src = get(fr, op.operands[0], op);
    if (src.kind != Value::Tensor) die(where + "tensor.pad of a scalar");
    LoopNestKernel k;
    std::string why;
    if (!buildPad(src.type, op.resultTypes[0], op.reassociation[0], value, k, why)) die(where + "tensor.pad: " + why);
    for (size_t d = 0; d < op.reassociation[1].size(); ++d)
      if (src.type.shape[d] + op.reassociation[0][d] + op.reassociation[1][d] != op.resultTypes[0].shape[d])
        die(where + "tensor.pad: low + extent + high differs from the result's extent");
    Value out = makeTensorExact(stream, op.resultTypes[0], false);
    std::vector<void *> ptrs = {src.buf->ptr, out.buf->ptr};
    ImexKernelDesc d = desc(IMEX_OP_LOOPNEST, 0, 0);
    d.dims[0] = k.threads;
    d.dims[3] = 2;
    launch(stream, d, ptrs, k.summary, k.source);
    fr.vals[op.results[0]] = out;
  }

  // How often `v` is used by the top-level ops of `b`; fusions that make `v` disappear are
  // only sound when these are ALL its uses (none hidden inside a nested loop body).
  static int visibleUses(const std::string &v, const Block &b) {
    int n = 0;
    for (auto &o : b.ops) {
      for (auto &x : o->ins) n += x == v;
      for (auto &x : o->outs) n += x == v;
      for (auto &x : o->operands) n += x == v;
      for (auto &x : o->iterInits) n += x == v;
    }
    return n;
  }
  static bool allUsesVisible(const std::string &v, const Block &b, const std::map<std::string, int> &uses) {
    auto it = uses.find(v);
    return it == uses.end() || it->second == visibleUses(v, b);
  }

  // Makes `name` available now when it is defined LATER in the block by a chain of view ops
  // (expand / collapse / cast) over values that already exist: a fusion looking ahead (the
  // bias of a matmul, test/Jax/janet/jit__net_loss.91_linalg.mlir:25-39) may need it early.
  bool forceViewChain(const std::string &name, Frame &fr, std::map<std::string, const Op *> &defs, int depth = 0) {
    if (fr.vals.count(name)) return true;
    auto it = defs.find(name);
    if (it == defs.end() || depth > 8) return false;
    const Op &o = *it->second;
    const std::string &n = o.name;
    if (n != "tensor.expand_shape" && n != "tensor.collapse_shape" && n != "tensor.cast") return false;
    if (o.operands.empty() || !forceViewChain(o.operands[0], fr, defs, depth + 1)) return false;
    Value v = fr.vals[o.operands[0]];
    if (v.lazy) return false;
    if (!o.resultTypes[0].unranked) v.type = o.resultTypes[0];
    fr.vals[o.results[0]] = v;
    return true;
  }

  std::vector<Value> runBlock(const Block &b, Frame &fr, void *stream, std::set<const Op *> &absorbed,
                              std::map<std::string, const Op *> &defs, std::map<std::string, int> &uses) {
    for (auto &up : b.ops) {
      const Op &op = *up;
      if (absorbed.count(&op)) continue;
      const std::string &n = op.name;
      if (n == "return" || n == "func.return" || n == "scf.yield" || n == "scf.condition") {
        std::vector<Value> out;  // scf.condition: the condition, then the forwarded values
        for (auto &v : op.operands) out.push_back(get(fr, v, op));
        return out;
      }
      if (n == "arith.constant") {
        Value v;
        v.type = op.resultTypes[0];
        if (v.type.isShaped()) {
          v = makeTensor(stream, op.resultTypes[0]);
          if (op.denseSplat) {
            v.isFill = true;
            v.fillValue = op.numbers[0];
          }
          upload(stream, v, encode(v.type, op.numbers, &op));
        } else {
          v.kind = Value::Scalar;
          v.scalar = op.numbers[0];
          if (op.isRaw[0]) {  // a hex literal holds the bits of the value
            const uint64_t bits = op.rawBits[0];
            if (v.type.elt == "f32") {
              uint32_t u = static_cast<uint32_t>(bits);
              float f;
              std::memcpy(&f, &u, 4);
              v.scalar = f;
            } else if (v.type.elt == "f64") {
              double d;
              std::memcpy(&d, &bits, 8);
              v.scalar = d;
            } else if (v.type.elt == "bf16") {
              uint32_t u = static_cast<uint32_t>(bits) << 16;
              float f;
              std::memcpy(&f, &u, 4);
              v.scalar = f;
            } else if (v.type.elt == "f16") {
              v.scalar = f16BitsToF32(static_cast<uint16_t>(bits));
            } else {
              v.scalar = static_cast<double>(static_cast<int64_t>(bits));
            }
          }
          fr.constants[op.results[0]] = v.scalar;
        }
        fr.vals[op.results[0]] = v;
      } else if (n == "tensor.empty") {
        // tensor.empty(%d0, %d1) : tensor<?x?xf32> -- the operands are the dynamic extents, in order
        // (test/PlaidML/OpTest.EltwiseAdd.dynamic.mlir:17)
        Type t = op.resultTypes[0];
        size_t next = 0;
        for (auto &d : t.shape)
          if (d < 0) {
            if (next >= op.operands.size()) die("line " + std::to_string(op.line) + ": tensor.empty with too few extents");
            d = static_cast<int64_t>(get(fr, op.operands[next++], op).scalar);
          }
        fr.vals[op.results[0]] = makeTensor(stream, t);
      } else if (n == "tensor.dim") {
        // the extent the value has here: every value of the runner carries its actual shape
        const Value &t = get(fr, op.operands[0], op);
        const int64_t d = static_cast<int64_t>(get(fr, op.operands[1], op).scalar);
        if (t.kind != Value::Tensor || d < 0 || d >= static_cast<int64_t>(t.type.shape.size()))
          die("line " + std::to_string(op.line) + ": tensor.dim outside the rank of its operand");
        Value v;
        v.kind = Value::Scalar;
        v.type = op.resultTypes[0];
        v.scalar = static_cast<double>(t.type.shape[d]);
        fr.constants[op.results[0]] = v.scalar;
        fr.vals[op.results[0]] = v;
      } else if (n == "tensor.cast" || n == "memref.cast" || n == "bufferization.to_memref" ||
                 n == "bufferization.to_buffer" || n == "bufferization.to_tensor") {
        Value v = get(fr, op.operands[0], op);
        if (!op.resultTypes[0].unranked) {
          // a cast to a type with dynamic extents forgets them in the IR only: the value keeps its shape
          Type to = op.resultTypes[0];
          if (to.shape.size() == v.type.shape.size())
            for (size_t d = 0; d < to.shape.size(); ++d)
              if (to.shape[d] < 0) to.shape[d] = v.type.shape[d];
          v.type = to;
        }
        fr.vals[op.results[0]] = v;
      } else if (n == "tensor.expand_shape" || n == "tensor.collapse_shape") {
        Value v = get(fr, op.operands[0], op);  // contiguous: only the shape changes
        v.type = op.resultTypes[0];
        fr.vals[op.results[0]] = v;
      } else if (n == "tensor.pad") {
        padOp(op, fr, stream);
      } else if (n == "tensor.extract_slice") {
        const std::string where = "line " + std::to_string(op.line) + ": ";
        Value &src = get(fr, op.operands[0], op);
        if (src.kind != Value::Tensor || op.reassociation.size() != 3) die(where + "tensor.extract_slice of a scalar");
        LoopNestKernel k;
        std::string why;
        if (!buildSlice(src.type, op.resultTypes[0], op.reassociation[0], op.reassociation[1], op.reassociation[2], k, why))
          die(where + why);
        Value out = makeTensorExact(stream, op.resultTypes[0], false);
        std::vector<void *> ptrs = {src.buf->ptr, out.buf->ptr};
        ImexKernelDesc d = desc(IMEX_OP_LOOPNEST, 0, 0);
        d.dims[0] = k.threads;
        d.dims[3] = 2;
        launch(stream, d, ptrs, k.summary, k.source);
        fr.vals[op.results[0]] = out;
      } else if (n == "tensor.extract") {
        Value &t = get(fr, op.operands[0], op);
        if (t.type.count() != 1) die("line " + std::to_string(op.line) + ": tensor.extract of a non-scalar tensor");
        Value v;
        v.kind = Value::Scalar;
        v.type = op.resultTypes[0];
        if (t.isFill) {
          v.scalar = t.fillValue;
        } else if (!g_plan) {
          std::vector<char> host(t.buf->bytes);
          gpuMemCopy(stream, host.data(), t.buf->ptr, host.size());
          const std::string &e = t.type.elt;
          if (e == "f32") { float f; std::memcpy(&f, host.data(), 4); v.scalar = f; }
          else if (e == "f64") { std::memcpy(&v.scalar, host.data(), 8); }
          else if (e == "i1" || e == "i8") { v.scalar = static_cast<double>(static_cast<int8_t>(host[0])); }
          else if (e == "i32") { int32_t i; std::memcpy(&i, host.data(), 4); v.scalar = i; }
          else if (e == "i64" || e == "index") { int64_t i; std::memcpy(&i, host.data(), 8); v.scalar = static_cast<double>(i); }
          else die("line " + std::to_string(op.line) + ": tensor.extract of element type " + e);
        }
        fr.constants[op.results[0]] = v.scalar;
        fr.vals[op.results[0]] = v;
      } else if (n == "shard.sharding" || n == "mesh.sharding") {
        Sharding sh;
        sh.grid = op.callee;
        sh.splitAxes = op.reassociation;
        fr.shardings[op.results[0]] = sh;
      } else if (n == "shard.shard" || n == "mesh.shard") {
        shardOp(op, fr, stream);
      } else if (n == "memref.dealloc" || n == "gpu.dealloc") {
        fr.vals.erase(op.operands[0]);
      } else if (n == "call" || n == "func.call" || n == "llvm.call") {
        doCall(op, fr, stream);
      } else if (n == "gpu.alloc" || n == "memref.alloc" || n == "memref.alloca") {
        // host code's own arrays are memory both sides can touch (managed), as gpu.alloc
        // host_shared is (lib/Transforms/InsertGPUAllocs.cpp:376-412); gpu.alloc () is device memory
        const bool host = n != "gpu.alloc" || op.predicate == "host_shared";
        fr.vals[op.results[0]] = makeTensorExact(stream, op.resultTypes[0], host);
      } else if (n == "gpu.memcpy") {
        Value &dst = get(fr, op.operands[0], op), &src = get(fr, op.operands[1], op);
        if (dst.kind != Value::Tensor || src.kind != Value::Tensor || dst.buf->bytes != src.buf->bytes)
          die("line " + std::to_string(op.line) + ": gpu.memcpy between arrays of different sizes");
        trace("gpuMemCopy(" + std::string(src.buf->hostVisible ? "host" : "device") + " -> " +
              (dst.buf->hostVisible ? "host" : "device") + ", " + std::to_string(dst.buf->bytes) + " bytes)");
        if (!g_plan && dst.buf->bytes) gpuMemCopy(stream, dst.buf->ptr, src.buf->ptr, dst.buf->bytes);
      } else if (n == "gpu.wait") {
        trace("gpuWait");
        if (!g_plan) gpuWait(stream);
      } else if (n == "gpu.launch_func") {
        launchFunc(op, fr, stream);
      } else if (n == "memref.load" || n == "memref.store") {
        hostElement(op, fr);
      } else if (n == "memref.subview") {
        subview(op, fr, stream);
      } else if (n == "vector.print") {
        if (g_plan) continue;
        if (op.operands.empty()) {
          std::string out;  // the string attribute with its escapes resolved
          for (size_t i = 0; i < op.text.size(); ++i) {
            if (op.text[i] == '\\' && i + 1 < op.text.size()) {
              const char e = op.text[++i];
              out += e == 'n' ? '\n' : e == 't' ? '\t' : e;
            } else {
              out += op.text[i];
            }
          }
          std::cout << out;
        } else {
          const Value &v = get(fr, op.operands[0], op);
          const std::string &e = op.operandTypes[0].elt;
          if (e == "f32" || e == "f64") std::cout << v.scalar << "\n";
          else std::cout << static_cast<long long>(v.scalar) << "\n";
        }
        std::cout.flush();
      } else if (n == "scf.while") {
        whileOp(op, fr, stream);
      } else if (n == "scf.for" && op.iterArgs.empty() && hostLoop(op, fr)) {
        // ran as a compiled host loop nest (host_loops.h)
      } else if (n == "scf.for") {
        const int64_t lb = static_cast<int64_t>(get(fr, op.operands[0], op).scalar);
        const int64_t ub = static_cast<int64_t>(get(fr, op.operands[1], op).scalar);
        const int64_t st = static_cast<int64_t>(get(fr, op.operands[2], op).scalar);
        if (st <= 0) die("scf.for with a non-positive step");
        std::vector<Value> carried;
        for (auto &i : op.iterInits) carried.push_back(get(fr, i, op));
        for (int64_t i = lb; i < ub; i += st) {
          if (g_plan && i != lb) break;  // a plan lists each launch of a loop body once
          Value iv;
          iv.kind = Value::Scalar;
          iv.type.kind = Type::Scalar;
          iv.type.elt = "index";
          iv.scalar = static_cast<double>(i);
          fr.vals[op.body->args[0]] = iv;
          for (size_t k = 0; k < op.iterArgs.size(); ++k) fr.vals[op.iterArgs[k]] = carried[k];
          std::set<const Op *> inner;
          std::vector<Value> y = runBlock(*op.body, fr, stream, inner, defs, uses);
          if (!op.iterArgs.empty()) carried = y;
        }
        for (size_t k = 0; k < op.results.size(); ++k) fr.vals[op.results[k]] = carried[k];
      } else if (n == "linalg.fill") {
        Value &s = get(fr, op.ins[0], op);
        Value v = makeTensor(stream, op.resultTypes.empty() ? op.outsTypes[0] : op.resultTypes[0]);
        v.isFill = true;
        v.fillValue = s.scalar;
        upload(stream, v, encode(v.type, {s.scalar}, nullptr));
        if (!op.results.empty()) fr.vals[op.results[0]] = v;
      } else if (n.rfind("linalg.", 0) == 0) {
        linalgOp(op, b, fr, stream, absorbed, defs, uses);
      } else if (n.rfind("arith.", 0) == 0 || n.rfind("math.", 0) == 0) {
        scalarOp(op, fr);
      } else {
        die("line " + std::to_string(op.line) + ": operation " + n + " is not supported by the runner");
      }
    }
    return {};
  }

  // %1 = shard.shard %0 to %s: with `split_axes = [[0]]` (dim 0 over the grid's axis 0,
  // test/Dialect/NDArray/Extensions/sharding_propagation.mlir:9-12) the result is this rank's
  // block of rows by the partition rule of lib/Dialect/NDArray/Extensions/MeshShardingExtensions.cpp:
  // 74-100; an unsplit sharding (replication) leaves the value whole.
  void shardOp(const Op &op, Frame &fr, void *stream) {
    const std::string where = "line " + std::to_string(op.line) + ": ";
    if (op.operands.size() != 2) die(where + "shard.shard takes a value and a sharding");
    auto sit = fr.shardings.find(op.operands[1]);
    if (sit == fr.shardings.end()) die(where + "unknown sharding " + op.operands[1]);
    const Sharding &sh = sit->second;
    Value &x = get(fr, op.operands[0], op);
    bool split0 = false;
    for (size_t axis = 0; axis < sh.splitAxes.size(); ++axis) {
      if (sh.splitAxes[axis].empty()) continue;
      if (axis != 0 || sh.splitAxes[axis] != std::vector<int64_t>{0})
        die(where + "only row sharding (split_axes = [[0]]) is mapped onto the ranks; columns stay whole");
      split0 = true;
    }
    const Grid *grid = nullptr;
    for (auto &g : mod.grids)
      if (g.name == sh.grid) grid = &g;
    if (!grid) die(where + "unknown grid " + sh.grid);
    if (!split0 || g_shardCount == 1 || x.kind != Value::Tensor || x.globalRows >= 0) {
      fr.vals[op.results[0]] = x;  // replicated, a single rank, or already this rank's rows
      return;
    }
    if (grid->shape.empty() || (grid->shape[0] >= 0 && grid->shape[0] != g_shardCount))
      die(where + "grid " + sh.grid + " has " + (grid->shape.empty() ? std::string("no") : std::to_string(grid->shape[0])) +
          " ranks on its first axis but the runner was started with --shard-count " + std::to_string(g_shardCount));
    if (x.type.shape.empty()) die(where + "a rank-0 tensor cannot be split");
    const int64_t G = x.type.shape[0];
    const int64_t r0 = imexShardOffset(g_shardRank, g_shardCount, G), rows = imexShardSize(g_shardRank, g_shardCount, G);
    trace("shard: rows [" + std::to_string(r0) + ", " + std::to_string(r0 + rows) + ") of " + std::to_string(G) +
          " on rank " + std::to_string(g_shardRank) + " of " + std::to_string(g_shardCount));
    fr.vals[op.results[0]] = rowBlock(stream, x, r0, rows);
  }

  // ---- GPU-dialect host code (gpu.launch_func of a recognised kernel, host memrefs) ---------
  // gpu.launch_func @module::@kernel ... args(...): the gpu.func is XeGPU-dialect device code;
  // what it computes is recognised from its data flow (gpu_kernels.h) and served by the GEMM
  // kernels of this runtime through a descriptor, with the launch's arguments put in the
  // descriptor's pointer order.
  void launchFunc(const Op &op, Frame &fr, void *stream) {
    const std::string where = "line " + std::to_string(op.line) + ": ";
    const GpuKernel *k = nullptr;
    for (auto &g : mod.gpuKernels)
      if (g.module + "::" + g.name == op.callee) k = &g;
    if (!k) die(where + "gpu.launch_func of unknown kernel " + op.callee);
    if (k->args.size() != op.operands.size()) die(where + "argument count differs from the kernel's signature");
    GpuGemm g;
    std::string why;
    if (!recogniseGpuGemm(*k, g, why))
      die(where + "the gpu.func " + op.callee + " is not a kernel this runtime can stand in for (" + why +
          "); its device code is of another dialect and cannot be compiled for sm_100a");
    auto arg = [&](int i) -> Value & {
      Value &v = get(fr, op.operands[i], op);
      if (v.kind != Value::Tensor) die(where + "kernel argument " + op.operands[i] + " is not a memref");
      return v;
    };
    Value &A = arg(g.a), &Bv = arg(g.b), &C = arg(g.c);
    ImexKernelDesc d = desc(IMEX_OP_GEMM, dtypeCode(A.type.elt), dtypeCode(C.type.elt));
    d.dims[0] = g.M;
    d.dims[1] = g.N;
    d.dims[2] = g.K;
    if (g.transA) d.flags |= IMEX_FLAG_TRANS_A;
    if (g.transB) d.flags |= IMEX_FLAG_TRANS_B;
    if (g.readsC) d.flags |= IMEX_FLAG_ACCUMULATE;
    std::vector<void *> ptrs = {A.buf->ptr, Bv.buf->ptr, C.buf->ptr};
    if (g.bias >= 0) {
      d.flags |= IMEX_FLAG_BIAS;
      ptrs.push_back(arg(g.bias).buf->ptr);
    }
    launch(stream, d, ptrs,
           std::string("gemm ") + A.type.elt + "->" + C.type.elt + (g.transA ? " A^T" : "") + (g.transB ? " B^T" : "") +
               (g.bias >= 0 ? " +bias" : "") + (g.readsC ? " +C" : "") + "  // gpu.func " + op.callee,
           std::string(), /*wait=*/false);
  }

  // memref.load / memref.store executed one at a time (outside compiled loop nests)
  void hostElement(const Op &op, Frame &fr) {
    const bool ld = op.name == "memref.load";
    Value &m = get(fr, op.operands[ld ? 0 : 1], op);
    if (m.kind != Value::Tensor || !m.buf->hostVisible)
      die("line " + std::to_string(op.line) + ": " + op.name + " needs a host-visible memref (memref.alloc or gpu.alloc host_shared)");
    if (g_plan) {
      if (ld) {
        Value v;
        v.kind = Value::Scalar;
        v.type = op.resultTypes[0];
        fr.vals[op.results[0]] = v;
      }
      return;
    }
    const size_t first = ld ? 1 : 2;
    int64_t lin = 0;
    for (size_t i = first; i < op.operands.size(); ++i)
      lin = lin * m.type.shape[i - first] + static_cast<int64_t>(get(fr, op.operands[i], op).scalar);
    char *p = static_cast<char *>(m.buf->ptr);
    const std::string &e = m.type.elt;
    if (e != "f32" && e != "i32" && e != "f64" && e != "i64" && e != "index")
      die("line " + std::to_string(op.line) + ": single " + op.name + " of " + e + " (use it inside an scf.for nest)");
    if (ld) {
      Value v;
      v.kind = Value::Scalar;
      v.type = op.resultTypes[0];
      if (e == "f32") { float f; std::memcpy(&f, p + 4 * lin, 4); v.scalar = f; }
      else if (e == "i32") { int32_t x; std::memcpy(&x, p + 4 * lin, 4); v.scalar = x; }
      else if (e == "f64") { std::memcpy(&v.scalar, p + 8 * lin, 8); }
      else { int64_t x; std::memcpy(&x, p + 8 * lin, 8); v.scalar = static_cast<double>(x); }
      fr.constants[op.results[0]] = v.scalar;
      fr.vals[op.results[0]] = v;
    } else {
      const double val = get(fr, op.operands[0], op).scalar;
      if (e == "f32") { float f = static_cast<float>(val); std::memcpy(p + 4 * lin, &f, 4); }
      else if (e == "i32") { int32_t x = static_cast<int32_t>(val); std::memcpy(p + 4 * lin, &x, 4); }
      else if (e == "f64") { std::memcpy(p + 8 * lin, &val, 8); }
      else { int64_t x = static_cast<int64_t>(val); std::memcpy(p + 8 * lin, &x, 8); }
    }
  }

  // memref.subview of whole leading rows ([r0, 0, ..][n, full, ..][1, 1, ..]): a copy of the
  // contiguous block (the tests only print such views)
  void subview(const Op &op, Frame &fr, void *stream) {
    const std::string where = "line " + std::to_string(op.line) + ": ";
    Value &m = get(fr, op.operands[0], op);
    const auto &off = op.reassociation[0], &size = op.reassociation[1], &stride = op.reassociation[2];
    const size_t rank = m.type.shape.size();
    if (off.size() != rank || size.size() != rank || stride.size() != rank) die(where + "memref.subview rank mismatch");
    for (size_t d = 0; d < rank; ++d)
      if (stride[d] != 1 || (d > 0 && (off[d] != 0 || size[d] != m.type.shape[d])))
        die(where + "only subviews of whole leading rows are supported");
    Type t = m.type;
    t.shape[0] = size[0];
    Value v = makeTensorExact(stream, t, m.buf->hostVisible);
    const size_t rowBytes = m.type.shape[0] ? m.buf->bytes / static_cast<size_t>(m.type.shape[0]) : 0;
    trace("gpuMemCopy(" + std::to_string(v.buf->bytes) + " bytes)  // subview rows [" + std::to_string(off[0]) + ", " +
          std::to_string(off[0] + size[0]) + ")");
    if (!g_plan && v.buf->bytes)
      gpuMemCopy(stream, v.buf->ptr, static_cast<char *>(m.buf->ptr) + static_cast<size_t>(off[0]) * rowBytes, v.buf->bytes);
    fr.vals[op.results[0]] = v;
  }

  // An scf.for nest of scalar code over host-visible memrefs, compiled and run (host_loops.h);
  // false when it holds anything else (kernel launches, calls, tensors): the interpreter's.
  bool hostLoop(const Op &op, Frame &fr) {
    HostLoopProgram prog;
    std::string why;
    bool touchesArrays = false;
    auto lookup = [&](const std::string &name, double &scalar, HostArray &arr, bool &isArray) {
      auto it = fr.vals.find(name);
      if (it == fr.vals.end()) return false;
      const Value &v = it->second;
      if (v.kind == Value::Scalar) {
        scalar = v.scalar;
        isArray = false;
        return true;
      }
      if (v.kind != Value::Tensor || v.lazy || !v.buf || !v.buf->hostVisible) return false;
      arr.data = v.buf->ptr;
      arr.elt = v.type.elt;
      arr.shape = v.type.shape;
      isArray = true;
      touchesArrays = true;
      return true;
    };
    if (!prog.compile(op, lookup, why)) return false;
    if (!touchesArrays) return false;  // pure scalar loops stay with the interpreter (they bind results)
    trace("host loop nest at line " + std::to_string(op.line) + " (compiled)");
    if (!g_plan) {
      if (curStream) gpuWait(curStream);  // the device is done with what the host is about to touch
      prog.run();
    }
    return true;
  }

  void scalarOp(const Op &op, Frame &fr) {
    auto a = [&](size_t i) { return get(fr, op.operands[i], op).scalar; };
    Value v;
    v.kind = Value::Scalar;
    v.type = op.resultTypes[0];
    const std::string &n = op.name;
    if (n == "arith.addf" || n == "arith.addi") v.scalar = a(0) + a(1);
    else if (n == "arith.subf" || n == "arith.subi") v.scalar = a(0) - a(1);
    else if (n == "arith.mulf" || n == "arith.muli") v.scalar = a(0) * a(1);
    else if (n == "arith.divf") v.scalar = a(0) / a(1);
    else if (n == "arith.index_cast" || n == "arith.sitofp" || n == "arith.extf" || n == "arith.truncf") v.scalar = a(0);
    else die("line " + std::to_string(op.line) + ": scalar operation " + n + " outside a linalg body is not supported");
    fr.constants[op.results[0]] = v.scalar;
    fr.vals[op.results[0]] = v;
  }

  void doCall(const Op &op, Frame &fr, void *stream) {
    const std::string &c = op.callee;
    if (c == "@rtclock") {
      Value v;
      v.kind = Value::Scalar;
      v.type = op.resultTypes[0];
      v.scalar = g_plan ? 0.0 : rtclock();
      fr.vals[op.results[0]] = v;
      return;
    }
    if (c == "@printF64") { if (!g_plan) printF64(get(fr, op.operands[0], op).scalar); return; }
    if (c == "@printF32") { if (!g_plan) printF32(static_cast<float>(get(fr, op.operands[0], op).scalar)); return; }
    if (c == "@printNewline") { if (!g_plan) printNewline(); return; }
    static const std::set<std::string> kHostUtils = {
        "@fillResource1DF32", "@fillResource1DF16", "@fillResource1DBF16", "@fillResource1DRandomF32",
        "@fillResource1DRandomF16", "@fillResource1DRandomBF16", "@gemmF16F16F32", "@gemmF16F16F16",
        "@gemmBF16BF16F32"};
    if (kHostUtils.count(c)) {
      // runner-utils functions that write a memref (lib/ExecutionEngine/ImexRunnerUtils.cpp:38-50,
      // 217-338): they run on the host, on the array itself when the host can see it, else on a
      // copy that is written back
      if (g_plan) { trace("host call " + c); return; }
      struct HostView {
        std::vector<char> copy;
        std::vector<int64_t> words;
        ImexUnrankedMemRef u;
        Value *v = nullptr;
      };
      std::vector<std::unique_ptr<HostView>> views;
      std::vector<double> scalars;
      gpuWait(stream);
      for (size_t i = 0; i < op.operands.size(); ++i) {
        Value &v = get(fr, op.operands[i], op);
        if (v.kind == Value::Scalar) { scalars.push_back(v.scalar); continue; }
        auto h = std::make_unique<HostView>();
        h->v = &v;
        void *base = v.buf->ptr;
        if (!v.buf->hostVisible) {
          h->copy.resize(v.buf->bytes ? v.buf->bytes : 1);
          if (v.buf->bytes) gpuMemCopy(stream, h->copy.data(), v.buf->ptr, v.buf->bytes);
          base = h->copy.data();
        }
        const int64_t rank = static_cast<int64_t>(v.type.shape.size());
        h->words.assign(3 + 2 * rank, 0);
        std::memcpy(&h->words[0], &base, 8);
        std::memcpy(&h->words[1], &base, 8);
        int64_t stride = 1;
        for (int64_t d = rank - 1; d >= 0; --d) {
          h->words[3 + d] = v.type.shape[d];
          h->words[3 + rank + d] = stride;
          stride *= v.type.shape[d];
        }
        h->u = ImexUnrankedMemRef{rank, h->words.data()};
        views.push_back(std::move(h));
      }
      auto elt = [&](size_t i) { return views.at(i)->v->type.elt; };
      const std::string where = "line " + std::to_string(op.line) + ": ";
      if (c.rfind("@fillResource1DRandom", 0) == 0) {
        if (views.size() != 1 || scalars.size() != 3) die(where + c + " takes a memref, two bounds and a flag");
        const float lo = static_cast<float>(scalars[0]), hi = static_cast<float>(scalars[1]);
        const bool ints = scalars[2] != 0;
        if (elt(0) == "f32") _mlir_ciface_fillResource1DRandomF32(&views[0]->u, lo, hi, ints);
        else if (elt(0) == "f16") _mlir_ciface_fillResource1DRandomF16(&views[0]->u, lo, hi, ints);
        else if (elt(0) == "bf16") _mlir_ciface_fillResource1DRandomBF16(&views[0]->u, lo, hi, ints);
        else die(where + c + " of " + elt(0));
      } else if (c.rfind("@fillResource1D", 0) == 0) {
        if (views.size() != 1 || scalars.size() != 1) die(where + c + " takes a memref and a value");
        const float val = static_cast<float>(scalars[0]);
        if (elt(0) == "f32") _mlir_ciface_fillResource1DF32(&views[0]->u, val);
        else if (elt(0) == "f16") _mlir_ciface_fillResource1DF16(&views[0]->u, val);
        else if (elt(0) == "bf16") _mlir_ciface_fillResource1DBF16(&views[0]->u, val);
        else die(where + c + " of " + elt(0));
      } else {
        if (views.size() != 3) die(where + c + " takes three memrefs");
        if (c == "@gemmF16F16F32") _mlir_ciface_gemmF16F16F32(&views[0]->u, &views[1]->u, &views[2]->u);
        else if (c == "@gemmF16F16F16") _mlir_ciface_gemmF16F16F16(&views[0]->u, &views[1]->u, &views[2]->u);
        else if (c == "@gemmBF16BF16F32") _mlir_ciface_gemmBF16BF16F32(&views[0]->u, &views[1]->u, &views[2]->u);
        else die(where + "unknown host GEMM " + c);
      }
      for (auto &h : views)  // the functions write their first (fill) or last (gemm) memref
        if (!h->copy.empty() && h->v->buf->bytes) gpuMemCopy(stream, h->v->buf->ptr, h->copy.data(), h->v->buf->bytes);
      return;
    }
    if (c.rfind("@printAllclose", 0) == 0 || c.rfind("@printMaxError", 0) == 0) {
      // the reference's result checks (lib/ExecutionEngine/ImexRunnerUtils.cpp:185-255): both
      // tensors come back to the host and go to the runner-utils function of that name
      if (op.operands.size() != 2) die("line " + std::to_string(op.line) + ": " + c + " takes two tensors");
      Value &t = get(fr, op.operands[0], op), &r = get(fr, op.operands[1], op);
      trace("gpuMemCopy(device -> host, " + std::to_string(t.buf ? t.buf->bytes : 0) + " bytes)  // " + c);
      trace("gpuMemCopy(device -> host, " + std::to_string(r.buf ? r.buf->bytes : 0) + " bytes)  // " + c);
      if (g_plan) return;
      struct HostCopy {
        std::vector<char> data;
        std::vector<int64_t> words;
        ImexUnrankedMemRef u;
      };
      auto fetch = [&](Value &v, HostCopy &h) {
        h.data.resize(v.buf->bytes ? v.buf->bytes : 1);
        if (v.buf->bytes) gpuMemCopy(stream, h.data.data(), v.buf->ptr, v.buf->bytes);
        const int64_t rank = static_cast<int64_t>(v.type.shape.size());
        h.words.assign(3 + 2 * rank, 0);
        void *base = h.data.data();
        std::memcpy(&h.words[0], &base, 8);
        std::memcpy(&h.words[1], &base, 8);
        int64_t stride = 1;
        for (int64_t d = rank - 1; d >= 0; --d) {
          h.words[3 + d] = v.type.shape[d];
          h.words[3 + rank + d] = stride;
          stride *= v.type.shape[d];
        }
        h.u = ImexUnrankedMemRef{rank, h.words.data()};
      };
      HostCopy a, b;
      fetch(t, a);
      fetch(r, b);
      const std::string &e = t.type.elt;
      const bool close = c.rfind("@printAllclose", 0) == 0;
      if (r.type.elt != "f32") die("line " + std::to_string(op.line) + ": the reference tensor of " + c + " is f32");
      if (e == "f32") close ? _mlir_ciface_printAllcloseF32(&a.u, &b.u) : _mlir_ciface_printMaxErrorF32(&a.u, &b.u);
      else if (e == "f16") close ? _mlir_ciface_printAllcloseF16(&a.u, &b.u) : _mlir_ciface_printMaxErrorF16(&a.u, &b.u);
      else if (e == "bf16") close ? _mlir_ciface_printAllcloseBF16(&a.u, &b.u) : _mlir_ciface_printMaxErrorBF16(&a.u, &b.u);
      else die(c + " of element type " + e);
      return;
    }
    if (c.rfind("@printMemref", 0) == 0) {
      Value &t = get(fr, op.operands[0], op);
      trace("gpuMemCopy(device -> host, " + std::to_string(t.buf ? t.buf->bytes : 0) + " bytes)  // " + c);
      if (g_plan) return;
      std::vector<char> host(t.buf->bytes ? t.buf->bytes : 1);
      if (t.buf->bytes) gpuMemCopy(stream, host.data(), t.buf->ptr, t.buf->bytes);
      const int64_t rank = static_cast<int64_t>(t.type.shape.size());
      std::vector<int64_t> words(3 + 2 * rank);
      void *base = host.data();
      std::memcpy(&words[0], &base, 8);
      std::memcpy(&words[1], &base, 8);
      words[2] = 0;
      int64_t stride = 1;
      for (int64_t d = rank - 1; d >= 0; --d) {
        words[3 + d] = t.type.shape[d];
        words[3 + rank + d] = stride;
        stride *= t.type.shape[d];
      }
      ImexUnrankedMemRef u{rank, words.data()};
      const std::string &e = t.type.elt;
      if (e == "f32") _mlir_ciface_printMemrefF32(&u);
      else if (e == "i32") _mlir_ciface_printMemrefI32(&u);
      else if (e == "i64") _mlir_ciface_printMemrefI64(&u);
      else if (e == "bf16") _mlir_ciface_printMemrefBF16(&u);
      else if (e == "f16") _mlir_ciface_printMemrefF16(&u);
      else if (e == "f64") _mlir_ciface_printMemrefF64(&u);
      else die("printMemref of element type " + e);
      return;
    }
    const Function *f = mod.find(c);
    if (!f || f->isDeclaration) die("line " + std::to_string(op.line) + ": call to unknown function " + c);
    std::vector<Value> args;
    for (auto &v : op.operands) args.push_back(get(fr, v, op));
    std::vector<Value> res = call(*f, args);
    for (size_t i = 0; i < op.results.size() && i < res.size(); ++i) {
      if (res[i].buf) res[i].buf->stream = stream;
      fr.vals[op.results[i]] = res[i];
    }
  }

  // ---- linalg ops and their fusions ---------------------------------------------
  const Op *producer(const std::string &v, std::map<std::string, const Op *> &defs) {
    auto it = defs.find(v);
    return it == defs.end() ? nullptr : it->second;
  }
  Classified classOf(const Op *o, Frame &fr) {
    if (!o || o->name.rfind("linalg.", 0) != 0) return Classified();
    return classify(*o, fr.constants);
  }

  // The later ops of `b` that consume `v` (top level only).
  std::vector<const Op *> usersOf(const std::string &v, const Block &b) {
    std::vector<const Op *> out;
    for (auto &o : b.ops) {
      bool u = false;
      for (auto &x : o->ins) u = u || x == v;
      for (auto &x : o->outs) u = u || x == v;
      for (auto &x : o->operands) u = u || x == v;
      if (u) out.push_back(o.get());
    }
    return out;
  }

  // This rank's block of rows of `v` (whose dim 0 has extent G): a copy of the contiguous rows.
  Value rowBlock(void *stream, Value &whole, int64_t r0, int64_t rows) {
    if (whole.lazy) materialise(whole);
    Type t = whole.type;
    const int64_t G = t.shape[0];
    t.shape[0] = rows;
    Value v = makeTensorExact(stream, t);
    v.isFill = whole.isFill;
    v.fillValue = whole.fillValue;
    v.globalRows = G;
    const size_t rowBytes = G ? whole.buf->bytes / static_cast<size_t>(G) : 0;
    trace("gpuMemCopy(device -> device, " + std::to_string(v.buf->bytes) + " bytes)  // rows [" + std::to_string(r0) +
          ", " + std::to_string(r0 + rows) + ") of " + std::to_string(G) + ": this rank's block");
    if (!g_plan && v.buf->bytes)
      gpuMemCopy(stream, v.buf->ptr, static_cast<char *>(whole.buf->ptr) + static_cast<size_t>(r0) * rowBytes, v.buf->bytes);
    return v;
  }

  // A linalg op one of whose operands is split by rows over the ranks of a shard.grid
  // (shard.shard ... split_axes = [[0]]): every rank runs the op on its own rows.  The loop
  // dimension that walks the split rows must be a parallel one and must index dim 0 of every
  // operand it indexes at all; those operands (and the result) are taken, or allocated, with
  // this rank's rows only.  Anything that would need an exchange between the ranks — a
  // reduction over the split dimension, a transpose of it — is refused.
  void linalgOp(const Op &op, const Block &b, Frame &fr, void *stream, std::set<const Op *> &absorbed,
                std::map<std::string, const Op *> &defs, std::map<std::string, int> &uses) {
    auto where = "line " + std::to_string(op.line) + ": ";
    int sharded = -1;
    for (size_t i = 0; i < op.ins.size() && sharded < 0; ++i) {
      auto it = fr.vals.find(op.ins[i]);
      if (it != fr.vals.end() && it->second.globalRows >= 0) sharded = static_cast<int>(i);
    }
    if (sharded < 0) {
      linalgOpBody(op, b, fr, stream, absorbed, defs, uses);
      return;
    }
    const Value &sv = fr.vals[op.ins[sharded]];
    ShardCtx ctx;
    ctx.active = true;
    ctx.G = sv.globalRows;
    ctx.L = sv.type.shape[0];
    ctx.r0 = imexShardOffset(g_shardRank, g_shardCount, ctx.G);
    // which loop dimension walks the split rows, and which operands it indexes
    const size_t nIn = op.ins.size(), nAll = nIn + op.outs.size();
    std::vector<int> pos(nAll, -1);  // position of that dimension in each operand's map, -1: not used
    if (op.name == "linalg.matmul" || op.name == "linalg.matmul_transpose_b") {
      if (sharded != 0) die(where + "only the rows of A (and C) of a matmul can be split over ranks");
      pos[0] = 0;
      pos[nIn] = 0;
    } else if (op.name == "linalg.generic" && op.maps.size() == nAll) {
      const MapResult &r0 = op.maps[sharded].results.empty() ? MapResult() : op.maps[sharded].results[0];
      if (op.maps[sharded].results.empty() || !r0.simple || r0.isConst)
        die(where + "the split dimension of a row-sharded operand must be indexed by a plain loop dimension");
      const int sd = static_cast<int>(r0.value);
      if (op.iterators[sd] != "parallel")
        die(where + "a reduction over the dimension that is split over ranks needs an exchange between them: not supported");
      for (size_t k = 0; k < nAll; ++k)
        for (size_t r = 0; r < op.maps[k].results.size(); ++r) {
          const MapResult &mr = op.maps[k].results[r];
          if (!mr.simple) {
            if (mr.expr.find("d" + std::to_string(sd)) != std::string::npos)
              die(where + "the split dimension inside a compound index expression is not supported");
            continue;
          }
          if (!mr.isConst && mr.value == sd) {
            if (r != 0) die(where + "the dimension that is split over ranks must index dim 0 of every operand (no transposes of it)");
            pos[k] = 0;
          }
        }
    } else {
      die(where + op.name + " on a row-sharded operand is not supported");
    }
    if (pos[nIn] != 0) die(where + "the result of an op on a row-sharded operand must be split the same way");
    // operands the split dimension indexes but that are still whole: take this rank's rows
    std::vector<std::pair<std::string, Value>> saved;
    for (size_t k = 0; k < nAll; ++k) {
      if (pos[k] != 0) continue;
      const std::string &name = k < nIn ? op.ins[k] : op.outs[k - nIn];
      auto it = fr.vals.find(name);
      if (it == fr.vals.end() || it->second.kind != Value::Tensor || it->second.globalRows >= 0) continue;
      if (it->second.type.shape.empty() || it->second.type.shape[0] != ctx.G) continue;
      saved.emplace_back(name, it->second);
      Value local = rowBlock(stream, it->second, ctx.r0, ctx.L);
      fr.vals[name] = local;
    }
    curShard = ctx;
    linalgOpBody(op, b, fr, stream, absorbed, defs, uses);
    curShard = ShardCtx();
    for (auto &sv2 : saved) fr.vals[sv2.first] = sv2.second;
  }

  void linalgOpBody(const Op &op, const Block &b, Frame &fr, void *stream, std::set<const Op *> &absorbed,
                    std::map<std::string, const Op *> &defs, std::map<std::string, int> &uses) {
    auto where = "line " + std::to_string(op.line) + ": ";
    if (op.results.empty())
      die(where + "linalg ops on buffers (no results) are not supported: the runner works on tensors");
    if (hasDynamicExtent(op) && !g_allLoopNests) {
      // the hot-path kernels are chosen from the static types of the IR; an op whose extents are
      // only known when it is reached runs as the loop nest written for the shapes at hand
      if (op.name == "linalg.generic") {
        loopNestOp(op, fr, stream, where, "dynamic extents in its types");
      } else {
        std::unique_ptr<Op> g = namedOpAsGeneric(op, where);
        loopNestOp(*g, fr, stream, where, "dynamic extents in its types");
      }
      return;
    }
    Classified c = classify(op, fr.constants);
    if (g_allLoopNests) {
      if (op.name == "linalg.generic") {
        loopNestOp(op, fr, stream, where, "every op is lowered to its loop nest in this mode");
      } else {
        std::unique_ptr<Op> g = namedOpAsGeneric(op, where);
        loopNestOp(*g, fr, stream, where, "every op is lowered to its loop nest in this mode");
      }
      return;
    }
    if (c.kind == Kind::Unknown) {
      loopNestOp(op, fr, stream, where, c.why);
      return;
    }
    const std::string res = op.results.empty() ? "" : op.results[0];
    const Type outT = localType(op.resultTypes.empty() ? op.outsTypes[0] : op.resultTypes[0]);

    switch (c.kind) {
    case Kind::Matmul: {
      // inputs: fold extf producers (16-bit data extended to f32 feeds an f32 multiply-add)
      std::string aName = op.ins[0], bName = op.ins[1];
      std::string inElt = get(fr, aName, op).type.elt;
      const Op *pa = producer(aName, defs), *pb = producer(bName, defs);
      if (classOf(pa, fr).kind == Kind::ExtF && classOf(pb, fr).kind == Kind::ExtF) {
        // the extended tensors were never materialised: see ExtF below
        aName = pa->ins[0];
        bName = pb->ins[0];
        inElt = get(fr, aName, op).type.elt;
      }
      Value &A = get(fr, aName, op), &Bv = get(fr, bName, op);
      if (A.type.elt != Bv.type.elt) die(where + "matmul operands of different element types");
      if (outT.elt != "f32") {
        // e.g. an f16 multiply-add (test/PlaidML/CppEdsl.DotF16.mlir): every step rounds to the
        // element type, which an f32-accumulating GEMM would not reproduce; the loop nest does
        if (op.name == "linalg.generic") {
          loopNestOp(op, fr, stream, where, "matmul accumulating in " + outT.elt + ": f32 accumulate only on the GEMM kernels");
          break;
        }
        die(where + "matmul accumulating in " + outT.elt + " is not mapped to a GEMM (f32 accumulate only)");
      }
      Value &C0 = get(fr, op.outs[0], op);
      // stored shapes: A [M,K] ([K,M] when transposed), B [K,N] ([N,K] when transposed)
      const int64_t M = A.type.shape[c.transA ? 1 : 0], K = A.type.shape[c.transA ? 0 : 1];
      const int64_t N = Bv.type.shape[c.transB ? 0 : 1];
      if (Bv.type.shape[c.transB ? 1 : 0] != K || outT.shape[0] != M || outT.shape[1] != N)
        die(where + "matmul shape mismatch");
      // fusions behind the matmul, in the order the IR applies them:
      //   + bias   add(result, broadcast_row(v[N]))
      //   epilogue relu, or sigmoid(x) followed by mul(sigmoid, x)
      //   truncf   the f32 result rounded once to bf16 / f16
      std::string finalRes = res;
      const Value *biasV = nullptr;
      // a value may be folded into the launch only when every use of it is in this block
      auto fusableUsers = [&](const std::string &v) {
        return allUsesVisible(v, b, uses) ? usersOf(v, b) : std::vector<const Op *>();
      };
      auto us = fusableUsers(finalRes);
      if (us.size() == 1 && classOf(us[0], fr).kind == Kind::Add) {
        const std::string &other = us[0]->ins[0] == finalRes ? us[0]->ins[1] : us[0]->ins[0];
        const Op *bp = producer(other, defs);
        if (classOf(bp, fr).kind == Kind::BroadcastRow && allUsesVisible(other, b, uses) &&
            usersOf(other, b).size() == 1 && forceViewChain(bp->ins[0], fr, defs)) {
          const Value &v = get(fr, bp->ins[0], *bp);
          if (v.type.elt == "f32" && v.type.shape.size() == 1 && v.type.shape[0] == N) {
            biasV = &v;
            absorbed.insert(us[0]);
            absorbed.insert(bp);  // the broadcast itself: nothing to materialise
            finalRes = us[0]->results[0];
            us = fusableUsers(finalRes);
          }
        }
      }
      uint32_t epi = IMEX_EPI_NONE;
      if (us.size() == 1 && classOf(us[0], fr).kind == Kind::Relu) {
        epi = IMEX_EPI_RELU;
        absorbed.insert(us[0]);
        finalRes = us[0]->results[0];
        us = fusableUsers(finalRes);
      } else if (us.size() == 2 && classOf(us[0], fr).kind == Kind::Sigmoid &&
                 classOf(us[1], fr).kind == Kind::Mul && us[1]->ins[0] == us[0]->results[0] &&
                 us[1]->ins[1] == finalRes) {
        epi = IMEX_EPI_SILU;
        absorbed.insert(us[0]);
        absorbed.insert(us[1]);
        finalRes = us[1]->results[0];
        us = fusableUsers(finalRes);
      }
      Type finalT = outT;
      if (us.size() == 1 && classOf(us[0], fr).kind == Kind::TruncF) {
        finalT = us[0]->resultTypes.empty() ? us[0]->outsTypes[0] : us[0]->resultTypes[0];
        absorbed.insert(us[0]);
        finalRes = us[0]->results[0];
      }
      const bool zeroInit = C0.isFill && C0.fillValue == 0.0;
      if (!zeroInit && finalT.elt != "f32")
        die(where + "matmul with a non-zero f32 initial value and a 16-bit result is not mapped");
      Value out = makeTensor(stream, finalT);
      ImexKernelDesc d = desc(IMEX_OP_GEMM, dtypeCode(inElt), dtypeCode(finalT.elt));
      d.epilogue = epi;
      if (c.transA) d.flags |= IMEX_FLAG_TRANS_A;
      if (c.transB) d.flags |= IMEX_FLAG_TRANS_B;
      if (biasV) d.flags |= IMEX_FLAG_BIAS;
      if (!zeroInit) {  // C is also an input: start from a copy of it
        d.flags |= IMEX_FLAG_ACCUMULATE;
        trace("gpuMemCopy(device -> device, " + std::to_string(out.buf->bytes) + " bytes)  // C init");
        if (!g_plan) gpuMemCopy(stream, out.buf->ptr, C0.buf->ptr, out.buf->bytes);
      }
      d.dims[0] = M;
      d.dims[1] = N;
      d.dims[2] = K;
      std::vector<void *> ptrs = {A.buf->ptr, Bv.buf->ptr, out.buf->ptr};
      if (biasV) ptrs.push_back(biasV->buf->ptr);
      launch(stream, d, ptrs,
             std::string("gemm ") + inElt + "->" + finalT.elt + (c.transA ? " A^T" : "") + (c.transB ? " B^T" : "") +
                 (biasV ? " +bias" : "") + (epi == IMEX_EPI_RELU ? " +relu" : epi == IMEX_EPI_SILU ? " +silu" : ""));
      fr.vals[finalRes] = out;
      if (finalRes != res) fr.vals[res] = out;
      break;
    }
    case Kind::BroadcastRow: {
      // only as the bias of a matmul: nothing is materialised, the GEMM epilogue adds v[j]
      auto us = usersOf(res, b);
      bool feedsBias = !us.empty();
      for (auto *u : us) {
        bool okUser = classOf(u, fr).kind == Kind::Add;
        if (okUser) {
          const std::string &other = u->ins[0] == res ? u->ins[1] : u->ins[0];
          okUser = classOf(producer(other, defs), fr).kind == Kind::Matmul;
        }
        feedsBias = feedsBias && okUser;
      }
      if (!feedsBias) {  // a broadcast on its own: the fused elementwise kernel with a row-vector input
        elementwiseOp(op, b, fr, where);
        break;
      }
      fr.vals[res] = get(fr, op.ins[0], op);
      break;
    }
    case Kind::Add:
    case Kind::Elementwise:
      elementwiseOp(op, b, fr, where);
      break;
    case Kind::ExtF: {
      // as the producer of matmul operands only, nothing is materialised: the GEMM reads
      // the 16-bit data itself
      auto us = usersOf(res, b);
      bool feedsMatmul = !us.empty();
      for (auto *u : us) feedsMatmul = feedsMatmul && classOf(u, fr).kind == Kind::Matmul;
      if (feedsMatmul) {
        Value v = get(fr, op.ins[0], op);  // alias of the 16-bit tensor; the matmul looks through it
        fr.vals[res] = v;
        break;
      }
      [[fallthrough]];
    }
    case Kind::TruncF: {
      Value &X = get(fr, op.ins[0], op);
      Value out = makeTensor(stream, outT);
      ImexKernelDesc d = desc(IMEX_OP_ELTWISE, dtypeCode(X.type.elt), dtypeCode(outT.elt));
      d.dims[0] = X.type.count();
      launch(stream, d, {X.buf->ptr, out.buf->ptr}, std::string("convert ") + X.type.elt + "->" + outT.elt);
      fr.vals[res] = out;
      break;
    }
    case Kind::Relu:
    case Kind::Sigmoid: {
      if (peek(fr, op.ins[0], op).type.elt != "f32" || peek(fr, op.ins[0], op).lazy) {
        // f16 / bf16 (the benchmark grid's other dtypes) or part of an open chain: the fused
        // elementwise kernel, which rounds every operation to the element type
        elementwiseOp(op, b, fr, where);
        break;
      }
      Value &X = get(fr, op.ins[0], op);
      uint32_t epi = IMEX_EPI_RELU;
      std::string finalRes = res;
      if (c.kind == Kind::Sigmoid) {
        auto us = usersOf(res, b);
        if (us.size() == 1 && allUsesVisible(res, b, uses) && classOf(us[0], fr).kind == Kind::Mul &&
            us[0]->ins[0] == res && us[0]->ins[1] == op.ins[0]) {
          epi = IMEX_EPI_SILU;
          absorbed.insert(us[0]);
          finalRes = us[0]->results[0];
        } else {  // a sigmoid on its own: an elementwise kernel like any other
          elementwiseOp(op, b, fr, where);
          break;
        }
      }
      Value out = makeTensor(stream, outT);
      ImexKernelDesc d = desc(IMEX_OP_ELTWISE, IMEX_F32, IMEX_F32);
      d.epilogue = epi;
      d.dims[0] = X.type.count();
      launch(stream, d, {X.buf->ptr, out.buf->ptr}, epi == IMEX_EPI_RELU ? "relu" : "silu");
      fr.vals[finalRes] = out;
      break;
    }
    case Kind::RowMax: {
      // head of the softmax chain: max -> x - max -> exp -> sum -> divide
      const std::string x = op.ins[0];
      Value &X = get(fr, x, op);
      Value &init = get(fr, op.outs[0], op);
      const Op *sub = nullptr, *ex = nullptr, *sum = nullptr, *dv = nullptr;
      for (auto *u : usersOf(res, b))
        if (classOf(u, fr).kind == Kind::SubRowBcast && u->ins[0] == x && u->ins[1] == res) sub = u;
      if (sub)
        for (auto *u : usersOf(sub->results[0], b))
          if (classOf(u, fr).kind == Kind::Exp) ex = u;
      if (ex)
        for (auto *u : usersOf(ex->results[0], b)) {
          Kind k = classOf(u, fr).kind;
          if (k == Kind::RowSum) sum = u;
          if (k == Kind::DivRowBcast && u->ins[0] == ex->results[0]) dv = u;
        }
      const bool negInf = init.isFill && std::isinf(init.fillValue) && init.fillValue < 0;
      bool chain = sub && ex && sum && dv && dv->ins[1] == sum->results[0] && init.isFill &&
                   (negInf || init.fillValue <= -3.4e38) && X.type.shape.size() == 2 &&
                   (X.type.elt == "f32" || X.type.elt == "f16" || X.type.elt == "bf16");
      // the chain's temporaries disappear: all of their uses must be the chain's own
      chain = chain && allUsesVisible(res, b, uses) && usersOf(res, b).size() == 1 &&
              allUsesVisible(sub->results[0], b, uses) && usersOf(sub->results[0], b).size() == 1 &&
              allUsesVisible(ex->results[0], b, uses) && usersOf(ex->results[0], b).size() == 2 &&
              allUsesVisible(sum->results[0], b, uses) && usersOf(sum->results[0], b).size() == 1;
      if (!chain) {  // a row max on its own (test/PlaidML/OpTest.Max.mlir): a loop nest, one thread per row
        loopNestOp(op, fr, stream, where, "a row max that does not start a softmax chain");
        break;
      }
      // The chain runs as one kernel when its LAST op (the divide) is reached: the row
      // sum's initial tensor may be defined between here and there.
      for (const Op *o : {sub, ex, sum}) absorbed.insert(o);
      SoftmaxPlan plan;
      plan.x = x;
      plan.sum = sum;
      plan.negInf = negInf || c.rowMaxOgt;
      pendingSoftmax[dv] = plan;
      break;
    }
    case Kind::DivRowBcast: {
      auto it = pendingSoftmax.find(&op);
      if (it == pendingSoftmax.end()) {  // a row-broadcast divide on its own
        elementwiseOp(op, b, fr, where);
        break;
      }
      const SoftmaxPlan plan = it->second;
      pendingSoftmax.erase(it);
      Value &X = get(fr, plan.x, op);
      Value &sumInit = get(fr, plan.sum->outs[0], *plan.sum);
      if (!(sumInit.isFill && sumInit.fillValue == 0.0)) die(where + "softmax row sum must start from 0");
      Value out = makeTensor(stream, outT);
      ImexKernelDesc d = desc(IMEX_OP_SOFTMAX, dtypeCode(X.type.elt), dtypeCode(X.type.elt));
      if (plan.negInf) d.flags |= IMEX_FLAG_SOFTMAX_NEG_INF;
      d.dims[0] = X.type.shape[0];
      d.dims[1] = X.type.shape[1];
      launch(stream, d, {X.buf->ptr, out.buf->ptr}, X.type.elt == "f32" ? "softmax" : "softmax " + X.type.elt);
      fr.vals[res] = out;
      break;
    }
    case Kind::RowSum:
    case Kind::ReduceLeading:
    case Kind::ReduceAll: {
      Value &maybeOpen = peek(fr, op.ins[0], op);
      if (c.kind == Kind::ReduceLeading && maybeOpen.type.shape.size() >= 2 &&
          (maybeOpen.lazy || maybeOpen.type.elt != "f32")) {
        // an elementwise chain feeding the column sum (kInputFusion.mlir.in:6-41), or a
        // 16-bit input: one pass, every add rounded to the element type
        Value &init = get(fr, op.outs[0], op);
        if (init.type.elt != maybeOpen.type.elt) die(where + "reduction changing the element type");
        XNodeP tree = maybeOpen.lazy ? maybeOpen.lazy : leaf(maybeOpen, 0);
        ExprProgram p;
        if (!compile(tree, p)) die("internal: an elementwise chain outgrew the fused kernel");
        Value out = makeTensor(stream, outT);
        ImexKernelDesc d = exprDesc(p, maybeOpen.type, dtypeCode(outT.elt), maybeOpen.type.shape[0],
                                    maybeOpen.type.count() / maybeOpen.type.shape[0]);
        d.flags |= IMEX_FLAG_REDUCE_LEADING;
        if (!(init.isFill && init.fillValue == 0.0)) {
          d.flags |= IMEX_FLAG_ACCUMULATE;
          trace("gpuMemCopy(device -> device, " + std::to_string(out.buf->bytes) + " bytes)  // reduction init");
          if (!g_plan) gpuMemCopy(stream, out.buf->ptr, init.buf->ptr, out.buf->bytes);
        }
        std::vector<void *> ptrs;
        for (auto &bf : p.inputs) ptrs.push_back(bf->ptr);
        ptrs.push_back(out.buf->ptr);
        launch(stream, d, ptrs, exprText(p) + " " + outT.elt + " +reduce_leading");
        fr.vals[res] = out;
        break;
      }
      if (maybeOpen.type.elt != "f32") {  // integer and f64 sums: a loop nest (exact, ascending order)
        loopNestOp(op, fr, stream, where, "the sum kernels are f32 only");
        break;
      }
      Value &X = get(fr, op.ins[0], op);
      Value &init = get(fr, op.outs[0], op);
      Value out = makeTensor(stream, outT);
      uint32_t opc = c.kind == Kind::RowSum ? IMEX_OP_REDUCE_ROWS
                     : c.kind == Kind::ReduceLeading ? IMEX_OP_REDUCE_LEADING : IMEX_OP_REDUCE_ALL;
      ImexKernelDesc d = desc(opc, IMEX_F32, IMEX_F32);
      if (!(init.isFill && init.fillValue == 0.0)) {
        d.flags |= IMEX_FLAG_ACCUMULATE;
        trace("gpuMemCopy(device -> device, " + std::to_string(out.buf->bytes) + " bytes)  // reduction init");
        if (!g_plan) gpuMemCopy(stream, out.buf->ptr, init.buf->ptr, out.buf->bytes);
      }
      if (c.kind == Kind::RowSum) {
        d.dims[0] = X.type.shape[0];
        d.dims[1] = X.type.shape[1];
      } else if (c.kind == Kind::ReduceLeading) {
        d.dims[0] = X.type.shape[0];
        d.dims[1] = X.type.count() / X.type.shape[0];
      } else {
        d.dims[0] = X.type.count();
      }
      launch(stream, d, {X.buf->ptr, out.buf->ptr}, kindName(c.kind));
      fr.vals[res] = out;
      break;
    }
    case Kind::Transpose: {
      Value &X = get(fr, op.ins[0], op);
      const size_t eb = eltBytes(X.type.elt);
      Value out = makeTensor(stream, outT);
      const auto &sh = X.type.shape;
      if (sh.size() == 2 && c.perm == std::vector<int>{1, 0}) {
        ImexKernelDesc d = desc(IMEX_OP_TRANSPOSE2D, eb == 4 ? IMEX_F32 : IMEX_BF16, eb == 4 ? IMEX_F32 : IMEX_BF16);
        if (eb != 4 && eb != 2) die(where + "transpose of " + X.type.elt);
        d.dims[0] = sh[0];
        d.dims[1] = sh[1];
        launch(stream, d, {X.buf->ptr, out.buf->ptr}, "transpose2d");
      } else if (sh.size() == 3 && (eb == 4 || eb == 2)) {
        ImexKernelDesc d = desc(IMEX_OP_TRANSPOSE3D, eb == 4 ? IMEX_F32 : IMEX_BF16, eb == 4 ? IMEX_F32 : IMEX_BF16);
        for (int i = 0; i < 3; ++i) {
          d.dims[i] = sh[i];
          d.dims[3 + i] = c.perm[i];
        }
        launch(stream, d, {X.buf->ptr, out.buf->ptr}, "transpose3d");
      } else {  // other ranks and element widths: a loop nest (one thread per element)
        loopNestOp(op, fr, stream, where, "the transpose kernels take rank 2 and 3, 2- and 4-byte elements");
        break;
      }
      fr.vals[res] = out;
      break;
    }
    default: {
      elementwiseOp(op, b, fr, where);  // e.g. an exp or a mul on its own; a loop nest when all else fails
      break;
    }
    }
  }
};

std::string readFile(const std::string &path) {
  std::ifstream in(path);
  if (!in) die("cannot open " + path);
  std::stringstream ss;
  ss << in.rdbuf();
  return ss.str();
}

} // namespace

int main(int argc, char **argv) {
  std::string file, entry = "main";
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    if (a == "-e" && i + 1 < argc) entry = argv[++i];
    else if (a.rfind("-e=", 0) == 0) entry = a.substr(3);
    else if (a == "--emit-plan") g_plan = true;
    else if (a == "--all-loopnests") g_allLoopNests = true;
    else if (a == "--shard-rank" && i + 1 < argc) g_shardRank = std::atoi(argv[++i]);
    else if (a == "--shard-count" && i + 1 < argc) g_shardCount = std::atoi(argv[++i]);
    else if (a == "--trace") g_trace = true;
    else if (a.rfind("--entry-point-result", 0) == 0 || a.rfind("-entry-point-result", 0) == 0) {
      if (a.find("void") == std::string::npos) die("only --entry-point-result=void is supported");
    } else if (a.rfind("--shared-libs", 0) == 0 || a.rfind("-shared-libs", 0) == 0) {
      // accepted for command-line compatibility: the runtime libraries are linked in
    } else if (!a.empty() && a[0] == '-') {
      die("unknown option " + a);
    } else {
      file = a;
    }
  }
  if (std::getenv("IMEX_B200_TRACE")) g_trace = true;
  if (std::getenv("IMEX_B200_ALL_LOOPNESTS")) g_allLoopNests = true;
  if (g_shardCount < 1 || g_shardRank < 0 || g_shardRank >= g_shardCount) die("--shard-rank must lie in [0, --shard-count)");
  if (file.empty()) die("usage: imex-b200-runner FILE.mlir [-e main] [--entry-point-result=void] [--emit-plan]");
  try {
    Module m = parseModule(readFile(file));
    Runner(m).runEntry(entry);
  } catch (const ParseError &e) {
    die(file + ": " + e.what());
  }
  return 0;
}
