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
//                    [--shared-libs=...] [--emit-plan] [--trace]
// --emit-plan: recognise and print the kernels and ABI calls without touching
//              a GPU.   --trace (or IMEX_B200_TRACE=1): log ABI calls to stderr.
#include "../../../include/imex_b200_blob.h"
#include "../../../include/imex_cuda_runtime.h"
#include "../../../include/imex_runner_utils.h"
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

// ---- runtime values ---------------------------------------------------------
struct Buffer {  // a device allocation, freed with the last reference
  void *stream = nullptr;
  void *ptr = nullptr;
  size_t bytes = 0;
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
};

struct Frame {
  std::map<std::string, Value> vals;
  ConstantTable constants;
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
  std::vector<std::unique_ptr<std::vector<char>>> blobs;  // modules are cached by blob address

  // ---- device helpers ---------------------------------------------------
  Value makeTensor(void *stream, const Type &t) {
    if (t.unranked) die("cannot allocate an unranked tensor");
    for (auto d : t.shape)
      if (d < 0) die("dynamic shapes are not supported: kernel arguments carry no shape");
    Value v;
    v.kind = Value::Tensor;
    v.type = t;
    v.buf = std::make_shared<Buffer>();
    v.buf->stream = stream;
    v.buf->bytes = static_cast<size_t>(t.count()) * eltBytes(t.elt);
    trace("gpuMemAlloc(" + std::to_string(v.buf->bytes) + " bytes, align 64, device)  // " + t.str());
    if (!g_plan) v.buf->ptr = gpuMemAlloc(stream, v.buf->bytes, 64, false);
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
  void launch(void *stream, ImexKernelDesc d, const std::vector<void *> &ptrs, const std::string &what) {
    std::snprintf(d.name, sizeof d.name, "imex_b200_kernel_%d", kernelCounter++);
    auto blob = std::make_unique<std::vector<char>>(sizeof(ImexBlobHeader) + sizeof(ImexKernelDesc));
    ImexBlobHeader h{IMEX_BLOB_MAGIC, IMEX_BLOB_VERSION, 1};
    std::memcpy(blob->data(), &h, sizeof h);
    std::memcpy(blob->data() + sizeof h, &d, sizeof d);
    std::ostringstream os;
    os << "kernel " << d.name << " = " << what << " dims=[" << d.dims[0] << "," << d.dims[1] << ","
       << d.dims[2] << "] epilogue=" << d.epilogue << " flags=" << d.flags;
    trace(os.str());
    trace(std::string("gpuModuleLoad(blob, ") + std::to_string(blob->size()) + " bytes)");
    trace(std::string("gpuKernelGet(\"") + d.name + "\")");
    trace("gpuLaunchKernel(" + std::to_string(ptrs.size()) + " pointer params)");
    trace("gpuWait");
    if (!g_plan) {
      void *m = gpuModuleLoad(stream, blob->data(), blob->size());
      void *k = gpuKernelGet(stream, m, d.name);
      std::vector<void *> slots(ptrs);
      std::vector<ImexParamDesc> params;
      for (auto &s : slots) params.push_back(ImexParamDesc{&s, sizeof(void *)});
      params.push_back(ImexParamDesc{nullptr, 0});
      ImexEventDesc none[1] = {{nullptr}};
      gpuLaunchKernel(stream, k, 1, 1, 1, 1, 1, 1, 0, params.data(), none);
      gpuWait(stream);
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
    curStream = stream;
    std::vector<Value> results = runBlock(f.body, fr, stream, absorbed, defs, uses);
    curStream = outerStream;
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

  static void index(const Block &b, std::map<std::string, const Op *> &defs, std::map<std::string, int> &uses) {
    for (auto &o : b.ops) {
      for (auto &r : o->results) defs[r] = o.get();
      for (auto &v : o->operands) uses[v]++;
      for (auto &v : o->ins) uses[v]++;
      for (auto &v : o->outs) uses[v]++;
      if (o->body && o->name == "scf.for") index(*o->body, defs, uses);
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
    Value out = makeTensor(curStream, v.type);
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
    if (!classifyElementwise(op, fr.constants, info))
      die(where + op.name + " is not a recognised hot-path op; no CPU fallback");
    const Type outT = op.resultTypes.empty() ? op.outsTypes[0] : op.resultTypes[0];
    if (outT.elt != "f32" && outT.elt != "f16" && outT.elt != "bf16") die(where + "elementwise ops on " + outT.elt);
    bool broadcast = false;
    for (int m : info.inputMode) broadcast = broadcast || m != 0;
    if (broadcast && outT.shape.size() != 2) die(where + "broadcasting elementwise ops are rank 2 only");
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
    const std::string res = op.results.empty() ? "" : op.results[0];
    bool defer = !res.empty();
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

  std::vector<Value> runBlock(const Block &b, Frame &fr, void *stream, std::set<const Op *> &absorbed,
                              std::map<std::string, const Op *> &defs, std::map<std::string, int> &uses) {
    for (auto &up : b.ops) {
      const Op &op = *up;
      if (absorbed.count(&op)) continue;
      const std::string &n = op.name;
      if (n == "return" || n == "func.return" || n == "scf.yield") {
        std::vector<Value> out;
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
          if (op.isRaw[0] && v.type.elt == "f32") {
            uint32_t u = static_cast<uint32_t>(op.rawBits[0]);
            float f;
            std::memcpy(&f, &u, 4);
            v.scalar = f;
          }
          fr.constants[op.results[0]] = v.scalar;
        }
        fr.vals[op.results[0]] = v;
      } else if (n == "tensor.empty") {
        fr.vals[op.results[0]] = makeTensor(stream, op.resultTypes[0]);
      } else if (n == "tensor.cast" || n == "memref.cast" || n == "bufferization.to_memref" ||
                 n == "bufferization.to_buffer" || n == "bufferization.to_tensor") {
        Value v = get(fr, op.operands[0], op);
        if (!op.resultTypes[0].unranked) v.type = op.resultTypes[0];
        fr.vals[op.results[0]] = v;
      } else if (n == "tensor.expand_shape" || n == "tensor.collapse_shape") {
        Value v = get(fr, op.operands[0], op);  // contiguous: only the shape changes
        v.type = op.resultTypes[0];
        fr.vals[op.results[0]] = v;
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
          float f = 0;
          if (t.type.elt == "f32") std::memcpy(&f, host.data(), 4);
          else die("tensor.extract supports f32 only");
          v.scalar = f;
        }
        fr.constants[op.results[0]] = v.scalar;
        fr.vals[op.results[0]] = v;
      } else if (n == "memref.dealloc" || n == "gpu.dealloc") {
        fr.vals.erase(op.operands[0]);
      } else if (n == "call" || n == "func.call" || n == "llvm.call") {
        doCall(op, fr, stream);
      } else if (n == "scf.for") {
        const int64_t lb = static_cast<int64_t>(get(fr, op.operands[0], op).scalar);
        const int64_t ub = static_cast<int64_t>(get(fr, op.operands[1], op).scalar);
        const int64_t st = static_cast<int64_t>(get(fr, op.operands[2], op).scalar);
        if (st <= 0) die("scf.for with a non-positive step");
        std::vector<Value> carried;
        for (auto &i : op.iterInits) carried.push_back(get(fr, i, op));
        for (int64_t i = lb; i < ub; i += st) {
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

  void linalgOp(const Op &op, const Block &b, Frame &fr, void *stream, std::set<const Op *> &absorbed,
                std::map<std::string, const Op *> &defs, std::map<std::string, int> &uses) {
    Classified c = classify(op, fr.constants);
    auto where = "line " + std::to_string(op.line) + ": ";
    if (c.kind == Kind::Unknown)
      die(where + op.name + " is not a recognised hot-path op (" + c.why + "); no CPU fallback");
    const std::string res = op.results.empty() ? "" : op.results[0];
    const Type outT = op.resultTypes.empty() ? op.outsTypes[0] : op.resultTypes[0];

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
      if (outT.elt != "f32") die(where + "matmul accumulating in " + outT.elt + " is not mapped to a GEMM (f32 accumulate only)");
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
      auto us = usersOf(finalRes, b);
      if (us.size() == 1 && classOf(us[0], fr).kind == Kind::Add) {
        const std::string &other = us[0]->ins[0] == finalRes ? us[0]->ins[1] : us[0]->ins[0];
        const Op *bp = producer(other, defs);
        if (classOf(bp, fr).kind == Kind::BroadcastRow) {
          const Value &v = get(fr, bp->ins[0], *bp);
          if (v.type.elt == "f32" && v.type.shape.size() == 1 && v.type.shape[0] == N) {
            biasV = &v;
            absorbed.insert(us[0]);
            finalRes = us[0]->results[0];
            us = usersOf(finalRes, b);
          }
        }
      }
      uint32_t epi = IMEX_EPI_NONE;
      if (us.size() == 1 && classOf(us[0], fr).kind == Kind::Relu) {
        epi = IMEX_EPI_RELU;
        absorbed.insert(us[0]);
        finalRes = us[0]->results[0];
        us = usersOf(finalRes, b);
      } else if (us.size() == 2 && classOf(us[0], fr).kind == Kind::Sigmoid &&
                 classOf(us[1], fr).kind == Kind::Mul && us[1]->ins[0] == us[0]->results[0] &&
                 us[1]->ins[1] == finalRes) {
        epi = IMEX_EPI_SILU;
        absorbed.insert(us[0]);
        absorbed.insert(us[1]);
        finalRes = us[1]->results[0];
        us = usersOf(finalRes, b);
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
        if (us.size() == 1 && classOf(us[0], fr).kind == Kind::Mul && us[0]->ins[0] == res &&
            us[0]->ins[1] == op.ins[0]) {
          epi = IMEX_EPI_SILU;
          absorbed.insert(us[0]);
          finalRes = us[0]->results[0];
        } else {
          die(where + "sigmoid generic that is not followed by x * sigmoid(x)");
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
      if (!(sub && ex && sum && dv && dv->ins[1] == sum->results[0]))
        die(where + "row max that does not start a softmax chain (max, subtract, exp, sum, divide)");
      if (!init.isFill) die(where + "softmax row max must start from a filled tensor");
      const bool negInf = std::isinf(init.fillValue) && init.fillValue < 0;
      if (!negInf && !(init.fillValue <= -3.4e38)) die(where + "softmax row max must start from -inf or -FLT_MAX");
      if ((X.type.elt != "f32" && X.type.elt != "f16" && X.type.elt != "bf16") || X.type.shape.size() != 2)
        die(where + "softmax is f32 / f16 / bf16, rank 2 only");
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
      if (it == pendingSoftmax.end())
        die(where + "row-broadcast divide outside a softmax chain; no CPU fallback");
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
      Value &X = get(fr, op.ins[0], op);
      Value &init = get(fr, op.outs[0], op);
      if (X.type.elt != "f32") die(where + "sum reductions are f32 only");
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
      } else {
        die(where + "only rank-2 and rank-3 permutations of 2- and 4-byte elements have kernels");
      }
      fr.vals[res] = out;
      break;
    }
    default: {
      ElementwiseInfo standalone;
      if (classifyElementwise(op, fr.constants, standalone)) {  // e.g. an exp or a mul on its own
        elementwiseOp(op, b, fr, where);
        break;
      }
      die(where + std::string(kindName(c.kind)) + " generic outside the chain it belongs to (softmax / silu); no CPU fallback");
    }
    }
    (void)uses;
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
  if (file.empty()) die("usage: imex-b200-runner FILE.mlir [-e main] [--entry-point-result=void] [--emit-plan]");
  try {
    Module m = parseModule(readFile(file));
    Runner(m).runEntry(entry);
  } catch (const ParseError &e) {
    die(file + ": " + e.what());
  }
  return 0;
}
