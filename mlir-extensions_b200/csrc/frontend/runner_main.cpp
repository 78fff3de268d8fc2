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

struct Value {
  enum { Empty, Scalar, Tensor } kind = Empty;
  Type type;
  double scalar = 0;
  std::shared_ptr<Buffer> buf;
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
    std::vector<Value> results = runBlock(f.body, fr, stream, absorbed, defs, uses);
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

  Value &get(Frame &fr, const std::string &name, const Op &at) {
    auto it = fr.vals.find(name);
    if (it == fr.vals.end()) die("line " + std::to_string(at.line) + ": use of undefined value " + name);
    return it->second;
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
      if (!feedsBias) die(where + "row broadcast that is not the bias of a matmul; no CPU fallback");
      fr.vals[res] = get(fr, op.ins[0], op);
      break;
    }
    case Kind::Add:
      die(where + "elementwise add that is not the bias of a matmul; no CPU fallback");
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
      Value &X = get(fr, op.ins[0], op);
      if (X.type.elt != "f32") die(where + "elementwise ops are f32 only");
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
      if (X.type.elt != "f32" || X.type.shape.size() != 2) die(where + "softmax is f32, rank 2 only");
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
      ImexKernelDesc d = desc(IMEX_OP_SOFTMAX, IMEX_F32, IMEX_F32);
      if (plan.negInf) d.flags |= IMEX_FLAG_SOFTMAX_NEG_INF;
      d.dims[0] = X.type.shape[0];
      d.dims[1] = X.type.shape[1];
      launch(stream, d, {X.buf->ptr, out.buf->ptr}, "softmax");
      fr.vals[res] = out;
      break;
    }
    case Kind::RowSum:
    case Kind::ReduceLeading:
    case Kind::ReduceAll: {
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
      } else if (sh.size() == 3 && eb == 4) {
        ImexKernelDesc d = desc(IMEX_OP_TRANSPOSE3D, IMEX_F32, IMEX_F32);
        for (int i = 0; i < 3; ++i) {
          d.dims[i] = sh[i];
          d.dims[3 + i] = c.perm[i];
        }
        launch(stream, d, {X.buf->ptr, out.buf->ptr}, "transpose3d");
      } else {
        die(where + "only rank-2 and rank-3 (4-byte) permutations have kernels");
      }
      fr.vals[res] = out;
      break;
    }
    default:
      die(where + std::string(kindName(c.kind)) + " generic outside the chain it belongs to (softmax / silu); no CPU fallback");
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
