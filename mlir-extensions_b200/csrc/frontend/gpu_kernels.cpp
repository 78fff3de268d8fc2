// Data-flow recognition of XeGPU GEMM kernels; see gpu_kernels.h.
#include "gpu_kernels.h"

#include <cctype>
#include <map>
#include <set>
#include <vector>

namespace imex {
namespace fe {
namespace {

struct Stmt {
  std::vector<std::string> results;
  std::string op;
  std::vector<std::string> operands;  // every %name on the right-hand side, in order
};

bool nameChar(char c) { return std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.' || c == '$' || c == '-'; }

// One statement per line of the body: "%r[, %r2] = dialect.op %a, %b ..." or "dialect.op %a, ...".
// scf.for's "iter_args(%x = %init)" gives an extra statement %x = iter_arg %init, and the values
// yielded in a loop body flow into the loop's results through the same accumulator names.
std::vector<Stmt> statements(const std::string &body) {
  std::vector<Stmt> out;
  size_t pos = 0;
  while (pos < body.size()) {
    size_t end = body.find('\n', pos);
    if (end == std::string::npos) end = body.size();
    std::string line = body.substr(pos, end - pos);
    pos = end + 1;
    const size_t comment = line.find("//");
    if (comment != std::string::npos) line.resize(comment);
    auto names = [](const std::string &t) {
      std::vector<std::string> v;
      for (size_t i = 0; i < t.size(); ++i)
        if (t[i] == '%') {
          size_t j = i + 1;
          while (j < t.size() && nameChar(t[j]) && !(t[j] == '-' && j + 1 < t.size() && t[j + 1] == '>')) ++j;
          v.push_back(t.substr(i, j - i));
          i = j - 1;
        }
      return v;
    };
    Stmt s;
    std::string rhs = line;
    const size_t eq = line.find(" = ");
    const size_t firstPct = line.find('%');
    if (eq != std::string::npos && firstPct != std::string::npos && firstPct < eq &&
        line.find_first_not_of(" \t") == firstPct) {
      s.results = names(line.substr(0, eq));
      rhs = line.substr(eq + 3);
    }
    size_t b = rhs.find_first_not_of(" \t");
    if (b == std::string::npos) continue;
    size_t e = b;
    while (e < rhs.size() && (nameChar(rhs[e]))) ++e;
    s.op = rhs.substr(b, e - b);
    s.operands = names(rhs.substr(e));
    if (s.op == "scf.for") {
      // %res = scf.for %iv = .. iter_args(%acc = %init) -> (..): %acc and %res both carry %init
      const size_t ia = rhs.find("iter_args(");
      if (ia != std::string::npos) {
        const size_t close = rhs.find(')', ia);
        std::vector<std::string> pairs = names(rhs.substr(ia, close - ia));
        for (size_t i = 0; i + 1 < pairs.size(); i += 2) {
          Stmt carry;
          carry.results = {pairs[i]};
          carry.op = "iter_arg";
          carry.operands = {pairs[i + 1]};
          out.push_back(carry);
          for (auto &r : s.results) {
            Stmt res;
            res.results = {r};
            res.op = "loop_result";
            res.operands = {pairs[i]};
            out.push_back(res);
          }
        }
      }
      continue;
    }
    if (s.op.empty() || s.op[0] == '^' || s.op[0] == '}') continue;
    out.push_back(s);
  }
  return out;
}

} // namespace

bool recogniseGpuGemm(const GpuKernel &k, GpuGemm &g, std::string &why) {
  const std::vector<Stmt> stmts = statements(k.body);
  std::map<std::string, const Stmt *> def;
  for (auto &s : stmts)
    for (auto &r : s.results) def[r] = &s;
  std::map<std::string, int> argIndex;
  for (size_t i = 0; i < k.args.size(); ++i) argIndex[k.args[i]] = static_cast<int>(i);

  // memref arguments a value depends on, and whether a vector.transpose lies on the way
  struct Origin {
    std::set<int> args;
    bool transposed = false;
  };
  auto trace = [&](const std::string &start) {
    Origin o;
    std::vector<std::string> todo{start};
    std::set<std::string> seen;
    while (!todo.empty()) {
      const std::string v = todo.back();
      todo.pop_back();
      if (!seen.insert(v).second) continue;
      auto a = argIndex.find(v);
      if (a != argIndex.end()) {
        if (k.argTypes[a->second].isShaped()) o.args.insert(a->second);
        continue;
      }
      auto d = def.find(v);
      if (d == def.end()) continue;
      if (d->second->op == "vector.transpose") o.transposed = true;
      for (auto &x : d->second->operands) todo.push_back(x);
    }
    return o;
  };

  const Stmt *dpas = nullptr;
  for (auto &s : stmts)
    if (s.op == "xegpu.dpas") {
      if (dpas) { why = "more than one xegpu.dpas"; return false; }
      dpas = &s;
    }
  if (!dpas) { why = "no xegpu.dpas: not a matrix product"; return false; }
  if (dpas->operands.size() < 2) { why = "xegpu.dpas without operands"; return false; }
  const Origin oa = trace(dpas->operands[0]), ob = trace(dpas->operands[1]);
  auto single16 = [&](const Origin &o, int &idx) {
    idx = -1;
    for (int a : o.args) {
      const Type &t = k.argTypes[a];
      if (t.shape.size() == 2 && (t.elt == "f16" || t.elt == "bf16")) {
        if (idx >= 0) return false;
        idx = a;
      }
    }
    return idx >= 0;
  };
  if (!single16(oa, g.a) || !single16(ob, g.b) || g.a == g.b) {
    why = "the operands of xegpu.dpas do not come from two distinct rank-2 f16 / bf16 arguments";
    return false;
  }
  g.transA = oa.transposed;
  g.transB = ob.transposed;
  // the result: the argument a store_nd's tensor descriptor was made from
  for (auto &s : stmts)
    if (s.op == "xegpu.store_nd" && s.operands.size() >= 2) {
      const Origin od = trace(s.operands[1]);
      for (int a : od.args)
        if (a != g.a && a != g.b && k.argTypes[a].shape.size() == 2) g.c = a;
    }
  if (g.c < 0) { why = "no xegpu.store_nd to a rank-2 argument"; return false; }
  if (dpas->operands.size() >= 3) {
    const Origin oc = trace(dpas->operands[2]);
    g.readsC = oc.args.count(g.c) != 0;
  }
  for (size_t i = 0; i < k.args.size(); ++i) {
    const int a = static_cast<int>(i);
    if (a == g.a || a == g.b || a == g.c || !k.argTypes[i].isShaped()) continue;
    if (k.argTypes[i].shape.size() == 1 && k.argTypes[i].elt == "f32" && g.bias < 0) g.bias = a;
    else { why = "argument " + k.args[i] + " has no role in a GEMM"; return false; }
  }
  if (g.bias >= 0) {  // it must be added to what is stored
    bool added = false;
    for (auto &s : stmts)
      if (s.op == "arith.addf")
        for (auto &x : s.operands) added = added || trace(x).args.count(g.bias) != 0;
    if (!added) { why = "a rank-1 f32 argument that is not added to the result"; return false; }
  }
  const Type &ta = k.argTypes[g.a], &tb = k.argTypes[g.b], &tc = k.argTypes[g.c];
  for (const Type *t : {&ta, &tb, &tc})
    for (auto d : t->shape)
      if (d <= 0) { why = "dynamic shapes"; return false; }
  g.M = ta.shape[g.transA ? 1 : 0];
  g.K = ta.shape[g.transA ? 0 : 1];
  g.N = tb.shape[g.transB ? 0 : 1];
  if (tb.shape[g.transB ? 1 : 0] != g.K || tc.shape[0] != g.M || tc.shape[1] != g.N) {
    why = "argument shapes do not form C[M,N] = A[M,K] . B[K,N]";
    return false;
  }
  if (ta.elt != tb.elt) { why = "A and B of different element types"; return false; }
  if (tc.elt != "f32" && tc.elt != "f16" && tc.elt != "bf16") { why = "result type " + tc.elt; return false; }
  if (g.bias >= 0 && k.argTypes[g.bias].shape[0] != g.N) { why = "bias length differs from N"; return false; }
  return true;
}

} // namespace fe
} // namespace imex
