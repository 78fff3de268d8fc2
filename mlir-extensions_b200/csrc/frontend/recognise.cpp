// Classification of linalg ops; see recognise.h.
#include "recognise.h"

#include "../../../include/imex_b200_blob.h"

#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <sstream>

namespace imex {
namespace fe {

const char *kindName(Kind k) {
  switch (k) {
  case Kind::Unknown: return "unknown";
  case Kind::Matmul: return "matmul";
  case Kind::Add: return "add";
  case Kind::BroadcastRow: return "broadcast_row";
  case Kind::Relu: return "relu";
  case Kind::Sigmoid: return "sigmoid";
  case Kind::Mul: return "mul";
  case Kind::RowMax: return "row_max";
  case Kind::SubRowBcast: return "sub_row_broadcast";
  case Kind::Exp: return "exp";
  case Kind::RowSum: return "row_sum";
  case Kind::DivRowBcast: return "div_row_broadcast";
  case Kind::Transpose: return "transpose";
  case Kind::ReduceLeading: return "reduce_leading";
  case Kind::ReduceAll: return "reduce_all";
  case Kind::ExtF: return "extf";
  case Kind::TruncF: return "truncf";
  case Kind::Elementwise: return "elementwise";
  case Kind::Fill: return "fill";
  }
  return "?";
}

namespace {

std::string fmtConst(double v) {
  std::ostringstream os;
  os << "c(" << v << ")";
  return os.str();
}

// Canonical expression of every yielded value of a linalg.generic body.
// Block arguments become in0.. / out0..; captured scalars become c(value);
// commutative ops sort their operands; tensor.from_elements / extract pairs on
// scalars are looked through (benchmarks/reduce/reduce_gpu.mlir.in:11-18).
std::vector<std::string> bodyExpressions(const Op &op, const ConstantTable &constants,
                                         std::string &why) {
  std::map<std::string, std::string> env;
  const Block &b = *op.body;
  const size_t nIn = op.ins.size();
  for (size_t i = 0; i < b.args.size(); ++i)
    env[b.args[i]] = (i < nIn ? "in" : "out") + std::to_string(i < nIn ? i : i - nIn);
  auto val = [&](const std::string &name) -> std::string {
    auto it = env.find(name);
    if (it != env.end()) return it->second;
    auto c = constants.find(name);
    if (c != constants.end()) return fmtConst(c->second);
    why = "body uses value " + name + " that is neither a block argument nor a known constant";
    return "?";
  };
  std::vector<std::string> yields;
  for (auto &o : b.ops) {
    const std::string &n = o->name;
    if (n == "linalg.yield") {
      for (auto &v : o->operands) yields.push_back(val(v));
      continue;
    }
    std::string e;
    auto fn = n.substr(n.find('.') + 1);
    if (n == "arith.constant") {
      e = fmtConst(o->isRaw[0] ? 0.0 : o->numbers[0]);
    } else if (n == "linalg.index") {
      e = "index" + std::to_string(o->intAttr);
    } else if (n == "arith.cmpf" || n == "arith.cmpi") {
      e = fn + "(" + o->predicate + "," + val(o->operands[0]) + "," + val(o->operands[1]) + ")";
    } else if (n == "arith.select") {
      e = "select(" + val(o->operands[0]) + "," + val(o->operands[1]) + "," + val(o->operands[2]) + ")";
    } else if (n == "tensor.from_elements" || n == "tensor.extract") {
      e = val(o->operands[0]);  // scalar <-> tensor<f32> round trip
    } else if (o->operands.size() == 1) {
      e = fn + "(" + val(o->operands[0]) + ")";
    } else if (o->operands.size() == 2) {
      std::string a = val(o->operands[0]), c = val(o->operands[1]);
      if (fn == "maxf") fn = "maximumf";  // older spelling of the same op
      const bool commutative = fn == "addf" || fn == "mulf" || fn == "maximumf" || fn == "addi" ||
                               fn == "muli" || fn == "maxnumf";
      if (commutative && c < a) std::swap(a, c);
      e = fn + "(" + a + "," + c + ")";
    } else {
      why = "unsupported operation " + n + " in a linalg body";
      e = "?";
    }
    for (auto &r : o->results) env[r] = e;
  }
  return yields;
}

bool mapIs(const AffineMap &m, std::initializer_list<int> dims) {
  if (m.results.size() != dims.size()) return false;
  size_t i = 0;
  for (int d : dims) {
    const MapResult &r = m.results[i++];
    if (d < 0) {  // -1: constant 0
      if (!r.isConst || r.value != 0) return false;
    } else if (r.isConst || r.value != d) {
      return false;
    }
  }
  return true;
}

bool allParallel(const Op &op) {
  return std::all_of(op.iterators.begin(), op.iterators.end(),
                     [](const std::string &s) { return s == "parallel"; });
}

// (d0,d1)->(d0,0) or (d0,d1)->(d0): one value per row
bool isRowVectorMap(const AffineMap &m) {
  return m.numDims == 2 && (mapIs(m, {0, -1}) || mapIs(m, {0}));
}

} // namespace

Classified classify(const Op &op, const ConstantTable &constants) {
  Classified c;
  if (op.name == "linalg.matmul" || op.name == "linalg.matmul_transpose_a" ||
      op.name == "linalg.matmul_transpose_b") {
    c.kind = Kind::Matmul;
    c.expr = op.name;
    c.transA = op.name == "linalg.matmul_transpose_a";
    c.transB = op.name == "linalg.matmul_transpose_b";
    return c;
  }
  if (op.name == "linalg.fill") {
    c.kind = Kind::Fill;
    return c;
  }
  if (op.name == "linalg.transpose") {
    c.kind = Kind::Transpose;
    for (auto &g : op.reassociation) c.perm.push_back(static_cast<int>(g[0]));
    return c;
  }
  if (op.name != "linalg.generic" || !op.body) {
    c.why = "not a linalg structured op";
    return c;
  }
  if (op.maps.size() != op.ins.size() + op.outs.size()) {
    c.why = "indexing_maps do not match the operand count";
    return c;
  }
  std::string why;
  std::vector<std::string> ys = bodyExpressions(op, constants, why);
  if (!why.empty() || ys.empty()) {
    c.why = why.empty() ? "empty body" : why;
    return c;
  }
  const std::string &y = ys[0];
  c.expr = y;
  const size_t nIn = op.ins.size(), nOut = op.outs.size();
  const int nd = op.maps[0].numDims;
  const AffineMap &outMap = op.maps[nIn];

  // ---- contractions ------------------------------------------------------
  if (nd == 3 && nIn == 2 && nOut == 1 && op.iterators.size() == 3 &&
      op.iterators[0] == "parallel" && op.iterators[1] == "parallel" &&
      op.iterators[2] == "reduction" && (mapIs(op.maps[0], {0, 2}) || mapIs(op.maps[0], {2, 0})) &&
      (mapIs(op.maps[1], {2, 1}) || mapIs(op.maps[1], {1, 2})) && mapIs(outMap, {0, 1})) {
    if (y == "addf(mulf(in0,in1),out0)" || y == "addf(mulf(extf(in0),extf(in1)),out0)") {
      c.kind = Kind::Matmul;
      c.transA = mapIs(op.maps[0], {2, 0});
      c.transB = mapIs(op.maps[1], {1, 2});
      return c;
    }
    c.why = "matmul-shaped generic with body " + y + " (only f32 mulf/addf is mapped to a GEMM)";
    return c;
  }

  // ---- reductions ----------------------------------------------------------
  const bool hasReduction = !allParallel(op);
  if (hasReduction) {
    if (nd == 2 && nIn == 1 && op.iterators[0] == "parallel" && op.iterators[1] == "reduction" &&
        op.maps[0].isIdentity() && isRowVectorMap(outMap)) {
      if (y == "addf(in0,out0)") {
        c.kind = Kind::RowSum;
        return c;
      }
      if (y == "maximumf(in0,out0)") {
        c.kind = Kind::RowMax;
        return c;
      }
      if (y == "select(cmpf(ogt,in0,out0),in0,out0)" || y == "select(cmpf(ogt,out0,in0),out0,in0)") {
        c.kind = Kind::RowMax;
        c.rowMaxOgt = true;
        return c;
      }
    }
    if (y == "addf(in0,out0)" && nIn == 1 && nOut == 1) {
      bool allRed = std::all_of(op.iterators.begin(), op.iterators.end(),
                                [](const std::string &s) { return s == "reduction"; });
      if (allRed && outMap.results.empty() && op.maps[0].isIdentity()) {
        c.kind = Kind::ReduceAll;
        return c;
      }
      // leading dim: in (d0..dn-1) -> (dn-1, d0, .., dn-2), out identity on the parallel dims,
      // last iterator is the reduction (benchmarks/reduce/reduce_gpu.mlir.in:1-2)
      bool lastRed = op.iterators.back() == "reduction";
      bool outIdent = static_cast<int>(outMap.results.size()) == nd - 1;
      for (int i = 0; outIdent && i < nd - 1; ++i)
        outIdent = !outMap.results[i].isConst && outMap.results[i].value == i;
      bool inRot = static_cast<int>(op.maps[0].results.size()) == nd;
      if (inRot) {
        inRot = !op.maps[0].results[0].isConst && op.maps[0].results[0].value == nd - 1;
        for (int i = 1; inRot && i < nd; ++i)
          inRot = !op.maps[0].results[i].isConst && op.maps[0].results[i].value == i - 1;
      }
      if (lastRed && outIdent && inRot) {
        c.kind = Kind::ReduceLeading;
        return c;
      }
    }
    c.why = "reduction with maps/body that match no hot-path reduction (body " + y + ")";
    return c;
  }

  // ---- elementwise / permutations -------------------------------------------
  if (y == "in0" && nIn == 1 && nOut == 1) {
    // pure data movement: out[outMap(d)] = in[inMap(d)]
    const AffineMap &inMap = op.maps[0];
    if (inMap.results.size() == outMap.results.size() &&
        static_cast<int>(inMap.results.size()) == nd) {
      // position of loop dim d in the input / output
      std::vector<int> inPos(nd, -1), outPos(nd, -1);
      bool permutation = true;
      for (int i = 0; i < nd; ++i) {
        const MapResult &ri = inMap.results[i], &ro = outMap.results[i];
        if (ri.isConst || ro.isConst || !ri.simple || !ro.simple) {
          permutation = false;
          break;
        }
        if (inPos[ri.value] >= 0 || outPos[ro.value] >= 0) permutation = false;  // a dim used twice
        inPos[ri.value] = i;
        outPos[ro.value] = i;
      }
      if (permutation) {
        c.perm.assign(nd, 0);
        for (int d = 0; d < nd; ++d) c.perm[outPos[d]] = inPos[d];
        c.kind = Kind::Transpose;
        return c;
      }
    }
  }
  bool identityAll = true;
  for (auto &m : op.maps) identityAll = identityAll && m.isIdentity();
  if (identityAll && nIn == 1) {
    if (y == "select(cmpf(ugt,in0,c(0)),in0,c(0))") { c.kind = Kind::Relu; return c; }
    if (y == "divf(c(1),addf(c(1),exp(negf(in0))))") { c.kind = Kind::Sigmoid; return c; }
    if (y == "exp(in0)") { c.kind = Kind::Exp; return c; }
    if (y == "extf(in0)") { c.kind = Kind::ExtF; return c; }
    if (y == "truncf(in0)") { c.kind = Kind::TruncF; return c; }
  }
  if (identityAll && nIn == 2 && y == "mulf(in0,in1)") {
    c.kind = Kind::Mul;
    return c;
  }
  if (identityAll && nIn == 2 && (y == "addf(in0,in1)" || y == "addf(in1,in0)")) {
    c.kind = Kind::Add;
    return c;
  }
  if (nd == 2 && nIn == 1 && nOut == 1 && y == "in0" && mapIs(op.maps[0], {1}) && outMap.isIdentity()) {
    c.kind = Kind::BroadcastRow;
    return c;
  }
  if (nd == 2 && nIn == 2 && op.maps[0].isIdentity() && isRowVectorMap(op.maps[1]) &&
      outMap.isIdentity()) {
    if (y == "subf(in0,in1)") { c.kind = Kind::SubRowBcast; return c; }
    if (y == "divf(in0,in1)") { c.kind = Kind::DivRowBcast; return c; }
  }
  ElementwiseInfo info;
  if (classifyElementwise(op, constants, info)) {
    c.kind = Kind::Elementwise;
    return c;
  }
  c.why = "elementwise body " + y + " matches no hot-path op";
  return c;
}

namespace {
struct ExprParser {
  const std::string &s;
  size_t pos = 0;
  explicit ExprParser(const std::string &text) : s(text) {}

  // the text of one balanced sub-expression starting at pos (without consuming it)
  std::string peekTerm() const {
    size_t i = pos;
    int depth = 0;
    for (; i < s.size(); ++i) {
      if (s[i] == '(') ++depth;
      else if (s[i] == ')') { if (depth == 0) break; --depth; }
      else if (s[i] == ',' && depth == 0) break;
    }
    return s.substr(pos, i - pos);
  }
  bool eat(char c) {
    if (pos < s.size() && s[pos] == c) { ++pos; return true; }
    return false;
  }
  std::shared_ptr<ExprTree> term() {
    size_t i = pos;
    while (i < s.size() && (std::isalnum(static_cast<unsigned char>(s[i])) || s[i] == '_')) ++i;
    const std::string name = s.substr(pos, i - pos);
    auto node = std::make_shared<ExprTree>();
    if (name.size() > 2 && name.compare(0, 2, "in") == 0 && std::isdigit(static_cast<unsigned char>(name[2])) &&
        (i == s.size() || s[i] != '(')) {
      node->kind = ExprTree::Input;
      node->index = std::atoi(name.c_str() + 2);
      pos = i;
      return node;
    }
    if (i >= s.size() || s[i] != '(') return nullptr;
    pos = i + 1;
    if (name == "c") {
      size_t j = s.find(')', pos);
      if (j == std::string::npos) return nullptr;
      node->kind = ExprTree::Const;
      node->value = std::strtod(s.substr(pos, j - pos).c_str(), nullptr);
      pos = j + 1;
      return node;
    }
    if (name == "select") {
      // only relu: select(cmpf(ugt,X,c(0)),X,c(0))
      if (s.compare(pos, 9, "cmpf(ugt,") != 0) return nullptr;
      pos += 9;
      const std::string x = peekTerm();
      auto xa = term();
      if (!xa || !eat(',')) return nullptr;
      auto zero = term();
      if (!zero || zero->kind != ExprTree::Const || zero->value != 0 || !eat(')') || !eat(',')) return nullptr;
      if (peekTerm() != x) return nullptr;
      auto xb = term();
      if (!xb || !eat(',')) return nullptr;
      auto zero2 = term();
      if (!zero2 || zero2->kind != ExprTree::Const || zero2->value != 0 || !eat(')')) return nullptr;
      node->kind = ExprTree::Unary;
      node->opcode = IMEX_X_RELU;
      node->a = xa;
      return node;
    }
    static const std::map<std::string, int> unary = {
        {"negf", IMEX_X_NEG}, {"absf", IMEX_X_ABS}, {"log", IMEX_X_LOG}, {"exp", IMEX_X_EXP},
        {"sqrt", IMEX_X_SQRT}, {"rsqrt", IMEX_X_RSQRT}, {"tanh", IMEX_X_TANH}};
    static const std::map<std::string, int> binary = {
        {"addf", IMEX_X_ADD}, {"subf", IMEX_X_SUB}, {"mulf", IMEX_X_MUL}, {"divf", IMEX_X_DIV},
        {"maximumf", IMEX_X_MAX}, {"minimumf", IMEX_X_MIN}};
    auto u = unary.find(name);
    auto bn = binary.find(name);
    if (u == unary.end() && bn == binary.end()) return nullptr;
    node->a = term();
    if (!node->a) return nullptr;
    if (u != unary.end()) {
      node->kind = ExprTree::Unary;
      node->opcode = u->second;
    } else {
      if (!eat(',')) return nullptr;
      node->b = term();
      if (!node->b) return nullptr;
      node->kind = ExprTree::Binary;
      node->opcode = bn->second;
    }
    if (!eat(')')) return nullptr;
    return node;
  }
};
} // namespace

std::shared_ptr<ExprTree> parseElementwiseExpr(const std::string &expr) {
  ExprParser p(expr);
  auto t = p.term();
  return (t && p.pos == expr.size()) ? t : nullptr;
}

bool classifyElementwise(const Op &op, const ConstantTable &constants, ElementwiseInfo &info) {
  if (op.name != "linalg.generic" || !op.body || op.outs.size() != 1 || op.ins.empty()) return false;
  if (op.maps.size() != op.ins.size() + 1 || !allParallel(op)) return false;
  const AffineMap &outMap = op.maps[op.ins.size()];
  if (!outMap.isIdentity()) return false;
  info.inputMode.clear();
  for (size_t i = 0; i < op.ins.size(); ++i) {
    const AffineMap &m = op.maps[i];
    if (m.isIdentity()) info.inputMode.push_back(0);
    else if (m.numDims == 2 && mapIs(m, {1})) info.inputMode.push_back(1);
    else if (m.numDims == 2 && (mapIs(m, {0}) || mapIs(m, {0, -1}))) info.inputMode.push_back(2);
    else return false;
  }
  std::string why;
  std::vector<std::string> ys = bodyExpressions(op, constants, why);
  if (!why.empty() || ys.size() != 1) return false;
  if (ys[0].find("out") != std::string::npos || ys[0].find("index") != std::string::npos) return false;
  info.expr = ys[0];
  info.tree = parseElementwiseExpr(info.expr);
  return info.tree != nullptr;
}

} // namespace fe
} // namespace imex
