// CUDA C++ text of a linalg.generic as a loop nest; see loopnest.h.
#include "loopnest.h"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <set>
#include <sstream>

namespace imex {
namespace fe {
namespace {

bool isFloat(const std::string &e) { return e == "f32" || e == "f64" || e == "f16" || e == "bf16"; }
bool isInt(const std::string &e) {
  return e == "i1" || e == "i8" || e == "i16" || e == "i32" || e == "i64" || e == "index";
}

// type a value of this element type is computed in
const char *computeType(const std::string &e) {
  if (e == "f32" || e == "f16" || e == "bf16") return "float";
  if (e == "f64") return "double";
  if (e == "i1") return "bool";
  if (e == "i8") return "signed char";
  if (e == "i16") return "short";
  if (e == "i32") return "int";
  if (e == "i64" || e == "index") return "i64";
  return nullptr;
}
const char *unsignedType(const std::string &e) {
  if (e == "i8") return "unsigned char";
  if (e == "i16") return "unsigned short";
  if (e == "i32") return "unsigned";
  if (e == "i64" || e == "index") return "u64";
  return nullptr;
}
// type of the array elements in memory
const char *storageType(const std::string &e) {
  if (e == "f16" || e == "bf16") return "u16";
  if (e == "i1") return "u8";
  return computeType(e);
}
std::string loadExpr(const std::string &e, const std::string &ref) {
  if (e == "f16") return "imx_f16_to_f32(" + ref + ")";
  if (e == "bf16") return "imx_bf16_to_f32(" + ref + ")";
  if (e == "i1") return "(" + ref + " != 0)";
  return ref;
}
std::string storeExpr(const std::string &e, const std::string &v) {
  if (e == "f16") return "imx_f32_to_f16(" + v + ")";
  if (e == "bf16") return "imx_f32_to_bf16(" + v + ")";
  if (e == "i1") return "(u8)(" + v + " ? 1 : 0)";
  return v;
}
// a float result rounded to the element type it belongs to
std::string rounded(const std::string &e, const std::string &v) {
  if (e == "f16") return "imx_rf16(" + v + ")";
  if (e == "bf16") return "imx_rbf16(" + v + ")";
  return v;
}

std::string literal(const std::string &e, double v) {
  char buf[64];
  if (isFloat(e)) {
    const bool dbl = e == "f64";
    std::string s;
    if (std::isnan(v)) s = dbl ? "imx_nan64()" : "imx_nan32()";
    else if (std::isinf(v)) s = std::string(v < 0 ? "(-" : "(") + (dbl ? "imx_inf64()" : "imx_inf32()") + ")";
    else {
      if (dbl) std::snprintf(buf, sizeof buf, "(%a)", v);
      else std::snprintf(buf, sizeof buf, "(%af)", static_cast<double>(static_cast<float>(v)));
      s = buf;
    }
    return rounded(e, s);
  }
  if (e == "i1") return v != 0 ? "true" : "false";
  std::snprintf(buf, sizeof buf, "((%s)%lldLL)", computeType(e), static_cast<long long>(v));
  return buf;
}

struct Val {
  std::string expr;  // C expression (a variable name or a literal)
  std::string elt;
};

class BodyWriter {
public:
  BodyWriter(const ConstantTable &c, std::ostringstream &o, const std::string &ind) : constants(c), os(o), indent(ind) {}
  std::map<std::string, Val> env;
  std::string why;
  // tensors of the enclosing function that the region reads with tensor.extract: extra
  // pointer arguments of the kernel (cap0, cap1, ...), in this order
  std::vector<std::pair<std::string, Type>> captured;

  Val use(const std::string &name, const std::string &eltHint) {
    auto it = env.find(name);
    if (it != env.end()) return it->second;
    auto c = constants.find(name);
    if (c != constants.end()) {
      if (!computeType(eltHint)) {
        why = "constant " + name + " of type " + eltHint;
        return Val{"0", eltHint};
      }
      return Val{literal(eltHint, c->second), eltHint};
    }
    why = "body uses value " + name + " that is neither a block argument nor a known constant";
    return Val{"0", eltHint};
  }

  std::string define(const std::string &name, const std::string &elt, const std::string &rhs) {
    const std::string var = "v" + std::to_string(counter++);
    os << indent << "const " << computeType(elt) << " " << var << " = " << rhs << ";\n";
    env[name] = Val{var, elt};
    return var;
  }

  // one operation of the region; false when it has no C counterpart
  bool emit(const Op &o) {
    const std::string &n = o.name;
    const std::string fn = n.substr(n.find('.') + 1);
    const std::string resElt = o.resultTypes.empty() ? "" : o.resultTypes[0].elt;
    const std::string opElt = o.operandTypes.empty() ? resElt : o.operandTypes[0].elt;
    if (!o.results.empty() && !computeType(resElt)) {
      why = "element type " + resElt + " in " + n;
      return false;
    }
    auto in = [&](size_t i, const std::string &e) { return use(o.operands[i], e).expr; };
    const bool dbl = opElt == "f64";
    auto mathName = [&](const std::string &base) { return dbl ? base : base + "f"; };

    if (n == "arith.constant") {
      double v = o.numbers.empty() ? 0.0 : o.numbers[0];
      if (!o.isRaw.empty() && o.isRaw[0]) {  // hex literal: the bits of the value
        if (resElt == "f32") {
          uint32_t u = static_cast<uint32_t>(o.rawBits[0]);
          float f;
          std::memcpy(&f, &u, 4);
          v = f;
        } else if (resElt == "f64") {
          std::memcpy(&v, &o.rawBits[0], 8);
        } else if (isFloat(resElt)) {
          why = "hex literal of type " + resElt;
          return false;
        } else {
          v = static_cast<double>(static_cast<int64_t>(o.rawBits[0]));
        }
      }
      define(o.results[0], resElt, literal(resElt, v));
      return true;
    }
    if (n == "linalg.index") {
      define(o.results[0], "index", "(i64)d" + std::to_string(o.intAttr));
      return true;
    }
    if (n == "arith.cmpf") {
      const std::string a = in(0, opElt), b = in(1, opElt), &p = o.predicate;
      std::string e;
      if (p == "oeq") e = a + " == " + b;
      else if (p == "ogt") e = a + " > " + b;
      else if (p == "oge") e = a + " >= " + b;
      else if (p == "olt") e = a + " < " + b;
      else if (p == "ole") e = a + " <= " + b;
      else if (p == "one") e = "(" + a + " < " + b + ") || (" + a + " > " + b + ")";
      else if (p == "ord") e = "(" + a + " == " + a + ") && (" + b + " == " + b + ")";
      else if (p == "ueq") e = "!((" + a + " < " + b + ") || (" + a + " > " + b + "))";
      else if (p == "ugt") e = "!(" + a + " <= " + b + ")";
      else if (p == "uge") e = "!(" + a + " < " + b + ")";
      else if (p == "ult") e = "!(" + a + " >= " + b + ")";
      else if (p == "ule") e = "!(" + a + " > " + b + ")";
      else if (p == "une") e = a + " != " + b;
      else if (p == "uno") e = "(" + a + " != " + a + ") || (" + b + " != " + b + ")";
      else if (p == "false" || p == "true") e = p;
      else { why = "cmpf predicate " + p; return false; }
      define(o.results[0], "i1", "(" + e + ")");
      return true;
    }
    if (n == "arith.cmpi") {
      std::string a = in(0, opElt), b = in(1, opElt);
      const std::string &p = o.predicate;
      if (p[0] == 'u' && opElt != "i1") {
        const char *ut = unsignedType(opElt);
        if (!ut) { why = "cmpi on " + opElt; return false; }
        a = "(" + std::string(ut) + ")" + a;
        b = "(" + std::string(ut) + ")" + b;
      }
      const char *c = p == "eq" ? "==" : p == "ne" ? "!=" : (p == "slt" || p == "ult") ? "<"
                    : (p == "sle" || p == "ule") ? "<=" : (p == "sgt" || p == "ugt") ? ">"
                    : (p == "sge" || p == "uge") ? ">=" : nullptr;
      if (!c) { why = "cmpi predicate " + p; return false; }
      define(o.results[0], "i1", "(" + a + " " + c + " " + b + ")");
      return true;
    }
    if (n == "arith.select") {
      define(o.results[0], resElt, "(" + in(0, "i1") + " ? " + in(1, resElt) + " : " + in(2, resElt) + ")");
      return true;
    }
    // ---- conversions ------------------------------------------------------------
    if (n == "arith.extf" || n == "arith.truncf") {
      const std::string a = in(0, opElt);
      if (resElt == "f64") define(o.results[0], resElt, "(double)" + a);
      else define(o.results[0], resElt, rounded(resElt, "(float)" + a));
      return true;
    }
    if (n == "arith.sitofp" || n == "arith.uitofp") {
      std::string a = in(0, opElt);
      if (opElt == "i1") a = n == "arith.sitofp" ? "(" + a + " ? -1 : 0)" : "(" + a + " ? 1 : 0)";
      else if (n == "arith.uitofp") a = "(" + std::string(unsignedType(opElt)) + ")" + a;
      define(o.results[0], resElt, rounded(resElt, "(" + std::string(computeType(resElt)) + ")" + a));
      return true;
    }
    if (n == "arith.fptosi" || n == "arith.fptoui") {
      const std::string a = in(0, opElt);
      if (resElt == "i1") define(o.results[0], resElt, "(((int)" + a + ") & 1) != 0");
      else if (n == "arith.fptoui")
        define(o.results[0], resElt, "(" + std::string(computeType(resElt)) + ")(" + unsignedType(resElt) + ")" + a);
      else define(o.results[0], resElt, "(" + std::string(computeType(resElt)) + ")" + a);
      return true;
    }
    if (n == "arith.extsi" || n == "arith.extui" || n == "arith.trunci" || n == "arith.index_cast" ||
        n == "arith.index_castui") {
      std::string a = in(0, opElt);
      if (opElt == "i1") a = n == "arith.extsi" ? "(" + a + " ? -1 : 0)" : "(" + a + " ? 1 : 0)";
      else if (n == "arith.extui" || n == "arith.index_castui") a = "(" + std::string(unsignedType(opElt)) + ")" + a;
      if (resElt == "i1") define(o.results[0], resElt, "((" + a + " & 1) != 0)");
      else define(o.results[0], resElt, "(" + std::string(computeType(resElt)) + ")" + a);
      return true;
    }
    if (n == "arith.bitcast") {
      const std::string a = in(0, opElt);
      if (opElt == resElt) define(o.results[0], resElt, a);
      else if (opElt == "f32" && resElt == "i32") define(o.results[0], resElt, "imx_f32_bits(" + a + ")");
      else if (opElt == "i32" && resElt == "f32") define(o.results[0], resElt, "imx_bits_f32(" + a + ")");
      else { why = "bitcast " + opElt + " to " + resElt; return false; }
      return true;
    }
    // ---- float arithmetic ------------------------------------------------------------
    if (isFloat(resElt) && !o.operands.empty()) {
      static const std::map<std::string, const char *> infix = {
          {"addf", "+"}, {"subf", "-"}, {"mulf", "*"}, {"divf", "/"}};
      auto ix = infix.find(fn);
      if (n.rfind("arith.", 0) == 0 && ix != infix.end() && o.operands.size() == 2) {
        define(o.results[0], resElt, rounded(resElt, "(" + in(0, resElt) + " " + ix->second + " " + in(1, resElt) + ")"));
        return true;
      }
      if (n == "arith.negf") {
        define(o.results[0], resElt, "(-" + in(0, resElt) + ")");
        return true;
      }
      if (n == "arith.remf") {
        define(o.results[0], resElt, rounded(resElt, mathName("fmod") + "(" + in(0, resElt) + ", " + in(1, resElt) + ")"));
        return true;
      }
      static const std::map<std::string, const char *> minmax = {
          {"maximumf", "imx_maximum"}, {"maxf", "imx_maximum"}, {"minimumf", "imx_minimum"},
          {"minf", "imx_minimum"}, {"maxnumf", "imx_maxnum"}, {"minnumf", "imx_minnum"}};
      auto mm = minmax.find(fn);
      if (n.rfind("arith.", 0) == 0 && mm != minmax.end()) {
        define(o.results[0], resElt, std::string(mm->second) + "(" + in(0, resElt) + ", " + in(1, resElt) + ")");
        return true;
      }
      if (n.rfind("math.", 0) == 0) {
        static const std::map<std::string, const char *> unary = {
            {"exp", "exp"}, {"exp2", "exp2"}, {"expm1", "expm1"}, {"log", "log"}, {"log2", "log2"},
            {"log10", "log10"}, {"log1p", "log1p"}, {"sqrt", "sqrt"}, {"cbrt", "cbrt"}, {"tanh", "tanh"},
            {"sin", "sin"}, {"cos", "cos"}, {"tan", "tan"}, {"atan", "atan"}, {"asin", "asin"},
            {"acos", "acos"}, {"sinh", "sinh"}, {"cosh", "cosh"}, {"asinh", "asinh"}, {"acosh", "acosh"},
            {"atanh", "atanh"}, {"erf", "erf"}, {"floor", "floor"}, {"ceil", "ceil"}, {"absf", "fabs"},
            {"round", "round"}, {"roundeven", "rint"}, {"trunc", "trunc"}};
        static const std::map<std::string, const char *> binary = {
            {"powf", "pow"}, {"atan2", "atan2"}, {"copysign", "copysign"}};
        auto u = unary.find(fn);
        if (fn == "exp" && (resElt == "f16" || resElt == "bf16") && o.operands.size() == 1) {
          // forms that round to libm's 16-bit value for every argument of the type (the kernel prelude)
          define(o.results[0], resElt, rounded(resElt, "imx_exp_" + resElt + "(" + in(0, resElt) + ")"));
          return true;
        }
        if (u != unary.end() && o.operands.size() == 1) {
          define(o.results[0], resElt, rounded(resElt, mathName(u->second) + "(" + in(0, resElt) + ")"));
          return true;
        }
        auto b = binary.find(fn);
        if (b != binary.end() && o.operands.size() == 2) {
          define(o.results[0], resElt,
                 rounded(resElt, mathName(b->second) + "(" + in(0, resElt) + ", " + in(1, resElt) + ")"));
          return true;
        }
        if (fn == "rsqrt") {  // expanded to 1 / sqrt(x) by the CPU pipeline
          define(o.results[0], resElt, rounded(resElt, "(" + std::string(dbl ? "1.0" : "1.0f") + " / " +
                                                           mathName("sqrt") + "(" + in(0, resElt) + "))"));
          return true;
        }
        if (fn == "fma" && o.operands.size() == 3) {
          define(o.results[0], resElt, rounded(resElt, mathName("fma") + "(" + in(0, resElt) + ", " + in(1, resElt) +
                                                           ", " + in(2, resElt) + ")"));
          return true;
        }
      }
    }
    // ---- integer arithmetic (wrapping) -----------------------------------------------
    if (isInt(resElt) && o.operands.size() == 2 && n.rfind("arith.", 0) == 0) {
      const std::string a = in(0, resElt), b = in(1, resElt);
      if (resElt == "i1") {
        const char *c = (fn == "andi" || fn == "muli") ? "&&" : fn == "ori" ? "||" : (fn == "xori" || fn == "addi" || fn == "subi") ? "!=" : nullptr;
        if (!c) { why = n + " on i1"; return false; }
        define(o.results[0], resElt, "(" + a + " " + c + " " + b + ")");
        return true;
      }
      const std::string T = computeType(resElt), U = unsignedType(resElt);
      auto wrap = [&](const char *c) { return "(" + T + ")((" + U + ")" + a + " " + c + " (" + U + ")" + b + ")"; };
      std::string e;
      if (fn == "addi") e = wrap("+");
      else if (fn == "subi") e = wrap("-");
      else if (fn == "muli") e = wrap("*");
      else if (fn == "andi") e = wrap("&");
      else if (fn == "ori") e = wrap("|");
      else if (fn == "xori") e = wrap("^");
      else if (fn == "shli") e = wrap("<<");
      else if (fn == "shrui") e = wrap(">>");
      else if (fn == "divui") e = wrap("/");
      else if (fn == "remui") e = wrap("%");
      else if (fn == "shrsi") e = "(" + T + ")(" + a + " >> " + b + ")";
      else if (fn == "divsi") e = "(" + T + ")(" + a + " / " + b + ")";
      else if (fn == "remsi") e = "(" + T + ")(" + a + " % " + b + ")";
      else if (fn == "maxsi") e = "(" + a + " > " + b + " ? " + a + " : " + b + ")";
      else if (fn == "minsi") e = "(" + a + " < " + b + " ? " + a + " : " + b + ")";
      else if (fn == "maxui") e = "((" + U + ")" + a + " > (" + U + ")" + b + " ? " + a + " : " + b + ")";
      else if (fn == "minui") e = "((" + U + ")" + a + " < (" + U + ")" + b + " ? " + a + " : " + b + ")";
      else { why = "integer operation " + n; return false; }
      define(o.results[0], resElt, e);
      return true;
    }
    if (n == "math.absi" && o.operands.size() == 1) {
      const std::string a = in(0, resElt);
      define(o.results[0], resElt, "(" + a + " < 0 ? (" + computeType(resElt) + ")(-" + a + ") : " + a + ")");
      return true;
    }
    // ---- values of the enclosing function, and branches (what a concatenation lowers to:
    //      test/Jax/janet/jit_prim_fun.50_linalg.mlir:21-40) ----------------------------
    if (n == "tensor.dim" && o.operands.size() == 2 && !o.operandTypes.empty()) {
      const Type &t = o.operandTypes[0];
      if (!t.isShaped() || t.unranked) { why = "tensor.dim of an unranked value"; return false; }
      const std::string idx = in(1, "index");
      std::string e = "0LL";
      for (int r = static_cast<int>(t.shape.size()) - 1; r >= 0; --r) {
        if (t.shape[r] < 0) { why = "tensor.dim of a dynamic extent"; return false; }
        e = "(" + idx + " == " + std::to_string(r) + " ? " + std::to_string(t.shape[r]) + "LL : " + e + ")";
      }
      define(o.results[0], "index", "(i64)" + e);
      return true;
    }
    if (n == "tensor.extract" && !o.operands.empty() && !o.operandTypes.empty()) {
      const Type &t = o.operandTypes[0];
      if (!t.isShaped() || t.unranked || !storageType(t.elt) || o.operands.size() != 1 + t.shape.size()) {
        why = "tensor.extract from " + o.operands[0];
        return false;
      }
      size_t k = 0;
      while (k < captured.size() && captured[k].first != o.operands[0]) ++k;
      if (k == captured.size()) captured.emplace_back(o.operands[0], t);
      std::string lin;
      int64_t stride = 1;
      for (int r = static_cast<int>(t.shape.size()) - 1; r >= 0; --r) {
        if (t.shape[r] < 0) { why = "tensor.extract from a dynamic shape"; return false; }
        std::string term = in(1 + r, "index");
        if (stride != 1) term += " * " + std::to_string(stride) + "LL";
        lin = lin.empty() ? term : term + " + " + lin;
        stride *= t.shape[r];
      }
      if (lin.empty()) lin = "0";
      define(o.results[0], t.elt, loadExpr(t.elt, "cap" + std::to_string(k) + "[" + lin + "]"));
      return true;
    }
    if (n == "scf.if" && o.operands.size() == 1 && o.body) {
      if (!o.results.empty() && !o.elseBody) { why = "scf.if with results and no else region"; return false; }
      std::vector<std::string> vars;
      for (size_t r = 0; r < o.results.size(); ++r) {
        const std::string &e = o.resultTypes[r].elt;
        if (!computeType(e)) { why = "scf.if result of type " + e; return false; }
        vars.push_back("v" + std::to_string(counter++));
        os << indent << computeType(e) << " " << vars.back() << ";\n";
      }
      os << indent << "if (" << in(0, "i1") << ") {\n";
      if (!region(*o.body, vars, o.resultTypes)) return false;
      if (o.elseBody) {
        os << indent << "} else {\n";
        if (!region(*o.elseBody, vars, o.resultTypes)) return false;
      }
      os << indent << "}\n";
      for (size_t r = 0; r < o.results.size(); ++r) env[o.results[r]] = Val{vars[r], o.resultTypes[r].elt};
      return true;
    }
    why = "operation " + n + " has no loop-nest translation";
    return false;
  }

  // a region of scf.if: its operations one level deeper, scf.yield assigning the results
  bool region(const Block &b, const std::vector<std::string> &vars, const std::vector<Type> &types) {
    const std::map<std::string, Val> outer = env;
    const std::string outerIndent = indent;
    indent += "  ";
    bool ok = true, yielded = vars.empty();
    for (auto &o : b.ops) {
      if (o->name == "scf.yield") {
        if (o->operands.size() != vars.size()) { why = "scf.yield count differs from the results"; ok = false; break; }
        for (size_t r = 0; r < vars.size(); ++r)
          os << indent << vars[r] << " = " << use(o->operands[r], types[r].elt).expr << ";\n";
        yielded = true;
        continue;
      }
      if (!emit(*o)) { ok = false; break; }
    }
    if (ok && !yielded) { why = "region without scf.yield"; ok = false; }
    env = outer;
    indent = outerIndent;
    return ok;
  }

private:
  const ConstantTable &constants;
  std::ostringstream &os;
  std::string indent;
  int counter = 0;
};

} // namespace

bool buildLoopNest(const Op &op, const ConstantTable &constants, LoopNestKernel &out, std::string &why,
                   const std::vector<Type> *types) {
  if (op.name != "linalg.generic" || !op.body) {
    why = "not a linalg.generic";
    return false;
  }
  const size_t nIn = op.ins.size(), nOut = op.outs.size();
  if (nOut == 0 || op.maps.size() != nIn + nOut || op.body->args.size() != nIn + nOut) {
    why = "operand, map and block-argument counts disagree";
    return false;
  }
  const int nd = op.maps[0].numDims;
  if (static_cast<int>(op.iterators.size()) != nd) {
    why = "iterator_types do not match the maps";
    return false;
  }
  for (auto &m : op.maps)
    if (m.numDims != nd) {
      why = "indexing maps over different iteration spaces";
      return false;
    }
  if (types && types->size() != nIn + nOut) {
    why = "operand type list of the wrong length";
    return false;
  }
  auto typeOf = [&](size_t k) -> const Type & {
    if (types) return (*types)[k];
    return k < nIn ? op.insTypes[k] : op.outsTypes[k - nIn];
  };
  for (size_t k = 0; k < nIn + nOut; ++k) {
    const Type &t = typeOf(k);
    if (!computeType(t.elt)) {
      why = "element type " + t.elt;
      return false;
    }
    if (t.isShaped()) {
      if (t.unranked) { why = "unranked operand"; return false; }
      for (auto d : t.shape)
        if (d < 0) { why = "dynamic shape"; return false; }
      if (t.shape.size() != op.maps[k].results.size()) { why = "map rank differs from operand rank"; return false; }
    } else if (k >= nIn) {
      why = "scalar output";
      return false;
    }
  }
  // extents of the iteration dimensions, from the operands they index directly
  std::vector<int64_t> extent(nd, -1);
  for (size_t k = 0; k < nIn + nOut; ++k) {
    const Type &t = typeOf(k);
    if (!t.isShaped()) continue;
    for (size_t r = 0; r < op.maps[k].results.size(); ++r) {
      const MapResult &mr = op.maps[k].results[r];
      if (!mr.simple || mr.isConst) continue;
      if (extent[mr.value] >= 0 && extent[mr.value] != t.shape[r]) {
        why = "operands disagree on the extent of d" + std::to_string(mr.value);
        return false;
      }
      extent[mr.value] = t.shape[r];
    }
  }
  for (int d = 0; d < nd; ++d)
    if (extent[d] < 0) {
      why = "extent of d" + std::to_string(d) + " cannot be inferred";
      return false;
    }
  // A dimension labelled "reduction" that every output is indexed by carries nothing from one
  // of its iterations to the next: each point updates an element of its own
  // (test/PlaidML/OpTest.ExplicitPaddingNegInf.mlir:29).  It is run as a parallel dimension, the
  // outputs keeping their initial contents where the iteration space does not reach.
  auto inEveryOutput = [&](int d) {
    for (size_t k = nIn; k < nIn + nOut; ++k) {
      bool found = false;
      for (auto &mr : op.maps[k].results)
        found = found || (mr.simple ? (!mr.isConst && mr.value == d) : mr.shiftDim == d);
      if (!found) return false;
    }
    return true;
  };
  std::vector<int> par, red;
  bool relabelled = false;
  for (int d = 0; d < nd; ++d) {
    if (op.iterators[d] == "reduction" && !inEveryOutput(d)) red.push_back(d);
    else {
      par.push_back(d);
      relabelled = relabelled || op.iterators[d] == "reduction";
    }
  }
  // outputs: indexed by parallel dimensions only, and by all of them
  // (a dimension moved by a constant, d0 + 2, still addresses every element at most once: the
  // part of the output the iteration space does not reach keeps its initial value,
  // test/PlaidML/OpTest.ExplicitPadding.mlir:29-40)
  std::vector<bool> partial(nOut, false);
  for (size_t k = nIn; k < nIn + nOut; ++k) {
    std::set<int> used;
    for (auto &mr : op.maps[k].results) {
      if (!mr.simple && mr.shiftDim < 0) { why = "output indexed by a compound expression"; return false; }
      if (!mr.simple) {
        used.insert(mr.shiftDim);
        partial[k - nIn] = true;
      } else if (!mr.isConst) {
        used.insert(static_cast<int>(mr.value));
      }
    }
    for (int d : red)
      if (used.count(d)) { why = "output indexed by a reduction dimension"; return false; }
    for (int d : par)
      if (!used.count(d) && extent[d] > 1) { why = "parallel dimension missing from an output map"; return false; }
  }

  auto linearIndex = [&](size_t k) {
    const Type &t = typeOf(k);
    std::string e;
    int64_t stride = 1;
    for (int r = static_cast<int>(t.shape.size()) - 1; r >= 0; --r) {
      std::string term = "(i64)(" + op.maps[k].results[r].expr + ")";
      if (stride != 1) term += " * " + std::to_string(stride) + "LL";
      e = e.empty() ? term : term + " + " + e;
      stride *= t.shape[r];
    }
    return e.empty() ? std::string("0") : e;
  };

  out.threads = 1;
  for (int d : par) out.threads *= extent[d];
  if (out.threads < 0 || out.threads > (int64_t(1) << 40)) { why = "iteration space too large"; return false; }
  for (int64_t e : extent)
    if (e == 0) out.threads = 0;

  // does the region read an output's block argument?
  std::set<std::string> usedNames;
  std::function<void(const Block &)> collect = [&](const Block &b) {
    for (auto &o : b.ops) {
      for (auto &v : o->operands) usedNames.insert(v);
      if (o->body) collect(*o->body);
      if (o->elseBody) collect(*o->elseBody);
    }
  };
  collect(*op.body);
  out.readsInit.assign(nOut, false);
  for (size_t k = 0; k < nOut; ++k)
    out.readsInit[k] = !red.empty() || relabelled || partial[k] || usedNames.count(op.body->args[nIn + k]) != 0;

  // the argument list is written last: the region tells which outer tensors it reads
  std::ostringstream sig, os;
  sig << "extern \"C\" __global__ void imex_loopnest(";
  out.pointerInputs.clear();
  bool first = true;
  for (size_t k = 0; k < nIn; ++k) {
    if (!typeOf(k).isShaped()) continue;
    out.pointerInputs.push_back(static_cast<int>(k));
    sig << (first ? "" : ", ") << "const " << storageType(typeOf(k).elt) << " *__restrict__ in" << k;
    first = false;
  }
  for (size_t k = 0; k < nOut; ++k) {
    sig << (first ? "" : ", ") << storageType(typeOf(nIn + k).elt) << " *__restrict__ out" << k;
    first = false;
  }
  os << "  const i64 p = IMX_THREAD_INDEX;\n"
     << "  if (p >= " << out.threads << "LL) return;\n"
     << "  i64 q = p;\n";
  for (int i = static_cast<int>(par.size()) - 1; i >= 0; --i) {
    const int d = par[i];
    if (i == 0) os << "  const i64 d" << d << " = q;\n";
    else os << "  const i64 d" << d << " = q % " << extent[d] << "LL; q /= " << extent[d] << "LL;\n";
  }
  os << "  (void)q;\n";
  for (size_t k = 0; k < nOut; ++k) {
    const std::string &e = typeOf(nIn + k).elt;
    os << "  const i64 o" << k << " = " << linearIndex(nIn + k) << ";\n";
    os << "  " << computeType(e) << " acc" << k << " = ";
    if (out.readsInit[k]) os << loadExpr(e, "out" + std::to_string(k) + "[o" + std::to_string(k) + "]") << ";\n";
    else os << literal(e, 0.0) << ";\n";
  }
  std::string indent = "  ";
  for (int d : red) {
    os << indent << "for (i64 d" << d << " = 0; d" << d << " < " << extent[d] << "LL; ++d" << d << ") {\n";
    indent += "  ";
  }
  BodyWriter body(constants, os, indent);
  for (size_t k = 0; k < nIn; ++k) {
    const Type &t = typeOf(k);
    const std::string &arg = op.body->args[k];
    if (!t.isShaped()) {  // a scalar operand: its value is known when the kernel is written
      auto c = constants.find(op.ins[k]);
      if (c == constants.end()) { why = "scalar operand " + op.ins[k] + " is not a known constant"; return false; }
      body.env[arg] = Val{literal(t.elt, c->second), t.elt};
      continue;
    }
    if (!usedNames.count(arg)) {
      bool yielded = false;
      for (auto &o : op.body->ops)
        if (o->name == "linalg.yield")
          for (auto &v : o->operands) yielded = yielded || v == arg;
      if (!yielded) continue;  // never read: no load
    }
    os << indent << "const " << computeType(t.elt) << " a" << k << " = "
       << loadExpr(t.elt, "in" + std::to_string(k) + "[" + linearIndex(k) + "]") << ";\n";
    body.env[arg] = Val{"a" + std::to_string(k), t.elt};
  }
  for (size_t k = 0; k < nOut; ++k)
    body.env[op.body->args[nIn + k]] = Val{"acc" + std::to_string(k), typeOf(nIn + k).elt};
  bool yielded = false;
  for (auto &o : op.body->ops) {
    if (o->name == "linalg.yield") {
      if (o->operands.size() != nOut) { why = "yield count differs from the outputs"; return false; }
      // all yielded values are read before any accumulator is overwritten
      std::vector<std::string> vals;
      for (size_t k = 0; k < nOut; ++k) vals.push_back(body.use(o->operands[k], typeOf(nIn + k).elt).expr);
      if (nOut > 1)
        for (size_t k = 0; k < nOut; ++k)
          os << indent << "const " << computeType(typeOf(nIn + k).elt) << " y" << k << " = " << vals[k] << ";\n";
      for (size_t k = 0; k < nOut; ++k)
        os << indent << "acc" << k << " = " << (nOut > 1 ? "y" + std::to_string(k) : vals[k]) << ";\n";
      yielded = true;
      continue;
    }
    if (!body.emit(*o)) {
      why = body.why;
      return false;
    }
  }
  if (!body.why.empty()) { why = body.why; return false; }
  if (!yielded) { why = "region without linalg.yield"; return false; }
  for (size_t i = 0; i < red.size(); ++i) {
    indent.resize(indent.size() - 2);
    os << indent << "}\n";
  }
  for (size_t k = 0; k < nOut; ++k)
    os << "  out" << k << "[o" << k << "] = " << storeExpr(typeOf(nIn + k).elt, "acc" + std::to_string(k)) << ";\n";
  os << "}\n";
  out.captured.clear();
  for (size_t k = 0; k < body.captured.size(); ++k) {
    sig << ", const " << storageType(body.captured[k].second.elt) << " *__restrict__ cap" << k;
    out.captured.push_back(body.captured[k].first);
  }
  sig << ") {\n";
  out.source = sig.str() + os.str();
  std::ostringstream sum;
  sum << "loopnest[" << par.size() << " parallel, " << red.size() << " reduction dims, " << out.threads << " threads]";
  out.summary = sum.str();
  return true;
}

bool buildPad(const Type &src, const Type &dst, const std::vector<int64_t> &low, double value,
              LoopNestKernel &out, std::string &why) {
  const size_t rank = dst.shape.size();
  if (!src.isShaped() || !dst.isShaped() || src.shape.size() != rank || low.size() != rank || src.elt != dst.elt) {
    why = "tensor.pad between arrays of different rank or element type";
    return false;
  }
  if (!storageType(dst.elt)) {
    why = "element type " + dst.elt + " has no C counterpart";
    return false;
  }
  int64_t n = 1;
  for (size_t d = 0; d < rank; ++d) {
    if (dst.shape[d] < 0 || src.shape[d] < 0) { why = "dynamic shape"; return false; }
    n *= dst.shape[d];
  }
  out.threads = n;
  out.pointerInputs = {0};
  out.readsInit = {false};
  std::ostringstream os;
  const char *st = storageType(dst.elt);
  os << "extern \"C\" __global__ void imex_loopnest(const " << st << " *__restrict__ in0, " << st
     << " *__restrict__ out0) {\n"
     << "  const i64 p = IMX_THREAD_INDEX;\n"
     << "  if (p >= " << n << "LL) return;\n"
     << "  i64 q = p, s = 0, stride = 1;\n"
     << "  bool inside = true;\n";
  // innermost dimension first: position in the source = position in the result - low
  for (int d = static_cast<int>(rank) - 1; d >= 0; --d) {
    os << "  {\n    const i64 c = q % " << dst.shape[d] << "LL - " << low[d] << "LL;\n    q /= " << dst.shape[d] << "LL;\n"
       << "    inside = inside && c >= 0 && c < " << src.shape[d] << "LL;\n"
       << "    s += c * stride;\n    stride *= " << src.shape[d] << "LL;\n  }\n";
  }
  os << "  out0[p] = inside ? in0[s] : " << storeExpr(dst.elt, literal(dst.elt, value)) << ";\n}\n";
  out.source = os.str();
  out.summary = "pad[" + std::to_string(n) + " threads]";
  return true;
}

bool buildSlice(const Type &src, const Type &dst, const std::vector<int64_t> &offsets,
                const std::vector<int64_t> &sizes, const std::vector<int64_t> &strides, LoopNestKernel &out,
                std::string &why) {
  const size_t rank = src.shape.size();
  if (!src.isShaped() || !dst.isShaped() || offsets.size() != rank || sizes.size() != rank || strides.size() != rank ||
      src.elt != dst.elt) {
    why = "tensor.extract_slice whose lists do not match the source";
    return false;
  }
  if (!storageType(dst.elt)) {
    why = "element type " + dst.elt + " has no C counterpart";
    return false;
  }
  int64_t n = 1;
  for (size_t d = 0; d < rank; ++d) {
    if (src.shape[d] < 0 || sizes[d] <= 0 || offsets[d] < 0 || strides[d] <= 0 ||
        offsets[d] + (sizes[d] - 1) * strides[d] >= src.shape[d]) {
      why = "tensor.extract_slice outside its source";
      return false;
    }
    n *= sizes[d];
  }
  if (dst.count() != n) {
    why = "tensor.extract_slice whose result does not hold sizes-many elements";
    return false;
  }
  out.threads = n;
  out.pointerInputs = {0};
  out.readsInit = {false};
  std::ostringstream os;
  const char *st = storageType(dst.elt);
  os << "extern \"C\" __global__ void imex_loopnest(const " << st << " *__restrict__ in0, " << st
     << " *__restrict__ out0) {\n"
     << "  const i64 p = IMX_THREAD_INDEX;\n"
     << "  if (p >= " << n << "LL) return;\n"
     << "  i64 q = p, s = 0, stride = 1;\n";
  for (int d = static_cast<int>(rank) - 1; d >= 0; --d)
    os << "  s += (" << offsets[d] << "LL + (q % " << sizes[d] << "LL) * " << strides[d] << "LL) * stride; q /= " << sizes[d]
       << "LL; stride *= " << src.shape[d] << "LL;\n";
  os << "  out0[p] = in0[s];\n}\n";
  out.source = os.str();
  out.summary = "slice[" + std::to_string(n) + " threads]";
  return true;
}

} // namespace fe
} // namespace imex
