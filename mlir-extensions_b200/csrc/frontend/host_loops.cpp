// Register program for host-side scalar loop nests; see host_loops.h.
#include "host_loops.h"

#include <cmath>
#include <cstring>

namespace imex {
namespace fe {
namespace {

float halfToFloat(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0x1f) u = sign | 0x7f800000u | (man << 13);
  else if (exp != 0) u = sign | ((exp + 112u) << 23) | (man << 13);
  else if (man == 0) u = sign;
  else {
    int e = -1;
    uint32_t m = man;
    do { ++e; m <<= 1; } while (!(m & 0x400u));
    u = sign | ((112u - e) << 23) | ((m & 0x3ffu) << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
uint16_t floatToHalf(float v) {
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
  if (e < -14) shift += -14 - e;
  else { base = static_cast<uint32_t>(e + 15) << 10; m &= 0x7fffffu; }
  uint32_t q = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  uint32_t r = base + q;
  if (r > 0x7c00u) r = 0x7c00u;
  return sign | static_cast<uint16_t>(r);
}
uint16_t floatToBf16(float v) {
  uint32_t u;
  std::memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

double loadElt(const HostArray &a, int64_t i) {
  const char *p = static_cast<const char *>(a.data);
  if (a.elt == "f32") { float f; std::memcpy(&f, p + 4 * i, 4); return f; }
  if (a.elt == "f64") { double d; std::memcpy(&d, p + 8 * i, 8); return d; }
  if (a.elt == "f16") { uint16_t h; std::memcpy(&h, p + 2 * i, 2); return halfToFloat(h); }
  if (a.elt == "bf16") { uint16_t h; std::memcpy(&h, p + 2 * i, 2); uint32_t u = static_cast<uint32_t>(h) << 16; float f; std::memcpy(&f, &u, 4); return f; }
  if (a.elt == "i32") { int32_t x; std::memcpy(&x, p + 4 * i, 4); return x; }
  if (a.elt == "i64" || a.elt == "index") { int64_t x; std::memcpy(&x, p + 8 * i, 8); return static_cast<double>(x); }
  if (a.elt == "i16") { int16_t x; std::memcpy(&x, p + 2 * i, 2); return x; }
  int8_t x; std::memcpy(&x, p + i, 1); return x;
}
void storeElt(const HostArray &a, int64_t i, double v) {
  char *p = static_cast<char *>(a.data);
  if (a.elt == "f32") { float f = static_cast<float>(v); std::memcpy(p + 4 * i, &f, 4); }
  else if (a.elt == "f64") std::memcpy(p + 8 * i, &v, 8);
  else if (a.elt == "f16") { uint16_t h = floatToHalf(static_cast<float>(v)); std::memcpy(p + 2 * i, &h, 2); }
  else if (a.elt == "bf16") { uint16_t h = floatToBf16(static_cast<float>(v)); std::memcpy(p + 2 * i, &h, 2); }
  else if (a.elt == "i32") { int32_t x = static_cast<int32_t>(v); std::memcpy(p + 4 * i, &x, 4); }
  else if (a.elt == "i64" || a.elt == "index") { int64_t x = static_cast<int64_t>(v); std::memcpy(p + 8 * i, &x, 8); }
  else if (a.elt == "i16") { int16_t x = static_cast<int16_t>(v); std::memcpy(p + 2 * i, &x, 2); }
  else { int8_t x = static_cast<int8_t>(v); std::memcpy(p + i, &x, 1); }
}

} // namespace

int HostLoopProgram::reg(const std::string &name, std::vector<std::pair<std::string, int>> &env, const Lookup &lookup,
                         std::string &why) {
  for (auto it = env.rbegin(); it != env.rend(); ++it)
    if (it->first == name) return it->second;
  double scalar = 0;
  HostArray arr;
  bool isArray = false;
  if (!lookup(name, scalar, arr, isArray) || isArray) {
    why = "value " + name + " is not a scalar known outside the loop";
    return -1;
  }
  regs.push_back(scalar);
  env.emplace_back(name, static_cast<int>(regs.size()) - 1);
  return env.back().second;
}

int HostLoopProgram::arrayOf(const std::string &name, const Lookup &lookup, std::string &why) {
  for (auto &p : arrayIndex)
    if (p.first == name) return p.second;
  double scalar = 0;
  HostArray arr;
  bool isArray = false;
  if (!lookup(name, scalar, arr, isArray) || !isArray) {
    why = name + " is not a host-visible memref";
    return -1;
  }
  arrays.push_back(arr);
  arrayIndex.emplace_back(name, static_cast<int>(arrays.size()) - 1);
  return arrayIndex.back().second;
}

bool HostLoopProgram::block(const Block &b, std::vector<std::pair<std::string, int>> &env, const Lookup &lookup,
                            std::string &why) {
  auto fresh = [&](const std::string &name) {
    regs.push_back(0.0);
    env.emplace_back(name, static_cast<int>(regs.size()) - 1);
    return env.back().second;
  };
  for (auto &up : b.ops) {
    const Op &o = *up;
    const std::string &n = o.name;
    if (n == "scf.yield") {
      if (!o.operands.empty()) { why = "loop-carried values"; return false; }
      continue;
    }
    if (n == "scf.for") {
      if (!o.iterArgs.empty() || !o.body) { why = "scf.for with iter_args"; return false; }
      Ins f;
      f.code = For;
      f.lb = reg(o.operands[0], env, lookup, why);
      f.ub = reg(o.operands[1], env, lookup, why);
      f.step = reg(o.operands[2], env, lookup, why);
      if (f.lb < 0 || f.ub < 0 || f.step < 0) return false;
      const size_t mark = env.size();
      f.dst = fresh(o.body->args[0]);
      const size_t at = code.size();
      code.push_back(f);
      if (!block(*o.body, env, lookup, why)) return false;
      Ins e;
      e.code = End;
      e.end = static_cast<int>(at);
      code.push_back(e);
      code[at].end = static_cast<int>(code.size()) - 1;
      env.resize(mark);
      continue;
    }
    if (n == "arith.constant") {
      if (o.resultTypes[0].isShaped() || o.numbers.empty() || (!o.isRaw.empty() && o.isRaw[0])) { why = "tensor or hex constant in a host loop"; return false; }
      Ins c;
      c.code = Const;
      c.imm = o.numbers[0];
      c.dst = fresh(o.results[0]);
      code.push_back(c);
      continue;
    }
    if (n == "memref.load" || n == "memref.store") {
      const bool ld = n == "memref.load";
      Ins m;
      m.code = ld ? Load : Store;
      const size_t first = ld ? 1 : 2;
      m.array = arrayOf(o.operands[ld ? 0 : 1], lookup, why);
      if (m.array < 0) return false;
      if (o.operands.size() - first != arrays[m.array].shape.size()) { why = "index count differs from the memref's rank"; return false; }
      for (size_t i = first; i < o.operands.size(); ++i) {
        const int r = reg(o.operands[i], env, lookup, why);
        if (r < 0) return false;
        m.idx.push_back(r);
      }
      if (ld) m.dst = fresh(o.results[0]);
      else if ((m.a = reg(o.operands[0], env, lookup, why)) < 0) return false;
      code.push_back(m);
      continue;
    }
    if (n.rfind("arith.", 0) == 0 && !o.results.empty() && !o.resultTypes.empty() && !o.resultTypes[0].isShaped()) {
      struct Entry { const char *name; Code code; int arity; };
      static const Entry table[] = {
          {"arith.addf", Add, 2}, {"arith.subf", Sub, 2}, {"arith.mulf", Mul, 2}, {"arith.divf", Div, 2},
          {"arith.negf", Neg, 1}, {"arith.maximumf", Max, 2}, {"arith.minimumf", Min, 2},
          {"arith.addi", AddI, 2}, {"arith.subi", SubI, 2}, {"arith.muli", MulI, 2}, {"arith.divsi", DivI, 2},
          {"arith.remsi", RemI, 2}, {"arith.index_cast", Copy, 1}, {"arith.sitofp", Copy, 1},
          {"arith.extf", Copy, 1}, {"arith.extsi", Copy, 1}, {"arith.trunci", Copy, 1},
          {"arith.truncf", F32, 1}, {"arith.fptosi", ToInt, 1}};
      const Entry *hit = nullptr;
      for (auto &t : table)
        if (n == t.name) hit = &t;
      if (!hit || static_cast<int>(o.operands.size()) != hit->arity) { why = "operation " + n + " in a host loop"; return false; }
      const std::string &elt = o.resultTypes[0].elt;
      if (n == "arith.truncf" && elt != "f32") { why = "truncf to " + elt + " in a host loop"; return false; }
      if ((hit->code <= Min) && elt != "f32" && elt != "f64") { why = elt + " arithmetic in a host loop"; return false; }
      Ins a;
      a.code = hit->code;
      a.f32 = elt == "f32";
      if ((a.a = reg(o.operands[0], env, lookup, why)) < 0) return false;
      if (hit->arity == 2 && (a.b = reg(o.operands[1], env, lookup, why)) < 0) return false;
      a.dst = fresh(o.results[0]);
      code.push_back(a);
      continue;
    }
    why = "operation " + n + " in a host loop";
    return false;
  }
  return true;
}

bool HostLoopProgram::compile(const Op &forOp, const Lookup &lookup, std::string &why) {
  code.clear();
  regs.clear();
  arrays.clear();
  arrayIndex.clear();
  Block wrapper;  // compile the loop itself as the only statement
  std::vector<std::pair<std::string, int>> env;
  // block() wants a Block; build the For by hand around the body
  if (forOp.name != "scf.for" || !forOp.iterArgs.empty() || !forOp.body) { why = "not a plain scf.for"; return false; }
  Ins f;
  f.code = For;
  f.lb = reg(forOp.operands[0], env, lookup, why);
  f.ub = reg(forOp.operands[1], env, lookup, why);
  f.step = reg(forOp.operands[2], env, lookup, why);
  if (f.lb < 0 || f.ub < 0 || f.step < 0) return false;
  regs.push_back(0.0);
  env.emplace_back(forOp.body->args[0], static_cast<int>(regs.size()) - 1);
  f.dst = env.back().second;
  code.push_back(f);
  if (!block(*forOp.body, env, lookup, why)) return false;
  Ins e;
  e.code = End;
  e.end = 0;
  code.push_back(e);
  code[0].end = static_cast<int>(code.size()) - 1;
  return true;
}

void HostLoopProgram::run() {
  double *r = regs.data();
  const int n = static_cast<int>(code.size());
  for (int pc = 0; pc < n; ++pc) {
    const Ins &i = code[pc];
    switch (i.code) {
    case Const: r[i.dst] = i.imm; break;
    case Add: r[i.dst] = i.f32 ? static_cast<double>(static_cast<float>(r[i.a]) + static_cast<float>(r[i.b])) : r[i.a] + r[i.b]; break;
    case Sub: r[i.dst] = i.f32 ? static_cast<double>(static_cast<float>(r[i.a]) - static_cast<float>(r[i.b])) : r[i.a] - r[i.b]; break;
    case Mul: r[i.dst] = i.f32 ? static_cast<double>(static_cast<float>(r[i.a]) * static_cast<float>(r[i.b])) : r[i.a] * r[i.b]; break;
    case Div: r[i.dst] = i.f32 ? static_cast<double>(static_cast<float>(r[i.a]) / static_cast<float>(r[i.b])) : r[i.a] / r[i.b]; break;
    case Neg: r[i.dst] = -r[i.a]; break;
    case Max: r[i.dst] = (r[i.a] != r[i.a]) ? r[i.a] : (r[i.b] != r[i.b]) ? r[i.b] : std::fmax(r[i.a], r[i.b]); break;
    case Min: r[i.dst] = (r[i.a] != r[i.a]) ? r[i.a] : (r[i.b] != r[i.b]) ? r[i.b] : std::fmin(r[i.a], r[i.b]); break;
    case AddI: r[i.dst] = static_cast<double>(static_cast<int64_t>(r[i.a]) + static_cast<int64_t>(r[i.b])); break;
    case SubI: r[i.dst] = static_cast<double>(static_cast<int64_t>(r[i.a]) - static_cast<int64_t>(r[i.b])); break;
    case MulI: r[i.dst] = static_cast<double>(static_cast<int64_t>(r[i.a]) * static_cast<int64_t>(r[i.b])); break;
    case DivI: r[i.dst] = static_cast<double>(static_cast<int64_t>(r[i.a]) / static_cast<int64_t>(r[i.b])); break;
    case RemI: r[i.dst] = static_cast<double>(static_cast<int64_t>(r[i.a]) % static_cast<int64_t>(r[i.b])); break;
    case Copy: r[i.dst] = r[i.a]; break;
    case ToInt: r[i.dst] = std::trunc(r[i.a]); break;
    case F32: r[i.dst] = static_cast<double>(static_cast<float>(r[i.a])); break;
    case Load:
    case Store: {
      const HostArray &a = arrays[i.array];
      int64_t lin = 0;
      for (size_t d = 0; d < i.idx.size(); ++d) lin = lin * a.shape[d] + static_cast<int64_t>(r[i.idx[d]]);
      if (i.code == Load) r[i.dst] = loadElt(a, lin);
      else storeElt(a, lin, r[i.a]);
      break;
    }
    case For:
      r[i.dst] = r[i.lb];
      if (!(r[i.dst] < r[i.ub])) pc = i.end;
      break;
    case End: {
      const Ins &f = code[i.end];
      r[f.dst] += r[f.step];
      if (r[f.dst] < r[f.ub]) pc = i.end;  // back to the first instruction of the body (the loop ++pc's)
      break;
    }
    }
  }
}

} // namespace fe
} // namespace imex
