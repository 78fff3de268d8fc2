// Reader for the MLIR-text subset of the hot-path programs; see mlir_text.h.
#include "mlir_text.h"

#include <cctype>
#include <cmath>
#include <cstring>
#include <limits>
#include <sstream>

namespace imex {
namespace fe {

std::string Type::str() const {
  if (kind == None) return "none";
  if (kind == Scalar) return elt;
  std::string s = kind == Tensor ? "tensor<" : "memref<";
  if (unranked) return s + "*x" + elt + ">";
  for (auto d : shape) s += (d < 0 ? std::string("?") : std::to_string(d)) + "x";
  return s + elt + ">";
}

bool AffineMap::isIdentity() const {
  if (static_cast<int>(results.size()) != numDims) return false;
  for (int i = 0; i < numDims; ++i)
    if (results[i].isConst || results[i].value != i) return false;
  return true;
}

std::string AffineMap::str() const {
  std::string s = "(";
  for (int i = 0; i < numDims; ++i) s += (i ? ", d" : "d") + std::to_string(i);
  s += ") -> (";
  for (size_t i = 0; i < results.size(); ++i)
    s += (i ? ", " : "") + (results[i].isConst ? std::to_string(results[i].value)
                                               : "d" + std::to_string(results[i].value));
  return s + ")";
}

const Function *Module::find(const std::string &symbol) const {
  for (auto &f : functions)
    if (f.name == symbol) return &f;
  return nullptr;
}

namespace {

class Parser {
public:
  explicit Parser(const std::string &t) : s(t) {}

  Module module() {
    Module m;
    skip();
    // affine map aliases and other top-level attribute aliases
    while (peek() == '#') {
      std::string alias = ident();
      expect('=');
      skip();
      if (startsWith("affine_map")) {
        maps[alias] = affineMapAttr();
      } else {
        skipAttrValue();
      }
      skip();
    }
    bool wrapped = false;
    if (startsWith("builtin.module") || startsWith("module")) {
      pos += startsWith("builtin.module") ? 14 : 6;
      skip();
      if (peek() == '@') m.name = ident();
      skip();
      if (startsWith("attributes")) {
        pos += 10;
        skip();
        skipBalanced('{', '}');
      }
      expect('{');
      wrapped = true;
    }
    for (;;) {
      skip();
      if (eof()) break;
      if (wrapped && peek() == '}') {
        ++pos;
        break;
      }
      if (startsWith("func.func") || startsWith("func ")) {
        m.functions.push_back(function());
      } else if (startsWith("gpu.module")) {
        gpuModule(m);
      } else if (startsWith("shard.grid") || startsWith("mesh.mesh")) {
        // shard.grid @mesh4(shape = 4)   (test/Dialect/NDArray/Extensions/sharding_propagation.mlir:4)
        pos += startsWith("shard.grid") ? 10 : 9;
        Grid g;
        g.name = ident();
        expect('(');
        expectWord("shape");
        expect('=');
        do {
          skip();
          if (peek() == '?') { ++pos; g.shape.push_back(-1); }
          else g.shape.push_back(static_cast<int64_t>(number().value));
          skip();
        } while (peek() == 'x' && ++pos);
        expect(')');
        m.grids.push_back(g);
      } else if (startsWith("memref.global") || startsWith("llvm.func") ||
                 startsWith("llvm.mlir.global")) {
        skipLineOrRegion();
      } else if (peek() == '#') {
        std::string alias = ident();
        expect('=');
        skip();
        if (startsWith("affine_map"))
          maps[alias] = affineMapAttr();
        else
          skipAttrValue();
      } else {
        fail("unsupported top-level construct '" + s.substr(pos, 24) + "'");
      }
    }
    return m;
  }

  Type typeOnly() {
    skip();
    Type t = type();
    skip();
    if (!eof()) fail("trailing characters after type");
    return t;
  }

private:
  const std::string &s;
  size_t pos = 0;
  std::map<std::string, AffineMap> maps;

  // ---- low level -----------------------------------------------------------
  bool eof() const { return pos >= s.size(); }
  char peek() const { return eof() ? '\0' : s[pos]; }
  int lineNo() const {
    int n = 1;
    for (size_t i = 0; i < pos && i < s.size(); ++i)
      if (s[i] == '\n') ++n;
    return n;
  }
  [[noreturn]] void fail(const std::string &msg) const {
    throw ParseError("line " + std::to_string(lineNo()) + ": " + msg);
  }
  void skip() {
    for (;;) {
      while (!eof() && std::isspace(static_cast<unsigned char>(s[pos]))) ++pos;
      if (pos + 1 < s.size() && s[pos] == '/' && s[pos + 1] == '/') {
        while (!eof() && s[pos] != '\n') ++pos;
        continue;
      }
      break;
    }
  }
  bool startsWith(const char *w) const { return s.compare(pos, std::strlen(w), w) == 0; }
  bool accept(char c) {
    skip();
    if (peek() == c) {
      ++pos;
      return true;
    }
    return false;
  }
  bool acceptWord(const char *w) {
    skip();
    size_t n = std::strlen(w);
    if (s.compare(pos, n, w) == 0) {
      char after = pos + n < s.size() ? s[pos + n] : '\0';
      if (std::isalnum(static_cast<unsigned char>(after)) || after == '_' || after == '.') return false;
      pos += n;
      return true;
    }
    return false;
  }
  void expect(char c) {
    skip();
    if (peek() != c) fail(std::string("expected '") + c + "' but found '" + s.substr(pos, 12) + "'");
    ++pos;
  }
  void expectWord(const char *w) {
    if (!acceptWord(w)) fail(std::string("expected '") + w + "' but found '" + s.substr(pos, 12) + "'");
  }
  void expectArrow() {
    skip();
    if (!startsWith("->")) fail("expected '->'");
    pos += 2;
  }
  static bool identChar(char c) {
    return std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.' || c == '$';
  }
  // %name, %4#0, @sym, #alias, ^bb0, bare.identifier
  std::string ident() {
    skip();
    size_t b = pos;
    if (peek() == '%' || peek() == '@' || peek() == '#' || peek() == '^') ++pos;
    if (peek() == '"') {  // @"quoted symbol"
      ++pos;
      while (!eof() && s[pos] != '"') ++pos;
      ++pos;
      return s.substr(b, pos - b);
    }
    while (!eof() && (identChar(s[pos]) ||
                      // value names may hold '-' (%c-1_i8), never directly before '>'
                      (s[b] == '%' && s[pos] == '-' && pos + 1 < s.size() && identChar(s[pos + 1]))))
      ++pos;
    if (s[b] == '%' && peek() == '#') {  // result index
      ++pos;
      while (!eof() && std::isdigit(static_cast<unsigned char>(s[pos]))) ++pos;
    }
    if (pos == b) fail("expected an identifier but found '" + s.substr(pos, 12) + "'");
    return s.substr(b, pos - b);
  }
  std::string stringLit() {
    expect('"');
    size_t b = pos;
    while (!eof() && s[pos] != '"') ++pos;
    std::string r = s.substr(b, pos - b);
    ++pos;
    return r;
  }
  void skipBalanced(char open, char close) {
    expect(open);
    int depth = 1;
    while (!eof() && depth) {
      char c = s[pos++];
      if (c == '"') {
        while (!eof() && s[pos] != '"') ++pos;
        ++pos;
      } else if (c == open) {
        ++depth;
      } else if (c == close) {
        --depth;
      }
    }
    if (depth) fail(std::string("unbalanced '") + open + "'");
  }
  void skipAttrValue() {  // to the end of the line, keeping brackets balanced
    int depth = 0;
    while (!eof()) {
      char c = s[pos];
      if (c == '\n' && depth <= 0) break;
      if (c == '<' || c == '(' || c == '[' || c == '{') ++depth;
      if (c == '>' || c == ')' || c == ']' || c == '}') --depth;
      ++pos;
    }
  }
  void skipLineOrRegion() {
    while (!eof() && s[pos] != '\n' && s[pos] != '{') ++pos;
    if (peek() == '{') skipBalanced('{', '}');
  }

  // ---- numbers -------------------------------------------------------------
  struct Number {
    double value = 0;
    bool raw = false;
    uint64_t bits = 0;
  };
  Number number() {
    skip();
    Number n;
    if (acceptWord("true")) { n.value = 1; return n; }
    if (acceptWord("false")) { n.value = 0; return n; }
    size_t b = pos;
    if (peek() == '-' || peek() == '+') ++pos;
    if (s.compare(pos, 2, "0x") == 0 || s.compare(pos, 2, "0X") == 0) {
      pos += 2;
      size_t h = pos;
      while (!eof() && std::isxdigit(static_cast<unsigned char>(s[pos]))) ++pos;
      n.raw = true;
      n.bits = std::stoull(s.substr(h, pos - h), nullptr, 16);
      n.value = static_cast<double>(n.bits);
      return n;
    }
    if (startsWith("inf")) { pos += 3; n.value = s[b] == '-' ? -INFINITY : INFINITY; return n; }
    if (startsWith("nan")) { pos += 3; n.value = NAN; return n; }
    while (!eof() && (std::isdigit(static_cast<unsigned char>(s[pos])) || s[pos] == '.')) ++pos;
    if (!eof() && (s[pos] == 'e' || s[pos] == 'E')) {
      ++pos;
      if (peek() == '-' || peek() == '+') ++pos;
      while (!eof() && std::isdigit(static_cast<unsigned char>(s[pos]))) ++pos;
    }
    if (pos == b) fail("expected a number but found '" + s.substr(pos, 12) + "'");
    n.value = std::stod(s.substr(b, pos - b));
    return n;
  }

  // ---- types -----------------------------------------------------------------
  Type type() {
    skip();
    Type t;
    if (startsWith("tensor<") || startsWith("memref<")) {
      t.kind = startsWith("tensor<") ? Type::Tensor : Type::MemRef;
      pos += 7;
      // dims: 10x20xf32 / *xf32 / ?x4xf32 / f32
      for (;;) {
        skip();
        if (peek() == '*') {
          t.unranked = true;
          ++pos;
          if (peek() != 'x') fail("expected 'x' after '*'");
          ++pos;
          continue;
        }
        if (peek() == '?') {
          t.shape.push_back(-1);
          ++pos;
          if (peek() != 'x') fail("expected 'x' after '?'");
          ++pos;
          continue;
        }
        if (std::isdigit(static_cast<unsigned char>(peek()))) {
          size_t b = pos;
          while (std::isdigit(static_cast<unsigned char>(peek()))) ++pos;
          if (peek() != 'x') fail("expected 'x' in shape");
          t.shape.push_back(std::stoll(s.substr(b, pos - b)));
          ++pos;
          continue;
        }
        break;
      }
      size_t b = pos;
      while (!eof() && identChar(s[pos])) ++pos;
      t.elt = s.substr(b, pos - b);
      if (t.elt.empty()) fail("missing element type");
      skip();
      if (peek() == ',') {  // layout / memory space: skip to the closing '>'
        int depth = 1;
        while (!eof() && depth) {
          if (s[pos] == '<') ++depth;
          if (s[pos] == '>') --depth;
          if (depth) ++pos;
        }
      }
      expect('>');
      return t;
    }
    if (startsWith("!llvm.ptr")) {
      pos += 9;
      if (peek() == '<') skipBalanced('<', '>');
      t.kind = Type::Scalar;
      t.elt = "ptr";
      return t;
    }
    size_t b = pos;
    while (!eof() && identChar(s[pos])) ++pos;
    if (pos == b) fail("expected a type but found '" + s.substr(pos, 12) + "'");
    t.kind = Type::Scalar;
    t.elt = s.substr(b, pos - b);
    return t;
  }
  std::vector<Type> typeList() {  // "(t, t)" or "t" or "()"
    std::vector<Type> out;
    skip();
    if (peek() == '(') {
      ++pos;
      skip();
      if (peek() == ')') {
        ++pos;
        return out;
      }
      do {
        out.push_back(type());
        skipTypeAttrs();
      } while (accept(','));
      expect(')');
    } else {
      out.push_back(type());
    }
    return out;
  }
  void skipTypeAttrs() {  // "{lmhlo.written}" after a function result type
    skip();
    if (peek() == '{') skipBalanced('{', '}');
  }

  // ---- affine maps ---------------------------------------------------------
  AffineMap affineMapAttr() {
    skip();
    if (!startsWith("affine_map")) fail("expected affine_map");
    pos += 10;
    expect('<');
    AffineMap m = affineMapBody();
    expect('>');
    return m;
  }
  AffineMap affineMapBody() {
    AffineMap m;
    expect('(');
    std::vector<std::string> dims;
    skip();
    if (peek() != ')') {
      do {
        dims.push_back(ident());
      } while (accept(','));
    }
    expect(')');
    m.numDims = static_cast<int>(dims.size());
    skip();
    if (peek() == '[') skipBalanced('[', ']');  // symbols: unused on this path
    expectArrow();
    expect('(');
    skip();
    if (peek() != ')') {
      do {
        AffineTerm t = affineSum(dims);
        MapResult r;
        r.expr = t.text;
        if (t.kind == AffineTerm::Const) {
          r.isConst = true;
          r.value = t.value;
        } else if (t.kind == AffineTerm::Dim) {
          r.value = t.value;
        } else {
          r.simple = false;
          r.value = -1;
          r.shiftDim = t.shiftDim;
          r.shift = t.shift;
        }
        m.results.push_back(r);
      } while (accept(','));
    }
    expect(')');
    return m;
  }
  // affine expressions: sums of products of dimensions and constants, floordiv / ceildiv /
  // mod by constants, parentheses.  Dimensions are non-negative, so C's `/` and `%` agree
  // with floordiv and mod for the positive divisors the syntax allows.
  struct AffineTerm {
    enum { Const, Dim, Other } kind = Other;
    int64_t value = 0;
    std::string text;
    int shiftDim = -1;   // Other of the form dim + constant
    int64_t shift = 0;
  };
  AffineTerm affineAtom(const std::vector<std::string> &dims) {
    skip();
    AffineTerm t;
    if (peek() == '(') {
      ++pos;
      t = affineSum(dims);
      expect(')');
      if (t.kind == AffineTerm::Other) t.text = "(" + t.text + ")";
      return t;
    }
    if (peek() == '-') {
      ++pos;
      AffineTerm a = affineAtom(dims);
      if (a.kind == AffineTerm::Const) {
        a.value = -a.value;
        a.text = std::to_string(a.value);
        return a;
      }
      t.text = "(-" + a.text + ")";
      return t;
    }
    if (std::isdigit(static_cast<unsigned char>(peek()))) {
      t.kind = AffineTerm::Const;
      t.value = static_cast<int64_t>(number().value);
      t.text = std::to_string(t.value);
      return t;
    }
    std::string d = ident();
    int idx = -1;
    for (size_t i = 0; i < dims.size(); ++i)
      if (dims[i] == d) idx = static_cast<int>(i);
    if (idx < 0) fail("unknown dimension '" + d + "' in affine map");
    t.kind = AffineTerm::Dim;
    t.value = idx;
    t.text = "d" + std::to_string(idx);
    return t;
  }
  AffineTerm affineProduct(const std::vector<std::string> &dims) {
    AffineTerm a = affineAtom(dims);
    for (;;) {
      skip();
      const char *op = nullptr;
      if (peek() == '*') { ++pos; op = "*"; }
      else if (acceptWord("floordiv")) op = "/";
      else if (acceptWord("ceildiv")) op = "ceil";
      else if (acceptWord("mod")) op = "%";
      else break;
      AffineTerm b = affineAtom(dims);
      AffineTerm r;
      if (std::string(op) == "ceil") r.text = "((" + a.text + " + " + b.text + " - 1) / " + b.text + ")";
      else r.text = "(" + a.text + " " + op + " " + b.text + ")";
      a = r;
    }
    return a;
  }
  AffineTerm affineSum(const std::vector<std::string> &dims) {
    AffineTerm a = affineProduct(dims);
    for (;;) {
      skip();
      char op = peek();
      if (op != '+' && op != '-') break;
      if (op == '-' && pos + 1 < s.size() && s[pos + 1] == '>') break;  // the map's arrow
      ++pos;
      AffineTerm b = affineProduct(dims);
      AffineTerm r;
      r.text = "(" + a.text + " " + op + " " + b.text + ")";
      if (a.kind == AffineTerm::Dim && b.kind == AffineTerm::Const) {
        r.shiftDim = static_cast<int>(a.value);
        r.shift = op == '+' ? b.value : -b.value;
      } else if (a.kind == AffineTerm::Const && b.kind == AffineTerm::Dim && op == '+') {
        r.shiftDim = static_cast<int>(b.value);
        r.shift = a.value;
      }
      a = r;
    }
    return a;
  }
  AffineMap mapRefOrInline() {
    skip();
    if (peek() == '#') {
      std::string a = ident();
      auto it = maps.find(a);
      if (it == maps.end()) fail("unknown map alias " + a);
      return it->second;
    }
    return affineMapAttr();
  }

  // gpu.module @name [targets] { gpu.func @k(%a: memref<..>, ...) kernel [attributes {..}] { body } ... }
  void gpuModule(Module &m) {
    pos += 10;
    const std::string modName = ident();
    while (!eof() && peek() != '{') ++pos;  // target attributes
    expect('{');
    for (;;) {
      skip();
      if (eof()) fail("unterminated gpu.module");
      if (peek() == '}') {
        ++pos;
        return;
      }
      if (!startsWith("gpu.func")) {
        skipLineOrRegion();
        continue;
      }
      pos += 8;
      GpuKernel k;
      k.module = modName;
      k.line = lineNo();
      k.name = ident();
      expect('(');
      skip();
      if (peek() != ')') {
        do {
          k.args.push_back(ident());
          expect(':');
          k.argTypes.push_back(type());
          skipTypeAttrs();
        } while (accept(','));
      }
      expect(')');
      acceptWord("kernel");
      if (acceptWord("attributes")) {
        skip();
        skipBalanced('{', '}');
      }
      skip();
      const size_t b = pos;
      skipBalanced('{', '}');
      k.body = s.substr(b, pos - b);
      m.gpuKernels.push_back(std::move(k));
    }
  }

  // ---- functions -------------------------------------------------------------
  Function function() {
    Function f;
    if (!acceptWord("func.func")) expectWord("func");
    if (acceptWord("private")) f.isDeclaration = true;
    acceptWord("public");
    f.name = ident();
    expect('(');
    skip();
    if (peek() != ')') {
      do {
        skip();
        if (peek() == '%') {
          f.args.push_back(ident());
          expect(':');
        } else {
          f.args.push_back("");
        }
        f.argTypes.push_back(type());
        skipTypeAttrs();
      } while (accept(','));
    }
    expect(')');
    skip();
    if (startsWith("->")) {
      pos += 2;
      f.resultTypes = typeList();  // result attributes only occur inside the parentheses
    }
    if (acceptWord("attributes")) {
      skip();
      skipBalanced('{', '}');
    }
    skip();
    if (peek() == '{') {
      ++pos;
      f.isDeclaration = false;
      block(f.body, /*allowLabel=*/false);
    } else {
      f.isDeclaration = true;
    }
    return f;
  }

  // ops until the closing '}' (consumed)
  void block(Block &b, bool allowLabel) {
    skip();
    if (allowLabel && peek() == '^') {
      ident();
      expect('(');
      skip();
      if (peek() != ')') {
        do {
          b.args.push_back(ident());
          expect(':');
          b.argTypes.push_back(type());
        } while (accept(','));
      }
      expect(')');
      expect(':');
    }
    for (;;) {
      skip();
      if (eof()) fail("unterminated block");
      if (peek() == '}') {
        ++pos;
        return;
      }
      b.ops.push_back(operation());
    }
  }

  void operandList(std::vector<std::string> &out) {  // %a, %b  (possibly empty)
    skip();
    while (peek() == '%') {
      out.push_back(ident());
      if (!accept(',')) break;
      skip();
    }
  }

  // "ins(%a, %b : tA, tB)" / "outs(...)"
  void insOuts(const char *word, std::vector<std::string> &vals, std::vector<Type> &types) {
    if (!acceptWord(word)) return;
    expect('(');
    operandList(vals);
    expect(':');
    do {
      types.push_back(type());
    } while (accept(','));
    expect(')');
  }

  void attrDict(Op &op) {  // { key = value, ... } — keeps what the recogniser needs
    expect('{');
    skip();
    if (peek() == '}') {
      ++pos;
      return;
    }
    do {
      skip();
      std::string key = peek() == '"' ? stringLit() : ident();
      skip();
      if (peek() != '=') continue;  // unit attribute
      ++pos;
      skip();
      if (key == "indexing_maps") {
        expect('[');
        do {
          op.maps.push_back(mapRefOrInline());
        } while (accept(','));
        expect(']');
      } else if (key == "iterator_types") {
        expect('[');
        skip();
        if (peek() != ']') {
          do {
            skip();
            if (peek() == '"') {
              op.iterators.push_back(stringLit());
            } else {  // #linalg.iterator_type<parallel>
              std::string a = ident();
              expect('<');
              op.iterators.push_back(ident());
              expect('>');
              (void)a;
            }
          } while (accept(','));
        }
        expect(']');
      } else {
        attrValue();
      }
    } while (accept(','));
    expect('}');
  }
  void attrValue() {  // skip one attribute value
    skip();
    int depth = 0;
    while (!eof()) {
      char c = s[pos];
      if (c == '"') {
        stringLit();
        continue;
      }
      if (c == '[' || c == '{' || c == '<' || c == '(') ++depth;
      if (c == ']' || c == '}' || c == '>' || c == ')') {
        if (depth == 0) return;
        --depth;
      }
      if (c == ',' && depth == 0) return;
      ++pos;
    }
  }

  void denseAttr(Op &op) {
    pos += 5;  // "dense"
    expect('<');
    op.hasDense = true;
    skip();
    if (peek() == '[') {
      denseList(op);
    } else {
      op.denseSplat = true;
      pushNumber(op, number());
    }
    expect('>');
  }
  void denseList(Op &op) {
    expect('[');
    skip();
    if (peek() == ']') {
      ++pos;
      return;
    }
    do {
      skip();
      if (peek() == '[')
        denseList(op);
      else
        pushNumber(op, number());
    } while (accept(','));
    expect(']');
  }
  static void pushNumber(Op &op, const Number &n) {
    op.numbers.push_back(n.value);
    op.rawBits.push_back(n.bits);
    op.isRaw.push_back(n.raw);
  }

  std::unique_ptr<Op> operation() {
    auto op = std::make_unique<Op>();
    skip();
    op->line = lineNo();
    if (peek() == '%') {
      do {
        std::string r = ident();
        skip();
        if (peek() == ':') {  // %4:2
          ++pos;
          int n = static_cast<int>(number().value);
          for (int i = 0; i < n; ++i) op->results.push_back(r + "#" + std::to_string(i));
        } else {
          op->results.push_back(r);
        }
      } while (accept(','));
      expect('=');
    }
    op->name = ident();
    const std::string &n = op->name;

    if (n == "arith.constant") {
      skip();
      if (startsWith("dense")) {
        denseAttr(*op);
      } else {
        skip();
        const bool boolean = startsWith("true") || startsWith("false");
        pushNumber(*op, number());
        skip();
        if (boolean && peek() != ':') {   // "arith.constant true": the type i1 goes without saying
          Type t;
          t.kind = Type::Scalar;
          t.elt = "i1";
          op->resultTypes.push_back(t);
          return op;
        }
      }
      expect(':');
      op->resultTypes.push_back(type());
    } else if (n == "tensor.empty") {
      expect('(');
      operandList(op->operands);  // the extents of the dynamic dimensions, in order
      expect(')');
      expect(':');
      op->resultTypes.push_back(type());
    } else if (n == "linalg.fill" || n == "linalg.matmul" || n == "linalg.generic" ||
               n == "linalg.transpose" || n == "linalg.copy") {
      skip();
      if (peek() == '{') attrDict(*op);
      insOuts("ins", op->ins, op->insTypes);
      insOuts("outs", op->outs, op->outsTypes);
      if (acceptWord("attrs")) {
        expect('=');
        Op scratch;
        attrDict(scratch);
      }
      if (acceptWord("permutation")) {
        expect('=');
        expect('[');
        do {
          op->reassociation.push_back({static_cast<int64_t>(number().value)});
        } while (accept(','));
        expect(']');
      }
      skip();
      if (peek() == '{') {
        ++pos;
        op->body = std::make_unique<Block>();
        block(*op->body, /*allowLabel=*/true);
      }
      skip();
      if (startsWith("->")) {
        pos += 2;
        op->resultTypes = typeList();
      }
    } else if (n == "linalg.yield" || n == "scf.yield" || n == "tensor.yield" || n == "return" || n == "func.return") {
      operandList(op->operands);
      if (accept(':')) {
        do {
          op->operandTypes.push_back(type());
        } while (accept(','));
      }
    } else if (n == "linalg.index") {
      op->intAttr = static_cast<int64_t>(number().value);
      expect(':');
      op->resultTypes.push_back(type());
    } else if (n == "call" || n == "func.call" || n == "llvm.call") {
      op->callee = ident();
      expect('(');
      operandList(op->operands);
      expect(')');
      expect(':');
      op->operandTypes = typeList();
      expectArrow();
      op->resultTypes = typeList();
    } else if (n == "arith.cmpf" || n == "arith.cmpi") {
      op->predicate = ident();
      expect(',');
      operandList(op->operands);
      expect(':');
      op->operandTypes.push_back(type());
      Type i1;
      i1.kind = Type::Scalar;
      i1.elt = "i1";
      op->resultTypes.push_back(i1);
    } else if (n == "arith.select") {
      operandList(op->operands);
      expect(':');
      Type t = type();
      if (accept(',')) t = type();  // "i1, f32" form
      op->resultTypes.push_back(t);
    } else if (n == "tensor.cast" || n == "memref.cast" || n == "arith.extf" || n == "arith.truncf" ||
               n == "arith.index_cast" || n == "arith.sitofp" || n == "arith.fptosi" ||
               n == "arith.extsi" || n == "arith.trunci" || n == "arith.uitofp" ||
               n == "bufferization.to_memref" || n == "bufferization.to_buffer" ||
               n == "bufferization.to_tensor") {
      operandList(op->operands);
      acceptWord("restrict");
      expect(':');
      Type from = type();
      Type to = from;
      if (acceptWord("to")) to = type();
      op->operandTypes.push_back(from);
      op->resultTypes.push_back(to);
    } else if (n == "tensor.extract") {
      operandList(op->operands);
      expect('[');
      std::vector<std::string> idx;
      operandList(idx);
      for (auto &i : idx) op->operands.push_back(i);
      expect(']');
      expect(':');
      Type t = type();
      op->operandTypes.push_back(t);
      Type e;
      e.kind = Type::Scalar;
      e.elt = t.elt;
      op->resultTypes.push_back(e);
    } else if (n == "tensor.from_elements") {
      operandList(op->operands);
      expect(':');
      op->resultTypes.push_back(type());
    } else if (n == "tensor.dim") {
      // %5 = tensor.dim %arg0, %c0_0 : tensor<1x6xf32>
      operandList(op->operands);
      expect(':');
      op->operandTypes.push_back(type());
      Type e;
      e.kind = Type::Scalar;
      e.elt = "index";
      op->resultTypes.push_back(e);
    } else if (n == "scf.if") {
      // %8 = scf.if %7 -> (f32) { ... scf.yield %10 : f32 } else { ... }
      operandList(op->operands);
      skip();
      if (peek() == '-') {
        expectArrow();
        op->resultTypes = typeList();
      }
      expect('{');
      op->body = std::make_unique<Block>();
      block(*op->body, /*allowLabel=*/false);
      if (acceptWord("else")) {
        expect('{');
        op->elseBody = std::make_unique<Block>();
        block(*op->elseBody, /*allowLabel=*/false);
      }
    } else if (n == "tensor.extract_slice") {
      // %r = tensor.extract_slice %x[49999] [1] [1] : tensor<50000xf32> to tensor<1xf32>
      //      (offsets, sizes, strides; static only; the result may drop unit dimensions)
      operandList(op->operands);
      for (int list = 0; list < 3; ++list) {
        expect('[');
        std::vector<int64_t> v;
        skip();
        if (peek() != ']') {
          do {
            skip();
            if (peek() == '%') fail("tensor.extract_slice with dynamic offsets, sizes or strides is outside the supported subset");
            v.push_back(static_cast<int64_t>(number().value));
          } while (accept(','));
        }
        expect(']');
        op->reassociation.push_back(v);
      }
      expect(':');
      op->operandTypes.push_back(type());
      expectWord("to");
      op->resultTypes.push_back(type());
    } else if (n == "tensor.pad") {
      // %r = tensor.pad %x low[0, 1, 1, 0] high[0, 1, 1, 0] { ^bb0(%i: index, ...): tensor.yield %c : f32 }
      //        : tensor<..> to tensor<..>      (static amounts only)
      operandList(op->operands);
      acceptWord("nofold");
      for (const char *word : {"low", "high"}) {
        expectWord(word);
        expect('[');
        std::vector<int64_t> amounts;
        skip();
        if (peek() != ']') {
          do {
            skip();
            if (peek() == '%') fail("tensor.pad with dynamic amounts is outside the supported subset");
            amounts.push_back(static_cast<int64_t>(number().value));
          } while (accept(','));
        }
        expect(']');
        op->reassociation.push_back(amounts);
      }
      expect('{');
      op->body = std::make_unique<Block>();
      block(*op->body, /*allowLabel=*/true);
      expect(':');
      op->operandTypes.push_back(type());
      expectWord("to");
      op->resultTypes.push_back(type());
    } else if (n == "tensor.expand_shape" || n == "tensor.collapse_shape") {
      operandList(op->operands);
      expect('[');
      skip();
      if (peek() != ']') {
        do {
          expect('[');
          std::vector<int64_t> grp;
          skip();
          if (peek() != ']') {
            do {
              grp.push_back(static_cast<int64_t>(number().value));
            } while (accept(','));
          }
          expect(']');
          op->reassociation.push_back(grp);
        } while (accept(','));
      }
      expect(']');
      if (acceptWord("output_shape")) skipBalanced('[', ']');
      expect(':');
      op->operandTypes.push_back(type());
      expectWord("into");
      op->resultTypes.push_back(type());
    } else if (n == "shard.sharding" || n == "mesh.sharding") {
      // %s = shard.sharding @mesh4 split_axes = [[0]] [sharded_dims_offsets = [..]] : !shard.sharding
      op->callee = ident();  // the grid
      expectWord("split_axes");
      expect('=');
      expect('[');
      skip();
      if (peek() != ']') {
        do {
          expect('[');
          std::vector<int64_t> axes;
          skip();
          if (peek() != ']') {
            do {
              axes.push_back(static_cast<int64_t>(number().value));
            } while (accept(','));
          }
          expect(']');
          op->reassociation.push_back(axes);
        } while (accept(','));
      }
      expect(']');
      for (const char *extra : {"halo_sizes", "sharded_dims_offsets", "partial"})
        if (acceptWord(extra)) {
          expect('=');
          skip();
          if (peek() == '[') skipBalanced('[', ']');
          else attrValue();
        }
      expect(':');
      skip();
      while (!eof() && (identChar(s[pos]) || s[pos] == '!')) ++pos;  // !shard.sharding
      Type t;
      t.kind = Type::Scalar;
      t.elt = "sharding";
      op->resultTypes.push_back(t);
    } else if (n == "shard.shard" || n == "mesh.shard") {
      // %1 = shard.shard %0 to %s [annotate_for_users] : tensor<..>
      operandList(op->operands);
      expectWord("to");
      operandList(op->operands);
      acceptWord("annotate_for_users");
      expect(':');
      op->resultTypes.push_back(type());
    } else if (n == "gpu.alloc" || n == "memref.alloc" || n == "memref.alloca") {
      // %m = gpu.alloc [host_shared] () : memref<..>    /    %m = memref.alloc() : memref<..>
      if (acceptWord("host_shared")) op->predicate = "host_shared";
      expect('(');
      expect(')');
      skip();
      if (peek() == '{') skipBalanced('{', '}');
      expect(':');
      op->resultTypes.push_back(type());
    } else if (n == "gpu.memcpy") {
      operandList(op->operands);  // dst, src
      expect(':');
      do {
        op->operandTypes.push_back(type());
      } while (accept(','));
    } else if (n == "gpu.wait") {
      acceptWord("async");
    } else if (n == "gpu.launch_func") {
      // gpu.launch_func @mod::@kernel blocks in (..) threads in (..) args(%a : t, ...)
      op->callee = ident();
      expect(':');
      expect(':');
      op->callee += "::" + ident();
      expectWord("blocks");
      expectWord("in");
      expect('(');
      std::vector<std::string> geometry;
      operandList(geometry);
      expect(')');
      expectWord("threads");
      expectWord("in");
      expect('(');
      operandList(geometry);
      expect(')');
      if (acceptWord("dynamic_shared_memory_size")) operandList(geometry);
      if (acceptWord("args")) {
        expect('(');
        skip();
        if (peek() != ')') {
          do {
            op->operands.push_back(ident());
            expect(':');
            op->operandTypes.push_back(type());
          } while (accept(','));
        }
        expect(')');
      }
    } else if (n == "memref.load") {
      operandList(op->operands);
      expect('[');
      operandList(op->operands);
      expect(']');
      expect(':');
      Type t = type();
      op->operandTypes.push_back(t);
      Type e;
      e.kind = Type::Scalar;
      e.elt = t.elt;
      op->resultTypes.push_back(e);
    } else if (n == "memref.store") {
      operandList(op->operands);  // value, memref
      expect('[');
      operandList(op->operands);
      expect(']');
      expect(':');
      op->operandTypes.push_back(type());
    } else if (n == "memref.subview") {
      // %v = memref.subview %m[o0, o1][s0, s1][t0, t1] : memref<..> to memref<.., strided<..>>
      operandList(op->operands);
      for (int part = 0; part < 3; ++part) {
        expect('[');
        std::vector<int64_t> vals;
        skip();
        if (peek() != ']') {
          do {
            skip();
            if (peek() == '%') fail("memref.subview with dynamic offsets or sizes is outside the supported subset");
            vals.push_back(static_cast<int64_t>(number().value));
          } while (accept(','));
        }
        expect(']');
        op->reassociation.push_back(vals);
      }
      expect(':');
      op->operandTypes.push_back(type());
      expectWord("to");
      op->resultTypes.push_back(type());
    } else if (n == "vector.print") {
      if (acceptWord("str")) {
        op->text = stringLit();
      } else {
        operandList(op->operands);
        expect(':');
        op->operandTypes.push_back(type());
      }
    } else if (n == "memref.dealloc" || n == "gpu.dealloc") {
      operandList(op->operands);
      expect(':');
      op->operandTypes.push_back(type());
    } else if (n == "scf.while") {
      // %0:6 = scf.while (%a = %init, ...) : (types) -> (types) { ... scf.condition(%c) %a, ... : types }
      //        do { ^bb0(%a: type, ...): ... scf.yield ... : types }
      // (test/Jax/janet/jit__get_age_weights_from_tables.8_linalg.mlir:389-591)
      expect('(');
      skip();
      if (peek() != ')') {
        do {
          op->iterArgs.push_back(ident());
          expect('=');
          op->iterInits.push_back(ident());
        } while (accept(','));
      }
      expect(')');
      expect(':');
      op->operandTypes = typeList();
      expectArrow();
      op->resultTypes = typeList();
      expect('{');
      op->body = std::make_unique<Block>();  // the "before" region: its arguments are the names above
      op->body->args = op->iterArgs;
      op->body->argTypes = op->operandTypes;
      block(*op->body, /*allowLabel=*/false);
      expectWord("do");
      expect('{');
      op->elseBody = std::make_unique<Block>();  // the "after" region
      block(*op->elseBody, /*allowLabel=*/true);
    } else if (n == "scf.condition") {
      expect('(');
      operandList(op->operands);  // the condition, then the forwarded values
      expect(')');
      operandList(op->operands);
      if (accept(':')) {
        do {
          op->operandTypes.push_back(type());
        } while (accept(','));
      }
    } else if (n == "scf.for") {
      op->body = std::make_unique<Block>();
      op->body->args.push_back(ident());  // induction variable
      expect('=');
      operandList(op->operands);  // lb
      expectWord("to");
      operandList(op->operands);  // ub
      expectWord("step");
      operandList(op->operands);  // step
      if (acceptWord("iter_args")) {
        expect('(');
        do {
          op->iterArgs.push_back(ident());
          expect('=');
          op->iterInits.push_back(ident());
        } while (accept(','));
        expect(')');
        expectArrow();
        op->resultTypes = typeList();
      }
      expect('{');
      block(*op->body, /*allowLabel=*/false);
    } else if (n.rfind("arith.", 0) == 0 || n.rfind("math.", 0) == 0) {
      // unary / binary scalar ops: "%r = arith.addf %a, %b [fastmath<..>] : f32", and the
      // conversions written "%r = arith.extui %a : i8 to i32"
      operandList(op->operands);
      skip();
      if (startsWith("fastmath")) {
        pos += 8;
        skipBalanced('<', '>');
      }
      skip();
      if (peek() == '{') skipBalanced('{', '}');  // e.g. {overflowFlags = ...}
      expect(':');
      Type from = type();
      Type to = from;
      if (acceptWord("to")) to = type();
      op->operandTypes.push_back(from);
      op->resultTypes.push_back(to);
    } else {
      fail("operation '" + n + "' is outside the supported subset");
    }
    return op;
  }
};

} // namespace

Module parseModule(const std::string &text) { return Parser(text).module(); }
Type parseTypeString(const std::string &text) { return Parser(text).typeOnly(); }

} // namespace fe
} // namespace imex
