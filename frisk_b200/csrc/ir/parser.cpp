// Reads the textual form of a module back into the IR: the custom assembly of the frisk ops as
// the reference's printers emit it (kernel FriskOps.cpp:922-951, parallel 991-1021, for
// 1118-1145, block 1220-1248, alloc_buffer 1483-1516, copy 1593-1640; gemm, fill and reduce use
// declarative formats, FriskOps.td:248-289, 348-410) and as this repository's printer reproduces
// it (ir.cpp).  A module printed by either side -- the reference's own logs included -- parses
// to a module that prints to the same text.
//
// Recursive descent over a character cursor; one function per construct.  Not supported (an
// error names them): func.func bodies, the generic "quoted" op form, #frisk.layout attributes.
#include "ir.h"

#include <cstring>

#include <cmath>

#include <cctype>
#include <cstdlib>
#include <map>
#include <stdexcept>

namespace fir {

namespace {

struct ParseError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Parser {
 public:
  Parser(const std::string& text, std::shared_ptr<Context> ctx) : s_(text), ctx_(std::move(ctx)) {}

  Operation* parseModule() {
    expectWord("module");
    Operation* mod = ctx_->newOp("builtin.module", Location{});
    if (peekWord("attributes")) {
      expectWord("attributes");
      parseAttrDict(mod);
    }
    Region* r = ctx_->newRegion(mod);
    Block* body = ctx_->newBlock();
    r->push_back(body);
    scopes_.emplace_back();
    expect('{');
    while (!peek('}')) parseOp(body);
    expect('}');
    scopes_.pop_back();
    skipWs();
    if (pos_ != s_.size()) fail("text after the module");
    return mod;
  }

 private:
  const std::string& s_;
  size_t pos_ = 0;
  std::shared_ptr<Context> ctx_;
  std::vector<std::map<std::string, Value>> scopes_;

  // ------------------------------------------------------------------ cursor
  [[noreturn]] void fail(const std::string& what) const {
    size_t line = 1, col = 1;
    for (size_t i = 0; i < pos_ && i < s_.size(); ++i) {
      if (s_[i] == '\n') {
        ++line;
        col = 1;
      } else {
        ++col;
      }
    }
    throw ParseError("line " + std::to_string(line) + ", column " + std::to_string(col) + ": " + what);
  }
  void skipWs() {
    while (pos_ < s_.size()) {
      if (std::isspace((unsigned char)s_[pos_])) {
        ++pos_;
      } else if (s_.compare(pos_, 2, "//") == 0) {
        while (pos_ < s_.size() && s_[pos_] != '\n') ++pos_;
      } else {
        break;
      }
    }
  }
  bool peek(char c) {
    skipWs();
    return pos_ < s_.size() && s_[pos_] == c;
  }
  bool accept(char c) {
    if (!peek(c)) return false;
    ++pos_;
    return true;
  }
  void expect(char c) {
    if (!accept(c)) fail(std::string("expected '") + c + "'");
  }
  bool peekStr(const std::string& w) {
    skipWs();
    return s_.compare(pos_, w.size(), w) == 0;
  }
  bool acceptStr(const std::string& w) {
    if (!peekStr(w)) return false;
    pos_ += w.size();
    return true;
  }
  void expectStr(const std::string& w) {
    if (!acceptStr(w)) fail("expected '" + w + "'");
  }
  static bool wordChar(char c) { return std::isalnum((unsigned char)c) || c == '_' || c == '.' || c == '$'; }
  bool peekWord(const std::string& w) {
    skipWs();
    return s_.compare(pos_, w.size(), w) == 0 && (pos_ + w.size() >= s_.size() || !wordChar(s_[pos_ + w.size()]));
  }
  bool acceptWord(const std::string& w) {
    if (!peekWord(w)) return false;
    pos_ += w.size();
    return true;
  }
  void expectWord(const std::string& w) {
    if (!acceptWord(w)) fail("expected '" + w + "'");
  }
  std::string word() {
    skipWs();
    const size_t b = pos_;
    while (pos_ < s_.size() && wordChar(s_[pos_])) ++pos_;
    if (b == pos_) fail("expected an identifier");
    return s_.substr(b, pos_ - b);
  }
  int64_t integer() {
    skipWs();
    const size_t b = pos_;
    if (pos_ < s_.size() && (s_[pos_] == '-' || s_[pos_] == '+')) ++pos_;
    while (pos_ < s_.size() && std::isdigit((unsigned char)s_[pos_])) ++pos_;
    if (b == pos_ || (pos_ == b + 1 && !std::isdigit((unsigned char)s_[b]))) fail("expected an integer");
    return std::strtoll(s_.substr(b, pos_ - b).c_str(), nullptr, 10);
  }
  std::string ssaName() {
    skipWs();
    if (pos_ >= s_.size() || s_[pos_] != '%') fail("expected an SSA value name");
    const size_t b = pos_++;
    while (pos_ < s_.size() && (wordChar(s_[pos_]) || s_[pos_] == '-')) ++pos_;
    return s_.substr(b, pos_ - b);
  }
  std::string quoted() {
    expect('"');
    const size_t b = pos_;
    while (pos_ < s_.size() && s_[pos_] != '"') ++pos_;
    if (pos_ >= s_.size()) fail("unterminated string");
    return s_.substr(b, pos_++ - b);
  }

  // ------------------------------------------------------------------ values
  void define(const std::string& name, Value v) { scopes_.back()[name] = v; }
  Value lookup(const std::string& name) {
    for (auto it = scopes_.rbegin(); it != scopes_.rend(); ++it) {
      auto f = it->find(name);
      if (f != it->end()) return f->second;
    }
    fail("use of undefined value " + name);
  }
  Value valueUse() { return lookup(ssaName()); }

  // ------------------------------------------------------------------ types
  Type parseType() {
    skipWs();
    if (acceptStr("memref<")) return parseShaped(true);
    if (acceptStr("tensor<")) return parseShaped(false);
    if (peek('(')) {
      std::vector<Type> in = parseTypeListParen();
      expectStr("->");
      std::vector<Type> out;
      if (peek('(')) out = parseTypeListParen();
      else out.push_back(parseType());
      return makeFunction(std::move(in), std::move(out));
    }
    const std::string w = word();
    if (w == "f16") return makeScalar(TypeKind::F16);
    if (w == "bf16") return makeScalar(TypeKind::BF16);
    if (w == "f32") return makeScalar(TypeKind::F32);
    if (w == "f64") return makeScalar(TypeKind::F64);
    if (w == "f8E4M3FN") return makeScalar(TypeKind::F8E4M3FN);
    if (w == "f8E5M2") return makeScalar(TypeKind::F8E5M2);
    if (w == "index") return makeScalar(TypeKind::Index);
    if (w.size() > 1 && w[0] == 'i' && std::isdigit((unsigned char)w[1]))
      return makeScalar(TypeKind::Integer, (unsigned)std::atoi(w.c_str() + 1));
    fail("unknown type '" + w + "'");
  }
  std::vector<Type> parseTypeListParen() {
    std::vector<Type> out;
    expect('(');
    if (!accept(')')) {
      do out.push_back(parseType());
      while (accept(','));
      expect(')');
    }
    return out;
  }
  // after "memref<" / "tensor<": dims 'x' elem [, affine_map<...>] [, space] '>'
  Type parseShaped(bool memref) {
    std::vector<int64_t> shape;
    for (;;) {
      skipWs();
      if (pos_ < s_.size() && s_[pos_] == '?') {
        ++pos_;
        shape.push_back(-1);
      } else if (pos_ < s_.size() && std::isdigit((unsigned char)s_[pos_])) {
        // a dimension is digits followed by 'x'; "8xf16" must not read "8xf16" as a word
        size_t e = pos_;
        while (e < s_.size() && std::isdigit((unsigned char)s_[e])) ++e;
        if (e >= s_.size() || s_[e] != 'x') fail("expected 'x' after a dimension");
        shape.push_back(std::strtoll(s_.substr(pos_, e - pos_).c_str(), nullptr, 10));
        pos_ = e;
      } else {
        break;
      }
      if (pos_ >= s_.size() || s_[pos_] != 'x') fail("expected 'x' after a dimension");
      ++pos_;
    }
    Type elem = parseType();
    AffineMap layout;
    unsigned space = 0;
    while (accept(',')) {
      if (acceptStr("affine_map<")) {
        layout = parseAffineMapBody();
        expect('>');
      } else {
        space = (unsigned)integer();
      }
    }
    expect('>');
    return memref ? makeMemRef(std::move(shape), std::move(elem), layout, space)
                  : makeTensor(std::move(shape), std::move(elem));
  }

  // ------------------------------------------------------------------ affine
  // Names usable inside an affine expression: d<i> / s<i> of a map, or SSA values of an index list.
  struct AffineNames {
    std::map<std::string, AffineExpr> fixed;       // d0, s0, ...
    std::vector<Value>* dimOperands = nullptr;     // SSA ids become dims in order of appearance
    std::vector<Value>* symOperands = nullptr;
  };

  AffineExpr affinePrimary(AffineNames& n) {
    skipWs();
    if (accept('(')) {
      AffineExpr e = affineSum(n);
      expect(')');
      return e;
    }
    if (accept('-')) return affineBinary(AffineKind::Mul, affinePrimary(n), affineConstant(-1));
    if (pos_ < s_.size() && std::isdigit((unsigned char)s_[pos_])) return affineConstant(integer());
    if (peek('%')) {
      if (!n.dimOperands) fail("SSA value in an affine map");
      Value v = valueUse();
      return operandExpr(*n.dimOperands, v, false);
    }
    if (acceptWord("symbol")) {
      if (!n.symOperands) fail("symbol(...) in an affine map");
      expect('(');
      Value v = valueUse();
      expect(')');
      return operandExpr(*n.symOperands, v, true);
    }
    const std::string w = word();
    auto it = n.fixed.find(w);
    if (it == n.fixed.end()) fail("unknown identifier '" + w + "' in an affine expression");
    return it->second;
  }
  static AffineExpr operandExpr(std::vector<Value>& ops, Value v, bool sym) {
    size_t i = 0;
    while (i < ops.size() && ops[i] != v) ++i;
    if (i == ops.size()) ops.push_back(v);
    return sym ? affineSymbol((unsigned)i) : affineDim((unsigned)i);
  }
  AffineExpr affineProduct(AffineNames& n) {
    AffineExpr e = affinePrimary(n);
    for (;;) {
      if (accept('*')) e = affineBinary(AffineKind::Mul, e, affinePrimary(n));
      else if (acceptWord("floordiv")) e = affineBinary(AffineKind::FloorDiv, e, affinePrimary(n));
      else if (acceptWord("ceildiv")) e = affineBinary(AffineKind::CeilDiv, e, affinePrimary(n));
      else if (acceptWord("mod")) e = affineBinary(AffineKind::Mod, e, affinePrimary(n));
      else return e;
    }
  }
  AffineExpr affineSum(AffineNames& n) {
    AffineExpr e = affineProduct(n);
    for (;;) {
      skipWs();
      if (accept('+')) {
        e = affineBinary(AffineKind::Add, e, affineProduct(n));
      } else if (peek('-') && !peekStr("->")) {
        ++pos_;
        e = affineBinary(AffineKind::Add, e,
                         affineBinary(AffineKind::Mul, affineProduct(n), affineConstant(-1)));
      } else {
        return e;
      }
    }
  }
  // "(d0, d1)[s0] -> (e0, e1)" (the text between affine_map< and >)
  AffineMap parseAffineMapBody() {
    AffineNames n;
    unsigned dims = 0, syms = 0;
    expect('(');
    if (!accept(')')) {
      do n.fixed[word()] = affineDim(dims++);
      while (accept(','));
      expect(')');
    }
    if (accept('[')) {
      if (!accept(']')) {
        do n.fixed[word()] = affineSymbol(syms++);
        while (accept(','));
        expect(']');
      }
    }
    expectStr("->");
    std::vector<AffineExpr> results;
    expect('(');
    if (!accept(')')) {
      do results.push_back(affineSum(n));
      while (accept(','));
      expect(')');
    }
    return AffineMap::get(dims, syms, std::move(results));
  }
  // "[e0, e1]" of a copy: SSA values are the map's inputs, dims first, then symbols
  AffineMap parseIndexList(std::vector<Value>& operands) {
    std::vector<Value> dimOps, symOps;
    AffineNames n;
    n.dimOperands = &dimOps;
    n.symOperands = &symOps;
    std::vector<AffineExpr> results;
    expect('[');
    if (!accept(']')) {
      do results.push_back(affineSum(n));
      while (accept(','));
      expect(']');
    }
    operands = dimOps;
    operands.insert(operands.end(), symOps.begin(), symOps.end());
    return AffineMap::get((unsigned)dimOps.size(), (unsigned)symOps.size(), std::move(results));
  }

  // ------------------------------------------------------------------ attributes
  Attribute parseAttrValue() {
    skipWs();
    if (peek('"')) return quoted();
    if (acceptWord("true")) return IntAttr{1, 1};
    if (acceptWord("false")) return IntAttr{0, 1};
    if (acceptWord("unit")) return std::monostate{};
    if (acceptStr("affine_map<")) {
      AffineMap m = parseAffineMapBody();
      expect('>');
      return m;
    }
    if (acceptStr("array<i64")) {
      DenseI64 d;
      if (accept(':')) {
        do d.values.push_back(integer());
        while (accept(','));
      }
      expect('>');
      return d;
    }
    if (acceptStr("#frisk<")) {
      EnumAttr e;
      e.mnemonic = word();
      e.value = word();
      expect('>');
      return e;
    }
    if (peekStr("#frisk.layout")) fail("#frisk.layout attributes are not read back");
    if (peekStr("memref<") || peekStr("tensor<")) return parseType();
    // a bit pattern "0x..." : type -- how infinities and NaNs of float attributes are printed
    if (peekStr("0x") || peekStr("0X")) {
      pos_ += 2;
      const size_t h = pos_;
      while (pos_ < s_.size() && std::isxdigit((unsigned char)s_[pos_])) ++pos_;
      if (h == pos_) fail("expected hexadecimal digits");
      const unsigned long long bits = std::strtoull(s_.substr(h, pos_ - h).c_str(), nullptr, 16);
      if (!accept(':')) return IntAttr{(int64_t)bits, 64};
      Type t = parseType();
      switch (t->kind) {
        case TypeKind::Integer: return IntAttr{(int64_t)bits, t->width};
        case TypeKind::Index: return IntAttr{(int64_t)bits, 64};
        case TypeKind::F64: { double d; const uint64_t u = bits; memcpy(&d, &u, 8); return FloatAttr{d, t}; }
        case TypeKind::F32: { float f; const uint32_t u = (uint32_t)bits; memcpy(&f, &u, 4); return FloatAttr{(double)f, t}; }
        case TypeKind::BF16: { float f; const uint32_t u = (uint32_t)bits << 16; memcpy(&f, &u, 4); return FloatAttr{(double)f, t}; }
        case TypeKind::F16: {
          const uint32_t sign = (bits >> 15) & 1u, ex = (bits >> 10) & 0x1Fu, man = bits & 0x3FFu;
          double v = ex == 0x1F ? (man ? std::nan("") : INFINITY)
                                : ex == 0 ? std::ldexp((double)man, -24) : std::ldexp(1.0 + man / 1024.0, (int)ex - 15);
          return FloatAttr{sign ? -v : v, t};
        }
        default: fail("a bit pattern needs an integer or a 16-, 32- or 64-bit float type");
      }
    }
    // number: integer ": iN" or float ": fN"
    const size_t b = pos_;
    if (pos_ < s_.size() && (s_[pos_] == '-' || s_[pos_] == '+')) ++pos_;
    bool isFloat = false;
    while (pos_ < s_.size() && (std::isdigit((unsigned char)s_[pos_]) || s_[pos_] == '.' || s_[pos_] == 'e' ||
                                s_[pos_] == 'E' ||
                                ((s_[pos_] == '+' || s_[pos_] == '-') && (s_[pos_ - 1] == 'e' || s_[pos_ - 1] == 'E')))) {
      if (!std::isdigit((unsigned char)s_[pos_])) isFloat = true;
      ++pos_;
    }
    if (b == pos_) {
      // a bare type (f16, i32, ...) or a float keyword
      if (acceptWord("inf") || acceptWord("nan")) fail("non-finite float attributes are not read back");
      return parseType();
    }
    const std::string num = s_.substr(b, pos_ - b);
    if (!accept(':')) {
      if (isFloat) return FloatAttr{std::strtod(num.c_str(), nullptr), makeScalar(TypeKind::F64)};
      return IntAttr{std::strtoll(num.c_str(), nullptr, 10), 64};
    }
    Type t = parseType();
    if (t->kind == TypeKind::Integer) return IntAttr{std::strtoll(num.c_str(), nullptr, 10), t->width};
    if (t->kind == TypeKind::Index) return IntAttr{std::strtoll(num.c_str(), nullptr, 10), 64};
    return FloatAttr{std::strtod(num.c_str(), nullptr), t};
  }
  void parseAttrDict(Operation* op) {
    expect('{');
    if (accept('}')) return;
    do {
      skipWs();
      const std::string key = peek('"') ? quoted() : word();
      if (accept('=')) op->attrs[key] = parseAttrValue();
      else op->attrs[key] = std::monostate{};
    } while (accept(','));
    expect('}');
  }
  std::vector<int64_t> parseI64Bracket() {
    std::vector<int64_t> v;
    expect('[');
    if (!accept(']')) {
      do v.push_back(integer());
      while (accept(','));
      expect(']');
    }
    return v;
  }
  std::vector<int64_t> parseI64Paren() {
    std::vector<int64_t> v;
    expect('(');
    if (!accept(')')) {
      do v.push_back(integer());
      while (accept(','));
      expect(')');
    }
    return v;
  }

  // ------------------------------------------------------------------ regions
  // "{ ops }" into a fresh block with the given argument names / types, ended by frisk.end.
  void parseBody(Operation* op, const std::vector<std::string>& argNames, const std::vector<Type>& argTypes) {
    Region* r = ctx_->newRegion(op);
    Block* body = ctx_->newBlock();
    r->push_back(body);
    scopes_.emplace_back();
    for (size_t i = 0; i < argTypes.size(); ++i) {
      Value a = body->addArgument(argTypes[i]);
      if (i < argNames.size()) define(argNames[i], a);
    }
    expect('{');
    while (!peek('}')) parseOp(body);
    expect('}');
    scopes_.pop_back();
    Operation* end = ctx_->newOp("frisk.end", Location{});
    body->insert(body->ops.size(), end);
  }

  // ------------------------------------------------------------------ operations
  void parseOp(Block* block) {
    skipWs();
    std::vector<std::string> results;
    if (peek('%')) {
      do results.push_back(ssaName());
      while (accept(','));
      expect('=');
    }
    skipWs();
    if (peek('"')) fail("the generic operation form is not read back");
    const std::string name = word();
    Operation* op = ctx_->newOp(name, Location{});
    block->insert(block->ops.size(), op);
    if (name == "frisk.kernel") parseKernel(op);
    else if (name == "frisk.parallel" || name == "frisk.block") parseGridOp(op, name == "frisk.parallel");
    else if (name == "frisk.for") parseFor(op);
    else if (name == "frisk.alloc_buffer") parseAlloc(op);
    else if (name == "frisk.copy") parseCopy(op);
    else if (name == "frisk.gemm") parseGemm(op);
    else if (name == "frisk.fill" || name == "frisk.reduce") parseOperandsDictTypes(op, false);
    else if (name == "frisk.end") { if (peek('{')) parseAttrDict(op); }
    else if (name == "arith.constant") parseConstant(op);
    else fail("operation '" + name + "' is not read back");
    if (results.size() != op->results.size())
      fail("'" + name + "' defines " + std::to_string(op->results.size()) + " value(s)");
    for (size_t i = 0; i < results.size(); ++i) define(results[i], op->results[i]);
  }

  void parseKernel(Operation* op) {
    expect('@');
    op->attrs["sym_name"] = word();
    std::vector<Type> in = parseTypeListParen(), out;
    if (acceptStr("->")) out = parseTypeListParen();
    op->attrs["function_type"] = makeFunction(in, out);
    std::vector<std::string> names;
    for (size_t i = 0; i < in.size(); ++i) names.push_back("%arg" + std::to_string(i));
    parseBody(op, names, in);
    if (peek('{')) parseAttrDict(op);
  }
  void parseGridOp(Operation* op, bool parallel) {
    std::vector<std::string> ivs;
    expect('(');
    if (!accept(')')) {
      do ivs.push_back(ssaName());
      while (accept(','));
      expect(')');
    }
    if (parallel) expect('=');
    else expectWord("to");
    op->attrs["ranges"] = DenseI64{parseI64Paren()};
    if (parallel) {
      expect(',');
      expectWord("threads");
      expect('=');
      op->attrs["threads"] = IntAttr{integer(), 64};
    }
    if (std::get<DenseI64>(op->attrs["ranges"]).values.size() != ivs.size())
      fail("one induction variable per range is needed");
    parseBody(op, ivs, std::vector<Type>(ivs.size(), makeScalar(TypeKind::Index)));
  }

  void parseFor(Operation* op) {
    const std::string iv = ssaName();
    expect('=');
    op->attrs["lower"] = IntAttr{integer(), 64};
    expectWord("to");
    op->attrs["upper"] = IntAttr{integer(), 64};
    int64_t step = 1;
    if (acceptWord("step")) {
      expect('=');
      step = integer();
    }
    op->attrs["step"] = IntAttr{step, 64};
    parseBody(op, {iv}, {makeScalar(TypeKind::Index)});
  }

  void parseAlloc(Operation* op) {
    Operation scratch;  // scope / alignment as printed; the rest follows from the result type
    parseAttrDict(&scratch);
    expectStr("->");
    Type t = parseType();
    if (t->kind != TypeKind::MemRef) fail("frisk.alloc_buffer must produce a memref");
    op->attrs["shape"] = DenseI64{t->shape};
    op->attrs["elementType"] = t->element;
    const Attribute* al = scratch.attr("alignment");
    op->attrs["alignment"] = al && std::holds_alternative<IntAttr>(*al) ? IntAttr{std::get<IntAttr>(*al).value, 64}
                                                                       : IntAttr{0, 64};
    op->attrs["memorySpace"] = IntAttr{(int64_t)t->memorySpace, 64};
    Value r = ctx_->newValue(t);
    r->defOp = op;
    op->results.push_back(r);
  }

  void parseCopy(Operation* op) {
    Value src = valueUse();
    std::vector<Value> srcIdx, dstIdx;
    AffineMap srcMap = parseIndexList(srcIdx);
    expect(',');
    Value dst = valueUse();
    AffineMap dstMap = parseIndexList(dstIdx);
    expect('{');
    expectWord("src_extents");
    expect('=');
    std::vector<int64_t> se = parseI64Bracket();
    expect(',');
    expectWord("dst_extents");
    expect('=');
    std::vector<int64_t> de = parseI64Bracket();
    expect('}');
    if (peek('{')) parseAttrDict(op);
    expect(':');
    Type st = parseType();
    expect(',');
    Type dt = parseType();
    if (!typeEqual(st, src->type) || !typeEqual(dt, dst->type)) fail("frisk.copy: operand types do not match");
    op->addOperand(src);
    op->addOperand(dst);
    for (Value v : srcIdx) op->addOperand(v);
    for (Value v : dstIdx) op->addOperand(v);
    op->segmentSizes = {1, 1, (int)srcIdx.size(), (int)dstIdx.size()};
    op->attrs["srcMap"] = srcMap;
    op->attrs["dstMap"] = dstMap;
    op->attrs["srcExtents"] = DenseI64{se};
    op->attrs["dstExtents"] = DenseI64{de};
  }

  void parseGemm(Operation* op) {
    expect('(');
    std::vector<Value> operands;
    do operands.push_back(valueUse());
    while (accept(','));
    expect(')');
    if (operands.size() != 3 && operands.size() != 5) fail("frisk.gemm takes A, B, C and optionally two scale vectors");
    if (peek('{')) parseAttrDict(op);
    expect(':');
    for (size_t i = 0; i < operands.size(); ++i) {
      if (i) expect(',');
      Type t = parseType();
      if (!typeEqual(t, operands[i]->type)) fail("frisk.gemm: operand types do not match");
      op->addOperand(operands[i]);
    }
  }

  // frisk.fill %m {..} : t      frisk.reduce %s, %d {..} : ts, td
  void parseOperandsDictTypes(Operation* op, bool) {
    std::vector<Value> operands;
    do operands.push_back(valueUse());
    while (accept(','));
    if (peek('{')) parseAttrDict(op);
    expect(':');
    for (size_t i = 0; i < operands.size(); ++i) {
      if (i) expect(',');
      Type t = parseType();
      if (!typeEqual(t, operands[i]->type)) fail(op->name + ": operand types do not match");
      op->addOperand(operands[i]);
    }
  }

  void parseConstant(Operation* op) {
    if (peekStr("dense<")) fail("dense constants are not read back");
    Attribute v = parseAttrValue();
    Type t;
    if (auto* i = std::get_if<IntAttr>(&v)) t = i->width == 1 ? makeScalar(TypeKind::Integer, 1) : makeScalar(TypeKind::Integer, i->width);
    else if (auto* f = std::get_if<FloatAttr>(&v)) t = f->type;
    else fail("arith.constant needs a typed number");
    op->attrs["value"] = v;
    Value r = ctx_->newValue(t);
    r->defOp = op;
    op->results.push_back(r);
  }
};

}  // namespace

Operation* parseModule(const std::string& text, std::shared_ptr<Context> ctx, std::string* error) {
  try {
    Parser p(text, std::move(ctx));
    return p.parseModule();
  } catch (const ParseError& e) {
    if (error) *error = e.what();
    return nullptr;
  }
}

}  // namespace fir
