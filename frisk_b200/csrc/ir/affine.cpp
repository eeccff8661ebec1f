// Affine expressions and maps: construction with MLIR's local simplifications, queries,
// substitution, evaluation and MLIR-compatible printing.
#include <algorithm>
#include <numeric>
#include <sstream>

#include "ir.h"

namespace fir {

namespace {

AffineExpr make(AffineKind k, int64_t v, AffineExpr l = nullptr, AffineExpr r = nullptr) {
  auto n = std::make_shared<AffineExprNode>();
  n->kind = k;
  n->value = v;
  n->lhs = std::move(l);
  n->rhs = std::move(r);
  return n;
}

bool isConst(const AffineExpr& e) { return e && e->kind == AffineKind::Constant; }
bool isBinary(const AffineExpr& e) { return e && e->kind <= AffineKind::CeilDiv; }

int64_t floorDiv(int64_t a, int64_t b) {
  int64_t q = a / b, r = a % b;
  return (r != 0 && ((r < 0) != (b < 0))) ? q - 1 : q;
}
int64_t ceilDiv(int64_t a, int64_t b) { return -floorDiv(-a, b); }
int64_t euclidMod(int64_t a, int64_t b) {
  int64_t r = a % b;
  return r < 0 ? r + b : r;
}

AffineExpr simplifyAdd(AffineExpr lhs, AffineExpr rhs) {
  if (isConst(lhs) && isConst(rhs)) return affineConstant(lhs->value + rhs->value);
  // constants, then symbolic expressions, go to the right
  if (isConst(lhs) || (isSymbolicOrConstant(lhs) && !isSymbolicOrConstant(rhs)))
    return affineBinary(AffineKind::Add, rhs, lhs);
  if (isConst(rhs) && rhs->value == 0) return lhs;
  // (x + c1) + c2 -> x + (c1 + c2)
  if (lhs->kind == AffineKind::Add && isConst(lhs->rhs) && isConst(rhs))
    return affineBinary(AffineKind::Add, lhs->lhs, affineConstant(lhs->rhs->value + rhs->value));
  // x * c1 + x * c2 -> x * (c1 + c2)   (a bare x counts as x * 1)
  auto split = [](const AffineExpr& e, AffineExpr& base, int64_t& coef) {
    if (e->kind == AffineKind::Mul && isConst(e->rhs)) {
      base = e->lhs;
      coef = e->rhs->value;
    } else {
      base = e;
      coef = 1;
    }
  };
  AffineExpr lb, rb;
  int64_t lc, rc;
  split(lhs, lb, lc);
  split(rhs, rb, rc);
  if (affineEqual(lb, rb)) return affineBinary(AffineKind::Mul, lb, affineConstant(lc + rc));
  // (x + c) + y -> (x + y) + c
  if (lhs->kind == AffineKind::Add && isConst(lhs->rhs))
    return affineBinary(AffineKind::Add, affineBinary(AffineKind::Add, lhs->lhs, rhs), lhs->rhs);
  // x - (x floordiv c) * c -> x mod c
  if (rhs->kind == AffineKind::Mul && isConst(rhs->rhs) && rhs->lhs->kind == AffineKind::FloorDiv &&
      isConst(rhs->lhs->rhs) && rhs->rhs->value == -rhs->lhs->rhs->value &&
      affineEqual(rhs->lhs->lhs, lhs))
    return affineBinary(AffineKind::Mod, lhs, rhs->lhs->rhs);
  return make(AffineKind::Add, 0, lhs, rhs);
}

AffineExpr simplifyMul(AffineExpr lhs, AffineExpr rhs) {
  if (isConst(lhs) && isConst(rhs)) return affineConstant(lhs->value * rhs->value);
  if (isConst(lhs) || (isSymbolicOrConstant(lhs) && !isSymbolicOrConstant(rhs)))
    return affineBinary(AffineKind::Mul, rhs, lhs);
  if (isConst(rhs)) {
    if (rhs->value == 1) return lhs;
    if (rhs->value == 0) return rhs;
  }
  // (x * c1) * c2 -> x * (c1 * c2)
  if (lhs->kind == AffineKind::Mul && isConst(lhs->rhs) && isConst(rhs))
    return affineBinary(AffineKind::Mul, lhs->lhs, affineConstant(lhs->rhs->value * rhs->value));
  // (x * c) * y -> (x * y) * c
  if (lhs->kind == AffineKind::Mul && isConst(lhs->rhs))
    return affineBinary(AffineKind::Mul, affineBinary(AffineKind::Mul, lhs->lhs, rhs), lhs->rhs);
  return make(AffineKind::Mul, 0, lhs, rhs);
}

AffineExpr simplifyFloorDiv(AffineExpr lhs, AffineExpr rhs) {
  if (!isConst(rhs) || rhs->value == 0) return make(AffineKind::FloorDiv, 0, lhs, rhs);
  const int64_t c = rhs->value;
  if (isConst(lhs)) return affineConstant(floorDiv(lhs->value, c));
  if (c == 1) return lhs;
  // (x * c1) floordiv c with c1 % c == 0 -> x * (c1 / c)
  if (lhs->kind == AffineKind::Mul && isConst(lhs->rhs) && lhs->rhs->value % c == 0)
    return affineBinary(AffineKind::Mul, lhs->lhs, affineConstant(lhs->rhs->value / c));
  // (a + b) floordiv c when a or b is a multiple of c
  if (lhs->kind == AffineKind::Add) {
    const int64_t ld = largestKnownDivisor(lhs->lhs), rd = largestKnownDivisor(lhs->rhs);
    if (ld % c == 0 || rd % c == 0)
      return affineBinary(AffineKind::Add, affineBinary(AffineKind::FloorDiv, lhs->lhs, rhs),
                          affineBinary(AffineKind::FloorDiv, lhs->rhs, rhs));
  }
  return make(AffineKind::FloorDiv, 0, lhs, rhs);
}

AffineExpr simplifyCeilDiv(AffineExpr lhs, AffineExpr rhs) {
  if (!isConst(rhs) || rhs->value == 0) return make(AffineKind::CeilDiv, 0, lhs, rhs);
  const int64_t c = rhs->value;
  if (isConst(lhs)) return affineConstant(ceilDiv(lhs->value, c));
  if (c == 1) return lhs;
  if (lhs->kind == AffineKind::Mul && isConst(lhs->rhs) && lhs->rhs->value % c == 0)
    return affineBinary(AffineKind::Mul, lhs->lhs, affineConstant(lhs->rhs->value / c));
  return make(AffineKind::CeilDiv, 0, lhs, rhs);
}

AffineExpr simplifyMod(AffineExpr lhs, AffineExpr rhs) {
  if (!isConst(rhs) || rhs->value < 1) return make(AffineKind::Mod, 0, lhs, rhs);
  const int64_t c = rhs->value;
  if (isConst(lhs)) return affineConstant(euclidMod(lhs->value, c));
  if (largestKnownDivisor(lhs) % c == 0) return affineConstant(0);
  // (a + b) mod c drops a term that is a multiple of c
  if (lhs->kind == AffineKind::Add) {
    if (largestKnownDivisor(lhs->lhs) % c == 0) return affineBinary(AffineKind::Mod, lhs->rhs, rhs);
    if (largestKnownDivisor(lhs->rhs) % c == 0) return affineBinary(AffineKind::Mod, lhs->lhs, rhs);
  }
  // (x mod c1) mod c with c1 % c == 0 -> x mod c
  if (lhs->kind == AffineKind::Mod && isConst(lhs->rhs) && lhs->rhs->value >= 1 &&
      lhs->rhs->value % c == 0)
    return affineBinary(AffineKind::Mod, lhs->lhs, rhs);
  return make(AffineKind::Mod, 0, lhs, rhs);
}

enum class Bind { Weak, Strong };

void printExpr(std::ostream& os, const AffineExpr& e, Bind enclosing,
               const std::function<std::string(bool, unsigned)>& name) {
  switch (e->kind) {
    case AffineKind::SymbolId:
      os << (name ? name(true, (unsigned)e->value) : "s" + std::to_string(e->value));
      return;
    case AffineKind::DimId:
      os << (name ? name(false, (unsigned)e->value) : "d" + std::to_string(e->value));
      return;
    case AffineKind::Constant: os << e->value; return;
    default: break;
  }
  const char* spelling = e->kind == AffineKind::Add        ? " + "
                         : e->kind == AffineKind::Mul      ? " * "
                         : e->kind == AffineKind::FloorDiv ? " floordiv "
                         : e->kind == AffineKind::CeilDiv  ? " ceildiv "
                                                           : " mod ";
  const AffineExpr &l = e->lhs, &r = e->rhs;
  if (e->kind != AffineKind::Add) {
    if (enclosing == Bind::Strong) os << '(';
    if (e->kind == AffineKind::Mul && isConst(r) && r->value == -1) {
      os << '-';
      printExpr(os, l, Bind::Strong, name);
    } else {
      printExpr(os, l, Bind::Strong, name);
      os << spelling;
      printExpr(os, r, Bind::Strong, name);
    }
    if (enclosing == Bind::Strong) os << ')';
    return;
  }
  if (enclosing == Bind::Strong) os << '(';
  bool done = false;
  // a + b * -c prints as a - b * c; a + -c as a - c
  if (r->kind == AffineKind::Mul && isConst(r->rhs)) {
    if (r->rhs->value == -1) {
      printExpr(os, l, Bind::Weak, name);
      os << " - ";
      printExpr(os, r->lhs, r->lhs->kind == AffineKind::Add ? Bind::Strong : Bind::Weak, name);
      done = true;
    } else if (r->rhs->value < -1) {
      printExpr(os, l, Bind::Weak, name);
      os << " - ";
      printExpr(os, r->lhs, Bind::Strong, name);
      os << " * " << -r->rhs->value;
      done = true;
    }
  }
  if (!done && isConst(r) && r->value < 0) {
    printExpr(os, l, Bind::Weak, name);
    os << " - " << -r->value;
    done = true;
  }
  if (!done) {
    printExpr(os, l, Bind::Weak, name);
    os << " + ";
    printExpr(os, r, Bind::Weak, name);
  }
  if (enclosing == Bind::Strong) os << ')';
}

}  // namespace

AffineExpr affineConstant(int64_t v) { return make(AffineKind::Constant, v); }
AffineExpr affineDim(unsigned pos) { return make(AffineKind::DimId, pos); }
AffineExpr affineSymbol(unsigned pos) { return make(AffineKind::SymbolId, pos); }

AffineExpr affineBinary(AffineKind kind, AffineExpr lhs, AffineExpr rhs) {
  if (!lhs || !rhs) return nullptr;
  switch (kind) {
    case AffineKind::Add: return simplifyAdd(std::move(lhs), std::move(rhs));
    case AffineKind::Mul: return simplifyMul(std::move(lhs), std::move(rhs));
    case AffineKind::FloorDiv: return simplifyFloorDiv(std::move(lhs), std::move(rhs));
    case AffineKind::CeilDiv: return simplifyCeilDiv(std::move(lhs), std::move(rhs));
    case AffineKind::Mod: return simplifyMod(std::move(lhs), std::move(rhs));
    default: return nullptr;
  }
}

bool affineEqual(const AffineExpr& a, const AffineExpr& b) {
  if (a == b) return true;
  if (!a || !b || a->kind != b->kind) return false;
  if (!isBinary(a)) return a->value == b->value;
  return affineEqual(a->lhs, b->lhs) && affineEqual(a->rhs, b->rhs);
}

bool isSymbolicOrConstant(const AffineExpr& e) {
  switch (e->kind) {
    case AffineKind::Constant:
    case AffineKind::SymbolId: return true;
    case AffineKind::DimId: return false;
    default: return isSymbolicOrConstant(e->lhs) && isSymbolicOrConstant(e->rhs);
  }
}

bool isPureAffine(const AffineExpr& e) {
  switch (e->kind) {
    case AffineKind::Constant:
    case AffineKind::SymbolId:
    case AffineKind::DimId: return true;
    case AffineKind::Add: return isPureAffine(e->lhs) && isPureAffine(e->rhs);
    case AffineKind::Mul:
      return isPureAffine(e->lhs) && isPureAffine(e->rhs) && (isConst(e->lhs) || isConst(e->rhs));
    default: return isPureAffine(e->lhs) && isConst(e->rhs);
  }
}

int64_t largestKnownDivisor(const AffineExpr& e) {
  switch (e->kind) {
    case AffineKind::DimId:
    case AffineKind::SymbolId: return 1;
    case AffineKind::Constant: return std::abs(e->value);
    case AffineKind::Mul: return largestKnownDivisor(e->lhs) * largestKnownDivisor(e->rhs);
    case AffineKind::Add:
    case AffineKind::Mod:
      return std::gcd(largestKnownDivisor(e->lhs), largestKnownDivisor(e->rhs));
    case AffineKind::FloorDiv:
    case AffineKind::CeilDiv: {
      if (isConst(e->rhs) && e->rhs->value != 0) {
        const int64_t d = largestKnownDivisor(e->lhs);
        if (d % e->rhs->value == 0) return std::abs(d / e->rhs->value);
      }
      return 1;
    }
  }
  return 1;
}

bool isFunctionOfDim(const AffineExpr& e, unsigned pos) {
  if (e->kind == AffineKind::DimId) return e->value == (int64_t)pos;
  if (isBinary(e)) return isFunctionOfDim(e->lhs, pos) || isFunctionOfDim(e->rhs, pos);
  return false;
}
bool isFunctionOfSymbol(const AffineExpr& e, unsigned pos) {
  if (e->kind == AffineKind::SymbolId) return e->value == (int64_t)pos;
  if (isBinary(e)) return isFunctionOfSymbol(e->lhs, pos) || isFunctionOfSymbol(e->rhs, pos);
  return false;
}

AffineExpr replaceDimsAndSymbols(const AffineExpr& e, const std::vector<AffineExpr>& dims,
                                 const std::vector<AffineExpr>& syms) {
  switch (e->kind) {
    case AffineKind::Constant: return e;
    case AffineKind::DimId:
      return (size_t)e->value < dims.size() && dims[e->value] ? dims[e->value] : e;
    case AffineKind::SymbolId:
      return (size_t)e->value < syms.size() && syms[e->value] ? syms[e->value] : e;
    default:
      return affineBinary(e->kind, replaceDimsAndSymbols(e->lhs, dims, syms),
                          replaceDimsAndSymbols(e->rhs, dims, syms));
  }
}

int64_t evaluate(const AffineExpr& e, const std::vector<int64_t>& dims,
                 const std::vector<int64_t>& syms) {
  switch (e->kind) {
    case AffineKind::Constant: return e->value;
    case AffineKind::DimId: return dims.at(e->value);
    case AffineKind::SymbolId: return syms.at(e->value);
    case AffineKind::Add: return evaluate(e->lhs, dims, syms) + evaluate(e->rhs, dims, syms);
    case AffineKind::Mul: return evaluate(e->lhs, dims, syms) * evaluate(e->rhs, dims, syms);
    case AffineKind::FloorDiv:
      return floorDiv(evaluate(e->lhs, dims, syms), evaluate(e->rhs, dims, syms));
    case AffineKind::CeilDiv:
      return ceilDiv(evaluate(e->lhs, dims, syms), evaluate(e->rhs, dims, syms));
    case AffineKind::Mod:
      return euclidMod(evaluate(e->lhs, dims, syms), evaluate(e->rhs, dims, syms));
  }
  return 0;
}

std::string printAffineExpr(const AffineExpr& e,
                            const std::function<std::string(bool, unsigned)>& name) {
  if (!e) return "<<NULL AFFINE EXPR>>";
  std::ostringstream os;
  printExpr(os, e, Bind::Weak, name);
  return os.str();
}

// ------------------------------------------------------------------------------- maps
AffineMap AffineMap::get(unsigned dims, unsigned syms, std::vector<AffineExpr> results) {
  AffineMap m;
  m.valid = true;
  m.numDims = dims;
  m.numSymbols = syms;
  m.results = std::move(results);
  return m;
}
AffineMap AffineMap::identity(unsigned rank) {
  std::vector<AffineExpr> r;
  for (unsigned i = 0; i < rank; ++i) r.push_back(affineDim(i));
  return get(rank, 0, r);
}
AffineMap AffineMap::constant(int64_t v) { return get(0, 0, {affineConstant(v)}); }
AffineMap AffineMap::minorIdentity(unsigned dims, unsigned results) {
  std::vector<AffineExpr> r;
  for (unsigned i = dims - results; i < dims; ++i) r.push_back(affineDim(i));
  return get(dims, 0, r);
}
AffineMap AffineMap::permutation(const std::vector<unsigned>& perm) {
  std::vector<AffineExpr> r;
  for (unsigned p : perm) r.push_back(affineDim(p));
  return get((unsigned)perm.size(), 0, r);
}
bool AffineMap::isIdentity() const {
  if (!valid || numDims != results.size()) return false;
  for (unsigned i = 0; i < results.size(); ++i)
    if (results[i]->kind != AffineKind::DimId || results[i]->value != (int64_t)i) return false;
  return true;
}
bool AffineMap::isMinorIdentity() const {
  if (!valid || results.size() > numDims) return false;
  const unsigned off = numDims - (unsigned)results.size();
  for (unsigned i = 0; i < results.size(); ++i)
    if (results[i]->kind != AffineKind::DimId || results[i]->value != (int64_t)(i + off)) return false;
  return true;
}
bool AffineMap::isProjectedPermutation(bool allowZero) const {
  if (!valid || numSymbols > 0 || results.size() > numDims) return false;
  std::vector<bool> seen(numDims, false);
  for (auto& e : results) {
    if (e->kind == AffineKind::DimId) {
      if (seen[e->value]) return false;
      seen[e->value] = true;
    } else if (!(allowZero && e->kind == AffineKind::Constant && e->value == 0)) {
      return false;
    }
  }
  return true;
}
bool AffineMap::isPermutation() const {
  return valid && numDims == results.size() && isProjectedPermutation(false);
}
bool AffineMap::operator==(const AffineMap& o) const {
  if (valid != o.valid) return false;
  if (!valid) return true;
  if (numDims != o.numDims || numSymbols != o.numSymbols || results.size() != o.results.size())
    return false;
  for (size_t i = 0; i < results.size(); ++i)
    if (!affineEqual(results[i], o.results[i])) return false;
  return true;
}
std::string AffineMap::str() const {
  if (!valid) return "<<NULL AFFINE MAP>>";
  std::ostringstream os;
  os << '(';
  for (unsigned i = 0; i < numDims; ++i) os << (i ? ", " : "") << 'd' << i;
  os << ')';
  if (numSymbols) {
    os << '[';
    for (unsigned i = 0; i < numSymbols; ++i) os << (i ? ", " : "") << 's' << i;
    os << ']';
  }
  os << " -> (";
  for (size_t i = 0; i < results.size(); ++i) os << (i ? ", " : "") << printAffineExpr(results[i]);
  os << ')';
  return os.str();
}

}  // namespace fir
