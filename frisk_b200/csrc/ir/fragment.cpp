// Register-fragment layouts of frisk.gemm and the layout a frisk.reduce gives its destination:
// which thread of the block owns element (i, j) of a tile, and in which of its registers.
//
// The reference builds these as affine expressions by repeated substitution
// (FriskOps.cpp:155-231 repeat / replicate, 233-287 the 8x4 / 8x8 / 8x16 / transposed-8x8 atoms,
// 304-347 the accumulator for mma.sync and wgmma, 349-451 operands A and B held in registers).
// Every such layout is a mixed-radix number: the thread id and the register index are sums of
// "digits" ((d floordiv div) mod ext) * weight taken from the row or the column coordinate.  Here
// a fragment is that digit list.  Repeating a fragment appends one digit per coordinate, evaluating
// it is a handful of integer operations, and the affine maps are written out from the digits at
// the end.  The maps equal the reference's as functions on the tile (its printed maps carry extra
// terms that are identically zero, such as "(d1 mod 8) floordiv 8"; those digits have extent 1
// and are dropped here).
//
// On sm_100a the accumulator is not a register fragment at all: it lives in tensor memory, row r
// of the tile in lane r and column c in column c.  inferGemmLayouts has that branch beside the
// Ampere and Hopper ones.
#include "ir.h"

#include <algorithm>
#include <array>
#include <cmath>
#include <cstdlib>
#include <limits>
#include <set>

namespace fir {

namespace {

struct Digit {
  int dim;          // 0: row coordinate, 1: column coordinate
  int64_t div, ext; // ((d floordiv div) mod ext)
  int64_t weight;
};

struct Fragment {
  std::array<int64_t, 2> shape{1, 1};
  std::vector<Digit> index, thread;
  int64_t indexExtent = 1, threadExtent = 1, replicate = 1;

  // One more level of tiling: the fragment is laid out r[0] x r[1] times; the copy number goes
  // to the thread id (other threads hold the copies) or to the register index (the same threads
  // hold them in further registers).  rowFastest: the row copy number is the low part of it
  // (FriskOps.cpp:163-219 with lowerDimFirst == false).
  Fragment repeat(std::array<int64_t, 2> r, bool onThread, bool rowFastest) const {
    Fragment n = *this;
    const int64_t base = onThread ? threadExtent : indexExtent;
    std::vector<Digit>& into = onThread ? n.thread : n.index;
    into.push_back({0, shape[0], r[0], base * (rowFastest ? 1 : r[1])});
    into.push_back({1, shape[1], r[1], base * (rowFastest ? r[0] : 1)});
    (onThread ? n.threadExtent : n.indexExtent) = base * r[0] * r[1];
    n.shape = {shape[0] * r[0], shape[1] * r[1]};
    return n;
  }
  // The same data in `times` groups of threads (FriskOps.cpp:224-229).
  Fragment replicated(int64_t times) const {
    Fragment n = *this;
    n.replicate *= times;
    return n;
  }

  static AffineExpr sum(const std::vector<Digit>& digits, const std::array<int64_t, 2>& shape) {
    AffineExpr e = affineConstant(0);
    for (const Digit& d : digits) {
      if (d.ext == 1) continue;
      AffineExpr x = affineDim(d.dim);
      if (d.div * d.ext < shape[d.dim]) x = affineBinary(AffineKind::Mod, x, affineConstant(d.div * d.ext));
      if (d.div > 1) x = affineBinary(AffineKind::FloorDiv, x, affineConstant(d.div));
      e = affineBinary(AffineKind::Add, e, affineBinary(AffineKind::Mul, x, affineConstant(d.weight)));
    }
    return e;
  }
  LayoutAttrData layout() const {
    LayoutAttrData l;
    l.inputShape = {shape[0], shape[1]};
    l.forwardIndex = AffineMap::get(2, 0, {sum(index, shape)});
    l.forwardThread = AffineMap::get(2, 0, {sum(thread, shape)});
    l.replicate = replicate;
    return l;
  }
};

// The atoms: 8 rows by 4 / 8 / 16 columns over one warp, `per` consecutive elements per thread,
// four threads across a row (FriskOps.cpp:233-273); `transposed` swaps the coordinates (275-287).
Fragment atom(int64_t cols, bool transposed = false) {
  const int64_t per = cols / 4;
  const int fast = transposed ? 0 : 1, slow = transposed ? 1 : 0;
  Fragment f;
  f.shape = {8, 8};
  f.shape[fast] = cols;
  f.index = {{fast, 1, per, 1}};
  f.indexExtent = per;
  f.thread = {{fast, per, 4, 1}, {slow, 1, 8, 4}};
  f.threadExtent = 32;
  return f;
}

// Accumulator for mma.sync.m16n8 (FriskOps.cpp:304-326): a 16x8 atom per warp, warps tiled over
// the block, then each warp's atoms repeated to fill its warp tile.
std::optional<Fragment> accumulatorMma(int64_t M, int64_t N, int64_t wm, int64_t wn) {
  if (wm % 16 || wn % 8 || M % wm || N % wn) return std::nullopt;
  return atom(8).repeat({2, 1}, false, false)
      .repeat({std::max<int64_t>(1, M / wm), std::max<int64_t>(1, N / wn)}, true, true)
      .repeat({std::max<int64_t>(1, wm / 16), std::max<int64_t>(1, wn / 8)}, false, true);
}

// Accumulator for wgmma (FriskOps.cpp:328-347): a warp owns 16 rows by the whole warp-tile width.
std::optional<Fragment> accumulatorWgmma(int64_t M, int64_t N, int64_t wm, int64_t wn) {
  if (wm % 16 || wn % 8 || M % wm || N % wn) return std::nullopt;
  return atom(8).repeat({2, std::max<int64_t>(1, wn / 8)}, false, true)
      .repeat({std::max<int64_t>(1, M / wm), std::max<int64_t>(1, N / wn)}, true, true)
      .repeat({std::max<int64_t>(1, wm / 16), 1}, false, true);
}

// Operand A in registers (FriskOps.cpp:349-418): 16 rows by one k-step per warp; the warps along N
// hold the same data (replicate).
std::optional<Fragment> operandA(int64_t M, int64_t N, int64_t K, int64_t wm, int64_t wn, unsigned bits,
                                 bool transposed) {
  if (M <= 0 || N <= 0 || K <= 0 || wm <= 0 || wn <= 0) return std::nullopt;
  if (M % wm || N % wn || wm % 16 || K % 16) return std::nullopt;
  if (bits != 8 && bits != 16 && bits != 32) return std::nullopt;
  const int64_t warpsM = M / wm, warpsN = N / wn;
  if (transposed)
    return atom(8, true).repeat({2, 2}, false, false).repeat({1, warpsM}, true, true)
        .replicated(warpsN).repeat({K / 16, wm / 16}, false, false);
  const int64_t kStep = bits == 8 ? 32 : bits == 16 ? 16 : 8;
  if (K % kStep) return std::nullopt;
  return atom(kStep / 2).repeat({2, 2}, false, true).repeat({warpsM, 1}, true, false)
      .replicated(warpsN).repeat({wm / 16, K / kStep}, false, true);
}

// Operand B in registers (FriskOps.cpp:420-451); the warps along M hold the same data.
std::optional<Fragment> operandB(int64_t M, int64_t N, int64_t K, int64_t wm, int64_t wn, bool transposed) {
  if (M <= 0 || N <= 0 || K <= 0 || wm <= 0 || wn <= 0) return std::nullopt;
  if (M % wm || N % wn || wn % 8 || K % 16) return std::nullopt;
  const int64_t warpsM = M / wm, warpsN = N / wn;
  if (transposed)
    return atom(8).repeat({1, 2}, false, true).replicated(warpsM).repeat({warpsN, 1}, true, true)
        .repeat({wn / 8, K / 16}, false, true);
  return atom(8, true).repeat({2, 1}, false, true).replicated(warpsM).repeat({1, warpsN}, true, false)
      .repeat({K / 16, wn / 8}, false, false);
}

struct Target {
  bool cuda = false;
  unsigned sm = 0;
  unsigned warp = 32;
};

// "sm_80", "sm90", "sm_100a" (the digits are read, a letter suffix is accepted), "gfx9.."; any
// other string counts as CUDA-like with no version (FriskOps.cpp:62-91).
std::optional<Target> targetOf(const Operation* op) {
  for (const Operation* cur = op; cur; cur = cur->parentOp()) {
    const Attribute* a = cur->attr("frisk.target");
    if (!a || !std::holds_alternative<std::string>(*a)) continue;
    std::string v = std::get<std::string>(*a);
    Target t;
    if (v.rfind("sm_", 0) == 0 || v.rfind("sm", 0) == 0) {
      v = v.substr(v[2] == '_' ? 3 : 2);
      t.cuda = true;
      t.sm = (unsigned)std::strtoul(v.c_str(), nullptr, 10);
    } else if (v.rfind("gfx", 0) == 0) {
      t.warp = v.size() > 3 && v[3] == '9' ? 64 : 32;
    } else {
      t.cuda = true;
    }
    return t;
  }
  return std::nullopt;
}

// Warps along M and N (FriskOps.cpp:825-888).
std::pair<int64_t, int64_t> warpPartition(const std::string& policy, int64_t M, int64_t N, int64_t threads,
                                          const Target& t) {
  const int64_t warps = t.warp ? threads / t.warp : 1;
  const int64_t perM = 16, perN = t.cuda && t.sm >= 70 ? 8 : 16;
  if (M == 0 || N == 0 || warps == 0) return {1, 1};
  int64_t m = 1, n = warps;
  if (policy == "FullRow") {
    m = warps;
    if (M % (m * perM) != 0) m = std::max<int64_t>(1, std::min(warps, std::max<int64_t>(1, M / perM)));
    n = std::max<int64_t>(1, warps / m);
  } else if (policy == "FullCol") {
    n = warps;
    if (N % (n * perN) != 0) n = std::max<int64_t>(1, std::min(warps, std::max<int64_t>(1, N / perN)));
    m = std::max<int64_t>(1, warps / n);
  } else {  // Square: the split whose per-warp aspect ratio is closest to the tile's
    const float ideal = (float)M / (float)N;
    float best = std::numeric_limits<float>::max();
    for (int64_t cm = 1; cm <= warps; ++cm) {
      if (warps % cm) continue;
      const int64_t cn = warps / cm;
      const float pm = (float)M / (cm * perM), pn = (float)N / (cn * perN);
      if (pm < 1 || pn < 1) continue;
      const float score = std::abs(pm / pn - ideal);
      if (score < best) {
        best = score;
        m = cm;
        n = cn;
      }
    }
  }
  return {std::max<int64_t>(m, 1), std::max<int64_t>(n, 1)};
}

}  // namespace

std::optional<int64_t> threadBlockSize(const Operation* op) {
  for (const Operation* cur = op; cur; cur = cur->parentOp()) {
    const Attribute* a = cur->attr("frisk.threads");
    if (a && std::holds_alternative<IntAttr>(*a)) return std::get<IntAttr>(*a).value;
    if (cur->name == "frisk.parallel") return cur->intAttr("threads");
  }
  return std::nullopt;
}

GemmLayouts inferGemmLayouts(const Operation* gemm) {
  GemmLayouts out;
  auto refuse = [&](const std::string& why) {
    out.ok = false;
    out.why = why;
    return out;
  };
  if (!gemm || gemm->name != "frisk.gemm") return refuse("not a frisk.gemm");
  const auto target = targetOf(gemm);
  if (!target) return refuse("layout inference requires a 'frisk.target' string attribute");
  const auto threads = threadBlockSize(gemm);
  if (!threads)
    return refuse("layout inference requires an enclosing 'frisk.parallel' operation to provide a thread count");
  const TypeStorage* ty[3];
  for (int i = 0; i < 3; ++i) {
    ty[i] = gemm->operands[i]->type.get();
    if (ty[i]->kind != TypeKind::MemRef) return refuse("all operands must be memref values for layout inference");
    const unsigned s = ty[i]->memorySpace;
    if (s != 0 && s != 1 && s != 3)
      return refuse(std::string("operand ") + "ABC"[i] + " resides in unsupported memory space " + std::to_string(s));
  }
  if (ty[2]->memorySpace != (unsigned)MemorySpace::Local) return refuse("operand C must reside in local memory space");
  for (int i = 0; i < 2; ++i)
    if (ty[i]->memorySpace == (unsigned)MemorySpace::Global)
      return refuse(std::string("operand ") + "AB"[i] +
                    " must reside in shared or local memory space for layout inference");
  const bool blackwell = target->cuda && target->sm >= 100;
  const bool hopper = target->cuda && target->sm >= 90;
  const bool ampere = target->cuda && target->sm >= 80 && target->sm < 90;
  if (!hopper && !ampere) return refuse("layout inference currently supports only Ampere or Hopper targets");

  const int64_t M = gemm->intAttr("M"), N = gemm->intAttr("N"), K = gemm->intAttr("K");
  const bool transA = gemm->intAttr("transA") != 0, transB = gemm->intAttr("transB") != 0;
  const std::string policy = std::get<EnumAttr>(*gemm->attr("policy")).value;
  // With tcgen05 one thread issues the MMA for the whole CTA tile: there is no split over warps.
  const auto [warpsM, warpsN] =
      blackwell ? std::pair<int64_t, int64_t>{1, 1} : warpPartition(policy, M, N, *threads, *target);
  if (M % warpsM || N % warpsN) return refuse("block shape must be divisible by warp partition");
  const int64_t wm = M / warpsM, wn = N / warpsN;
  out.warpsM = warpsM;
  out.warpsN = warpsN;
  const bool wgmma = hopper && *threads % 128 == 0 && M >= 64 && N >= 64;  // FriskOps.cpp:620-625
  out.instruction = blackwell ? "tcgen05" : wgmma ? "wgmma" : "mma";

  if (blackwell) {
    // tcgen05.mma reads both operands through shared-memory descriptors and accumulates in
    // tensor memory: 128 (or 64) lanes by up to 512 32-bit columns per CTA.
    if (ty[0]->memorySpace != (unsigned)MemorySpace::Shared || ty[1]->memorySpace != (unsigned)MemorySpace::Shared)
      return refuse("on sm_100 operands A and B of a gemm must reside in shared memory");
    if ((M != 64 && M != 128) || N % 8 || N < 8 || N > 512)
      return refuse("a tensor-memory accumulator tile has 64 or 128 rows and a multiple of 8 up to 512 columns");
  }

  auto shared = [&](int i, bool kInner) { return sharedLayoutForOperand(ty[i]->shape, bitWidth(ty[i]->element), kInner, hopper); };
  if (ty[0]->memorySpace == (unsigned)MemorySpace::Shared) {
    auto l = shared(0, !transA);
    if (!l) return refuse("unable to materialize shared-memory layout for operand A");
    out.a = *l;
  } else {
    auto f = operandA(M, N, K, wm, wn, bitWidth(ty[0]->element), transA);
    if (!f) return refuse("unable to build fragment layout for operand A; check tile shape and element type");
    out.a = f->layout();
  }
  if (ty[1]->memorySpace == (unsigned)MemorySpace::Shared) {
    auto l = shared(1, transB);
    if (!l) return refuse("unable to materialize shared-memory layout for operand B");
    out.b = *l;
  } else {
    auto f = operandB(M, N, K, wm, wn, transB);
    if (!f) return refuse("unable to build fragment layout for operand B; check warp policy and tile shape");
    out.b = f->layout();
  }
  if (blackwell) {
    out.c.inputShape = {M, N};
    out.c.forwardIndex = AffineMap::get(2, 0, {affineDim(1)});
    out.c.forwardThread = AffineMap::get(2, 0, {affineDim(0)});
    out.c.replicate = 1;
  } else {
    auto f = wgmma ? accumulatorWgmma(M, N, wm, wn) : accumulatorMma(M, N, wm, wn);
    if (!f) return refuse("unable to build accumulator fragment for current warp shape; check warp policy and target");
    out.c = f->layout();
  }
  out.ok = true;
  return out;
}

// ------------------------------------------------------------------------------------ reduce
// frisk.reduce removes one dimension of a register-resident buffer.  The destination keeps the
// source's maps with that coordinate taken out: in the register index it is set to 0, in the
// thread map it becomes a free symbol (every thread that held a piece of the reduced line ends up
// holding the result), and the replicate count grows by the number of distinct thread groups the
// coordinate selected (FriskOps_Reduce.cpp:214-357; the count, LayoutUtils.cpp:37-218).

namespace {

bool usesDim(const AffineExpr& e, unsigned dim) { return isFunctionOfDim(e, dim); }

int64_t ceilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

const AffineExprNode* constantOf(const AffineExpr& e) {
  return e && e->kind == AffineKind::Constant ? e.get() : nullptr;
}

// How many values the expression can take when `dim` runs over `extent` values and everything
// else is fixed: an upper estimate built bottom-up (LayoutUtils.cpp:37-111).
std::optional<int64_t> spanOf(const AffineExpr& e, unsigned dim, int64_t extent) {
  switch (e->kind) {
    case AffineKind::Constant:
    case AffineKind::SymbolId:
      return 1;
    case AffineKind::DimId:
      return (unsigned)e->value == dim ? extent : 1;
    default:
      break;
  }
  const auto l = spanOf(e->lhs, dim, extent), r = spanOf(e->rhs, dim, extent);
  if (!l || !r) return std::nullopt;
  switch (e->kind) {
    case AffineKind::Add:
      return std::max<int64_t>(1, *l + *r - 1);
    case AffineKind::Mul:
      if (auto* c = constantOf(e->rhs)) return *l * std::llabs(c->value);
      if (auto* c = constantOf(e->lhs)) return *r * std::llabs(c->value);
      return std::nullopt;
    case AffineKind::FloorDiv:
      if (auto* c = constantOf(e->rhs); c && c->value > 0) return ceilDiv(*l, c->value);
      return std::nullopt;
    case AffineKind::Mod:
      if (auto* c = constantOf(e->rhs); c && c->value > 0) return std::min(*l, c->value);
      return std::nullopt;
    default:
      return std::nullopt;
  }
}

// Every place `dim` enters the expression, as (stride it is divided by, extent that survives the
// enclosing mod / floordiv) -- LayoutUtils.cpp:113-176.
bool collectSplits(const AffineExpr& e, unsigned dim, int64_t extent, int64_t lower,
                   std::set<std::pair<int64_t, int64_t>>& splits) {
  if (!usesDim(e, dim)) return true;
  switch (e->kind) {
    case AffineKind::DimId:
      splits.insert({lower, extent});
      return true;
    case AffineKind::Add:
      return collectSplits(e->lhs, dim, extent, lower, splits) && collectSplits(e->rhs, dim, extent, lower, splits);
    case AffineKind::Mul:
      if (constantOf(e->lhs)) return collectSplits(e->rhs, dim, extent, lower, splits);
      if (constantOf(e->rhs)) return collectSplits(e->lhs, dim, extent, lower, splits);
      return false;
    case AffineKind::FloorDiv: {
      auto* c = constantOf(e->rhs);
      if (!c || c->value <= 0) return false;
      const auto span = spanOf(e->lhs, dim, extent);
      if (!span) return false;
      return collectSplits(e->lhs, dim, ceilDiv(*span, c->value), lower * c->value, splits);
    }
    case AffineKind::Mod: {
      auto* c = constantOf(e->rhs);
      if (!c || c->value <= 0) return false;
      const auto span = spanOf(e->lhs, dim, extent);
      if (!span) return false;
      return collectSplits(e->lhs, dim, std::min(*span, c->value), lower, splits);
    }
    default:
      return false;
  }
}

}  // namespace

std::optional<int64_t> usedExtentOfDim(const AffineMap& map, unsigned dim, int64_t extent) {
  if (!map.valid) return 1;
  if (extent <= 0 || dim >= map.numDims) return std::nullopt;
  std::set<std::pair<int64_t, int64_t>> splits;
  for (const AffineExpr& r : map.results)
    if (usesDim(r, dim) && !collectSplits(r, dim, extent, 1, splits)) return std::nullopt;
  int64_t used = 1;
  for (const auto& s : splits) {
    if (s.second <= 0) return std::nullopt;
    used *= s.second;
  }
  return used;
}

ReduceLayout inferReduceLayout(const Operation* reduce, const LayoutAttrData* src, const LayoutAttrData* existing) {
  ReduceLayout out;
  auto refuse = [&](const std::string& why) {
    out.ok = false;
    out.why = why;
    return out;
  };
  if (!reduce || reduce->name != "frisk.reduce") return refuse("not a frisk.reduce");
  const TypeStorage* st = reduce->operands[0]->type.get();
  const TypeStorage* dt = reduce->operands[1]->type.get();
  if (st->kind != TypeKind::MemRef || dt->kind != TypeKind::MemRef)
    return refuse("layout inference requires memref operands");
  for (const TypeStorage* t : {st, dt})
    if (t->memorySpace != 0 && t->memorySpace != 1 && t->memorySpace != 3)
      return refuse(std::string("operand ") + (t == st ? "src" : "dst") + " resides in unsupported memory space " +
                    std::to_string(t->memorySpace));
  out.ok = true;
  // Only register-resident buffers carry thread ownership; without a source fragment there is
  // nothing to derive from.
  if (st->memorySpace != (unsigned)MemorySpace::Local || dt->memorySpace != (unsigned)MemorySpace::Local) return out;
  if (!src || !src->forwardIndex.valid || !src->forwardThread.valid) return out;

  const unsigned rank = (unsigned)st->shape.size();
  if (src->inputShape.size() != rank) return refuse("source layout rank does not match source memref rank");
  const int64_t dim = reduce->intAttr("dim");
  if (dim < 0 || dim >= (int64_t)rank) return refuse("invalid reduce dimension " + std::to_string(dim));
  const int64_t extent = st->shape[dim];
  if (extent < 0) return refuse("layout inference requires static extent along the reduce dimension");
  if (extent == 0) return refuse("reduce extent must be positive for layout inference");

  // Step 1: renumber the coordinates; the reduced one moves to the last position ("placeholder").
  auto remap = [&](const AffineMap& m) {
    std::vector<AffineExpr> dims, syms;
    const AffineExpr placeholder = affineDim(rank - 1);
    for (unsigned i = 0; i < m.numDims; ++i) {
      if ((int64_t)i < dim) dims.push_back(affineDim(i));
      else if ((int64_t)i == dim)
        dims.push_back(extent == 1 ? affineConstant(0)
                                   : affineBinary(AffineKind::Mod, placeholder, affineConstant(extent)));
      else dims.push_back(affineDim(i - 1));
    }
    for (unsigned i = 0; i < m.numSymbols; ++i) syms.push_back(affineSymbol(i));
    std::vector<AffineExpr> results;
    for (const AffineExpr& r : m.results) results.push_back(replaceDimsAndSymbols(r, dims, syms));
    return AffineMap::get(rank, m.numSymbols, std::move(results));
  };
  if (src->forwardIndex.numDims != rank || src->forwardThread.numDims != rank)
    return refuse("source layout rank does not match source memref rank");
  const AffineMap index = remap(src->forwardIndex), thread = remap(src->forwardThread);

  // Step 2: how many thread groups the reduced coordinate ranged over.
  const auto used = usedExtentOfDim(thread, rank - 1, extent);
  if (!used) return refuse("unable to analyze reduce dimension usage in thread map for layout inference");
  const int64_t factor = std::max<int64_t>(1, *used);

  // Step 3: drop the placeholder (0 in the index map, a new symbol in the thread map).
  auto condense = [&](const AffineMap& m, bool keepAsSymbol) {
    const unsigned placeholder = m.numDims - 1;
    bool usedHere = false;
    for (const AffineExpr& r : m.results) usedHere = usedHere || usesDim(r, placeholder);
    unsigned nsyms = m.numSymbols;
    AffineExpr value = affineConstant(0);
    if (keepAsSymbol && usedHere) value = affineSymbol(nsyms++);
    std::vector<AffineExpr> dims, syms;
    for (unsigned i = 0; i < placeholder; ++i) dims.push_back(affineDim(i));
    dims.push_back(value);
    for (unsigned i = 0; i < m.numSymbols; ++i) syms.push_back(affineSymbol(i));
    std::vector<AffineExpr> results;
    for (const AffineExpr& r : m.results) results.push_back(replaceDimsAndSymbols(r, dims, syms));
    return AffineMap::get(placeholder, nsyms, std::move(results));
  };
  LayoutAttrData dst;
  dst.inputShape = dt->shape.empty() ? std::vector<int64_t>{1} : dt->shape;
  dst.forwardIndex = condense(index, false);
  dst.forwardThread = condense(thread, true);
  const int64_t base = src->replicate ? *src->replicate : 1;
  if (base <= 0) return refuse("source layout replicate extent must be positive");
  dst.replicate = base * factor;

  if (const auto threads = threadBlockSize(reduce); threads && *threads > 0) {
    const int64_t rep = *dst.replicate;
    if (*threads % rep != 0 && rep % *threads != 0)
      return refuse("reduce layout inference requires thread count divisible by replicate extent (threads=" +
                    std::to_string(*threads) + ", replicate=" + std::to_string(rep) + ")");
  }

  // A layout the destination already has must agree (FriskOps_Reduce.cpp:178-209).
  if (existing) {
    auto sameMap = [](const AffineMap& a, const AffineMap& b) { return a.valid == b.valid && (!a.valid || a == b); };
    const char* conflict = nullptr;
    if (existing->inputShape != dst.inputShape) conflict = "input shapes disagree";
    else if (!sameMap(existing->forwardIndex, dst.forwardIndex)) conflict = "forward index maps differ";
    else if (!sameMap(existing->forwardThread, dst.forwardThread)) conflict = "thread maps differ";
    else if (existing->replicate && *dst.replicate > *existing->replicate)
      conflict = "existing layout replicates fewer lanes than inferred";
    if (conflict) return refuse(std::string("destination layout conflicts with reduce inference: ") + conflict);
    out.layout = *existing;
    return out;
  }
  out.layout = dst;
  out.inferred = true;
  return out;
}

std::string layoutDebugString(const LayoutAttrData& l) {
  const bool fragment = l.forwardThread.valid;
  std::string s = fragment ? "Fragment(shape=[" : "Layout(shape=[";
  for (size_t i = 0; i < l.inputShape.size(); ++i) s += (i ? ", " : "") + std::to_string(l.inputShape[i]);
  s += "], index=affine_map<" + l.forwardIndex.str() + ">";
  if (fragment) s += ", thread=affine_map<" + l.forwardThread.str() + ">";
  if (l.replicate) s += ", replicate=" + std::to_string(*l.replicate);
  return s + ")";
}

}  // namespace fir
