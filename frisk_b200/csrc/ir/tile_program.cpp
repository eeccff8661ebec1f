// Recognises the tiled matrix product written with the ops around frisk.gemm and lifts it to one
// whole-problem GEMM.
//
// The reference's sketch of the intended program (tmp/ir.mlir:1-17) is
//
//   frisk.kernel @matmul(%A, %B, %C)
//     frisk.parallel %by, %bx : ((GY, GX), threads)
//       %a = alloc_buffer [TM, TK] shared      %b = alloc_buffer [TK, TN] shared
//       %c = alloc_buffer [TM, TN] local       frisk.fill %c, 0.0
//       frisk.for %k = lb to ub step st
//         frisk.copy A[by*TM, k*..] -> %a      frisk.copy B[k*.., bx*TN] -> %b
//         frisk.gemm(%a, %b, %c)
//       frisk.copy %c -> C[by*TM, bx*TN]
//
// built from FriskOps.td:81-228 (parallel, for, alloc_buffer), 348-410 (copy, fill) and 248-289
// (gemm).  On a B200 the tile sizes, the staging through shared memory and the grid are the back
// end's own choice, so the program is not interpreted op by op: it is checked to be exactly this
// product (every tile of C written once, every k-slice visited once, plain sub-block copies) and
// then handed to the GEMM planner as C = A x B over the kernel's arguments.  Anything that does not
// match is refused with the reason; nothing is guessed.
#include "ir.h"

#include <array>
#include <limits>
#include <stdexcept>
#include <string>

namespace fir {

namespace {

struct Fail {
  std::string why;
};

[[noreturn]] void fail(const std::string& why) { throw Fail{why}; }

bool isTerminatorOrNothing(const Operation* op) { return op->isTerminator(); }

const std::vector<int64_t>& dense(const Operation* op, const char* name) {
  const Attribute* a = op->attr(name);
  if (!a || !std::holds_alternative<DenseI64>(*a)) fail(op->name + ": missing attribute " + name);
  return std::get<DenseI64>(*a).values;
}

const AffineMap& mapAttr(const Operation* op, const char* name) {
  const Attribute* a = op->attr(name);
  if (!a || !std::holds_alternative<AffineMap>(*a)) fail(op->name + ": missing attribute " + name);
  return std::get<AffineMap>(*a);
}

// The three loop variables an index may be: the two block indices and the k-loop variable.
struct Ivs {
  Value by = nullptr, bx = nullptr, k = nullptr;
};

// origin[r] = coef[r][0]*by + coef[r][1]*bx + coef[r][2]*k + coef[r][3], for both coordinates.
struct Origin {
  std::array<std::array<int64_t, 4>, 2> coef{};
};

// Evaluates the copy's map at probe points to read the origin off as a linear form of
// (by, bx, k), and checks with a mixed point that it is linear at all.
Origin originOf(const Operation* copy, bool srcSide, const Ivs& ivs) {
  const AffineMap& map = mapAttr(copy, srcSide ? "srcMap" : "dstMap");
  if (map.results.size() != 2) fail("frisk.copy: only rank-2 buffers are lifted");
  const int first = srcSide ? 2 : 2 + copy->segmentSizes[2];
  const int count = srcSide ? copy->segmentSizes[2] : copy->segmentSizes[3];
  if ((int)(map.numDims + map.numSymbols) != count) fail("frisk.copy: map inputs and indices differ");
  std::vector<int> which(count);
  for (int i = 0; i < count; ++i) {
    Value v = copy->operands[first + i];
    which[i] = v == ivs.by ? 0 : v == ivs.bx ? 1 : v == ivs.k ? 2 : -1;
    if (which[i] < 0) fail("frisk.copy: an index is neither a block index nor the loop variable");
  }
  auto at = [&](std::array<int64_t, 3> p, int r) {
    std::vector<int64_t> dims(map.numDims), syms(map.numSymbols);
    for (int i = 0; i < count; ++i) {
      const int64_t val = p[which[i]];
      if (i < (int)map.numDims) dims[i] = val;
      else syms[i - map.numDims] = val;
    }
    return evaluate(map.results[r], dims, syms);
  };
  Origin o;
  for (int r = 0; r < 2; ++r) {
    const int64_t c = at({0, 0, 0}, r);
    o.coef[r] = {at({1, 0, 0}, r) - c, at({0, 1, 0}, r) - c, at({0, 0, 1}, r) - c, c};
    const int64_t want = 3 * o.coef[r][0] + 5 * o.coef[r][1] + 7 * o.coef[r][2] + c;
    if (at({3, 5, 7}, r) != want) fail("frisk.copy: the origin is not linear in the loop variables");
  }
  return o;
}

bool isZeroOrigin(const Origin& o) {
  for (auto& row : o.coef)
    for (int64_t v : row)
      if (v != 0) return false;
  return true;
}

int argIndex(const Block* entry, Value v) {
  if (!v || v->block != entry) return -1;
  return (int)v->index;
}

const TypeStorage* memref2d(Value v, const char* what) {
  if (!v || !v->type || v->type->kind != TypeKind::MemRef || v->type->shape.size() != 2)
    fail(std::string(what) + " is not a rank-2 memref");
  return v->type.get();
}

}  // namespace

TiledGemm liftTiledGemm(Operation* kernel) {
  TiledGemm out;
  try {
    if (!kernel || kernel->name != "frisk.kernel" || kernel->regions.empty() ||
        kernel->regions[0]->blocks.empty())
      fail("not a frisk.kernel with a body");
    const Block* entry = kernel->regions[0]->blocks[0];

    // ---- the kernel body: one parallel op
    const Operation* par = nullptr;
    for (const Operation* op : entry->ops) {
      if (isTerminatorOrNothing(op)) continue;
      if (op->name != "frisk.parallel" || par) fail("the kernel body must be one frisk.parallel");
      par = op;
    }
    if (!par || par->regions.empty() || par->regions[0]->blocks.empty())
      fail("the kernel body must be one frisk.parallel");
    const std::vector<int64_t>& grid = dense(par, "ranges");
    const Block* pbody = par->regions[0]->blocks[0];
    if (grid.size() != 2 || pbody->args.size() != 2) fail("the grid must have two dimensions");
    Ivs ivs;
    ivs.by = pbody->args[0];
    ivs.bx = pbody->args[1];

    // ---- the block body: allocs, at most one fill / one load of the accumulator, one for, one
    // store; then, optionally, a frisk.reduce of the accumulator tile and the copy of its result
    const Operation *loop = nullptr, *fill = nullptr, *store = nullptr, *preload = nullptr;
    const Operation *reduce = nullptr, *rstore = nullptr;
    for (const Operation* op : pbody->ops) {
      if (isTerminatorOrNothing(op) || op->name == "frisk.alloc_buffer") continue;
      if (op->name == "frisk.fill" && !loop && !fill) fill = op;
      else if (op->name == "frisk.for" && !loop) loop = op;
      else if (op->name == "frisk.copy" && !loop && !preload) preload = op;
      else if (op->name == "frisk.copy" && loop && !store) store = op;
      else if (op->name == "frisk.reduce" && store && !reduce) reduce = op;
      else if (op->name == "frisk.copy" && reduce && !rstore) rstore = op;
      else fail("unexpected " + op->name + " in the block body");
    }
    if (reduce && !rstore) fail("the reduce of the accumulator tile needs a frisk.copy of its result after it");
    if (!loop || !store) fail("the block body needs a frisk.for and a frisk.copy of the result after it");
    const Block* lbody = loop->regions.at(0)->blocks.at(0);
    ivs.k = lbody->args.at(0);
    const int64_t lb = loop->intAttr("lower"), ub = loop->intAttr("upper"), st = loop->intAttr("step");
    if (st <= 0 || ub <= lb) fail("the k loop must run forwards at least once");
    const int64_t trips = (ub - lb + st - 1) / st;

    // ---- the loop body: two copies into tiles and the gemm on them
    const Operation* gemm = nullptr;
    std::vector<const Operation*> loads;
    for (const Operation* op : lbody->ops) {
      if (isTerminatorOrNothing(op)) continue;
      if (op->name == "frisk.gemm" && !gemm) gemm = op;
      else if (op->name == "frisk.copy" && !gemm) loads.push_back(op);
      else fail("unexpected " + op->name + " in the k loop");
    }
    if (!gemm || loads.size() != 2) fail("the k loop must be two frisk.copy and one frisk.gemm");
    // scale vectors of an 8-bit float gemm have no meaning per tile, and the tiles are copied in
    // row-major [TM,TK] / [TK,TN] order, so a transposed operand cannot be what the program means
    if (gemm->operands.size() != 3) fail("the gemm in the loop must not carry scale operands");
    if (gemm->intAttr("transA") || gemm->intAttr("transB"))
      fail("the gemm in the loop must not transpose its tiles (transA = transB = false)");
    Value ta = gemm->operands.at(0), tb = gemm->operands.at(1), tc = gemm->operands.at(2);
    for (Value t : {ta, tb, tc})
      if (!t->defOp || t->defOp->name != "frisk.alloc_buffer" || t->defOp->parent != pbody)
        fail("the gemm operands must be buffers allocated in the block body");
    if (ta == tb || ta == tc || tb == tc) fail("the gemm operands must be three different buffers");
    const TypeStorage *tat = memref2d(ta, "the A tile"), *tbt = memref2d(tb, "the B tile"),
                      *tct = memref2d(tc, "the C tile");
    const int64_t TM = tat->shape[0], TK = tat->shape[1], TN = tbt->shape[1];
    if (tbt->shape[0] != TK || tct->shape[0] != TM || tct->shape[1] != TN || TM <= 0 || TN <= 0 || TK <= 0)
      fail("tile shapes must be [TM,TK], [TK,TN], [TM,TN]");

    auto loadOf = [&](Value tile, const char* what) -> const Operation* {
      const Operation* found = nullptr;
      for (const Operation* c : loads)
        if (c->operands.at(1) == tile) {
          if (found) fail(std::string("two copies write ") + what);
          found = c;
        }
      if (!found) fail(std::string("no copy writes ") + what);
      return found;
    };
    const Operation *la = loadOf(ta, "the A tile"), *lbop = loadOf(tb, "the B tile");

    // a load: global argument -> whole tile
    auto checkLoad = [&](const Operation* c, int64_t rows, int64_t cols, const char* what) {
      const int arg = argIndex(entry, c->operands.at(0));
      if (arg < 0) fail(std::string(what) + " is not loaded from a kernel argument");
      const TypeStorage* g = memref2d(c->operands.at(0), what);
      if (g->memorySpace != 1) fail(std::string(what) + " must be loaded from GLOBAL memory");
      const auto &se = dense(c, "srcExtents"), &de = dense(c, "dstExtents");
      if (se != std::vector<int64_t>{rows, cols} || de != se)
        fail(std::string(what) + ": the copy must cover exactly the tile");
      if (!isZeroOrigin(originOf(c, false, ivs))) fail(std::string(what) + ": the tile must be filled from its origin");
      return arg;
    };
    out.argA = checkLoad(la, TM, TK, "A");
    out.argB = checkLoad(lbop, TK, TN, "B");
    const Origin oa = originOf(la, true, ivs), ob = originOf(lbop, true, ivs);

    // rows of A follow by, columns of A follow k; rows of B follow k, columns of B follow bx
    const std::array<int64_t, 4> rowsA{TM, 0, 0, 0}, colsB{0, TN, 0, 0};
    if (oa.coef[0] != rowsA) fail("A tile rows must start at by * TM");
    if (ob.coef[1] != colsB) fail("B tile columns must start at bx * TN");
    if (oa.coef[1] != ob.coef[0]) fail("A and B must walk K the same way");
    const auto& kc = oa.coef[1];
    if (kc[0] != 0 || kc[1] != 0) fail("the K offset may depend on the loop variable only");
    // k = lb, lb+st, ...: offsets kc[2]*k + kc[3] must be 0, TK, 2 TK, ...
    if (kc[2] * lb + kc[3] != 0 || kc[2] * st != TK) fail("the k loop must visit consecutive slices of TK");

    // ---- the result: accumulator tile -> global argument at (by*TM, bx*TN)
    if (store->operands.at(0) != tc) fail("the copy after the loop must read the C tile");
    out.argC = argIndex(entry, store->operands.at(1));
    if (out.argC < 0) fail("C is not stored to a kernel argument");
    const TypeStorage* gc = memref2d(store->operands.at(1), "C");
    if (gc->memorySpace != 1) fail("C must be stored to GLOBAL memory");
    if (dense(store, "srcExtents") != std::vector<int64_t>{TM, TN} ||
        dense(store, "dstExtents") != std::vector<int64_t>{TM, TN})
      fail("C: the copy must cover exactly the tile");
    if (!isZeroOrigin(originOf(store, true, ivs))) fail("C: the tile must be read from its origin");
    const Origin oc = originOf(store, false, ivs);
    const std::array<int64_t, 4> colsC{0, TN, 0, 0};
    if (oc.coef[0] != rowsA || oc.coef[1] != colsC) fail("C tiles must land at (by * TM, bx * TN)");

    // ---- how the accumulator starts
    if (fill) {
      if (fill->operands.at(0) != tc) fail("the fill before the loop must clear the C tile");
      const Attribute* v = fill->attr("value");
      if (!v || !std::holds_alternative<FloatAttr>(*v) || std::get<FloatAttr>(*v).value != 0.0)
        fail("the C tile must be filled with zero");
      if (preload) fail("the C tile is both filled and loaded");
      out.clearAccum = true;
    } else if (preload) {
      if (preload->operands.at(1) != tc || preload->operands.at(0) != store->operands.at(1))
        fail("the copy before the loop must load the C tile from C");
      const Origin op0 = originOf(preload, true, ivs);
      if (op0.coef[0] != rowsA || op0.coef[1] != colsC || !isZeroOrigin(originOf(preload, false, ivs)))
        fail("the C tile must be loaded from (by * TM, bx * TN)");
      out.clearAccum = false;
    } else {
      fail("the C tile is neither cleared nor loaded before the loop");
    }
    if (gemm->intAttr("clear_accum")) fail("the gemm in the loop must accumulate (clear_accum = false)");

    // ---- the whole problem
    out.M = grid[0] * TM;
    out.N = grid[1] * TN;
    out.K = trips * TK;
    const TypeStorage *ga = la->operands[0]->type.get(), *gb = lbop->operands[0]->type.get();
    if (ga->shape != std::vector<int64_t>{out.M, out.K}) fail("the grid and the loop must cover A exactly");
    if (gb->shape != std::vector<int64_t>{out.K, out.N}) fail("the grid and the loop must cover B exactly");
    if (gc->shape != std::vector<int64_t>{out.M, out.N}) fail("the grid must cover C exactly");
    if (out.argA == out.argC || out.argB == out.argC) fail("C must not alias A or B");
    out.elemAB = ga->element;
    out.elemC = gc->element;
    if (!typeEqual(ga->element, gb->element)) fail("A and B must have one element type");
    out.tile = {TM, TN, TK};
    out.grid = {grid[0], grid[1]};

    // ---- the row fold behind the product (the reference's attention sketch reduces the
    // accumulator of its first gemm this way, tmp/ir.mlir:112-135)
    if (reduce) {
      if (grid[1] != 1) fail("a reduce of the accumulator tile is lifted only when a tile holds whole rows of C (one tile column)");
      if (reduce->operands.at(0) != tc) fail("the reduce must read the accumulator tile");
      if (reduce->intAttr("dim") != 1) fail("the reduce must fold the accumulator's columns (dim = 1)");
      const Attribute* kind = reduce->attr("kind");
      if (!kind || !std::holds_alternative<std::string>(*kind)) fail("frisk.reduce: missing kind");
      Value rt = reduce->operands.at(1);
      if (!rt->defOp || rt->defOp->name != "frisk.alloc_buffer" || rt->defOp->parent != pbody)
        fail("the reduce must write a buffer allocated in the block body");
      if (!rt->type || rt->type->kind != TypeKind::MemRef || rt->type->shape != std::vector<int64_t>{TM})
        fail("the reduce's destination must have one element per row of the tile");
      if (rstore->operands.at(0) != rt) fail("the copy after the reduce must read its destination");
      out.argR = argIndex(entry, rstore->operands.at(1));
      if (out.argR < 0) fail("the reduce's result is not copied to a kernel argument");
      const TypeStorage* gr = rstore->operands.at(1)->type.get();
      if (!gr || gr->kind != TypeKind::MemRef || gr->memorySpace != 1 || gr->shape != std::vector<int64_t>{out.M})
        fail("the reduce's result must go to a GLOBAL buffer of M elements");
      if (!typeEqual(gr->element, gc->element)) fail("the reduce's result must have C's element type");
      if (out.argR == out.argA || out.argR == out.argB || out.argR == out.argC)
        fail("the reduce's result must not alias A, B or C");
      if (dense(rstore, "srcExtents") != std::vector<int64_t>{TM} || dense(rstore, "dstExtents") != std::vector<int64_t>{TM})
        fail("the copy of the reduce's result must cover exactly the tile's rows");
      // rank-1 origins: the source from 0, the destination at by * TM
      const AffineMap& sm = mapAttr(rstore, "srcMap");
      const AffineMap& dm = mapAttr(rstore, "dstMap");
      if (sm.results.size() != 1 || dm.results.size() != 1) fail("the copy of the reduce's result must be rank 1");
      const int nsrc = rstore->segmentSizes[2], ndst = rstore->segmentSizes[3];
      auto eval1 = [&](const AffineMap& map, int first, int count, int64_t by) {
        if ((int)(map.numDims + map.numSymbols) != count) fail("frisk.copy: map inputs and indices differ");
        std::vector<int64_t> dims(map.numDims), syms(map.numSymbols);
        for (int i = 0; i < count; ++i) {
          if (rstore->operands[first + i] != ivs.by) fail("the reduce's result may be placed by the row block index only");
          if (i < (int)map.numDims) dims[i] = by;
          else syms[i - map.numDims] = by;
        }
        return evaluate(map.results[0], dims, syms);
      };
      if (eval1(sm, 2, nsrc, 0) != 0 || eval1(sm, 2, nsrc, 3) != 0) fail("the reduce's result must be read from its origin");
      if (eval1(dm, 2 + nsrc, ndst, 0) != 0 || eval1(dm, 2 + nsrc, ndst, 1) != TM || eval1(dm, 2 + nsrc, ndst, 5) != 5 * TM)
        fail("the reduce's result must land at by * TM");
      out.reduceKind = std::get<std::string>(*kind);
      out.reduceClear = reduce->intAttr("clear", 1) != 0;
    }
    out.ok = true;
  } catch (const Fail& f) {
    out.ok = false;
    out.why = f.why;
  } catch (const std::out_of_range&) {
    out.ok = false;
    out.why = "malformed operation (missing operand or region)";
  }
  return out;
}

// ---------------------------------------------------------------------------------------------
// The tiled reduce.  The reference's online-softmax sketch (tmp/ir.mlir:22-36) walks a row of a
// GLOBAL matrix in tiles inside a frisk.parallel body and reduces every tile with frisk.reduce;
// written with the ops the builder has (FriskOps.td:81-228 parallel / for / alloc_buffer, 348-410
// copy / fill, FriskOps_Reduce.cpp reduce) the whole-row fold is
//
//   frisk.kernel @k(%X: [R, C] global, %Y: [R] global)            (dim = 1; dim = 0 mirrored)
//     frisk.parallel %b : ((G), threads)
//       %x = alloc_buffer [TR, TC]        %m = alloc_buffer [TR]
//       frisk.fill %m, identity of the kind      |  frisk.copy Y[b*TR] -> %m
//       frisk.for %i = lb to ub step st
//         frisk.copy X[b*TR, i*..] -> %x
//         frisk.reduce %x -> %m  {dim = 1, clear = false}
//       frisk.copy %m -> Y[b*TR]
//
// (without the loop when one tile spans the reduced dimension).  As with the matrix product, the
// program is checked to be exactly this fold -- every element of X visited once, every element of
// Y written once -- and run as ONE whole-buffer reduce; tile sizes and the grid are the back end's.
namespace {

// origin of a rank-1 copy side as a * b + c, the only index allowed being the block index
std::array<int64_t, 2> origin1(const Operation* copy, bool srcSide, Value b) {
  const AffineMap& map = mapAttr(copy, srcSide ? "srcMap" : "dstMap");
  if (map.results.size() != 1) fail("frisk.copy: the accumulator moves as a rank-1 buffer");
  const int first = srcSide ? 2 : 2 + copy->segmentSizes[2];
  const int count = srcSide ? copy->segmentSizes[2] : copy->segmentSizes[3];
  if ((int)(map.numDims + map.numSymbols) != count) fail("frisk.copy: map inputs and indices differ");
  auto at = [&](int64_t v) {
    std::vector<int64_t> dims(map.numDims), syms(map.numSymbols);
    for (int i = 0; i < count; ++i) {
      if (copy->operands[first + i] != b) fail("frisk.copy: the accumulator may be placed by the block index only");
      if (i < (int)map.numDims) dims[i] = v;
      else syms[i - map.numDims] = v;
    }
    return evaluate(map.results[0], dims, syms);
  };
  const int64_t c = at(0), a = at(1) - c;
  if (at(5) != 5 * a + c) fail("frisk.copy: the origin is not linear in the block index");
  return {a, c};
}

double identityOf(const std::string& kind) {
  if (kind == "add") return 0.0;
  if (kind == "mul") return 1.0;
  if (kind == "min") return std::numeric_limits<double>::infinity();
  return -std::numeric_limits<double>::infinity();
}

}  // namespace

TiledReduce liftTiledReduce(Operation* kernel) {
  TiledReduce out;
  try {
    if (!kernel || kernel->name != "frisk.kernel" || kernel->regions.empty() ||
        kernel->regions[0]->blocks.empty())
      fail("not a frisk.kernel with a body");
    const Block* entry = kernel->regions[0]->blocks[0];
    const Operation* par = nullptr;
    for (const Operation* op : entry->ops) {
      if (isTerminatorOrNothing(op)) continue;
      if (op->name != "frisk.parallel" || par) fail("the kernel body must be one frisk.parallel");
      par = op;
    }
    if (!par || par->regions.empty() || par->regions[0]->blocks.empty())
      fail("the kernel body must be one frisk.parallel");
    const std::vector<int64_t>& grid = dense(par, "ranges");
    const Block* pbody = par->regions[0]->blocks[0];
    if (grid.size() != 1 || pbody->args.size() != 1) fail("the grid of a tiled reduce has one dimension");
    Ivs ivs;
    ivs.by = pbody->args[0];

    // ---- the block body: allocs, a fill or a load of the accumulator, a loop (or the bare tile
    // load and reduce), the store of the accumulator
    const Operation *loop = nullptr, *fill = nullptr, *preload = nullptr, *store = nullptr;
    const Operation *load = nullptr, *reduce = nullptr;
    auto body = [&](const Block* blk, bool inLoop) {
      for (const Operation* op : blk->ops) {
        if (isTerminatorOrNothing(op)) continue;
        if (!inLoop && op->name == "frisk.alloc_buffer") continue;
        if (!inLoop && op->name == "frisk.for" && !loop && !load && !store) { loop = op; continue; }
        if (!inLoop && loop) {
          if (op->name == "frisk.copy" && !store) { store = op; continue; }
          fail("unexpected " + op->name + " behind the loop");
        }
        if (op->name == "frisk.fill" && !inLoop && !fill && !load) fill = op;
        else if (op->name == "frisk.copy" && !reduce && !load && !inLoop && !preload && !fill &&
                 op->operands.at(1)->type && op->operands.at(1)->type->shape.size() == 1) preload = op;
        else if (op->name == "frisk.copy" && !load) load = op;
        else if (op->name == "frisk.reduce" && load && !reduce) reduce = op;
        else if (op->name == "frisk.copy" && reduce && !inLoop && !store) store = op;
        else fail("unexpected " + op->name + (inLoop ? " in the loop" : " in the block body"));
      }
    };
    body(pbody, false);
    int64_t lb = 0, st = 1, trips = 1;
    if (loop) {
      const Block* lbody = loop->regions.at(0)->blocks.at(0);
      ivs.k = lbody->args.at(0);
      lb = loop->intAttr("lower");
      st = loop->intAttr("step");
      const int64_t ub = loop->intAttr("upper");
      if (st <= 0 || ub <= lb) fail("the loop must run forwards at least once");
      trips = (ub - lb + st - 1) / st;
      body(lbody, true);
    }
    if (!load || !reduce) fail("the body needs a frisk.copy into a tile and a frisk.reduce of the tile");
    if (!store) fail("the accumulator is not copied out");

    // ---- the tile, the accumulator, the reduce between them
    Value tx = reduce->operands.at(0), tm = reduce->operands.at(1);
    for (Value t : {tx, tm})
      if (!t->defOp || t->defOp->name != "frisk.alloc_buffer" || t->defOp->parent != pbody)
        fail("the reduce must work on buffers allocated in the block body");
    const TypeStorage* xt = memref2d(tx, "the tile");
    const int64_t dim = reduce->intAttr("dim");
    if (dim != 0 && dim != 1) fail("the reduce must fold dimension 0 or 1 of the tile");
    const int64_t keep = 1 - dim;   // the tile dimension that survives
    const int64_t T[2] = {xt->shape[0], xt->shape[1]};
    if (T[0] <= 0 || T[1] <= 0) fail("the tile must have a static shape");
    if (!tm->type || tm->type->kind != TypeKind::MemRef || tm->type->shape != std::vector<int64_t>{T[keep]})
      fail("the accumulator must have one element per kept row or column of the tile");
    const Attribute* kind = reduce->attr("kind");
    if (!kind || !std::holds_alternative<std::string>(*kind)) fail("frisk.reduce: missing kind");
    out.kind = std::get<std::string>(*kind);
    const bool opClear = reduce->intAttr("clear", 1) != 0;
    if (loop && trips > 1 && opClear)
      fail("the reduce in the loop must fold into the accumulator (clear = false): with clear = true only the last tile would count");

    // ---- the load: GLOBAL argument -> whole tile, walking the reduced dimension with the loop
    if (load->operands.at(1) != tx) fail("the copy before the reduce must fill the tile the reduce reads");
    out.argSrc = argIndex(entry, load->operands.at(0));
    if (out.argSrc < 0) fail("the tile is not loaded from a kernel argument");
    const TypeStorage* gx = memref2d(load->operands.at(0), "the source");
    if (gx->memorySpace != 1) fail("the source must live in GLOBAL memory");
    const std::vector<int64_t> whole{T[0], T[1]};
    if (dense(load, "srcExtents") != whole || dense(load, "dstExtents") != whole)
      fail("the load must cover exactly the tile");
    if (!isZeroOrigin(originOf(load, false, ivs))) fail("the tile must be filled from its origin");
    const Origin ox = originOf(load, true, ivs);
    const std::array<int64_t, 4> keptWant{T[keep], 0, 0, 0};
    if (ox.coef[keep] != keptWant) fail("the kept dimension of the tile must start at block index * tile extent");
    const auto& rc = ox.coef[dim];
    if (rc[0] != 0 || rc[1] != 0) fail("the offset along the reduced dimension may depend on the loop variable only");
    if (loop) {
      if (rc[2] * lb + rc[3] != 0 || (trips > 1 && rc[2] * st != T[dim]))
        fail("the loop must visit consecutive tiles of the reduced dimension");
    } else if (rc[2] != 0 || rc[3] != 0) {
      fail("without a loop the tile must start at the origin of the reduced dimension");
    }
    std::vector<int64_t> shape(2);
    shape[keep] = grid[0] * T[keep];
    shape[dim] = trips * T[dim];
    if (gx->shape != shape) fail("the grid and the loop must cover the source exactly");

    // ---- the store: accumulator -> GLOBAL argument at block index * tile extent
    if (store->operands.at(0) != tm) fail("the copy at the end must read the accumulator");
    out.argDst = argIndex(entry, store->operands.at(1));
    if (out.argDst < 0) fail("the result is not copied to a kernel argument");
    const TypeStorage* gy = store->operands.at(1)->type.get();
    if (!gy || gy->kind != TypeKind::MemRef || gy->memorySpace != 1 || gy->shape != std::vector<int64_t>{shape[keep]})
      fail("the result must go to a GLOBAL buffer with one element per kept row or column");
    if (!typeEqual(gy->element, gx->element)) fail("source and result must have one element type");
    if (out.argDst == out.argSrc) fail("the result must not alias the source");
    const std::vector<int64_t> accAll{T[keep]};
    if (dense(store, "srcExtents") != accAll || dense(store, "dstExtents") != accAll)
      fail("the copy of the result must cover exactly the accumulator");
    if (origin1(store, true, ivs.by) != std::array<int64_t, 2>{0, 0}) fail("the accumulator must be read from its origin");
    if (origin1(store, false, ivs.by) != std::array<int64_t, 2>{T[keep], 0}) fail("the result must land at block index * tile extent");

    // ---- how the accumulator starts
    if (fill) {
      if (fill->operands.at(0) != tm) fail("the fill must set the accumulator");
      const Attribute* v = fill->attr("value");
      if (!v || !std::holds_alternative<FloatAttr>(*v) || std::get<FloatAttr>(*v).value != identityOf(out.kind))
        fail("the accumulator must start at the identity of the reduce kind (0 for add, 1 for mul, +inf for min, -inf for max)");
      out.clear = true;
    } else if (preload) {
      if (preload->operands.at(1) != tm || preload->operands.at(0) != store->operands.at(1))
        fail("the copy before the loop must load the accumulator from the result buffer");
      if (dense(preload, "srcExtents") != accAll || dense(preload, "dstExtents") != accAll)
        fail("the load of the accumulator must cover it exactly");
      if (origin1(preload, false, ivs.by) != std::array<int64_t, 2>{0, 0} ||
          origin1(preload, true, ivs.by) != std::array<int64_t, 2>{T[keep], 0})
        fail("the accumulator must be loaded from block index * tile extent");
      out.clear = false;
    } else if (opClear) {
      out.clear = true;   // a single tile, cleared by the reduce itself
    } else {
      fail("the accumulator is neither filled nor loaded before it is folded into");
    }
    if ((fill || preload) && opClear) fail("the reduce clears the accumulator that was just set");
    out.shape = shape;
    out.dim = dim;
    out.elem = gx->element;
    out.tile = {T[0], T[1]};
    out.grid = grid[0];
    out.ok = true;
  } catch (const Fail& f) {
    out.ok = false;
    out.why = f.why;
  } catch (const std::out_of_range&) {
    out.ok = false;
    out.why = "malformed operation (missing operand or region)";
  }
  return out;
}

}  // namespace fir
