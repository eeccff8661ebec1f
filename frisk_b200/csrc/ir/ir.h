// A small self-contained IR with the surface of the reference's `frisk` dialect and of the MLIR
// objects its Python binding exposes (ffi/ir.cpp), without MLIR: contexts, types, attributes,
// affine expressions and maps, values, blocks, regions and operations, plus a printer that
// reproduces MLIR's textual conventions for the ops the reference's tests emit.
//
// Ownership: a Context owns every object created through it (an arena); handles given to Python
// keep the context alive, so nothing dangles when a module is dropped before its ops.
#pragma once
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <variant>
#include <vector>

namespace fir {

struct Context;
struct Operation;
struct Block;
struct Region;

// ---------------------------------------------------------------------------- affine
enum class AffineKind { Add = 0, Mul, Mod, FloorDiv, CeilDiv, Constant, DimId, SymbolId };

struct AffineExprNode {
  AffineKind kind;
  int64_t value = 0;  // constant value or dim / symbol position
  std::shared_ptr<const AffineExprNode> lhs, rhs;
};
using AffineExpr = std::shared_ptr<const AffineExprNode>;  // null = "no expression"

AffineExpr affineConstant(int64_t v);
AffineExpr affineDim(unsigned pos);
AffineExpr affineSymbol(unsigned pos);
// Builders apply the local simplifications of MLIR's AffineExpr operators (constant folding,
// constants and symbols moved to the right, x*1, x+0, (x+c1)+c2, x*c1*c2, x*c + x*d, ...).
AffineExpr affineBinary(AffineKind kind, AffineExpr lhs, AffineExpr rhs);
bool affineEqual(const AffineExpr& a, const AffineExpr& b);
bool isSymbolicOrConstant(const AffineExpr& e);
bool isPureAffine(const AffineExpr& e);
int64_t largestKnownDivisor(const AffineExpr& e);
bool isFunctionOfDim(const AffineExpr& e, unsigned pos);
bool isFunctionOfSymbol(const AffineExpr& e, unsigned pos);
AffineExpr replaceDimsAndSymbols(const AffineExpr& e, const std::vector<AffineExpr>& dims,
                                 const std::vector<AffineExpr>& syms);
int64_t evaluate(const AffineExpr& e, const std::vector<int64_t>& dims,
                 const std::vector<int64_t>& syms);
std::string printAffineExpr(const AffineExpr& e,
                            const std::function<std::string(bool isSymbol, unsigned pos)>& name = {});

struct AffineMap {
  bool valid = false;  // a default-constructed map is "null" (bool(map) is False)
  unsigned numDims = 0, numSymbols = 0;
  std::vector<AffineExpr> results;
  static AffineMap get(unsigned dims, unsigned syms, std::vector<AffineExpr> results);
  static AffineMap identity(unsigned rank);
  static AffineMap constant(int64_t v);
  static AffineMap minorIdentity(unsigned dims, unsigned results);
  static AffineMap permutation(const std::vector<unsigned>& perm);
  bool isIdentity() const;
  bool isMinorIdentity() const;
  bool isPermutation() const;
  bool isProjectedPermutation(bool allowZero) const;
  bool operator==(const AffineMap& o) const;
  std::string str() const;
};

// ---------------------------------------------------------------------------- types
enum class TypeKind { F16, BF16, F32, F64, F8E4M3FN, F8E5M2, Integer, Index, MemRef, RankedTensor,
                      Function };
struct TypeStorage;
using Type = std::shared_ptr<const TypeStorage>;
struct TypeStorage {
  TypeKind kind;
  unsigned width = 0;               // Integer
  std::vector<int64_t> shape;       // MemRef / RankedTensor
  Type element;                     // MemRef / RankedTensor
  AffineMap layout;                 // MemRef (invalid = identity)
  unsigned memorySpace = 0;         // MemRef: 0 local, 1 global, 3 shared
  std::vector<Type> inputs, outputs;  // Function
};
Type makeScalar(TypeKind k, unsigned width = 0);
Type makeMemRef(std::vector<int64_t> shape, Type elem, AffineMap layout, unsigned space);
Type makeTensor(std::vector<int64_t> shape, Type elem);
Type makeFunction(std::vector<Type> in, std::vector<Type> out);
bool typeEqual(const Type& a, const Type& b);
std::string printType(const Type& t);
bool isFloat(const Type& t);
unsigned bitWidth(const Type& t);

// ---------------------------------------------------------------------------- attributes
enum class MemorySpace : unsigned { Local = 0, Global = 1, Shared = 3 };
enum class GemmWarpPolicy : unsigned { Square = 0, FullRow = 1, FullCol = 2 };

struct EnumAttr { std::string mnemonic, value; };  // prints #frisk<mnemonic value>
struct FloatAttr { double value; Type type; };
struct IntAttr { int64_t value; unsigned width; };  // width 1 = bool
struct DenseI64 { std::vector<int64_t> values; };
struct LayoutAttrData {
  std::vector<int64_t> inputShape;
  AffineMap forwardIndex, forwardThread;  // forwardThread may be invalid
  std::optional<int64_t> replicate;
};
using Attribute = std::variant<std::monostate, IntAttr, FloatAttr, std::string, Type, DenseI64,
                               AffineMap, EnumAttr, LayoutAttrData>;
std::string printAttribute(const Attribute& a);

// ---------------------------------------------------------------------------- IR
struct Location { std::string file; int line = 0, col = 0; };

struct ValueImpl {
  Type type;
  Operation* defOp = nullptr;  // op result
  Block* block = nullptr;      // block argument
  unsigned index = 0;
  std::vector<std::pair<Operation*, unsigned>> uses;
  Context* ctx = nullptr;
};
using Value = ValueImpl*;

struct Operation {
  std::string name;  // e.g. "frisk.gemm"
  std::vector<Value> operands;
  std::vector<Value> results;
  std::map<std::string, Attribute> attrs;  // sorted: MLIR prints attribute dictionaries sorted
  std::vector<Region*> regions;
  std::vector<int> segmentSizes;  // frisk.copy: operand groups
  Block* parent = nullptr;
  Location loc;
  Context* ctx = nullptr;

  void setOperand(unsigned i, Value v);
  void addOperand(Value v);
  const Attribute* attr(const std::string& n) const;
  int64_t intAttr(const std::string& n, int64_t dflt = 0) const;
  bool isTerminator() const { return name == "frisk.end" || name == "func.return"; }
  Operation* parentOp() const;
};

struct Block {
  std::vector<Value> args;
  std::vector<Operation*> ops;
  Region* parent = nullptr;
  Context* ctx = nullptr;
  Value addArgument(Type t);
  void insert(size_t pos, Operation* op);
  void erase(Operation* op);
};

struct Region {
  std::vector<Block*> blocks;
  Operation* parentOp = nullptr;
  Context* ctx = nullptr;
  void push_back(Block* b);
};

struct Context : std::enable_shared_from_this<Context> {
  bool multithreading = true;
  bool friskLoaded = false;
  std::vector<std::unique_ptr<Operation>> ops;
  std::vector<std::unique_ptr<Block>> blocks;
  std::vector<std::unique_ptr<Region>> regions;
  std::vector<std::unique_ptr<ValueImpl>> values;
  Operation* newOp(const std::string& name, const Location& loc);
  Block* newBlock();
  Region* newRegion(Operation* parent);
  Value newValue(Type t);
};

void walk(Operation* op, const std::function<void(Operation*)>& fn);  // post-order
void replaceAllUsesWith(Value from, Value to);

// Printing (MLIR-compatible SSA numbering: %argN for block arguments, %N for results, numbered
// per region scope the way mlir::AsmState does).
std::string printOperation(Operation* op);
std::string printBlock(Block* b);
std::string printValueName(Value v);

// Verification: the checks of the reference's verifiers (FriskOps.cpp) for kernel, gemm,
// alloc_buffer, copy, fill and reduce.  Returns an empty string on success, else the message.
std::string verify(Operation* op);

struct InsertPoint { Block* block = nullptr; size_t index = 0; };

// The reference's OpBuilderWithLoc (include/Dialect/Frisk/Utils/Utils.h:17-92): an insertion point
// plus the last location, stamped on every created op.
struct Builder {
  std::shared_ptr<Context> ctx;
  InsertPoint ip;
  Location lastLoc;
  explicit Builder(std::shared_ptr<Context> c) : ctx(std::move(c)) {}
  Operation* create(const std::string& name);  // inserts at the insertion point when one is set
  void setInsertionPointToStart(Block* b) { ip = {b, 0}; }
  void setInsertionPointToEnd(Block* b);
  void setInsertionPointAfter(Operation* op);
};

// Shared-memory layout the reference's GemmOp::inferLayout picks for an operand tile
// (FriskOps.cpp:500-618): returns the LayoutAttr data with the (tc, ts, index) maps.
std::optional<LayoutAttrData> sharedLayoutForOperand(const std::vector<int64_t>& shape,
                                                     unsigned elemBits, bool kInner, bool hopper);

// Layout inference of frisk.gemm (FriskOps.cpp:1285-1407): a shared-memory layout for an operand
// in shared memory, a register fragment (thread map + register index map + replicate count) for an
// operand in local memory and for the accumulator.  Needs a 'frisk.target' string on an enclosing
// op and a thread count ('frisk.threads' on an enclosing op, or an enclosing frisk.parallel).
// Targets sm_80..89 (mma.sync fragments), sm_90..99 (wgmma accumulator when it applies) and, as
// an addition, sm_100 and later: operands in shared memory, accumulator in tensor memory.
struct GemmLayouts {
  bool ok = false;
  std::string why;           // the refusal, in the reference's words where it has them
  LayoutAttrData a, b, c;
  int64_t warpsM = 1, warpsN = 1;
  std::string instruction;   // "mma", "wgmma" or "tcgen05"
};
GemmLayouts inferGemmLayouts(const Operation* gemm);

// Layout inference of frisk.reduce (FriskOps_Reduce.cpp:214-357): the destination's fragment
// derived from the source's.  ok && !inferred: nothing to infer (an operand outside local memory,
// or a source without a thread map), or `existing` was given and agrees (it is returned).
struct ReduceLayout {
  bool ok = false;
  bool inferred = false;
  std::string why;
  LayoutAttrData layout;
};
ReduceLayout inferReduceLayout(const Operation* reduce, const LayoutAttrData* src,
                               const LayoutAttrData* existing = nullptr);

// Number of distinct values of the thread map that one coordinate selects, the factor by which a
// reduce over that coordinate grows the replicate count (LayoutUtils.cpp:181-218).
std::optional<int64_t> usedExtentOfDim(const AffineMap& map, unsigned dim, int64_t extent);
std::optional<int64_t> threadBlockSize(const Operation* op);
// "Fragment(shape=[..], index=affine_map<..>, thread=affine_map<..>, replicate=N)" or
// "Layout(shape=[..], index=affine_map<..>)" (FriskAttributes.cpp:38-64).
std::string layoutDebugString(const LayoutAttrData& l);

// The tiled matrix product of the reference's sketch (tmp/ir.mlir:1-17: parallel grid, tiles in
// shared / local buffers, a k loop of two copies and a gemm, a copy of the result) recognised and
// lifted to one whole-problem GEMM C = A x B over kernel arguments; `ok` is false, with the
// reason in `why`, for anything else.
struct TiledGemm {
  bool ok = false;
  std::string why;
  int64_t M = 0, N = 0, K = 0;
  int argA = -1, argB = -1, argC = -1;  // kernel argument positions
  bool clearAccum = true;               // false: the C tile is loaded from C before the loop
  Type elemAB, elemC;
  std::vector<int64_t> tile;            // TM, TN, TK of the program (a hint; not used to execute)
  std::vector<int64_t> grid;            // GY, GX
  // A frisk.reduce of the accumulator tile over its columns, written out to a rank-1 kernel
  // argument of M elements (only when the grid has one tile column, so that a tile row holds a
  // whole row of C): the fold the GEMM's epilogue can do.  argR < 0: the program has none.
  int argR = -1;
  std::string reduceKind;
  bool reduceClear = true;
};
TiledGemm liftTiledGemm(Operation* kernel);

// A tiled reduce (tile_program.cpp): a one-dimensional frisk.parallel grid whose body walks the
// reduced dimension of a rank-2 GLOBAL argument tile by tile (copy into a tile buffer,
// frisk.reduce of the tile into a rank-1 accumulator buffer with clear = false) and copies the
// accumulator out, recognised and lifted to one whole-buffer frisk.reduce over kernel arguments.
struct TiledReduce {
  bool ok = false;
  std::string why;
  std::vector<int64_t> shape;  // of the source argument: [R, C]
  int64_t dim = 0;             // the reduced dimension
  std::string kind;
  bool clear = true;           // false: the accumulator is loaded from the destination first
  int argSrc = -1, argDst = -1;
  Type elem;
  std::vector<int64_t> tile;   // the program's tile [TR, TC] (a hint; not used to execute)
  int64_t grid = 0;
};
TiledReduce liftTiledReduce(Operation* kernel);

// Reads a module from its textual form (the custom assembly the printers above and the reference's
// own printers emit).  Returns nullptr and sets *error ("line L, column C: what") on anything it
// cannot read.  The module's objects belong to `ctx`.
Operation* parseModule(const std::string& text, std::shared_ptr<Context> ctx, std::string* error);

}  // namespace fir
