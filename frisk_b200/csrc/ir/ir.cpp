// Types, attributes, the operation / block / region graph, the textual printer and the verifiers.
#include "ir.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <sstream>
#include <unordered_map>

namespace fir {

// ---------------------------------------------------------------------------------- types
Type makeScalar(TypeKind k, unsigned width) {
  auto t = std::make_shared<TypeStorage>();
  t->kind = k;
  t->width = width;
  return t;
}
Type makeMemRef(std::vector<int64_t> shape, Type elem, AffineMap layout, unsigned space) {
  auto t = std::make_shared<TypeStorage>();
  t->kind = TypeKind::MemRef;
  t->shape = std::move(shape);
  t->element = std::move(elem);
  if (layout.valid && !layout.isIdentity()) t->layout = std::move(layout);  // identity is the default
  t->memorySpace = space;
  return t;
}
Type makeTensor(std::vector<int64_t> shape, Type elem) {
  auto t = std::make_shared<TypeStorage>();
  t->kind = TypeKind::RankedTensor;
  t->shape = std::move(shape);
  t->element = std::move(elem);
  return t;
}
Type makeFunction(std::vector<Type> in, std::vector<Type> out) {
  auto t = std::make_shared<TypeStorage>();
  t->kind = TypeKind::Function;
  t->inputs = std::move(in);
  t->outputs = std::move(out);
  return t;
}
bool typeEqual(const Type& a, const Type& b) {
  if (a == b) return true;
  if (!a || !b || a->kind != b->kind) return false;
  switch (a->kind) {
    case TypeKind::Integer: return a->width == b->width;
    case TypeKind::MemRef:
      return a->shape == b->shape && typeEqual(a->element, b->element) &&
             a->memorySpace == b->memorySpace && a->layout == b->layout;
    case TypeKind::RankedTensor: return a->shape == b->shape && typeEqual(a->element, b->element);
    case TypeKind::Function: {
      if (a->inputs.size() != b->inputs.size() || a->outputs.size() != b->outputs.size()) return false;
      for (size_t i = 0; i < a->inputs.size(); ++i)
        if (!typeEqual(a->inputs[i], b->inputs[i])) return false;
      for (size_t i = 0; i < a->outputs.size(); ++i)
        if (!typeEqual(a->outputs[i], b->outputs[i])) return false;
      return true;
    }
    default: return true;
  }
}
bool isFloat(const Type& t) { return t && t->kind <= TypeKind::F8E5M2; }
unsigned bitWidth(const Type& t) {
  switch (t->kind) {
    case TypeKind::F16:
    case TypeKind::BF16: return 16;
    case TypeKind::F32: return 32;
    case TypeKind::F64: return 64;
    case TypeKind::F8E4M3FN:
    case TypeKind::F8E5M2: return 8;
    case TypeKind::Integer: return t->width;
    case TypeKind::Index: return 64;
    default: return 0;
  }
}
static void printShape(std::ostream& os, const std::vector<int64_t>& shape) {
  for (int64_t d : shape) {
    if (d < 0) os << '?';
    else os << d;
    os << 'x';
  }
}
std::string printType(const Type& t) {
  if (!t) return "<<NULL TYPE>>";
  std::ostringstream os;
  switch (t->kind) {
    case TypeKind::F16: return "f16";
    case TypeKind::BF16: return "bf16";
    case TypeKind::F32: return "f32";
    case TypeKind::F64: return "f64";
    case TypeKind::F8E4M3FN: return "f8E4M3FN";
    case TypeKind::F8E5M2: return "f8E5M2";
    case TypeKind::Integer: return "i" + std::to_string(t->width);
    case TypeKind::Index: return "index";
    case TypeKind::MemRef:
      os << "memref<";
      printShape(os, t->shape);
      os << printType(t->element);
      if (t->layout.valid) os << ", affine_map<" << t->layout.str() << ">";
      if (t->memorySpace != 0) os << ", " << t->memorySpace;
      os << ">";
      return os.str();
    case TypeKind::RankedTensor:
      os << "tensor<";
      printShape(os, t->shape);
      os << printType(t->element) << ">";
      return os.str();
    case TypeKind::Function: {
      os << "(";
      for (size_t i = 0; i < t->inputs.size(); ++i) os << (i ? ", " : "") << printType(t->inputs[i]);
      os << ") -> ";
      if (t->outputs.size() == 1 && t->outputs[0]->kind != TypeKind::Function) {
        os << printType(t->outputs[0]);
      } else {
        os << "(";
        for (size_t i = 0; i < t->outputs.size(); ++i)
          os << (i ? ", " : "") << printType(t->outputs[i]);
        os << ")";
      }
      return os.str();
    }
  }
  return "";
}

// ---------------------------------------------------------------------------------- attributes
static std::string printFloat(double v) {
  // MLIR prints floats in scientific notation with six digits when that round-trips
  char buf[64];
  snprintf(buf, sizeof buf, "%.6e", v);
  if (std::strtod(buf, nullptr) == v) return buf;
  snprintf(buf, sizeof buf, "%.17g", v);
  return buf;
}
static void printI64List(std::ostream& os, const std::vector<int64_t>& v) {
  for (size_t i = 0; i < v.size(); ++i) os << (i ? ", " : "") << v[i];
}
std::string printAttribute(const Attribute& a) {
  std::ostringstream os;
  if (auto* i = std::get_if<IntAttr>(&a)) {
    if (i->width == 1) return i->value ? "true" : "false";
    os << i->value << " : i" << i->width;
  } else if (auto* f = std::get_if<FloatAttr>(&a)) {
    if (std::isfinite(f->value)) {
      os << printFloat(f->value);
    } else {
      // MLIR prints infinities and NaNs as the bit pattern of the attribute's type
      const bool neg = std::signbit(f->value), nan = std::isnan(f->value);
      char buf[32];
      switch (f->type ? f->type->kind : TypeKind::F64) {
        case TypeKind::F16: snprintf(buf, sizeof buf, "0x%04X", (nan ? 0x7E00u : 0x7C00u) | (neg ? 0x8000u : 0u)); break;
        case TypeKind::BF16: snprintf(buf, sizeof buf, "0x%04X", (nan ? 0x7FC0u : 0x7F80u) | (neg ? 0x8000u : 0u)); break;
        case TypeKind::F32: snprintf(buf, sizeof buf, "0x%08X", (nan ? 0x7FC00000u : 0x7F800000u) | (neg ? 0x80000000u : 0u)); break;
        default:
          snprintf(buf, sizeof buf, "0x%016llX",
                   (unsigned long long)((nan ? 0x7FF8000000000000ull : 0x7FF0000000000000ull) | (neg ? 0x8000000000000000ull : 0ull)));
      }
      os << buf;
    }
    os << " : " << printType(f->type);
  } else if (auto* s = std::get_if<std::string>(&a)) {
    os << '"' << *s << '"';
  } else if (auto* t = std::get_if<Type>(&a)) {
    os << printType(*t);
  } else if (auto* d = std::get_if<DenseI64>(&a)) {
    os << "array<i64";
    if (!d->values.empty()) {
      os << ": ";
      printI64List(os, d->values);
    }
    os << ">";
  } else if (auto* m = std::get_if<AffineMap>(&a)) {
    os << "affine_map<" << m->str() << ">";
  } else if (auto* e = std::get_if<EnumAttr>(&a)) {
    os << "#frisk<" << e->mnemonic << " " << e->value << ">";
  } else if (auto* l = std::get_if<LayoutAttrData>(&a)) {
    os << "#frisk.layout<[";
    printI64List(os, l->inputShape);
    os << "], affine_map<" << l->forwardIndex.str() << ">";
    if (l->forwardThread.valid) os << ", affine_map<" << l->forwardThread.str() << ">";
    if (l->replicate) os << ", " << *l->replicate;
    os << ">";
  } else {
    os << "unit";
  }
  return os.str();
}

// ---------------------------------------------------------------------------------- IR graph
Operation* Context::newOp(const std::string& name, const Location& loc) {
  ops.push_back(std::make_unique<Operation>());
  Operation* op = ops.back().get();
  op->name = name;
  op->loc = loc;
  op->ctx = this;
  return op;
}
Block* Context::newBlock() {
  blocks.push_back(std::make_unique<Block>());
  blocks.back()->ctx = this;
  return blocks.back().get();
}
Region* Context::newRegion(Operation* parent) {
  regions.push_back(std::make_unique<Region>());
  Region* r = regions.back().get();
  r->parentOp = parent;
  r->ctx = this;
  if (parent) parent->regions.push_back(r);
  return r;
}
Value Context::newValue(Type t) {
  values.push_back(std::make_unique<ValueImpl>());
  Value v = values.back().get();
  v->type = std::move(t);
  v->ctx = this;
  return v;
}

void Operation::addOperand(Value v) {
  operands.push_back(v);
  if (v) v->uses.emplace_back(this, (unsigned)operands.size() - 1);
}
void Operation::setOperand(unsigned i, Value v) {
  Value old = operands.at(i);
  if (old) {
    auto& u = old->uses;
    u.erase(std::remove(u.begin(), u.end(), std::make_pair(this, i)), u.end());
  }
  operands[i] = v;
  if (v) v->uses.emplace_back(this, i);
}
const Attribute* Operation::attr(const std::string& n) const {
  auto it = attrs.find(n);
  return it == attrs.end() ? nullptr : &it->second;
}
int64_t Operation::intAttr(const std::string& n, int64_t dflt) const {
  if (auto* a = attr(n))
    if (auto* i = std::get_if<IntAttr>(a)) return i->value;
  return dflt;
}
Operation* Operation::parentOp() const {
  return parent && parent->parent ? parent->parent->parentOp : nullptr;
}

Value Block::addArgument(Type t) {
  Value v = ctx->newValue(std::move(t));
  v->block = this;
  v->index = (unsigned)args.size();
  args.push_back(v);
  return v;
}
void Block::insert(size_t pos, Operation* op) {
  pos = std::min(pos, ops.size());
  ops.insert(ops.begin() + (long)pos, op);
  op->parent = this;
}
void Block::erase(Operation* op) {
  ops.erase(std::remove(ops.begin(), ops.end(), op), ops.end());
  op->parent = nullptr;
}
void Region::push_back(Block* b) {
  blocks.push_back(b);
  b->parent = this;
}

void walk(Operation* op, const std::function<void(Operation*)>& fn) {
  for (Region* r : op->regions)
    for (Block* b : r->blocks) {
      std::vector<Operation*> copy = b->ops;  // the callback may erase ops
      for (Operation* o : copy) walk(o, fn);
    }
  fn(op);
}

void replaceAllUsesWith(Value from, Value to) {
  auto uses = from->uses;
  for (auto& [op, idx] : uses) op->setOperand(idx, to);
}

Operation* Builder::create(const std::string& name) {
  Operation* op = ctx->newOp(name, lastLoc);
  if (ip.block) {
    ip.block->insert(ip.index, op);
    ++ip.index;
  }
  return op;
}
void Builder::setInsertionPointToEnd(Block* b) { ip = {b, b->ops.size()}; }
void Builder::setInsertionPointAfter(Operation* op) {
  Block* b = op->parent;
  if (!b) return;
  auto it = std::find(b->ops.begin(), b->ops.end(), op);
  ip = {b, (size_t)(it - b->ops.begin()) + 1};
}

// ---------------------------------------------------------------------------------- printer
namespace {

struct Names {
  std::unordered_map<const ValueImpl*, std::string> name;
};

// mlir::AsmState numbering: a region is numbered with the counters as they stood after its
// parent REGION was numbered completely, so sibling regions reuse numbers.
void numberRegion(Region* r, unsigned nextValue, unsigned nextArg, Names& n) {
  unsigned cst = 0;
  for (Block* b : r->blocks) {
    for (Value a : b->args) n.name[a] = "%arg" + std::to_string(nextArg++);
    for (Operation* op : b->ops) {
      for (Value res : op->results) {
        if (op->name == "arith.constant") {
          // constants get descriptive names, as MLIR's OpAsmOpInterface gives them
          std::string base;
          const Attribute* v = op->attr("value");
          if (v && std::holds_alternative<IntAttr>(*v)) {
            const IntAttr& i = std::get<IntAttr>(*v);
            base = "%c" + std::string(i.value < 0 ? "-" : "") + std::to_string(std::llabs(i.value)) +
                   "_i" + std::to_string(i.width);
          } else {
            base = cst == 0 ? "%cst" : "%cst_" + std::to_string(cst - 1);
            ++cst;
          }
          n.name[res] = base;
        } else {
          n.name[res] = "%" + std::to_string(nextValue++);
        }
      }
    }
  }
  for (Block* b : r->blocks)
    for (Operation* op : b->ops)
      for (Region* sub : op->regions) numberRegion(sub, nextValue, nextArg, n);
}

Operation* topLevel(Operation* op) {
  while (Operation* p = op->parentOp()) op = p;
  return op;
}

void numberFrom(Operation* top, Names& n) {
  unsigned v = 0;
  for (Value res : top->results) n.name[res] = "%" + std::to_string(v++);
  for (Region* r : top->regions) numberRegion(r, v, 0, n);
}

std::string nameOf(const Names& n, Value v) {
  auto it = n.name.find(v);
  return it == n.name.end() ? "<<UNKNOWN SSA VALUE>>" : it->second;
}

void printAttrDict(std::ostream& os, const Operation* op, const std::vector<std::string>& elide,
                   bool leadingSpace = true) {
  bool any = false;
  for (auto& [k, v] : op->attrs) {
    if (std::find(elide.begin(), elide.end(), k) != elide.end()) continue;
    os << (any ? ", " : (leadingSpace ? " {" : "{")) << k;
    if (!std::holds_alternative<std::monostate>(v)) os << " = " << printAttribute(v);
    any = true;
  }
  if (any) os << "}";
}

void printOp(std::ostream& os, Operation* op, int indent, const Names& n);

void printRegion(std::ostream& os, Region* r, int indent, const Names& n, bool printTerminators) {
  os << "{\n";
  for (Block* b : r->blocks)
    for (Operation* op : b->ops) {
      if (op->isTerminator() && !printTerminators && op->name == "frisk.end") continue;
      os << std::string((size_t)indent + 2, ' ');
      printOp(os, op, indent + 2, n);
      os << "\n";
    }
  os << std::string((size_t)indent, ' ') << "}";
}

void printIndexList(std::ostream& os, const Operation* op, const char* mapName, size_t first,
                    size_t count, const Names& n) {
  const Attribute* a = op->attr(mapName);
  const AffineMap* m = a ? std::get_if<AffineMap>(a) : nullptr;
  if (!m || !m->valid) return;
  // mlir::OpAsmPrinter::printAffineMapOfSSAIds: every result with dims / symbols replaced by names
  for (size_t i = 0; i < m->results.size(); ++i) {
    os << (i ? ", " : "");
    os << printAffineExpr(m->results[i], [&](bool isSym, unsigned pos) {
      size_t idx = first + (isSym ? m->numDims + pos : pos);
      std::string nm = idx < first + count ? nameOf(n, op->operands[idx]) : "<<?>>";
      return isSym ? "symbol(" + nm + ")" : nm;
    });
  }
}

void printOp(std::ostream& os, Operation* op, int indent, const Names& n) {
  if (!op->results.empty()) {
    for (size_t i = 0; i < op->results.size(); ++i) os << (i ? ", " : "") << nameOf(n, op->results[i]);
    os << " = ";
  }
  const std::string& nm = op->name;
  if (nm == "builtin.module") {
    os << "module";
    bool any = !op->attrs.empty();
    if (any) {
      os << " attributes";
      printAttrDict(os, op, {});
    }
    os << " ";
    printRegion(os, op->regions[0], indent, n, false);
  } else if (nm == "frisk.kernel") {
    const Type& ft = std::get<Type>(*op->attr("function_type"));
    os << nm << " @" << std::get<std::string>(*op->attr("sym_name")) << "(";
    for (size_t i = 0; i < ft->inputs.size(); ++i) os << (i ? ", " : "") << printType(ft->inputs[i]);
    os << ")";
    if (!ft->outputs.empty()) {
      os << " -> (";
      for (size_t i = 0; i < ft->outputs.size(); ++i) os << (i ? ", " : "") << printType(ft->outputs[i]);
      os << ")";
    }
    os << " ";
    printRegion(os, op->regions[0], indent, n, false);
    printAttrDict(os, op, {"sym_name", "function_type"});
  } else if (nm == "frisk.parallel" || nm == "frisk.block") {
    os << nm << " (";
    Block* body = op->regions[0]->blocks.empty() ? nullptr : op->regions[0]->blocks[0];
    if (body)
      for (size_t i = 0; i < body->args.size(); ++i) os << (i ? ", " : "") << nameOf(n, body->args[i]);
    const DenseI64& ranges = std::get<DenseI64>(*op->attr("ranges"));
    os << (nm == "frisk.parallel" ? ") = (" : ") to (");
    printI64List(os, ranges.values);
    os << ")";
    if (nm == "frisk.parallel") os << ", threads = " << op->intAttr("threads");
    os << " ";
    printRegion(os, op->regions[0], indent, n, false);
  } else if (nm == "frisk.for") {
    Block* body = op->regions[0]->blocks[0];
    os << nm << " " << nameOf(n, body->args[0]) << " = " << op->intAttr("lower") << " to "
       << op->intAttr("upper");
    if (op->intAttr("step") > 1) os << " step = " << op->intAttr("step");
    os << " ";
    printRegion(os, op->regions[0], indent, n, false);
  } else if (nm == "frisk.alloc_buffer") {
    static const char* scope[] = {"local", "global", "unknown", "shared"};
    const unsigned ms = (unsigned)op->intAttr("memorySpace");
    os << nm << " {scope = \"" << (ms < 4 ? scope[ms] : "unknown") << "\"";
    if (op->intAttr("alignment") != 0) os << ", alignment = " << op->intAttr("alignment");
    os << "} -> " << printType(op->results[0]->type);
  } else if (nm == "frisk.copy") {
    const size_t nSrc = (size_t)op->segmentSizes.at(2), nDst = (size_t)op->segmentSizes.at(3);
    os << nm << " " << nameOf(n, op->operands[0]) << "[";
    printIndexList(os, op, "srcMap", 2, nSrc, n);
    os << "], " << nameOf(n, op->operands[1]) << "[";
    printIndexList(os, op, "dstMap", 2 + nSrc, nDst, n);
    os << "] {src_extents = [";
    printI64List(os, std::get<DenseI64>(*op->attr("srcExtents")).values);
    os << "], dst_extents = [";
    printI64List(os, std::get<DenseI64>(*op->attr("dstExtents")).values);
    os << "]} ";
    printAttrDict(os, op, {"srcMap", "dstMap", "srcExtents", "dstExtents"}, /*leadingSpace=*/false);
    os << " : " << printType(op->operands[0]->type) << ", " << printType(op->operands[1]->type);
  } else if (nm == "frisk.gemm") {
    // three operands as in the reference; five when the (additional) scale vectors are present
    os << nm << "(";
    for (size_t i = 0; i < op->operands.size(); ++i) os << (i ? ", " : "") << nameOf(n, op->operands[i]);
    os << ")";
    printAttrDict(os, op, {});
    os << " : ";
    for (size_t i = 0; i < op->operands.size(); ++i)
      os << (i ? ", " : "") << printType(op->operands[i]->type);
  } else if (nm == "frisk.fill" || nm == "frisk.reduce") {
    os << nm << " ";
    for (size_t i = 0; i < op->operands.size(); ++i) os << (i ? ", " : "") << nameOf(n, op->operands[i]);
    printAttrDict(os, op, {});
    os << " : ";
    for (size_t i = 0; i < op->operands.size(); ++i)
      os << (i ? ", " : "") << printType(op->operands[i]->type);
  } else if (nm == "frisk.end") {
    os << nm;
    printAttrDict(os, op, {});
  } else if (nm == "arith.constant") {
    os << nm << " ";
    const Attribute* v = op->attr("value");
    if (v && std::holds_alternative<IntAttr>(*v)) {
      const IntAttr& i = std::get<IntAttr>(*v);
      os << i.value << " : i" << i.width;
    } else if (v && std::holds_alternative<FloatAttr>(*v)) {
      os << printAttribute(*v);
    } else if (v && std::holds_alternative<std::string>(*v)) {
      os << std::get<std::string>(*v) << " : " << printType(op->results[0]->type);  // dense<...>
    }
  } else if (nm == "func.func") {
    const Type& ft = std::get<Type>(*op->attr("function_type"));
    os << nm << " @" << std::get<std::string>(*op->attr("sym_name")) << "(";
    Block* body = op->regions[0]->blocks.empty() ? nullptr : op->regions[0]->blocks[0];
    for (size_t i = 0; i < ft->inputs.size(); ++i) {
      os << (i ? ", " : "");
      if (body) os << nameOf(n, body->args[i]) << ": ";
      os << printType(ft->inputs[i]);
    }
    os << ")";
    if (!ft->outputs.empty()) {
      os << " -> ";
      if (ft->outputs.size() == 1) os << printType(ft->outputs[0]);
      else {
        os << "(";
        for (size_t i = 0; i < ft->outputs.size(); ++i) os << (i ? ", " : "") << printType(ft->outputs[i]);
        os << ")";
      }
    }
    if (body) {
      os << " ";
      printRegion(os, op->regions[0], indent, n, true);
    }
  } else if (nm == "func.return") {
    os << "return";
    for (size_t i = 0; i < op->operands.size(); ++i) os << (i ? ", " : " ") << nameOf(n, op->operands[i]);
    if (!op->operands.empty()) {
      os << " : ";
      for (size_t i = 0; i < op->operands.size(); ++i)
        os << (i ? ", " : "") << printType(op->operands[i]->type);
    }
  } else {
    // generic form
    os << '"' << nm << "\"(";
    for (size_t i = 0; i < op->operands.size(); ++i) os << (i ? ", " : "") << nameOf(n, op->operands[i]);
    os << ")";
    printAttrDict(os, op, {});
    os << " : (";
    for (size_t i = 0; i < op->operands.size(); ++i)
      os << (i ? ", " : "") << printType(op->operands[i]->type);
    os << ") -> (";
    for (size_t i = 0; i < op->results.size(); ++i)
      os << (i ? ", " : "") << printType(op->results[i]->type);
    os << ")";
  }
}

}  // namespace

std::string printOperation(Operation* op) {
  Names n;
  numberFrom(topLevel(op), n);
  std::ostringstream os;
  printOp(os, op, 0, n);
  return os.str();
}

std::string printBlock(Block* b) {
  Names n;
  if (b->parent && b->parent->parentOp) numberFrom(topLevel(b->parent->parentOp), n);
  else {
    unsigned a = 0, v = 0;
    for (Value x : b->args) n.name[x] = "%arg" + std::to_string(a++);
    for (Operation* op : b->ops)
      for (Value r : op->results) n.name[r] = "%" + std::to_string(v++);
  }
  std::ostringstream os;
  if (!b->args.empty()) {
    os << "^bb0(";
    for (size_t i = 0; i < b->args.size(); ++i)
      os << (i ? ", " : "") << nameOf(n, b->args[i]) << ": " << printType(b->args[i]->type);
    os << "):\n";
  }
  for (Operation* op : b->ops) {
    os << "  ";
    printOp(os, op, 2, n);
    os << "\n";
  }
  return os.str();
}

std::string printValueName(Value v) {
  Names n;
  Operation* top = nullptr;
  if (v->defOp) top = topLevel(v->defOp);
  else if (v->block && v->block->parent && v->block->parent->parentOp)
    top = topLevel(v->block->parent->parentOp);
  if (top) numberFrom(top, n);
  auto it = n.name.find(v);
  if (it != n.name.end()) return it->second;
  return v->block ? "<block argument>" : "%0";
}

// ---------------------------------------------------------------------------------- verifier
static std::string verifyOne(Operation* op) {
  auto memref = [](Value v) -> const TypeStorage* {
    return v && v->type && v->type->kind == TypeKind::MemRef ? v->type.get() : nullptr;
  };
  const std::string& nm = op->name;
  if (nm == "frisk.kernel") {  // FriskOps.cpp:901-920
    const Attribute* a = op->attr("function_type");
    if (!a || !std::holds_alternative<Type>(*a)) return "requires a 'function_type' attribute";
    const Type& ft = std::get<Type>(*a);
    if (ft->kind != TypeKind::Function) return "requires a function type";
    if (op->regions.empty() || op->regions[0]->blocks.empty()) return "";
    Block* b = op->regions[0]->blocks[0];
    if (b->args.size() != ft->inputs.size()) return "region argument count does not match function type";
    for (size_t i = 0; i < b->args.size(); ++i)
      if (!typeEqual(b->args[i]->type, ft->inputs[i])) return "region argument type mismatch";
  } else if (nm == "frisk.gemm") {  // FriskOps.cpp:1264-1283
    auto *A = memref(op->operands[0]), *B = memref(op->operands[1]), *C = memref(op->operands[2]);
    if (!A || !B || !C) return "operands must be memrefs";
    const bool sameAB = typeEqual(A->element, B->element);
    const bool fp8 = A->element->kind == TypeKind::F8E4M3FN || A->element->kind == TypeKind::F8E5M2;
    // extension: 8-bit float inputs may produce a wider C (the reference has no fp8 GEMM)
    if (!sameAB || (!typeEqual(A->element, C->element) && !fp8))
      return "all operands must have the same element type";
    if (A->shape[1] != B->shape[0]) return "A columns must equal B rows for matrix multiplication";
    if (A->shape[0] != C->shape[0] || B->shape[1] != C->shape[1])
      return "C dimensions must match matrix multiplication result";
  } else if (nm == "frisk.alloc_buffer") {  // FriskOps.cpp:1436-1481
    auto* R = memref(op->results.empty() ? nullptr : op->results[0]);
    if (!R) return "result must be a memref type";
    if (R->shape != std::get<DenseI64>(*op->attr("shape")).values)
      return "shape attribute must match result memref shape";
    if (!typeEqual(R->element, std::get<Type>(*op->attr("elementType"))))
      return "elementType attribute must match result memref element type";
    if ((int64_t)R->memorySpace != op->intAttr("memorySpace"))
      return "memorySpace attribute must match result memref memory space";
    const int64_t al = op->intAttr("alignment");
    if (al < 0) return "alignment must be non-negative";
    if (al > 0 && (al & (al - 1)) != 0) return "alignment must be a power of 2";
  } else if (nm == "frisk.copy") {  // FriskOps.cpp:1664-1683
    const AffineMap& sm = std::get<AffineMap>(*op->attr("srcMap"));
    const AffineMap& dm = std::get<AffineMap>(*op->attr("dstMap"));
    if ((size_t)op->segmentSizes[2] != sm.numDims + sm.numSymbols)
      return "expected " + std::to_string(sm.numDims + sm.numSymbols) + " source indices, but got " +
             std::to_string(op->segmentSizes[2]);
    if ((size_t)op->segmentSizes[3] != dm.numDims + dm.numSymbols)
      return "expected " + std::to_string(dm.numDims + dm.numSymbols) +
             " destination indices, but got " + std::to_string(op->segmentSizes[3]);
  } else if (nm == "frisk.fill") {  // FriskOps.cpp:1688-1701
    auto* M = memref(op->operands[0]);
    const Attribute* v = op->attr("value");
    if (!M) return "operand must be a memref";
    if (!v || !std::holds_alternative<FloatAttr>(*v)) return "fill value must be a float attribute";
    if (!typeEqual(std::get<FloatAttr>(*v).type, M->element))
      return "value type " + printType(std::get<FloatAttr>(*v).type) +
             " does not match memref element type " + printType(M->element);
  } else if (nm == "frisk.reduce") {  // FriskOps.cpp:1734-1767
    auto *S = memref(op->operands[0]), *D = memref(op->operands[1]);
    if (!S || !D) return "source and destination must be memref types";
    const int64_t dim = op->intAttr("dim");
    const int64_t rank = (int64_t)S->shape.size();
    if (dim < 0 || dim >= rank) return "dimension " + std::to_string(dim) + " is out of range for source of rank " + std::to_string(rank);
    const std::string& kind = std::get<std::string>(*op->attr("kind"));
    if (kind != "add" && kind != "mul" && kind != "min" && kind != "max")
      return "unsupported reduce kind: " + kind + ". Supported: add, mul, min, max";
    if (S->shape.size() != D->shape.size() + 1) return "destination rank must be one less than source rank";
    for (int64_t i = 0, j = 0; i < rank; ++i) {
      if (i == dim) continue;
      if (S->shape[i] != D->shape[j]) return "non-reduced dimension mismatch";
      ++j;
    }
    if (!typeEqual(S->element, D->element)) return "source and destination must have the same element type";
  }
  return "";
}

std::string verify(Operation* op) {
  std::string err;
  walk(op, [&](Operation* o) {
    if (!err.empty()) return;
    std::string e = verifyOne(o);
    if (!e.empty()) err = "'" + o->name + "' op " + e;
  });
  return err;
}

// ---------------------------------------------------------------------------------- layouts
// The swizzled shared-memory layouts of FriskOps.cpp:500-558 as (tc, ts, index) maps of (i, j).
static LayoutAttrData swizzleLayout(int64_t rows, int64_t cols, unsigned elemBits, int chunks) {
  // chunks = 16-byte chunks per row of one atom: 8 (full bank), 4 (half), 2 (quarter)
  const int64_t vec = 128 / elemBits;
  AffineExpr i = affineDim(0), j = affineDim(1);
  auto C = [](int64_t v) { return affineConstant(v); };
  auto fd = [&](AffineExpr a, int64_t c) { return affineBinary(AffineKind::FloorDiv, a, C(c)); };
  auto md = [&](AffineExpr a, int64_t c) { return affineBinary(AffineKind::Mod, a, C(c)); };
  auto add = [&](AffineExpr a, AffineExpr b) { return affineBinary(AffineKind::Add, a, b); };
  auto mul = [&](AffineExpr a, int64_t c) { return affineBinary(AffineKind::Mul, a, C(c)); };
  // XOR of two small non-negative operands written in affine form, bit by bit:
  // a ^ b = sum_k 2^k * ((a_k + b_k) mod 2)
  auto xorBits = [&](AffineExpr a, AffineExpr b, int bits) {
    AffineExpr r = C(0);
    for (int k = 0; k < bits; ++k) {
      AffineExpr ak = md(fd(a, 1ll << k), 2), bk = md(fd(b, 1ll << k), 2);
      r = add(r, mul(md(add(ak, bk), 2), 1ll << k));
    }
    return r;
  };
  AffineExpr ts = fd(i, 8), s = md(i, 8);
  AffineExpr block = fd(j, vec);
  AffineExpr tc = fd(block, chunks), c = md(block, chunks);
  AffineExpr v = md(j, vec);
  AffineExpr sw = chunks == 8 ? xorBits(c, s, 3) : chunks == 4 ? xorBits(c, fd(s, 2), 2)
                                                               : xorBits(c, fd(s, 4), 1);
  AffineExpr index = add(v, mul(add(sw, mul(s, chunks)), vec));
  LayoutAttrData l;
  l.inputShape = {rows, cols};
  l.forwardIndex = AffineMap::get(2, 0, {tc, ts, index});
  return l;
}

std::optional<LayoutAttrData> sharedLayoutForOperand(const std::vector<int64_t>& shape,
                                                     unsigned elemBits, bool kInner, bool hopper) {
  if (shape.size() < 2 || elemBits == 0 || elemBits == 64) return std::nullopt;
  const int64_t rows = shape[shape.size() - 2], cont = shape.back();
  const int64_t vec = 128 / elemBits;
  auto linear = [&](int64_t stride) {
    LayoutAttrData l;
    l.inputShape = {rows, cont};
    l.forwardIndex = AffineMap::get(
        2, 0, {affineBinary(AffineKind::Add,
                            affineBinary(AffineKind::Mul, affineDim(0), affineConstant(stride)),
                            affineDim(1))});
    return l;
  };
  auto padded = [&]() {
    int64_t p = cont;
    if ((elemBits * cont) % 256 == 0) p += 128 / elemBits;
    return linear(p);
  };
  if (!hopper) {  // buildAmpereSharedLayout, FriskOps.cpp:560-587
    if (!kInner && elemBits == 8) return padded();
    if (cont % (vec * 8) == 0) return swizzleLayout(rows, cont, elemBits, 8);
    if (cont % (vec * 4) == 0) return swizzleLayout(rows, cont, elemBits, 4);
    return padded();
  }
  // buildHopperSharedLayout, FriskOps.cpp:589-618 (also what an sm_100 target string selects)
  if (cont % (vec * 8) == 0) return swizzleLayout(rows, cont, elemBits, 8);
  if (cont % (vec * 4) == 0) return swizzleLayout(rows, cont, elemBits, 4);
  if (cont % (vec * 2) == 0) return swizzleLayout(rows, cont, elemBits, 2);
  if (cont % vec == 0) return linear(cont);
  return std::nullopt;
}

}  // namespace fir
