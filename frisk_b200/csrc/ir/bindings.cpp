// pybind11 module `frisk_ffi` with submodule `ir` (and `ir.frisk`): the Python surface of the
// reference's binding (ffi/ffi.cpp:3-7, ffi/ir.cpp:33-1087) on top of the MLIR-free IR of ir.h.
// Names, argument orders, defaults and error types follow the reference; additions are marked.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <iostream>
#include <stdexcept>

#include "ir.h"

namespace py = pybind11;
using namespace fir;
using ret = py::return_value_policy;

namespace {

using CtxPtr = std::shared_ptr<Context>;

struct PyType { Type t; };
struct PyMemRef : PyType {};
struct PyTensor : PyType {};
struct PyFunctionType : PyType {};
struct PyValue { Value v = nullptr; CtxPtr keep; };
struct PyOpResult : PyValue {};
struct PyBlockArg : PyValue {};
struct PyBlock { Block* b = nullptr; CtxPtr keep; };
struct PyRegion { Region* r = nullptr; CtxPtr keep; };
struct PyOperation { Operation* op = nullptr; CtxPtr keep; };  // the reference's `operation`
struct PyOpState { Operation* op = nullptr; CtxPtr keep; };    // the reference's `OpState`
struct PyModule : PyOpState {};
struct PyGemm : PyOpState {};
struct PyKernel : PyOpState {};
struct PyParallel : PyOpState {};
struct PyBlockOp : PyOpState {};
struct PyFor : PyOpState {};
struct PyAlloc : PyOpState {};
struct PyCopy : PyOpState {};
struct PyFill : PyOpState {};
struct PyReduce : PyOpState {};
struct PyConstant : PyOpState {};
struct PyFunction : PyOpState {};
struct PyAttribute { Attribute a; };
struct PyValueRange { std::vector<PyValue> vals; };
struct PyLocation { Location loc; };
struct PyAffineExpr { AffineExpr e; };
struct PyBinaryExpr : PyAffineExpr {};
struct PyDimExpr : PyAffineExpr {};
struct PySymbolExpr : PyAffineExpr {};
struct PyConstExpr : PyAffineExpr {};
struct PyBuilder { Builder b; explicit PyBuilder(CtxPtr c) : b(std::move(c)) {} };

CtxPtr keepOf(Context* c) { return c->shared_from_this(); }

py::object castType(const Type& t) {
  if (!t) return py::none();
  switch (t->kind) {
    case TypeKind::MemRef: { PyMemRef m; m.t = t; return py::cast(m); }
    case TypeKind::RankedTensor: { PyTensor m; m.t = t; return py::cast(m); }
    case TypeKind::Function: { PyFunctionType m; m.t = t; return py::cast(m); }
    default: { PyType m; m.t = t; return py::cast(m); }
  }
}

py::object castValue(Value v) {
  if (!v) return py::none();
  if (v->defOp) { PyOpResult r; r.v = v; r.keep = keepOf(v->ctx); return py::cast(r); }
  PyBlockArg a; a.v = v; a.keep = keepOf(v->ctx); return py::cast(a);
}

template <class T>
T wrapOp(Operation* op) {
  T t;
  t.op = op;
  t.keep = keepOf(op->ctx);
  return t;
}
PyBlock wrapBlock(Block* b) { return PyBlock{b, keepOf(b->ctx)}; }

py::object castExpr(const AffineExpr& e) {
  if (!e) return py::cast(PyAffineExpr{});
  return py::cast(PyAffineExpr{e});
}

Type dtypeFromString(const std::string& dtype, bool allowBf16) {
  if (dtype == "e4m3fn") return makeScalar(TypeKind::F8E4M3FN);
  if (dtype == "e5m2") return makeScalar(TypeKind::F8E5M2);
  if (dtype == "fp16") return makeScalar(TypeKind::F16);
  if (dtype == "fp32") return makeScalar(TypeKind::F32);
  if (dtype == "fp64") return makeScalar(TypeKind::F64);
  if (allowBf16 && dtype == "bf16") return makeScalar(TypeKind::BF16);  // addition: the reference lacks bf16 here
  throw std::invalid_argument("invalid float type");
}

Operation* lookupSymbol(Operation* module, const std::string& name, const std::string& opName) {
  for (Block* b : module->regions[0]->blocks)
    for (Operation* op : b->ops) {
      const Attribute* s = op->attr("sym_name");
      if (s && std::get<std::string>(*s) == name && (opName.empty() || op->name == opName)) return op;
    }
  return nullptr;
}

// Entry block of frisk.kernel / frisk.parallel / func.func (FriskOps.td:56-73, 119-132).
Block* addEntryBlock(Operation* op, const std::vector<Type>& argTypes, bool withEnd) {
  Region* r = op->regions[0];
  if (!r->blocks.empty()) throw std::runtime_error("entry block already exists");
  Block* b = op->ctx->newBlock();
  r->push_back(b);
  for (auto& t : argTypes) b->addArgument(t);
  if (withEnd) {
    Operation* end = op->ctx->newOp("frisk.end", op->loc);
    b->insert(0, end);
  }
  return b;
}

// Regions built by a body callback (frisk.for / frisk.block): FriskOps.cpp:1097-1116, 1198-1218.
template <class Fn>
void buildBody(PyBuilder& self, Operation* op, size_t numIvs, Fn&& callBody) {
  Context* ctx = op->ctx;
  Region* r = ctx->newRegion(op);
  Block* body = ctx->newBlock();
  r->push_back(body);
  for (size_t i = 0; i < numIvs; ++i) body->addArgument(makeScalar(TypeKind::Index));
  const InsertPoint saved = self.b.ip;  // InsertionGuard
  self.b.setInsertionPointToStart(body);
  try {
    callBody(body);
  } catch (...) {
    self.b.ip = saved;
    throw;
  }
  self.b.setInsertionPointToEnd(body);
  self.b.create("frisk.end");
  self.b.ip = saved;
}

const TypeStorage* requireMemRef(Value v, const char* what) {
  if (v && v->type && v->type->kind == TypeKind::MemRef) return v->type.get();
  throw std::invalid_argument(std::string("create_gemm_op expects memref for operand ") + what);
}

void initCommon(py::module_& m) {
  py::class_<Context, CtxPtr>(m, "context", py::module_local())
      .def(py::init([] { return std::make_shared<Context>(); }))
      .def("disable_multithreading", [](Context& c) { c.multithreading = false; });

  py::class_<PyType>(m, "type", py::module_local())
      .def("__str__", [](PyType& t) { return printType(t.t); })
      .def("__eq__", [](PyType& a, PyType& b) { return typeEqual(a.t, b.t); })
      .def("__hash__", [](PyType& t) { return std::hash<std::string>()(printType(t.t)); })
      .def("to_ranked_tensor_ty", [](PyType& t) -> py::object {
        return t.t && t.t->kind == TypeKind::RankedTensor ? castType(t.t) : py::none();
      })
      .def("is_f16", [](PyType& t) { return t.t->kind == TypeKind::F16; })
      .def("is_bf16", [](PyType& t) { return t.t->kind == TypeKind::BF16; })  // addition
      .def("is_f32", [](PyType& t) { return t.t->kind == TypeKind::F32; })
      .def("is_f64", [](PyType& t) { return t.t->kind == TypeKind::F64; })
      .def("is_float", [](PyType& t) { return isFloat(t.t); })
      .def("is_index", [](PyType& t) { return t.t->kind == TypeKind::Index; })
      .def("is_int", [](PyType& t) { return t.t->kind == TypeKind::Integer; })
      .def("is_signed_int", [](PyType&) { return false; })
      .def("is_unsigned_int", [](PyType&) { return false; })
      .def("is_signless_int", [](PyType& t) { return t.t->kind == TypeKind::Integer; });

  py::class_<PyTensor, PyType>(m, "ranked_tensor", py::module_local())
      .def("get_rank", [](PyTensor& t) { return (int64_t)t.t->shape.size(); })
      .def("get_shape", [](PyTensor& t) { return t.t->shape; })
      .def("get_element_ty", [](PyTensor& t) { return castType(t.t->element); });

  py::class_<PyMemRef, PyType>(m, "memref_buffer", py::module_local())
      .def("get_rank", [](PyMemRef& t) { return (int64_t)t.t->shape.size(); })
      .def("get_dim_size", [](PyMemRef& t, unsigned i) { return t.t->shape.at(i); })
      .def("get_elem_width", [](PyMemRef& t) { return bitWidth(t.t->element); })
      .def("get_shape", [](PyMemRef& t) { return t.t->shape; })
      .def("get_element_ty", [](PyMemRef& t) { return castType(t.t->element); })
      .def("get_memory_space", [](PyMemRef& t) -> std::optional<MemorySpace> {
        const unsigned s = t.t->memorySpace;
        if (s == 0 || s == 1 || s == 3) return static_cast<MemorySpace>(s);
        return std::nullopt;
      })
      .def("get_layout_map", [](PyMemRef& t) {
        return t.t->layout.valid ? t.t->layout : AffineMap::identity((unsigned)t.t->shape.size());
      });

  py::class_<PyFunctionType, PyType>(m, "function_type", py::module_local())
      .def("param_types", [](PyFunctionType& t) {
        py::list l;
        for (auto& x : t.t->inputs) l.append(castType(x));
        return l;
      });

  py::class_<PyLocation>(m, "location", py::module_local()).def("__str__", [](PyLocation& l) {
    if (l.loc.file.empty()) return std::string("loc(unknown)");
    return "loc(\"" + l.loc.file + "\":" + std::to_string(l.loc.line) + ":" + std::to_string(l.loc.col) + ")";
  });

  py::class_<PyValue>(m, "value", py::module_local())
      .def("get_context", [](PyValue& v) { return v.keep; })
      .def("get_defining_op", [](PyValue& v) -> py::object {
        if (!v.v->defOp) return py::none();
        return py::cast(wrapOp<PyOperation>(v.v->defOp));
      })
      .def("get_users", [](PyValue& v) {
        py::list l;
        for (auto& u : v.v->uses) l.append(wrapOp<PyOperation>(u.first));
        return l;
      })
      .def("replace_all_uses_with", [](PyValue& v, PyValue& n) { replaceAllUsesWith(v.v, n.v); })
      .def("get_type", [](PyValue& v) { return castType(v.v->type); })
      .def("id", [](PyValue& v) { return (uint64_t)(uintptr_t)v.v; })
      .def("__eq__", [](PyValue& a, PyValue& b) { return a.v == b.v; })
      .def("__hash__", [](PyValue& v) { return std::hash<const void*>()(v.v); })
      .def("__repr__", [](PyValue& v) { return "Value(" + std::to_string((uintptr_t)v.v) + ")"; })
      .def("__str__", [](PyValue& v) { return printValueName(v.v); });

  py::class_<PyValueRange>(m, "value_range", py::module_local())
      .def(py::init<>())
      .def(py::init([](PyValue& v) { return PyValueRange{{v}}; }))
      .def(py::init([](std::vector<PyValue> v) { return PyValueRange{std::move(v)}; }))
      .def("empty", [](PyValueRange& r) { return r.vals.empty(); })
      .def("size", [](PyValueRange& r) { return r.vals.size(); })
      .def("__len__", [](PyValueRange& r) { return r.vals.size(); })
      .def("__getitem__", [](PyValueRange& r, size_t i) {
        if (i >= r.vals.size()) throw py::index_error("ValueRange index out of range");
        return castValue(r.vals[i].v);
      })
      .def("__iter__", [](PyValueRange& r) {
        py::list l;
        for (auto& v : r.vals) l.append(castValue(v.v));
        return py::iter(l);
      })
      .def("to_vector", [](PyValueRange& r) {
        py::list l;
        for (auto& v : r.vals) l.append(castValue(v.v));
        return l;
      })
      .def("__eq__", [](PyValueRange& a, PyValueRange& b) {
        if (a.vals.size() != b.vals.size()) return false;
        for (size_t i = 0; i < a.vals.size(); ++i)
          if (a.vals[i].v != b.vals[i].v) return false;
        return true;
      })
      .def("__repr__", [](PyValueRange& r) {
        std::string s = "ValueRange([";
        for (size_t i = 0; i < r.vals.size(); ++i)
          s += (i ? ", " : "") + std::string("Value(") + std::to_string((uintptr_t)r.vals[i].v) + ")";
        return s + "])";
      })
      .def("__str__", [](PyValueRange& r) { return "ValueRange(size=" + std::to_string(r.vals.size()) + ")"; });

  py::class_<PyOpResult, PyValue>(m, "op_result", py::module_local());
  py::class_<PyBlockArg, PyValue>(m, "block_argument", py::module_local());

  py::class_<PyRegion>(m, "region", py::module_local())
      .def("get_parent_region", [](PyRegion& r) -> py::object {
        Operation* p = r.r->parentOp;
        if (!p || !p->parent || !p->parent->parent) return py::none();
        return py::cast(PyRegion{p->parent->parent, r.keep});
      })
      .def("size", [](PyRegion& r) { return r.r->blocks.size(); })
      .def("front", [](PyRegion& r) {
        if (r.r->blocks.empty()) throw py::index_error("region has no blocks");
        return wrapBlock(r.r->blocks.front());
      })
      .def("empty", [](PyRegion& r) { return r.r->blocks.empty(); })
      .def("push_back", [](PyRegion& r, PyBlock& b) { r.r->push_back(b.b); })  // used by FriskHelper
      .def("id", [](PyRegion& r) { return (uint64_t)(uintptr_t)r.r; });

  py::class_<PyBlock>(m, "block", py::module_local())
      .def("arg", [](PyBlock& b, int i) {
        if (i < 0 || (size_t)i >= b.b->args.size())
          throw py::index_error("Block argument index out of range");
        return castValue(b.b->args[(size_t)i]);
      })
      .def("add_argument", [](PyBlock& b, PyType& t) { b.b->addArgument(t.t); })
      .def("get_num_arguments", [](PyBlock& b) { return b.b->args.size(); })
      .def("get_argument", [](PyBlock& b, unsigned i) {
        if (i >= b.b->args.size()) throw py::index_error("Block argument index out of range");
        return castValue(b.b->args[i]);
      })
      .def("dump", [](PyBlock& b) { std::cerr << printBlock(b.b) << std::endl; })
      .def("get_parent", [](PyBlock& b) -> py::object {
        if (!b.b->parent) return py::none();
        return py::cast(PyRegion{b.b->parent, b.keep});
      })
      .def("move_before", [](PyBlock& b, PyBlock& dst) {
        Region* r = dst.b->parent;
        if (!r) throw std::runtime_error("destination block has no parent region");
        if (b.b->parent) {
          auto& v = b.b->parent->blocks;
          v.erase(std::remove(v.begin(), v.end(), b.b), v.end());
        }
        auto it = std::find(r->blocks.begin(), r->blocks.end(), dst.b);
        r->blocks.insert(it, b.b);
        b.b->parent = r;
      })
      .def("insert_before", [](PyBlock& b, PyBlock& dst) {
        Region* r = dst.b->parent;
        if (!r) throw std::runtime_error("destination block has no parent region");
        auto it = std::find(r->blocks.begin(), r->blocks.end(), dst.b);
        r->blocks.insert(it, b.b);
        b.b->parent = r;
      })
      .def("merge_block_before", [](PyBlock& b, PyBlock& dst) {
        if (!b.b->args.empty()) throw std::runtime_error("This block has arguments, don't merge");
        std::vector<Operation*> moved = b.b->ops;
        b.b->ops.clear();
        size_t pos = 0;
        for (Operation* op : moved) dst.b->insert(pos++, op);
        if (b.b->parent) {
          auto& v = b.b->parent->blocks;
          v.erase(std::remove(v.begin(), v.end(), b.b), v.end());
          b.b->parent = nullptr;
        }
      })
      .def("replace_use_in_block_with", [](PyBlock& b, PyValue& v, PyValue& nv) {
        auto uses = v.v->uses;
        for (auto& [op, idx] : uses) {
          for (Block* cur = op->parent; cur;) {
            if (cur == b.b) { op->setOperand(idx, nv.v); break; }
            Operation* p = cur->parent ? cur->parent->parentOp : nullptr;
            cur = p ? p->parent : nullptr;
          }
        }
      })
      .def("__str__", [](PyBlock& b) { return printBlock(b.b); })
      .def("has_terminator", [](PyBlock& b) { return !b.b->ops.empty() && b.b->ops.back()->isTerminator(); })
      .def("has_return", [](PyBlock& b) { return !b.b->ops.empty() && b.b->ops.back()->isTerminator(); })
      .def("erase", [](PyBlock& b) {
        if (b.b->parent) {
          auto& v = b.b->parent->blocks;
          v.erase(std::remove(v.begin(), v.end(), b.b), v.end());
          b.b->parent = nullptr;
        }
      })
      .def("walk", [](PyBlock& b, const std::function<void(PyOperation)>& fn) {
        std::vector<Operation*> copy = b.b->ops;
        for (Operation* op : copy) walk(op, [&](Operation* o) { fn(wrapOp<PyOperation>(o)); });
      })
      .def("id", [](PyBlock& b) { return (uint64_t)(uintptr_t)b.b; });

  py::class_<PyAttribute>(m, "attribute", py::module_local())
      .def("__str__", [](PyAttribute& a) { return printAttribute(a.a); });
}

void initOperation(py::module_& m) {
  py::class_<PyOpState>(m, "OpState", py::module_local())
      .def("set_attr", [](PyOpState& s, const std::string& n, PyAttribute& a) { s.op->attrs[n] = a.a; })
      .def("get_num_results", [](PyOpState& s) { return s.op->results.size(); })
      .def("get_result", [](PyOpState& s, unsigned i) {
        if (i >= s.op->results.size()) throw py::index_error("Op result index out of range");
        return castValue(s.op->results[i]);
      })
      .def("get_region", [](PyOpState& s, unsigned i) {
        if (i >= s.op->regions.size()) throw py::index_error("Op region index out of range");
        return PyRegion{s.op->regions[i], s.keep};
      })
      .def("dump", [](PyOpState& s) { std::cerr << printOperation(s.op) << std::endl; })
      .def("__str__", [](PyOpState& s) { return printOperation(s.op); })
      .def("append_operand", [](PyOpState& s, PyValue& v) { s.op->addOperand(v.v); })
      .def("verify", [](PyOpState& s) { return verify(s.op).empty(); })
      .def("verify_message", [](PyOpState& s) { return verify(s.op); })  // addition: the reason
      .def("get_operation", [](PyOpState& s) { return wrapOp<PyOperation>(s.op); });  // addition

  py::class_<PyOperation>(m, "operation", py::module_local())
      .def("__str__", [](PyOperation& o) { return o.op->name; })
      .def("__repr__", [](PyOperation& o) { return o.op->name; })
      .def("get_name", [](PyOperation& o) { return o.op->name; })
      .def("get_num_operands", [](PyOperation& o) { return o.op->operands.size(); })
      .def("get_operand", [](PyOperation& o, unsigned i) { return castValue(o.op->operands.at(i)); })
      .def("set_operand", [](PyOperation& o, unsigned i, PyValue& v) { o.op->setOperand(i, v.v); })
      .def("get_num_results", [](PyOperation& o) { return o.op->results.size(); })
      .def("get_result", [](PyOperation& o, unsigned i) { return castValue(o.op->results.at(i)); })
      .def("get_num_regions", [](PyOperation& o) { return o.op->regions.size(); })
      .def("get_region", [](PyOperation& o, unsigned i) { return PyRegion{o.op->regions.at(i), o.keep}; })
      .def("get_block", [](PyOperation& o) -> py::object {
        if (!o.op->parent) return py::none();
        return py::cast(wrapBlock(o.op->parent));
      })
      .def("get_str_attr", [](PyOperation& o, const std::string& n) -> py::object {
        const Attribute* a = o.op->attr(n);
        if (a && std::holds_alternative<std::string>(*a)) return py::str(std::get<std::string>(*a));
        return py::none();
      })
      .def("get_flat_symbol_ref_attr", [](PyOperation&, const std::string&) -> py::object { return py::none(); })
      .def("get_int_attr", [](PyOperation& o, const std::string& n) -> py::object {  // addition
        const Attribute* a = o.op->attr(n);
        if (a && std::holds_alternative<IntAttr>(*a)) return py::int_(std::get<IntAttr>(*a).value);
        return py::none();
      })
      .def("is_constant_op", [](PyOperation& o) { return o.op->name == "arith.constant"; })
      .def("to_constant_op", [](PyOperation& o) -> py::object {
        if (o.op->name == "arith.constant") return py::cast(wrapOp<PyConstant>(o.op));
        return py::none();
      })
      .def("to_gemm_op", [](PyOperation& o) -> py::object {  // addition (GemmOp.from_operation)
        if (o.op->name == "frisk.gemm") return py::cast(wrapOp<PyGemm>(o.op));
        return py::none();
      })
      .def("to_reduce_op", [](PyOperation& o) -> py::object {  // addition
        if (o.op->name == "frisk.reduce") return py::cast(wrapOp<PyReduce>(o.op));
        return py::none();
      });
}

void initCommonOps(py::module_& m) {
  py::class_<PyModule, PyOpState>(m, "module", py::module_local(), py::dynamic_attr())
      .def("dump", [](PyModule& s, const std::string& log) {
        if (!log.empty()) py::print(log);
        py::print(printOperation(s.op));
      }, py::arg("log") = "")
      .def("__str__", [](PyModule& s) { return printOperation(s.op); })
      .def("push_back", [](PyModule& s, PyOpState& fnOrKernel) {
        Block* body = s.op->regions[0]->blocks[0];
        if (fnOrKernel.op->parent) return;  // already inserted
        body->insert(body->ops.size(), fnOrKernel.op);
      })
      .def("has_function", [](PyModule& s, const std::string& n) { return lookupSymbol(s.op, n, "func.func") != nullptr; })
      .def("get_function", [](PyModule& s, const std::string& n) -> py::object {
        Operation* op = lookupSymbol(s.op, n, "func.func");
        return op ? py::cast(wrapOp<PyFunction>(op)) : py::none();
      })
      .def("get_kernel", [](PyModule& s, const std::string& n) -> py::object {
        Operation* op = lookupSymbol(s.op, n, "frisk.kernel");
        return op ? py::cast(wrapOp<PyKernel>(op)) : py::none();
      })
      .def("erase_kernel", [](PyModule& s, const std::string& n) {
        if (Operation* op = lookupSymbol(s.op, n, "frisk.kernel")) op->parent->erase(op);
      })
      .def("get_int_attr", [](PyModule& s, const std::string& n) -> py::object {
        const Attribute* a = s.op->attr(n);
        if (a && std::holds_alternative<IntAttr>(*a)) return py::int_(std::get<IntAttr>(*a).value);
        return py::none();
      })
      .def("set_str_attr", [](PyModule& s, const std::string& n, const std::string& v) {  // addition:
        s.op->attrs[n] = v;                                                                // e.g. frisk.target
      })
      .def("get_str_attr", [](PyModule& s, const std::string& n) -> py::object {  // addition
        const Attribute* a = s.op->attr(n);
        if (a && std::holds_alternative<std::string>(*a)) return py::str(std::get<std::string>(*a));
        return py::none();
      })
      .def("walk", [](PyModule& s, const std::function<void(PyOperation)>& fn) {
        walk(s.op, [&](Operation* o) { fn(wrapOp<PyOperation>(o)); });
      });

  py::class_<PyConstant, PyOpState>(m, "constant", py::module_local())
      .def("get_splat_float_value", [](PyConstant& c) -> py::object {
        const Attribute* a = c.op->attr("splat");
        if (a && std::holds_alternative<FloatAttr>(*a)) return py::float_(std::get<FloatAttr>(*a).value);
        return py::none();
      });

  py::class_<PyFunction, PyOpState>(m, "function", py::module_local())
      .def("arg", [](PyFunction& f, unsigned i) {
        Block* b = f.op->regions[0]->blocks.empty() ? nullptr : f.op->regions[0]->blocks[0];
        if (!b || i >= b->args.size()) throw py::index_error("Function argument index out of range");
        return castValue(b->args[i]);
      })
      .def("get_num_arguments", [](PyFunction& f) { return std::get<Type>(*f.op->attr("function_type"))->inputs.size(); })
      .def("get_callable_region", [](PyFunction& f) { return PyRegion{f.op->regions[0], f.keep}; })
      .def("get_terminator", [](PyFunction& f) -> py::object {
        Block* b = f.op->regions[0]->blocks.empty() ? nullptr : f.op->regions[0]->blocks[0];
        if (!b || b->ops.empty()) return py::none();
        return py::cast(wrapOp<PyOperation>(b->ops.back()));
      })
      .def("add_entry_block", [](PyFunction& f) {
        return wrapBlock(addEntryBlock(f.op, std::get<Type>(*f.op->attr("function_type"))->inputs, false));
      })
      .def("set_arg_attr", [](PyFunction& f, int argNo, const std::string& name, int val) {
        if (argNo < 0 || (size_t)argNo >= std::get<Type>(*f.op->attr("function_type"))->inputs.size())
          throw py::index_error("Function argument index out of range");
        f.op->attrs["arg" + std::to_string(argNo) + "." + name] = IntAttr{val, 32};
      })
      .def_property_readonly("type", [](PyFunction& f) { return castType(std::get<Type>(*f.op->attr("function_type"))); })
      .def("reset_type", [](PyFunction& f, PyType& t) { f.op->attrs["function_type"] = t.t; });
}

void initAffine(py::module_& m) {
  py::class_<AffineMap>(m, "AffineMap", py::module_local())
      .def(py::init<>())
      .def_static("get", [](CtxPtr) { return AffineMap::get(0, 0, {}); })
      .def_static("get", [](unsigned d, unsigned s, CtxPtr) { return AffineMap::get(d, s, {}); })
      .def_static("get", [](unsigned d, unsigned s, PyAffineExpr& e) { return AffineMap::get(d, s, {e.e}); })
      .def_static("get", [](unsigned d, unsigned s, std::vector<PyAffineExpr> r, CtxPtr) {
        std::vector<AffineExpr> v;
        for (auto& e : r) v.push_back(e.e);
        return AffineMap::get(d, s, v);
      })
      .def_static("get_constant_map", [](int64_t v, CtxPtr) { return AffineMap::constant(v); })
      .def_static("get_multi_dim_identity_map", [](unsigned n, CtxPtr) { return AffineMap::identity(n); })
      .def_static("get_minor_identity_map", [](unsigned d, unsigned r, CtxPtr) { return AffineMap::minorIdentity(d, r); })
      .def_static("get_permutation_map", [](std::vector<int64_t> p, CtxPtr) {
        std::vector<unsigned> u(p.begin(), p.end());
        return AffineMap::permutation(u);
      })
      .def_static("get_multi_dim_map_with_targets", [](unsigned n, CtxPtr) { return AffineMap::identity(n); })
      .def("__eq__", [](const AffineMap& a, const AffineMap& b) { return a == b; })
      .def("__ne__", [](const AffineMap& a, const AffineMap& b) { return !(a == b); })
      .def("__bool__", [](const AffineMap& a) { return a.valid; })
      .def("__nonzero__", [](const AffineMap& a) { return a.valid; })
      .def("__str__", [](const AffineMap& a) { return a.str(); })
      .def("__repr__", [](const AffineMap& a) { return "AffineMap(" + a.str() + ")"; })
      .def("get_num_dims", [](const AffineMap& a) { return a.numDims; })
      .def("get_num_symbols", [](const AffineMap& a) { return a.numSymbols; })
      .def("get_num_results", [](const AffineMap& a) { return a.results.size(); })
      .def("get_num_inputs", [](const AffineMap& a) { return a.numDims + a.numSymbols; })
      .def("get_results", [](const AffineMap& a) {
        py::list l;
        for (auto& e : a.results) l.append(castExpr(e));
        return l;
      })
      .def("get_result", [](const AffineMap& a, unsigned i) { return castExpr(a.results.at(i)); })
      .def("is_identity", &AffineMap::isIdentity)
      .def("is_symbol_identity", [](const AffineMap& a) {
        if (!a.valid || a.numSymbols != a.results.size()) return false;
        for (unsigned i = 0; i < a.results.size(); ++i)
          if (a.results[i]->kind != AffineKind::SymbolId || a.results[i]->value != (int64_t)i) return false;
        return true;
      })
      .def("is_minor_identity", &AffineMap::isMinorIdentity)
      .def("is_empty", [](const AffineMap& a) { return a.valid && a.numDims == 0 && a.numSymbols == 0 && a.results.empty(); })
      .def("is_single_constant", [](const AffineMap& a) { return a.results.size() == 1 && a.results[0]->kind == AffineKind::Constant; })
      .def("is_constant", [](const AffineMap& a) {
        for (auto& e : a.results) if (e->kind != AffineKind::Constant) return false;
        return true;
      })
      .def("is_permutation", &AffineMap::isPermutation)
      .def("is_projected_permutation", &AffineMap::isProjectedPermutation, py::arg("allow_zero_in_results") = false)
      .def("get_single_constant_result", [](const AffineMap& a) { return a.results.at(0)->value; })
      .def("get_constant_results", [](const AffineMap& a) {
        std::vector<int64_t> v;
        for (auto& e : a.results) v.push_back(e->value);
        return v;
      })
      .def("get_dim_position", [](const AffineMap& a, unsigned i) { return (unsigned)a.results.at(i)->value; }, py::arg("idx"))
      .def("get_result_position", [](const AffineMap& a, PyAffineExpr& in) -> py::object {
        for (size_t i = 0; i < a.results.size(); ++i)
          if (affineEqual(a.results[i], in.e)) return py::int_(i);
        return py::none();
      }, py::arg("input"))
      .def("evaluate", [](const AffineMap& a, std::vector<int64_t> dims, std::vector<int64_t> syms) {  // addition
        std::vector<int64_t> out;
        for (auto& e : a.results) out.push_back(evaluate(e, dims, syms));
        return out;
      }, py::arg("dims"), py::arg("symbols") = std::vector<int64_t>{});

  py::enum_<AffineKind>(m, "AffineExprKind", py::module_local())
      .value("Add", AffineKind::Add)
      .value("Mul", AffineKind::Mul)
      .value("Mod", AffineKind::Mod)
      .value("FloorDiv", AffineKind::FloorDiv)
      .value("CeilDiv", AffineKind::CeilDiv)
      .value("Constant", AffineKind::Constant)
      .value("DimId", AffineKind::DimId)
      .value("SymbolId", AffineKind::SymbolId)
      .export_values();
  m.attr("AffineExprKind").attr("LAST_AFFINE_BINARY_OP") = m.attr("AffineExprKind").attr("CeilDiv");

  auto bin = [](AffineKind k) {
    return [k](const PyAffineExpr& a, const PyAffineExpr& b) { return castExpr(affineBinary(k, a.e, b.e)); };
  };
  auto binc = [](AffineKind k) {
    return [k](const PyAffineExpr& a, int64_t v) { return castExpr(affineBinary(k, a.e, affineConstant(v))); };
  };
  py::class_<PyAffineExpr>(m, "AffineExpr", py::module_local())
      .def(py::init<>())
      .def("__eq__", [](const PyAffineExpr& a, const PyAffineExpr& b) { return affineEqual(a.e, b.e); })
      .def("__eq__", [](const PyAffineExpr& a, int64_t v) { return a.e && a.e->kind == AffineKind::Constant && a.e->value == v; })
      .def("__ne__", [](const PyAffineExpr& a, const PyAffineExpr& b) { return !affineEqual(a.e, b.e); })
      .def("__ne__", [](const PyAffineExpr& a, int64_t v) { return !(a.e && a.e->kind == AffineKind::Constant && a.e->value == v); })
      .def("__bool__", [](const PyAffineExpr& a) { return (bool)a.e; })
      .def("__nonzero__", [](const PyAffineExpr& a) { return (bool)a.e; })
      .def("__hash__", [](const PyAffineExpr& a) { return std::hash<std::string>()(printAffineExpr(a.e)); })
      .def("__str__", [](const PyAffineExpr& a) { return printAffineExpr(a.e); })
      .def("__repr__", [](const PyAffineExpr& a) { return "AffineExpr(" + printAffineExpr(a.e) + ")"; })
      .def("get_kind", [](const PyAffineExpr& a) { return a.e->kind; })
      .def("is_symbolic_or_constant", [](const PyAffineExpr& a) { return isSymbolicOrConstant(a.e); })
      .def("is_pure_affine", [](const PyAffineExpr& a) { return isPureAffine(a.e); })
      .def("get_largest_known_divisor", [](const PyAffineExpr& a) { return largestKnownDivisor(a.e); })
      .def("is_multiple_of", [](const PyAffineExpr& a, int64_t f) { return f != 0 && largestKnownDivisor(a.e) % f == 0; })
      .def("is_function_of_dim", [](const PyAffineExpr& a, unsigned p) { return isFunctionOfDim(a.e, p); })
      .def("is_function_of_symbol", [](const PyAffineExpr& a, unsigned p) { return isFunctionOfSymbol(a.e, p); })
      .def("replace_dims_and_symbols", [](const PyAffineExpr& a, std::vector<PyAffineExpr> d, std::vector<PyAffineExpr> s) {
        std::vector<AffineExpr> dv, sv;
        for (auto& x : d) dv.push_back(x.e);
        for (auto& x : s) sv.push_back(x.e);
        return castExpr(replaceDimsAndSymbols(a.e, dv, sv));
      })
      .def("replace_dims", [](const PyAffineExpr& a, std::vector<PyAffineExpr> d) {
        std::vector<AffineExpr> dv;
        for (auto& x : d) dv.push_back(x.e);
        return castExpr(replaceDimsAndSymbols(a.e, dv, {}));
      })
      .def("replace_symbols", [](const PyAffineExpr& a, std::vector<PyAffineExpr> s) {
        std::vector<AffineExpr> sv;
        for (auto& x : s) sv.push_back(x.e);
        return castExpr(replaceDimsAndSymbols(a.e, {}, sv));
      })
      .def("shift_dims", [](const PyAffineExpr& a, unsigned numDims, unsigned shift, unsigned offset) {
        std::vector<AffineExpr> d;
        for (unsigned i = 0; i < numDims; ++i) d.push_back(affineDim(i < offset ? i : i + shift));
        return castExpr(replaceDimsAndSymbols(a.e, d, {}));
      }, py::arg("num_dims"), py::arg("shift"), py::arg("offset") = 0)
      .def("shift_symbols", [](const PyAffineExpr& a, unsigned numSyms, unsigned shift, unsigned offset) {
        std::vector<AffineExpr> s;
        for (unsigned i = 0; i < numSyms; ++i) s.push_back(affineSymbol(i < offset ? i : i + shift));
        return castExpr(replaceDimsAndSymbols(a.e, {}, s));
      }, py::arg("num_symbols"), py::arg("shift"), py::arg("offset") = 0)
      .def("__add__", binc(AffineKind::Add))
      .def("__add__", bin(AffineKind::Add))
      .def("__radd__", binc(AffineKind::Add))
      .def("__neg__", [](const PyAffineExpr& a) { return castExpr(affineBinary(AffineKind::Mul, a.e, affineConstant(-1))); })
      .def("__sub__", [](const PyAffineExpr& a, int64_t v) { return castExpr(affineBinary(AffineKind::Add, a.e, affineConstant(-v))); })
      .def("__sub__", [](const PyAffineExpr& a, const PyAffineExpr& b) {
        return castExpr(affineBinary(AffineKind::Add, a.e, affineBinary(AffineKind::Mul, b.e, affineConstant(-1))));
      })
      .def("__rsub__", [](const PyAffineExpr& a, int64_t v) {
        return castExpr(affineBinary(AffineKind::Add, affineConstant(v), affineBinary(AffineKind::Mul, a.e, affineConstant(-1))));
      })
      .def("__mul__", binc(AffineKind::Mul))
      .def("__mul__", bin(AffineKind::Mul))
      .def("__rmul__", binc(AffineKind::Mul))
      .def("floor_div", binc(AffineKind::FloorDiv))
      .def("floor_div", bin(AffineKind::FloorDiv))
      .def("ceil_div", binc(AffineKind::CeilDiv))
      .def("ceil_div", bin(AffineKind::CeilDiv))
      .def("__mod__", binc(AffineKind::Mod))
      .def("__mod__", bin(AffineKind::Mod))
      .def("compose", [](const PyAffineExpr& a, const AffineMap& map) {
        return castExpr(replaceDimsAndSymbols(a.e, map.results, {}));
      })
      .def("as_binary", [](const PyAffineExpr& a) -> py::object {
        if (a.e && a.e->kind <= AffineKind::CeilDiv) { PyBinaryExpr b; b.e = a.e; return py::cast(b); }
        return py::none();
      })
      .def("as_dim", [](const PyAffineExpr& a) -> py::object {
        if (a.e && a.e->kind == AffineKind::DimId) { PyDimExpr b; b.e = a.e; return py::cast(b); }
        return py::none();
      })
      .def("as_symbol", [](const PyAffineExpr& a) -> py::object {
        if (a.e && a.e->kind == AffineKind::SymbolId) { PySymbolExpr b; b.e = a.e; return py::cast(b); }
        return py::none();
      })
      .def("as_constant", [](const PyAffineExpr& a) -> py::object {
        if (a.e && a.e->kind == AffineKind::Constant) { PyConstExpr b; b.e = a.e; return py::cast(b); }
        return py::none();
      });
  py::class_<PyBinaryExpr, PyAffineExpr>(m, "AffineBinaryOpExpr", py::module_local())
      .def("get_lhs", [](PyBinaryExpr& b) { return castExpr(b.e->lhs); })
      .def("get_rhs", [](PyBinaryExpr& b) { return castExpr(b.e->rhs); });
  py::class_<PyDimExpr, PyAffineExpr>(m, "AffineDimExpr", py::module_local())
      .def("get_position", [](PyDimExpr& b) { return (unsigned)b.e->value; });
  py::class_<PySymbolExpr, PyAffineExpr>(m, "AffineSymbolExpr", py::module_local())
      .def("get_position", [](PySymbolExpr& b) { return (unsigned)b.e->value; });
  py::class_<PyConstExpr, PyAffineExpr>(m, "AffineConstantExpr", py::module_local())
      .def("get_value", [](PyConstExpr& b) { return b.e->value; });

  m.def("get_affine_dim_expr", [](unsigned p, CtxPtr) { return castExpr(affineDim(p)); });
  m.def("get_affine_symbol_expr", [](unsigned p, CtxPtr) { return castExpr(affineSymbol(p)); });
  m.def("get_affine_constant_expr", [](int64_t v, CtxPtr) { return castExpr(affineConstant(v)); });
  m.def("get_affine_constant_exprs", [](std::vector<int64_t> vs, CtxPtr) {
    py::list l;
    for (int64_t v : vs) l.append(castExpr(affineConstant(v)));
    return l;
  });
  m.def("get_affine_binary_op_expr", [](AffineKind k, PyAffineExpr& a, PyAffineExpr& b) {
    return castExpr(affineBinary(k, a.e, b.e));
  });
  m.def("simplify_affine_expr", [](PyAffineExpr& e, unsigned, unsigned) {
    // expressions are kept simplified as they are built; rebuilding re-applies the rules bottom-up
    return castExpr(replaceDimsAndSymbols(e.e, {}, {}));
  });
}

void initBuilder(py::module_& m) {
  py::class_<InsertPoint>(m, "InsertPoint", py::module_local());

  py::enum_<MemorySpace>(m, "MemorySpace", py::arithmetic())
      .value("GLOBAL", MemorySpace::Global)
      .value("SHARED", MemorySpace::Shared)
      .value("LOCAL", MemorySpace::Local)
      .export_values();

  auto constantOp = [](PyBuilder& self, Attribute value, Type type) {
    Operation* op = self.b.create("arith.constant");
    op->attrs["value"] = std::move(value);
    Value r = self.b.ctx->newValue(std::move(type));
    r->defOp = op;
    op->results.push_back(r);
    return castValue(r);
  };
  auto tensorConstant = [](PyBuilder& self, const std::vector<double>& v, std::vector<int64_t> shape, Type elem, bool isInt) {
    Type tt = makeTensor(std::move(shape), elem);
    std::string text = "dense<";
    bool splat = !v.empty() && std::all_of(v.begin(), v.end(), [&](double x) { return x == v[0]; });
    auto one = [&](double x) {
      if (isInt) return std::to_string((int64_t)x);
      char buf[64];
      snprintf(buf, sizeof buf, "%.6e", x);
      return std::string(buf);
    };
    if (splat) text += one(v[0]);
    else {
      text += "[";
      for (size_t i = 0; i < v.size(); ++i) text += (i ? ", " : "") + one(v[i]);
      text += "]";
    }
    text += ">";
    Operation* op = self.b.create("arith.constant");
    op->attrs["value"] = text;
    if (splat && !isInt) op->attrs["splat"] = FloatAttr{v[0], elem};
    Value r = self.b.ctx->newValue(tt);
    r->defOp = op;
    op->results.push_back(r);
    return castValue(r);
  };

  py::class_<PyBuilder>(m, "builder")
      .def(py::init<CtxPtr>())
      .def("create_module", [](PyBuilder& self) {
        Operation* op = self.b.ctx->newOp("builtin.module", self.b.lastLoc);  // never auto-inserted
        Region* r = self.b.ctx->newRegion(op);
        r->push_back(self.b.ctx->newBlock());
        return wrapOp<PyModule>(op);
      })
      .def("set_insertion_point_to_start", [](PyBuilder& self, PyBlock& b) { self.b.setInsertionPointToStart(b.b); })
      .def("set_insertion_point_to_end", [](PyBuilder& self, PyBlock& b) { self.b.setInsertionPointToEnd(b.b); })
      .def("set_insertion_point_after", [](PyBuilder& self, PyOperation& op) { self.b.setInsertionPointAfter(op.op); })
      .def("set_insertion_point_after", [](PyBuilder& self, PyOpState& op) { self.b.setInsertionPointAfter(op.op); })
      .def("get_insertion_block", [](PyBuilder& self) -> py::object {
        if (!self.b.ip.block) return py::none();
        return py::cast(wrapBlock(self.b.ip.block));
      })
      .def("get_insertion_point", [](PyBuilder& self) { return self.b.ip; })
      .def("restore_insertion_point", [](PyBuilder& self, InsertPoint ip) { self.b.ip = ip; })
      // attributes
      .def("get_bool_attr", [](PyBuilder&, bool v) { return PyAttribute{IntAttr{v, 1}}; })
      .def("get_int32_attr", [](PyBuilder&, int32_t v) { return PyAttribute{IntAttr{v, 32}}; })
      .def("get_int64_attr", [](PyBuilder&, int64_t v) { return PyAttribute{IntAttr{v, 64}}; })  // addition
      .def("get_str_attr", [](PyBuilder&, const std::string& v) { return PyAttribute{v}; })       // addition
      .def("get_float_attr", [](PyBuilder&, float v, const std::string& dtype) {
        return PyAttribute{FloatAttr{v, dtypeFromString(dtype, false)}};
      })
      // constants
      .def("get_int64", [constantOp](PyBuilder& s, int64_t v) { return constantOp(s, IntAttr{v, 64}, makeScalar(TypeKind::Integer, 64)); })
      .def("get_f16", [constantOp](PyBuilder& s, float v) { Type t = makeScalar(TypeKind::F16); return constantOp(s, FloatAttr{v, t}, t); })
      .def("get_f32", [constantOp](PyBuilder& s, float v) { Type t = makeScalar(TypeKind::F32); return constantOp(s, FloatAttr{v, t}, t); })
      .def("get_f64", [constantOp](PyBuilder& s, double v) { Type t = makeScalar(TypeKind::F64); return constantOp(s, FloatAttr{v, t}, t); })
      .def("get_f16_tensor", [tensorConstant](PyBuilder& s, std::vector<double> v, std::vector<int64_t> sh) { return tensorConstant(s, v, sh, makeScalar(TypeKind::F16), false); })
      .def("get_f32_tensor", [tensorConstant](PyBuilder& s, std::vector<double> v, std::vector<int64_t> sh) { return tensorConstant(s, v, sh, makeScalar(TypeKind::F32), false); })
      .def("get_f64_tensor", [tensorConstant](PyBuilder& s, std::vector<double> v, std::vector<int64_t> sh) { return tensorConstant(s, v, sh, makeScalar(TypeKind::F64), false); })
      .def("get_int64_tensor", [tensorConstant](PyBuilder& s, std::vector<double> v, std::vector<int64_t> sh) { return tensorConstant(s, v, sh, makeScalar(TypeKind::Integer, 64), true); })
      // types
      .def("get_bool_ty", [](PyBuilder&) { return castType(makeScalar(TypeKind::Integer, 8)); })
      .def("get_int64_ty", [](PyBuilder&) { return castType(makeScalar(TypeKind::Integer, 64)); })
      .def("get_index_ty", [](PyBuilder&) { return castType(makeScalar(TypeKind::Index)); })  // addition
      .def("get_f64_ty", [](PyBuilder&) { return castType(makeScalar(TypeKind::F64)); })
      .def("get_f16_ty", [](PyBuilder&) { return castType(makeScalar(TypeKind::F16)); })
      .def("get_bf16_ty", [](PyBuilder&) { return castType(makeScalar(TypeKind::BF16)); })
      .def("get_f32_ty", [](PyBuilder&) { return castType(makeScalar(TypeKind::F32)); })
      .def("get_f8e4m3fn_ty", [](PyBuilder&) { return castType(makeScalar(TypeKind::F8E4M3FN)); })  // addition
      .def("get_f8e5m2_ty", [](PyBuilder&) { return castType(makeScalar(TypeKind::F8E5M2)); })      // addition
      .def("get_ranked_tensor_ty", [](PyBuilder&, PyType& e, std::vector<int64_t> shape) { return castType(makeTensor(shape, e.t)); })
      .def("get_memref_ty", [](PyBuilder&, PyType& e, std::vector<int64_t> shape, AffineMap map, MemorySpace space) {
        return castType(makeMemRef(shape, e.t, map, (unsigned)space));
      }, py::arg("elementType"), py::arg("shape"), py::arg("map") = AffineMap(), py::arg("space") = MemorySpace::Global)
      .def("get_function_ty", [](PyBuilder&, std::vector<PyType> in, std::vector<PyType> out) {
        std::vector<Type> i, o;
        for (auto& t : in) i.push_back(t.t);
        for (auto& t : out) o.push_back(t.t);
        return castType(makeFunction(i, o));
      })
      .def("get_kernel_ty", [](PyBuilder&, std::vector<PyType> in) {
        std::vector<Type> i;
        for (auto& t : in) i.push_back(t.t);
        return castType(makeFunction(i, {}));
      })
      // locations
      .def("set_loc", [](PyBuilder& s, PyLocation& l) { s.b.lastLoc = l.loc; })
      .def("set_loc", [](PyBuilder& s, const std::string& f, int line, int col) { s.b.lastLoc = Location{f, line, col}; })
      .def("get_loc", [](PyBuilder& s) { return PyLocation{s.b.lastLoc}; })
      // generic ops
      .def("get_or_insert_function", [](PyBuilder& s, PyModule& mod, const std::string& name, PyType& ty) {
        if (Operation* f = lookupSymbol(mod.op, name, "func.func")) return wrapOp<PyFunction>(f);
        if (!ty.t || ty.t->kind != TypeKind::Function) throw std::invalid_argument("invalid function type");
        Operation* op = s.b.create("func.func");
        op->attrs["sym_name"] = name;
        op->attrs["function_type"] = ty.t;
        s.b.ctx->newRegion(op);
        return wrapOp<PyFunction>(op);
      })
      .def("create_block", [](PyBuilder& s) {
        if (!s.b.ip.block || !s.b.ip.block->parent) throw std::runtime_error("no insertion block");
        Block* b = s.b.ctx->newBlock();
        s.b.ip.block->parent->push_back(b);
        s.b.setInsertionPointToStart(b);
        return wrapBlock(b);
      })
      .def("create_block_with_parent", [](PyBuilder& s, PyRegion& parent, std::vector<PyType> argTypes) {
        Block* b = s.b.ctx->newBlock();
        parent.r->push_back(b);
        for (auto& t : argTypes) b->addArgument(t.t);
        s.b.setInsertionPointToStart(b);
        return wrapBlock(b);
      })
      .def("new_block", [](PyBuilder& s) { return wrapBlock(s.b.ctx->newBlock()); })
      .def("ret", [](PyBuilder& s, std::vector<PyValue> vals) {
        Operation* op = s.b.create("func.return");
        for (auto& v : vals) op->addOperand(v.v);
        return wrapOp<PyOpState>(op);
      })
      // affine helpers
      .def("get_affine_dim_expr", [](PyBuilder&, unsigned p) { return castExpr(affineDim(p)); })
      .def("get_affine_symbol_expr", [](PyBuilder&, unsigned p) { return castExpr(affineSymbol(p)); })
      .def("get_affine_constant_expr", [](PyBuilder&, int64_t v) { return castExpr(affineConstant(v)); })
      .def("get_empty_affine_map", [](PyBuilder&) { return AffineMap::get(0, 0, {}); })
      .def("get_dim_identity_map", [](PyBuilder&) { return AffineMap::identity(1); })
      .def("get_multi_dim_identity_map", [](PyBuilder&, unsigned r) { return AffineMap::identity(r); })
      .def("get_symbol_identity_map", [](PyBuilder&) { return AffineMap::get(0, 1, {affineSymbol(0)}); })
      .def("get_single_dim_shift_affine_map", [](PyBuilder&, int64_t shift) {
        return AffineMap::get(1, 0, {affineBinary(AffineKind::Add, affineDim(0), affineConstant(shift))});
      })
      .def("get_shifted_affine_map", [](PyBuilder&, AffineMap map, int64_t shift) {
        std::vector<AffineExpr> r;
        for (auto& e : map.results) r.push_back(affineBinary(AffineKind::Add, e, affineConstant(shift)));
        return AffineMap::get(map.numDims, map.numSymbols, r);
      })
      // frisk ops
      .def("create_gemm_op", [](PyBuilder& s, PyValue& A, PyValue& B, PyValue& C, bool transA, bool transB, bool clearAccum,
                                std::optional<PyValue> scaleA, std::optional<PyValue> scaleB) {
        const TypeStorage* a = requireMemRef(A.v, "A");
        const TypeStorage* b = requireMemRef(B.v, "B");
        const TypeStorage* c = requireMemRef(C.v, "C");
        if (a->shape.size() != 2 || b->shape.size() != 2 || c->shape.size() != 2)
          throw std::invalid_argument("create_gemm_op expects rank-2 memrefs");
        auto need = [](int64_t d, const char* what) {
          if (d < 0) throw std::invalid_argument(std::string("create_gemm_op requires static ") + what);
          return d;
        };
        const int64_t mm = need(a->shape[0], "M dimension of A"), k = need(a->shape[1], "K dimension of A");
        if (k != need(b->shape[0], "K dimension of B"))
          throw std::invalid_argument("create_gemm_op expects A and B inner dimensions to match");
        const int64_t n = need(b->shape[1], "N dimension of B");
        if (mm != need(c->shape[0], "M dimension of C") || n != need(c->shape[1], "N dimension of C"))
          throw std::invalid_argument("create_gemm_op expects C shape to match A/B product");
        const bool fp8 = a->element->kind == TypeKind::F8E4M3FN || a->element->kind == TypeKind::F8E5M2;
        // the reference requires one element type for all three (ffi/ir.cpp:357-359); 8-bit float
        // inputs, which it cannot express at all, may pair with a wider C
        if (!typeEqual(a->element, b->element) || (!typeEqual(a->element, c->element) && !fp8))
          throw std::invalid_argument("create_gemm_op expects operands to have matching element types");
        // addition: per-row scales of A and per-column scales of B (fp32 vectors of M and N
        // entries) for 8-bit float inputs; the reference's op has three operands only
        if (scaleA.has_value() != scaleB.has_value())
          throw std::invalid_argument("create_gemm_op expects scale_a and scale_b together");
        if (scaleA) {
          if (!fp8) throw std::invalid_argument("create_gemm_op takes scales only with 8-bit float operands");
          auto vec = [](Value v, int64_t n, const char* what) {
            const TypeStorage* t = requireMemRef(v, what);
            if (t->shape.size() != 1 || t->shape[0] != n || t->element->kind != TypeKind::F32)
              throw std::invalid_argument(std::string("create_gemm_op expects ") + what + " to be a rank-1 f32 memref of matching length");
          };
          vec(scaleA->v, mm, "scale_a");
          vec(scaleB->v, n, "scale_b");
        }
        Operation* op = s.b.create("frisk.gemm");
        op->addOperand(A.v);
        op->addOperand(B.v);
        op->addOperand(C.v);
        if (scaleA) {
          op->addOperand(scaleA->v);
          op->addOperand(scaleB->v);
        }
        op->attrs["transA"] = IntAttr{transA, 1};
        op->attrs["transB"] = IntAttr{transB, 1};
        op->attrs["M"] = IntAttr{mm, 64};
        op->attrs["N"] = IntAttr{n, 64};
        op->attrs["K"] = IntAttr{k, 64};
        op->attrs["policy"] = EnumAttr{"gemm_warp_policy", "Square"};
        op->attrs["clear_accum"] = IntAttr{clearAccum, 1};
        return wrapOp<PyGemm>(op);
      }, py::arg("A"), py::arg("B"), py::arg("C"), py::arg("transA") = false, py::arg("transB") = false, py::arg("clear_accum") = false,
         py::arg("scale_a") = py::none(), py::arg("scale_b") = py::none())
      .def("create_kernel_op", [](PyBuilder& s, PyModule& mod, const std::string& name, PyType& ty) {
        if (Operation* k = lookupSymbol(mod.op, name, "frisk.kernel")) return wrapOp<PyKernel>(k);
        if (!ty.t || ty.t->kind != TypeKind::Function) throw std::invalid_argument("invalid kernel function type");
        Operation* op = s.b.create("frisk.kernel");
        op->attrs["sym_name"] = name;
        op->attrs["function_type"] = ty.t;
        s.b.ctx->newRegion(op);
        return wrapOp<PyKernel>(op);
      })
      .def("create_parallel_op", [](PyBuilder& s, std::vector<int64_t> grid, int64_t threads) {
        // the reference accepts a parallel op only as the sole op (besides the hidden terminator)
        if (!s.b.ip.block || s.b.ip.block->ops.size() != 1) throw std::invalid_argument("invalid parallel create");
        Operation* op = s.b.create("frisk.parallel");
        op->attrs["threads"] = IntAttr{threads, 64};
        op->attrs["ranges"] = DenseI64{grid};
        s.b.ctx->newRegion(op);
        return wrapOp<PyParallel>(op);
      })
      .def("create_block_op", [](PyBuilder& s, std::vector<int64_t> ranges, py::function fn) {
        Operation* op = s.b.create("frisk.block");
        op->attrs["ranges"] = DenseI64{ranges};
        py::object self = py::cast(&s, ret::reference);
        buildBody(s, op, ranges.size(), [&](Block* body) {
          PyValueRange ivs;
          for (Value v : body->args) ivs.vals.push_back(PyValue{v, keepOf(v->ctx)});
          fn(self, ivs);
        });
        return wrapOp<PyBlockOp>(op);
      })
      .def("create_for_op", [](PyBuilder& s, int64_t lower, int64_t upper, int64_t step, py::function fn) {
        Operation* op = s.b.create("frisk.for");
        op->attrs["lower"] = IntAttr{lower, 64};
        op->attrs["upper"] = IntAttr{upper, 64};
        op->attrs["step"] = IntAttr{step, 64};
        py::object self = py::cast(&s, ret::reference);
        buildBody(s, op, 1, [&](Block* body) { fn(self, castValue(body->args[0])); });
        return wrapOp<PyFor>(op);
      })
      .def("create_alloc_buffer_op", [](PyBuilder& s, std::vector<int64_t> shape, const std::string& dtype, MemorySpace space, int64_t alignment) {
        Type elem = dtypeFromString(dtype, true);
        if (alignment < 0) throw std::invalid_argument("alignment must be non-negative");
        Operation* op = s.b.create("frisk.alloc_buffer");
        op->attrs["shape"] = DenseI64{shape};
        op->attrs["elementType"] = elem;
        op->attrs["alignment"] = IntAttr{alignment, 64};
        op->attrs["memorySpace"] = IntAttr{(int64_t)space, 64};
        Value r = s.b.ctx->newValue(makeMemRef(shape, elem, AffineMap(), (unsigned)space));
        r->defOp = op;
        op->results.push_back(r);
        return wrapOp<PyAlloc>(op);
      }, py::arg("shape"), py::arg("dtype"), py::arg("space") = MemorySpace::Global, py::arg("alignment") = 0)
      .def("create_copy_op", [](PyBuilder& s, PyValue& src, PyValue& dst, std::vector<PyValue> srcIdx, std::vector<PyValue> dstIdx,
                                AffineMap srcMap, AffineMap dstMap, std::vector<int64_t> srcExt, std::vector<int64_t> dstExt) {
        auto *st = src.v->type.get(), *dt = dst.v->type.get();
        if (st->kind != TypeKind::MemRef || dt->kind != TypeKind::MemRef) throw std::invalid_argument("create_copy_op expects memref operands");
        const bool maps = srcMap.valid && dstMap.valid, noMaps = !srcMap.valid && !dstMap.valid;
        const bool exts = !srcExt.empty() && !dstExt.empty(), noExts = srcExt.empty() && dstExt.empty();
        if (!((noMaps && noExts) || (maps && noExts) || (maps && exts)))
          throw std::invalid_argument("copy op map error.");  // the reference aborts the process here
        if (noMaps) {
          srcMap = AffineMap::identity((unsigned)st->shape.size());
          dstMap = AffineMap::identity((unsigned)dt->shape.size());
        }
        if (srcMap.numDims + srcMap.numSymbols != srcIdx.size() || dstMap.numDims + dstMap.numSymbols != dstIdx.size())
          throw std::invalid_argument("copy op: number of indices must match the map inputs");
        if (noExts) {  // FriskOps.cpp:1578-1590: extents follow the destination shape
          if (st->shape.size() < dt->shape.size()) throw std::invalid_argument("src rank must be >= dst rank");
          dstExt = dt->shape;
          const size_t diff = st->shape.size() - dt->shape.size();
          for (size_t i = 0; i < st->shape.size(); ++i) srcExt.push_back(i < diff ? 1 : dstExt[i - diff]);
        }
        Operation* op = s.b.create("frisk.copy");
        op->addOperand(src.v);
        op->addOperand(dst.v);
        for (auto& v : srcIdx) op->addOperand(v.v);
        for (auto& v : dstIdx) op->addOperand(v.v);
        op->segmentSizes = {1, 1, (int)srcIdx.size(), (int)dstIdx.size()};
        op->attrs["srcMap"] = srcMap;
        op->attrs["dstMap"] = dstMap;
        op->attrs["srcExtents"] = DenseI64{srcExt};
        op->attrs["dstExtents"] = DenseI64{dstExt};
        return wrapOp<PyCopy>(op);
      }, py::arg("src"), py::arg("dst"), py::arg("srcIndices"), py::arg("dstIndices"), py::arg("srcMap") = AffineMap(),
         py::arg("dstMap") = AffineMap(), py::arg("srcExtents") = std::vector<int64_t>{}, py::arg("dstExtents") = std::vector<int64_t>{})
      .def("create_fill_op", [](PyBuilder& s, PyValue& memref, float value, const std::string& dtype) {
        Type t = dtypeFromString(dtype, true);
        Operation* op = s.b.create("frisk.fill");
        op->addOperand(memref.v);
        op->attrs["value"] = FloatAttr{value, t};
        return wrapOp<PyFill>(op);
      })
      .def("create_reduce_op", [](PyBuilder& s, PyValue& src, PyValue& dst, const std::string& kind, int64_t dim, bool clear) {
        Operation* op = s.b.create("frisk.reduce");
        op->addOperand(src.v);
        op->addOperand(dst.v);
        op->attrs["kind"] = kind;
        op->attrs["dim"] = IntAttr{dim, 64};
        op->attrs["clear"] = IntAttr{clear, 1};
        return wrapOp<PyReduce>(op);
      }, py::arg("src"), py::arg("dst"), py::arg("kind"), py::arg("dim"), py::arg("clear") = true);
}

void initFrisk(py::module_ m) {
  m.def("load_dialects", [](Context& c) { c.friskLoaded = true; });
  // addition: the inverse of str(module) -- reads the custom assembly back, the reference's own
  // printed modules included; raises ValueError("line L, column C: ...") on text it cannot read
  m.def("parse_module", [](const std::string& text, CtxPtr ctx) {
    std::string err;
    Operation* op = parseModule(text, ctx, &err);
    if (!op) throw std::invalid_argument("cannot parse module: " + err);
    return wrapOp<PyModule>(op);
  });
  // addition: the tiled matrix product around a frisk.gemm (tmp/ir.mlir:1-17) lifted to one
  // whole-problem GEMM; raises ValueError with the reason when the kernel is anything else
  m.def("lift_tiled_gemm", [](PyKernel& k) {
    TiledGemm t = liftTiledGemm(k.op);
    if (!t.ok) throw std::invalid_argument("not a tiled matrix product: " + t.why);
    py::dict d;
    d["M"] = t.M;
    d["N"] = t.N;
    d["K"] = t.K;
    d["arg_a"] = t.argA;
    d["arg_b"] = t.argB;
    d["arg_c"] = t.argC;
    d["clear_accum"] = t.clearAccum;
    d["ab_type"] = castType(t.elemAB);
    d["c_type"] = castType(t.elemC);
    d["tile"] = t.tile;
    d["grid"] = t.grid;
    if (t.argR >= 0) {  // a row fold of the accumulator rides along
      d["arg_r"] = t.argR;
      d["reduce_kind"] = t.reduceKind;
      d["reduce_clear"] = t.reduceClear;
    }
    return d;
  });
  // addition: the tiled reduce (a grid of tiles folded into a rank-1 accumulator with frisk.reduce)
  // lifted to one whole-buffer reduce; raises ValueError with the reason for anything else
  m.def("lift_tiled_reduce", [](PyKernel& k) {
    TiledReduce t = liftTiledReduce(k.op);
    if (!t.ok) throw std::invalid_argument("not a tiled reduce: " + t.why);
    py::dict d;
    d["shape"] = t.shape;
    d["dim"] = t.dim;
    d["kind"] = t.kind;
    d["clear"] = t.clear;
    d["arg_src"] = t.argSrc;
    d["arg_dst"] = t.argDst;
    d["type"] = castType(t.elem);
    d["tile"] = t.tile;
    d["grid"] = t.grid;
    return d;
  });

  py::class_<PyGemm, PyOpState>(m, "GemmOp", py::module_local())
      .def_static("from_operation", [](PyOperation& o) -> py::object {
        if (o.op->name == "frisk.gemm") return py::cast(wrapOp<PyGemm>(o.op));
        return py::none();
      })
      .def("get_matrix_A", [](PyGemm& g) { return castValue(g.op->operands[0]); })
      .def("get_matrix_B", [](PyGemm& g) { return castValue(g.op->operands[1]); })
      .def("get_matrix_C", [](PyGemm& g) { return castValue(g.op->operands[2]); })
      .def("get_all_matrix", [](PyGemm& g) {
        PyValueRange r;
        for (size_t i = 0; i < 3; ++i) r.vals.push_back(PyValue{g.op->operands[i], g.keep});
        return r;
      })
      // additions: the scale vectors of an 8-bit float gemm (None when the op has none)
      .def("get_scale_A", [](PyGemm& g) -> py::object {
        return g.op->operands.size() == 5 ? castValue(g.op->operands[3]) : py::object(py::none());
      })
      .def("get_scale_B", [](PyGemm& g) -> py::object {
        return g.op->operands.size() == 5 ? castValue(g.op->operands[4]) : py::object(py::none());
      })
      // additions: the op's attributes, and the shared-memory layout the reference infers for an
      // operand tile together with its Blackwell mapping inputs
      .def("get_attrs", [](PyGemm& g) {
        py::dict d;
        for (const char* k : {"M", "N", "K"}) d[k] = g.op->intAttr(k);
        for (const char* k : {"transA", "transB", "clear_accum"}) d[k] = g.op->intAttr(k) != 0;
        d["policy"] = std::get<EnumAttr>(*g.op->attr("policy")).value;
        return d;
      })
      .def("infer_shared_layout", [](PyGemm& g, const std::string& operand, bool hopper) -> py::object {
        const unsigned idx = operand == "A" ? 0 : 1;
        const TypeStorage* t = g.op->operands[idx]->type.get();
        const bool kInner = idx == 0 ? g.op->intAttr("transA") == 0 : g.op->intAttr("transB") != 0;
        auto l = sharedLayoutForOperand(t->shape, bitWidth(t->element), kInner, hopper);
        if (!l) return py::none();
        return py::cast(PyAttribute{*l});
      }, py::arg("operand"), py::arg("hopper") = true)
      // addition: GemmOp::inferLayout (FriskOps.cpp:1285-1407), which the reference reaches only
      // from C++ (test_pass/attr_test.cpp:155-232): {"A", "B", "C"} -> #frisk.layout attribute,
      // plus the warp split and the instruction family it implies.  ValueError with the
      // reference's message when inference fails.
      .def("infer_layout", [](PyGemm& g) {
        GemmLayouts l = inferGemmLayouts(g.op);
        if (!l.ok) throw std::invalid_argument("'frisk.gemm' op " + l.why);
        py::dict d;
        d["A"] = PyAttribute{l.a};
        d["B"] = PyAttribute{l.b};
        d["C"] = PyAttribute{l.c};
        d["warps"] = py::make_tuple(l.warpsM, l.warpsN);
        d["instruction"] = l.instruction;
        return d;
      })
      // addition: where the accumulator of a 128-row tile lives on sm_100a.  The reference's
      // GemmOp::inferLayout gives C a register fragment (FriskOps.cpp:304-347, per-thread ownership
      // for mma.sync / wgmma); with tcgen05 the accumulator is in tensor memory, row r of the tile
      // in lane r, column c in column c, and `tcgen05.ld.32x32b` hands thread t of the warp that
      // owns lanes 32q .. 32q+31 (warp index mod 4 == q) row 32q + t with consecutive columns as
      // consecutive registers.  As a layout: index (d0, d1) -> (d1), thread (d0, d1) -> (d0).
      .def("infer_accumulator_layout_sm100", [](PyGemm& g, int64_t tileRows, int64_t tileCols) {
        if (tileRows != 128) throw std::invalid_argument("a tcgen05 accumulator tile has 128 rows per CTA");
        if (tileCols < 8 || tileCols > 256 || tileCols % 8 != 0)
          throw std::invalid_argument("accumulator columns must be a multiple of 8 up to 256");
        (void)g;
        LayoutAttrData l;
        l.inputShape = {tileRows, tileCols};
        l.forwardIndex = AffineMap::get(2, 0, {affineDim(1)});
        l.forwardThread = AffineMap::get(2, 0, {affineDim(0)});
        l.replicate = 1;
        return PyAttribute{l};
      }, py::arg("tile_rows") = 128, py::arg("tile_cols") = 256);

  py::class_<PyKernel, PyOpState>(m, "KernelOp", py::module_local())
      .def("arg", [](PyKernel& k, unsigned i) {
        Block* b = k.op->regions[0]->blocks.empty() ? nullptr : k.op->regions[0]->blocks[0];
        if (!b || i >= b->args.size()) throw py::index_error("Kernel argument index out of range");
        return castValue(b->args[i]);
      })
      .def("get_num_arguments", [](PyKernel& k) {
        Block* b = k.op->regions[0]->blocks.empty() ? nullptr : k.op->regions[0]->blocks[0];
        return b ? b->args.size() : (size_t)0;
      })
      .def("add_entry_block", [](PyKernel& k) {
        return wrapBlock(addEntryBlock(k.op, std::get<Type>(*k.op->attr("function_type"))->inputs, true));
      })
      .def("get_name", [](PyKernel& k) { return std::get<std::string>(*k.op->attr("sym_name")); })  // addition
      .def_property_readonly("type", [](PyKernel& k) { return castType(std::get<Type>(*k.op->attr("function_type"))); });

  py::class_<PyParallel, PyOpState>(m, "ParallelOp", py::module_local())
      .def("get_ivs", [](PyParallel& p) {
        py::list l;
        if (!p.op->regions[0]->blocks.empty())
          for (Value v : p.op->regions[0]->blocks[0]->args) l.append(castValue(v));
        return l;
      })
      .def("get_grid", [](PyParallel& p) { return std::get<DenseI64>(*p.op->attr("ranges")).values; })
      .def("get_thread_num", [](PyParallel& p) { return p.op->intAttr("threads"); })
      .def("get_grid_dim", [](PyParallel& p) { return std::get<DenseI64>(*p.op->attr("ranges")).values.size(); })
      .def("add_entry_block", [](PyParallel& p) {
        const size_t n = std::get<DenseI64>(*p.op->attr("ranges")).values.size();
        return wrapBlock(addEntryBlock(p.op, std::vector<Type>(n, makeScalar(TypeKind::Index)), true));
      });

  py::class_<PyBlockOp, PyOpState>(m, "BlockOp", py::module_local())
      .def("get_ivs", [](PyBlockOp& p) {
        py::list l;
        for (Value v : p.op->regions[0]->blocks[0]->args) l.append(castValue(v));
        return l;
      })
      .def("get_block_ranges", [](PyBlockOp& p) { return std::get<DenseI64>(*p.op->attr("ranges")).values; })
      .def("get_iteration_num", [](PyBlockOp& p) {
        int64_t n = 1;
        for (int64_t v : std::get<DenseI64>(*p.op->attr("ranges")).values) n *= v;
        return n;
      })
      .def("get_block_dim", [](PyBlockOp& p) { return std::get<DenseI64>(*p.op->attr("ranges")).values.size(); });

  py::class_<PyFor, PyOpState>(m, "ForOp", py::module_local())
      .def("get_induction_var", [](PyFor& f) { return castValue(f.op->regions[0]->blocks[0]->args[0]); })
      .def("get_lower_bound", [](PyFor& f) { return f.op->intAttr("lower"); })
      .def("get_upper_bound", [](PyFor& f) { return f.op->intAttr("upper"); })
      .def("get_step", [](PyFor& f) { return f.op->intAttr("step"); });

  py::class_<PyAlloc, PyOpState>(m, "AllocBufferOp", py::module_local())
      .def("get_alignment", [](PyAlloc& a) { return a.op->intAttr("alignment"); })
      .def("get_memroy_space", [](PyAlloc& a) { return static_cast<MemorySpace>(a.op->intAttr("memorySpace")); })
      .def("get_memory_space", [](PyAlloc& a) { return static_cast<MemorySpace>(a.op->intAttr("memorySpace")); })  // addition (spelling)
      .def("get_result", [](PyAlloc& a) { return castValue(a.op->results[0]); })
      .def("get_result", [](PyAlloc& a, unsigned i) {
        if (i >= a.op->results.size()) throw py::index_error("Op result index out of range");
        return castValue(a.op->results[i]);
      })
      .def("get_memref_ty", [](PyAlloc& a) { return castType(a.op->results[0]->type); });

  py::class_<PyCopy, PyOpState>(m, "CopyOp", py::module_local())
      .def("get_src_affine_map", [](PyCopy& c) { return std::get<AffineMap>(*c.op->attr("srcMap")); })
      .def("get_dst_affine_map", [](PyCopy& c) { return std::get<AffineMap>(*c.op->attr("dstMap")); })
      .def("get_src_memref", [](PyCopy& c) { return castValue(c.op->operands[0]); })
      .def("get_dst_memref", [](PyCopy& c) { return castValue(c.op->operands[1]); })
      .def("get_src_memref_ty", [](PyCopy& c) { return castType(c.op->operands[0]->type); })
      .def("get_dst_memref_ty", [](PyCopy& c) { return castType(c.op->operands[1]->type); })
      .def("get_src_indices", [](PyCopy& c) {
        PyValueRange r;
        for (int i = 0; i < c.op->segmentSizes[2]; ++i) r.vals.push_back(PyValue{c.op->operands[2 + (size_t)i], c.keep});
        return r;
      })
      .def("get_dst_indices", [](PyCopy& c) {
        PyValueRange r;
        const size_t first = 2 + (size_t)c.op->segmentSizes[2];
        for (int i = 0; i < c.op->segmentSizes[3]; ++i) r.vals.push_back(PyValue{c.op->operands[first + (size_t)i], c.keep});
        return r;
      })
      .def("get_src_extents", [](PyCopy& c) { return std::get<DenseI64>(*c.op->attr("srcExtents")).values; })
      .def("get_dst_extents", [](PyCopy& c) { return std::get<DenseI64>(*c.op->attr("dstExtents")).values; });

  py::class_<PyFill, PyOpState>(m, "FillOp", py::module_local())
      .def("get_memref", [](PyFill& f) { return castValue(f.op->operands[0]); });

  py::class_<PyReduce, PyOpState>(m, "ReduceOp", py::module_local())
      .def("get_src_memref", [](PyReduce& r) { return castValue(r.op->operands[0]); })
      .def("get_dst_memref", [](PyReduce& r) { return castValue(r.op->operands[1]); })
      .def("get_reduce_dim", [](PyReduce& r) { return r.op->intAttr("dim"); })
      .def("get_kind", [](PyReduce& r) { return std::get<std::string>(*r.op->attr("kind")); })  // addition
      .def("get_clear", [](PyReduce& r) { return r.op->intAttr("clear") != 0; })              // addition
      // addition: ReduceOp::inferLayout (FriskOps_Reduce.cpp:214-357).  Returns the destination's
      // #frisk.layout, or None when there is nothing to infer; ValueError on a conflict.
      .def("infer_layout", [](PyReduce& r, py::object src, py::object existing) -> py::object {
        auto data = [](py::object o) -> const LayoutAttrData* {
          if (o.is_none()) return nullptr;
          auto* l = std::get_if<LayoutAttrData>(&o.cast<PyAttribute&>().a);
          if (!l) throw std::invalid_argument("'frisk.reduce' op source layout entry must be a frisk.layout attribute");
          return l;
        };
        ReduceLayout l = inferReduceLayout(r.op, data(src), data(existing));
        if (!l.ok) throw std::invalid_argument("'frisk.reduce' op " + l.why);
        if (!l.inferred && existing.is_none()) return py::none();
        return py::cast(PyAttribute{l.layout});
      }, py::arg("src_layout"), py::arg("existing") = py::none());

  // addition: LayoutAttr as an object (the reference constructs it only from C++)
  m.def("layout_attr", [](std::vector<int64_t> shape, AffineMap index, AffineMap thread, py::object replicate) {
    LayoutAttrData l;
    l.inputShape = std::move(shape);
    l.forwardIndex = std::move(index);
    l.forwardThread = std::move(thread);
    if (!replicate.is_none()) l.replicate = replicate.cast<int64_t>();
    return PyAttribute{l};
  }, py::arg("shape"), py::arg("index"), py::arg("thread") = AffineMap(), py::arg("replicate") = py::none());
  m.def("layout_index_map", [](PyAttribute& a) -> py::object {
    if (auto* l = std::get_if<LayoutAttrData>(&a.a)) return py::cast(l->forwardIndex);
    return py::none();
  });
  m.def("layout_thread_map", [](PyAttribute& a) -> py::object {
    auto* l = std::get_if<LayoutAttrData>(&a.a);
    if (l && l->forwardThread.valid) return py::cast(l->forwardThread);
    return py::none();
  });
  m.def("layout_replicate", [](PyAttribute& a) -> py::object {
    auto* l = std::get_if<LayoutAttrData>(&a.a);
    if (l && l->replicate) return py::int_(*l->replicate);
    return py::none();
  });
  m.def("layout_shape", [](PyAttribute& a) -> py::object {
    if (auto* l = std::get_if<LayoutAttrData>(&a.a)) return py::cast(l->inputShape);
    return py::none();
  });
  m.def("layout_debug_string", [](PyAttribute& a) -> std::string {
    if (auto* l = std::get_if<LayoutAttrData>(&a.a)) return layoutDebugString(*l);
    return "<null layout>";
  });
  m.def("used_extent_of_dim", [](const AffineMap& map, unsigned dim, int64_t extent) -> py::object {
    auto v = usedExtentOfDim(map, dim, extent);
    return v ? py::object(py::int_(*v)) : py::object(py::none());
  });
  m.def("enum_attr", [](const std::string& mnemonic, const std::string& value) {
    return PyAttribute{EnumAttr{mnemonic, value}};
  });
}

}  // namespace

PYBIND11_MODULE(frisk_ffi, m) {
  m.doc() = "MLIR-free re-creation of Frisk's IR-builder binding (ffi/ffi.cpp, ffi/ir.cpp)";
  py::module_ ir = m.def_submodule("ir");
  initCommon(ir);
  initOperation(ir);
  initCommonOps(ir);
  initAffine(ir);
  initBuilder(ir);
  initFrisk(ir.def_submodule("frisk"));
}
