// Operator builders: shape/dtype checks, result allocation and function naming of the
// reference Frontend (src/Frontend/Operators.cc), recorded as plain data instead of MLIR.
#include "Frontend/Operators.h"

#include <algorithm>
#include <cstdio>
#include <iostream>

namespace KernelCodeGen {

Log KCGLog::level = Log::Release;

// ---- dtypes (reference: Operators.cc:5-29, plus the two extensions) ---------------------
DType getDType(const std::string& dtype) {
  static const std::map<std::string, DType> table = {
      {"float32", DType::f32}, {"float64", DType::f64}, {"float16", DType::f16}, {"int64", DType::i64},
      {"int32", DType::i32},   {"int16", DType::i16},   {"index", DType::i64},   {"bool", DType::boolean},
      {"bfloat16", DType::bf16}, {"float8_e4m3", DType::f8e4m3}};
  auto it = table.find(dtype);
  return it == table.end() ? DType::invalid : it->second;
}

std::string toStr(DType type) {
  switch (type) {
    case DType::f32: return "float32";
    case DType::f64: return "float64";
    case DType::f16: return "float16";
    case DType::i64: return "int64";
    case DType::i32: return "int32";
    case DType::i16: return "int16";
    case DType::boolean: return "bool";
    case DType::bf16: return "bfloat16";
    case DType::f8e4m3: return "float8_e4m3";
    default: return "";
  }
}

size_t dtypeSize(DType type) {
  switch (type) {
    case DType::f32: case DType::i32: return 4;
    case DType::f64: case DType::i64: return 8;
    case DType::f16: case DType::bf16: case DType::i16: return 2;
    case DType::f8e4m3: case DType::boolean: return 1;
    default: return 0;
  }
}

// ---- handles and graph queries -----------------------------------------------------------
const std::vector<int64_t>& Value::shape() const { return owner->tensors[id].shape; }
std::vector<int64_t> Value::strides() const { return owner->tensors[id].effective_strides(); }

std::vector<int64_t> TensorInfo::effective_strides() const {
  if (!strides.empty()) return strides;
  std::vector<int64_t> st(shape.size(), 1);
  for (int d = static_cast<int>(shape.size()) - 2; d >= 0; --d) st[d] = st[d + 1] * shape[d + 1];
  return st;
}

bool TensorInfo::dense() const {
  if (strides.empty()) return true;
  TensorInfo plain;
  plain.shape = shape;
  return strides == plain.effective_strides();
}
DType Value::dtype() const { return owner->tensors[id].dtype; }
int64_t Value::numel() const {
  int64_t n = 1;
  for (auto d : shape()) n *= d;
  return n;
}
size_t Value::bytes() const { return static_cast<size_t>(numel()) * dtypeSize(dtype()); }

int GraphData::root(int tensor) const {
  while (tensor >= 0 && tensors[tensor].alias_of >= 0) tensor = tensors[tensor].alias_of;
  return tensor;
}

int GraphData::users(int tensor) const {
  int n = 0;
  for (const auto& op : ops) {
    if (op.erased) continue;
    for (int in : op.inputs)
      if (in == tensor) ++n;
  }
  return n;
}

namespace {

std::string dims(const std::vector<int64_t>& shape, const char* sep = "_") {
  std::string s;
  for (auto d : shape) s += sep + std::to_string(d);
  return s;
}

// The reference names a function after its operator and shapes only, so two calls that differ in
// element type would share one function (and one optimizer decision).  All-float32 functions keep
// the reference's exact name; any other element type is appended ("_bfloat16"), and a result type
// that differs from the operand type as well ("_float32_to_int32").
std::string dtype_suffix(DType in, DType out) {
  if (in == DType::f32 && out == DType::f32) return "";
  std::string s = "_" + toStr(in);
  if (out != in) s += "_to_" + toStr(out);
  return s;
}

bool valid(ComputeDAG* graph, Value v, const char* what, bool allow_strided = false) {
  if (!graph || !graph->data) {
    std::cerr << "No graph: call KernelCodeGenerator::createGraph first.\n";
    return false;
  }
  if (!v || v.owner != graph->data.get()) {
    std::cerr << what;
    return false;
  }
  if (!allow_strided && !graph->data->tensors[v.id].dense()) {
    std::cerr << "This operator takes dense row-major tensors; strided PlaceHolders are accepted by BatchedMatmul only.\n";
    return false;
  }
  return true;
}

Value new_tensor(ComputeDAG* graph, const std::vector<int64_t>& shape, DType dt, MemorySpace ms, int producer,
                 int alias_of = -1) {
  TensorInfo t;
  t.shape = shape;
  t.dtype = dt;
  t.space = ms;
  t.producer = producer;
  t.alias_of = alias_of;
  graph->data->tensors.push_back(t);
  return Value{static_cast<int>(graph->data->tensors.size()) - 1, graph->data.get()};
}

// Find-or-create of the per-(op, shape) function (reference: buildFuction, Operators.cc:69-110;
// new functions are inserted at the start of the module).  Every call re-tags it "cpu".
void touch_func(ComputeDAG* graph, const std::string& name) {
  auto& g = *graph->data;
  if (!g.funcs.count(name)) g.func_order.insert(g.func_order.begin(), name);
  g.funcs[name].state = "cpu";
  g.funcs[name].optimizer.clear();
}

Value add_op(ComputeDAG* graph, OpNode node, const std::vector<int64_t>& out_shape, DType out_dt, MemorySpace ms,
             int alias_of) {
  auto& g = *graph->data;
  const int op_index = static_cast<int>(g.ops.size());
  Value out = new_tensor(graph, out_shape, out_dt, ms == MemorySpace::inplace ? MemorySpace::global : ms, op_index,
                         alias_of);
  node.output = out.id;
  touch_func(graph, node.func);
  g.ops.push_back(node);
  return out;
}

// dtype_ == "" means "the element type of the first operand".
bool resolve_dtype(const std::string& dtype_, DType fallback, DType& out, const char* op) {
  out = dtype_.empty() ? fallback : getDType(dtype_);
  if (out == DType::invalid) {
    std::cerr << "Unknown dtype \"" << dtype_ << "\" for " << op << ".\n";
    return false;
  }
  return true;
}

}  // namespace

// ---- ComputeDAG ---------------------------------------------------------------------------
void ComputeDAG::dump(const std::string& info) {
  if (KCGLog::level == Log::Release || !data) return;
  std::cerr << "-----------------------------------------------------------\n";
  std::cerr << "           " << info << "\n";
  std::cerr << "-----------------------------------------------------------\n";
  std::cerr << "module @" << data->name << " {\n";
  for (const auto& f : data->func_order)
    std::cerr << "  func @" << f << " {func.state = \"" << data->funcs[f].state << "\"}\n";
  for (size_t i = 0; i < data->tensors.size(); ++i) {
    const auto& t = data->tensors[i];
    if (t.producer < 0)
      std::cerr << "  %" << i << " = alloc() : <" << dims(t.shape, "x").substr(1) << "x" << toStr(t.dtype) << ", "
                << static_cast<int>(t.space) << ">\n";
  }
  for (const auto& op : data->ops) {
    if (op.erased) continue;
    std::cerr << "  %" << op.output << " = call @" << op.func << "(";
    for (size_t k = 0; k < op.inputs.size(); ++k) std::cerr << (k ? ", %" : "%") << op.inputs[k];
    std::cerr << ")\n";
  }
  std::cerr << "}\n";
}

// ---- PlaceHolder (reference: Operators.cc:112-118) ------------------------------------------
Value PlaceHolder::build(ComputeDAG* graph, const std::vector<int64_t>& shapes, const std::string& dtype,
                         const std::vector<int64_t>& strides) {
  if (!graph || !graph->data) {
    std::cerr << "No graph: call KernelCodeGenerator::createGraph first.\n";
    return {};
  }
  const DType dt = getDType(dtype);
  if (dt == DType::invalid) {
    std::cerr << "Unknown dtype \"" << dtype << "\" for PlaceHolder.\n";
    return {};
  }
  for (auto d : shapes)
    if (d < 0) {
      std::cerr << "PlaceHolder needs static non-negative dims.\n";
      return {};
    }
  if (!strides.empty()) {
    bool ok = strides.size() == shapes.size() && strides.back() == 1;
    for (auto s : strides) ok = ok && s > 0;
    if (!ok) {
      std::cerr << "PlaceHolder strides: one positive element stride per dim, the innermost equal to 1.\n";
      return {};
    }
  }
  Value v = new_tensor(graph, shapes, dt, MemorySpace::global, -1);
  graph->data->tensors[v.id].strides = strides;
  if (graph->data->tensors[v.id].dense()) graph->data->tensors[v.id].strides.clear();
  return v;
}

// ---- Matmul (reference: Operators.cc:120-220) ------------------------------------------------
Value Matmul::build(ComputeDAG* graph, Value A, Value B, const std::string& dtype_) {
  if (!valid(graph, A, "Type of left operand of Matmul is not Memref.\n")) return {};
  if (!valid(graph, B, "Type of right operand of Matmul is not Memref.\n")) return {};
  if (A.shape().size() != 2 || B.shape().size() != 2) {
    std::cerr << "Matmul takes rank-2 operands.\n";
    return {};
  }
  const int64_t m = A.shape()[0], k1 = A.shape()[1], k2 = B.shape()[0], n = B.shape()[1];
  if (k1 != k2) {
    std::cerr << "Can't apply Matmul Operation due to imcompatible K-dim.\n";
    return {};
  }
  DType dt;
  // FP8 inputs accumulate in fp32 and are written as bfloat16 unless asked otherwise.
  const DType fallback = A.dtype() == DType::f8e4m3 ? DType::bf16 : A.dtype();
  if (!resolve_dtype(dtype_, fallback, dt, "Matmul")) return {};
  OpNode node;
  node.kind = OpKind::Matmul;
  node.func = "Matmul_m" + std::to_string(m) + "n" + std::to_string(n) + "k" + std::to_string(k1) +
              dtype_suffix(A.dtype(), dt);
  node.inputs = {A.id, B.id};
  return add_op(graph, node, {m, n}, dt, MemorySpace::global, -1);
}

Value Matmul::build(ComputeDAG* graph, Value A, Value B, MemorySpace, const std::string& dtype_) {
  return build(graph, A, B, dtype_);
}

Value Matmul::build(ComputeDAG* graph, Value A, Value B, Value scaleA, Value scaleB, const std::string& dtype_) {
  if (!valid(graph, scaleA, "Matmul: scale of A is not a tensor of this graph.\n")) return {};
  if (!valid(graph, scaleB, "Matmul: scale of B is not a tensor of this graph.\n")) return {};
  if (scaleA.dtype() != DType::f32 || scaleB.dtype() != DType::f32 || scaleA.numel() != 1 || scaleB.numel() != 1) {
    std::cerr << "Matmul: per-tensor scales are one-element float32 tensors.\n";
    return {};
  }
  Value C = build(graph, A, B, dtype_);
  if (!C) return C;
  auto& op = graph->data->ops.back();
  op.scale_a = scaleA.id;
  op.scale_b = scaleB.id;
  op.inputs.push_back(scaleA.id);
  op.inputs.push_back(scaleB.id);
  return C;
}

// ---- Relu (reference: Operators.cc:222-289) ---------------------------------------------------
Value Relu::build(ComputeDAG* graph, Value input, MemorySpace ms, const std::string& dtype_) {
  if (!valid(graph, input, "Type of input of Relu is not Memref.\n")) return {};
  DType dt;
  if (!resolve_dtype(dtype_, input.dtype(), dt, "Relu")) return {};
  OpNode node;
  node.kind = OpKind::ElementWise;
  node.operation = "Relu";
  const DType out_dt = ms == MemorySpace::inplace ? input.dtype() : dt;
  node.func = "Relu_Elementwise" + dims(input.shape()) + dtype_suffix(input.dtype(), out_dt);
  node.inputs = {input.id};
  return add_op(graph, node, input.shape(), out_dt, ms, ms == MemorySpace::inplace ? input.id : -1);
}

// ---- BatchedMatmul (reference: Operators.cc:291-457) ------------------------------------------
Value BatchedMatmul::build(ComputeDAG* graph, Value A, Layout layoutA, Value B, Layout layoutB,
                           const std::string& dtype_, Value out) {
  if (!valid(graph, A, "Type of left operand of BatchedMatmul is not Memref.\n", true)) return {};
  if (!valid(graph, B, "Type of right operand of BatchedMatmul is not Memref.\n", true)) return {};
  const auto& sa = A.shape();
  const auto& sb = B.shape();
  const int total = static_cast<int>(sa.size());
  if (total < 2) {
    // the reference exits the process here (Operators.cc:306-309); a null handle is kinder
    std::cerr << "BatchedMatmul needs at least 2 dim but got " << total << "\n";
    return {};
  }
  if (sb.size() != sa.size()) {
    std::cerr << "BatchedMatmul: A, B dim not matched.\n";
    return {};
  }
  for (int i = 0; i < total - 2; ++i)
    if (sa[i] != sb[i]) {
      std::cerr << "BatchedMatmul: A, B dim not matched.\n";
      return {};
    }
  const int64_t m = layoutA == Layout::rowMajor ? sa[total - 2] : sa[total - 1];
  const int64_t k1 = layoutA == Layout::rowMajor ? sa[total - 1] : sa[total - 2];
  const int64_t n = layoutB == Layout::colMajor ? sb[total - 2] : sb[total - 1];
  const int64_t k2 = layoutB == Layout::colMajor ? sb[total - 1] : sb[total - 2];
  if (k1 != k2) {
    std::cerr << "Can't apply BatchedMatmul Operation due to imcompatible K-dim.\n";
    return {};
  }
  DType dt;
  const DType fallback = A.dtype() == DType::f8e4m3 ? DType::bf16 : A.dtype();
  if (!resolve_dtype(dtype_, fallback, dt, "BatchedMatmul")) return {};
  std::vector<int64_t> sc(sa.begin(), sa.end() - 2);
  std::string name = "BatchMatmul" + dims(sc);
  sc.push_back(m);
  sc.push_back(n);
  name += "_m" + std::to_string(m) + "_n" + std::to_string(n) + "_k" + std::to_string(k1) + "_";
  name += layoutA == Layout::rowMajor ? 'N' : 'T';
  name += layoutB == Layout::rowMajor ? 'N' : 'T';
  name += dtype_suffix(A.dtype(), dt);
  OpNode node;
  node.kind = OpKind::BatchedMatmul;
  node.func = name;
  node.inputs = {A.id, B.id};
  node.layoutA = layoutA;
  node.layoutB = layoutB;
  if (out) {
    if (!valid(graph, out, "BatchedMatmul: out is not a tensor of this graph.\n", true)) return {};
    const auto& ot = graph->data->tensors[out.id];
    if (ot.producer >= 0 || ot.shape != sc || ot.dtype != dt) {
      std::cerr << "BatchedMatmul: out must be a PlaceHolder with the result's shape and element type.\n";
      return {};
    }
    const std::vector<int64_t> out_strides = ot.strides;
    Value c = add_op(graph, node, sc, dt, MemorySpace::global, out.id);
    graph->data->tensors[c.id].strides = out_strides;
    return c;
  }
  return add_op(graph, node, sc, dt, MemorySpace::global, -1);
}

// ---- Softmax (reference: Operators.cc:462-578) -------------------------------------------------
Value Softmax::build(ComputeDAG* graph, Value input, int axis, MemorySpace, const std::string& dtype_, float scale,
                     bool causal) {
  if (!valid(graph, input, "Type of input of Softmax is not Memref.\n")) return {};
  const int total = static_cast<int>(input.shape().size());
  if (total < 1) {
    std::cerr << "Illegal reduction axis in Softmax.\n";
    return {};
  }
  if (axis != -1 && (axis < 0 || axis >= total)) {
    std::cerr << "Illegal reduction axis in Softmax.\n";
    return {};
  }
  const int start = axis == -1 ? total - 1 : axis;
  if (total - start != 1) {
    std::cerr << "At present, only support reduction on the last dim.\n";
    return {};
  }
  DType dt;
  if (!resolve_dtype(dtype_, input.dtype(), dt, "Softmax")) return {};
  OpNode node;
  node.kind = OpKind::Softmax;
  node.func = "Softmax" + dims(input.shape()) + "_axis" + std::to_string(start) + dtype_suffix(input.dtype(), input.dtype());
  node.inputs = {input.id};
  node.axis = start;
  node.scale = scale;
  node.causal = causal;
  // always in place: the reference stores into and returns its input buffer (Operators.cc:573)
  return add_op(graph, node, input.shape(), input.dtype(), MemorySpace::inplace, input.id);
}

// The reference declares Transpose with one operand and leaves the body empty
// (Operators.h:97-99, Operators.cc:459-460); here it swaps the two innermost dims.
Value Transpose::build(ComputeDAG* graph, Value input) {
  if (!valid(graph, input, "Type of operand of Transpose is not Memref.\n")) return {};
  const auto& in = input.shape();
  if (in.size() < 2) {
    std::cerr << "Transpose takes an operand of rank 2 or more.\n";
    return {};
  }
  std::vector<int64_t> out = in;
  std::swap(out[out.size() - 1], out[out.size() - 2]);
  OpNode node;
  node.kind = OpKind::Transpose;
  node.func = "Transpose" + dims(in) + dtype_suffix(input.dtype(), input.dtype());
  node.inputs = {input.id};
  return add_op(graph, node, out, input.dtype(), MemorySpace::global, -1);
}

// ---- Binary (reference: Operators.cc:772-889) ---------------------------------------------------
const std::vector<std::string>& Binary::operations() {
  static const std::vector<std::string> ops = {"Add", "Mul", "Div", "Sub", "Pow", "Equal", "Greater"};
  return ops;
}

Value Binary::build(ComputeDAG* graph, Value A, Value B, std::string operation, MemorySpace ms,
                    const std::string& dtype_) {
  if (!valid(graph, A, ("Type of left operand of" + operation + "is not Memref.\n").c_str())) return {};
  if (!valid(graph, B, ("Type of right operand of " + operation + " is not Memref.\n").c_str())) return {};
  const auto& known = operations();
  if (std::find(known.begin(), known.end(), operation) == known.end()) {
    std::cerr << "Unknown Binary operation \"" << operation << "\".\n";
    return {};
  }
  DType dt;
  if (!resolve_dtype(dtype_, A.dtype(), dt, "Binary")) return {};
  if (A.dtype() != B.dtype()) {
    std::cerr << "Binary operands must share an element type.\n";
    return {};
  }
  // broadcast shape: align at the trailing dim; unequal extents need a 1 (Operators.cc:797-821)
  std::vector<int64_t> ra(A.shape().rbegin(), A.shape().rend()), rb(B.shape().rbegin(), B.shape().rend());
  const size_t mn = std::min(ra.size(), rb.size());
  std::vector<int64_t> out;
  for (size_t i = 0; i < mn; ++i) {
    if (ra[i] != rb[i] && ra[i] != 1 && rb[i] != 1) {
      std::cerr << "dim not equal\n";
      return {};
    }
    out.push_back(ra[i] == 1 ? rb[i] : ra[i]);
  }
  const auto& longer = ra.size() >= rb.size() ? ra : rb;
  out.insert(out.end(), longer.begin() + mn, longer.end());
  std::reverse(out.begin(), out.end());
  OpNode node;
  node.kind = OpKind::Binary;
  node.operation = operation;
  node.func = operation + "_Binary" + dims(A.shape()) + "_" + operation + dims(B.shape()) +
              dtype_suffix(A.dtype(), ms == MemorySpace::inplace ? A.dtype() : dt);
  node.inputs = {A.id, B.id};
  int alias = -1;
  if (ms == MemorySpace::inplace) {
    if (out != A.shape()) {
      std::cerr << "Binary: inplace needs the left operand to have the output shape.\n";
      return {};
    }
    alias = A.id;
  }
  return add_op(graph, node, out, ms == MemorySpace::inplace ? A.dtype() : dt, ms, alias);
}

// ---- ElementWise (reference: Operators.cc:960-1074) ----------------------------------------------
const std::vector<std::string>& ElementWise::operations() {
  static const std::vector<std::string> ops = {"Tanh", "Sqrt", "Log", "Relu", "Cast", "Gelu"};
  return ops;
}

Value ElementWise::build(ComputeDAG* graph, Value input, std::string operation, MemorySpace ms,
                         const std::string& dtype_) {
  if (!valid(graph, input, ("Type of operand of " + operation + " is not Memref.\n").c_str())) return {};
  const auto& known = operations();
  if (std::find(known.begin(), known.end(), operation) == known.end()) {
    std::cerr << "Unknown ElementWise operation \"" << operation << "\".\n";
    return {};
  }
  DType dt;
  if (!resolve_dtype(dtype_, input.dtype(), dt, "ElementWise")) return {};
  if (operation != "Cast" && dt != input.dtype()) {
    std::cerr << "ElementWise " << operation << " keeps the element type; only Cast changes it.\n";
    return {};
  }
  if (ms == MemorySpace::inplace && dtypeSize(dt) != dtypeSize(input.dtype())) {
    std::cerr << "ElementWise: an inplace Cast needs element types of equal size.\n";
    return {};
  }
  OpNode node;
  node.kind = OpKind::ElementWise;
  node.operation = operation;
  node.func = operation + "_Elementwise" + dims(input.shape()) + dtype_suffix(input.dtype(), dt);
  node.inputs = {input.id};
  return add_op(graph, node, input.shape(), dt, ms, ms == MemorySpace::inplace ? input.id : -1);
}

// ---- LayerNorm (reference: Operators.cc:1076-1251) -------------------------------------------------
Value LayerNorm::build(ComputeDAG* graph, Value input, Value scale, Value bias, int64_t axis, const float& eps,
                       MemorySpace ms, const std::string& dtype_) {
  if (!valid(graph, input, "Type of operand of LayerNorm is not Memref.\n")) return {};
  if (!valid(graph, scale, "Type of scale of LayerNorm is not Memref.\n")) return {};
  if (!valid(graph, bias, "Type of bias of LayerNorm is not Memref.\n")) return {};
  DType dt;
  if (!resolve_dtype(dtype_, input.dtype(), dt, "LayerNorm")) return {};
  const auto& in = input.shape();
  const int64_t dim = static_cast<int64_t>(in.size());
  auto check = [&](const std::vector<int64_t>& s, const char* what) {
    if (s.size() > in.size()) {
      std::cerr << what << " dim is not equal.\n";
      return false;
    }
    for (size_t i = 0; i < s.size(); ++i)
      if (s[s.size() - 1 - i] != in[in.size() - 1 - i] && s[s.size() - 1 - i] != 1) {
        std::cerr << what << " dim is not equal.\n";
        return false;
      }
    return true;
  };
  if (!check(scale.shape(), "scale") || !check(bias.shape(), "bias")) return {};
  if (axis >= dim || axis <= -dim) {
    std::cerr << "axis is out of bounds for array of dimension.\n";
    return {};
  }
  if (axis < 0) axis += dim;
  if (scale.dtype() != input.dtype() || bias.dtype() != input.dtype()) {
    std::cerr << "LayerNorm: scale and bias must have the input's element type.\n";
    return {};
  }
  OpNode node;
  node.kind = OpKind::LayerNorm;
  node.func = "LayerNorm" + dims(in) + "_axis_" + std::to_string(axis) + dtype_suffix(input.dtype(), input.dtype());
  node.inputs = {input.id, scale.id, bias.id};
  node.axis = axis;
  node.eps = eps;
  return add_op(graph, node, in, input.dtype(), ms, ms == MemorySpace::inplace ? input.id : -1);
}

// ---- Gather (reference: Operators.cc:1253-1352) ------------------------------------------------------
Value Gather::build(ComputeDAG* graph, Value input, Value indices, const std::int64_t& axis, const std::string& dtype_) {
  if (!valid(graph, input, "Type of operand of Gather is not Memref.\n")) return {};
  if (!valid(graph, indices, "Type of operand of Gather is not Memref.\n")) return {};
  const auto& in = input.shape();
  const auto& idx = indices.shape();
  if (axis < 0 || axis >= static_cast<int64_t>(in.size())) {
    std::cerr << "Can't apply Gather Operation due to axis is greater than shape of input.\n";
    return {};
  }
  if (indices.dtype() != DType::i32 && indices.dtype() != DType::i64) {
    std::cerr << "Gather: indices must be int32 or int64 (index).\n";
    return {};
  }
  DType dt;
  if (!resolve_dtype(dtype_, input.dtype(), dt, "Gather")) return {};
  if (dt != input.dtype()) {
    std::cerr << "Gather moves elements; it cannot change the element type.\n";
    return {};
  }
  // the axis is erased and, unless the indices are a single [1] vector, their dims take its place
  std::vector<int64_t> out = in;
  out.erase(out.begin() + axis);
  if (!(idx.size() == 1 && idx[0] == 1)) out.insert(out.begin() + axis, idx.begin(), idx.end());
  OpNode node;
  node.kind = OpKind::Gather;
  std::string name = "Gather";
  for (auto d : in) name += "_" + std::to_string(d);
  name += "_indices";
  for (auto d : idx) name += "_" + std::to_string(d);
  name += "_axis_" + std::to_string(axis);
  name += dtype_suffix(input.dtype(), input.dtype());
  if (indices.dtype() == DType::i32) name += "_idx32";   // the reference's indices are `index` (64-bit)
  node.func = name;
  node.inputs = {input.id, indices.id};
  node.axis = axis;
  return add_op(graph, node, out, input.dtype(), MemorySpace::global, -1);
}

}  // namespace KernelCodeGen
