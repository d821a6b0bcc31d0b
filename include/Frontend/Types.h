// Value types shared by the KernelCodeGen front end: enums that appear in operator
// signatures, the log switch, tensor handles and the recorded graph.
//
// The reference builds its graph as MLIR (memref values, func.func per operator,
// func.call at graph level).  This front end keeps the same user-visible API but records
// the graph as plain C++ data: a tensor table, an operator list and a function table
// keyed by the reference's function names, which is all the dispatch layer needs.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

// Log level (global enum, as user code writes Log::Debug / Log::Release;
// reference: include/log.h).
enum Log {
  Debug = 0,
  Release = 1,
};

namespace KernelCodeGen {

struct KCGLog {
  static Log level;
};

// reference: include/enum.h — the numeric values are part of the API (MemorySpace is
// stored as the memref memory-space attribute there).
enum class Target { CUDA = 0, ROCm = 1 };
enum class MemorySpace { global = 1, shared = 2, local = 3, constant = 4, unallocated = 5, inplace = 6 };
enum class Position { before = 0, after = 1, begin = 2, end = 3 };
enum class Layout { rowMajor = 0, colMajor = 1 };

// Element types accepted by getDType (reference: src/Frontend/Operators.cc:5-15) plus
// "bfloat16" and "float8_e4m3".  Values match enum kcg_dtype of the C ABI.
enum class DType : int {
  f32 = 0, f16 = 1, bf16 = 2, f8e4m3 = 3, i32 = 4, f64 = 5, i64 = 6, i16 = 7, boolean = 8, invalid = -1
};
DType getDType(const std::string& dtype);
std::string toStr(DType type);
size_t dtypeSize(DType type);

struct GraphData;

// Handle to a tensor of a graph.  A default-constructed handle is the "null value" the
// reference returns (as a null mlir::Value) when an operator rejects its arguments.
struct Value {
  int id = -1;
  GraphData* owner = nullptr;
  explicit operator bool() const { return id >= 0; }
  bool operator==(const Value& o) const { return id == o.id && owner == o.owner; }
  const std::vector<int64_t>& shape() const;
  // element strides, one per dim; the dense row-major strides unless the PlaceHolder gave others
  std::vector<int64_t> strides() const;
  DType dtype() const;
  int64_t numel() const;
  size_t bytes() const;
};

struct TensorInfo {
  std::vector<int64_t> shape;
  // Element strides per dim; empty = dense row-major (the only layout the reference has).
  // Extension: a PlaceHolder may declare others, e.g. a [B,H,S,D] view of a [B,S,H,D] buffer.
  std::vector<int64_t> strides;
  bool dense() const;                        // strides are absent or equal to the row-major ones
  std::vector<int64_t> effective_strides() const;
  DType dtype = DType::f32;
  MemorySpace space = MemorySpace::global;
  int producer = -1;       // index into GraphData::ops, -1 for a PlaceHolder
  int alias_of = -1;       // tensor whose storage this one shares (inplace results)
};

enum class OpKind { Matmul, BatchedMatmul, Softmax, LayerNorm, ElementWise, Binary, Gather, Transpose, FusedAttention,
                    FusedLayerNormGeluAdd };

// One recorded operator call (the reference's func.call); `func` names the per-(op, shape)
// function it calls (the reference's func.func symbol).
struct OpNode {
  OpKind kind;
  std::string func;
  std::vector<int> inputs;
  int output = -1;
  // attributes
  std::string operation;               // ElementWise / Binary operation name
  Layout layoutA = Layout::rowMajor, layoutB = Layout::rowMajor;
  int64_t axis = -1;
  float eps = 1e-5f;
  float scale = 1.0f;                  // Softmax / attention extension
  bool causal = false;                 // Softmax / attention extension
  int scale_a = -1, scale_b = -1;      // tensors holding per-tensor fp32 scales (FP8 Matmul)
  int bias = -1;                       // fused GEMM epilogue: tensor of N values added to every row
  std::string activation;              // fused GEMM epilogue: "", "Relu" or "Gelu"
  bool erased = false;                 // consumed by a fusion
};

struct FuncInfo {
  std::string state = "cpu";           // "cpu" as built; "gpu" once an optimizer selected a kernel
  std::string optimizer;               // name of the optimizer that selected it
  std::map<std::string, int> config;   // the optimizer's tile-config table at selection time
};

struct GraphData {
  std::string name;
  std::vector<TensorInfo> tensors;
  std::vector<OpNode> ops;
  std::vector<std::string> func_order;           // creation order, newest first like the reference module
  std::map<std::string, FuncInfo> funcs;
  int users(int tensor) const;                   // number of live ops reading `tensor`
  int root(int tensor) const;                    // storage owner after following alias_of
};

}  // namespace KernelCodeGen
