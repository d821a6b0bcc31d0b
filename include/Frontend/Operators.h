// Graph builder: ComputeDAG and the operator structs, with the parameter lists and
// defaults of the reference (include/Frontend/Operators.h:17-133).  `build` returns a
// tensor handle; on invalid arguments it prints the reference's message to stderr and
// returns a null handle, as the reference does.
#pragma once

#include <string>
#include <utility>
#include <vector>

#include "Frontend/Types.h"

namespace KernelCodeGen {

// Builds the graph and holds it.  Copies share the same recorded graph, so a copy taken
// from KernelCodeGenerator::createGraph stays a valid view (the reference's test does that).
struct ComputeDAG {
  ComputeDAG() = default;
  template <typename OperatorType, typename... Args>
  Value create(Args&&... args) {
    return OperatorType::build(this, std::forward<Args>(args)...);
  }
  // Prints the recorded graph to stderr in Debug mode (reference: Operators.h:34-44).
  void dump(const std::string& info = "");
  std::shared_ptr<GraphData> data;
};

// Interface to define operators (reference: Operators.h:66-72).
template <typename T>
struct Operator {
  template <typename... Args>
  static Value build(ComputeDAG* graph, Args&&... args) {
    return T::build(graph, std::forward<Args>(args)...);
  }
};

struct PlaceHolder : Operator<PlaceHolder> {
  // `strides` (extension; elements, one per dim, innermost must be 1) declares a tensor that is
  // not dense row-major, e.g. shape [B,H,S,D] with strides {S*H*D, D, H*D, 1} for data stored as
  // [B,S,H,D].  Empty (the default) is the reference's dense layout.  Strided tensors are
  // accepted by BatchedMatmul only (the attention chain); every other operator refuses them.
  static Value build(ComputeDAG* graph, const std::vector<int64_t>& shapes, const std::string& dtype,
                     const std::vector<int64_t>& strides = {});
};

struct Matmul : Operator<Matmul> {
  static Value build(ComputeDAG* graph, Value A, Value B, const std::string& dtype = {""});
  // Old call sites pass a MemorySpace third (reference: test/test.cc:89).
  static Value build(ComputeDAG* graph, Value A, Value B, MemorySpace ms, const std::string& dtype = {""});
  // Extension: FP8 inputs with per-tensor fp32 scales (one-element float32 tensors).
  static Value build(ComputeDAG* graph, Value A, Value B, Value scaleA, Value scaleB, const std::string& dtype);
};

struct Relu : Operator<Relu> {
  static Value build(ComputeDAG* graph, Value input, MemorySpace ms, const std::string& dtype = {""});
};

struct BatchedMatmul : Operator<BatchedMatmul> {
  // `out` (extension): a PlaceHolder of the result's shape and element type to write into, which
  // is how a result gets a layout of its own (the reference allocates C itself, dense).  The
  // returned handle names out's storage.
  static Value build(ComputeDAG* graph, Value A, Layout layoutA, Value B, Layout layoutB,
                     const std::string& dtype = {""}, Value out = {});
};

// Softmax over the last dim, always in place (the reference returns its input buffer).
// `scale` and `causal` are extensions with neutral defaults.
struct Softmax : Operator<Softmax> {
  static Value build(ComputeDAG* graph, Value input, int axis = -1, MemorySpace ms = MemorySpace::global,
                     const std::string& dtype = {""}, float scale = 1.0f, bool causal = false);
};

struct Transpose : Operator<Transpose> {
  static Value build(ComputeDAG* graph, Value input);  // declared but empty in the reference
};

struct Binary : Operator<Binary> {
  static Value build(ComputeDAG* graph, Value A, Value B, std::string operation,
                     MemorySpace ms = MemorySpace::global, const std::string& dtype = {""});
  static const std::vector<std::string>& operations();  // keys of the reference's operationMap
};

struct ElementWise : Operator<ElementWise> {
  static Value build(ComputeDAG* graph, Value input, std::string operation, MemorySpace ms,
                     const std::string& dtype = {""});
  static const std::vector<std::string>& operations();
};

struct LayerNorm : Operator<LayerNorm> {
  static Value build(ComputeDAG* graph, Value input, Value scale, Value bias, int64_t axis,
                     const float& eps = 1e-5, MemorySpace ms = MemorySpace::global, const std::string& dtype_ = {""});
};

struct Gather : Operator<Gather> {
  static Value build(ComputeDAG* graph, Value input, Value indices, const std::int64_t& axis = 0,
                     const std::string& dtype_ = {""});  // out = take(input, indices, axis); runs kcg_gather
};

}  // namespace KernelCodeGen
