// Optimizers: in the reference each one pattern-matches functions by name and rewrites
// their loop nests into a GPU schedule (include/Optimizer/Optimizer.h:29-286).  Here the
// schedules are the hand-written sm_100a kernels, so an optimizer only SELECTS: `applicable`
// finds the functions of its family that are still tagged "cpu", `applyOptimzer` tags them
// "gpu" and records the kernel that will run them.  The static tile-config maps are kept
// (KernelCodeGenerator fills them from its tables) and recorded with the selection; they are
// per host thread, so generators on different threads can optimize at the same time.
#pragma once

#include <map>
#include <string>
#include <vector>

#include "Frontend/Operators.h"

namespace KernelCodeGen {

struct Module;      // defined in KernelCodeGen.h
struct OpBuilder {};  // placeholder for the reference's mlir::OpBuilder parameter

struct Optimizer {
  virtual ~Optimizer() = default;
  virtual bool applicable(Module& module) = 0;
  virtual void applyOptimzer(Module& module, OpBuilder& builder) = 0;
  bool operator==(const Optimizer& other) { return name == other.name; }
  std::string name;

 protected:
  // functions whose name contains `needle` (and not `exclude`) and that are still "cpu"
  std::vector<std::string> collect(Module& module, const std::string& needle, const std::string& exclude = "");
  void select(Module& module, const std::vector<std::string>& funcs, const std::map<std::string, int>& config);
  std::vector<std::string> matched;
};

#define KCG_DECLARE_OPTIMIZER(Class, Name, configMember)                 \
  struct Class : Optimizer {                                             \
    Class() { this->name = Name; }                                       \
    bool applicable(Module& module) override;                            \
    void applyOptimzer(Module& module, OpBuilder& builder) override;     \
    static thread_local std::map<std::string, int> configMember;         \
  }

KCG_DECLARE_OPTIMIZER(MatmulOptimizer, "Matmul", matmulConfig);
KCG_DECLARE_OPTIMIZER(BinaryOptimizer, "Binary", binaryConfig);
KCG_DECLARE_OPTIMIZER(ElementWiseOptimizer, "ElementWise", elementWiseConfig);
KCG_DECLARE_OPTIMIZER(LayerNormOptimizer, "LayerNorm", layerNormConfig);
KCG_DECLARE_OPTIMIZER(GatherOptimizer, "Gather", gatherConfig);
KCG_DECLARE_OPTIMIZER(BatchMatmulOptimizer, "BatchMatmul", batchMatmulConfig);
// Extension: the reference has no stand-alone softmax schedule (softmax only exists fused).
KCG_DECLARE_OPTIMIZER(SoftmaxOptimizer, "Softmax", softmaxConfig);
// Extension: Transpose is declared by the reference without a body or a schedule.
KCG_DECLARE_OPTIMIZER(TransposeOptimizer, "Transpose", transposeConfig);

// Finds BatchMatmul(NT) -> Softmax -> BatchMatmul(NN) chains whose intermediate results have
// a single user (reference: src/Optimizer/Optimizer.cc:2113-2199) and replaces each by one
// Fused_Multi_Head_Attention call.
struct FMHAOptimizer : Optimizer {
  FMHAOptimizer() { this->name = "FMHA"; }
  bool applicable(Module& module) override;
  void applyOptimzer(Module& module, OpBuilder& builder) override;
  static thread_local std::map<std::string, int> fmhaConfig;

 private:
  struct Chain { int qk, softmax, pv; };
  std::vector<Chain> chains;
};

// The "KernelFusion Optimizer" of the reference's roadmap (doc/Plan.md:68, :110; not implemented
// there).  Two patterns, both requiring every intermediate to have a single user:
//   Matmul / BatchedMatmul [-> Binary "Add" with an [N] bias] [-> Relu | ElementWise "Relu"/"Gelu"]
//       becomes one GEMM launch with a fused epilogue (test/test.cc:62-63 is Matmul -> Relu);
//   LayerNorm (last dim) -> ElementWise "Gelu" -> Binary "Add" with a same-shape tensor
//       becomes one pass over memory.
// Push it before the family optimizers so that it sees the chains still unselected.
struct KernelFusionOptimizer : Optimizer {
  KernelFusionOptimizer() { this->name = "KernelFusion"; }
  bool applicable(Module& module) override;
  void applyOptimzer(Module& module, OpBuilder& builder) override;
  static thread_local std::map<std::string, int> fusionConfig;

 private:
  struct GemmChain { int gemm, add, act; };     // op indices, -1 where absent
  struct LnChain { int ln, gelu, add; };
  std::vector<GemmChain> gemm_chains;
  std::vector<LnChain> ln_chains;
};

#undef KCG_DECLARE_OPTIMIZER

}  // namespace KernelCodeGen
