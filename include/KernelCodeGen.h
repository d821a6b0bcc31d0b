// KernelCodeGenerator: the session object of the reference API (include/KernelCodeGen.h:25-165)
// over the sm_100a kernel library.
//
//   KernelCodeGenerator generator("CUDA");
//   auto graph = generator.createGraph("demo");
//   generator.opts.push_back(std::make_unique<MatmulOptimizer>());
//   auto A = graph.create<PlaceHolder>(std::vector<int64_t>{m, k}, std::string{"bfloat16"});
//   auto B = graph.create<PlaceHolder>(std::vector<int64_t>{k, n}, std::string{"bfloat16"});
//   auto C = graph.create<Matmul>(A, B);
//   auto module = generator.optimize(graph);
//   auto plan = generator.codegen(module);                  // text: the dispatch plan
//   Bindings bind; bind.set(A, dA); bind.set(B, dB); bind.set(C, dC);
//   int status = generator.run(module, bind, stream);       // launches the kernels
//
// `run` is the one addition: the reference stops at source text and leaves compiling and
// launching to an external harness.
#pragma once

#include <cfloat>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "Backend/CUDA.h"
#include "Frontend/Operators.h"
#include "Optimizer/Optimizer.h"

namespace KernelCodeGen {

// One kernel launch of the plan.
struct KernelCall {
  OpKind kind;
  std::string func;        // reference-style function name this launch implements
  std::string entry;       // C-ABI entry point
  int op = -1;             // index into GraphData::ops
};

// The optimized module: a private copy of the graph plus the launches selected for it.
struct Module {
  std::shared_ptr<GraphData> graph;
  std::vector<KernelCall> calls;   // rebuilt by KernelCodeGenerator::optimize
  void dump() const;               // prints functions (with their cpu/gpu tag) and calls to stderr
};

// Device pointers for the tensors of a graph.  The caller owns every buffer, inputs,
// outputs and intermediates alike; in-place results share their input's pointer.
struct Bindings {
  void set(Value v, void* device_ptr) { ptrs[v.id] = device_ptr; }
  void* get(int id) const {
    auto it = ptrs.find(id);
    return it == ptrs.end() ? nullptr : it->second;
  }
  std::map<int, void*> ptrs;
};

// How run() splits a module over the GPUs of one node (one process per GPU; extension, the
// reference is single-GPU).  Every operator is cut along its independent units — Matmul rows of
// A / C in granules of 128, BatchedMatmul and attention batches, LayerNorm / Softmax / elementwise
// rows — by kcg_shard_range; rank `rank` of `world` launches the ordinary kernel on its block
// only.  Buffers are bound at FULL size on every rank (inputs replicated).  With `gather` the
// output of each sharded operator is all-gathered in place over `nccl_comm` (an ncclComm_t) on
// the same stream, so every rank ends with the whole tensor and later operators may read all of
// it; without it a rank's buffer holds its own block only (enough for a chain of row-wise
// operators, which all cut the rows the same way).  Operators with no row-like unit (Gather,
// a 2-D Transpose, a Binary that broadcasts along dim 0) run whole on every rank.
struct ShardSpec {
  int world = 1;
  int rank = 0;
  void* nccl_comm = nullptr;
  bool gather = false;
};

class KernelCodeGenerator {
 public:
  KernelCodeGenerator(const std::string& platform_ = {"CUDA"});
  KernelCodeGenerator() = delete;

  ComputeDAG& createGraph(const std::string& graphName);
  ComputeDAG& getGraph() { return graph; }

  void dump(Module& module, const std::string& info = "");
  // Writes `str` to `file`, or to stdout when file == "terminal".
  void save(const std::string& str, const std::string& file);

  void resetModule(Module& module);
  void backupModule(Module& module);
  void saveBestModule(Module& module);

  // Applies every optimizer in `opts`, once per entry of its family's config table, and
  // returns the best module (reference: src/KernelCodeGen.cc:8-120).
  Module& optimize(ComputeDAG& graph_);

  // Latency of a candidate module.  With `autotune` off (the default) it returns 0 like the
  // reference (include/KernelCodeGen.h:134-136), so the first config of each table wins.  With
  // `autotune` on and a GPU present it runs the module's selected kernels on scratch buffers
  // (zero-filled, allocated and freed here) and returns the mean device time in milliseconds.
  float evaluate(Module& module);

  // Candidate tile/variant configurations of one optimizer family ("Matmul", "BatchMatmul",
  // "LayerNorm", "FMHA", ...); optimize() tries each entry in turn.  Empty name -> nullptr.
  std::vector<std::map<std::string, int>>* configs(const std::string& family);

  std::string codegen(Module module);

  // Launches the module's kernels in order on `stream` (a cudaStream_t).  Every tensor a
  // launch touches must be bound.  Returns a kcg_status; functions no optimizer selected
  // are an error (there is no CPU execution path).
  int run(Module& module, const Bindings& bindings, void* stream = nullptr);
  // The same, sharded over the ranks `shard` describes (see ShardSpec).  Collective when
  // shard.gather is set: every rank calls it with the same module.
  int run(Module& module, const Bindings& bindings, const ShardSpec& shard, void* stream = nullptr);

  // Time every candidate config on the device inside optimize() (see evaluate()).
  bool autotune = false;
  // Latency evaluate() returned for the candidate the last optimizer kept (0 without autotuning).
  float bestLatency() const { return minLatency; }

  void setLogMode(Log level) { KCGLog::level = level; }

 public:
  std::vector<std::unique_ptr<Optimizer>> opts;

 private:
  Module backupModule_;
  Module bestModule;
  ComputeDAG graph;
  std::string platform;
  float minLatency = FLT_MAX;
  int runSelected(Module& module, const Bindings& bindings, void* stream, bool skipUnselected,
                  const ShardSpec* shard = nullptr);
  std::vector<std::map<std::string, int>> matmulConfigs, fmhaConfigs, binaryConfigs, elementWiseConfigs,
      gatherConfigs, layerNormConfigs, batchMatmulConfigs, softmaxConfigs, fusionConfigs;
};

}  // namespace KernelCodeGen
