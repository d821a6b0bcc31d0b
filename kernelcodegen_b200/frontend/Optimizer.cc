// Optimizers as kernel selectors.  Matching follows the reference: functions are found by
// substring of their name (Analyzer::collectFunctions, src/Optimizer/Analyzer.cc:62-74),
// "Matmul" skips names containing "BatchMatmul" (src/Optimizer/Optimizer.cc:243-256), and
// the attention chain is recognised structurally (src/Optimizer/Optimizer.cc:2113-2199).
#include "KernelCodeGen.h"

#include <iostream>

namespace KernelCodeGen {

std::map<std::string, int> MatmulOptimizer::matmulConfig;
std::map<std::string, int> FMHAOptimizer::fmhaConfig;
std::map<std::string, int> BinaryOptimizer::binaryConfig;
std::map<std::string, int> ElementWiseOptimizer::elementWiseConfig;
std::map<std::string, int> LayerNormOptimizer::layerNormConfig;
std::map<std::string, int> GatherOptimizer::gatherConfig;
std::map<std::string, int> BatchMatmulOptimizer::batchMatmulConfig;
std::map<std::string, int> SoftmaxOptimizer::softmaxConfig;

std::vector<std::string> Optimizer::collect(Module& module, const std::string& needle, const std::string& exclude) {
  std::vector<std::string> out;
  for (const auto& name : module.graph->func_order) {
    if (name.find(needle) == std::string::npos) continue;
    if (!exclude.empty() && name.find(exclude) != std::string::npos) continue;
    if (module.graph->funcs[name].state != "cpu") continue;
    out.push_back(name);
  }
  return out;
}

void Optimizer::select(Module& module, const std::vector<std::string>& funcs, const std::map<std::string, int>& config) {
  for (const auto& f : funcs) {
    auto& info = module.graph->funcs[f];
    info.state = "gpu";
    info.optimizer = name;
    info.config = config;
  }
}

#define KCG_SIMPLE_OPTIMIZER(Class, needle, exclude, configMember)                          \
  bool Class::applicable(Module& module) {                                                  \
    matched = collect(module, needle, exclude);                                             \
    return !matched.empty();                                                                \
  }                                                                                         \
  void Class::applyOptimzer(Module& module, OpBuilder&) { select(module, matched, configMember); }

KCG_SIMPLE_OPTIMIZER(MatmulOptimizer, "Matmul", "BatchMatmul", matmulConfig)
KCG_SIMPLE_OPTIMIZER(BinaryOptimizer, "Binary", "", binaryConfig)
KCG_SIMPLE_OPTIMIZER(ElementWiseOptimizer, "Elementwise", "", elementWiseConfig)
KCG_SIMPLE_OPTIMIZER(LayerNormOptimizer, "LayerNorm", "", layerNormConfig)
KCG_SIMPLE_OPTIMIZER(BatchMatmulOptimizer, "BatchMatmul", "", batchMatmulConfig)
KCG_SIMPLE_OPTIMIZER(SoftmaxOptimizer, "Softmax", "", softmaxConfig)
#undef KCG_SIMPLE_OPTIMIZER

// No Gather kernel exists in this library, so there is never anything to select.
bool GatherOptimizer::applicable(Module&) { return false; }
void GatherOptimizer::applyOptimzer(Module&, OpBuilder&) {}

bool FMHAOptimizer::applicable(Module& module) {
  chains.clear();
  auto& g = *module.graph;
  auto cpu = [&](const OpNode& op) { return g.funcs[op.func].state == "cpu"; };
  for (int i = 0; i < static_cast<int>(g.ops.size()); ++i) {
    const OpNode& qk = g.ops[i];
    if (qk.erased || qk.kind != OpKind::BatchedMatmul || !cpu(qk)) continue;
    if (qk.layoutA != Layout::rowMajor || qk.layoutB != Layout::colMajor) continue;
    if (g.users(qk.output) != 1) continue;
    int si = -1, pi = -1;
    for (int j = 0; j < static_cast<int>(g.ops.size()); ++j) {
      const OpNode& op = g.ops[j];
      if (!op.erased && !op.inputs.empty() && op.inputs[0] == qk.output && op.kind == OpKind::Softmax) si = j;
    }
    if (si < 0 || !cpu(g.ops[si]) || g.users(g.ops[si].output) != 1) continue;
    for (int j = 0; j < static_cast<int>(g.ops.size()); ++j) {
      const OpNode& op = g.ops[j];
      if (!op.erased && op.kind == OpKind::BatchedMatmul && !op.inputs.empty() && op.inputs[0] == g.ops[si].output) pi = j;
    }
    if (pi < 0 || !cpu(g.ops[pi])) continue;
    const OpNode& pv = g.ops[pi];
    if (pv.layoutA != Layout::rowMajor || pv.layoutB != Layout::rowMajor) continue;
    const auto& q = g.tensors[qk.inputs[0]];
    const auto& k = g.tensors[qk.inputs[1]];
    const auto& v = g.tensors[pv.inputs[1]];
    const size_t r = q.shape.size();
    if (r < 3 || r > 4 || k.shape.size() != r || v.shape.size() != r) continue;
    // same batch, m1 == m2, n1 == k2 (reference: Optimizer.cc:2177-2180)
    bool same = true;
    for (size_t d = 0; d + 2 < r; ++d) same = same && q.shape[d] == k.shape[d] && q.shape[d] == v.shape[d];
    if (!same || k.shape[r - 2] != v.shape[r - 2]) continue;
    const int64_t hd = q.shape[r - 1];
    const bool kernel_ok = (q.dtype == DType::bf16 || q.dtype == DType::f16) && k.dtype == q.dtype &&
                           v.dtype == q.dtype && (hd == 64 || hd == 128) && v.shape[r - 1] == hd &&
                           g.tensors[pv.output].dtype == q.dtype;
    if (!kernel_ok) {
      if (KCGLog::level == Log::Debug)
        std::cerr << "FMHA: chain at @" << qk.func << " left unfused (the fused kernel takes bfloat16/float16 with "
                     "head dimension 64 or 128)\n";
      continue;
    }
    chains.push_back({i, si, pi});
  }
  return !chains.empty();
}

void FMHAOptimizer::applyOptimzer(Module& module, OpBuilder&) {
  auto& g = *module.graph;
  for (const auto& c : chains) {
    OpNode& qk = g.ops[c.qk];
    OpNode& sm = g.ops[c.softmax];
    OpNode& pv = g.ops[c.pv];
    const auto& q = g.tensors[qk.inputs[0]];
    const size_t r = q.shape.size();
    OpNode fused;
    fused.kind = OpKind::FusedAttention;
    fused.func = "Fused_Multi_Head_Attention";
    for (size_t d = 0; d + 2 < r; ++d) fused.func += "_" + std::to_string(q.shape[d]);
    fused.func += "_SL" + std::to_string(q.shape[r - 2]) + "_HD" + std::to_string(q.shape[r - 1]);
    fused.inputs = {qk.inputs[0], qk.inputs[1], pv.inputs[1]};
    fused.output = pv.output;
    fused.scale = sm.scale;
    fused.causal = sm.causal;
    g.tensors[fused.output].producer = c.pv;
    qk.erased = true;
    sm.erased = true;
    if (!g.funcs.count(fused.func)) g.func_order.insert(g.func_order.begin(), fused.func);
    auto& info = g.funcs[fused.func];
    info.state = "gpu";
    info.optimizer = name;
    info.config = fmhaConfig;
    pv = fused;  // the fused call takes the place of the last call of the chain
  }
  // functions that lost their last caller disappear, as the reference erases the three calls
  for (auto it = g.func_order.begin(); it != g.func_order.end();) {
    bool used = false;
    for (const auto& op : g.ops) used = used || (!op.erased && op.func == *it);
    if (!used) {
      g.funcs.erase(*it);
      it = g.func_order.erase(it);
    } else {
      ++it;
    }
  }
}

}  // namespace KernelCodeGen
