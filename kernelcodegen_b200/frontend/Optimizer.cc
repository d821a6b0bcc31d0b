// Optimizers as kernel selectors.  Matching follows the reference: functions are found by
// substring of their name (Analyzer::collectFunctions, src/Optimizer/Analyzer.cc:62-74),
// "Matmul" skips names containing "BatchMatmul" (src/Optimizer/Optimizer.cc:243-256), and
// the attention chain is recognised structurally (src/Optimizer/Optimizer.cc:2113-2199).
#include "KernelCodeGen.h"

#include <iostream>

namespace KernelCodeGen {

thread_local std::map<std::string, int> MatmulOptimizer::matmulConfig;
thread_local std::map<std::string, int> FMHAOptimizer::fmhaConfig;
thread_local std::map<std::string, int> BinaryOptimizer::binaryConfig;
thread_local std::map<std::string, int> ElementWiseOptimizer::elementWiseConfig;
thread_local std::map<std::string, int> LayerNormOptimizer::layerNormConfig;
thread_local std::map<std::string, int> GatherOptimizer::gatherConfig;
thread_local std::map<std::string, int> TransposeOptimizer::transposeConfig;
thread_local std::map<std::string, int> BatchMatmulOptimizer::batchMatmulConfig;
thread_local std::map<std::string, int> SoftmaxOptimizer::softmaxConfig;

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
KCG_SIMPLE_OPTIMIZER(GatherOptimizer, "Gather", "", gatherConfig)
KCG_SIMPLE_OPTIMIZER(TransposeOptimizer, "Transpose", "", transposeConfig)
#undef KCG_SIMPLE_OPTIMIZER

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
    // the kernel addresses each tensor as base + b*s0 + h*s1 + s*s2 + d: any strides whose
    // innermost is 1 and whose others are multiples of 8 elements (16-byte rows for TMA)
    auto strides_ok = [](const TensorInfo& t) {
      for (size_t d = 0; d + 1 < t.strides.size(); ++d)
        if (t.strides[d] % 8 != 0) return false;
      return true;
    };
    const auto& o = g.tensors[pv.output];
    const bool kernel_ok = (q.dtype == DType::bf16 || q.dtype == DType::f16) && k.dtype == q.dtype &&
                           v.dtype == q.dtype && (hd == 64 || hd == 128) && v.shape[r - 1] == hd &&
                           o.dtype == q.dtype && strides_ok(q) && strides_ok(k) && strides_ok(v) && strides_ok(o) &&
                           g.tensors[qk.output].dense() && g.tensors[g.ops[si].output].dense();
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
    fused.func += "_SL" + std::to_string(q.shape[r - 2]) + "_HD" + std::to_string(q.shape[r - 1]) + "_" + toStr(q.dtype);
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

// ---------------------------------------------------------------------------- KernelFusion
namespace KernelCodeGen {

thread_local std::map<std::string, int> KernelFusionOptimizer::fusionConfig;

namespace {
// The single live op that reads `tensor` as its first input, or -1 (also -1 when the tensor has
// more than one reader: a second reader needs the intermediate in memory).
int sole_consumer(const GraphData& g, int tensor) {
  if (g.users(tensor) != 1) return -1;
  for (int j = 0; j < static_cast<int>(g.ops.size()); ++j) {
    const OpNode& op = g.ops[j];
    if (op.erased) continue;
    for (int in : op.inputs)
      if (in == tensor) return j;
  }
  return -1;
}
}  // namespace

bool KernelFusionOptimizer::applicable(Module& module) {
  gemm_chains.clear();
  ln_chains.clear();
  auto& g = *module.graph;
  auto cpu = [&](int op) { return op >= 0 && g.funcs[g.ops[op].func].state == "cpu"; };
  for (int i = 0; i < static_cast<int>(g.ops.size()); ++i) {
    const OpNode& op = g.ops[i];
    if (op.erased || !cpu(i)) continue;
    if (op.kind == OpKind::Matmul || op.kind == OpKind::BatchedMatmul) {
      if (op.bias >= 0 || !op.activation.empty()) continue;  // already fused
      GemmChain c{i, -1, -1};
      int tail = op.output;
      const int64_t n = g.tensors[op.output].shape.back();
      int next = sole_consumer(g, tail);
      if (cpu(next) && g.ops[next].kind == OpKind::Binary && g.ops[next].operation == "Add" &&
          g.ops[next].inputs[0] == tail) {
        const auto& bias = g.tensors[g.ops[next].inputs[1]];
        if (bias.shape.size() == 1 && bias.shape[0] == n && bias.dtype == g.tensors[tail].dtype &&
            g.tensors[g.ops[next].output].shape == g.tensors[tail].shape) {
          c.add = next;
          tail = g.ops[next].output;
          next = sole_consumer(g, tail);
        }
      }
      if (cpu(next) && g.ops[next].kind == OpKind::ElementWise && g.ops[next].inputs[0] == tail &&
          (g.ops[next].operation == "Relu" || g.ops[next].operation == "Gelu") &&
          g.tensors[g.ops[next].output].dtype == g.tensors[tail].dtype)
        c.act = next;
      if (c.add >= 0 || c.act >= 0) gemm_chains.push_back(c);
    } else if (op.kind == OpKind::LayerNorm) {
      const auto& x = g.tensors[op.inputs[0]];
      if (op.axis != static_cast<int64_t>(x.shape.size()) - 1) continue;
      const int64_t cols = x.shape.back();
      const auto& sc = g.tensors[op.inputs[1]];
      const auto& bi = g.tensors[op.inputs[2]];
      if (sc.shape != std::vector<int64_t>{cols} || bi.shape != std::vector<int64_t>{cols}) continue;
      const int ge = sole_consumer(g, op.output);
      if (!cpu(ge) || g.ops[ge].kind != OpKind::ElementWise || g.ops[ge].operation != "Gelu") continue;
      const int ad = sole_consumer(g, g.ops[ge].output);
      if (!cpu(ad) || g.ops[ad].kind != OpKind::Binary || g.ops[ad].operation != "Add") continue;
      const OpNode& add = g.ops[ad];
      const int other = add.inputs[0] == g.ops[ge].output ? add.inputs[1] : add.inputs[0];
      if (other == g.ops[ge].output) continue;  // y + y
      if (g.tensors[other].shape != x.shape || g.tensors[other].dtype != x.dtype) continue;
      // Rows the one-pass kernel does not take (not a whole number of 16-byte vectors, or more
      // than 4096 of them) run as three launches in place in the output, which then must not be
      // the residual's own storage (an inplace Add on the residual): leave that chain unfused.
      const int64_t vw = 16 / static_cast<int64_t>(dtypeSize(x.dtype));
      const bool one_pass = cols % vw == 0 && cols / vw <= 4096;
      if (!one_pass && g.root(add.output) == g.root(other)) continue;
      ln_chains.push_back({i, ge, ad});
    }
  }
  return !gemm_chains.empty() || !ln_chains.empty();
}

void KernelFusionOptimizer::applyOptimzer(Module& module, OpBuilder&) {
  auto& g = *module.graph;
  auto add_func = [&](const std::string& name) {
    if (!g.funcs.count(name)) g.func_order.insert(g.func_order.begin(), name);
    auto& info = g.funcs[name];
    info.state = "gpu";
    info.optimizer = this->name;
    info.config = fusionConfig;
  };
  for (const auto& c : gemm_chains) {
    OpNode fused = g.ops[c.gemm];
    const int last = c.act >= 0 ? c.act : c.add;
    fused.func = "Fused_" + g.ops[c.gemm].func;
    if (c.add >= 0) {
      fused.bias = g.ops[c.add].inputs[1];
      fused.inputs.push_back(fused.bias);
      fused.func += "_Bias";
    }
    if (c.act >= 0) {
      fused.activation = g.ops[c.act].operation;
      fused.func += "_" + fused.activation;
    }
    // the fused launch writes the last tensor of the chain; an in-place result keeps naming the
    // storage of the tensor it was a view of, so a pointer bound to either handle is found
    fused.output = g.ops[last].output;
    g.tensors[fused.output].producer = last;
    g.ops[c.gemm].erased = true;
    if (c.add >= 0) g.ops[c.add].erased = true;
    if (c.act >= 0) g.ops[c.act].erased = true;
    g.ops[last] = fused;
    add_func(fused.func);
  }
  for (const auto& c : ln_chains) {
    const OpNode& ln = g.ops[c.ln];
    const OpNode& add = g.ops[c.add];
    OpNode fused = ln;
    fused.kind = OpKind::FusedLayerNormGeluAdd;
    fused.func = "Fused_" + ln.func + "_Gelu_Add";
    const int other = add.inputs[0] == g.ops[c.gelu].output ? add.inputs[1] : add.inputs[0];
    fused.inputs = {ln.inputs[0], ln.inputs[1], ln.inputs[2], other};
    fused.output = add.output;
    g.tensors[fused.output].producer = c.add;
    g.ops[c.ln].erased = true;
    g.ops[c.gelu].erased = true;
    g.ops[c.add] = fused;
    add_func(fused.func);
  }
  // functions that lost their last caller disappear
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
