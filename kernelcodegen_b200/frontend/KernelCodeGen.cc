// KernelCodeGenerator: config tables, the optimize() sweep, the textual plan and run().
#include "KernelCodeGen.h"

#include <fstream>
#include <iostream>
#include <sstream>

#include "kcg_kernels.h"

namespace KernelCodeGen {

namespace {

std::shared_ptr<GraphData> clone(const std::shared_ptr<GraphData>& g) {
  return g ? std::make_shared<GraphData>(*g) : nullptr;
}

const char* entry_for(OpKind k) {
  switch (k) {
    case OpKind::Matmul: case OpKind::BatchedMatmul: return "kcg_gemm";
    case OpKind::Softmax: return "kcg_softmax";
    case OpKind::LayerNorm: return "kcg_layernorm";
    case OpKind::ElementWise: return "kcg_eltwise";
    case OpKind::Binary: return "kcg_binary";
    case OpKind::Gather: return "kcg_gather";
    case OpKind::Transpose: return "kcg_transpose";
    case OpKind::FusedAttention: return "kcg_fmha_fwd";
    case OpKind::FusedLayerNormGeluAdd: return "kcg_layernorm_gelu_add";
  }
  return "?";
}

void rebuild_calls(Module& m) {
  m.calls.clear();
  if (!m.graph) return;
  for (int i = 0; i < static_cast<int>(m.graph->ops.size()); ++i) {
    const auto& op = m.graph->ops[i];
    if (op.erased) continue;
    m.calls.push_back({op.kind, op.func, entry_for(op.kind), i});
  }
}

std::string shape_str(const std::vector<int64_t>& s) {
  std::string r = "[";
  for (size_t i = 0; i < s.size(); ++i) r += (i ? "," : "") + std::to_string(s[i]);
  return r + "]";
}

int act_code(const std::string& a) { return a == "Relu" ? 1 : (a == "Gelu" ? 2 : 0); }

int index_of(const std::vector<std::string>& v, const std::string& s) {
  for (size_t i = 0; i < v.size(); ++i)
    if (v[i] == s) return static_cast<int>(i);
  return -1;
}

}  // namespace

void Module::dump() const {
  if (!graph) return;
  std::cerr << "module @" << graph->name << " {\n";
  for (const auto& f : graph->func_order) {
    const auto& info = graph->funcs.at(f);
    std::cerr << "  func @" << f << " {func.state = \"" << info.state << "\"";
    if (!info.optimizer.empty()) std::cerr << ", optimizer = \"" << info.optimizer << "\"";
    std::cerr << "}\n";
  }
  for (const auto& c : calls) std::cerr << "  launch " << c.entry << " for @" << c.func << "\n";
  std::cerr << "}\n";
}

KernelCodeGenerator::KernelCodeGenerator(const std::string& platform_) : platform(platform_) {
  // Default tile-config tables with the reference's keys (include/KernelCodeGen.h:35-58).  The
  // matmul / fmha entries describe the sm_100a kernels: CTA tile, k-block, ring depth.
  // Candidates differ in the keys the kernels really switch on: CTA_PAIR (256x256 tiles on two
  // SMs with cta_group::2, or 128x256 on one), WARP_ROW_VECS (LayerNorm rows of up to 32*v
  // 16-byte vectors are handled by one warp), VARIANT (attention data path).
  matmulConfigs = {{{"BLOCK_SIZE_M", 256}, {"BLOCK_SIZE_N", 256}, {"BLOCK_SIZE_K", 64}, {"GROUP_SIZE_M", 8},
                    {"STAGES", 6}, {"ACCUMULATORS", 2}, {"WARP_SIZE", 32}, {"CTA_PAIR", 1}},
                   {{"BLOCK_SIZE_M", 128}, {"BLOCK_SIZE_N", 256}, {"BLOCK_SIZE_K", 64}, {"GROUP_SIZE_M", 16},
                    {"STAGES", 4}, {"ACCUMULATORS", 2}, {"WARP_SIZE", 32}, {"CTA_PAIR", 0}},
                   {{"BLOCK_SIZE_M", 128}, {"BLOCK_SIZE_N", 128}, {"BLOCK_SIZE_K", 64}, {"GROUP_SIZE_M", 16},
                    {"STAGES", 6}, {"ACCUMULATORS", 2}, {"WARP_SIZE", 32}, {"CTA_PAIR", 0}},
                   {{"BLOCK_SIZE_M", 128}, {"BLOCK_SIZE_N", 64}, {"BLOCK_SIZE_K", 64}, {"GROUP_SIZE_M", 16},
                    {"STAGES", 8}, {"ACCUMULATORS", 2}, {"WARP_SIZE", 32}, {"CTA_PAIR", 0}}};
  batchMatmulConfigs = matmulConfigs;
  binaryConfigs = {{{"BLOCK_SIZE", 256}, {"UNROLL", 4}, {"VECTORIZE_WIDTH", 16}}};
  elementWiseConfigs = {{{"BLOCK_SIZE", 256}, {"UNROLL", 4}, {"VECTORIZE_WIDTH", 16}}};
  // THREAD_VECS 0: the library picks the vectors per thread of the block-per-row kernel by row length
  layerNormConfigs = {{{"WARP_ROW_VECS", 8}, {"THREAD_VECS", 0}, {"VECTORIZE_WIDTH", 16}},
                      {{"WARP_ROW_VECS", 16}, {"THREAD_VECS", 0}, {"VECTORIZE_WIDTH", 16}},
                      {{"WARP_ROW_VECS", 8}, {"THREAD_VECS", 8}, {"VECTORIZE_WIDTH", 16}},
                      {{"WARP_ROW_VECS", 8}, {"THREAD_VECS", 4}, {"VECTORIZE_WIDTH", 16}},
                      {{"WARP_ROW_VECS", 0}, {"THREAD_VECS", 0}, {"VECTORIZE_WIDTH", 16}}};
  gatherConfigs = {{{"BLOCK_SIZE", 256}, {"VECTORIZE_WIDTH", 16}}};
  softmaxConfigs = {{{"BLOCK_SIZE", 256}}};
  fusionConfigs = {{{"EPILOGUE", 1}}};
  // VARIANT -1: the library picks the attention kernel by shape (CTA pair, two tiles, one tile)
  fmhaConfigs = {{{"BLOCK_SIZE", 384}, {"Br", 512}, {"Bc", 128}, {"KV_STAGES", 2}, {"WARP_SIZE", 32}, {"VARIANT", -1}},
                 {{"BLOCK_SIZE", 384}, {"Br", 256}, {"Bc", 128}, {"KV_STAGES", 2}, {"WARP_SIZE", 32}, {"VARIANT", 5}},
                 {{"BLOCK_SIZE", 384}, {"Br", 512}, {"Bc", 128}, {"KV_STAGES", 2}, {"WARP_SIZE", 32}, {"VARIANT", 3}},
                 {{"BLOCK_SIZE", 384}, {"Br", 256}, {"Bc", 128}, {"KV_STAGES", 3}, {"WARP_SIZE", 32}, {"VARIANT", 4}},
                 {{"BLOCK_SIZE", 384}, {"Br", 256}, {"Bc", 128}, {"KV_STAGES", 2}, {"WARP_SIZE", 32}, {"VARIANT", 2}},
                 {{"BLOCK_SIZE", 192}, {"Br", 128}, {"Bc", 128}, {"KV_STAGES", 2}, {"WARP_SIZE", 32}, {"VARIANT", 1}}};
}

ComputeDAG& KernelCodeGenerator::createGraph(const std::string& graphName) {
  minLatency = FLT_MAX;
  graph.data = std::make_shared<GraphData>();
  graph.data->name = graphName;
  return graph;
}

void KernelCodeGenerator::dump(Module& module, const std::string& info) {
  if (KCGLog::level == Log::Release) return;
  std::cerr << "----------------------------------------------------------\n";
  std::cerr << "           " << info << "\n";
  std::cerr << "----------------------------------------------------------\n";
  module.dump();
}

void KernelCodeGenerator::save(const std::string& str, const std::string& file) {
  if (file == "terminal") {
    std::cout << str;
    return;
  }
  std::ofstream w(file.c_str());
  if (!w.is_open()) {
    std::cerr << "Can't open file \"" << file << "\"\n";
    return;
  }
  w << str;
}

void KernelCodeGenerator::resetModule(Module& module) { module.graph = clone(backupModule_.graph); }
void KernelCodeGenerator::backupModule(Module& module) { backupModule_.graph = clone(module.graph); }
void KernelCodeGenerator::saveBestModule(Module& module) {
  bestModule.graph = clone(module.graph);
  rebuild_calls(bestModule);
}

Module& KernelCodeGenerator::optimize(ComputeDAG& graph_) {
  graph = graph_;
  Module module;
  module.graph = clone(graph.data);
  saveBestModule(module);
  OpBuilder builder;
  for (auto& opt : opts) {
    backupModule(module);
    std::vector<std::map<std::string, int>>* table = nullptr;
    std::map<std::string, int>* slot = nullptr;
    if (*opt == FMHAOptimizer()) { table = &fmhaConfigs; slot = &FMHAOptimizer::fmhaConfig; }
    else if (*opt == MatmulOptimizer()) { table = &matmulConfigs; slot = &MatmulOptimizer::matmulConfig; }
    else if (*opt == BinaryOptimizer()) { table = &binaryConfigs; slot = &BinaryOptimizer::binaryConfig; }
    else if (*opt == ElementWiseOptimizer()) { table = &elementWiseConfigs; slot = &ElementWiseOptimizer::elementWiseConfig; }
    else if (*opt == LayerNormOptimizer()) { table = &layerNormConfigs; slot = &LayerNormOptimizer::layerNormConfig; }
    else if (*opt == GatherOptimizer()) { table = &gatherConfigs; slot = &GatherOptimizer::gatherConfig; }
    else if (*opt == BatchMatmulOptimizer()) { table = &batchMatmulConfigs; slot = &BatchMatmulOptimizer::batchMatmulConfig; }
    else if (*opt == SoftmaxOptimizer()) { table = &softmaxConfigs; slot = &SoftmaxOptimizer::softmaxConfig; }
    else if (*opt == KernelFusionOptimizer()) { table = &fusionConfigs; slot = &KernelFusionOptimizer::fusionConfig; }
    bool applied = false;
    if (table) {
      // Each candidate is applied to a fresh copy of the module and timed; the fastest one is
      // kept.  With evaluate() == 0 (no autotuning) the comparison is strict, so the first entry
      // of the table wins, as in the reference (src/KernelCodeGen.cc:15-118).
      float best = FLT_MAX;
      std::map<std::string, int> bestCfg;
      for (auto& cfg : *table) {
        *slot = cfg;
        resetModule(module);
        if (opt->applicable(module)) {
          opt->applyOptimzer(module, builder);
          const float latency = evaluate(module);
          if (KCGLog::level == Log::Debug && autotune) {
            std::cerr << "autotune " << opt->name << ":";
            for (const auto& kv : cfg) std::cerr << " " << kv.first << "=" << kv.second;
            std::cerr << " -> " << latency << " ms\n";
          }
          if (latency < best) {
            best = latency;
            bestCfg = cfg;
            saveBestModule(module);
            applied = true;
          }
        }
      }
      if (!applied) resetModule(module);
      else {
        module.graph = clone(bestModule.graph);
        *slot = bestCfg;
        minLatency = best;
      }
    } else if (opt->applicable(module)) {
      opt->applyOptimzer(module, builder);
      minLatency = evaluate(module);
      saveBestModule(module);
    }
  }
  return bestModule;
}

std::string CUDAGen(Module& module) {
  std::ostringstream os;
  if (!module.graph) return "";
  const auto& g = *module.graph;
  os << "// dispatch plan for graph \"" << g.name << "\": one line per sm_100a kernel launch\n";
  for (const auto& c : module.calls) {
    const auto& op = g.ops[c.op];
    const auto& info = g.funcs.at(op.func);
    os << (info.state == "gpu" ? "launch " : "// no optimizer selected @");
    if (info.state == "gpu") os << c.entry << "  // @";
    os << op.func << " (";
    for (size_t i = 0; i < op.inputs.size(); ++i) {
      const auto& t = g.tensors[op.inputs[i]];
      os << (i ? ", " : "") << "%" << op.inputs[i] << ":" << toStr(t.dtype) << shape_str(t.shape);
    }
    const auto& o = g.tensors[op.output];
    os << ") -> %" << op.output << ":" << toStr(o.dtype) << shape_str(o.shape);
    if (o.alias_of >= 0) os << " inplace(%" << g.root(op.output) << ")";
    if (!info.optimizer.empty()) {
      os << "  [" << info.optimizer;
      for (const auto& kv : info.config) os << " " << kv.first << "=" << kv.second;
      os << "]";
    }
    os << "\n";
  }
  return os.str();
}

std::string KernelCodeGenerator::codegen(Module module) {
  if (platform == "CUDA") {
    std::string text = CUDAGen(module);
    if (KCGLog::level == Log::Debug) std::cerr << text;
    return text;
  }
  std::cerr << "Platform \"" << platform << "\" has no back end (only \"CUDA\").\n";
  return "";
}

std::vector<std::map<std::string, int>>* KernelCodeGenerator::configs(const std::string& family) {
  if (family == "Matmul") return &matmulConfigs;
  if (family == "BatchMatmul") return &batchMatmulConfigs;
  if (family == "FMHA") return &fmhaConfigs;
  if (family == "Binary") return &binaryConfigs;
  if (family == "ElementWise") return &elementWiseConfigs;
  if (family == "Gather") return &gatherConfigs;
  if (family == "LayerNorm") return &layerNormConfigs;
  if (family == "Softmax") return &softmaxConfigs;
  if (family == "KernelFusion") return &fusionConfigs;
  return nullptr;
}

float KernelCodeGenerator::evaluate(Module& module) {
  if (!autotune || !module.graph) return 0.0f;
  int devices = 0;
  kcg_device_count(&devices);
  if (devices <= 0) return 0.0f;
  rebuild_calls(module);
  const auto& g = *module.graph;
  // one zero-filled scratch buffer per tensor that owns storage (zeros are valid indices for
  // Gather and harmless operands for everything else; timing does not depend on the values)
  Bindings bind;
  std::vector<void*> owned;
  bool ok = true;
  for (size_t t = 0; t < g.tensors.size() && ok; ++t) {
    if (g.tensors[t].alias_of >= 0) continue;
    size_t bytes = dtypeSize(g.tensors[t].dtype);
    for (auto d : g.tensors[t].shape) bytes *= static_cast<size_t>(d);
    bytes = (bytes + 255) / 256 * 256 + 256;
    void* p = nullptr;
    if (kcg_peer_alloc(bytes, &p) != KCG_OK || kcg_device_memset(p, 0, bytes, nullptr) != KCG_OK) { ok = false; break; }
    owned.push_back(p);
    bind.ptrs[static_cast<int>(t)] = p;
  }
  float ms = FLT_MAX;
  if (ok && runSelected(module, bind, nullptr, true) == KCG_OK) {  // warm-up (first-use set-up, caches)
    constexpr int kRuns = 5;
    void* timer = nullptr;
    if (kcg_timer_begin(nullptr, &timer) == KCG_OK) {
      int rc = KCG_OK;
      for (int i = 0; i < kRuns && rc == KCG_OK; ++i) rc = runSelected(module, bind, nullptr, true);
      float total = 0.f;
      if (kcg_timer_end(nullptr, timer, &total) == KCG_OK && rc == KCG_OK && kcg_device_status() == KCG_OK)
        ms = total / kRuns;
    }
  }
  for (void* p : owned) kcg_peer_free(p);
  return ms;
}

namespace {
// The kernels' process-wide switches that a function's chosen config maps to.
void apply_knobs(OpKind kind, const std::map<std::string, int>& cfg, bool restore) {
  auto find = [&](const char* key, int& v) {
    auto it = cfg.find(key);
    if (it == cfg.end()) return false;
    v = it->second;
    return true;
  };
  int v = 0;
  switch (kind) {
    case OpKind::Matmul: case OpKind::BatchedMatmul:
      if (find("CTA_PAIR", v)) {
        int bn = 256;
        find("BLOCK_SIZE_N", bn);
        // CTA_PAIR=1: the library's own choice; 0: single-CTA tiles of the stated width
        kcg_gemm_set_pair_mode(restore ? -1 : (v ? -1 : (bn == 128 ? 2 : (bn == 64 ? 3 : 0))));
      }
      break;
    case OpKind::LayerNorm: case OpKind::FusedLayerNormGeluAdd:
      if (find("WARP_ROW_VECS", v)) kcg_layernorm_set_warp_row_limit(restore ? 8 : v);
      if (find("THREAD_VECS", v)) kcg_layernorm_set_block_shape(restore ? 0 : v, 1);
      break;
    case OpKind::FusedAttention:
      if (find("VARIANT", v)) kcg_fmha_set_p_in_tmem(restore ? -1 : v);
      break;
    default: break;
  }
}
}  // namespace

int KernelCodeGenerator::run(Module& module, const Bindings& bindings, void* stream) {
  return runSelected(module, bindings, stream, false);
}

int KernelCodeGenerator::run(Module& module, const Bindings& bindings, const ShardSpec& shard, void* stream) {
  if (shard.world < 1 || shard.rank < 0 || shard.rank >= shard.world) {
    std::cerr << "run: ShardSpec with world " << shard.world << ", rank " << shard.rank << ".\n";
    return KCG_ERR_INVALID_ARG;
  }
  if (shard.gather && shard.world > 1 && !shard.nccl_comm) {
    std::cerr << "run: ShardSpec::gather needs an NCCL communicator.\n";
    return KCG_ERR_INVALID_ARG;
  }
  return runSelected(module, bindings, stream, false, &shard);
}

namespace {

// This rank's block of `total` units (all of them when the run is not sharded).
struct Cut {
  int64_t begin = 0, count = 0;
  bool on = false;
};

// Leading dimension and batch stride of a tensor used as a (batched) GEMM operand: the innermost
// stride must be 1 and the batch dims must collapse to one stride.
bool gemm_view(const TensorInfo& t, int64_t& ld, int64_t& batch_stride) {
  const auto st = t.effective_strides();
  const size_t r = st.size();
  if (r < 2 || st[r - 1] != 1) return false;
  ld = st[r - 2];
  batch_stride = r > 2 ? st[r - 3] : 0;
  for (size_t d = 0; d + 3 < r; ++d)
    if (st[d] != st[d + 1] * t.shape[d + 1]) return false;
  return true;
}

char* shifted(void* p, int64_t elements, size_t esize) { return static_cast<char*>(p) + elements * static_cast<int64_t>(esize); }

}  // namespace

int KernelCodeGenerator::runSelected(Module& module, const Bindings& bindings, void* stream, bool skipUnselected,
                                     const ShardSpec* shard) {
  if (!module.graph) return KCG_ERR_INVALID_ARG;
  const auto& g = *module.graph;
  const bool sharded = shard && shard->world > 1;
  auto ptr = [&](int id) -> void* {
    for (int t = id; t >= 0; t = g.tensors[t].alias_of)
      if (void* p = bindings.get(t)) return p;
    return nullptr;
  };
  auto numel = [&](int id) {
    int64_t n = 1;
    for (auto d : g.tensors[id].shape) n *= d;
    return n;
  };
  auto cut = [&](int64_t total, int64_t granule) {
    Cut c;
    c.count = total;
    if (sharded && kcg_shard_range(total, shard->world, shard->rank, granule, &c.begin, &c.count) == KCG_OK) c.on = true;
    return c;
  };
  // all-gather of a sharded output, in place, on the same stream (only when the spec asks for it)
  auto gather = [&](const Cut& c, void* out, int64_t units, int64_t unit_bytes, int64_t granule) -> int {
    if (!c.on || !shard->gather) return KCG_OK;
    return kcg_shard_allgather(out, units, unit_bytes, granule, shard->world, shard->rank, shard->nccl_comm, stream);
  };
  for (const auto& c : module.calls) {
    const auto& op = g.ops[c.op];
    const auto& info = g.funcs.at(op.func);
    if (info.state != "gpu" && skipUnselected) continue;
    if (info.state != "gpu") {
      std::cerr << "run: no optimizer selected a kernel for @" << op.func
                << " (push the matching Optimizer into opts); there is no CPU execution path.\n";
      return KCG_ERR_UNSUPPORTED;
    }
    std::vector<void*> in;
    for (int id : op.inputs) {
      void* p = ptr(id);
      if (!p) {
        std::cerr << "run: tensor %" << id << " of @" << op.func << " has no device pointer bound.\n";
        return KCG_ERR_INVALID_ARG;
      }
      in.push_back(p);
    }
    void* out = ptr(op.output);
    if (!out) {
      std::cerr << "run: result %" << op.output << " of @" << op.func << " has no device pointer bound.\n";
      return KCG_ERR_INVALID_ARG;
    }
    const auto& t0 = g.tensors[op.inputs[0]];
    const auto& to = g.tensors[op.output];
    const size_t es_in = dtypeSize(t0.dtype), es_out = dtypeSize(to.dtype);
    int rc = KCG_OK;
    apply_knobs(op.kind, info.config, false);
    switch (op.kind) {
      case OpKind::Matmul: {
        const int64_t m = t0.shape[0], k = t0.shape[1], n = g.tensors[op.inputs[1]].shape[1];
        const float* sa = op.scale_a >= 0 ? static_cast<const float*>(ptr(op.scale_a)) : nullptr;
        const float* sb = op.scale_b >= 0 ? static_cast<const float*>(ptr(op.scale_b)) : nullptr;
        const Cut r = cut(m, 128);   // rows of A and C; B is replicated
        if (r.count > 0)
          rc = kcg_gemm_fused(static_cast<int>(t0.dtype), static_cast<int>(to.dtype), r.count, n, k, 1, 0, 0,
                              shifted(in[0], r.begin * k, es_in), k, 0, in[1], n, 0, shifted(out, r.begin * n, es_out), n, 0,
                              sa, sb, op.bias >= 0 ? ptr(op.bias) : nullptr, act_code(op.activation), stream);
        if (rc == KCG_OK) rc = gather(r, out, m, n * static_cast<int64_t>(es_out), 128);
        break;
      }
      case OpKind::BatchedMatmul: {
        const auto& tb = g.tensors[op.inputs[1]];
        const auto& sa = t0.shape;
        const auto& sb = tb.shape;
        const size_t r = sa.size();
        const bool ta = op.layoutA == Layout::colMajor, tbt = op.layoutB == Layout::colMajor;
        const int64_t m = ta ? sa[r - 1] : sa[r - 2], k = ta ? sa[r - 2] : sa[r - 1];
        const int64_t n = tbt ? sb[r - 2] : sb[r - 1];
        int64_t batch = 1;
        for (size_t d = 0; d + 2 < r; ++d) batch *= sa[d];
        int64_t lda, ldb, ldc, stride_a, stride_b, stride_c;
        if (!gemm_view(t0, lda, stride_a) || !gemm_view(tb, ldb, stride_b) || !gemm_view(to, ldc, stride_c)) {
          std::cerr << "run: @" << op.func << " has a strided operand the GEMM kernel cannot address (one leading "
                       "dimension and one batch stride); such layouts run only as part of the fused attention chain.\n";
          return KCG_ERR_UNSUPPORTED;
        }
        const void* bias = op.bias >= 0 ? ptr(op.bias) : nullptr;
        if (batch > 1) {
          const Cut bc = cut(batch, 1);   // whole matrices per rank
          if (bc.count > 0)
            rc = kcg_gemm_fused(static_cast<int>(t0.dtype), static_cast<int>(to.dtype), m, n, k, bc.count, ta, tbt,
                                shifted(in[0], bc.begin * stride_a, es_in), lda, stride_a,
                                shifted(in[1], bc.begin * stride_b, es_in), ldb, stride_b,
                                shifted(out, bc.begin * stride_c, es_out), ldc, stride_c, nullptr, nullptr, bias,
                                act_code(op.activation), stream);
          if (rc == KCG_OK && bc.on && shard->gather) {
            if (!to.dense()) {
              std::cerr << "run: the gather of @" << op.func << " needs a dense result.\n";
              return KCG_ERR_UNSUPPORTED;
            }
            rc = gather(bc, out, batch, m * n * static_cast<int64_t>(es_out), 1);
          }
        } else {
          const Cut rc_rows = cut(m, 128);
          if (rc_rows.count > 0)
            rc = kcg_gemm_fused(static_cast<int>(t0.dtype), static_cast<int>(to.dtype), rc_rows.count, n, k, 1, ta, tbt,
                                shifted(in[0], ta ? rc_rows.begin : rc_rows.begin * lda, es_in), lda, 0, in[1], ldb, 0,
                                shifted(out, rc_rows.begin * ldc, es_out), ldc, 0, nullptr, nullptr, bias,
                                act_code(op.activation), stream);
          if (rc == KCG_OK && rc_rows.on && shard->gather) {
            if (!to.dense()) {
              std::cerr << "run: the gather of @" << op.func << " needs a dense result.\n";
              return KCG_ERR_UNSUPPORTED;
            }
            rc = gather(rc_rows, out, m, n * static_cast<int64_t>(es_out), 128);
          }
        }
        break;
      }
      case OpKind::Softmax: {
        const int64_t cols = t0.shape.back();
        const int64_t rows = cols ? numel(op.inputs[0]) / cols : 0;
        const int64_t q_len = t0.shape.size() >= 2 ? t0.shape[t0.shape.size() - 2] : 1;
        // a causal mask depends on the row's position inside its [q_len, cols] matrix: keep matrices whole
        const int64_t gran = op.causal && q_len > 0 ? q_len : 1;
        const Cut r = cut(rows, gran);
        if (r.count > 0)
          rc = kcg_softmax(static_cast<int>(t0.dtype), r.count, cols, op.scale, op.causal, q_len,
                           shifted(in[0], r.begin * cols, es_in), shifted(out, r.begin * cols, es_out), stream);
        if (rc == KCG_OK) rc = gather(r, out, rows, cols * static_cast<int64_t>(es_out), gran);
        break;
      }
      case OpKind::LayerNorm: {
        int64_t cols = 1;
        for (size_t d = static_cast<size_t>(op.axis); d < t0.shape.size(); ++d) cols *= t0.shape[d];
        const int64_t rows = cols ? numel(op.inputs[0]) / cols : 0;
        if (numel(op.inputs[1]) != cols || numel(op.inputs[2]) != cols) {
          std::cerr << "run: LayerNorm scale/bias with broadcast (1) dims must be bound pre-expanded to the "
                       "normalised shape.\n";
          return KCG_ERR_UNSUPPORTED;
        }
        const Cut r = cut(rows, 1);
        if (r.count > 0)
          rc = kcg_layernorm(static_cast<int>(t0.dtype), r.count, cols, shifted(in[0], r.begin * cols, es_in), in[1], in[2],
                             op.eps, shifted(out, r.begin * cols, es_out), stream);
        if (rc == KCG_OK) rc = gather(r, out, rows, cols * static_cast<int64_t>(es_out), 1);
        break;
      }
      case OpKind::ElementWise: {
        const int opi = index_of(ElementWise::operations(), op.operation);
        const int64_t n_all = numel(op.inputs[0]);
        const int64_t units = !t0.shape.empty() && t0.shape[0] > 0 ? t0.shape[0] : 1;
        const int64_t inner = n_all / units;
        const Cut r = cut(units, 1);
        if (r.count * inner > 0)
          rc = kcg_eltwise(opi, static_cast<int>(t0.dtype), static_cast<int>(to.dtype), r.count * inner,
                           shifted(in[0], r.begin * inner, es_in), shifted(out, r.begin * inner, es_out), stream);
        if (rc == KCG_OK && n_all > 0) rc = gather(r, out, units, inner * static_cast<int64_t>(es_out), 1);
        break;
      }
      case OpKind::Binary: {
        std::vector<int64_t> sa = t0.shape, sb = g.tensors[op.inputs[1]].shape;
        // Rows can be split when A already has the output's shape and B either has it too or does
        // not extend along dim 0 (a bias-like operand); any other broadcast runs whole on every rank.
        const bool b_same = sb == sa;
        const bool b_fixed = sb.size() < sa.size() || (sb.size() == sa.size() && !sb.empty() && sb[0] == 1 && sa[0] != 1);
        const bool splittable = sharded && to.shape == sa && !sa.empty() && sa[0] > 0 && (b_same || b_fixed);
        void* a_ptr = in[0];
        void* b_ptr = in[1];
        void* c_ptr = out;
        Cut r;
        r.count = sa.empty() ? 1 : sa[0];
        if (splittable) {
          r = cut(sa[0], 1);
          const int64_t inner = numel(op.inputs[0]) / sa[0];
          a_ptr = shifted(in[0], r.begin * inner, es_in);
          c_ptr = shifted(out, r.begin * inner, es_out);
          if (b_same) b_ptr = shifted(in[1], r.begin * inner, es_in);
          sa[0] = r.count;
          if (b_same) sb[0] = r.count;
        }
        if (!splittable || r.count > 0)
          rc = kcg_binary(index_of(Binary::operations(), op.operation), static_cast<int>(t0.dtype),
                          static_cast<int>(sa.size()), sa.data(), static_cast<int>(sb.size()), sb.data(), a_ptr, b_ptr, c_ptr,
                          stream);
        if (rc == KCG_OK && splittable)
          rc = gather(r, out, t0.shape[0], numel(op.inputs[0]) / t0.shape[0] * static_cast<int64_t>(es_out), 1);
        break;
      }
      case OpKind::Gather: {
        const auto& ti = g.tensors[op.inputs[1]];
        int64_t outer = 1, inner = 1;
        for (int64_t d = 0; d < op.axis; ++d) outer *= t0.shape[d];
        for (size_t d = op.axis + 1; d < t0.shape.size(); ++d) inner *= t0.shape[d];
        rc = kcg_gather(static_cast<int>(t0.dtype), static_cast<int>(ti.dtype), outer, t0.shape[op.axis], inner,
                        numel(op.inputs[1]), in[0], in[1], out, stream);
        break;
      }
      case OpKind::Transpose: {
        const size_t r = t0.shape.size();
        const int64_t rows = t0.shape[r - 2], cols = t0.shape[r - 1];
        const int64_t batch = (rows != 0 && cols != 0) ? numel(op.inputs[0]) / (rows * cols) : 0;
        Cut bc;
        bc.count = batch;
        if (batch > 1) bc = cut(batch, 1);
        if (bc.count > 0)
          rc = kcg_transpose(static_cast<int>(t0.dtype), bc.count, rows, cols, shifted(in[0], bc.begin * rows * cols, es_in),
                             shifted(out, bc.begin * rows * cols, es_out), stream);
        if (rc == KCG_OK && batch > 1) rc = gather(bc, out, batch, rows * cols * static_cast<int64_t>(es_out), 1);
        break;
      }
      case OpKind::FusedLayerNormGeluAdd: {
        const int64_t cols = t0.shape.back();
        const int64_t rows = cols ? numel(op.inputs[0]) / cols : 0;
        const Cut r = cut(rows, 1);
        if (r.count > 0)
          rc = kcg_layernorm_gelu_add(static_cast<int>(t0.dtype), r.count, cols, shifted(in[0], r.begin * cols, es_in), in[1],
                                      in[2], op.eps, shifted(in[3], r.begin * cols, es_in),
                                      shifted(out, r.begin * cols, es_out), stream);
        if (rc == KCG_OK) rc = gather(r, out, rows, cols * static_cast<int64_t>(es_out), 1);
        break;
      }
      case OpKind::FusedAttention: {
        const auto& tk = g.tensors[op.inputs[1]];
        const auto& tv = g.tensors[op.inputs[2]];
        const auto& q = t0.shape;
        const size_t r = q.size();
        const int64_t D = q[r - 1], Sq = q[r - 2], Skv = tk.shape[r - 2];
        const int64_t H = r == 4 ? q[1] : 1, B = q[0];
        // (batch, head, sequence) element strides of each tensor, whatever layout it was declared with
        auto bhs = [&](const TensorInfo& t, int64_t (&st)[3]) {
          const auto e = t.effective_strides();
          st[0] = e[0];
          st[1] = r == 4 ? e[1] : e[0];
          st[2] = e[r - 2];
        };
        int64_t qs[3], ks[3], vs[3], os[3];
        bhs(t0, qs); bhs(tk, ks); bhs(tv, vs); bhs(to, os);
        const Cut bc = cut(B, 1);   // whole batches per rank
        if (bc.count > 0)
          rc = kcg_fmha_fwd(static_cast<int>(t0.dtype), bc.count, H, Sq, Skv, D, op.scale, op.causal,
                            shifted(in[0], bc.begin * qs[0], es_in), qs, shifted(in[1], bc.begin * ks[0], es_in), ks,
                            shifted(in[2], bc.begin * vs[0], es_in), vs, shifted(out, bc.begin * os[0], es_out), os, stream);
        if (rc == KCG_OK && bc.on && shard->gather) {
          if (os[0] != H * Sq * D) {
            std::cerr << "run: the gather of @" << op.func << " needs each batch of the result to be one contiguous block.\n";
            return KCG_ERR_UNSUPPORTED;
          }
          rc = gather(bc, out, B, os[0] * static_cast<int64_t>(es_out), 1);
        }
        break;
      }
    }
    apply_knobs(op.kind, info.config, true);
    if (rc != KCG_OK) {
      std::cerr << "run: " << c.entry << " for @" << op.func << " failed: " << kcg_last_error() << "\n";
      return rc;
    }
  }
  return KCG_OK;
}

}  // namespace KernelCodeGen
