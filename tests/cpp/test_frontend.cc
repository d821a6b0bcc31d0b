// Front-end tests in the style of the reference's own test program (test/test.cc): each
// case builds a graph with the reference call sequence, optimizes it and checks the result.
//   test_frontend cpu    graph construction, naming, dedup, error handling, plans (no GPU)
//   test_frontend gpu    runs the plans on the current device and compares with the CPU oracle
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include "KernelCodeGen.h"
#include "kcg_kernels.h"

using namespace KernelCodeGen;

static int failures = 0;
#define CHECK(cond)                                                              \
  do {                                                                           \
    if (!(cond)) {                                                               \
      std::fprintf(stderr, "CHECK failed %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++failures;                                                                \
    }                                                                            \
  } while (0)

static bool has(const std::string& text, const std::string& needle) { return text.find(needle) != std::string::npos; }

// ---------------------------------------------------------------------------------- cpu mode
static void test_operators_cast() {  // test/test.cc:8-49, the live sequence
  KernelCodeGenerator generator("CUDA");
  auto graph = generator.createGraph("demo");
  generator.setLogMode(Log::Release);
  generator.opts.push_back(std::move(std::make_unique<ElementWiseOptimizer>()));
  auto A = graph.create<PlaceHolder>(std::vector<int64_t>{2, 768, 768}, std::string{"float32"});
  auto gelu = graph.create<ElementWise>(A, "Cast", MemorySpace::global, "int32");
  CHECK(bool(A) && bool(gelu));
  CHECK(gelu.dtype() == DType::i32 && gelu.shape() == A.shape());
  graph.dump();
  auto module = generator.optimize(graph);
  generator.dump(module);
  auto&& sourceCode = generator.codegen(module);
  CHECK(has(sourceCode, "launch kcg_eltwise") && has(sourceCode, "@Cast_Elementwise_2_768_768_float32_to_int32"));
  CHECK(module.graph->funcs.at("Cast_Elementwise_2_768_768_float32_to_int32").state == "gpu");
  // the graph the user holds is untouched by optimize (the reference optimizes a clone)
  CHECK(graph.data->funcs.at("Cast_Elementwise_2_768_768_float32_to_int32").state == "cpu");
}

static void test_commented_sequences() {  // test/test.cc:26-46, the commented-out variants
  KernelCodeGenerator generator("CUDA");
  generator.opts.push_back(std::make_unique<LayerNormOptimizer>());
  generator.opts.push_back(std::make_unique<BinaryOptimizer>());
  generator.opts.push_back(std::make_unique<MatmulOptimizer>());
  generator.opts.push_back(std::make_unique<BatchMatmulOptimizer>());
  generator.opts.push_back(std::make_unique<ElementWiseOptimizer>());
  auto graph = generator.createGraph("demo");
  {
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{2, 768, 768}, std::string{"float32"});
    int64_t axis_ = 1;
    float eps = 1e-5;
    auto scale = graph.create<PlaceHolder>(std::vector<int64_t>{768, 768}, std::string{"float32"});
    auto bias = graph.create<PlaceHolder>(std::vector<int64_t>{768, 768}, std::string{"float32"});
    auto layernorm = graph.create<LayerNorm>(A, scale, bias, axis_, eps);
    CHECK(bool(layernorm) && layernorm.shape() == A.shape());
  }
  {
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{16, 1, 1, 256}, std::string{"float32"});
    auto B = graph.create<PlaceHolder>(std::vector<int64_t>{1, 128, 256}, std::string{"float32"});
    auto C = graph.create<Binary>(A, B, "Add");
    CHECK(bool(C) && C.shape() == (std::vector<int64_t>{16, 1, 128, 256}));
  }
  {
    int m = 2048, n = 2048, k = 1024;
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{m, k}, std::string{"float32"});
    auto B = graph.create<PlaceHolder>(std::vector<int64_t>{k, n}, std::string{"float32"});
    auto C = graph.create<Matmul>(A, B);
    auto D = graph.create<Relu>(C, MemorySpace::inplace);  // test/test.cc:62-63
    auto C2 = graph.create<Matmul>(A, B, MemorySpace::global);  // old call form, test/test.cc:89
    CHECK(bool(C) && bool(D) && bool(C2));
    CHECK(graph.data->tensors[D.id].alias_of == C.id);
  }
  {
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{256, 2048, 64}, std::string{"float32"});
    auto B = graph.create<PlaceHolder>(std::vector<int64_t>{256, 2048, 64}, std::string{"float32"});
    auto C = graph.create<BatchedMatmul>(A, Layout::rowMajor, B, Layout::colMajor);
    CHECK(bool(C) && C.shape() == (std::vector<int64_t>{256, 2048, 2048}));
  }
  const auto& f = graph.data->funcs;
  CHECK(f.count("LayerNorm_2_768_768_axis_1"));
  CHECK(f.count("Add_Binary_16_1_1_256_Add_1_128_256"));
  CHECK(f.count("Matmul_m2048n2048k1024"));
  CHECK(f.count("Relu_Elementwise_2048_2048"));
  CHECK(f.count("BatchMatmul_256_m2048_n2048_k64_NT"));
  // two calls of the same (op, shape) share one function
  int matmul_funcs = 0;
  for (const auto& name : graph.data->func_order) matmul_funcs += name == "Matmul_m2048n2048k1024";
  CHECK(matmul_funcs == 1);
  auto module = generator.optimize(graph);
  for (const auto& kv : module.graph->funcs) CHECK(kv.second.state == "gpu");
  // "Matmul" must not claim the batched function (reference: Optimizer.cc:255)
  CHECK(module.graph->funcs.at("BatchMatmul_256_m2048_n2048_k64_NT").optimizer == "BatchMatmul");
  CHECK(module.graph->funcs.at("Matmul_m2048n2048k1024").optimizer == "Matmul");
  CHECK(module.graph->funcs.at("Relu_Elementwise_2048_2048").optimizer == "ElementWise");
  auto plan = generator.codegen(module);
  CHECK(has(plan, "launch kcg_layernorm") && has(plan, "launch kcg_binary") && has(plan, "launch kcg_gemm"));
  CHECK(has(plan, "inplace(%"));
  generator.save(plan, "/tmp/kcg_plan_test.txt");
  FILE* fp = std::fopen("/tmp/kcg_plan_test.txt", "r");
  CHECK(fp != nullptr);
  if (fp) std::fclose(fp);
}

static void test_flash_attention_graph() {  // test/test.cc:107-147
  KernelCodeGenerator generator("CUDA");
  auto graph = generator.createGraph("flash_attn_demo");
  generator.opts.push_back(std::move(std::make_unique<FMHAOptimizer>()));
  int64_t head_dim = 64L, seq_len = 2048L, batch_size = 8, head_num = 32;
  for (const char* dtype : {"float32", "bfloat16"}) {
    graph = generator.createGraph("flash_attn_demo");
    auto Q = graph.create<PlaceHolder>(std::vector<int64_t>{batch_size, head_num, seq_len, head_dim}, std::string{dtype});
    auto K = graph.create<PlaceHolder>(std::vector<int64_t>{batch_size, head_num, seq_len, head_dim}, std::string{dtype});
    auto V = graph.create<PlaceHolder>(std::vector<int64_t>{batch_size, head_num, seq_len, head_dim}, std::string{dtype});
    auto S = graph.create<BatchedMatmul>(Q, Layout::rowMajor, K, Layout::colMajor);
    auto P = graph.create<Softmax>(S, -1, MemorySpace::inplace);
    auto O = graph.create<BatchedMatmul>(P, Layout::rowMajor, V, Layout::rowMajor);
    CHECK(bool(O) && O.shape() == Q.shape());
    // float32 functions carry the reference's exact names; other element types are appended
    const std::string sfx = std::string(dtype) == "float32" ? "" : "_" + std::string(dtype);
    CHECK(graph.data->funcs.count("BatchMatmul_8_32_m2048_n2048_k64_NT" + sfx));
    CHECK(graph.data->funcs.count("Softmax_8_32_2048_2048_axis3" + sfx));
    CHECK(graph.data->funcs.count("BatchMatmul_8_32_m2048_n64_k2048_NN" + sfx));
    auto module = generator.optimize(graph);
    auto plan = generator.codegen(module);
    if (std::string(dtype) == "bfloat16") {
      CHECK(module.calls.size() == 1);
      CHECK(has(plan, "launch kcg_fmha_fwd") && has(plan, "@Fused_Multi_Head_Attention_8_32_SL2048_HD64_bfloat16"));
      CHECK(!module.graph->funcs.count("Softmax_8_32_2048_2048_axis3_bfloat16"));
    } else {
      // the fused kernel is a 16-bit tensor-core kernel: the fp32 chain stays three calls
      CHECK(module.calls.size() == 3 && !has(plan, "kcg_fmha_fwd"));
    }
  }
  // a second user of the scores blocks the fusion (single-user rule, Optimizer.cc:2131-2135)
  graph = generator.createGraph("no_fuse");
  auto Q = graph.create<PlaceHolder>(std::vector<int64_t>{2, 128, 64}, std::string{"bfloat16"});
  auto S = graph.create<BatchedMatmul>(Q, Layout::rowMajor, Q, Layout::colMajor);
  auto P = graph.create<Softmax>(S, -1, MemorySpace::inplace);
  auto O = graph.create<BatchedMatmul>(P, Layout::rowMajor, Q, Layout::rowMajor);
  auto extra = graph.create<ElementWise>(P, "Tanh", MemorySpace::global);
  (void)O; (void)extra;
  auto module = generator.optimize(graph);
  CHECK(module.calls.size() == 4);
}

static void test_kernel_fusion() {
  KernelCodeGenerator generator("CUDA");
  generator.opts.push_back(std::make_unique<KernelFusionOptimizer>());
  generator.opts.push_back(std::make_unique<MatmulOptimizer>());
  generator.opts.push_back(std::make_unique<LayerNormOptimizer>());
  generator.opts.push_back(std::make_unique<ElementWiseOptimizer>());
  generator.opts.push_back(std::make_unique<BinaryOptimizer>());
  auto graph = generator.createGraph("fusion");
  auto A = graph.create<PlaceHolder>(std::vector<int64_t>{512, 128}, std::string{"bfloat16"});
  auto B = graph.create<PlaceHolder>(std::vector<int64_t>{128, 256}, std::string{"bfloat16"});
  auto bias = graph.create<PlaceHolder>(std::vector<int64_t>{256}, std::string{"bfloat16"});
  auto C = graph.create<Matmul>(A, B);
  auto Cb = graph.create<Binary>(C, bias, "Add");
  auto D = graph.create<ElementWise>(Cb, "Gelu", MemorySpace::global);
  // Matmul -> Relu(inplace), the reference's own sequence (test/test.cc:62-63)
  auto E = graph.create<Matmul>(A, B);
  auto F = graph.create<Relu>(E, MemorySpace::inplace);
  // LayerNorm -> Gelu -> Add
  auto X = graph.create<PlaceHolder>(std::vector<int64_t>{64, 256}, std::string{"bfloat16"});
  auto G = graph.create<PlaceHolder>(std::vector<int64_t>{256}, std::string{"bfloat16"});
  auto R = graph.create<PlaceHolder>(std::vector<int64_t>{64, 256}, std::string{"bfloat16"});
  auto Y = graph.create<LayerNorm>(X, G, G, int64_t(-1));
  auto Z = graph.create<ElementWise>(Y, "Gelu", MemorySpace::global);
  auto W = graph.create<Binary>(Z, R, "Add");
  // a Gelu whose input has a second reader must stay unfused
  auto H = graph.create<Matmul>(A, B);
  auto I = graph.create<ElementWise>(H, "Gelu", MemorySpace::global);
  auto J = graph.create<ElementWise>(H, "Tanh", MemorySpace::global);
  (void)D; (void)F; (void)W; (void)I; (void)J;
  auto module = generator.optimize(graph);
  auto plan = generator.codegen(module);
  CHECK(module.calls.size() == 6);  // fused gemm+bias+gelu, fused gemm+relu, fused LN chain, gemm, gelu, tanh
  CHECK(has(plan, "@Fused_Matmul_m512n256k128_bfloat16_Bias_Gelu"));
  CHECK(has(plan, "@Fused_Matmul_m512n256k128_bfloat16_Relu"));
  CHECK(has(plan, "launch kcg_layernorm_gelu_add") && has(plan, "@Fused_LayerNorm_64_256_axis_1_bfloat16_Gelu_Add"));
  CHECK(has(plan, "@Gelu_Elementwise_512_256_bfloat16") && has(plan, "@Tanh_Elementwise_512_256_bfloat16"));
  for (const auto& kv : module.graph->funcs) CHECK(kv.second.state == "gpu");
}

static void test_gather_transpose_graph() {  // test/test.cc:17-23 (the commented Gather sequence)
  KernelCodeGenerator generator("CUDA");
  generator.opts.push_back(std::make_unique<GatherOptimizer>());
  generator.opts.push_back(std::make_unique<TransposeOptimizer>());
  auto graph = generator.createGraph("gather_demo");
  auto A = graph.create<PlaceHolder>(std::vector<int64_t>{4, 9, 6}, std::string{"float32"});
  auto idx = graph.create<PlaceHolder>(std::vector<int64_t>{3, 2}, std::string{"int64"});
  auto one = graph.create<PlaceHolder>(std::vector<int64_t>{1}, std::string{"int32"});
  int64_t axis = 1;
  auto G = graph.create<Gather>(A, idx, axis);
  auto G1 = graph.create<Gather>(A, one, axis);
  auto G0 = graph.create<Gather>(A, idx);                   // axis defaults to 0
  auto T = graph.create<Transpose>(G);
  CHECK(bool(G) && G.shape() == (std::vector<int64_t>{4, 3, 2, 6}));
  CHECK(bool(G1) && G1.shape() == (std::vector<int64_t>{4, 6}));   // a [1] index drops the axis
  CHECK(bool(G0) && G0.shape() == (std::vector<int64_t>{3, 2, 9, 6}));
  CHECK(bool(T) && T.shape() == (std::vector<int64_t>{4, 3, 6, 2}));
  const auto& f = graph.data->funcs;
  CHECK(f.count("Gather_4_9_6_indices_3_2_axis_1") && f.count("Gather_4_9_6_indices_1_axis_1_idx32"));
  CHECK(f.count("Transpose_4_3_2_6"));
  auto module = generator.optimize(graph);
  for (const auto& kv : module.graph->funcs) CHECK(kv.second.state == "gpu");
  CHECK(module.graph->funcs.at("Gather_4_9_6_indices_3_2_axis_1").optimizer == "Gather");
  auto plan = generator.codegen(module);
  CHECK(has(plan, "launch kcg_gather") && has(plan, "launch kcg_transpose"));
}

static void test_config_candidates_without_autotune() {
  // evaluate() is 0 without autotuning, so the first entry of each table is the one recorded
  KernelCodeGenerator generator("CUDA");
  generator.opts.push_back(std::make_unique<MatmulOptimizer>());
  generator.opts.push_back(std::make_unique<LayerNormOptimizer>());
  CHECK(generator.configs("Matmul") && generator.configs("Matmul")->size() >= 2);
  CHECK(generator.configs("nope") == nullptr);
  auto graph = generator.createGraph("cands");
  auto A = graph.create<PlaceHolder>(std::vector<int64_t>{512, 256}, std::string{"bfloat16"});
  auto B = graph.create<PlaceHolder>(std::vector<int64_t>{256, 512}, std::string{"bfloat16"});
  auto C = graph.create<Matmul>(A, B);
  auto gm = graph.create<PlaceHolder>(std::vector<int64_t>{512}, std::string{"bfloat16"});
  auto Y = graph.create<LayerNorm>(C, gm, gm, int64_t(1), 1e-5f);
  auto module = generator.optimize(graph);
  CHECK(generator.evaluate(module) == 0.0f && generator.bestLatency() == 0.0f);
  CHECK(module.graph->funcs.at("Matmul_m512n512k256_bfloat16").config.at("CTA_PAIR") == generator.configs("Matmul")->front().at("CTA_PAIR"));
  CHECK(module.graph->funcs.at("LayerNorm_512_512_axis_1_bfloat16").config.at("WARP_ROW_VECS") == 8);
  auto plan = generator.codegen(module);
  CHECK(has(plan, "CTA_PAIR=1") && has(plan, "WARP_ROW_VECS=8"));   // the choice is part of the saved plan
  (void)Y;
}

static void test_errors() {
  KernelCodeGenerator generator("CUDA");
  auto graph = generator.createGraph("errors");
  auto A = graph.create<PlaceHolder>(std::vector<int64_t>{4, 5}, std::string{"float32"});
  auto B = graph.create<PlaceHolder>(std::vector<int64_t>{4, 3}, std::string{"float32"});
  CHECK(!graph.create<Matmul>(A, B));                       // incompatible K
  CHECK(!graph.create<Binary>(A, B, "Add"));                // dim not equal
  CHECK(!graph.create<Binary>(A, A, "Nope"));
  CHECK(!graph.create<LayerNorm>(A, A, A, int64_t(2)));     // axis out of bounds
  CHECK(!graph.create<LayerNorm>(A, B, A, int64_t(1)));     // scale dim is not equal
  CHECK(!graph.create<Softmax>(A, 0));                      // only the last dim
  CHECK(!graph.create<PlaceHolder>(std::vector<int64_t>{4}, std::string{"complex64"}));
  CHECK(!graph.create<Matmul>(Value{}, B));                 // null operand
  auto V1 = graph.create<PlaceHolder>(std::vector<int64_t>{7}, std::string{"float32"});
  CHECK(!graph.create<Transpose>(V1));                      // rank below 2
  CHECK(!graph.create<Gather>(A, A));                       // indices must be integers
  auto I1 = graph.create<PlaceHolder>(std::vector<int64_t>{3}, std::string{"int64"});
  CHECK(!graph.create<Gather>(A, I1, int64_t(2)));          // axis past the input's rank
  CHECK(getDType("bfloat16") == DType::bf16 && getDType("float8_e4m3") == DType::f8e4m3 && toStr(DType::f16) == "float16");
  // run() refuses functions no optimizer selected, and unbound tensors
  auto C = graph.create<ElementWise>(A, "Gelu", MemorySpace::global);
  auto module = generator.optimize(graph);
  Bindings bind;
  CHECK(generator.run(module, bind) == KCG_ERR_UNSUPPORTED);
  generator.opts.push_back(std::make_unique<ElementWiseOptimizer>());
  auto module2 = generator.optimize(graph);
  CHECK(generator.run(module2, bind) == KCG_ERR_INVALID_ARG);
  (void)C;
  KernelCodeGenerator rocm("ROCm");
  auto g2 = rocm.createGraph("x");
  auto m2 = rocm.optimize(g2);
  CHECK(rocm.codegen(m2).empty());
}

static void test_dtype_is_part_of_the_function_key() {
  // The reference names functions by operator and shape only; two calls that differ in element
  // type must still be two functions here (own state, optimizer decision, autotuned config).
  KernelCodeGenerator generator("CUDA");
  generator.opts.push_back(std::make_unique<LayerNormOptimizer>());
  auto graph = generator.createGraph("keys");
  Value y[2];
  int i = 0;
  for (const char* dtype : {"float32", "bfloat16"}) {
    auto X = graph.create<PlaceHolder>(std::vector<int64_t>{64, 512}, std::string{dtype});
    auto G = graph.create<PlaceHolder>(std::vector<int64_t>{512}, std::string{dtype});
    y[i++] = graph.create<LayerNorm>(X, G, G, int64_t(1));
  }
  CHECK(bool(y[0]) && bool(y[1]));
  const auto& f = graph.data->funcs;
  CHECK(f.size() == 2 && f.count("LayerNorm_64_512_axis_1") && f.count("LayerNorm_64_512_axis_1_bfloat16"));
  // same shape and type again: the existing function is reused (the reference's dedup)
  auto X = graph.create<PlaceHolder>(std::vector<int64_t>{64, 512}, std::string{"bfloat16"});
  auto G = graph.create<PlaceHolder>(std::vector<int64_t>{512}, std::string{"bfloat16"});
  CHECK(bool(graph.create<LayerNorm>(X, G, G, int64_t(1))) && graph.data->funcs.size() == 2);
  // a Cast is keyed by both types
  auto c1 = graph.create<ElementWise>(X, "Cast", MemorySpace::global, "float32");
  auto c2 = graph.create<ElementWise>(X, "Cast", MemorySpace::global, "float16");
  CHECK(bool(c1) && bool(c2) && f.count("Cast_Elementwise_64_512_bfloat16_to_float32") &&
        f.count("Cast_Elementwise_64_512_bfloat16_to_float16"));
}

static void test_strided_placeholders() {
  // Q, K, V stored [B,S,H,D] and declared as [B,H,S,D] views; O written into a [B,S,H,D] buffer
  KernelCodeGenerator generator("CUDA");
  generator.opts.push_back(std::make_unique<FMHAOptimizer>());
  generator.opts.push_back(std::make_unique<BatchMatmulOptimizer>());
  generator.opts.push_back(std::make_unique<SoftmaxOptimizer>());
  auto graph = generator.createGraph("bshd");
  const int64_t B = 2, H = 4, S = 256, D = 128;
  const std::vector<int64_t> shape{B, H, S, D}, bshd{S * H * D, D, H * D, 1};
  auto Q = graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, bshd);
  auto K = graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, bshd);
  auto V = graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, bshd);
  auto Obuf = graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, bshd);
  CHECK(bool(Q) && Q.strides() == bshd && !graph.data->tensors[Q.id].dense());
  auto dense = graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, std::vector<int64_t>{H * S * D, S * D, D, 1});
  CHECK(bool(dense) && graph.data->tensors[dense.id].dense());       // row-major strides are the default layout
  CHECK(!graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, std::vector<int64_t>{1, 2, 3}));      // one per dim
  CHECK(!graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, std::vector<int64_t>{8, 8, 8, 2}));   // innermost 1
  auto Sc = graph.create<BatchedMatmul>(Q, Layout::rowMajor, K, Layout::colMajor);
  auto P = graph.create<Softmax>(Sc, -1, MemorySpace::inplace, "", 0.0883883f, true);
  auto O = graph.create<BatchedMatmul>(P, Layout::rowMajor, V, Layout::rowMajor, "", Obuf);
  CHECK(bool(O) && O.strides() == bshd && graph.data->root(O.id) == Obuf.id);
  // every other operator takes dense tensors only
  CHECK(!graph.create<ElementWise>(Q, "Gelu", MemorySpace::global));
  CHECK(!graph.create<Binary>(Q, Q, "Add"));
  // out must be a PlaceHolder of the result's shape and type
  CHECK(!graph.create<BatchedMatmul>(P, Layout::rowMajor, V, Layout::rowMajor, "", Sc));
  auto module = generator.optimize(graph);
  auto plan = generator.codegen(module);
  CHECK(module.calls.size() == 1 && module.calls[0].entry == "kcg_fmha_fwd");
  // unfused, the strided operands have no single batch stride: run() must refuse, not mis-address
  KernelCodeGenerator plain("CUDA");
  plain.opts.push_back(std::make_unique<BatchMatmulOptimizer>());
  plain.opts.push_back(std::make_unique<SoftmaxOptimizer>());
  auto m2 = plain.optimize(graph);
  CHECK(m2.calls.size() == 3);
  Bindings bind;
  int dummy[4];
  for (int t = 0; t < static_cast<int>(graph.data->tensors.size()); ++t) bind.ptrs[t] = dummy;
  CHECK(plain.run(m2, bind) == KCG_ERR_UNSUPPORTED);
}

static void test_shard_spec_validation() {
  KernelCodeGenerator generator("CUDA");
  generator.opts.push_back(std::make_unique<ElementWiseOptimizer>());
  auto graph = generator.createGraph("shard");
  auto A = graph.create<PlaceHolder>(std::vector<int64_t>{4, 5}, std::string{"float32"});
  auto C = graph.create<ElementWise>(A, "Gelu", MemorySpace::global);
  (void)C;
  auto module = generator.optimize(graph);
  Bindings bind;
  ShardSpec bad;
  bad.world = 2; bad.rank = 2;
  CHECK(generator.run(module, bind, bad) == KCG_ERR_INVALID_ARG);
  ShardSpec no_comm;
  no_comm.world = 2; no_comm.rank = 0; no_comm.gather = true;
  CHECK(generator.run(module, bind, no_comm) == KCG_ERR_INVALID_ARG);
  // the C entry refuses bad arguments before it looks for NCCL
  CHECK(kcg_shard_allgather(nullptr, 8, 4, 1, 2, 0, nullptr, nullptr) == KCG_ERR_INVALID_ARG);
  CHECK(kcg_shard_allgather(nullptr, 8, 0, 1, 2, 0, nullptr, nullptr) == KCG_ERR_INVALID_ARG);
  CHECK(kcg_shard_allgather(nullptr, 0, 4, 1, 2, 0, nullptr, nullptr) == KCG_OK);   // nothing to exchange
  CHECK(kcg_shard_allgather(nullptr, 8, 4, 1, 1, 0, nullptr, nullptr) == KCG_OK);   // one rank
}

// ---------------------------------------------------------------------------------- gpu mode
extern "C" {
int cudaMalloc(void**, size_t);
int cudaFree(void*);
int cudaMemcpy(void*, const void*, size_t, int);
int cudaDeviceSynchronize(void);
// CPU oracle (oracle/kcg_oracle.c)
void oracle_matmul_f32(const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t, int64_t, int);
void oracle_layernorm_f32(const float*, const float*, const float*, float*, int64_t, int64_t, float, int);
void oracle_unary_f32(int, const float*, float*, int64_t, int);
int64_t oracle_binary_f32(int, int, const int64_t*, int, const int64_t*, const float*, const float*, float*);
void oracle_attention_f32(const float*, const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t, int64_t,
                          float, int, const int64_t*, const int64_t*, const int64_t*, const int64_t*, int64_t, int64_t, int);
}

static std::vector<float> randn(size_t n, unsigned seed, float std_ = 1.f, float mean = 0.f) {
  std::mt19937 gen(seed);
  std::normal_distribution<float> d(mean, std_);
  std::vector<float> v(n);
  for (auto& x : v) x = d(gen);
  return v;
}
static void* upload(const void* h, size_t bytes) {
  void* d = nullptr;
  if (cudaMalloc(&d, bytes) != 0) { std::fprintf(stderr, "cudaMalloc failed\n"); std::exit(2); }
  if (h) cudaMemcpy(d, h, bytes, 1);
  return d;
}
static std::vector<float> download(void* d, size_t n) {
  std::vector<float> v(n);
  cudaMemcpy(v.data(), d, n * 4, 2);
  return v;
}
static double rel_fro(const std::vector<float>& got, const std::vector<float>& want) {
  double num = 0, den = 0;
  for (size_t i = 0; i < want.size(); ++i) {
    num += (double(got[i]) - want[i]) * (double(got[i]) - want[i]);
    den += double(want[i]) * want[i];
  }
  return std::sqrt(num / (den > 0 ? den : 1));
}
static uint16_t to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  u += 0x7FFF + ((u >> 16) & 1);
  return uint16_t(u >> 16);
}
static float from_bf16(uint16_t h) {
  uint32_t u = uint32_t(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

static void gpu_matmul_relu() {  // Matmul -> Relu inplace, fp32 (test/test.cc:59-63 scaled down)
  KernelCodeGenerator generator("CUDA");
  auto graph = generator.createGraph("matmul_demo");
  generator.opts.push_back(std::make_unique<MatmulOptimizer>());
  generator.opts.push_back(std::make_unique<ElementWiseOptimizer>());
  const int m = 512, n = 256, k = 128;
  auto A = graph.create<PlaceHolder>(std::vector<int64_t>{m, k}, std::string{"float32"});
  auto B = graph.create<PlaceHolder>(std::vector<int64_t>{k, n}, std::string{"float32"});
  auto C = graph.create<Matmul>(A, B);
  auto D = graph.create<Relu>(C, MemorySpace::inplace);
  auto module = generator.optimize(graph);
  auto hA = randn(size_t(m) * k, 1), hB = randn(size_t(k) * n, 2);
  Bindings bind;
  void* dC = upload(nullptr, size_t(m) * n * 4);
  bind.set(A, upload(hA.data(), hA.size() * 4));
  bind.set(B, upload(hB.data(), hB.size() * 4));
  bind.set(C, dC);  // D aliases C
  CHECK(generator.run(module, bind) == KCG_OK);
  cudaDeviceSynchronize();
  std::vector<float> want(size_t(m) * n), relu(size_t(m) * n);
  oracle_matmul_f32(hA.data(), hB.data(), want.data(), m, n, k, 0, m, 0);
  oracle_unary_f32(3, want.data(), relu.data(), relu.size(), 0);
  CHECK(rel_fro(download(dC, relu.size()), relu) <= 1e-5);
  (void)D;
}

static void gpu_layernorm_gelu_add() {  // the headline chain through the graph API, fp32
  KernelCodeGenerator generator("CUDA");
  auto graph = generator.createGraph("ln_gelu_add");
  generator.opts.push_back(std::make_unique<LayerNormOptimizer>());
  generator.opts.push_back(std::make_unique<ElementWiseOptimizer>());
  generator.opts.push_back(std::make_unique<BinaryOptimizer>());
  const int64_t rows = 96, cols = 4096;
  auto X = graph.create<PlaceHolder>(std::vector<int64_t>{rows, cols}, std::string{"float32"});
  auto G = graph.create<PlaceHolder>(std::vector<int64_t>{cols}, std::string{"float32"});
  auto Bt = graph.create<PlaceHolder>(std::vector<int64_t>{cols}, std::string{"float32"});
  auto R = graph.create<PlaceHolder>(std::vector<int64_t>{rows, cols}, std::string{"float32"});
  auto Y = graph.create<LayerNorm>(X, G, Bt, int64_t(-1));
  auto Z = graph.create<ElementWise>(Y, "Gelu", MemorySpace::global);
  auto W = graph.create<Binary>(Z, R, "Add");
  auto module = generator.optimize(graph);
  CHECK(module.calls.size() == 3);
  auto hX = randn(rows * cols, 3), hG = randn(cols, 4, 0.1f, 1.f), hB = randn(cols, 5, 0.1f), hR = randn(rows * cols, 6);
  Bindings bind;
  void* dW = upload(nullptr, rows * cols * 4);
  bind.set(X, upload(hX.data(), hX.size() * 4));
  bind.set(G, upload(hG.data(), hG.size() * 4));
  bind.set(Bt, upload(hB.data(), hB.size() * 4));
  bind.set(R, upload(hR.data(), hR.size() * 4));
  bind.set(Y, upload(nullptr, rows * cols * 4));
  bind.set(Z, upload(nullptr, rows * cols * 4));
  bind.set(W, dW);
  CHECK(generator.run(module, bind) == KCG_OK);
  cudaDeviceSynchronize();
  std::vector<float> y(rows * cols), z(rows * cols), w(rows * cols);
  oracle_layernorm_f32(hX.data(), hG.data(), hB.data(), y.data(), rows, cols, 1e-5f, 0);
  oracle_unary_f32(5, y.data(), z.data(), z.size(), 0);
  const int64_t sh[2] = {rows, cols};
  oracle_binary_f32(0, 2, sh, 2, sh, z.data(), hR.data(), w.data());
  CHECK(rel_fro(download(dW, w.size()), w) <= 1e-5);
}

static void gpu_kernel_fusion() {  // LayerNorm -> Gelu -> Add fused by KernelFusionOptimizer, fp32
  KernelCodeGenerator generator("CUDA");
  auto graph = generator.createGraph("ln_gelu_add_fused");
  generator.opts.push_back(std::make_unique<KernelFusionOptimizer>());
  const int64_t rows = 96, cols = 4096;
  auto X = graph.create<PlaceHolder>(std::vector<int64_t>{rows, cols}, std::string{"float32"});
  auto G = graph.create<PlaceHolder>(std::vector<int64_t>{cols}, std::string{"float32"});
  auto Bt = graph.create<PlaceHolder>(std::vector<int64_t>{cols}, std::string{"float32"});
  auto R = graph.create<PlaceHolder>(std::vector<int64_t>{rows, cols}, std::string{"float32"});
  auto Y = graph.create<LayerNorm>(X, G, Bt, int64_t(-1));
  auto Z = graph.create<ElementWise>(Y, "Gelu", MemorySpace::global);
  auto W = graph.create<Binary>(Z, R, "Add");
  auto module = generator.optimize(graph);
  CHECK(module.calls.size() == 1 && module.calls[0].entry == "kcg_layernorm_gelu_add");
  auto hX = randn(rows * cols, 13), hG = randn(cols, 14, 0.1f, 1.f), hB = randn(cols, 15, 0.1f), hR = randn(rows * cols, 16);
  Bindings bind;
  void* dW = upload(nullptr, rows * cols * 4);
  bind.set(X, upload(hX.data(), hX.size() * 4));
  bind.set(G, upload(hG.data(), hG.size() * 4));
  bind.set(Bt, upload(hB.data(), hB.size() * 4));
  bind.set(R, upload(hR.data(), hR.size() * 4));
  bind.set(W, dW);  // Y and Z never exist in memory
  CHECK(generator.run(module, bind) == KCG_OK);
  cudaDeviceSynchronize();
  std::vector<float> y(rows * cols), z(rows * cols), w(rows * cols);
  oracle_layernorm_f32(hX.data(), hG.data(), hB.data(), y.data(), rows, cols, 1e-5f, 0);
  oracle_unary_f32(5, y.data(), z.data(), z.size(), 0);
  const int64_t sh[2] = {rows, cols};
  oracle_binary_f32(0, 2, sh, 2, sh, z.data(), hR.data(), w.data());
  CHECK(rel_fro(download(dW, w.size()), w) <= 1e-5);
  // Matmul -> Relu(inplace) fused into the GEMM epilogue; the pointer is bound to C only
  auto g2 = generator.createGraph("matmul_relu_fused");
  const int m = 256, n = 128, k = 64;
  auto A = g2.create<PlaceHolder>(std::vector<int64_t>{m, k}, std::string{"float32"});
  auto B = g2.create<PlaceHolder>(std::vector<int64_t>{k, n}, std::string{"float32"});
  auto C = g2.create<Matmul>(A, B);
  auto D = g2.create<Relu>(C, MemorySpace::inplace);
  (void)D;
  auto m2 = generator.optimize(g2);
  CHECK(m2.calls.size() == 1 && m2.calls[0].entry == "kcg_gemm");
  auto hA = randn(size_t(m) * k, 17), hBm = randn(size_t(k) * n, 18);
  Bindings b2;
  void* dC = upload(nullptr, size_t(m) * n * 4);
  b2.set(A, upload(hA.data(), hA.size() * 4));
  b2.set(B, upload(hBm.data(), hBm.size() * 4));
  b2.set(C, dC);
  CHECK(generator.run(m2, b2) == KCG_OK);
  cudaDeviceSynchronize();
  std::vector<float> want(size_t(m) * n), relu(size_t(m) * n);
  oracle_matmul_f32(hA.data(), hBm.data(), want.data(), m, n, k, 0, m, 0);
  oracle_unary_f32(3, want.data(), relu.data(), relu.size(), 0);
  CHECK(rel_fro(download(dC, relu.size()), relu) <= 1e-5);
}

static void gpu_fused_attention() {  // BatchedMatmul -> Softmax -> BatchedMatmul, bf16, fused
  KernelCodeGenerator generator("CUDA");
  auto graph = generator.createGraph("flash_attn_demo");
  generator.opts.push_back(std::make_unique<FMHAOptimizer>());
  const int64_t B = 2, H = 3, S = 256, D = 64;
  auto Q = graph.create<PlaceHolder>(std::vector<int64_t>{B, H, S, D}, std::string{"bfloat16"});
  auto K = graph.create<PlaceHolder>(std::vector<int64_t>{B, H, S, D}, std::string{"bfloat16"});
  auto V = graph.create<PlaceHolder>(std::vector<int64_t>{B, H, S, D}, std::string{"bfloat16"});
  auto Sc = graph.create<BatchedMatmul>(Q, Layout::rowMajor, K, Layout::colMajor);
  auto P = graph.create<Softmax>(Sc, -1, MemorySpace::inplace, "", 0.125f, true);
  auto O = graph.create<BatchedMatmul>(P, Layout::rowMajor, V, Layout::rowMajor);
  auto module = generator.optimize(graph);
  CHECK(module.calls.size() == 1 && module.calls[0].entry == "kcg_fmha_fwd");
  const size_t n = size_t(B) * H * S * D;
  auto fq = randn(n, 7), fk = randn(n, 8), fv = randn(n, 9);
  std::vector<uint16_t> hq(n), hk(n), hv(n);
  for (size_t i = 0; i < n; ++i) {
    hq[i] = to_bf16(fq[i]); hk[i] = to_bf16(fk[i]); hv[i] = to_bf16(fv[i]);
    fq[i] = from_bf16(hq[i]); fk[i] = from_bf16(hk[i]); fv[i] = from_bf16(hv[i]);
  }
  Bindings bind;
  void* dO = upload(nullptr, n * 2);
  bind.set(Q, upload(hq.data(), n * 2));
  bind.set(K, upload(hk.data(), n * 2));
  bind.set(V, upload(hv.data(), n * 2));
  bind.set(O, dO);  // the scores and probabilities never exist in memory
  CHECK(generator.run(module, bind) == KCG_OK);
  cudaDeviceSynchronize();
  CHECK(kcg_device_status() == KCG_OK);
  std::vector<uint16_t> ho(n);
  cudaMemcpy(ho.data(), dO, n * 2, 2);
  std::vector<float> got(n), want(n);
  for (size_t i = 0; i < n; ++i) got[i] = from_bf16(ho[i]);
  const int64_t st[3] = {H * S * D, S * D, D};
  oracle_attention_f32(fq.data(), fk.data(), fv.data(), want.data(), B, H, S, S, D, 0.125f, 1, st, st, st, st, 0, B * H, 0);
  CHECK(rel_fro(got, want) <= 1e-2);
}

static void gpu_gather_transpose() {  // embedding-style row gather, then a transpose, fp32
  KernelCodeGenerator generator("CUDA");
  generator.opts.push_back(std::make_unique<GatherOptimizer>());
  generator.opts.push_back(std::make_unique<TransposeOptimizer>());
  auto graph = generator.createGraph("gather_run");
  const int rows = 300, cols = 72, n = 129;
  auto A = graph.create<PlaceHolder>(std::vector<int64_t>{rows, cols}, std::string{"float32"});
  auto I = graph.create<PlaceHolder>(std::vector<int64_t>{n}, std::string{"int32"});
  auto G = graph.create<Gather>(A, I);
  auto T = graph.create<Transpose>(G);
  auto module = generator.optimize(graph);
  auto hA = randn(size_t(rows) * cols, 31);
  std::vector<int32_t> hI(n);
  for (int i = 0; i < n; ++i) hI[i] = (i * 37 + 11) % rows;
  void* dG = upload(nullptr, size_t(n) * cols * 4);
  void* dT = upload(nullptr, size_t(n) * cols * 4);
  Bindings bind;
  bind.set(A, upload(hA.data(), hA.size() * 4));
  bind.set(I, upload(hI.data(), hI.size() * 4));
  bind.set(G, dG);
  bind.set(T, dT);
  CHECK(generator.run(module, bind) == KCG_OK);
  cudaDeviceSynchronize();
  CHECK(kcg_device_status() == KCG_OK);
  auto g = download(dG, size_t(n) * cols), t = download(dT, size_t(n) * cols);
  bool ok = true;
  for (int i = 0; i < n && ok; ++i)
    for (int c = 0; c < cols; ++c) {
      const float want = hA[size_t(hI[i]) * cols + c];   // the reference's loop nest, Operators.cc:1320-1340
      if (g[size_t(i) * cols + c] != want || t[size_t(c) * n + i] != want) { ok = false; break; }
    }
  CHECK(ok);
}

// Every candidate is timed on the device and the fastest kept.  The GEMM tile shapes accumulate in one
// order, so the product is the same bits whatever was chosen; the LayerNorm block shapes sum a row in
// different orders, so that output is held to the operator's tolerance instead.
static void gpu_autotune() {
  auto build = [](KernelCodeGenerator& generator, Value& A, Value& B, Value& gm, Value& C, Value& Y) {
    generator.opts.push_back(std::make_unique<MatmulOptimizer>());
    generator.opts.push_back(std::make_unique<LayerNormOptimizer>());
    auto graph = generator.createGraph("tuned");
    A = graph.create<PlaceHolder>(std::vector<int64_t>{1024, 512}, std::string{"bfloat16"});
    B = graph.create<PlaceHolder>(std::vector<int64_t>{512, 2048}, std::string{"bfloat16"});
    C = graph.create<Matmul>(A, B);
    gm = graph.create<PlaceHolder>(std::vector<int64_t>{2048}, std::string{"bfloat16"});
    Y = graph.create<LayerNorm>(C, gm, gm, int64_t(1), 1e-5f);
    return graph;
  };
  auto hA32 = randn(size_t(1024) * 512, 51), hB32 = randn(size_t(512) * 2048, 52), hg32 = randn(2048, 53);
  std::vector<uint16_t> hA(hA32.size()), hB(hB32.size()), hg(hg32.size());
  for (size_t i = 0; i < hA.size(); ++i) hA[i] = to_bf16(hA32[i] * 0.05f);
  for (size_t i = 0; i < hB.size(); ++i) hB[i] = to_bf16(hB32[i]);
  for (size_t i = 0; i < hg.size(); ++i) hg[i] = to_bf16(1.0f + 0.1f * hg32[i]);
  std::vector<std::vector<uint16_t>> results, products;
  for (int tuned = 0; tuned < 2; ++tuned) {
    KernelCodeGenerator generator("CUDA");
    generator.autotune = tuned == 1;
    Value A, B, gm, C, Y;
    auto graph = build(generator, A, B, gm, C, Y);
    auto module = generator.optimize(graph);
    if (tuned) {
      CHECK(generator.bestLatency() > 0.0f && generator.bestLatency() < 1e3f);   // a measured time, in ms
      const auto& cfg = module.graph->funcs.at("LayerNorm_1024_2048_axis_1_bfloat16").config;
      bool known = false;
      for (const auto& cand : *generator.configs("LayerNorm")) known = known || cand == cfg;
      CHECK(known);
      std::printf("autotune kept CTA_PAIR=%d WARP_ROW_VECS=%d, %.4f ms\n",
                  module.graph->funcs.at("Matmul_m1024n2048k512_bfloat16").config.at("CTA_PAIR"), cfg.at("WARP_ROW_VECS"),
                  generator.bestLatency());
    }
    Bindings bind;
    void* dY = upload(nullptr, size_t(1024) * 2048 * 2);
    bind.set(A, upload(hA.data(), hA.size() * 2));
    bind.set(B, upload(hB.data(), hB.size() * 2));
    bind.set(gm, upload(hg.data(), hg.size() * 2));
    void* dC = upload(nullptr, size_t(1024) * 2048 * 2);
    bind.set(C, dC);
    bind.set(Y, dY);
    CHECK(generator.run(module, bind) == KCG_OK);
    cudaDeviceSynchronize();
    CHECK(kcg_device_status() == KCG_OK);
    std::vector<uint16_t> out(size_t(1024) * 2048), prod(size_t(1024) * 2048);
    cudaMemcpy(out.data(), dY, out.size() * 2, 2);
    cudaMemcpy(prod.data(), dC, prod.size() * 2, 2);
    results.push_back(out);
    products.push_back(prod);
  }
  CHECK(products[0] == products[1]);
  std::vector<float> y0(results[0].size()), y1(results[1].size());
  for (size_t i = 0; i < y0.size(); ++i) { y0[i] = from_bf16(results[0][i]); y1[i] = from_bf16(results[1][i]); }
  CHECK(rel_fro(y1, y0) <= 1e-2);
}

static void gpu_fused_attention_bshd() {
  // The attention benchmark's layout through the graph API: Q, K, V held as [B,S,H,D], O written
  // as [B,S,H,D], all declared as [B,H,S,D] views with strides; bf16, D = 128, causal, scaled.
  KernelCodeGenerator generator("CUDA");
  generator.opts.push_back(std::make_unique<FMHAOptimizer>());
  auto graph = generator.createGraph("attn_bshd");
  const int64_t B = 2, H = 4, S = 384, D = 128;
  const std::vector<int64_t> shape{B, H, S, D}, bshd{S * H * D, D, H * D, 1};
  auto Q = graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, bshd);
  auto K = graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, bshd);
  auto V = graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, bshd);
  auto Ob = graph.create<PlaceHolder>(shape, std::string{"bfloat16"}, bshd);
  const float scale = 1.0f / std::sqrt(float(D));
  auto Sc = graph.create<BatchedMatmul>(Q, Layout::rowMajor, K, Layout::colMajor);
  auto P = graph.create<Softmax>(Sc, -1, MemorySpace::inplace, "", scale, true);
  auto O = graph.create<BatchedMatmul>(P, Layout::rowMajor, V, Layout::rowMajor, "", Ob);
  auto module = generator.optimize(graph);
  CHECK(bool(O) && module.calls.size() == 1 && module.calls[0].entry == "kcg_fmha_fwd");
  const size_t n = size_t(B) * H * S * D;
  auto fq = randn(n, 71), fk = randn(n, 72), fv = randn(n, 73);
  std::vector<uint16_t> hq(n), hk(n), hv(n);
  for (size_t i = 0; i < n; ++i) {
    hq[i] = to_bf16(fq[i]); hk[i] = to_bf16(fk[i]); hv[i] = to_bf16(fv[i]);
    fq[i] = from_bf16(hq[i]); fk[i] = from_bf16(hk[i]); fv[i] = from_bf16(hv[i]);
  }
  Bindings bind;
  void* dO = upload(nullptr, n * 2);
  bind.set(Q, upload(hq.data(), n * 2));
  bind.set(K, upload(hk.data(), n * 2));
  bind.set(V, upload(hv.data(), n * 2));
  bind.set(Ob, dO);   // O names Ob's storage
  CHECK(generator.run(module, bind) == KCG_OK);
  cudaDeviceSynchronize();
  CHECK(kcg_device_status() == KCG_OK);
  std::vector<uint16_t> ho(n);
  cudaMemcpy(ho.data(), dO, n * 2, 2);
  std::vector<float> got(n), want(n);
  for (size_t i = 0; i < n; ++i) got[i] = from_bf16(ho[i]);
  const int64_t st[3] = {S * H * D, D, H * D};   // (batch, head, sequence) strides of a [B,S,H,D] buffer
  oracle_attention_f32(fq.data(), fk.data(), fv.data(), want.data(), B, H, S, S, D, scale, 1, st, st, st, st, 0, B * H, 0);
  CHECK(rel_fro(got, want) <= 1e-2);
}

// One generator per "rank" on one GPU, no collective: rank r of `world` writes only its block of
// each output, so running the ranks one after the other on the same full-size buffers must
// reproduce the unsharded run bit for bit.  This checks every operator's pointer arithmetic.
// (Without the gather a chain is only valid while all its operators cut the rows alike, so the
// row-wise chain and the GEMMs, whose rows go in granules of 128, are separate graphs here.)
static void gpu_sharded_run_matches_unsharded() {
  const int64_t rows = 1000, cols = 512, n = 384, nb = 5;
  auto hx32 = randn(rows * cols, 81), hg32 = randn(cols, 82, 0.1f, 1.f), hw32 = randn(cols * n, 83, 0.05f);
  std::vector<uint16_t> hx(hx32.size()), hg(hg32.size()), hw(hw32.size());
  for (size_t i = 0; i < hx.size(); ++i) hx[i] = to_bf16(hx32[i]);
  for (size_t i = 0; i < hg.size(); ++i) hg[i] = to_bf16(hg32[i]);
  for (size_t i = 0; i < hw.size(); ++i) hw[i] = to_bf16(hw32[i]);
  void* dX = upload(hx.data(), hx.size() * 2);
  void* dG = upload(hg.data(), hg.size() * 2);
  void* dW = upload(hw.data(), hw.size() * 2);
  std::vector<std::vector<uint16_t>> outs[3];
  for (int world : {1, 3}) {
    auto run_all = [&](KernelCodeGenerator& generator, Module& module, Bindings& bind) {
      for (int r = 0; r < world; ++r) {
        ShardSpec spec;
        spec.world = world; spec.rank = r;
        CHECK(generator.run(module, bind, spec) == KCG_OK);
      }
      cudaDeviceSynchronize();
      CHECK(kcg_device_status() == KCG_OK);
    };
    auto fetch = [&](void* d, size_t count) {
      std::vector<uint16_t> out(count);
      cudaMemcpy(out.data(), d, count * 2, 2);
      return out;
    };
    auto fresh = [&](size_t count) {
      void* p = upload(nullptr, count * 2);
      kcg_device_memset(p, 0xFF, count * 2, nullptr);
      return p;
    };
    {  // row-wise chain: 1000 rows over 3 ranks = 334 + 333 + 333
      KernelCodeGenerator generator("CUDA");
      generator.opts.push_back(std::make_unique<LayerNormOptimizer>());
      generator.opts.push_back(std::make_unique<ElementWiseOptimizer>());
      generator.opts.push_back(std::make_unique<BinaryOptimizer>());
      generator.opts.push_back(std::make_unique<SoftmaxOptimizer>());
      auto graph = generator.createGraph("rows");
      auto X = graph.create<PlaceHolder>(std::vector<int64_t>{rows, cols}, std::string{"bfloat16"});
      auto G = graph.create<PlaceHolder>(std::vector<int64_t>{cols}, std::string{"bfloat16"});
      auto Y = graph.create<LayerNorm>(X, G, G, int64_t(1));
      auto Z = graph.create<ElementWise>(Y, "Gelu", MemorySpace::global);
      auto A = graph.create<Binary>(Z, X, "Add");      // same-shape operand
      auto M = graph.create<Binary>(A, G, "Mul");      // row-broadcast operand
      auto S = graph.create<Softmax>(M);               // in place
      (void)S;
      auto module = generator.optimize(graph);
      Bindings bind;
      bind.set(X, dX); bind.set(G, dG);
      bind.set(Y, fresh(rows * cols)); bind.set(Z, fresh(rows * cols)); bind.set(A, fresh(rows * cols));
      void* dM = fresh(rows * cols);
      bind.set(M, dM);
      run_all(generator, module, bind);
      outs[0].push_back(fetch(dM, rows * cols));
    }
    {  // Matmul with a fused Relu: 1000 rows in granules of 128 = 384 + 384 + 232
      KernelCodeGenerator generator("CUDA");
      generator.opts.push_back(std::make_unique<KernelFusionOptimizer>());
      generator.opts.push_back(std::make_unique<MatmulOptimizer>());
      auto graph = generator.createGraph("gemm");
      auto X = graph.create<PlaceHolder>(std::vector<int64_t>{rows, cols}, std::string{"bfloat16"});
      auto W = graph.create<PlaceHolder>(std::vector<int64_t>{cols, n}, std::string{"bfloat16"});
      auto C = graph.create<Matmul>(X, W);
      auto R = graph.create<Relu>(C, MemorySpace::inplace);
      (void)R;
      auto module = generator.optimize(graph);
      Bindings bind;
      void* dC = fresh(rows * n);
      bind.set(X, dX); bind.set(W, dW); bind.set(C, dC);
      run_all(generator, module, bind);
      outs[1].push_back(fetch(dC, rows * n));
    }
    {  // BatchedMatmul NT: 5 matrices over 3 ranks = 2 + 2 + 1
      KernelCodeGenerator generator("CUDA");
      generator.opts.push_back(std::make_unique<BatchMatmulOptimizer>());
      auto graph = generator.createGraph("bmm");
      const int64_t bm = rows / nb;   // 200 rows per matrix out of the same buffer
      auto A = graph.create<PlaceHolder>(std::vector<int64_t>{nb, bm, cols}, std::string{"bfloat16"});
      auto C = graph.create<BatchedMatmul>(A, Layout::rowMajor, A, Layout::colMajor);
      auto module = generator.optimize(graph);
      Bindings bind;
      void* dC = fresh(nb * bm * bm);
      bind.set(A, dX); bind.set(C, dC);
      run_all(generator, module, bind);
      outs[2].push_back(fetch(dC, nb * bm * bm));
    }
  }
  for (int g = 0; g < 3; ++g) CHECK(outs[g].size() == 2 && outs[g][0] == outs[g][1]);
  // nothing was left unwritten (the buffers started as 0xFFFF words, a bf16 NaN)
  bool filled = true;
  for (int g = 0; g < 3; ++g)
    for (uint16_t w : outs[g][0]) filled = filled && w != 0xFFFF;
  CHECK(filled);
}

// Two host threads, each with its own generator whose optimizer picked a different GEMM tile
// (a setting of the calling thread in the kernel library), run at the same time on their own
// streams: neither may see the other's setting, and both must give the bits of a lone run.
extern "C" {
int cudaStreamCreate(void**);
int cudaStreamSynchronize(void*);
}
#include <thread>
static void gpu_two_generators_two_threads() {
  const int m = 1024, n = 1024, k = 512;
  auto hA32 = randn(size_t(m) * k, 91, 0.05f), hB32 = randn(size_t(k) * n, 92);
  std::vector<uint16_t> hA(hA32.size()), hB(hB32.size());
  for (size_t i = 0; i < hA.size(); ++i) hA[i] = to_bf16(hA32[i]);
  for (size_t i = 0; i < hB.size(); ++i) hB[i] = to_bf16(hB32[i]);
  void* dA = upload(hA.data(), hA.size() * 2);
  void* dB = upload(hB.data(), hB.size() * 2);
  std::vector<uint16_t> out[2];
  int status[2] = {-1, -1};
  auto worker = [&](int which) {
    KernelCodeGenerator generator("CUDA");
    generator.opts.push_back(std::make_unique<MatmulOptimizer>());
    // thread 0 keeps the first candidate (CTA pairs), thread 1 only has the 128x128 single-CTA tile
    if (which == 1) {
      auto* table = generator.configs("Matmul");
      auto narrow = table->back();
      table->clear();
      table->push_back(narrow);
    }
    auto graph = generator.createGraph("mt");
    auto A = graph.create<PlaceHolder>(std::vector<int64_t>{m, k}, std::string{"bfloat16"});
    auto B = graph.create<PlaceHolder>(std::vector<int64_t>{k, n}, std::string{"bfloat16"});
    auto C = graph.create<Matmul>(A, B);
    auto module = generator.optimize(graph);
    void* stream = nullptr;
    cudaStreamCreate(&stream);
    void* dC = upload(nullptr, size_t(m) * n * 2);
    Bindings bind;
    bind.set(A, dA); bind.set(B, dB); bind.set(C, dC);
    int rc = KCG_OK;
    for (int i = 0; i < 200 && rc == KCG_OK; ++i) rc = generator.run(module, bind, stream);
    cudaStreamSynchronize(stream);
    status[which] = rc;
    out[which].resize(size_t(m) * n);
    cudaMemcpy(out[which].data(), dC, out[which].size() * 2, 2);
  };
  std::thread t0(worker, 0), t1(worker, 1);
  t0.join();
  t1.join();
  CHECK(status[0] == KCG_OK && status[1] == KCG_OK && kcg_device_status() == KCG_OK);
  CHECK(out[0] == out[1]);   // every tile shape accumulates in the same order
}

// Run by two (or more) processes, one per GPU: `test_frontend shard <world> <rank> <id file>`.
// Each builds the same graph, runs it sharded with the in-place NCCL gather after every operator,
// and compares every rank's full result with an unsharded run on its own GPU, bit for bit.
extern "C" int cudaSetDevice(int);
#include <chrono>
#include <fstream>
static int shard_main(int world, int rank, const std::string& id_file) {
  if (cudaSetDevice(rank) != 0) { std::fprintf(stderr, "cudaSetDevice(%d) failed\n", rank); return 2; }
  unsigned char id[128];
  if (rank == 0) {
    if (kcg_nccl_unique_id(id) != KCG_OK) { std::fprintf(stderr, "%s\n", kcg_last_error()); return 2; }
    std::ofstream w(id_file + ".tmp", std::ios::binary);
    w.write(reinterpret_cast<const char*>(id), 128);
    w.close();
    std::rename((id_file + ".tmp").c_str(), id_file.c_str());
  } else {
    bool got = false;
    for (int i = 0; i < 600 && !got; ++i) {
      std::ifstream r(id_file, std::ios::binary);
      if (r && r.read(reinterpret_cast<char*>(id), 128)) got = true;
      else std::this_thread::sleep_for(std::chrono::milliseconds(100));
    }
    if (!got) { std::fprintf(stderr, "rank %d: no NCCL id\n", rank); return 2; }
  }
  void* comm = nullptr;
  if (kcg_nccl_comm_create(world, rank, id, &comm) != KCG_OK) { std::fprintf(stderr, "%s\n", kcg_last_error()); return 2; }
  const int64_t rows = 1000, cols = 512, n = 384;
  auto hx32 = randn(rows * cols, 81), hg32 = randn(cols, 82, 0.1f, 1.f), hw32 = randn(cols * n, 83, 0.05f);
  std::vector<uint16_t> hx(hx32.size()), hg(hg32.size()), hw(hw32.size());
  for (size_t i = 0; i < hx.size(); ++i) hx[i] = to_bf16(hx32[i]);
  for (size_t i = 0; i < hg.size(); ++i) hg[i] = to_bf16(hg32[i]);
  for (size_t i = 0; i < hw.size(); ++i) hw[i] = to_bf16(hw32[i]);
  std::vector<uint16_t> outs[2];
  for (int pass = 0; pass < 2; ++pass) {   // 0: unsharded, 1: sharded with gather
    KernelCodeGenerator generator("CUDA");
    generator.opts.push_back(std::make_unique<LayerNormOptimizer>());
    generator.opts.push_back(std::make_unique<MatmulOptimizer>());
    generator.opts.push_back(std::make_unique<ElementWiseOptimizer>());
    auto graph = generator.createGraph("sharded");
    auto X = graph.create<PlaceHolder>(std::vector<int64_t>{rows, cols}, std::string{"bfloat16"});
    auto G = graph.create<PlaceHolder>(std::vector<int64_t>{cols}, std::string{"bfloat16"});
    auto W = graph.create<PlaceHolder>(std::vector<int64_t>{cols, n}, std::string{"bfloat16"});
    auto Y = graph.create<LayerNorm>(X, G, G, int64_t(1));
    auto C = graph.create<Matmul>(Y, W);              // rows cut in granules of 128: ragged blocks
    auto Z = graph.create<ElementWise>(C, "Gelu", MemorySpace::global);   // rows cut evenly
    auto module = generator.optimize(graph);
    Bindings bind;
    bind.set(X, upload(hx.data(), hx.size() * 2));
    bind.set(G, upload(hg.data(), hg.size() * 2));
    bind.set(W, upload(hw.data(), hw.size() * 2));
    bind.set(Y, upload(nullptr, rows * cols * 2));
    bind.set(C, upload(nullptr, rows * n * 2));
    void* dZ = upload(nullptr, rows * n * 2);
    kcg_device_memset(dZ, 0xFF, rows * n * 2, nullptr);
    bind.set(Z, dZ);
    int rc;
    if (pass == 0) {
      rc = generator.run(module, bind);
    } else {
      ShardSpec spec;
      spec.world = world; spec.rank = rank; spec.nccl_comm = comm; spec.gather = true;
      rc = generator.run(module, bind, spec);
    }
    CHECK(rc == KCG_OK);
    cudaDeviceSynchronize();
    CHECK(kcg_device_status() == KCG_OK);
    outs[pass].resize(rows * n);
    cudaMemcpy(outs[pass].data(), dZ, outs[pass].size() * 2, 2);
  }
  CHECK(outs[0] == outs[1]);
  CHECK(kcg_nccl_comm_destroy(comm) == KCG_OK);
  if (failures) return 1;
  std::printf("frontend shard rank %d of %d passed\n", rank, world);
  return 0;
}

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "cpu";
  if (mode == "shard" && argc == 5) return shard_main(std::atoi(argv[2]), std::atoi(argv[3]), argv[4]);
  if (mode == "cpu") {
    test_operators_cast();
    test_commented_sequences();
    test_flash_attention_graph();
    test_kernel_fusion();
    test_gather_transpose_graph();
    test_config_candidates_without_autotune();
    test_errors();
    test_dtype_is_part_of_the_function_key();
    test_strided_placeholders();
    test_shard_spec_validation();
  } else {
    gpu_matmul_relu();
    gpu_layernorm_gelu_add();
    gpu_kernel_fusion();
    gpu_fused_attention();
    gpu_fused_attention_bshd();
    gpu_sharded_run_matches_unsharded();
    gpu_two_generators_two_threads();
    gpu_gather_transpose();
    gpu_autotune();
  }
  if (failures) {
    std::fprintf(stderr, "%d check(s) failed\n", failures);
    return 1;
  }
  std::printf("frontend %s tests passed\n", mode.c_str());
  return 0;
}
