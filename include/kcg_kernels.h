/*
 * kcg_kernels.h — C ABI of the B200 (sm_100a) operator kernels.
 *
 * The reference project (KernelCodeGen) never executes a kernel itself: its
 * Optimizer + Backend print CUDA C source, one `__global__ kernelN(T* arg0, ...)`
 * per operator, whose parameters are flat row-major device pointers in
 * function-argument order followed by the outputs, with the static shape baked
 * into the text (src/Backend/CUDA.cc:1019-1064) and the launch geometry passed
 * out of band as a comment.  An external harness compiled and launched that
 * text.  This header is the replacement for that boundary: one entry point per
 * operator family, taking the same flat device pointers plus the shape the
 * reference baked in, and launching a hand-written sm_100a kernel.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller; nothing here
 *     synchronises the stream or copies to the host unless stated;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - every function returns a kcg_status (0 = success) and never aborts;
 *   - tensors are dense row-major unless a leading dimension / stride is given;
 *   - element counts and strides are in ELEMENTS, not bytes;
 *   - functions are re-entrant: they may be called from several host threads at
 *     once.  The tuning switches (kcg_*_set_*) are settings of the CALLING THREAD
 *     only: they affect the launches that thread makes afterwards and nothing else,
 *     so two threads can tune, or autotune, side by side;
 *   - kernels launched on different streams do not share state, except the
 *     per-device scratch buffers documented at kcg_layernorm() and
 *     kcg_gemm_set_fp32_mode().  Scratch rules: a scratch buffer that has been handed
 *     to a launch is never freed before the process exits (a larger request gets a
 *     new buffer and the old one is parked), so CUDA graphs captured earlier stay
 *     valid; a call that would have to GROW a scratch buffer while its stream is
 *     being captured returns KCG_ERR_UNSUPPORTED instead of allocating inside the
 *     capture — make one call of that size before capturing.
 */
#ifndef KCG_KERNELS_H_
#define KCG_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define KCG_API
#else
#define KCG_API __attribute__((visibility("default")))
#endif

/* dtype strings of the reference Frontend (src/Frontend/Operators.cc:5-15)
 * plus the two storage types the B200 configs add. */
typedef enum kcg_dtype {
  KCG_F32 = 0,    /* "float32"      */
  KCG_F16 = 1,    /* "float16"      */
  KCG_BF16 = 2,   /* "bfloat16"     (extension) */
  KCG_F8E4M3 = 3, /* "float8_e4m3"  (extension) */
  KCG_I32 = 4,    /* "int32"        (ElementWise "Cast" target) */
  KCG_F64 = 5,    /* "float64"      (accepted by the graph builder only) */
  KCG_I64 = 6,    /* "int64"        (accepted by the graph builder only) */
  KCG_I16 = 7,    /* "int16"        (accepted by the graph builder only) */
  KCG_BOOL = 8    /* "bool"         (accepted by the graph builder only) */
} kcg_dtype;

typedef enum kcg_status {
  KCG_OK = 0,
  KCG_ERR_INVALID_ARG = 1,  /* null pointer, non-positive size, bad enum      */
  KCG_ERR_UNSUPPORTED = 2,  /* legal request this build has no kernel for     */
  KCG_ERR_ALIGNMENT = 3,    /* pointer / leading dimension not 16-byte aligned */
  KCG_ERR_CUDA = 4,         /* a CUDA runtime / driver call failed            */
  KCG_ERR_TIMEOUT = 5,      /* a bounded device-side wait gave up             */
  KCG_ERR_NO_DEVICE = 6     /* no sm_100 device is current                    */
} kcg_status;

/* ElementWise::operationMap keys (src/Frontend/Operators.cc:997-1000). */
typedef enum kcg_unary_op {
  KCG_UNARY_TANH = 0,
  KCG_UNARY_SQRT = 1,
  KCG_UNARY_LOG = 2,
  KCG_UNARY_RELU = 3,
  KCG_UNARY_CAST = 4,
  KCG_UNARY_GELU = 5
} kcg_unary_op;

/* Binary::operationMap keys (src/Frontend/Operators.cc:609-612). */
typedef enum kcg_binary_op {
  KCG_BINARY_ADD = 0,
  KCG_BINARY_MUL = 1,
  KCG_BINARY_DIV = 2,
  KCG_BINARY_SUB = 3,
  KCG_BINARY_POW = 4,
  KCG_BINARY_EQUAL = 5,
  KCG_BINARY_GREATER = 6
} kcg_binary_op;

#define KCG_MAX_RANK 8

KCG_API const char* kcg_status_string(int status);
/* Text of the most recent failure on the calling thread ("" if none). */
KCG_API const char* kcg_last_error(void);
KCG_API int kcg_version(void);
/*
 * Kernels that wait on hardware barriers bound every wait; one that gives up stores a
 * kcg_status in a host-mapped word instead of hanging.  Call this after the stream has
 * been synchronised: it returns that word (KCG_OK if no kernel reported anything) and
 * clears it.
 */
KCG_API int kcg_device_status(void);
KCG_API size_t kcg_dtype_size(int dtype);

/*
 * LayerNorm — replaces the kernel emitted for `LayerNorm_{dims}_axis_{a}`
 * (builder: src/Frontend/Operators.cc:1076-1251; schedule:
 * src/Optimizer/Optimizer.cc:1802-1930).
 *
 *   rows = product of the dims before `axis`, cols = product of the dims from
 *   `axis` on.  For each row: mean = sum(x)/cols; d = x - mean;
 *   var = sum(d*d)/cols (biased); y = gamma * (d / sqrt(var + eps)) + beta.
 *   gamma and beta hold `cols` elements of the same dtype as x.  Statistics are
 *   accumulated in fp32 whatever the storage dtype.  y may alias x (the
 *   reference's MemorySpace::inplace).
 *
 *   dtype: KCG_F32, KCG_BF16 or KCG_F16.
 *
 *   Rows too long to be held on chip by one thread block are split over several
 *   blocks; that path keeps per-chunk statistics in a per-device scratch buffer
 *   that the library allocates (cudaMalloc) on first use and re-uses afterwards.
 *   Two such calls running concurrently on one device from different streams
 *   would share it: serialise them.
 */
KCG_API int kcg_layernorm(int dtype, int64_t rows, int64_t cols, const void* x,
                          const void* gamma, const void* beta, float eps, void* y,
                          void* stream);

/*
 * y = Gelu(LayerNorm(x)) + residual in one pass over memory — the fusion of the chain
 * LayerNorm -> ElementWise "Gelu" -> Binary "Add" that the reference's roadmap calls the
 * "KernelFusion Optimizer" (doc/Plan.md:68, :110; no implementation exists there).
 * x, residual and y are [rows, cols]; gamma and beta hold `cols` elements.  The value is
 * rounded to the storage dtype after each of the three steps, exactly where the separate
 * kernels would store it, so the result is bit-identical to calling kcg_layernorm,
 * kcg_eltwise(Gelu) and kcg_binary(Add) in turn, at 3 instead of 7 tensor passes.  y may
 * alias x or residual.  Rows the one-pass kernels do not take (longer than 32768 bf16 /
 * 16384 fp32 elements, or not 16-byte vectorisable) run as those three launches, in place in
 * y: for such rows y may still alias x but must not overlap residual (KCG_ERR_UNSUPPORTED).
 */
KCG_API int kcg_layernorm_gelu_add(int dtype, int64_t rows, int64_t cols, const void* x,
                                   const void* gamma, const void* beta, float eps,
                                   const void* residual, void* y, void* stream);

/*
 * LayerNorm through the split-row kernels, with no allocation of any kind.  This entry
 * point has no counterpart in the reference (which never runs a kernel, let alone manages
 * scratch memory).
 *
 * It is meant for callers that must not trigger a device allocation from inside a library
 * call: a process that has handed all of HBM to its own memory pool (so a hidden
 * cudaMalloc could fail), or a latency-critical loop in which cudaMalloc's implicit
 * device-wide synchronisation, and the chance of an out-of-memory error in the middle of
 * the loop, are not acceptable.  kcg_layernorm() may allocate (its split-row path grows a
 * cached per-device buffer); this function never calls cudaMalloc, cudaFree or any
 * allocating routine.
 *
 * Same arithmetic, arguments and result as kcg_layernorm(), always computed by the
 * split-row kernels: each row is cut into chunks of 8192 elements, a first kernel writes
 * the (mean, sum of squared deviations) of every chunk, a second merges them per row and
 * normalises.  The per-chunk statistics live in a fixed array inside the library image
 * (256 KiB of device memory on every GPU that loads the library, held until exit).
 *
 * Limit: rows * ceil(cols / 8192) <= 32768 and rows <= 65535; anything larger returns
 * KCG_ERR_UNSUPPORTED with an explanatory kcg_last_error().
 *
 * The first call on each device looks up the device address of that array (one
 * cudaGetSymbolAddress with that device current) and caches it; make that first call
 * before starting any stream capture on the device.  All calls on a device share the one
 * array and it keeps the previous call's contents; that is harmless because every entry
 * read is first rewritten by the same call, so nothing needs clearing — but two calls that
 * overlap on the GPU (different streams, or different host threads on one device) race on
 * it: serialise them.  The cached address belongs to the device's current primary context:
 * after a cudaDeviceReset() in the process it is stale and this entry point must not be
 * called again.
 */
KCG_API int kcg_layernorm_split_static(int dtype, int64_t rows, int64_t cols, const void* x,
                                       const void* gamma, const void* beta, float eps, void* y,
                                       void* stream);

/*
 * LayerNorm that also returns the per-row statistics, with optional scale and bias — the
 * argument list the reference's authors planned for the emitted kernel,
 * `(X, scale, bias, Y, mean, invStdDev)` (doc/pass.md:789-791, :806-822; the shipped builder
 * returns Y only, src/Frontend/Operators.cc:1076-1251).  y is computed exactly as by
 * kcg_layernorm (bit-identical for the same gamma/beta); mean[r] and inv_std[r] are the fp32
 * row mean and 1/sqrt(var + eps) it used, `rows` values each.  gamma == NULL means a scale of
 * one, beta == NULL a bias of zero; the library then reads a constant vector that it keeps
 * per device (allocated and filled, with one stream synchronisation, the first time a call
 * needs `cols` elements of it).
 */
KCG_API int kcg_layernorm_stats(int dtype, int64_t rows, int64_t cols, const void* x,
                                const void* gamma, const void* beta, float eps, void* y,
                                float* mean, float* inv_std, void* stream);

/*
 * Tuning switch with no counterpart in the reference: rows of up to 32 * vecs_per_lane
 * 16-byte vectors are normalised by one warp each (no block barrier); longer rows get one
 * thread block each.  Range 0..16, default 8.  A setting of the calling thread.
 */
KCG_API void kcg_layernorm_set_warp_row_limit(int vecs_per_lane);

/*
 * Tuning switch with no counterpart in the reference: the shape of the block-per-row kernel that
 * takes the rows too long for one warp.  A row is held by ceil(vectors / vecs_per_thread) threads
 * (vecs_per_thread 2, 4 or 8 16-byte vectors each; 0, the default, picks 4 for rows of up to 768
 * vectors and 8 beyond) and a thread block holds rows_per_block (1, the default, 2 or 4) such
 * groups, each with its own barrier; a negative rows_per_block runs a persistent grid of that
 * many blocks per SM, each prefetching its next row.  rows_per_block does not change the result;
 * vecs_per_thread changes the order in which the fp32 partial sums are added, so results agree
 * to rounding, not bit for bit.  A setting of the calling thread.
 */
KCG_API void kcg_layernorm_set_block_shape(int vecs_per_thread, int rows_per_block);

/*
 * Unary elementwise map — replaces `{Op}_Elementwise_{dims}` and
 * `Relu_Elementwise_{dims}` (builders: src/Frontend/Operators.cc:222-289 and
 * :1003-1074; schedule: src/Optimizer/Optimizer.cc:1080-1175).
 *
 *   Gelu is the tanh form with the reference's literal constants:
 *   0.5*x*(1 + tanh(0.797884*(x + 0.044715*x^3))).  Cast is a value conversion
 *   (the generated code prints static_cast, src/Backend/CUDA.cc:537-548);
 *   float -> int32 truncates toward zero.  For every op other than Cast
 *   dtype_out must equal dtype_in.  y may alias x when the dtypes have equal size.
 *
 *   dtype_in: KCG_F32, KCG_BF16, KCG_F16 (and KCG_I32 for Cast).
 */
KCG_API int kcg_eltwise(int op, int dtype_in, int dtype_out, int64_t n, const void* x,
                        void* y, void* stream);

/*
 * Binary elementwise map with numpy-style broadcasting — replaces
 * `{Op}_Binary_{dimsA}_{Op}_{dimsB}` (builder:
 * src/Frontend/Operators.cc:772-889; schedule: src/Optimizer/Optimizer.cc:928-991).
 *
 *   Shapes are aligned at the trailing dimension; where they differ one of the
 *   two extents must be 1.  The output has the broadcast shape and the dtype of
 *   the inputs.  Equal / Greater write 1 or 0 in that dtype.
 *   rank_a, rank_b <= KCG_MAX_RANK.  c may alias a when a has the output shape.
 */
KCG_API int kcg_binary(int op, int dtype, int rank_a, const int64_t* shape_a, int rank_b,
                       const int64_t* shape_b, const void* a, const void* b, void* c,
                       void* stream);

/*
 * Row softmax over the last dimension — replaces `Softmax_{dims}_axis{a}`
 * (builder: src/Frontend/Operators.cc:462-578):  y = exp(s*x) / sum(exp(s*x)),
 * evaluated in the max-subtracted form.  `scale` (s) and `causal` are extensions
 * with neutral defaults 1.0f / 0: with causal != 0 the row index within the
 * trailing [q_len, cols] matrix masks columns j > i + (cols - q_len).
 * y may alias x (the reference's Softmax is always in place).
 */
KCG_API int kcg_softmax(int dtype, int64_t rows, int64_t cols, float scale, int causal,
                        int64_t q_len, const void* x, void* y, void* stream);

/*
 * GEMM — replaces `Matmul_m{m}n{n}k{k}` and
 * `BatchMatmul_{b..}_m{m}_n{n}_k{k}_{N|T}{N|T}` (builders:
 * src/Frontend/Operators.cc:120-220 and :291-457; schedules:
 * src/Optimizer/Optimizer.cc:406-570 and :3290-3445).
 *
 *   For each batch index g in [0, batch):
 *     C_g[m, n] = alpha * sum_k opA(A_g)[m, k] * opB(B_g)[k, n]
 *   trans_a == 0: A_g is [M, K] row-major with leading dimension lda (Layout::rowMajor);
 *   trans_a != 0: A_g is [K, M] row-major with leading dimension lda (Layout::colMajor);
 *   trans_b == 0: B_g is [K, N] row-major, ldb (Layout::rowMajor);
 *   trans_b != 0: B_g is [N, K] row-major, ldb (Layout::colMajor).
 *   X_g = X + g * stride_x (elements).  C_g is [M, N] row-major, ldc.
 *   alpha = (scale_a ? *scale_a : 1) * (scale_b ? *scale_b : 1), read on the
 *   device (per-tensor FP8 de-quantisation scales); pass NULL for 1.
 *
 *   dtype_in / dtype_out combinations:
 *     KCG_BF16 -> KCG_BF16 | KCG_F32, KCG_F16 -> KCG_F16 | KCG_F32
 *         tcgen05 tensor-core kernel, fp32 accumulation in tensor memory;
 *     KCG_F8E4M3 -> KCG_BF16 | KCG_F32   tcgen05 kind::f8f6f4, fp32 accumulation;
 *     KCG_F32 -> KCG_F32   by default (M N K >= 256^3) the tensor cores, as three tf32
 *         products of hi/lo-split operands with K cut into chunks of 256 (within ~3e-6 of
 *         a float64 product); smaller problems, or kcg_gemm_set_fp32_mode(0), take the
 *         CUDA-core FFMA kernel with the reference's sequential-k fp32 accumulation.
 *   Tensor-core paths need 16-byte aligned base pointers and leading dimensions
 *   / batch strides that are multiples of 16 bytes; M, N, K are arbitrary.
 */
KCG_API int kcg_gemm(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K,
                     int64_t batch, int trans_a, int trans_b, const void* A, int64_t lda,
                     int64_t stride_a, const void* B, int64_t ldb, int64_t stride_b, void* C,
                     int64_t ldc, int64_t stride_c, const float* scale_a,
                     const float* scale_b, void* stream);

/*
 * GEMM with a fused epilogue: C = act(alpha * op(A) op(B) + bias) — the fusion of
 * Matmul -> Binary "Add" (bias of N elements broadcast over rows) -> ElementWise / Relu, e.g.
 * the reference's own Matmul -> Relu(inplace) sequence (test/test.cc:62-63), which its
 * roadmap assigns to a "KernelFusion Optimizer" (doc/Plan.md:68, :110).
 *   bias: N values of dtype_out, or NULL.  activation: 0 none, 1 Relu, 2 Gelu.
 * The value is rounded to dtype_out after each step, exactly where the separate kernels would
 * store it, so the result is bit-identical to the unfused chain.  All other arguments as
 * kcg_gemm(), which is this function with bias = NULL and activation = 0.
 */
KCG_API int kcg_gemm_fused(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K,
                           int64_t batch, int trans_a, int trans_b, const void* A, int64_t lda,
                           int64_t stride_a, const void* B, int64_t ldb, int64_t stride_b, void* C,
                           int64_t ldc, int64_t stride_c, const float* scale_a,
                           const float* scale_b, const void* bias, int activation, void* stream);

/*
 * Tuning switch with no counterpart in the reference, choosing the tile of the tensor-core
 * GEMM: -1 (default) picks, per problem, whichever of the shapes below fills the SMs most
 * evenly (large problems get CTA pairs); 0 forces 128x256 tiles on single CTAs; 1 forces CTA
 * pairs (tcgen05 cta_group::2, one 256x256 tile per two SMs) whenever M > 128; 2 forces 128x128
 * and 3 forces 128x64 tiles on single CTAs (the latter for 16-bit inputs; 8-bit and tf32 inputs
 * get 128x128).  Results are identical.  A setting of the calling thread.
 */
KCG_API void kcg_gemm_set_pair_mode(int mode);

/*
 * Fused multi-head attention forward — replaces
 * `Fused_Multi_Head_Attention_{batch..}_SL{S}_HD{D}`, the kernel the reference
 * builds when it finds BatchMatmul(NT) -> Softmax -> BatchMatmul(NN)
 * (match: src/Optimizer/Optimizer.cc:2113-2199; build: :2606-2860).
 *
 *   O[b,h,i,:] = sum_j softmax_j(softmax_scale * Q[b,h,i,:].K[b,h,j,:]) * V[b,h,j,:]
 *   causal != 0 masks j > i + (Skv - Sq).  The reference has neither scale nor
 *   mask: pass 1.0f and 0 for its semantics.
 *   Each tensor is addressed as base + b*stride[0] + h*stride[1] + s*stride[2] + d
 *   (elements; the head dimension is contiguous), so [B,H,S,D] and [B,S,H,D]
 *   layouts are both expressible.  dtype: KCG_BF16 or KCG_F16; D in {64, 128}.
 *   Softmax statistics are kept in fp32.
 */
KCG_API int kcg_fmha_fwd(int dtype, int64_t B, int64_t H, int64_t Sq, int64_t Skv, int64_t D,
                         float softmax_scale, int causal, const void* Q,
                         const int64_t q_strides[3], const void* K, const int64_t k_strides[3],
                         const void* V, const int64_t v_strides[3], void* O,
                         const int64_t o_strides[3], void* stream);

/*
 * Tuning switch with no counterpart in the reference: which attention kernel runs.
 *   -1 (default)  chosen by shape: variant 5 when Sq > 128 (variant 2 for the gather epilogues), else 1;
 *    5            the two-tile kernel as a persistent grid: a CTA stays resident and walks over
 *                 (tile pair, batch x head) work items, loading the next item's Q and K_0 and issuing
 *                 its first QK^T under the current item's last key block, the output leaving through
 *                 TMA stores staged in the idle K / V ring entry; with a causal mask the items are dealt
 *                 so that every CTA gets long and short tile pairs alike (no gather epilogue; Sq <= 128
 *                 runs variant 1);
 *    4            CTA pair with one query tile per CTA, two score buffers and P in tensor-memory
 *                 columns of its own; the two softmax warpgroups take alternate key blocks and
 *                 two threads issue the MMAs (D = 128 only, no gather epilogue);
 *    3            CTA pair (tcgen05 cta_group::2): four 128-query tiles per two SMs, each SM staging
 *                 half of every K and V tile (D = 128 only; other head dimensions run variant 2);
 *    2            two 128-query tiles per CTA, P handed to the second MMA through tensor memory;
 *    1            one query tile per CTA, P through tensor memory;
 *    0            one query tile per CTA, P through a swizzled shared-memory tile.
 * All variants give results within the same tolerance; kept so the data paths can be compared
 * on one build.  A setting of the calling thread.
 */
KCG_API void kcg_fmha_set_p_in_tmem(int variant);

/*
 * Gather along one axis — replaces the kernel emitted for
 * `Gather_{dims}_indices_{dims}_axis_{a}` (builder: src/Frontend/Operators.cc:1253-1352;
 * schedule: src/Optimizer/Optimizer.cc:1934-2074).
 *
 *   The input is viewed as [outer, axis_len, inner] (dims before, at and after `axis`), the
 *   indices as n_idx values in row-major order: out[o, i, r] = in[o, indices[i], r], an
 *   [outer, n_idx, inner] tensor (the reference's output shape is the input's with the axis
 *   replaced by the shape of `indices`, or dropped when `indices` has shape [1]).
 *   dtype: any kcg_dtype (elements are moved, not interpreted).  index_dtype: KCG_I32 or
 *   KCG_I64.  A negative index counts from the end of the axis.  An index still out of range
 *   is not dereferenced: the output slice is zero-filled and kcg_device_status() reports
 *   KCG_ERR_INVALID_ARG after the stream has been synchronised.
 */
KCG_API int kcg_gather(int dtype, int index_dtype, int64_t outer, int64_t axis_len, int64_t inner,
                       int64_t n_idx, const void* input, const void* indices, void* output,
                       void* stream);

/*
 * Transpose of the two innermost dims, out[b, j, i] = in[b, i, j] for a [batch, rows, cols]
 * input — `Transpose::build(graph, input)` is declared by the reference but its body is empty
 * (include/Frontend/Operators.h:97-99, src/Frontend/Operators.cc:459-460); this is the meaning
 * its signature (one operand, no permutation) admits.  dtype: any kcg_dtype.  Input and output
 * must not alias.
 */
KCG_API int kcg_transpose(int dtype, int64_t batch, int64_t rows, int64_t cols, const void* input,
                          void* output, void* stream);

/*
 * How float32 GEMMs are computed (no counterpart in the reference, whose SGEMM is CUDA-core
 * code): 0 = the CUDA-core FFMA kernel, one fp32 accumulator per output summed in increasing k
 * like the reference's loop nest; 1 = the tensor cores, as three tf32 products of operands
 * split into hi + lo parts (a b = a_hi b_hi + a_lo b_hi + a_hi b_lo, fp32 accumulation; results
 * within ~1e-6 relative of a float64 product, several times faster; uses a cached per-device
 * scratch buffer of 12 (M + N) K bytes per batch entry plus up to 1 GiB of partial products,
 * shared by all float32 GEMMs of a device: serialise float32 GEMMs that could overlap on one
 * device from different streams); -1 (default) = 1 when M N K >= 256^3, else 0.  A setting of
 * the calling thread.
 */
KCG_API void kcg_gemm_set_fp32_mode(int mode);

/*
 * GEMM with the all-gather of C done by its epilogue (no counterpart in the reference, which
 * has no multi-GPU code; the sharding is the one kcg_shard_range describes).  Rank `rank` of
 * `world` (<= 8) computes its M x N block C = op(A) op(B) exactly as kcg_gemm_fused would
 * (same kernel, same bits) and stores every tile into rows [row_offset, row_offset + M) of
 * each of the `world` gathered matrices gathered[r] (leading dimension ldc, `N` columns used):
 * gathered[rank] is this GPU's own buffer, the others are the peers' buffers mapped into this
 * process (kcg_peer_open).  Stores to peers are whole 128-byte row segments written straight
 * from the epilogue, so the transfer overlaps the tensor-core work of the following tiles.
 * The call only launches; the rows written by the other ranks are complete once every rank's
 * launch has finished (synchronise the ranks, e.g. with a barrier on the stream, before reading
 * and before the next call overwrites the buffers).  Tensor-core input dtypes only, M > 128,
 * 16-byte aligned pointers / ldc / N.
 */
KCG_API int kcg_gemm_allgather(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K,
                               int trans_a, int trans_b, const void* A, int64_t lda,
                               const void* B, int64_t ldb, void* const* gathered, int world,
                               int rank, int64_t row_offset, int64_t ldc, const float* scale_a,
                               const float* scale_b, const void* bias, int activation,
                               void* stream);

/*
 * Attention forward with the all-gather of O done by its epilogue (no counterpart in the
 * reference).  Rank `rank` of `world` (<= 8) computes its B batches exactly as kcg_fmha_fwd would
 * (two-tile kernel, same bits) and stores every output row into batches [batch_offset,
 * batch_offset + B) of each rank's gathered tensor gathered[r] (element strides o_strides, as
 * for kcg_fmha_fwd); gathered[rank] is local, the others are peers' buffers mapped with
 * kcg_peer_open.  Rows leave as whole D-element lines (256 bytes at D = 128).  Synchronise the
 * ranks as for kcg_gemm_allgather.
 */
KCG_API int kcg_fmha_fwd_allgather(int dtype, int64_t B, int64_t H, int64_t Sq, int64_t Skv,
                                   int64_t D, float softmax_scale, int causal, const void* Q,
                                   const int64_t q_strides[3], const void* K,
                                   const int64_t k_strides[3], const void* V,
                                   const int64_t v_strides[3], void* const* gathered, int world,
                                   int rank, int64_t batch_offset, const int64_t o_strides[3],
                                   void* stream);

/*
 * The two fused gathers with the replication done by NVSwitch (no counterpart in the reference).
 * `gathered_multicast` is the address of the gathered matrix / tensor inside a multicast mapping
 * to which every rank has bound its own buffer (an NVLink multicast object, e.g. the
 * `multicast_ptr` of a torch symmetric-memory allocation), `gathered_local` this rank's own
 * buffer.  Each tile (output row) is stored ONCE, with multimem.st to the multicast address, and
 * the switch delivers it to every rank's buffer, this rank's included: a GPU sends its block over
 * its links once instead of world - 1 times, which is what keeps the gather under the math at 8
 * GPUs.  Same kernels, same bits and same synchronisation rules as kcg_gemm_allgather /
 * kcg_fmha_fwd_allgather.  All ranks must unbind / release the mapping before any of them exits.
 */
KCG_API int kcg_gemm_allgather_multicast(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K,
                                         int trans_a, int trans_b, const void* A, int64_t lda,
                                         const void* B, int64_t ldb, void* gathered_local,
                                         void* gathered_multicast, int64_t row_offset, int64_t ldc,
                                         const float* scale_a, const float* scale_b, const void* bias,
                                         int activation, void* stream);
KCG_API int kcg_fmha_fwd_allgather_multicast(int dtype, int64_t B, int64_t H, int64_t Sq, int64_t Skv,
                                             int64_t D, float softmax_scale, int causal, const void* Q,
                                             const int64_t q_strides[3], const void* K,
                                             const int64_t k_strides[3], const void* V,
                                             const int64_t v_strides[3], void* gathered_local,
                                             void* gathered_multicast, int64_t batch_offset,
                                             const int64_t o_strides[3], void* stream);

/*
 * LayerNorm of this rank's `rows` rows with the all-gather of the result done by NVSwitch: row r is
 * stored, with multimem.st, to row row_offset + r of `gathered_multicast` (the multicast address
 * of the [total_rows, cols] gathered tensor, see kcg_gemm_allgather_multicast) and arrives in every
 * rank's buffer.  Rows the one-pass kernels take only (16-byte vectorisable, at most 4096 vectors).
 * Same arithmetic and bits as kcg_layernorm; no counterpart in the reference.
 */
KCG_API int kcg_layernorm_allgather_multicast(int dtype, int64_t rows, int64_t cols, const void* x,
                                              const void* gamma, const void* beta, float eps,
                                              void* gathered_multicast, int64_t row_offset,
                                              void* stream);

/*
 * Device memory that other processes on the node can map (CUDA IPC).  kcg_peer_alloc returns a
 * plain device allocation; kcg_peer_export fills a 64-byte handle that another process passes
 * to kcg_peer_open to obtain a pointer valid on its own GPU (peer access is enabled on first
 * use; loads and stores through it cross NVLink).  Close every opened pointer before the owner
 * frees the allocation.
 */
KCG_API int kcg_peer_alloc(size_t bytes, void** ptr);
KCG_API int kcg_peer_free(void* ptr);
KCG_API int kcg_peer_export(void* ptr, unsigned char handle[64]);
KCG_API int kcg_peer_open(const unsigned char handle[64], void** ptr);
KCG_API int kcg_peer_close(void* ptr);

/*
 * Device utilities for host code that does not link the CUDA runtime itself (the C++ front
 * end's autotuner): number of visible devices (0 without a driver, never an error), an
 * asynchronous byte fill, and a stream timer — kcg_timer_begin records an event on `stream`,
 * kcg_timer_end records a second one, waits for it and returns the elapsed device time,
 * releasing the timer.  Buffers come from kcg_peer_alloc / kcg_peer_free.
 */
KCG_API int kcg_device_count(int* count);
KCG_API int kcg_device_memset(void* ptr, int byte_value, size_t bytes, void* stream);
KCG_API int kcg_timer_begin(void* stream, void** timer);
KCG_API int kcg_timer_end(void* stream, void* timer, float* milliseconds);

/*
 * Diagnostic: launches one thread block that waits, with the same bounded wait all tensor-core
 * kernels use, on a barrier that nothing signals, for at most budget_ns (<= 100 ms) nanoseconds.
 * The kernel then gives up exactly as a real kernel would: it writes KCG_ERR_TIMEOUT to the word
 * kcg_device_status() reports, stores the time it waited to *waited_ns_device (device memory)
 * and exits normally, leaving the context usable.  No counterpart in the reference.
 */
KCG_API int kcg_selftest_bounded_wait(uint64_t budget_ns, unsigned long long* waited_ns_device,
                                      void* stream);

/*
 * Row-range owned by one rank when `total` independent units (GEMM rows of A/C,
 * attention batch*head slices, LayerNorm / elementwise rows) are split over
 * `world` GPUs in contiguous blocks rounded to `granule` units.  The reference
 * has no multi-GPU code; this is the only sharding rule the library uses.
 */
KCG_API int kcg_shard_range(int64_t total, int world, int rank, int64_t granule,
                            int64_t* begin, int64_t* count);

/*
 * The optional exchange after a sharded operator: an in-place all-gather over NCCL.  `buffer`
 * holds the whole output, `total_units` units of `unit_bytes` bytes each (GEMM / LayerNorm /
 * elementwise rows, attention batches); on entry the block kcg_shard_range(total_units, world,
 * rank, granule) assigns to this rank is valid, and once the work queued on `stream` has run,
 * every rank's block is.  Blocks of equal size go through one in-place ncclAllGather, ragged
 * ones through one ncclBroadcast per owner inside a group.  `nccl_comm` is an ncclComm_t of
 * `world` ranks in which this process is rank `rank` (checked).  Collective: every rank calls it
 * with the same sizes.  No counterpart in the reference (which has no multi-GPU code); NCCL is
 * looked up at run time in the libnccl.so.2 already loaded in the process, not linked.
 */
KCG_API int kcg_shard_allgather(void* buffer, int64_t total_units, int64_t unit_bytes,
                                int64_t granule, int world, int rank, void* nccl_comm,
                                void* stream);

/*
 * Thin wrappers for host code that does not include nccl.h itself (the C++ front end's tests, a
 * ctypes caller): kcg_nccl_unique_id fills the 128-byte ncclUniqueId that rank 0 hands to the
 * others by its own means; kcg_nccl_comm_create is ncclCommInitRank on the current device
 * (collective); kcg_nccl_comm_destroy is ncclCommDestroy.  A communicator created elsewhere with
 * the same NCCL library works just as well.
 */
KCG_API int kcg_nccl_unique_id(unsigned char id[128]);
KCG_API int kcg_nccl_comm_create(int world, int rank, const unsigned char id[128], void** comm);
KCG_API int kcg_nccl_comm_destroy(void* comm);

#ifdef __cplusplus
}
#endif
#endif /* KCG_KERNELS_H_ */
