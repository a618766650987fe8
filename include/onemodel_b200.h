/*
 * onemodel_b200.h - C ABI of libonemodel_b200.so: the B200 (sm_100a) training backend for the autograd
 * hot path of RecursiveAI.OneModel.Training (forward ops that fill the tape's saved slots, every per-op
 * backward function, the fused optimizer step, gradient clipping, data-parallel gradient exchange).
 *
 * Conventions
 *  - Every function returns an om_status (0 = OM_OK). The message of the last failure on a context is read
 *    with om_last_error. No C++ exception crosses this boundary.
 *  - All tensor pointers are DEVICE pointers unless a parameter name ends in _host. Tensors are float32,
 *    row-major and contiguous unless strides are passed explicitly. The caller owns all memory it passes;
 *    the library keeps no pointer past a call except registered data-parallel buckets.
 *  - One om_ctx per device; calls on one context are serialised by the caller (the reference engine is
 *    single-threaded: src/OneModel/Tensors/Autograd/Engine.cs:112-120). Work is asynchronous on the
 *    context's stream until om_sync or a device-to-host copy.
 *  - Results never depend on launch geometry chosen at run time: every reduction has a fixed partition and
 *    a fixed combine order and no kernel uses floating-point atomics (the reference's rule that a result
 *    must not depend on the thread count, src/OneModel/Tensors/TensorKernels.cs:57-61).
 *  - The reference has no FFI for this path (tests/OneModel.Tests/PackageGuardTests.cs:54-66 bans P/Invoke
 *    under src/). Each entry point names the managed function whose body it replaces.
 */
#ifndef ONEMODEL_B200_H
#define ONEMODEL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

typedef struct om_ctx om_ctx;

typedef enum om_status {
  OM_OK = 0,
  OM_ERR_SHAPE = 1,       /* TensorShapeException in the reference */
  OM_ERR_INDEX = 2,       /* ArgumentOutOfRangeException: embedding id / NLL target / CTC label out of range
                             (src/OneModel/Tensors/Ops.Layers.cs:590-600,667-676) */
  OM_ERR_OOM = 3,
  OM_ERR_CUDA = 4,
  OM_ERR_NCCL = 5,
  OM_ERR_TIMEOUT = 6,     /* a bounded device-side or host-side wait ran out */
  OM_ERR_UNSUPPORTED = 7,
  OM_ERR_ARG = 8,
  OM_ERR_CANARY = 9       /* OM_CHECKED: the guard bytes behind a released buffer were overwritten */
} om_status;

/* Context flags. OM_TF32: matrix products run on the tcgen05 tensor pipe with TF32 operands and fp32
 * accumulation (TensorCompute.Mode = Fast); without it they run on an fp32 FMA kernel that keeps the
 * reference's one-accumulator, increasing-k order (TensorCompute.Mode = Exact tier of tolerance,
 * src/OneModel/Tensors/Autograd/TensorCompute.cs:22-78). OM_BF16_OPERANDS (with OM_TF32): the host layer above this
 * library keeps bfloat16 copies of the tensors that feed the Linear products and calls the om_*_bf16 entry points below
 * (bfloat16 operands rounded to nearest even, fp32 accumulation); the fp32-operand entry points are unchanged by it.
 * OM_CHECKED (the reference's CHECKED build, docs/tensors.md:108-110): memory from om_alloc (and every pooled scratch
 * block) is filled with 0xFF when handed out and again when returned (NaN for floats, -1 for integers: reads of unwritten
 * or released memory stand out), and 64 guard bytes (0xA5) follow its length; om_free verifies them on the device and a
 * kernel that wrote past the end shows as OM_ERR_CANARY at the next om_sync. Index operands are range-checked on the
 * device with or without the flag. A debugging mode: two extra small launches per allocation. OM_PAIR_TILES (with OM_TF32): every plain product the
 * CTA-pair kernel can take runs on it (tcgen05 cta_group::2, 256-row tiles: fewer operand bytes per SM); without the
 * flag only products with several rounds of tiles over the device do.
 * OM_TWO_STREAMS: a backward entry point whose gradients are independent of one another (om_linear_bwd: the input
 * gradient on one side, the weight and bias gradients on the other) runs them on two streams of the context, forked
 * and joined inside the call, so that products too small to fill the device overlap; om_linear_bwd_bf16_b16 runs the
 * bias column sum (bound by memory) beside its products (bound by the tensor pipe). Results are the same bits.
 * OM_SEQ_KERNELS (with OM_TF32): an LSTM layer whose shape fits (hidden a multiple of 16, batch <= 256 for the backward)
 * runs all its time steps in one cooperative launch with fp32 recurrent products, instead of a product and a gate
 * kernel per step. OM_OVERLAP_LAUNCHES: the frequent kernels are launched as programmatic dependents of their
 * predecessor in the stream, so that launch latency and prologue overlap the predecessor's tail (same results).
 * OM_PERSISTENT_TILES (with OM_TF32): plain products run on the persistent CTA-pair kernel that the bfloat16 products
 * always use (two accumulator buffers in tensor memory: a tile's read-back and stores run under the next tile's MMAs). */
#define OM_TF32 1u
#define OM_BF16_OPERANDS 2u
#define OM_CHECKED 4u
#define OM_PAIR_TILES 8u
#define OM_TWO_STREAMS 16u
#define OM_SEQ_KERNELS 32u
#define OM_OVERLAP_LAUNCHES 64u
#define OM_PERSISTENT_TILES 128u

typedef enum om_dtype { OM_F32 = 0, OM_I32 = 1, OM_I64 = 2 } om_dtype;

/* ---- context, memory, streams ---------------------------------------------------------------------- */

int32_t om_version(void);
int32_t om_ctx_create(int32_t device, uint32_t flags, om_ctx** out);
int32_t om_ctx_destroy(om_ctx* ctx);
int32_t om_ctx_set_flags(om_ctx* ctx, uint32_t flags);
int32_t om_ctx_get_flags(om_ctx* ctx, uint32_t* flags);
/* Every device-side wait of the tensor-pipe kernels (on an mbarrier: operands landed, stage free, accumulator ready)
 * is bounded; when the bound runs out the kernel stores OM_ERR_TIMEOUT in the context's status word, every role leaves
 * its loop, tensor memory is released and the kernel returns, so the next om_sync reports the timeout and the context
 * stays usable. The bound is about one second of SM clock; this sets another one for the context (0 = the default
 * again; budgets under a quarter of a millisecond act as a quarter of a millisecond). Synchronises the stream. No
 * counterpart in the reference (its kernels are host loops). */
int32_t om_ctx_set_wait_budget_us(om_ctx* ctx, int64_t microseconds);
/* Launches one warp that waits, under the context's wait budget, on a barrier nothing ever arrives at: the timeout
 * path above in isolation. The next om_sync returns OM_ERR_TIMEOUT (detail 99). For tests of error handling. */
int32_t om_selftest_bounded_wait(om_ctx* ctx);
/* Copies the last error message (NUL terminated, truncated to n) of this context; ctx may be NULL for
 * errors of om_ctx_create. */
int32_t om_last_error(om_ctx* ctx, char* buf, size_t n);
/* The CUDA stream (cudaStream_t) all work of this context is ordered on. */
int32_t om_ctx_stream(om_ctx* ctx, void** stream);

/* Pooled device memory with the reference pool's size classes b*{1.25,1.5,1.75,2}
 * (replaces BufferPool.Rent / release, src/OneModel/Tensors/Memory/BufferPool.cs:67; docs/tensors.md:93-118).
 * Freed blocks are reused in stream order; om_pool_trim returns cached blocks to the driver. */
int32_t om_alloc(om_ctx* ctx, size_t bytes, int32_t zero, void** dptr);
int32_t om_free(om_ctx* ctx, void* dptr);
int32_t om_pool_trim(om_ctx* ctx);
int32_t om_pool_stats(om_ctx* ctx, uint64_t* bytes_in_use, uint64_t* bytes_cached, uint64_t* driver_allocs);
int32_t om_memcpy_h2d(om_ctx* ctx, void* dst, const void* src_host, size_t bytes);
int32_t om_memcpy_d2h(om_ctx* ctx, void* dst_host, const void* src, size_t bytes); /* synchronises */
int32_t om_memcpy_d2d(om_ctx* ctx, void* dst, const void* src, size_t bytes);
int32_t om_memset(om_ctx* ctx, void* dst, int32_t byte, size_t bytes);
/* Staging of input batches one or more steps ahead (the device side of DataLoader's prefetch ring,
 * src/OneModel.Training/Data/DataLoader.cs:35, docs/data-loading.md section 1: a batch waits in slot `step mod Prefetch`
 * until its step takes it). The copies run on a copy stream of the context, beside the compute stream:
 *   om_stage_h2d(slot, dst, src)  copy pinned host memory to device memory on the copy stream, after the step that
 *                                 used the slot's previous batch has taken it;
 *   om_stage_commit(slot)         the slot's batch is complete (an event on the copy stream);
 *   om_stage_acquire(slot)        the compute stream waits for that event (no host wait);
 *   om_stage_release(slot)        the work queued so far on the compute stream has taken the batch: the slot may be refilled;
 *   om_stage_wait_taken(slot)     host wait for that point.
 * Slots 0..15. The host memory must stay unchanged until the copy has run (keep it in the loader's ring). */
int32_t om_stage_h2d(om_ctx* ctx, int32_t slot, void* dst, const void* src_pinned, size_t bytes);
int32_t om_stage_commit(om_ctx* ctx, int32_t slot);
int32_t om_stage_acquire(om_ctx* ctx, int32_t slot);
int32_t om_stage_release(om_ctx* ctx, int32_t slot);
/* Host wait until the slot's last om_stage_release has been reached by the compute stream (the loader's back-pressure:
 * the pinned buffer behind the slot may be rewritten after it). Returns at once when the slot was never released. */
int32_t om_stage_wait_taken(om_ctx* ctx, int32_t slot);
int32_t om_host_alloc_pinned(om_ctx* ctx, size_t bytes, void** hptr);
int32_t om_host_free_pinned(om_ctx* ctx, void* hptr);
/* Waits for the stream and returns the device status word: OM_ERR_INDEX if a checked kernel saw an index
 * out of range, OM_ERR_TIMEOUT if a bounded device wait expired. The word is cleared. */
int32_t om_sync(om_ctx* ctx);

/* Whole-step CUDA graph capture of the calls made between begin and end on this context. */
int32_t om_graph_begin(om_ctx* ctx);
int32_t om_graph_end(om_ctx* ctx, void** graph_exec);
int32_t om_graph_launch(om_ctx* ctx, void* graph_exec);
/* Number of kernel nodes in the graph produced by the last om_graph_end on this context. */
int32_t om_graph_last_kernel_nodes(om_ctx* ctx, int32_t* n);
int32_t om_graph_destroy(om_ctx* ctx, void* graph_exec);

/* Per-entry-point device timers (CUDA events on the context's stream around every call).
 * om_profile_read writes up to cap rows; names are the entry point names. */
typedef struct om_profile_row {
  char name[48];
  uint64_t calls;
  double ms;
  double flops; /* algorithmic flops reported by the entry point (0 for bandwidth-bound kernels) */
  double bytes; /* algorithmic bytes reported by the entry point */
} om_profile_row;
int32_t om_profile_enable(om_ctx* ctx, int32_t on);
int32_t om_profile_reset(om_ctx* ctx);
int32_t om_profile_read(om_ctx* ctx, om_profile_row* rows, int32_t cap, int32_t* n);

/* ---- dense products --------------------------------------------------------------------------------- */

/* C[m,n] = op(A)[m,k] * op(B)[k,n] (+ C when accumulate != 0), row-major, leading dimensions in elements.
 * op(X) = X^T when transX != 0 (X is then stored [k,m] resp. [n,k]).
 * Replaces Dense.Gemm (src/OneModel/Tensors/Autograd/Dense.cs:12-48) under Ops.MatMul (Ops.cs:117-144) and
 * both products of the MatMul backward (BackwardOps.cs:69-82): dA = g*B^T, dB = A^T*g with no transposed copy.
 * Each output element has one accumulator summed in increasing k (fp32 path), or a fixed split of k into
 * equal parts combined in increasing order (tensor-pipe path). */
int32_t om_matmul(om_ctx* ctx, int32_t transA, int32_t transB, int32_t m, int32_t n, int32_t k,
                  const float* A, int32_t lda, const float* B, int32_t ldb, float* C, int32_t ldc,
                  int32_t accumulate);
/* Same, over `batch` matrices at the given element strides (0 broadcasts an operand).
 * Replaces Ops.MatMulBatched and BatchMatMul backward (Ops.GraphOps.cs:24; BackwardGraphOps.cs:10-66). */
int32_t om_matmul_batched(om_ctx* ctx, int32_t transA, int32_t transB, int32_t m, int32_t n, int32_t k,
                          const float* A, int32_t lda, int64_t strideA, const float* B, int32_t ldb,
                          int64_t strideB, float* C, int32_t ldc, int64_t strideC, int32_t batch,
                          int32_t accumulate);
/* y[rows,out] = x[rows,in] * W[out,in]^T + bias[out] (bias may be NULL), optionally followed by an
 * activation (om_unary_op, OM_UNARY_NONE for none) whose pre-activation is written to pre (may be NULL).
 * Fuses the Reshape/MatMul/Add chain of Ops.Linear (Ops.Layers.cs:715-733). */
int32_t om_linear_fwd(om_ctx* ctx, const float* x, const float* W, const float* bias, int32_t rows,
                      int32_t in_features, int32_t out_features, float* y);
/* The same with an explicit row pitch of y / g in elements (>= out_features). A pitch that is a multiple of four
 * keeps wide outputs whose width is not (the 30522-column vocabulary logits) on the tensor pipe, whose TMA loads need
 * 16-byte aligned rows. */
int32_t om_linear_fwd_ld(om_ctx* ctx, const float* x, const float* W, const float* bias, int32_t rows,
                         int32_t in_features, int32_t out_features, float* y, int32_t ldy);
int32_t om_linear_bwd_ld(om_ctx* ctx, const float* g, int32_t ldg, const float* x, const float* W, int32_t rows,
                         int32_t in_features, int32_t out_features, float* dx, float* dW, float* dbias,
                         int32_t accumulate_w);
/* Backward of om_linear_fwd: dx = g*W (NULL to skip), dW = g^T*x (NULL to skip), dbias = column sums of g
 * (NULL to skip). accumulate_w bit 0 adds into dW/dbias, bit 1 adds into dx (Engine.AddInto, Engine.cs:330-344: the
 * product's epilogue adds to a gradient that already holds another branch's contribution instead of a separate pass).
 * Replaces the Reshape/Add/MatMul/Permute records of one Linear (call stack: BackwardOps.cs:69-82,107-122,156-194). */
int32_t om_linear_bwd(om_ctx* ctx, const float* g, const float* x, const float* W, int32_t rows,
                      int32_t in_features, int32_t out_features, float* dx, float* dW, float* dbias,
                      int32_t accumulate_w);

/* ---- products with bfloat16 operands (OM_BF16_OPERANDS) ------------------------------------------------------------
 * The tier BERT-base-shape training is configured for: product operands rounded to bfloat16 (round to nearest even,
 * the rule of docs/tensors.md section 10 / BFloat16.FromSingleBits, src/OneModel/Tensors/Float16.cs:121-160),
 * fp32 accumulation, fp32 results, fp32 master weights. The reference has no such path on the CPU (its Dense.Gemm,
 * Dense.cs:12-48, multiplies fp32); these entry points stand where om_matmul / om_linear_fwd / om_linear_bwd stand, with
 * the operands given as bfloat16 copies that the caller keeps beside the fp32 tensors (one om_cast_bf16 per tensor and
 * version, reused by every product that reads it: forward and weight gradient share x, forward and input gradient share
 * W, the two gradients share g). Operand pitches must be multiples of 8 elements, the pitch of C a multiple of 4, base
 * addresses 16-byte aligned (OM_ERR_UNSUPPORTED otherwise: use the fp32-operand entry point). */
/* dst[i] = bfloat16(src[i]), round to nearest even. */
int32_t om_cast_bf16(om_ctx* ctx, const float* src, uint16_t* dst, int64_t n);
int32_t om_matmul_bf16(om_ctx* ctx, int32_t transA, int32_t transB, int32_t m, int32_t n, int32_t k, const uint16_t* A,
                       int32_t lda, const uint16_t* B, int32_t ldb, float* C, int32_t ldc, int32_t accumulate);
int32_t om_linear_fwd_bf16(om_ctx* ctx, const uint16_t* x, const uint16_t* W, const float* bias, int32_t rows,
                           int32_t in_features, int32_t out_features, float* y, int32_t ldy);
/* The forward product and the input gradient with the bfloat16 copy of their result (y16 / dx16, same pitch in elements as
 * the fp32 result, may be NULL) written by the product's epilogue (y may be NULL instead when only the bfloat16 result is
 * wanted and k is not split, i.e. the shape passes om_linear_act_bf16_supported): the packed q | k | v projections and the gradient of the
 * attention output are read as bfloat16 by the attention kernels. */
int32_t om_linear_fwd_bf16_b16(om_ctx* ctx, const uint16_t* x, const uint16_t* W, const float* bias, int32_t rows,
                               int32_t in_features, int32_t out_features, float* y, uint16_t* y16, int32_t ldy);
int32_t om_linear_bwd_bf16_b16(om_ctx* ctx, const uint16_t* g16, const float* g, int32_t ldg, const uint16_t* x,
                               const uint16_t* W, int32_t rows, int32_t in_features, int32_t out_features, float* dx,
                               uint16_t* dx16, float* dW, float* dbias, int32_t accumulate_w);
/* Producers that write the bfloat16 copy of their result in the same pass (the copy pointer may be NULL: then they are
 * om_unary, om_unary_bwd, om_layernorm_fwd, om_layernorm_bwd): the activation, its gradient and the two sides of a
 * layer norm are what feeds the Linear products of an encoder layer, so no separate cast pass is left for them.
 * With a copy requested, OM_GELU_ERF and its derivative evaluate erf in a short branch-free form (within 4e-7 absolute of
 * erf; the copy then rounds to 8 significant bits), the same form that om_linear_fwd_bf16_act and
 * om_linear_dgrad_bf16_act apply in their epilogues, so that the fused and the separate calls give the same bits. */
int32_t om_unary_b16(om_ctx* ctx, int32_t op, const float* x, float* y, uint16_t* y16, int64_t n);
int32_t om_unary_bwd_b16(om_ctx* ctx, int32_t op, const float* g, const float* saved, float* dx, uint16_t* dx16, int64_t n);
int32_t om_layernorm_fwd_b16(om_ctx* ctx, const float* x, const float* gamma, const float* beta, int32_t rows,
                             int32_t cols, float eps, float* y, uint16_t* y16, float* mean, float* inv);
/* The residual sum in front of a layer norm formed in the same pass: sum = x + addend (written out, the layer norm's
 * input for the backward pass), y = LayerNorm(sum). The values are those of om_binary(OM_ADD) followed by om_layernorm_fwd;
 * one read of the two operands instead of a write and a read of the sum between two launches. addend and sum NULL: plain
 * om_layernorm_fwd_b16. Rows up to 1024 wide. */
int32_t om_add_layernorm_fwd_b16(om_ctx* ctx, const float* x, const float* addend, float* sum, const float* gamma,
                                 const float* beta, int32_t rows, int32_t cols, float eps, float* y, uint16_t* y16,
                                 float* mean, float* inv);
int32_t om_layernorm_bwd_b16(om_ctx* ctx, const float* g, const float* x, const float* gamma, const float* mean,
                             const float* inv, int32_t rows, int32_t cols, float* dx, uint16_t* dx16, float* dgamma,
                             float* dbeta, int32_t accumulate_params);
/* g16 is the bfloat16 copy of g (same pitch ldg). The bias gradient g^T 1 sums the fp32 g when one is given; with g NULL
 * it sums g16, the operand that the weight gradient g^T x reads (om_colsum_bf16), and the fp32 gradient need not exist.
 * The same holds for om_linear_bwd_bf16_b16. */
int32_t om_linear_bwd_bf16(om_ctx* ctx, const uint16_t* g16, const float* g, int32_t ldg, const uint16_t* x,
                           const uint16_t* W, int32_t rows, int32_t in_features, int32_t out_features, float* dx,
                           float* dW, float* dbias, int32_t accumulate_w);
/* A Linear layer together with the activation that follows it (op: OM_GELU_ERF or OM_GELU_TANH), for the pair
 * Linear -> activation -> Linear of a feed-forward block (the reference composes Ops.Linear, Ops.Gelu, Ops.Linear,
 * Ops.Layers.cs:715-733 and Ops.cs Gelu; the values are those of the composition, bit for bit):
 *   om_linear_fwd_bf16_act: y = x W^T + bias (fp32, what the activation's backward needs) and a16 = bfloat16(op(y)), the
 *     next layer's operand, from the product's epilogue; op(y) is not stored as fp32.
 *   om_linear_dgrad_bf16_act: dx = op'(pre) * (g W), the input gradient of the layer AFTER the activation already
 *     multiplied by the activation's derivative at its saved input `pre` ([rows, in_features] with pitch ldpre), as
 *     fp32 and as bfloat16 (either of dx and dx16 may be NULL: with dx NULL only the bfloat16 result is written, which is
 *     all that the gradient products of the layer in front of the activation read).
 * om_linear_act_bf16_supported tells (1 / 0) whether the shape can take the fused form (widths that are multiples of 8, at
 * least 256 result columns, no split of k); otherwise the caller composes the unfused calls. */
int32_t om_linear_act_bf16_supported(om_ctx* ctx, int32_t rows, int32_t in_features, int32_t out_features, int32_t op,
                                     int32_t backward);
int32_t om_linear_fwd_bf16_act(om_ctx* ctx, const uint16_t* x, const uint16_t* W, const float* bias, int32_t rows,
                               int32_t in_features, int32_t out_features, int32_t op, float* y, uint16_t* a16, int32_t ldy);
int32_t om_linear_dgrad_bf16_act(om_ctx* ctx, const uint16_t* g16, int32_t ldg, const uint16_t* W, int32_t rows,
                                 int32_t in_features, int32_t out_features, int32_t op, const float* pre, int32_t ldpre,
                                 float* dx, uint16_t* dx16);
/* The same pair with the activation's derivative left behind by the forward pass, so that the backward epilogue only
 * multiplies: om_linear_fwd_bf16_actd writes deriv = op'(x W^T + bias) as IEEE half (binary16, round to nearest even: the
 * derivative of GELU lies in [-0.13, 1.13], where half carries 11 significant bits, eight times finer than the bfloat16
 * rounding of the gradient it multiplies) and a16 = bfloat16(op(x W^T + bias)), both with pitch ldd (a multiple of 8);
 * om_linear_dgrad_bf16_mul writes dx = factor * (g W) with factor = that derivative ([rows, in_features] half, pitch ldf, a
 * multiple of 8), as fp32 and / or bfloat16 (either of dx and dx16 may be NULL). a16 has the bits om_linear_fwd_bf16_act
 * writes; dx is om_linear_dgrad_bf16_act's up to the half rounding of the factor. The derivative is evaluated once, where the
 * activation is, and costs 2 bytes per element to keep instead of the 4 of the saved input. Supported shapes as for those
 * (om_linear_act_bf16_supported). */
int32_t om_linear_fwd_bf16_actd(om_ctx* ctx, const uint16_t* x, const uint16_t* W, const float* bias, int32_t rows,
                                int32_t in_features, int32_t out_features, int32_t op, uint16_t* deriv, uint16_t* a16,
                                int32_t ldd);
int32_t om_linear_dgrad_bf16_mul(om_ctx* ctx, const uint16_t* g16, int32_t ldg, const uint16_t* W, int32_t rows,
                                 int32_t in_features, int32_t out_features, const uint16_t* factor, int32_t ldf, float* dx,
                                 uint16_t* dx16);
/* dx = residual + g W, out of place: the input gradient of a Linear layer whose input already holds a gradient from
 * another branch (a residual connection). The sum is formed in the product's epilogue from a plain read of `residual`
 * ([rows, in_features] fp32 with pitch ldres), so that tensor is not modified and may stay shared with its other readers
 * (the engine of the reference adds later gradients into the first one that arrived, Engine.cs:124-344; the values are the
 * same). dx16 (may be NULL) receives the bfloat16 copy. om_linear_dgrad_bf16_add_supported tells (1 / 0) whether the shape
 * can take it (widths multiples of 8, at least 256 result columns, no split of k). */
int32_t om_linear_dgrad_bf16_add_supported(om_ctx* ctx, int32_t rows, int32_t in_features, int32_t out_features);
int32_t om_linear_dgrad_bf16_add(om_ctx* ctx, const uint16_t* g16, int32_t ldg, const uint16_t* W, int32_t rows,
                                 int32_t in_features, int32_t out_features, const float* residual, int32_t ldres, float* dx,
                                 uint16_t* dx16);
/* out[c] (+)= sum over rows of the bfloat16 matrix g16[rows, cols] with pitch ld (a multiple of 8, 16-byte aligned base):
 * om_colsum on the bfloat16 copy of a gradient, with the same partition of the rows (chunks of 512 rows, 32 lanes of 16 rows).
 * A lane adds its 16 rows (lane, lane + 32, ...) in fp32 in increasing order; the 32 lane sums of a chunk, then the chunks,
 * are added in double in increasing order. The order is fixed, so the result is the same from run to run. */
int32_t om_colsum_bf16(om_ctx* ctx, const uint16_t* g16, int32_t rows, int32_t cols, int32_t ld, float* out,
                       int32_t accumulate);

/* ---- elementwise ------------------------------------------------------------------------------------ */

typedef enum om_binary_op { OM_ADD = 0, OM_SUB = 1, OM_MUL = 2, OM_DIV = 3 } om_binary_op;
typedef enum om_unary_op {
  OM_UNARY_NONE = 0, OM_RELU = 1, OM_GELU_ERF = 2, OM_GELU_TANH = 3, OM_SIGMOID = 4, OM_TANH = 5,
  OM_NEG = 6, OM_EXP = 7, OM_SQRT = 8, OM_ERF = 9
} om_unary_op;

/* out = a (op) b over a broadcast shape of rank <= 8; strides in elements, 0 on broadcast axes; out is
 * contiguous. Replaces ITensorKernels.Binary (src/OneModel/Tensors/TensorKernels.cs:62-98) under
 * Ops.Add/Sub/Mul/Div (Ops.cs:15-96). */
int32_t om_binary(om_ctx* ctx, int32_t op, int32_t rank, const int32_t* shape, const float* a,
                  const int64_t* a_strides, const float* b, const int64_t* b_strides, float* out);
/* y = f(x) over n contiguous elements. Replaces ITensorKernels.Unary under Ops.Relu/Neg (Ops.cs:98-115),
 * Ops.Gelu/Sigmoid/Tanh (Ops.Nn.cs:86-160), Ops.Erf/Exp/Sqrt (Ops.GraphOps.cs:100-200). */
int32_t om_unary(om_ctx* ctx, int32_t op, const float* x, float* y, int64_t n);
/* dx = g * f'(saved). saved is the OUTPUT for RELU, SIGMOID, TANH, EXP, SQRT and the INPUT for GELU_*, ERF,
 * exactly as the reference's records save them. Replaces ReluGradBin, SigmoidGradBin, TanhGradBin,
 * GeluGradBin (src/OneModel/Kernels/TrainElementwise.cs:42-85; BackwardOps.cs:66-68; BackwardNn.cs:12-21)
 * and the Erf/Exp/Sqrt cases of BackwardGraphOps.cs:10-139. */
int32_t om_unary_bwd(om_ctx* ctx, int32_t op, const float* g, const float* saved, float* dx, int64_t n);
/* dst[i] += src[i] in element order. Replaces Engine.AddInto (Engine.cs:330-344). */
int32_t om_add_into(om_ctx* ctx, float* dst, const float* src, int64_t n);
/* y[i] = x[i] * s (Mean backward division is x * (1/n) only when exact; this entry divides: y = x / d). */
int32_t om_div_scalar(om_ctx* ctx, const float* x, float d, float* y, int64_t n);
int32_t om_fill(om_ctx* ctx, float* dst, float value, int64_t n);
/* Zero-fills count buffers in one launch. Replaces Optimizer.ZeroGrad -> Backprop.ZeroGrad
 * (src/OneModel.Training/Optimizers.cs:222-228; Engine.cs:77-91). ptrs_host/len_host are host arrays. */
int32_t om_zero(om_ctx* ctx, int32_t count, float* const* ptrs_host, const int64_t* len_host);

/* y = x^p with the reference's exact cases for p in {1, 2, 0.5, -1} (Ops.Pow / PowScalar, Ops.GraphOps.cs:175-206), and
 * dx = g * d/dx x^p (PowDerivative, BackwardGraphOps.cs:44-76); x is the saved input. */
int32_t om_pow(om_ctx* ctx, const float* x, float exponent, float* y, int64_t n);
int32_t om_pow_bwd(om_ctx* ctx, const float* g, const float* x, float exponent, float* dx, int64_t n);
/* out = condition ? a : b over n contiguous elements (all three already broadcast to one shape, as Ops.Where does
 * before its loop, Ops.GraphOps.cs:244-300). The condition is Int32, non-zero = true: this ABI has no one-byte tensor
 * type, the binding widens the reference's Bool tensor when it uploads it. om_where_bwd: out = (condition == wanted) ? g : 0
 * (WhereBackward, BackwardGraphOps.cs:78-103). */
int32_t om_where(om_ctx* ctx, const int32_t* condition, const float* a, const float* b, float* out, int64_t n);
int32_t om_where_bwd(om_ctx* ctx, const int32_t* condition, const float* g, int32_t wanted, float* out, int64_t n);
/* Gather along one axis of data viewed as [outer, n, inner] with `count` indices (Int32 / Int64, negative counts from
 * the end): out [outer, count, inner] (Ops.Gather, Ops.GraphOps.cs:306-394). An index outside the axis sets the device
 * status word to OM_ERR_INDEX. om_gather_bwd: dx [outer, n, inner] = slices of g added per destination in increasing
 * index position (GatherBackward, BackwardGraphOps.cs:105-139); every destination element is written (zero when no
 * index points at it). */
int32_t om_gather_fwd(om_ctx* ctx, const float* data, const void* ids, int32_t id_dtype, int64_t outer, int64_t count,
                      int64_t n, int64_t inner, float* out);
int32_t om_gather_bwd(om_ctx* ctx, const float* g, const void* ids, int32_t id_dtype, int64_t outer, int64_t count,
                      int64_t n, int64_t inner, float* dx);

/* ---- data movement and broadcast sums ---------------------------------------------------------------- */

/* dst (strided) = src (strided) over `shape`, rank <= 8, strides in elements (negative allowed for Flip).
 * Covers Permute/Slice/Select/Expand/Flip/Concat clones and the slice-write of Slice/Select backward
 * (BackwardOps.cs:86-140; BackwardNn.cs:112-128; Tensor.Views.cs:11-21). */
int32_t om_strided_copy(om_ctx* ctx, int32_t rank, const int32_t* shape, const float* src,
                        const int64_t* src_strides, float* dst, const int64_t* dst_strides);
/* out[target] = sum of g over broadcast axes; g contiguous of `shape`; t_strides are the target's element
 * strides per axis of g, 0 where the target was broadcast. Sums in increasing element order with a double
 * accumulator per output (fixed two-level order). Replaces BackwardOps.SumTo (BackwardOps.cs:201-269). */
int32_t om_sum_to(om_ctx* ctx, int32_t rank, const int32_t* shape, const float* g,
                  const int64_t* t_strides, float* out, int64_t out_len);
/* out[cols] = column sums of g[rows,cols] (bias gradient; the common case of SumTo), double accumulation. */
int32_t om_colsum(om_ctx* ctx, const float* g, int32_t rows, int32_t cols, float* out, int32_t accumulate);
/* om_colsum without any device allocation. No counterpart in the reference: an addition for hosts that must not
 * allocate device memory once they are running (their whole device budget is handed out at start-up, or a driver
 * allocation's device-wide synchronisation and late out-of-memory failure are not acceptable in the middle of a run).
 * The per-chunk partial sums go to a fixed 1 MiB array inside the loaded module instead of the context's pool, so the
 * call takes nothing from the pool or the driver. Same arithmetic and same bits as om_colsum.
 * Limit: ceil(rows / 512) * cols <= 131072 and ceil(rows / 512) <= 65535; beyond it the call returns OM_ERR_UNSUPPORTED and
 * om_colsum is the one to use.
 * The first call on a device looks the array's address up (set-up work: make it before any stream capture). The array
 * is shared by every call on the device and keeps its last contents; calls that overlap on one device race on it, so
 * the caller serialises them. */
int32_t om_colsum_static(om_ctx* ctx, const float* g, int32_t rows, int32_t cols, float* out, int32_t accumulate);
/* Sum/Mean forward over one axis or all (axis < 0) of a contiguous tensor viewed as [outer, n, inner]
 * (Ops.Nn.cs:162-231), double accumulation in increasing order. */
int32_t om_reduce_fwd(om_ctx* ctx, const float* x, int64_t outer, int64_t n, int64_t inner, int32_t mean,
                      float* y);
/* Sum/Mean backward: dx[outer,n,inner] = g[outer,inner] (/ n when mean). Replaces ReduceBackward
 * (BackwardNn.cs:145-168). */
int32_t om_reduce_bwd(om_ctx* ctx, const float* g, int64_t outer, int64_t n, int64_t inner, int32_t mean,
                      float* dx);

/* ---- softmax family and losses ------------------------------------------------------------------------ */

/* Rows of `cols` elements. Forward: Ops.Softmax / Ops.LogSoftmax (Ops.Layers.cs:17-96): row max subtracted,
 * exp summed in double, lse = max + log(sum). Backward: BackwardNn.cs:26-80 (row sums in double). */
int32_t om_softmax_fwd(om_ctx* ctx, const float* x, int32_t rows, int32_t cols, float* y);
int32_t om_softmax_bwd(om_ctx* ctx, const float* g, const float* y, int32_t rows, int32_t cols, float* dx);
int32_t om_logsoftmax_fwd(om_ctx* ctx, const float* x, int32_t rows, int32_t cols, float* y);
int32_t om_logsoftmax_bwd(om_ctx* ctx, const float* g, const float* y, int32_t rows, int32_t cols, float* dx);
/* loss = -(sum or mean over counted rows) logp[n, target[n]]; rows whose target == ignore_index are skipped.
 * count (device int32, may be NULL) receives the number of counted rows. Out-of-range targets set the
 * device status word to OM_ERR_INDEX. Replaces Ops.NllLoss (Ops.Layers.cs:644-699). */
int32_t om_nll_fwd(om_ctx* ctx, const float* logp, const void* targets, int32_t target_dtype, int32_t rows,
                   int32_t cols, int32_t mean, int64_t ignore_index, float* loss, int32_t* count);
/* dx[rows,cols] = 0 except -g/count (mean) or -g at [n, target[n]]; g is the device scalar gradient of the
 * loss. Replaces NllBackward (BackwardNn.cs:602-634). */
int32_t om_nll_bwd(om_ctx* ctx, const float* g, const void* targets, int32_t target_dtype, int32_t rows,
                   int32_t cols, int32_t mean, int64_t ignore_index, float* dx);
/* Fused LogSoftmax + NllLoss of Losses.CrossEntropy (src/OneModel.Training/Losses.cs:21-32): forward writes
 * logp (may be NULL when only the loss is wanted... it is needed by the backward) and the loss; backward
 * writes dlogits = g*(exp(logp) * s - onehot)/count directly, the composition of NllBackward and the
 * LogSoftmax backward above. `denominator` > 0 overrides the counted-row divisor (data-parallel shards
 * divide by the global count). */
int32_t om_cross_entropy_fwd(om_ctx* ctx, const float* logits, const void* targets, int32_t target_dtype,
                             int32_t rows, int32_t cols, int32_t mean, int64_t ignore_index,
                             float denominator, float* logp, float* loss, int32_t* count);
int32_t om_cross_entropy_bwd(om_ctx* ctx, const float* g, const float* logp, const void* targets,
                             int32_t target_dtype, int32_t rows, int32_t cols, int32_t mean,
                             int64_t ignore_index, float denominator, float* dlogits);
/* The same with one row pitch `ld` (elements, >= cols) shared by logits, logp and dlogits. */
int32_t om_cross_entropy_fwd_ld(om_ctx* ctx, const float* logits, const void* targets, int32_t target_dtype,
                                int32_t rows, int32_t cols, int32_t ld, int32_t mean, int64_t ignore_index,
                                float denominator, float* logp, float* loss, int32_t* count);
int32_t om_cross_entropy_bwd_ld(om_ctx* ctx, const float* g, const float* logp, const void* targets,
                                int32_t target_dtype, int32_t rows, int32_t cols, int32_t ld, int32_t mean,
                                int64_t ignore_index, float denominator, float* dlogits);

/* ---- normalisation ------------------------------------------------------------------------------------ */

/* y = (x-mean)*inv*gamma + beta per row; mean[rows], inv[rows] (may be NULL) receive the saved statistics.
 * Replaces Ops.LayerNorm -> NormKernels.Rows (Ops.Layers.cs:109-145; Kernels/Exact/NormKernels.cs:39-128). */
int32_t om_layernorm_fwd(om_ctx* ctx, const float* x, const float* gamma, const float* beta, int32_t rows,
                         int32_t cols, float eps, float* y, float* mean, float* inv);
/* dx, dgamma, dbeta (each may be NULL). Row sums and the column accumulators of dgamma/dbeta are double,
 * combined in a fixed order. Replaces LayerNormBackward (BackwardNn.cs:170-242). */
int32_t om_layernorm_bwd(om_ctx* ctx, const float* g, const float* x, const float* gamma, const float* mean,
                         const float* inv, int32_t rows, int32_t cols, float* dx, float* dgamma,
                         float* dbeta, int32_t accumulate_params);
/* NCHW batch normalisation. Training: batch statistics in double, running stats updated in place with the
 * unbiased variance (Ops.Layers.cs:158-277). mean[C], inv[C] receive the saved statistics. */
int32_t om_batchnorm_fwd(om_ctx* ctx, const float* x, const float* gamma, const float* beta,
                         float* running_mean, float* running_var, int32_t n, int32_t c, int32_t plane,
                         int32_t training, float momentum, float eps, float* y, float* mean, float* inv);
/* Replaces BatchNormBackward (BackwardNn.cs:244-307). */
int32_t om_batchnorm_bwd(om_ctx* ctx, const float* g, const float* x, const float* gamma, const float* mean,
                         const float* inv, int32_t n, int32_t c, int32_t plane, int32_t training, float* dx,
                         float* dgamma, float* dbeta, int32_t accumulate_params);

/* ---- embedding ------------------------------------------------------------------------------------------ */

/* out[i,:] = table[ids[i],:]. Ids outside [0,V) set OM_ERR_INDEX. Replaces Ops.Embedding (Ops.Layers.cs:549-628). */
int32_t om_embedding_fwd(om_ctx* ctx, const float* table, int32_t v, int32_t dim, const void* ids,
                         int32_t id_dtype, int64_t n, float* out);
/* dtable[V,dim]: rows of g added per id in increasing position order starting from zero (or from the
 * existing contents when accumulate != 0), padding id skipped. No atomics: positions are sorted by id on the
 * device and each table row is summed by one thread in position order. Replaces EmbeddingBackward
 * (BackwardNn.cs:508-546). */
int32_t om_embedding_bwd(om_ctx* ctx, const float* g, const void* ids, int32_t id_dtype, int64_t n,
                         int32_t v, int32_t dim, int64_t padding_index, float* dtable, int32_t accumulate);

/* ---- attention ------------------------------------------------------------------------------------------ */

/* out = softmax(scale*Q*K^T + mask)*V per (batch, head); q [B,H,Lq,D], k,v [B,H,Lk,D] contiguous; mask
 * additive [Lq,Lk] (mask_batch_stride 0) or [B,Lq,Lk] (stride Lq*Lk) or NULL. lse [B,H,Lq] (may be NULL)
 * receives the row log-sum-exp for the backward. Replaces Ops.Attention -> AttentionDriver.Run
 * (Ops.Layers.cs:746-807; Kernels/AttentionDriver.cs:29). */
int32_t om_attention_fwd(om_ctx* ctx, const float* q, const float* k, const float* v, const float* mask,
                         int64_t mask_batch_stride, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d,
                         float scale, float* out, float* lse);
/* dq, dk, dv (each may be NULL) from g = dOut, recomputing P from q,k (and lse when given).
 * Replaces AttentionBackward (BackwardNn.cs:636-701). */
int32_t om_attention_bwd(om_ctx* ctx, const float* g, const float* q, const float* k, const float* v,
                         const float* mask, int64_t mask_batch_stride, const float* lse, int32_t b,
                         int32_t h, int32_t lq, int32_t lk, int32_t d, float scale, float* dq, float* dk,
                         float* dv);

/* Element strides of an activation seen as [B, H, L, D] with D contiguous: where the [L, D] matrix of (batch, head)
 * starts (batch, head) and how far apart its rows are (row >= D). [B,H,L,D] contiguous is {H*L*D, L*D, D}; the output
 * of a Linear, [B, L, H*D], read per head without a copy is {L*H*D, D, H*D}. */
typedef struct om_head_strides {
  int64_t batch, head, row;
} om_head_strides;
/* om_attention_fwd / om_attention_bwd on activations addressed through om_head_strides, so that the head split
 * ([B,L,H*D] -> [B,H,L,D]) and merge permutes around Ops.Attention (the Reshape + Permute pairs of
 * MultiHeadAttention.Forward, Layers.cs:503-520, and their inverse-permute copies in the backward, BackwardOps.cs:86-99)
 * need no copy: the tensor-map (or the fp32 kernel's index arithmetic) walks the strided layout directly. */
int32_t om_attention_fwd_strided(om_ctx* ctx, const float* q, const om_head_strides* qs, const float* k,
                                 const om_head_strides* ks, const float* v, const om_head_strides* vs,
                                 const float* mask, int64_t mask_batch_stride, int32_t b, int32_t h, int32_t lq,
                                 int32_t lk, int32_t d, float scale, float* out, const om_head_strides* os,
                                 float* lse);
int32_t om_attention_bwd_strided(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q,
                                 const om_head_strides* qs, const float* k, const om_head_strides* ks,
                                 const float* v, const om_head_strides* vs, const float* mask,
                                 int64_t mask_batch_stride, const float* lse, int32_t b, int32_t h, int32_t lq,
                                 int32_t lk, int32_t d, float scale, float* dq, const om_head_strides* dqs,
                                 float* dk, const om_head_strides* dks, float* dv, const om_head_strides* dvs);
/* om_attention_bwd_strided with the forward's output `out` (strides os) at hand. The reference recomputes the row dots
 * rowsum(P dP) from the probabilities (BackwardNn.cs:660-676); with O = P V they equal rowsum(dO O), which lets the
 * several-tile kernel walk the key tiles once instead of twice. out == NULL is om_attention_bwd_strided. */
int32_t om_attention_bwd_strided_out(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q,
                                     const om_head_strides* qs, const float* k, const om_head_strides* ks,
                                     const float* v, const om_head_strides* vs, const float* out,
                                     const om_head_strides* os, const float* mask, int64_t mask_batch_stride,
                                     const float* lse, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d,
                                     float scale, float* dq, const om_head_strides* dqs, float* dk,
                                     const om_head_strides* dks, float* dv, const om_head_strides* dvs);
/* Ops.Attention forward (src/OneModel/Tensors/Ops.Layers.cs, the attention op that AttentionBackward differentiates) with
 * bfloat16 product operands, for sequences of several tiles: out = softmax(scale q k^T + mask) v per (batch, head), from the
 * bfloat16 copies of q, k, v. A CTA per (128 queries, batch, head) walks the key tiles twice (row maxima first; then
 * exponentials, their fp32 row sums and the second product with the exponentials rounded to bfloat16), two CTAs per SM.
 * Without a mask it walks them once where scale |q_i| max_j |k_j| (a bound on row i's scores; the key norms come from a
 * small kernel in front) is at most 40 for every row of the tile: the exponentials are taken against that bound instead
 * of the row maximum, which changes neither the normalised result nor the log-sum-exp beyond rounding.
 * out is fp32, out16 (may be NULL) its bfloat16 copy with the same strides, lse (may be NULL) the row log-sum-exp
 * [b * h, lq] that om_attention_bwd_bf16 takes. Built for head dimension 64, any lq and lk, a positive scale, at most 65535
 * (batch, head) pairs (om_attention_fwd_bf16_supported tells); operand strides multiples of 8. */
int32_t om_attention_fwd_bf16_supported(om_ctx* ctx, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d, float scale);
int32_t om_attention_fwd_bf16(om_ctx* ctx, const uint16_t* q16, const om_head_strides* qs, const uint16_t* k16,
                              const om_head_strides* ks, const uint16_t* v16, const om_head_strides* vs, const float* mask,
                              int64_t mask_batch_stride, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d, float scale,
                              float* out, uint16_t* out16, const om_head_strides* os, float* lse);
/* AttentionBackward (src/OneModel/Tensors/Autograd/BackwardNn.cs:636-701) for sequences of several 128-key tiles with
 * bfloat16 product operands: a CTA per (batch, head, 128-key tile) forms S = Q K^T and dP = dO V^T half a tile at a time
 * in two alternating accumulator buffers of tensor memory, P = exp(scale S + mask - lse) and dS = P (dP - rowsum(dO o O))
 * scale in registers (rounded to bfloat16 as the operands of the three output products), accumulates dV and dK of its key
 * tile over the query tiles in tensor memory, and writes its part of dQ per query tile to a pooled workspace; a second
 * launch sums the parts of dQ over the key tiles in increasing order (a first one forms the row dots). Nothing of size
 * Lq x Lk is written to memory. q16 / k16 / v16 / g16 are the bfloat16 copies of q, k, v and of the output gradient g; g and
 * out (the forward's output) are read in fp32 for the row dots; lse is the forward's row log-sum-exp. Each of dq, dk, dv
 * is written as fp32, as bfloat16 (dq16 / dk16 / dv16, same strides) or both: pass NULL for the form that is not wanted
 * (bfloat16 alone is all that a following product reads). Built for head dimension 64, any Lq and Lk, at most
 * 65535 (batch, head) pairs (om_attention_bwd_bf16_supported tells); strides of the bfloat16 operands multiples of 8. */
int32_t om_attention_bwd_bf16_supported(om_ctx* ctx, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d);
int32_t om_attention_bwd_bf16(om_ctx* ctx, const uint16_t* g16, const float* g, const om_head_strides* gs,
                              const uint16_t* q16, const om_head_strides* qs, const uint16_t* k16, const om_head_strides* ks,
                              const uint16_t* v16, const om_head_strides* vs, const float* out, const om_head_strides* os,
                              const float* mask, int64_t mask_batch_stride, const float* lse, int32_t b, int32_t h,
                              int32_t lq, int32_t lk, int32_t d, float scale, float* dq, uint16_t* dq16,
                              const om_head_strides* dqs, float* dk, uint16_t* dk16, const om_head_strides* dks, float* dv,
                              uint16_t* dv16, const om_head_strides* dvs);

/* ---- pooling and convolution ---------------------------------------------------------------------------- */

/* The 16 integers of ConvShape (src/OneModel/Kernels/Conv.cs:11-13) in the reference's order. */
typedef struct om_conv_shape {
  int32_t n, cin, h, w, cout, kh, kw;
  int32_t stride_h, stride_w, pad_top, pad_left, pad_bottom, pad_right, dil_h, dil_w, groups;
} om_conv_shape;
/* y [N,Cout,OH,OW] = conv(x [N,Cin,H,W], w [Cout,Cin/g,KH,KW]) + bias (may be NULL).
 * Replaces Ops.Conv2d -> Conv.Run (Ops.Layers.cs:279-348). */
int32_t om_conv2d_fwd(om_ctx* ctx, const om_conv_shape* s, const float* x, const float* w, const float* bias,
                      float* y);
/* Replaces the three branches of ConvBackward (BackwardNn.cs:317-402). */
int32_t om_conv2d_dgrad(om_ctx* ctx, const om_conv_shape* s, const float* g, const float* w, float* dx);
int32_t om_conv2d_wgrad(om_ctx* ctx, const om_conv_shape* s, const float* g, const float* x, float* dw,
                        int32_t accumulate);
int32_t om_conv2d_dbias(om_ctx* ctx, const om_conv_shape* s, const float* g, float* dbias, int32_t accumulate);

/* Max pooling over NCHW planes; idx receives the Int32 flat NCHW index of each maximum (first wins ties,
 * NaN wins), bit-exact with ReferenceKernels.MaxPool2d (src/OneModel/Tensors/TensorKernels.cs:242-295). */
int32_t om_maxpool_fwd(om_ctx* ctx, const float* x, int32_t planes, int32_t h, int32_t w, int32_t kh,
                       int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw, float* y, int32_t* idx);
/* dx[idx[i]] += g[i] in output order from zero, without atomics (each input element gathers the outputs
 * that selected it in increasing output index). Replaces MaxPoolBackward (BackwardOps.cs:285-298). */
int32_t om_maxpool_bwd(om_ctx* ctx, const float* g, const int32_t* idx, int32_t planes, int32_t h, int32_t w,
                       int32_t oh, int32_t ow, int32_t kh, int32_t kw, int32_t sh, int32_t sw, int32_t ph,
                       int32_t pw, float* dx);
/* Average pooling (Ops.Layers.cs:414-461) and AvgPoolBackward / PoolWindow (BackwardNn.cs:464-506). */
int32_t om_avgpool_fwd(om_ctx* ctx, const float* x, int32_t planes, int32_t h, int32_t w, int32_t kh,
                       int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t count_include_pad,
                       float* y);
int32_t om_avgpool_bwd(om_ctx* ctx, const float* g, int32_t planes, int32_t h, int32_t w, int32_t kh,
                       int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t count_include_pad,
                       float* dx);

/* Resize of NCHW planes [planes, H, W] to [planes, out_h, out_w]: mode 0 nearest (source index min(floor(dst*in/out), in-1)),
 * mode 1 bilinear with or without aligned corners; the source coordinate rule of Ops.SourceCoord (Ops.Spatial.cs:200-235).
 * Replaces Ops.Resize2d (Ops.Spatial.cs:148-197). The backward gathers, per input pixel, the weighted terms the
 * reference scatters in output order (ResizeBackward, BackwardRecurrent.cs:371-412). */
int32_t om_resize2d_fwd(om_ctx* ctx, const float* x, int64_t planes, int32_t h, int32_t w, int32_t out_h, int32_t out_w,
                        int32_t mode, int32_t align_corners, float* y);
int32_t om_resize2d_bwd(om_ctx* ctx, const float* g, int64_t planes, int32_t h, int32_t w, int32_t out_h, int32_t out_w,
                        int32_t mode, int32_t align_corners, float* dx);

/* ---- recurrent and CTC ---------------------------------------------------------------------------------- */

/* One LSTM layer direction over x [T,B,I]: gates = x*W_ih^T + b_ih + h*W_hh^T + b_hh in i,f,g,o order.
 * Outputs y [T,B,H] and the saved slots gates [T,B,4H] (post-activation), c [T,B,H], tanh_c [T,B,H].
 * h0/c0 may be NULL (zeros). Replaces Ops.LstmLayer (src/OneModel/Tensors/Ops.Recurrent.cs:40-146). */
int32_t om_lstm_layer_fwd(om_ctx* ctx, int32_t reverse, int32_t t, int32_t b, int32_t i, int32_t h,
                          const float* x, const float* w_ih, const float* w_hh, const float* b_ih,
                          const float* b_hh, const float* h0, const float* c0, float* y, float* gates,
                          float* c, float* tanh_c);
/* Backward through time. gy [T,B,H]; ghn, gcn (may be NULL) are gradients of the final states. Outputs (each
 * may be NULL): dx [T,B,I], dw_ih [4H,I], dw_hh [4H,H], db_ih [4H], db_hh [4H], dh0, dc0 [B,H].
 * Replaces LstmBackward + ColumnSums (BackwardRecurrent.cs:10-113,224-246). */
int32_t om_lstm_layer_bwd(om_ctx* ctx, int32_t reverse, int32_t t, int32_t b, int32_t i, int32_t h,
                          const float* gy, const float* ghn, const float* gcn, const float* x,
                          const float* y, const float* w_ih, const float* w_hh, const float* h0,
                          const float* c0, const float* gates, const float* c, const float* tanh_c,
                          float* dx, float* dw_ih, float* dw_hh, float* db_ih, float* db_hh, float* dh0,
                          float* dc0);

/* Both directions of one bidirectional LSTM layer over the same input, zero initial states: the forward direction runs on
 * the context's stream and the reverse direction concurrently on an auxiliary stream (fork / join by events; inside
 * om_graph_begin/end both become branches of the graph), since one direction's per-step kernels fill only a few SMs.
 * Index 0 of every array = forward direction, 1 = reverse. b_ih / b_hh may be NULL arrays. Per direction the arithmetic
 * is that of om_lstm_layer_fwd / om_lstm_layer_bwd (Recurrent.Forward, src/OneModel.Training/Recurrent.cs:28-67). */
int32_t om_lstm_bilayer_fwd(om_ctx* ctx, int32_t t, int32_t b, int32_t i, int32_t h, const float* x,
                            const float* const* w_ih, const float* const* w_hh, const float* const* b_ih,
                            const float* const* b_hh, float* const* y, float* const* gates, float* const* c,
                            float* const* tanh_c);
/* dx[0] and dx[1] are the two directions' input gradients (the caller adds them); any output array may be NULL. */
int32_t om_lstm_bilayer_bwd(om_ctx* ctx, int32_t t, int32_t b, int32_t i, int32_t h, const float* const* gy,
                            const float* x, const float* const* y, const float* const* w_ih,
                            const float* const* w_hh, const float* const* gates, const float* const* c,
                            const float* const* tanh_c, float* const* dx, float* const* dw_ih,
                            float* const* dw_hh, float* const* db_ih, float* const* db_hh);

/* One direction of one GRU layer over a whole sequence, PyTorch's gate formulation. x [T,B,I], w_ih [3H,I],
 * w_hh [3H,H], b_ih / b_hh [3H] or NULL, h0 [B,H] or NULL (zeros). Outputs: y [T,B,H] and the saved slots of the
 * backward: gates [T,B,3H] (activated r, z, n) and hn [T,B,H] (the hidden side of n, W_hn h' + b_hn).
 * Replaces Ops.GruLayer (Ops.Recurrent.cs:148-260). */
int32_t om_gru_layer_fwd(om_ctx* ctx, int32_t reverse, int32_t t, int32_t b, int32_t i, int32_t h, const float* x,
                         const float* w_ih, const float* w_hh, const float* b_ih, const float* b_hh,
                         const float* h0, float* y, float* gates, float* hn);
/* Backward through time of om_gru_layer_fwd from gy [T,B,H]. Each output may be NULL: dx [T,B,I], dw_ih [3H,I],
 * dw_hh [3H,H], db_ih [3H] (column sums of the input-side gate gradients), db_hh [3H] (of the hidden-side ones,
 * whose n column carries the factor r), dh0 [B,H]. Replaces GruBackward + ColumnSums (BackwardRecurrent.cs:115-246). */
int32_t om_gru_layer_bwd(om_ctx* ctx, int32_t reverse, int32_t t, int32_t b, int32_t i, int32_t h, const float* gy,
                         const float* x, const float* y, const float* w_ih, const float* w_hh, const float* h0,
                         const float* gates, const float* hn, float* dx, float* dw_ih, float* dw_hh,
                         float* db_ih, float* db_hh, float* dh0);

/* CTC negative log-likelihood per sequence from log-probabilities lp [T,B,C] (double-precision alpha
 * recursion in log space), targets concatenated (int32) with target_lengths[B], input_lengths[B].
 * nll[B] receives the per-sequence losses (zero_infinity replaces +inf by 0); loss receives the reduction
 * (0 = none: loss unused, 1 = mean over batch of nll/max(1,len), 2 = sum).
 * Replaces Ops.CtcLoss -> CtcLossMath.Alpha (src/OneModel/Tensors/CtcLoss.cs:40-217). */
int32_t om_ctc_loss(om_ctx* ctx, const float* lp, int32_t t, int32_t b, int32_t c, const int32_t* targets,
                    const int32_t* target_lengths, const int32_t* input_lengths, int32_t blank,
                    int32_t reduction, int32_t zero_infinity, float* nll, float* loss);
/* grad [T,B,C] of the reduced loss with respect to lp given g (device: scalar for mean/sum, [B] for none).
 * Replaces CtcBackward -> CtcLossMath.Gradient (BackwardRecurrent.cs:253-296; CtcLoss.cs:219-281). */
int32_t om_ctc_grad(om_ctx* ctx, const float* g, const float* lp, int32_t t, int32_t b, int32_t c,
                    const int32_t* targets, const int32_t* target_lengths, const int32_t* input_lengths,
                    const float* nll, int32_t blank, int32_t reduction, int32_t zero_infinity, float* grad);
/* Greedy CTC decode of lp [T,B,C]: per step argmax (lowest index on ties, NaN never wins over a number),
 * merged runs, blanks dropped. labels, first_step, last_step are [B,T] padded with -1 (first/last may be
 * NULL): the label of each kept run and the first and last frame it covers; lengths [B]. Integers are
 * bit-exact with Ctc.Greedy (src/OneModel/Tensors/Ctc.cs:89-190). */
int32_t om_ctc_greedy(om_ctx* ctx, const float* lp, int32_t t, int32_t b, int32_t c,
                      const int32_t* input_lengths, int32_t blank, int32_t* labels, int32_t* first_step,
                      int32_t* last_step, int32_t* lengths);

/* ---- optimizers ------------------------------------------------------------------------------------------ */

/* Per-step scalars of Adam/AdamW computed on the host in double exactly as Adam.BeginStep does
 * (src/OneModel.Training/Optimizers.cs:501-508): step_size = (float)(lr / (1 - beta1^t)),
 * sqrt_bc2 = (float)sqrt(1 - beta2^t). grad_scale multiplies every gradient first (1 = the reference;
 * data-parallel runs pass 1 because the loss is already divided by the global row count). */
typedef struct om_adam_hyper {
  float lr, beta1, beta2, eps, weight_decay, step_size, sqrt_bc2, grad_scale;
  int32_t decoupled; /* AdamW */
  int32_t amsgrad;
} om_adam_hyper;
/* One fused multi-tensor launch over n_tensors parameters: per element exactly the rounding sequence of
 * Adam.UpdateRange (Optimizers.cs:554-589), no fused multiply-add. Host arrays of device pointers; vmax may be
 * NULL unless amsgrad. If hyper_dev is not NULL the kernel reads the scalars from that device struct instead
 * (so a captured graph can be replayed with new per-step scalars). */
int32_t om_optim_adam_step(om_ctx* ctx, int32_t n_tensors, float* const* p_host, const float* const* g_host,
                           float* const* m_host, float* const* v_host, float* const* vmax_host,
                           const int64_t* len_host, const om_adam_hyper* hyper_host,
                           const om_adam_hyper* hyper_dev);
/* The same step that also refreshes the bfloat16 copies of the parameters it updates (p16_host[i] may be NULL: no copy for
 * that parameter): the weights of the Linear layers are product operands under OM_BF16_OPERANDS, and their copies are then
 * current without a cast pass after the step. */
int32_t om_optim_adam_step_b16(om_ctx* ctx, int32_t n_tensors, float* const* p_host, const float* const* g_host,
                               float* const* m_host, float* const* v_host, float* const* vmax_host,
                               uint16_t* const* p16_host, const int64_t* len_host, const om_adam_hyper* hyper_host,
                               const om_adam_hyper* hyper_dev);
typedef struct om_sgd_hyper {
  float lr, weight_decay, momentum, dampening, grad_scale;
  int32_t nesterov;
  int32_t has_momentum;
} om_sgd_hyper;
/* Sgd.Update (Optimizers.cs:335-373). first_host[i] != 0 marks a momentum buffer not yet initialised. */
int32_t om_optim_sgd_step(om_ctx* ctx, int32_t n_tensors, float* const* p_host, const float* const* g_host,
                          float* const* buf_host, const int32_t* first_host, const int64_t* len_host,
                          const om_sgd_hyper* hyper_host, const om_sgd_hyper* hyper_dev);
/* Global gradient-norm clipping: norm = sqrt(sum g^2) accumulated in double in parameter and element order
 * (fixed two-level partition), coef = (float)(max_norm/(norm+1e-6)); gradients are scaled when coef < 1 and
 * the norm is finite. total_norm (device float, may be NULL) receives the norm.
 * Replaces GradClip.ClipNorm (src/OneModel.Training/Schedules.cs:22-100). */
int32_t om_grad_norm_clip(om_ctx* ctx, int32_t n_tensors, float* const* g_host, const int64_t* len_host,
                          float max_norm, int32_t infinity_norm, float* total_norm);
/* Replaces GradClip.ClipValue (Schedules.cs:120-143). */
int32_t om_grad_clip_value(om_ctx* ctx, int32_t n_tensors, float* const* g_host, const int64_t* len_host,
                           float clip);

/* Dropout (the mask of the reference's Dropout module, src/OneModel.Training/Layers.cs:308-371; row a29 of the forward
 * ops). Element i of call number `draw` is kept, scaled by 1/(1-p), when u >= p with
 * u = (Mix(Mix(seed + draw*G) + (i+1)*G) >> 40) * 2^-24, Mix the SplitMix64 finaliser and G = 0x9E3779B97F4A7C15
 * (Generator.cs:10-48): the same bits as the reference. `draws` is the module's call counter in DEVICE memory (int64[1],
 * the "draws" buffer of the state dict): om_dropout_fwd reads it, writes y = x * mask (and the mask when `mask` is not
 * NULL), notes the value it used in draw_used (device int64[1], may be NULL) and then advances the counter by one in
 * stream order, so a captured step draws a new mask on every replay. om_dropout_bwd forms the mask again from draw_used:
 * dx = g * mask (MulBackward of the reference's Ops.Mul(input, mask), BackwardOps.cs:23-40). om_dropout_mask writes the
 * mask of the call number in `draw` without touching a counter. p in [0, 1). x and y (g and dx) may alias. */
int32_t om_dropout_mask(om_ctx* ctx, uint64_t seed, const int64_t* draw, float p, int64_t n, float* mask);
int32_t om_dropout_fwd(om_ctx* ctx, const float* x, int64_t n, float p, uint64_t seed, int64_t* draws, int64_t* draw_used,
                       float* y, float* mask);
int32_t om_dropout_bwd(om_ctx* ctx, const float* g, int64_t n, float p, uint64_t seed, const int64_t* draw_used, float* dx);
/* mask[i] = 1 where targets[i] != ignore_index, else 0 (the counted rows of Losses.CrossEntropy's label-smoothing term,
 * Losses.cs:33-46). */
int32_t om_target_mask(om_ctx* ctx, const void* targets, int32_t target_dtype, int32_t rows, int64_t ignore_index, float* mask);

/* Row-sparse updates for embedding tables (SparseAdam and the sparse path of Sgd, Optimizers.cs:377-397,625-722). The
 * reference carries a RowSparseGradient (sorted unique rows + coalesced values); here the same information is the
 * dense-format table gradient of om_embedding_bwd plus touched[rows] from om_rows_touched (how many positions of the
 * step's id list name each row; ids equal to padding_index are skipped, an id outside [0, rows) sets OM_ERR_INDEX).
 * Only rows with touched != 0 are updated; the moments of the other rows do not decay. step_size is the host-computed
 * lr * sqrt(1 - beta2^t) / (1 - beta1^t) of SparseAdam.BeginStep (double arithmetic, rounded once). */
int32_t om_rows_touched(om_ctx* ctx, const void* ids, int32_t id_dtype, int64_t n, int32_t rows, int64_t padding_index,
                        int32_t* touched);
int32_t om_optim_sparse_adam_step(om_ctx* ctx, float* p, const float* g, float* m, float* v, const int32_t* touched,
                                  int32_t rows, int32_t width, float beta1, float beta2, float eps, float step_size);
int32_t om_optim_sparse_sgd_step(om_ctx* ctx, float* p, const float* g, const int32_t* touched, int32_t rows,
                                 int32_t width, float lr);

/* The row-sparse table gradient as an object of its own (RowSparseGradient.cs:14-120 of the reference): rows[k], k <
 * *row_count, are the looked-up row numbers in strictly ascending order, each once (the padding row is absent), and
 * values[k, 0..dim) is the gradient of row rows[k]: the sum of the output gradients g[pos, :] of the row's lookups in
 * increasing position order starting from zero (EmbeddingSparseBackward, BackwardNn.cs:548-600), which are the bits of the
 * dense gradient's row. rows, values and row_count are device memory; the count is not read back by any entry point, so the
 * calls can be captured in a graph. The arrays have `capacity` entries, at least min(n, v); the entries behind the count
 * are row -1 with zero values, so values can be scaled or normed as a plain [capacity, dim] tensor (gradient clipping,
 * Schedules.cs:33). An id outside [0, v) sets OM_ERR_INDEX as in om_embedding_bwd. */
int32_t om_embedding_bwd_sparse(om_ctx* ctx, const float* g, const void* ids, int32_t id_dtype, int64_t n, int32_t v,
                                int32_t dim, int64_t padding_index, int32_t* rows, float* values, int32_t capacity,
                                int32_t* row_count);
/* dense[rows[k], :] += values[k, :] for k < *row_count (RowSparseGradient.AddTo, :47-63; ToDense is this into zeros).
 * dense is [v, dim]. */
int32_t om_rowsparse_add_to(om_ctx* ctx, const int32_t* rows, const float* values, const int32_t* row_count,
                            int32_t capacity, int32_t dim, float* dense, int32_t v);
/* a + b (RowSparseGradient.Merge, :66-116): the union of the rows in ascending order; a row in both gets a's values plus
 * b's (a first), a row in one gets that one's values (b's added to zero). The result needs capacity
 * min(capacity_a + capacity_b, v). */
int32_t om_rowsparse_merge(om_ctx* ctx, const int32_t* rows_a, const float* values_a, const int32_t* count_a,
                           int32_t capacity_a, const int32_t* rows_b, const float* values_b, const int32_t* count_b,
                           int32_t capacity_b, int32_t v, int32_t dim, int32_t* rows_out, float* values_out,
                           int32_t capacity_out, int32_t* count_out);
/* SparseAdam.UpdateSparse / Sgd.UpdateSparse (Optimizers.cs:696-722, 377-397) from such a row list: the arithmetic of the
 * two entry points above on the listed rows only, so the table has the same bits as when it is updated from the
 * dense-format gradient with touched counts. p, m, v are [table_rows, width]. */
int32_t om_optim_sparse_adam_step_rows(om_ctx* ctx, float* p, const int32_t* rows, const float* values,
                                       const int32_t* row_count, int32_t capacity, float* m, float* v, int32_t table_rows,
                                       int32_t width, float beta1, float beta2, float eps, float step_size);
int32_t om_optim_sparse_sgd_step_rows(om_ctx* ctx, float* p, const int32_t* rows, const float* values,
                                      const int32_t* row_count, int32_t capacity, int32_t table_rows, int32_t width, float lr);

/* ---- data parallel ---------------------------------------------------------------------------------------- */

/* The reference is single-process; these have no counterpart there. One rank per process and GPU.
 * om_dp_unique_id fills a 128-byte NCCL id on rank 0 which the caller distributes to all ranks;
 * om_dp_init joins the communicator. Buckets are contiguous ranges of gradient memory registered once;
 * om_dp_allreduce_bucket launches ncclAllReduce(sum, fp32) on a communication stream after the work
 * already queued on the context stream; om_dp_wait makes the context stream wait for all launched buckets
 * and polls the communicator for asynchronous errors with a host deadline (OM_ERR_TIMEOUT / OM_ERR_NCCL). */
int32_t om_dp_unique_id(om_ctx* ctx, uint8_t id128[128]);
int32_t om_dp_init(om_ctx* ctx, const uint8_t id128[128], int32_t rank, int32_t world);
int32_t om_dp_register_bucket(om_ctx* ctx, int32_t bucket_id, float* base, int64_t count);
int32_t om_dp_allreduce_bucket(om_ctx* ctx, int32_t bucket_id);
int32_t om_dp_allreduce(om_ctx* ctx, void* buf, int64_t count, int32_t dtype); /* small in-stream sums */
int32_t om_dp_wait(om_ctx* ctx, int32_t timeout_ms);
/* Makes the context stream wait for ONE launched bucket: the optimizer can update the parameters of a bucket while
 * later buckets are still being reduced. om_dp_wait afterwards collects the rest and checks the communicator. */
int32_t om_dp_wait_bucket(om_ctx* ctx, int32_t bucket_id);
int32_t om_dp_finalize(om_ctx* ctx);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* ONEMODEL_B200_H */
