// Products with bfloat16 operands and fp32 accumulation (the OM_BF16_OPERANDS tier): the caller keeps, beside each fp32
// tensor that feeds a product, a bfloat16 copy rounded to nearest even (om_cast_bf16, or the fused producers that write it
// on their way out), and the entry points here multiply those copies on the tensor pipe (om_gemm_ws.cu, kind::f16) into
// fp32 results. Master weights, gradients, bias sums and everything that is not a product operand stay fp32.
#include <cuda_bf16.h>

#include "om_common.cuh"

namespace om {

bool gemm_ws_supported(om_ctx* ctx, int elem, int m, int n, int k, const void* A, long long lda, const void* B, long long ldb, const float* C,
                       long long ldc);
int32_t gemm_ws(om_ctx* ctx, int elem, int ta, int tb, int m, int n, int k, const void* A, long long lda, const void* B, long long ldb, float* C,
                long long ldc, int acc, const float* bias, uint16_t* C16);
int32_t gemm_ws_act(om_ctx* ctx, int elem, int ta, int tb, int m, int n, int k, const void* A, long long lda, const void* B, long long ldb, float* C,
                    long long ldc, int acc, const float* bias, uint16_t* C16, int act, int op, const float* aux, long long ld_aux);
bool gemm_ws_act_ok(int act, int op, int m, int n, int k, const float* C, long long ldc, const uint16_t* C16, const float* aux, long long ld_aux);
int32_t colsum_ld(om_ctx* ctx, const float* g, int32_t rows, int32_t cols, int64_t ld, float* out, int32_t accumulate);
int32_t colsum16_ld(om_ctx* ctx, const uint16_t* g16, int32_t rows, int32_t cols, int64_t ld, float* out, int32_t accumulate);

// Eight elements per thread: two 16-byte loads, one 16-byte store.
__global__ void cast_bf16_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, int64_t n) {
  pdl_enter();
  const int64_t n8 = n >> 3;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += stride) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(src) + 2 * i);
    const float4 b = __ldg(reinterpret_cast<const float4*>(src) + 2 * i + 1);
    __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
    uint4 o;
    o.x = *reinterpret_cast<uint32_t*>(&p0);
    o.y = *reinterpret_cast<uint32_t*>(&p1);
    o.z = *reinterpret_cast<uint32_t*>(&p2);
    o.w = *reinterpret_cast<uint32_t*>(&p3);
    reinterpret_cast<uint4*>(dst)[i] = o;
  }
  // Tail (fewer than eight elements), by the first threads of the grid.
  const int64_t t = (n8 << 3) + blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t < n) {
    __nv_bfloat16 v = __float2bfloat16_rn(src[t]);
    dst[t] = *reinterpret_cast<uint16_t*>(&v);
  }
}

// The bfloat16 copy of a row-pitched matrix, element for element (the pitch columns are converted along: harmless).
int32_t cast_bf16_rows(om_ctx* ctx, const float* src, uint16_t* dst, int rows, int cols, long long ld) {
  if (rows < 1 || cols < 1) return OM_OK;
  const int64_t n = (int64_t)(rows - 1) * ld + cols;
  launch_chained(ctx, cast_bf16_kernel, grid_for(ctx, (n + 7) / 8, 256), 256, 0, src, dst, n);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? OM_OK : check_cuda(ctx, e, "cast_bf16_rows");
}

static int32_t check_args(om_ctx* ctx, const char* who, int m, int n, int k, const void* A, long long lda, const void* B, long long ldb, const float* C,
                          long long ldc) {
  if (m < 0 || n < 0 || k < 1) return fail(ctx, OM_ERR_SHAPE, "%s: m %d n %d k %d", who, m, n, k);
  if (m == 0 || n == 0) return OM_OK;
  if (!gemm_ws_supported(ctx, 1, m, n, k, A, lda, B, ldb, C, ldc))
    return fail(ctx, OM_ERR_UNSUPPORTED,
                "%s: bfloat16 operands need pitches that are multiples of 8 elements (A %lld, B %lld), a C pitch that is a multiple of 4 (%lld) "
                "and 16-byte aligned base addresses; use the fp32-operand entry point for this shape",
                who, lda, ldb, ldc);
  return OM_OK;
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_cast_bf16(om_ctx* ctx, const float* src, uint16_t* dst, int64_t n) {
  OM_CHECK_CTX(ctx);
  if (n < 0) return fail(ctx, OM_ERR_SHAPE, "om_cast_bf16: n %lld", (long long)n);
  if (n == 0) return OM_OK;
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
    return fail(ctx, OM_ERR_ARG, "om_cast_bf16: source and destination must be 16-byte aligned");
  ProfileScope prof(ctx, "om_cast_bf16", 0.0, 6.0 * (double)n);
  launch_chained(ctx, cast_bf16_kernel, grid_for(ctx, (n + 7) / 8, 256), 256, 0, src, dst, n);
  OM_LAUNCH_CHECK(ctx, "om_cast_bf16");
  return OM_OK;
}

int32_t om_matmul_bf16(om_ctx* ctx, int32_t transA, int32_t transB, int32_t m, int32_t n, int32_t k, const uint16_t* A, int32_t lda,
                       const uint16_t* B, int32_t ldb, float* C, int32_t ldc, int32_t accumulate) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check_args(ctx, "om_matmul_bf16", m, n, k, A, lda, B, ldb, C, ldc));
  if (m == 0 || n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_matmul", 2.0 * m * n * k, 2.0 * ((double)m * k + (double)k * n) + 4.0 * (double)m * n);
  return gemm_ws(ctx, 1, transA, transB, m, n, k, A, lda, B, ldb, C, ldc, accumulate, nullptr, nullptr);
}

int32_t om_linear_fwd_bf16_b16(om_ctx* ctx, const uint16_t* x, const uint16_t* W, const float* bias, int32_t rows, int32_t in_features,
                               int32_t out_features, float* y, uint16_t* y16, int32_t ldy) {
  OM_CHECK_CTX(ctx);
  if (y16 && (reinterpret_cast<uintptr_t>(y16) & 15)) return fail(ctx, OM_ERR_ARG, "om_linear_fwd_bf16_b16: the bfloat16 copy must be 16-byte aligned");
  if (rows < 0 || in_features < 1 || out_features < 1 || ldy < out_features)
    return fail(ctx, OM_ERR_SHAPE, "om_linear_fwd_bf16: rows %d in %d out %d ldy %d", rows, in_features, out_features, ldy);
  OM_TRY(check_args(ctx, "om_linear_fwd_bf16", rows, out_features, in_features, x, in_features, W, in_features, y, ldy));
  if (rows == 0) return OM_OK;
  ProfileScope prof(ctx, "om_linear_fwd", 2.0 * rows * in_features * out_features,
                    2.0 * ((double)rows * in_features + (double)in_features * out_features) + 4.0 * (double)rows * out_features);
  return gemm_ws(ctx, 1, 0, 1, rows, out_features, in_features, x, in_features, W, in_features, y, ldy, 0, bias, y16);
}

int32_t om_linear_fwd_bf16(om_ctx* ctx, const uint16_t* x, const uint16_t* W, const float* bias, int32_t rows, int32_t in_features,
                           int32_t out_features, float* y, int32_t ldy) {
  return om_linear_fwd_bf16_b16(ctx, x, W, bias, rows, in_features, out_features, y, nullptr, ldy);
}

int32_t om_linear_bwd_bf16_b16(om_ctx* ctx, const uint16_t* g16, const float* g, int32_t ldg, const uint16_t* x, const uint16_t* W, int32_t rows,
                               int32_t in_features, int32_t out_features, float* dx, uint16_t* dx16, float* dW, float* dbias,
                               int32_t accumulate_w) {
  OM_CHECK_CTX(ctx);
  if (dx16 && (!dx || (reinterpret_cast<uintptr_t>(dx16) & 15)))
    return fail(ctx, OM_ERR_ARG, "om_linear_bwd_bf16_b16: the bfloat16 copy needs dx and 16-byte alignment");
  if (rows < 0 || in_features < 1 || out_features < 1 || ldg < out_features)
    return fail(ctx, OM_ERR_SHAPE, "om_linear_bwd_bf16: rows %d in %d out %d ldg %d", rows, in_features, out_features, ldg);
  if (rows == 0) return OM_OK;
  const double flops = 2.0 * rows * in_features * out_features;
  auto products = [&]() -> int32_t {
    if (dx) {
      // dx[rows, in] = g[rows, out] * W[out, in]
      OM_TRY(check_args(ctx, "om_linear_bwd_bf16 (input gradient)", rows, in_features, out_features, g16, ldg, W, in_features, dx, in_features));
      ProfileScope prof(ctx, "om_linear_bwd.dgrad", flops, 2.0 * ((double)rows * out_features + (double)in_features * out_features) + 4.0 * (double)rows * in_features);
      OM_TRY(gemm_ws(ctx, 1, 0, 0, rows, in_features, out_features, g16, ldg, W, in_features, dx, in_features, (accumulate_w >> 1) & 1, nullptr, dx16));
    }
    if (dW) {
      // dW[out, in] = g[rows, out]^T * x[rows, in]
      OM_TRY(check_args(ctx, "om_linear_bwd_bf16 (weight gradient)", out_features, in_features, rows, g16, ldg, x, in_features, dW, in_features));
      ProfileScope prof(ctx, "om_linear_bwd.wgrad", flops, 2.0 * ((double)rows * out_features + (double)rows * in_features) + 4.0 * (double)in_features * out_features);
      OM_TRY(gemm_ws(ctx, 1, 1, 0, out_features, in_features, rows, g16, ldg, x, in_features, dW, in_features, accumulate_w & 1, nullptr, nullptr));
    }
    return OM_OK;
  };
  // The bias gradient g^T 1: from the fp32 gradient when the caller has one, else from the same bfloat16 copy that the weight
  // gradient g^T x reads (half the bytes, and the fp32 gradient need not exist at all).
  auto bias_sum = [&]() -> int32_t {
    if (!dbias) return OM_OK;
    if (g) return colsum_ld(ctx, g, rows, out_features, ldg, dbias, accumulate_w & 1);
    return colsum16_ld(ctx, g16, rows, out_features, ldg, dbias, accumulate_w & 1);
  };
  // With OM_TWO_STREAMS the column sum runs beside the products: they are bound by the tensor pipe and leave most of the
  // memory bandwidth idle, the sum is bound by memory alone, and a product's CTA leaves room on its SM for one of the sum's.
  // The products are launched first so that they hold their SMs when the sum's CTAs arrive.
  const bool fork = (ctx->flags & OM_TWO_STREAMS) && !ctx->profiling && !ctx->aux_active && dbias && (dx || dW) && rows >= 512;
  if (fork) return run_forked(ctx, products, bias_sum);
  OM_TRY(products());
  return bias_sum();
}

int32_t om_linear_bwd_bf16(om_ctx* ctx, const uint16_t* g16, const float* g, int32_t ldg, const uint16_t* x, const uint16_t* W, int32_t rows,
                           int32_t in_features, int32_t out_features, float* dx, float* dW, float* dbias, int32_t accumulate_w) {
  return om_linear_bwd_bf16_b16(ctx, g16, g, ldg, x, W, rows, in_features, out_features, dx, nullptr, dW, dbias, accumulate_w);
}

// ---- a Linear layer with the activation that follows it, and the input gradient of the layer after that activation ----

int32_t om_linear_act_bf16_supported(om_ctx* ctx, int32_t rows, int32_t in_features, int32_t out_features, int32_t op, int32_t backward) {
  if (!ctx) return 0;
  // Aligned stand-ins for the pointers: the query is about the shape (the calls check their own pointers).
  const float* aligned = reinterpret_cast<const float*>(uintptr_t(256));
  const uint16_t* aligned16 = reinterpret_cast<const uint16_t*>(uintptr_t(256));
  if (backward) {
    if (out_features % 8 || in_features % 8) return 0;
    return gemm_ws_act_ok(2, op, rows, in_features, out_features, aligned, in_features, aligned16, aligned, in_features) ? 1 : 0;
  }
  if (in_features % 8 || out_features % 8) return 0;
  return gemm_ws_act_ok(1, op, rows, out_features, in_features, aligned, out_features, aligned16, nullptr, 0) ? 1 : 0;
}

int32_t om_linear_fwd_bf16_act(om_ctx* ctx, const uint16_t* x, const uint16_t* W, const float* bias, int32_t rows, int32_t in_features,
                               int32_t out_features, int32_t op, float* y, uint16_t* a16, int32_t ldy) {
  OM_CHECK_CTX(ctx);
  if (rows < 1 || in_features < 1 || out_features < 1 || ldy < out_features)
    return fail(ctx, OM_ERR_SHAPE, "om_linear_fwd_bf16_act: rows %d in %d out %d ldy %d", rows, in_features, out_features, ldy);
  if (!y || !a16) return fail(ctx, OM_ERR_ARG, "om_linear_fwd_bf16_act: y and a16 are both written");
  OM_TRY(check_args(ctx, "om_linear_fwd_bf16_act", rows, out_features, in_features, x, in_features, W, in_features, y, ldy));
  ProfileScope prof(ctx, "om_linear_fwd", 2.0 * rows * in_features * out_features,
                    2.0 * ((double)rows * in_features + (double)in_features * out_features) + 6.0 * (double)rows * out_features);
  return gemm_ws_act(ctx, 1, 0, 1, rows, out_features, in_features, x, in_features, W, in_features, y, ldy, 0, bias, a16, 1, op, nullptr, 0);
}

int32_t om_linear_dgrad_bf16_act(om_ctx* ctx, const uint16_t* g16, int32_t ldg, const uint16_t* W, int32_t rows, int32_t in_features,
                                 int32_t out_features, int32_t op, const float* pre, int32_t ldpre, float* dx, uint16_t* dx16) {
  OM_CHECK_CTX(ctx);
  if (rows < 1 || in_features < 1 || out_features < 1 || ldg < out_features || ldpre < in_features)
    return fail(ctx, OM_ERR_SHAPE, "om_linear_dgrad_bf16_act: rows %d in %d out %d ldg %d ldpre %d", rows, in_features, out_features, ldg, ldpre);
  if ((!dx && !dx16) || !pre) return fail(ctx, OM_ERR_ARG, "om_linear_dgrad_bf16_act: a result (dx or dx16) and the activation's saved input are needed");
  OM_TRY(check_args(ctx, "om_linear_dgrad_bf16_act", rows, in_features, out_features, g16, ldg, W, in_features, dx, in_features));
  ProfileScope prof(ctx, "om_linear_bwd.dgrad", 2.0 * rows * in_features * out_features,
                    2.0 * ((double)rows * out_features + (double)in_features * out_features) + (4.0 + (dx ? 4.0 : 0.0) + (dx16 ? 2.0 : 0.0)) * (double)rows * in_features);
  return gemm_ws_act(ctx, 1, 0, 0, rows, in_features, out_features, g16, ldg, W, in_features, dx, in_features, 0, nullptr, dx16, 2, op, pre, ldpre);
}

// ---- the same pair with the activation's derivative left behind by the forward pass ----

int32_t om_linear_fwd_bf16_actd(om_ctx* ctx, const uint16_t* x, const uint16_t* W, const float* bias, int32_t rows, int32_t in_features,
                                int32_t out_features, int32_t op, uint16_t* deriv, uint16_t* a16, int32_t ldd) {
  OM_CHECK_CTX(ctx);
  if (rows < 1 || in_features < 1 || out_features < 1 || ldd < out_features)
    return fail(ctx, OM_ERR_SHAPE, "om_linear_fwd_bf16_actd: rows %d in %d out %d ldd %d", rows, in_features, out_features, ldd);
  if (!deriv || !a16) return fail(ctx, OM_ERR_ARG, "om_linear_fwd_bf16_actd: deriv and a16 are both written");
  OM_TRY(check_args(ctx, "om_linear_fwd_bf16_actd", rows, out_features, in_features, x, in_features, W, in_features, reinterpret_cast<const float*>(deriv), ldd));
  ProfileScope prof(ctx, "om_linear_fwd", 2.0 * rows * in_features * out_features,
                    2.0 * ((double)rows * in_features + (double)in_features * out_features) + 4.0 * (double)rows * out_features);
  return gemm_ws_act(ctx, 1, 0, 1, rows, out_features, in_features, x, in_features, W, in_features, reinterpret_cast<float*>(deriv), ldd, 0, bias, a16,
                     5, op, nullptr, 0);
}

int32_t om_linear_dgrad_bf16_mul(om_ctx* ctx, const uint16_t* g16, int32_t ldg, const uint16_t* W, int32_t rows, int32_t in_features,
                                 int32_t out_features, const uint16_t* factor, int32_t ldf, float* dx, uint16_t* dx16) {
  OM_CHECK_CTX(ctx);
  if (rows < 1 || in_features < 1 || out_features < 1 || ldg < out_features || ldf < in_features)
    return fail(ctx, OM_ERR_SHAPE, "om_linear_dgrad_bf16_mul: rows %d in %d out %d ldg %d ldf %d", rows, in_features, out_features, ldg, ldf);
  if ((!dx && !dx16) || !factor) return fail(ctx, OM_ERR_ARG, "om_linear_dgrad_bf16_mul: a result (dx or dx16) and the factor are needed");
  OM_TRY(check_args(ctx, "om_linear_dgrad_bf16_mul", rows, in_features, out_features, g16, ldg, W, in_features, dx, in_features));
  ProfileScope prof(ctx, "om_linear_bwd.dgrad", 2.0 * rows * in_features * out_features,
                    2.0 * ((double)rows * out_features + (double)in_features * out_features) + (2.0 + (dx ? 4.0 : 0.0) + (dx16 ? 2.0 : 0.0)) * (double)rows * in_features);
  return gemm_ws_act(ctx, 1, 0, 0, rows, in_features, out_features, g16, ldg, W, in_features, dx, in_features, 0, nullptr, dx16, 4, 0,
                     reinterpret_cast<const float*>(factor), ldf);
}

// ---- an input gradient that joins another branch's gradient: dx = residual + g W, out of place ----

int32_t om_linear_dgrad_bf16_add_supported(om_ctx* ctx, int32_t rows, int32_t in_features, int32_t out_features) {
  if (!ctx || in_features % 8 || out_features % 8) return 0;
  const float* aligned = reinterpret_cast<const float*>(uintptr_t(256));
  return gemm_ws_act_ok(3, 0, rows, in_features, out_features, aligned, in_features, nullptr, aligned, in_features) ? 1 : 0;
}

int32_t om_linear_dgrad_bf16_add(om_ctx* ctx, const uint16_t* g16, int32_t ldg, const uint16_t* W, int32_t rows, int32_t in_features,
                                 int32_t out_features, const float* residual, int32_t ldres, float* dx, uint16_t* dx16) {
  OM_CHECK_CTX(ctx);
  if (rows < 1 || in_features < 1 || out_features < 1 || ldg < out_features || ldres < in_features)
    return fail(ctx, OM_ERR_SHAPE, "om_linear_dgrad_bf16_add: rows %d in %d out %d ldg %d ldres %d", rows, in_features, out_features, ldg, ldres);
  if (!dx || !residual || dx == residual) return fail(ctx, OM_ERR_ARG, "om_linear_dgrad_bf16_add: dx and a distinct residual are needed");
  OM_TRY(check_args(ctx, "om_linear_dgrad_bf16_add", rows, in_features, out_features, g16, ldg, W, in_features, dx, in_features));
  ProfileScope prof(ctx, "om_linear_bwd.dgrad", 2.0 * rows * in_features * out_features,
                    2.0 * ((double)rows * out_features + (double)in_features * out_features) + (dx16 ? 10.0 : 8.0) * (double)rows * in_features);
  return gemm_ws_act(ctx, 1, 0, 0, rows, in_features, out_features, g16, ldg, W, in_features, dx, in_features, 0, nullptr, dx16, 3, 0, residual, ldres);
}

}  // extern "C"
