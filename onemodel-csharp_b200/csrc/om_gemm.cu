// Entry points of the dense products: pick the tensor-pipe kernel (tcgen05, om_gemm_tc.cu) when the context asks
// for TF32 or BF16 operands and the shape qualifies, else the fp32 FMA kernel (om_gemm_simt.cu). Both run on the
// GPU; there is no host path.
#include "om_common.cuh"

namespace om {

void splitk_reduce_launch(om_ctx* ctx, const float* part, int splits, int64_t mn, int n, int64_t ldc, const float* bias, float* out, int accumulate);
int32_t gemm_simt(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, int64_t sA,
                  const float* B, int ldb, int64_t sB, float* C, int ldc, int64_t sC, int batch, int acc);
bool gemm_tc_supported(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B,
                       int ldb, const float* C, int ldc);
int32_t gemm_tc(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B, int ldb,
                float* C, int ldc, int acc, const float* bias);
bool gemm_tc_batched_supported(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA,
                               const float* B, int ldb, long long sB, int batch);
int32_t gemm_tc_batched(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA, const float* B,
                        int ldb, long long sB, float* C, int ldc, long long sC, int batch, int acc, const float* bias);

__global__ void add_bias_rows_kernel(float* __restrict__ y, const float* __restrict__ bias, int64_t rows, int32_t cols, int64_t ld) {
  int64_t total = rows * cols;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (ld != cols) {
    for (int64_t j = i; j < total; j += stride) y[(j / cols) * ld + (j % cols)] += bias[j % cols];
  } else if ((cols & 3) == 0) {
    int64_t n4 = total >> 2;
    int32_t c4 = cols >> 2;
    float4* y4 = reinterpret_cast<float4*>(y);
    const float4* b4 = reinterpret_cast<const float4*>(bias);
    for (int64_t j = i; j < n4; j += stride) {
      float4 v = y4[j], b = b4[j % c4];
      v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
      y4[j] = v;
    }
  } else {
    for (int64_t j = i; j < total; j += stride) y[j] += bias[j % cols];
  }
}

static int32_t check_gemm_args(om_ctx* ctx, const char* who, int ta, int tb, int m, int n, int k, int lda, int ldb, int ldc) {
  if (m < 0 || n < 0 || k < 0) return fail(ctx, OM_ERR_SHAPE, "%s: m %d n %d k %d", who, m, n, k);
  int min_lda = ta ? m : k, min_ldb = tb ? k : n;
  if (lda < (min_lda > 1 ? min_lda : 1) || ldb < (min_ldb > 1 ? min_ldb : 1) || ldc < (n > 1 ? n : 1))
    return fail(ctx, OM_ERR_SHAPE, "%s: leading dimensions lda %d ldb %d ldc %d too small for m %d n %d k %d", who, lda, ldb, ldc, m, n, k);
  return OM_OK;
}

int32_t gemm_dispatch(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B,
                      int ldb, float* C, int ldc, int acc, const float* bias) {
  if (m == 0 || n == 0) return OM_OK;
  if ((ctx->flags & OM_TF32) && gemm_tc_supported(ctx, ta, tb, m, n, k, A, lda, B, ldb, C, ldc))
    return gemm_tc(ctx, ta, tb, m, n, k, A, lda, B, ldb, C, ldc, acc, bias);
  // A deep product with a small result that the tensor-pipe kernel cannot take (a pitch that is not a multiple of 16
  // bytes, e.g. the weight gradient of a 97-class output layer) would run as a handful of CTAs each walking all of k.
  // In the fast tier (where the one-accumulator order of the exact tier is not promised) k is cut into a fixed number
  // of equal slices computed as a batch and added in slice order.
  if ((ctx->flags & OM_TF32) && k >= 1024 && (int64_t)m * n <= 262144) {
    int slices = 0;
    for (int cand : {32, 16, 8, 4, 2})
      if (k % cand == 0 && k / cand >= 128) {
        slices = cand;
        break;
      }
    if (slices > 0) {
      const int ks = k / slices;
      float* part = nullptr;
      OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)slices * m * n, false, (void**)&part));
      int32_t st = gemm_simt(ctx, ta, tb, m, n, ks, A, lda, ta ? (long long)ks * lda : ks, B, ldb, tb ? ks : (long long)ks * ldb, part, n,
                             (long long)m * n, slices, 0);
      if (st == OM_OK) splitk_reduce_launch(ctx, part, slices, (int64_t)m * n, n, ldc, bias, C, acc);
      pool_free(ctx, part);
      return st;
    }
  }
  OM_TRY(gemm_simt(ctx, ta, tb, m, n, k, A, lda, 0, B, ldb, 0, C, ldc, 0, 1, acc));
  if (bias) {
    add_bias_rows_kernel<<<grid_for(ctx, ((int64_t)m * n + 3) / 4, 256), 256, 0, ctx->stream>>>(C, bias, m, n, ldc);
    OM_LAUNCH_CHECK(ctx, "add_bias_rows");
  }
  return OM_OK;
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_colsum(om_ctx* ctx, const float* g, int32_t rows, int32_t cols, float* out, int32_t accumulate);
}
namespace om {
int32_t colsum_ld(om_ctx* ctx, const float* g, int32_t rows, int32_t cols, int64_t ld, float* out, int32_t accumulate);
}
extern "C" {

int32_t om_matmul(om_ctx* ctx, int32_t transA, int32_t transB, int32_t m, int32_t n, int32_t k, const float* A,
                  int32_t lda, const float* B, int32_t ldb, float* C, int32_t ldc, int32_t accumulate) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check_gemm_args(ctx, "om_matmul", transA, transB, m, n, k, lda, ldb, ldc));
  ProfileScope prof(ctx, "om_matmul", 2.0 * m * n * k, 4.0 * ((double)m * k + (double)k * n + (double)m * n));
  return gemm_dispatch(ctx, transA, transB, m, n, k, A, lda, B, ldb, C, ldc, accumulate, nullptr);
}

int32_t om_matmul_batched(om_ctx* ctx, int32_t transA, int32_t transB, int32_t m, int32_t n, int32_t k,
                          const float* A, int32_t lda, int64_t strideA, const float* B, int32_t ldb, int64_t strideB,
                          float* C, int32_t ldc, int64_t strideC, int32_t batch, int32_t accumulate) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check_gemm_args(ctx, "om_matmul_batched", transA, transB, m, n, k, lda, ldb, ldc));
  if (batch < 0 || batch > 65535) return fail(ctx, OM_ERR_SHAPE, "om_matmul_batched: batch %d", batch);
  ProfileScope prof(ctx, "om_matmul_batched", 2.0 * m * n * k * batch,
                    4.0 * batch * ((double)m * k + (double)k * n + (double)m * n));
  if (batch > 1 && (ldc & 3) == 0 && (strideC & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
      gemm_tc_batched_supported(ctx, transA, transB, m, n, k, A, lda, strideA, B, ldb, strideB, batch))
    return gemm_tc_batched(ctx, transA, transB, m, n, k, A, lda, strideA, B, ldb, strideB, C, ldc, strideC, batch, accumulate, nullptr);
  return gemm_simt(ctx, transA, transB, m, n, k, A, lda, strideA, B, ldb, strideB, C, ldc, strideC, batch, accumulate);
}

int32_t om_linear_fwd_ld(om_ctx* ctx, const float* x, const float* W, const float* bias, int32_t rows, int32_t in_features,
                         int32_t out_features, float* y, int32_t ldy) {
  OM_CHECK_CTX(ctx);
  if (rows < 0 || in_features < 1 || out_features < 1 || ldy < out_features)
    return fail(ctx, OM_ERR_SHAPE, "om_linear_fwd: rows %d in %d out %d ldy %d", rows, in_features, out_features, ldy);
  ProfileScope prof(ctx, "om_linear_fwd", 2.0 * rows * in_features * out_features,
                    4.0 * ((double)rows * in_features + (double)in_features * out_features + (double)rows * out_features));
  return gemm_dispatch(ctx, 0, 1, rows, out_features, in_features, x, in_features, W, in_features, y, ldy, 0, bias);
}

int32_t om_linear_fwd(om_ctx* ctx, const float* x, const float* W, const float* bias, int32_t rows, int32_t in_features,
                      int32_t out_features, float* y) {
  return om_linear_fwd_ld(ctx, x, W, bias, rows, in_features, out_features, y, out_features);
}

int32_t om_linear_bwd_ld(om_ctx* ctx, const float* g, int32_t ldg, const float* x, const float* W, int32_t rows,
                         int32_t in_features, int32_t out_features, float* dx, float* dW, float* dbias, int32_t accumulate_w) {
  OM_CHECK_CTX(ctx);
  if (rows < 0 || in_features < 1 || out_features < 1 || ldg < out_features)
    return fail(ctx, OM_ERR_SHAPE, "om_linear_bwd: rows %d in %d out %d ldg %d", rows, in_features, out_features, ldg);
  const double flops = 2.0 * rows * in_features * out_features;
  const double bytes = 4.0 * ((double)rows * in_features + (double)in_features * out_features + (double)rows * out_features);
  auto input_side = [&]() -> int32_t {
    if (!dx) return OM_OK;
    ProfileScope prof(ctx, "om_linear_bwd.dgrad", flops, bytes);
    // dx[rows, in] = g[rows, out] * W[out, in]
    return gemm_dispatch(ctx, 0, 0, rows, in_features, out_features, g, ldg, W, in_features, dx, in_features, (accumulate_w >> 1) & 1, nullptr);
  };
  auto parameter_side = [&]() -> int32_t {
    if (dW) {
      ProfileScope prof(ctx, "om_linear_bwd.wgrad", flops, bytes);
      // dW[out, in] = g[rows, out]^T * x[rows, in]
      OM_TRY(gemm_dispatch(ctx, 1, 0, out_features, in_features, rows, g, ldg, x, in_features, dW, in_features, accumulate_w & 1, nullptr));
    }
    if (dbias) OM_TRY(colsum_ld(ctx, g, rows, out_features, ldg, dbias, accumulate_w & 1));
    return OM_OK;
  };
  // The two sides share only inputs. With OM_TWO_STREAMS they overlap (not while per-entry times are being taken,
  // which need one stream, and not for products so small that the fork and join cost more than they hide).
  const bool fork = (ctx->flags & OM_TWO_STREAMS) && !ctx->profiling && !ctx->aux_active && dx && (dW || dbias) && rows >= 512;
  if (fork) return run_forked(ctx, input_side, parameter_side);
  OM_TRY(input_side());
  return parameter_side();
}

int32_t om_linear_bwd(om_ctx* ctx, const float* g, const float* x, const float* W, int32_t rows, int32_t in_features,
                      int32_t out_features, float* dx, float* dW, float* dbias, int32_t accumulate_w) {
  return om_linear_bwd_ld(ctx, g, out_features, x, W, rows, in_features, out_features, dx, dW, dbias, accumulate_w);
}

}  // extern "C"
