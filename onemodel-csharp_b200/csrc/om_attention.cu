// Scaled dot-product attention, forward and backward, per (batch, head).
//
// Data flow of the backward, as AttentionBackward in the reference (BackwardNn.cs:636-701): recompute
// S = Q K^T, P = softmax(scale S + mask); dV = P^T dO; dP = dO V^T; dS = P (dP - rowsum(dP P)) scale;
// dQ = dS K; dK = dS^T Q. The [B*H, Lq, Lk] score and probability matrices live in pooled scratch for the duration
// of the call; every product is a strided-batched fp32 GEMM over all heads at once and the row operations are one
// fused kernel each (scale + mask + softmax, and the dS row transform with its double-precision row dot).
#include "om_common.cuh"

namespace om {

int32_t gemm_simt(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, int64_t sA,
                  const float* B, int ldb, int64_t sB, float* C, int ldc, int64_t sC, int batch, int acc);
bool gemm_tc_batched_supported(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA,
                               const float* B, int ldb, long long sB, int batch);
int32_t gemm_tc_batched(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA, const float* B,
                        int ldb, long long sB, float* C, int ldc, long long sC, int batch, int acc, const float* bias);

// One product per (batch, head): on the tensor pipe (TF32) when the context asks for it and the strides allow TMA,
// else on the fp32 FMA kernel.
static int32_t head_gemm(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, int64_t sA, const float* B,
                         int ldb, int64_t sB, float* C, int ldc, int64_t sC, int batch) {
  if (batch > 1 && (ldc & 3) == 0 && (sC & 3) == 0 && gemm_tc_batched_supported(ctx, ta, tb, m, n, k, A, lda, sA, B, ldb, sB, batch))
    return gemm_tc_batched(ctx, ta, tb, m, n, k, A, lda, sA, B, ldb, sB, C, ldc, sC, batch, 0, nullptr);
  return gemm_simt(ctx, ta, tb, m, n, k, A, lda, sA, B, ldb, sB, C, ldc, sC, batch, 0);
}

__device__ __forceinline__ double att_wsum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float att_wmax_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// In place over s [BH*Lq, Lk]: p = softmax(s*scale + mask). One warp per row. lse (may be NULL) gets max + log(sum).
__global__ void __launch_bounds__(256)
att_softmax_kernel(float* __restrict__ s, const float* __restrict__ mask, int64_t mask_batch_stride, int32_t heads,
                   int32_t lq, int32_t lk, int64_t rows, float scale, float* __restrict__ lse) {
  int lane = threadIdx.x & 31;
  int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t r = warp; r < rows; r += warps) {
    float* sr = s + r * lk;
    const float* mr = nullptr;
    if (mask) {
      int64_t i = r % lq;
      int64_t b = r / ((int64_t)lq * heads);
      mr = mask + b * mask_batch_stride + i * lk;
    }
    float mx = -INFINITY;
    for (int j = lane; j < lk; j += 32) {
      float v = (sr[j] * scale) + (mr ? mr[j] : 0.f);
      sr[j] = v;
      mx = fmaxf(mx, v);
    }
    mx = att_wmax_f(mx);
    // A fully masked row (all -inf) gives exp(nan); keep the reference's behaviour of propagating it.
    double sum = 0.0;
    for (int j = lane; j < lk; j += 32) {
      float e = expf(sr[j] - mx);
      sr[j] = e;
      sum += (double)e;
    }
    float fs = (float)att_wsum_d(sum);
    for (int j = lane; j < lk; j += 32) sr[j] = sr[j] / fs;
    if (lse && lane == 0) lse[r] = mx + logf(fs);
  }
}

// In place over dp: ds = p * (dp - dot) * scale with dot = sum_j dp*p in double.
__global__ void __launch_bounds__(256)
att_ds_kernel(float* __restrict__ dp, const float* __restrict__ p, int32_t lk, int64_t rows, float scale) {
  int lane = threadIdx.x & 31;
  int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t r = warp; r < rows; r += warps) {
    float* d = dp + r * lk;
    const float* pr = p + r * lk;
    double dot = 0.0;
    for (int j = lane; j < lk; j += 32) dot += (double)(d[j] * pr[j]);
    float df = (float)att_wsum_d(dot);
    for (int j = lane; j < lk; j += 32) d[j] = (pr[j] * (d[j] - df)) * scale;
  }
}

static int32_t check_att(om_ctx* ctx, const char* who, int b, int h, int lq, int lk, int d) {
  if (b < 0 || h < 0 || lq < 0 || lk < 0 || d < 0 || (d & 1))
    return fail(ctx, OM_ERR_SHAPE, "%s needs [B,H,L,D] tensors with matching batch, heads and even D (B %d H %d Lq %d Lk %d D %d)", who, b, h, lq, lk, d);
  if ((int64_t)b * h > 65535) return fail(ctx, OM_ERR_UNSUPPORTED, "%s: more than 65535 heads in one call", who);
  return OM_OK;
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_attention_fwd(om_ctx* ctx, const float* q, const float* k, const float* v, const float* mask,
                         int64_t mask_batch_stride, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d, float scale,
                         float* out, float* lse) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check_att(ctx, "Attention", b, h, lq, lk, d));
  int bh = b * h;
  if (bh == 0 || lq == 0) return OM_OK;
  if (lk == 0) return fail(ctx, OM_ERR_SHAPE, "Attention: no keys");
  ProfileScope prof(ctx, "om_attention_fwd", 4.0 * bh * (double)lq * lk * d, 4.0 * bh * ((double)lq * d * 2 + (double)lk * d * 2));
  float* s = nullptr;
  int64_t rows = (int64_t)bh * lq;
  OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)rows * lk, false, (void**)&s));
  int32_t st = head_gemm(ctx, 0, 1, lq, lk, d, q, d, (int64_t)lq * d, k, d, (int64_t)lk * d, s, lk, (int64_t)lq * lk, bh);
  if (st == OM_OK) {
    int grid = (int)std::min<int64_t>(ceil_div(rows, 8), (int64_t)ctx->sm_count * 16);
    att_softmax_kernel<<<grid, 256, 0, ctx->stream>>>(s, mask, mask_batch_stride, h, lq, lk, rows, scale, lse);
    st = head_gemm(ctx, 0, 0, lq, d, lk, s, lk, (int64_t)lq * lk, v, d, (int64_t)lk * d, out, d, (int64_t)lq * d, bh);
  }
  pool_free(ctx, s);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_attention_fwd");
  return OM_OK;
}

int32_t om_attention_bwd(om_ctx* ctx, const float* g, const float* q, const float* k, const float* v, const float* mask,
                         int64_t mask_batch_stride, const float* lse, int32_t b, int32_t h, int32_t lq, int32_t lk,
                         int32_t d, float scale, float* dq, float* dk, float* dv) {
  OM_CHECK_CTX(ctx);
  (void)lse;
  OM_TRY(check_att(ctx, "Attention backward", b, h, lq, lk, d));
  int bh = b * h;
  if (bh == 0 || lq == 0 || lk == 0) return OM_OK;
  ProfileScope prof(ctx, "om_attention_bwd", 8.0 * bh * (double)lq * lk * d, 4.0 * bh * ((double)lq * d * 4 + (double)lk * d * 4));
  int64_t rows = (int64_t)bh * lq;
  float *p = nullptr, *dp = nullptr;
  OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)rows * lk, false, (void**)&p));
  int32_t st = pool_alloc(ctx, sizeof(float) * (size_t)rows * lk, false, (void**)&dp);
  if (st != OM_OK) {
    pool_free(ctx, p);
    return st;
  }
  const int64_t sq = (int64_t)lq * d, sk = (int64_t)lk * d, ss = (int64_t)lq * lk;
  int grid = (int)std::min<int64_t>(ceil_div(rows, 8), (int64_t)ctx->sm_count * 16);
  st = head_gemm(ctx, 0, 1, lq, lk, d, q, d, sq, k, d, sk, p, lk, ss, bh);
  if (st == OM_OK) {
    att_softmax_kernel<<<grid, 256, 0, ctx->stream>>>(p, mask, mask_batch_stride, h, lq, lk, rows, scale, nullptr);
    // dV = P^T dO
    if (dv) st = head_gemm(ctx, 1, 0, lk, d, lq, p, lk, ss, g, d, sq, dv, d, sk, bh);
  }
  if (st == OM_OK && (dq || dk)) {
    // dP = dO V^T, then dS in place
    st = head_gemm(ctx, 0, 1, lq, lk, d, g, d, sq, v, d, sk, dp, lk, ss, bh);
    if (st == OM_OK) {
      att_ds_kernel<<<grid, 256, 0, ctx->stream>>>(dp, p, lk, rows, scale);
      if (dq) st = head_gemm(ctx, 0, 0, lq, d, lk, dp, lk, ss, k, d, sk, dq, d, sq, bh);
      if (st == OM_OK && dk) st = head_gemm(ctx, 1, 0, lk, d, lq, dp, lk, ss, q, d, sq, dk, d, sk, bh);
    }
  }
  pool_free(ctx, p);
  pool_free(ctx, dp);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_attention_bwd");
  return OM_OK;
}

}  // extern "C"
