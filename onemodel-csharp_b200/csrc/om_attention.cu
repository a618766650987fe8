// Scaled dot-product attention, forward and backward, per (batch, head).
//
// Data flow of the backward, as AttentionBackward in the reference (BackwardNn.cs:636-701): recompute
// S = Q K^T, P = softmax(scale S + mask); dV = P^T dO; dP = dO V^T; dS = P (dP - rowsum(dP P)) scale;
// dQ = dS K; dK = dS^T Q. The [B*H, Lq, Lk] score and probability matrices live in pooled scratch for the duration
// of the call; every product is a strided-batched fp32 GEMM over all heads at once and the row operations are one
// fused kernel each (scale + mask + softmax, and the dS row transform with its double-precision row dot).
#include "om_common.cuh"

namespace om {

int32_t gemm_simt_heads(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, int64_t sA, int64_t iA,
                        const float* B, int ldb, int64_t sB, int64_t iB, float* C, int ldc, int64_t sC, int64_t iC, int batch,
                        int inner, int acc);
bool gemm_tc_heads_supported(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA, long long iA,
                             const float* B, int ldb, long long sB, long long iB, int batch, int inner);
int32_t gemm_tc_heads(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA, long long iA,
                      const float* B, int ldb, long long sB, long long iB, float* C, int ldc, long long sC, long long iC, int batch,
                      int inner, int acc, const float* bias);

bool attention_tc_fwd_supported(om_ctx* ctx, const float* q, const om_head_strides* qs, const float* k, const om_head_strides* ks,
                                const float* v, const om_head_strides* vs, const float* out, const om_head_strides* os, int b, int h,
                                int lq, int lk, int d);
bool attention_bwd_front_supported(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q, const om_head_strides* qs,
                                   const float* k, const om_head_strides* ks, const float* v, const om_head_strides* vs, const float* lse,
                                   int b, int h, int lq, int lk, int d);
int32_t attention_bwd_front(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q, const om_head_strides* qs, const float* k,
                            const om_head_strides* ks, const float* v, const om_head_strides* vs, const float* o, const om_head_strides* os,
                            const float* mask, long long mask_batch_stride, const float* lse, int b, int h, int lq, int lk, int d, float scale,
                            float* p_out, float* ds_out);
int32_t attention_tc_fwd(om_ctx* ctx, const float* q, const om_head_strides* qs, const float* k, const om_head_strides* ks, const float* v,
                         const om_head_strides* vs, const float* mask, long long mask_batch_stride, int b, int h, int lq, int lk, int d,
                         float scale, float* out, const om_head_strides* os, float* lse);

bool attention_tc_bwd_supported(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q, const om_head_strides* qs,
                                const float* k, const om_head_strides* ks, const float* v, const om_head_strides* vs, const float* lse,
                                int b, int h, int lq, int lk, int d, const float* dq, const om_head_strides* dqs, const float* dk,
                                const om_head_strides* dks, const float* dv, const om_head_strides* dvs);
int32_t attention_tc_bwd(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q, const om_head_strides* qs, const float* k,
                         const om_head_strides* ks, const float* v, const om_head_strides* vs, const float* mask, long long mask_batch_stride,
                         const float* lse, int b, int h, int lq, int lk, float scale, float* dq, const om_head_strides* dqs, float* dk,
                         const om_head_strides* dks, float* dv, const om_head_strides* dvs);

// Where the [l, d] matrix of (batch b, head h) of an activation starts and how its rows are spaced: element strides.
struct HeadView {
  const float* p;
  int64_t batch, head, row;
};

// One product per (batch, head): on the tensor pipe (TF32) when the context asks for it and the strides allow TMA,
// else on the fp32 FMA kernel.
static int32_t head_gemm(om_ctx* ctx, int ta, int tb, int m, int n, int k, HeadView A, HeadView B, float* C, HeadView Cv, int bh,
                         int heads) {
  if (bh > 1 && (Cv.row & 3) == 0 && (Cv.batch & 3) == 0 && (Cv.head & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
      A.row <= INT32_MAX && B.row <= INT32_MAX &&
      gemm_tc_heads_supported(ctx, ta, tb, m, n, k, A.p, (int)A.row, A.batch, A.head, B.p, (int)B.row, B.batch, B.head, bh, heads))
    return gemm_tc_heads(ctx, ta, tb, m, n, k, A.p, (int)A.row, A.batch, A.head, B.p, (int)B.row, B.batch, B.head, C, (int)Cv.row,
                         Cv.batch, Cv.head, bh, heads, 0, nullptr);
  return gemm_simt_heads(ctx, ta, tb, m, n, k, A.p, (int)A.row, A.batch, A.head, B.p, (int)B.row, B.batch, B.head, C, (int)Cv.row,
                         Cv.batch, Cv.head, bh, heads, 0);
}

static HeadView view_of(const float* p, const om_head_strides* s) { return HeadView{p, s->batch, s->head, s->row}; }
static HeadView scores_view(const float* p, int heads, int lq, int lk) {
  return HeadView{p, (int64_t)heads * lq * lk, (int64_t)lq * lk, (int64_t)lk};
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
// NP > 0: the row (lk <= 32 * NP) stays in registers between the three sweeps - one read and one write of the scores.
// NP == 0: any length, the sweeps go through memory. Same arithmetic and summation order in both.
template <int NP>
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
    if (NP > 0) {
      float v[NP > 0 ? NP : 1];
      float mx = -INFINITY;
#pragma unroll
      for (int u = 0; u < NP; u++) {
        int j = lane + 32 * u;
        v[u] = j < lk ? (sr[j] * scale) + (mr ? mr[j] : 0.f) : -INFINITY;
        mx = fmaxf(mx, v[u]);
      }
      mx = att_wmax_f(mx);
      // A fully masked row (all -inf) gives exp(nan); keep the reference's behaviour of propagating it.
      double sum = 0.0;
#pragma unroll
      for (int u = 0; u < NP; u++) {
        if (lane + 32 * u < lk) {
          v[u] = expf(v[u] - mx);
          sum += (double)v[u];
        }
      }
      float fs = (float)att_wsum_d(sum);
#pragma unroll
      for (int u = 0; u < NP; u++)
        if (lane + 32 * u < lk) sr[lane + 32 * u] = v[u] / fs;
      if (lse && lane == 0) lse[r] = mx + logf(fs);
    } else {
      float mx = -INFINITY;
      for (int j = lane; j < lk; j += 32) {
        float v = (sr[j] * scale) + (mr ? mr[j] : 0.f);
        sr[j] = v;
        mx = fmaxf(mx, v);
      }
      mx = att_wmax_f(mx);
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
}

// In place over dp: ds = p * (dp - dot) * scale with dot = sum_j dp*p in double. NP as above.
template <int NP>
__global__ void __launch_bounds__(256)
att_ds_kernel(float* __restrict__ dp, const float* __restrict__ p, int32_t lk, int64_t rows, float scale) {
  int lane = threadIdx.x & 31;
  int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t r = warp; r < rows; r += warps) {
    float* d = dp + r * lk;
    const float* pr = p + r * lk;
    if (NP > 0) {
      float dv[NP > 0 ? NP : 1], pv[NP > 0 ? NP : 1];
      double dot = 0.0;
#pragma unroll
      for (int u = 0; u < NP; u++) {
        int j = lane + 32 * u;
        if (j < lk) {
          dv[u] = d[j];
          pv[u] = pr[j];
          dot += (double)(dv[u] * pv[u]);
        }
      }
      float df = (float)att_wsum_d(dot);
#pragma unroll
      for (int u = 0; u < NP; u++)
        if (lane + 32 * u < lk) d[lane + 32 * u] = (pv[u] * (dv[u] - df)) * scale;
    } else {
      double dot = 0.0;
      for (int j = lane; j < lk; j += 32) dot += (double)(d[j] * pr[j]);
      float df = (float)att_wsum_d(dot);
      for (int j = lane; j < lk; j += 32) d[j] = (pr[j] * (d[j] - df)) * scale;
    }
  }
}

static void launch_att_softmax(om_ctx* ctx, int grid, float* s, const float* mask, int64_t mbs, int h, int lq, int lk, int64_t rows,
                               float scale, float* lse) {
  if (lk <= 128) att_softmax_kernel<4><<<grid, 256, 0, ctx->stream>>>(s, mask, mbs, h, lq, lk, rows, scale, lse);
  else if (lk <= 512) att_softmax_kernel<16><<<grid, 256, 0, ctx->stream>>>(s, mask, mbs, h, lq, lk, rows, scale, lse);
  else att_softmax_kernel<0><<<grid, 256, 0, ctx->stream>>>(s, mask, mbs, h, lq, lk, rows, scale, lse);
}
static void launch_att_ds(om_ctx* ctx, int grid, float* dp, const float* p, int lk, int64_t rows, float scale) {
  if (lk <= 128) att_ds_kernel<4><<<grid, 256, 0, ctx->stream>>>(dp, p, lk, rows, scale);
  else if (lk <= 512) att_ds_kernel<16><<<grid, 256, 0, ctx->stream>>>(dp, p, lk, rows, scale);
  else att_ds_kernel<0><<<grid, 256, 0, ctx->stream>>>(dp, p, lk, rows, scale);
}

static int32_t check_att(om_ctx* ctx, const char* who, int b, int h, int lq, int lk, int d) {
  if (b < 0 || h < 0 || lq < 0 || lk < 0 || d < 0 || (d & 1))
    return fail(ctx, OM_ERR_SHAPE, "%s needs [B,H,L,D] tensors with matching batch, heads and even D (B %d H %d Lq %d Lk %d D %d)", who, b, h, lq, lk, d);
  if ((int64_t)b * h > 65535) return fail(ctx, OM_ERR_UNSUPPORTED, "%s: more than 65535 heads in one call", who);
  return OM_OK;
}

static int32_t check_strides(om_ctx* ctx, const char* who, const om_head_strides* s, int d) {
  if (s == nullptr || s->row < d || s->batch < 0 || s->head < 0 || s->row > INT32_MAX)
    return fail(ctx, OM_ERR_SHAPE, "%s: rows of an activation must be at least D = %d elements apart and strides non-negative", who, d);
  return OM_OK;
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_attention_fwd_strided(om_ctx* ctx, const float* q, const om_head_strides* qs, const float* k, const om_head_strides* ks,
                                 const float* v, const om_head_strides* vs, const float* mask, int64_t mask_batch_stride, int32_t b,
                                 int32_t h, int32_t lq, int32_t lk, int32_t d, float scale, float* out, const om_head_strides* os,
                                 float* lse) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check_att(ctx, "Attention", b, h, lq, lk, d));
  OM_TRY(check_strides(ctx, "Attention", qs, d));
  OM_TRY(check_strides(ctx, "Attention", ks, d));
  OM_TRY(check_strides(ctx, "Attention", vs, d));
  OM_TRY(check_strides(ctx, "Attention", os, d));
  int bh = b * h;
  if (bh == 0 || lq == 0) return OM_OK;
  if (lk == 0) return fail(ctx, OM_ERR_SHAPE, "Attention: no keys");
  ProfileScope prof(ctx, "om_attention_fwd", 4.0 * bh * (double)lq * lk * d, 4.0 * bh * ((double)lq * d * 2 + (double)lk * d * 2));
  // Sequences that fit one tile run as one fused tensor-pipe kernel per (batch, head); the scores stay in tensor memory.
  if (attention_tc_fwd_supported(ctx, q, qs, k, ks, v, vs, out, os, b, h, lq, lk, d))
    return attention_tc_fwd(ctx, q, qs, k, ks, v, vs, mask, mask_batch_stride, b, h, lq, lk, d, scale, out, os, lse);
  float* s = nullptr;
  int64_t rows = (int64_t)bh * lq;
  OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)rows * lk, false, (void**)&s));
  const HeadView Q = view_of(q, qs), K = view_of(k, ks), V = view_of(v, vs), O = view_of(out, os), S = scores_view(s, h, lq, lk);
  int32_t st = head_gemm(ctx, 0, 1, lq, lk, d, Q, K, s, S, bh, h);
  if (st == OM_OK) {
    int grid = (int)std::min<int64_t>(ceil_div(rows, 8), (int64_t)ctx->sm_count * 16);
    launch_att_softmax(ctx, grid, s, mask, mask_batch_stride, h, lq, lk, rows, scale, lse);
    st = head_gemm(ctx, 0, 0, lq, d, lk, S, V, out, O, bh, h);
  }
  pool_free(ctx, s);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_attention_fwd");
  return OM_OK;
}

int32_t om_attention_fwd(om_ctx* ctx, const float* q, const float* k, const float* v, const float* mask,
                         int64_t mask_batch_stride, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d, float scale,
                         float* out, float* lse) {
  const om_head_strides sq = {(int64_t)h * lq * d, (int64_t)lq * d, d}, sk = {(int64_t)h * lk * d, (int64_t)lk * d, d};
  return om_attention_fwd_strided(ctx, q, &sq, k, &sk, v, &sk, mask, mask_batch_stride, b, h, lq, lk, d, scale, out, &sq, lse);
}

int32_t om_attention_bwd_strided_out(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q, const om_head_strides* qs,
                                     const float* k, const om_head_strides* ks, const float* v, const om_head_strides* vs,
                                     const float* out, const om_head_strides* os, const float* mask, int64_t mask_batch_stride,
                                     const float* lse, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d, float scale, float* dq,
                                     const om_head_strides* dqs, float* dk, const om_head_strides* dks, float* dv,
                                     const om_head_strides* dvs) {
  OM_CHECK_CTX(ctx);
  if (out) OM_TRY(check_strides(ctx, "Attention backward", os, d));
  OM_TRY(check_att(ctx, "Attention backward", b, h, lq, lk, d));
  OM_TRY(check_strides(ctx, "Attention backward", gs, d));
  OM_TRY(check_strides(ctx, "Attention backward", qs, d));
  OM_TRY(check_strides(ctx, "Attention backward", ks, d));
  OM_TRY(check_strides(ctx, "Attention backward", vs, d));
  if (dq) OM_TRY(check_strides(ctx, "Attention backward", dqs, d));
  if (dk) OM_TRY(check_strides(ctx, "Attention backward", dks, d));
  if (dv) OM_TRY(check_strides(ctx, "Attention backward", dvs, d));
  int bh = b * h;
  if (bh == 0 || lq == 0 || lk == 0) return OM_OK;
  ProfileScope prof(ctx, "om_attention_bwd", 8.0 * bh * (double)lq * lk * d, 4.0 * bh * ((double)lq * d * 4 + (double)lk * d * 4));
  // One-tile sequences with the forward's log-sum-exp at hand: one fused tensor-pipe kernel per (batch, head).
  if (attention_tc_bwd_supported(ctx, g, gs, q, qs, k, ks, v, vs, lse, b, h, lq, lk, d, dq, dqs, dk, dks, dv, dvs))
    return attention_tc_bwd(ctx, g, gs, q, qs, k, ks, v, vs, mask, mask_batch_stride, lse, b, h, lq, lk, scale, dq, dqs, dk, dks, dv, dvs);
  int64_t rows = (int64_t)bh * lq;
  float *p = nullptr, *dp = nullptr;
  OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)rows * lk, false, (void**)&p));
  int32_t st = pool_alloc(ctx, sizeof(float) * (size_t)rows * lk, false, (void**)&dp);
  if (st != OM_OK) {
    pool_free(ctx, p);
    return st;
  }
  const HeadView G = view_of(g, gs), Q = view_of(q, qs), K = view_of(k, ks), V = view_of(v, vs);
  const HeadView P = scores_view(p, h, lq, lk), DP = scores_view(dp, h, lq, lk);
  int grid = (int)std::min<int64_t>(ceil_div(rows, 8), (int64_t)ctx->sm_count * 16);
  if (attention_bwd_front_supported(ctx, g, gs, q, qs, k, ks, v, vs, lse, b, h, lq, lk, d)) {
    // P and dS from one tensor-pipe kernel per 128 queries (the forward's log-sum-exp makes P a single pass), then the three
    // output products.
    st = attention_bwd_front(ctx, g, gs, q, qs, k, ks, v, vs, out, os, mask, mask_batch_stride, lse, b, h, lq, lk, d, scale, p, dp);
    if (st == OM_OK && dv) st = head_gemm(ctx, 1, 0, lk, d, lq, P, G, dv, view_of(dv, dvs), bh, h);
    if (st == OM_OK && dq) st = head_gemm(ctx, 0, 0, lq, d, lk, DP, K, dq, view_of(dq, dqs), bh, h);
    if (st == OM_OK && dk) st = head_gemm(ctx, 1, 0, lk, d, lq, DP, Q, dk, view_of(dk, dks), bh, h);
    pool_free(ctx, p);
    pool_free(ctx, dp);
    OM_TRY(st);
    OM_LAUNCH_CHECK(ctx, "om_attention_bwd");
    return OM_OK;
  }
  st = head_gemm(ctx, 0, 1, lq, lk, d, Q, K, p, P, bh, h);
  if (st == OM_OK) {
    launch_att_softmax(ctx, grid, p, mask, mask_batch_stride, h, lq, lk, rows, scale, nullptr);
    // dV = P^T dO
    if (dv) st = head_gemm(ctx, 1, 0, lk, d, lq, P, G, dv, view_of(dv, dvs), bh, h);
  }
  if (st == OM_OK && (dq || dk)) {
    // dP = dO V^T, then dS in place
    st = head_gemm(ctx, 0, 1, lq, lk, d, G, V, dp, DP, bh, h);
    if (st == OM_OK) {
      launch_att_ds(ctx, grid, dp, p, lk, rows, scale);
      if (dq) st = head_gemm(ctx, 0, 0, lq, d, lk, DP, K, dq, view_of(dq, dqs), bh, h);
      if (st == OM_OK && dk) st = head_gemm(ctx, 1, 0, lk, d, lq, DP, Q, dk, view_of(dk, dks), bh, h);
    }
  }
  pool_free(ctx, p);
  pool_free(ctx, dp);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_attention_bwd");
  return OM_OK;
}

int32_t om_attention_bwd_strided(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q, const om_head_strides* qs,
                                 const float* k, const om_head_strides* ks, const float* v, const om_head_strides* vs,
                                 const float* mask, int64_t mask_batch_stride, const float* lse, int32_t b, int32_t h, int32_t lq,
                                 int32_t lk, int32_t d, float scale, float* dq, const om_head_strides* dqs, float* dk,
                                 const om_head_strides* dks, float* dv, const om_head_strides* dvs) {
  return om_attention_bwd_strided_out(ctx, g, gs, q, qs, k, ks, v, vs, nullptr, nullptr, mask, mask_batch_stride, lse, b, h, lq, lk, d, scale,
                                      dq, dqs, dk, dks, dv, dvs);
}

int32_t om_attention_bwd(om_ctx* ctx, const float* g, const float* q, const float* k, const float* v, const float* mask,
                         int64_t mask_batch_stride, const float* lse, int32_t b, int32_t h, int32_t lq, int32_t lk,
                         int32_t d, float scale, float* dq, float* dk, float* dv) {
  const om_head_strides sq = {(int64_t)h * lq * d, (int64_t)lq * d, d}, sk = {(int64_t)h * lk * d, (int64_t)lk * d, d};
  return om_attention_bwd_strided(ctx, g, &sq, q, &sq, k, &sk, v, &sk, mask, mask_batch_stride, lse, b, h, lq, lk, d, scale, dq, &sq,
                                  dk, &sk, dv, &sk);
}

}  // extern "C"
