/*
 * TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT.
 * CPU restatement, in plain C, of the reference's training hot path (RecursiveAI.OneModel, C#), used only as the
 * checker in tests/, in __graft_entry__.smoke() and as the timed CPU baseline of bench.py. Nothing under the
 * package directory may link or call this file.
 *
 * Every function names the reference code it follows (paths relative to the reference repository). Loop orders,
 * accumulator types (double where the reference uses double) and operation order are kept; transcendental functions
 * use the C library (the reference's own polynomials agree with it to a few ulp, docs/exact-transcendentals.md).
 * Build: see oracle/Makefile (-ffp-contract=off, so a*b+c rounds twice unless written as fmaf).
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

/* Dense.Gemm -> Kernels.Gemm.Run (src/OneModel/Tensors/Autograd/Dense.cs:12-48; docs/kernels-gemm.md:73-79):
 * one accumulator per output element, from +0, increasing k, fused multiply-add. A transposed operand is first
 * copied to row-major scratch (Dense.Transpose, Dense.cs:51-69), as the reference does. The i-k-j loop order below
 * gives each C[i][j] exactly the sequence fmaf(a[i][0],b[0][j],0), fmaf(a[i][1],b[1][j],.), ... */
API void orc_gemm(int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B, int ldb, float* C,
                  int ldc, int accumulate) {
  float *At = NULL, *Bt = NULL;
  if (ta) {
    At = (float*)malloc(sizeof(float) * (size_t)m * k + 4);
    for (int i = 0; i < m; i++)
      for (int p = 0; p < k; p++) At[(size_t)i * k + p] = A[(size_t)p * lda + i];
    A = At;
    lda = k;
  }
  if (tb) {
    Bt = (float*)malloc(sizeof(float) * (size_t)k * n + 4);
#pragma omp parallel for schedule(static)
    for (int p = 0; p < k; p++)
      for (int j = 0; j < n; j++) Bt[(size_t)p * n + j] = B[(size_t)j * ldb + p];
    B = Bt;
    ldb = n;
  }
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; i++) {
    float* tmp = (float*)malloc(sizeof(float) * (size_t)n + 4);
    for (int j = 0; j < n; j++) tmp[j] = 0.0f;
    for (int p = 0; p < k; p++) {
      float a = A[(size_t)i * lda + p];
      const float* b = B + (size_t)p * ldb;
      for (int j = 0; j < n; j++) tmp[j] = fmaf(a, b[j], tmp[j]);
    }
    float* c = C + (size_t)i * ldc;
    if (accumulate)
      for (int j = 0; j < n; j++) c[j] += tmp[j];
    else
      for (int j = 0; j < n; j++) c[j] = tmp[j];
    free(tmp);
  }
  free(At);
  free(Bt);
}

/* Same with operands rounded to bfloat16 (round to nearest even, docs/tensors.md:177) before multiplication and fp32
 * accumulation: the arithmetic the bf16-operand configuration asks for. */
static float bf16_round(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return x;
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  memcpy(&x, &u, 4);
  return x;
}
API void orc_round_bf16(const float* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) y[i] = bf16_round(x[i]);
}
/* Thread count of the OpenMP regions below (the products, attention heads and softmax rows): set explicitly by the timed
 * CPU baseline so that it does not depend on what a launcher put into OMP_NUM_THREADS. Returns the count in effect. */
API int orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* TF32 operand rounding (10 explicit mantissa bits): mode 0 drops the low 13 bits (what the tensor pipe does to raw
 * fp32 operands), mode 1 rounds to nearest, ties to even (what the product's TMA loads do; measured on B200). */
API void orc_round_tf32(const float* x, float* y, int64_t n, int nearest) {
  for (int64_t i = 0; i < n; i++) {
    uint32_t u;
    memcpy(&u, &x[i], 4);
    if ((u & 0x7f800000u) != 0x7f800000u && nearest) u += 0xfffu + ((u >> 13) & 1u);
    u &= 0xffffe000u;
    memcpy(&y[i], &u, 4);
  }
}

/* ---- elementwise (src/OneModel/Kernels/TrainElementwise.cs:42-98; Kernels/Exact/ExactUnary.cs) ------------------- */
API void orc_unary(int op, const float* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    float v = x[i];
    switch (op) {
      case 1: y[i] = v > 0.0f ? v : (v == v ? 0.0f : v); break;                 /* ReluUn */
      case 2: y[i] = (0.5f * v) * (1.0f + erff(v * 0.70710677f)); break;         /* GeluErf */
      case 3: {
        float u = 0.79788456f * (v + ((0.044715f * v) * v) * v);
        y[i] = (0.5f * v) * (1.0f + tanhf(u));
        break;
      }
      case 4: y[i] = 1.0f / (1.0f + expf(-v)); break;
      case 5: y[i] = tanhf(v); break;
      case 6: y[i] = v * -1.0f; break;
      case 7: y[i] = expf(v); break;
      case 8: y[i] = sqrtf(v); break;
      case 9: y[i] = erff(v); break;
      default: y[i] = v;
    }
  }
}

API void orc_unary_bwd(int op, const float* g, const float* s, float* dx, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    float gv = g[i], v = s[i];
    switch (op) {
      case 1: dx[i] = v > 0.0f ? gv : 0.0f; break;                               /* ReluGradBin */
      case 2: {                                                                  /* GeluGradBin, erf form */
        float cdf = 0.5f * (1.0f + erff(v * 0.70710677f));
        float pdf = expf((-0.5f * v) * v) * 0.3989423f;
        dx[i] = gv * (cdf + v * pdf);
        break;
      }
      case 3: {                                                                  /* GeluGradBin, tanh form */
        float u = 0.79788456f * (v + ((0.044715f * v) * v) * v);
        float t = tanhf(u);
        float left = 0.5f * (1.0f + t);
        float right = (((0.5f * v) * (1.0f - t * t)) * 0.79788456f) * (1.0f + ((3.0f * 0.044715f) * v) * v);
        dx[i] = gv * (left + right);
        break;
      }
      case 4: dx[i] = (gv * v) * (1.0f - v); break;                              /* SigmoidGradBin */
      case 5: dx[i] = gv * (1.0f - v * v); break;                                /* TanhGradBin */
      case 6: dx[i] = gv * -1.0f; break;
      default: dx[i] = gv;
    }
  }
}

/* BackwardOps.SumTo (src/OneModel/Tensors/Autograd/BackwardOps.cs:201-269): g of `shape` summed onto the target
 * whose per-axis strides are ts (0 on broadcast axes); double accumulators, increasing source order. */
API void orc_sum_to(int rank, const int32_t* shape, const float* g, const int64_t* ts, float* out, int64_t out_len) {
  double* sum = (double*)calloc((size_t)(out_len > 0 ? out_len : 1), sizeof(double));
  int64_t n = 1;
  for (int i = 0; i < rank; i++) n *= shape[i];
  int32_t idx[8] = {0};
  int64_t off = 0;
  for (int64_t e = 0; e < n; e++) {
    sum[off] += g[e];
    for (int ax = rank - 1; ax >= 0; ax--) {
      idx[ax]++;
      off += ts[ax];
      if (idx[ax] < shape[ax]) break;
      off -= ts[ax] * shape[ax];
      idx[ax] = 0;
    }
  }
  for (int64_t i = 0; i < out_len; i++) out[i] = (float)sum[i];
  free(sum);
}

/* Ops.Reduce (src/OneModel/Tensors/Ops.Nn.cs:162-231). */
API void orc_reduce_fwd(const float* x, int64_t outer, int64_t n, int64_t inner, int mean, float* y) {
  for (int64_t o = 0; o < outer; o++)
    for (int64_t i = 0; i < inner; i++) {
      double acc = 0;
      for (int64_t k = 0; k < n; k++) acc += x[((o * n) + k) * inner + i];
      y[o * inner + i] = mean ? (float)(acc / (double)n) : (float)acc;
    }
}
/* ReduceBackward (BackwardNn.cs:145-168). */
API void orc_reduce_bwd(const float* g, int64_t outer, int64_t n, int64_t inner, int mean, float* dx) {
  float fn = (float)n;
  for (int64_t o = 0; o < outer; o++)
    for (int64_t k = 0; k < n; k++)
      for (int64_t i = 0; i < inner; i++) {
        float v = g[o * inner + i];
        dx[((o * n) + k) * inner + i] = mean ? v / fn : v;
      }
}

/* ---- softmax family (Ops.Layers.cs:17-96; BackwardNn.cs:26-80) --------------------------------------------------- */
API void orc_softmax_fwd(const float* x, int rows, int cols, float* y) {
  for (int r = 0; r < rows; r++) {
    const float* s = x + (size_t)r * cols;
    float* d = y + (size_t)r * cols;
    float max = -INFINITY;
    for (int j = 0; j < cols; j++)
      if (s[j] > max) max = s[j];
    double sum = 0;
    for (int j = 0; j < cols; j++) {
      d[j] = expf(s[j] - max);
      sum += d[j];
    }
    float fs = (float)sum;
    for (int j = 0; j < cols; j++) d[j] = d[j] / fs;
  }
}
API void orc_logsoftmax_fwd(const float* x, int rows, int cols, float* y) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; r++) {
    const float* s = x + (size_t)r * cols;
    float* d = y + (size_t)r * cols;
    float max = -INFINITY;
    for (int j = 0; j < cols; j++)
      if (s[j] > max) max = s[j];
    double sum = 0;
    for (int j = 0; j < cols; j++) sum += expf(s[j] - max);
    float lse = max + logf((float)sum);
    for (int j = 0; j < cols; j++) d[j] = s[j] - lse;
  }
}
API void orc_softmax_bwd(const float* g, const float* y, int rows, int cols, float* dx) {
  for (int r = 0; r < rows; r++) {
    size_t o = (size_t)r * cols;
    double dot = 0;
    for (int j = 0; j < cols; j++) dot += (double)(g[o + j] * y[o + j]);
    float dotf = (float)dot;
    for (int j = 0; j < cols; j++) dx[o + j] = y[o + j] * (g[o + j] - dotf);
  }
}
API void orc_logsoftmax_bwd(const float* g, const float* y, int rows, int cols, float* dx) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; r++) {
    size_t o = (size_t)r * cols;
    double sum = 0;
    for (int j = 0; j < cols; j++) sum += g[o + j];
    float s = (float)sum;
    for (int j = 0; j < cols; j++) dx[o + j] = g[o + j] - (expf(y[o + j]) * s);
  }
}

/* Ops.NllLoss (Ops.Layers.cs:644-699). Returns -1 on an out-of-range target, else the counted rows. */
API int orc_nll_fwd(const float* logp, const int64_t* targets, int rows, int cols, int mean, int64_t ignore, float* loss) {
  double sum = 0;
  int count = 0;
  for (int i = 0; i < rows; i++) {
    int64_t t = targets[i];
    if (t == ignore) continue;
    if (t < 0 || t >= cols) return -1;
    sum -= logp[(size_t)i * cols + t];
    count++;
  }
  *loss = (float)(mean ? sum / (count > 1 ? count : 1) : sum);
  return count;
}
/* NllBackward (BackwardNn.cs:602-634). */
API void orc_nll_bwd(float g, const int64_t* targets, int rows, int cols, int mean, int64_t ignore, float* dx) {
  int count = 0;
  for (int i = 0; i < rows; i++)
    if (targets[i] != ignore) count++;
  float scale = mean ? g / (float)(count > 1 ? count : 1) : g;
  memset(dx, 0, sizeof(float) * (size_t)rows * cols);
  for (int i = 0; i < rows; i++)
    if (targets[i] != ignore) dx[(size_t)i * cols + targets[i]] = -scale;
}

/* ---- layer norm (Kernels/Exact/NormKernels.cs:66-128; BackwardNn.cs:170-242) --------------------------------------- */
/* RowReduce.Sum16 (src/OneModel/Kernels/Softmax.cs:136-175): 16 partial sums, element j added to partial j mod 16 in
 * increasing j (tail included), then combined by halving (p[t] + p[t+8], then +4, +2, +1). */
static float sum16(const float* x, int n) {
  float p[16] = {0};
  for (int j = 0; j < n; j++) p[j & 15] += x[j];
  for (int s = 8; s > 0; s >>= 1)
    for (int l = 0; l < s; l++) p[l] += p[l + s];
  return p[0];
}
API void orc_layernorm_fwd(const float* x, const float* gamma, const float* beta, int rows, int cols, float eps, float* y,
                           float* mean_out, float* inv_out) {
  float* dev = (float*)malloc(sizeof(float) * (size_t)cols + 4);
  float n = (float)cols;
  for (int r = 0; r < rows; r++) {
    const float* xr = x + (size_t)r * cols;
    float* yr = y + (size_t)r * cols;
    float mean = sum16(xr, cols) / n;
    for (int j = 0; j < cols; j++) {
      float d = xr[j] - mean;
      dev[j] = d * d;
    }
    float ssq = sum16(dev, cols);
    float inv = 1.0f / sqrtf((ssq / n) + eps);
    if (mean_out) mean_out[r] = mean;
    if (inv_out) inv_out[r] = inv;
    for (int j = 0; j < cols; j++) yr[j] = (((xr[j] - mean) * inv) * gamma[j]) + beta[j];
  }
  free(dev);
}
API void orc_layernorm_bwd(const float* g, const float* x, const float* gamma, const float* mean, const float* inv, int rows,
                           int cols, float* dx, float* dgamma, float* dbeta) {
  double* sg = (double*)calloc((size_t)cols, sizeof(double));
  double* sb = (double*)calloc((size_t)cols, sizeof(double));
  for (int r = 0; r < rows; r++) {
    size_t o = (size_t)r * cols;
    float m = mean[r], s = inv[r];
    double sum1 = 0, sum2 = 0;
    for (int j = 0; j < cols; j++) {
      float xhat = (x[o + j] - m) * s;
      float dxhat = g[o + j] * gamma[j];
      sum1 += dxhat;
      sum2 += (double)(dxhat * xhat);
      sg[j] += (double)(g[o + j] * xhat);
      sb[j] += g[o + j];
    }
    if (dx) {
      float m1 = (float)(sum1 / cols), m2 = (float)(sum2 / cols);
      for (int j = 0; j < cols; j++) {
        float xhat = (x[o + j] - m) * s;
        dx[o + j] = s * ((g[o + j] * gamma[j]) - m1 - (xhat * m2));
      }
    }
  }
  for (int j = 0; j < cols; j++) {
    if (dgamma) dgamma[j] = (float)sg[j];
    if (dbeta) dbeta[j] = (float)sb[j];
  }
  free(sg);
  free(sb);
}

/* ---- batch norm (Ops.Layers.cs:158-277; BackwardNn.cs:244-307) ------------------------------------------------------ */
API void orc_batchnorm_fwd(const float* x, const float* gamma, const float* beta, float* rm, float* rv, int n, int c,
                           int plane, int training, float momentum, float eps, float* y, float* mu, float* iv) {
  if (training) {
    double m = (double)n * plane;
    for (int ch = 0; ch < c; ch++) {
      double sum = 0;
      for (int i = 0; i < n; i++) {
        const float* pl = x + ((size_t)i * c + ch) * plane;
        for (int p = 0; p < plane; p++) sum += pl[p];
      }
      double mu64 = sum / m, ss = 0;
      for (int i = 0; i < n; i++) {
        const float* pl = x + ((size_t)i * c + ch) * plane;
        for (int p = 0; p < plane; p++) {
          double dd = pl[p] - mu64;
          ss += dd * dd;
        }
      }
      double var = ss / m;
      mu[ch] = (float)mu64;
      iv[ch] = 1.0f / sqrtf((float)var + eps);
      double unbiased = m > 1 ? var * m / (m - 1) : var;
      rm[ch] = (float)(((1 - momentum) * rm[ch]) + (momentum * mu64));
      rv[ch] = (float)(((1 - momentum) * rv[ch]) + (momentum * unbiased));
    }
  } else {
    for (int ch = 0; ch < c; ch++) {
      mu[ch] = rm[ch];
      iv[ch] = 1.0f / sqrtf(rv[ch] + eps);
    }
  }
  for (int i = 0; i < n; i++)
    for (int ch = 0; ch < c; ch++) {
      size_t o = ((size_t)i * c + ch) * plane;
      float mm = mu[ch], s = iv[ch], gg = gamma[ch], bb = beta[ch];
      for (int p = 0; p < plane; p++) y[o + p] = (((x[o + p] - mm) * s) * gg) + bb;
    }
}
API void orc_batchnorm_bwd(const float* g, const float* x, const float* gamma, const float* mu, const float* iv, int n, int c,
                           int plane, int training, float* dx, float* dgamma, float* dbeta) {
  double m = (double)n * plane;
  double* sg = (double*)calloc((size_t)c, sizeof(double));
  double* sb = (double*)calloc((size_t)c, sizeof(double));
  for (int i = 0; i < n; i++)
    for (int ch = 0; ch < c; ch++) {
      size_t o = ((size_t)i * c + ch) * plane;
      float mm = mu[ch], s = iv[ch];
      double a = 0, b = 0;
      for (int p = 0; p < plane; p++) {
        float gg = g[o + p];
        a += (double)(gg * ((x[o + p] - mm) * s));
        b += gg;
      }
      sg[ch] += a;
      sb[ch] += b;
    }
  if (dx)
    for (int i = 0; i < n; i++)
      for (int ch = 0; ch < c; ch++) {
        size_t o = ((size_t)i * c + ch) * plane;
        float mm = mu[ch], s = iv[ch], k = gamma[ch] * s;
        float cb = (float)(sb[ch] / m), cg = (float)(sg[ch] / m);
        for (int p = 0; p < plane; p++)
          dx[o + p] = training ? k * (g[o + p] - cb - (((x[o + p] - mm) * s) * cg)) : k * g[o + p];
      }
  for (int ch = 0; ch < c; ch++) {
    if (dgamma) dgamma[ch] = (float)sg[ch];
    if (dbeta) dbeta[ch] = (float)sb[ch];
  }
  free(sg);
  free(sb);
}

/* ---- embedding (Ops.Layers.cs:549-628; BackwardNn.cs:508-546) ------------------------------------------------------- */
API int orc_embedding_fwd(const float* table, int v, int dim, const int64_t* ids, int64_t n, float* out) {
  for (int64_t i = 0; i < n; i++) {
    if (ids[i] < 0 || ids[i] >= v) return -1;
    memcpy(out + i * dim, table + ids[i] * dim, sizeof(float) * (size_t)dim);
  }
  return 0;
}
API void orc_embedding_bwd(const float* g, const int64_t* ids, int64_t n, int v, int dim, int64_t pad, float* dtable) {
  memset(dtable, 0, sizeof(float) * (size_t)v * dim);
  for (int64_t i = 0; i < n; i++) {
    if (ids[i] == pad) continue;
    float* row = dtable + ids[i] * dim;
    const float* src = g + i * dim;
    for (int j = 0; j < dim; j++) row[j] += src[j];
  }
}

/* ---- attention (Ops.Layers.cs:746-807 forward; BackwardNn.cs:636-701 backward) -------------------------------------- */
/* The forward restates the definition softmax(scale QK^T + mask) V per head with the reference's GEMM and row-softmax
 * arithmetic (the fused CPU kernel, Kernels/AttentionDriver.cs:29, is within 3.4e-6 of it, docs/kernels-attention.md:53-57). */
API void orc_attention_fwd(const float* q, const float* k, const float* v, const float* mask, int64_t mask_bs, int b, int h,
                           int lq, int lk, int d, float scale, float* out) {
#pragma omp parallel for schedule(dynamic)
  for (int bh = 0; bh < b * h; bh++) {
    int bi = bh / h;
    float* s = (float*)malloc(sizeof(float) * (size_t)lq * lk);
    const float *qh = q + (size_t)bh * lq * d, *kh = k + (size_t)bh * lk * d, *vh = v + (size_t)bh * lk * d;
    orc_gemm(0, 1, lq, lk, d, qh, d, kh, d, s, lk, 0);
    for (int i = 0; i < lq; i++)
      for (int j = 0; j < lk; j++)
        s[(size_t)i * lk + j] = (s[(size_t)i * lk + j] * scale) + (mask ? mask[bi * mask_bs + (size_t)i * lk + j] : 0.0f);
    orc_softmax_fwd(s, lq, lk, s);
    orc_gemm(0, 0, lq, d, lk, s, lk, vh, d, out + (size_t)bh * lq * d, d, 0);
    free(s);
  }
}
API void orc_attention_bwd(const float* g, const float* q, const float* k, const float* v, const float* mask, int64_t mask_bs,
                           int b, int h, int lq, int lk, int d, float scale, float* dq, float* dk, float* dv) {
#pragma omp parallel for schedule(dynamic)
  for (int bh = 0; bh < b * h; bh++) {
    int bi = bh / h;
    size_t qo = (size_t)bh * lq * d, ko = (size_t)bh * lk * d;
    float* sv = (float*)malloc(sizeof(float) * (size_t)lq * lk);
    float* dp = (float*)malloc(sizeof(float) * (size_t)lq * lk);
    orc_gemm(0, 1, lq, lk, d, q + qo, d, k + ko, d, sv, lk, 0);
    for (int i = 0; i < lq; i++)
      for (int j = 0; j < lk; j++)
        sv[(size_t)i * lk + j] = (sv[(size_t)i * lk + j] * scale) + (mask ? mask[bi * mask_bs + (size_t)i * lk + j] : 0.0f);
    orc_softmax_fwd(sv, lq, lk, sv);
    orc_gemm(1, 0, lk, d, lq, sv, lk, g + qo, d, dv + ko, d, 0);
    orc_gemm(0, 1, lq, lk, d, g + qo, d, v + ko, d, dp, lk, 0);
    for (int i = 0; i < lq; i++) {
      size_t o = (size_t)i * lk;
      double dot = 0;
      for (int j = 0; j < lk; j++) dot += (double)(dp[o + j] * sv[o + j]);
      float df = (float)dot;
      for (int j = 0; j < lk; j++) dp[o + j] = sv[o + j] * (dp[o + j] - df) * scale;
    }
    orc_gemm(0, 0, lq, d, lk, dp, lk, k + ko, d, dq + qo, d, 0);
    orc_gemm(1, 0, lk, d, lq, dp, lk, q + qo, d, dk + ko, d, 0);
    free(sv);
    free(dp);
  }
}

/* ---- optimizers (src/OneModel.Training/Optimizers.cs:335-373,501-508,554-589) ---------------------------------------- */
static double int_pow(double b, int64_t n) {
  double r = 1.0;
  while (n > 0) {
    if (n & 1) r *= b;
    b *= b;
    n >>= 1;
  }
  return r;
}
/* One Adam/AdamW step over one tensor; t is the 1-based step. */
API void orc_adam_step(float* p, const float* grad, float* m, float* v, float* vmax, int64_t n, float lr, float beta1,
                       float beta2, float eps, float wd, int decoupled, int amsgrad, int64_t t) {
  double bc1 = 1.0 - int_pow(beta1, t), bc2 = 1.0 - int_pow(beta2, t);
  float step_size = (float)((double)lr / bc1), sq = (float)sqrt(bc2);
  float b1 = beta1, b2 = beta2, omb1 = 1.0f - beta1, omb2 = 1.0f - beta2;
  float decay = 1.0f - lr * wd;
  for (int64_t i = 0; i < n; i++) {
    float g = grad[i], pi = p[i];
    if (wd != 0.0f) {
      if (decoupled) pi *= decay; else g += wd * pi;
    }
    float mi = b1 * m[i] + omb1 * g;
    float vi = b2 * v[i] + omb2 * g * g;
    m[i] = mi;
    v[i] = vi;
    float vd = vi;
    if (amsgrad) {
      vd = vmax[i] > vi ? vmax[i] : vi;
      vmax[i] = vd;
    }
    float denom = sqrtf(vd) / sq + eps;
    p[i] = pi - step_size * mi / denom;
  }
}
API void orc_sgd_step(float* p, const float* grad, float* buf, int64_t n, float lr, float wd, float mu, float dampening,
                      int nesterov, int has_momentum, int first) {
  float keep = 1.0f - dampening;
  for (int64_t i = 0; i < n; i++) {
    float g = grad[i];
    if (wd != 0.0f) g += wd * p[i];
    if (has_momentum) {
      float b = first ? g : mu * buf[i] + keep * g;
      buf[i] = b;
      g = nesterov ? g + mu * b : b;
    }
    p[i] -= lr * g;
  }
}
/* GradClip.ClipNorm pieces (src/OneModel.Training/Schedules.cs:22-100): running double sum across tensors. */
API double orc_sumsq(const float* g, int64_t n, double acc, int infinity) {
  for (int64_t i = 0; i < n; i++) {
    if (infinity) {
      double a = fabs((double)g[i]);
      if (a > acc || a != a) acc = a;
    } else {
      acc += (double)g[i] * g[i];
    }
  }
  return acc;
}
API void orc_scale(float* g, int64_t n, float coef) {
  for (int64_t i = 0; i < n; i++) g[i] *= coef;
}
