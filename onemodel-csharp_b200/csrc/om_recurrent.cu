// LSTM layer (forward and backward through time) and CTC (loss, gradient, greedy decode).
//
// LSTM follows Ops.LstmLayer and LstmBackward of the reference (Ops.Recurrent.cs:40-146, BackwardRecurrent.cs:10-113):
// the input projection of all steps is one product; each step is one small recurrent product plus one fused cell
// kernel (gate activations, cell and hidden update - or, backward, all gate gradients); the weight and input
// gradients are three large products after the time loop; bias gradients are double-precision column sums.
//
// CTC follows CtcLossMath.Alpha / Gradient (CtcLoss.cs:170-281) in double precision in log space with the reference's
// own exp/log polynomials (Ctc.cs:515-616), one CTA per sequence; per-class sums run in increasing extended-label
// order so the result has the reference's bits.
#include "om_common.cuh"
#include "om_lstm_seq.cuh"

namespace om {

int32_t gemm_dispatch(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B,
                      int ldb, float* C, int ldc, int acc, const float* bias);
int32_t colsum_ld(om_ctx* ctx, const float* g, int32_t rows, int32_t cols, int64_t ld, float* out, int32_t accumulate);

__device__ __forceinline__ float sigm(float x) { return 1.0f / (1.0f + expf(-x)); }

__global__ void lstm_bias_kernel(const float* __restrict__ a, const float* __restrict__ b, int n, float* __restrict__ out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = a ? a[i] : 0.f;
  if (b) v += b[i];
  out[i] = v;
}

// One time step for all batch rows: g = gates_t (+ rec) (+ bias), activations in place, c, tanh(c), h.
__global__ void lstm_cell_fwd_kernel(float* __restrict__ gates_t, const float* __restrict__ rec, const float* __restrict__ bias,
                                     const float* __restrict__ cprev, int batch, int h, float* __restrict__ c_t,
                                     float* __restrict__ tanhc_t, float* __restrict__ y_t) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= batch * h) return;
  int b = idx / h, j = idx % h;
  float* g = gates_t + (size_t)b * 4 * h;
  const float* rr = rec + (size_t)b * 4 * h;
  float v[4];
#pragma unroll
  for (int q = 0; q < 4; q++) {
    float t = g[q * h + j] + rr[q * h + j];
    if (bias) t = t + bias[q * h + j];
    v[q] = t;
  }
  float gi = sigm(v[0]), gf = sigm(v[1]), gg = tanhf(v[2]), go = sigm(v[3]);
  g[j] = gi;
  g[h + j] = gf;
  g[2 * h + j] = gg;
  g[3 * h + j] = go;
  float fc = gf * (cprev ? cprev[idx] : 0.f);
  float ig = gi * gg;
  float c = fc + ig;
  c_t[idx] = c;
  float tc = tanhf(c);
  tanhc_t[idx] = tc;
  y_t[idx] = go * tc;
}

// Gate gradients of one step (BackwardRecurrent.cs:37-57). dh may be null on the first processed step (zeros).
__global__ void lstm_cell_bwd_kernel(const float* __restrict__ gates_t, const float* __restrict__ tanhc_t,
                                     const float* __restrict__ gy_t, const float* __restrict__ dh, float* __restrict__ dc,
                                     const float* __restrict__ cprev, int batch, int h, float* __restrict__ dg_t) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= batch * h) return;
  int b = idx / h, j = idx % h;
  const float* g = gates_t + (size_t)b * 4 * h;
  float* d = dg_t + (size_t)b * 4 * h;
  float gi = g[j], gf = g[h + j], gg = g[2 * h + j], go = g[3 * h + j];
  float tc = tanhc_t[idx];
  float dH = gy_t[idx] + dh[idx];
  float dO = dH * tc;
  float dC = dc[idx] + ((dH * go) * (1.f - (tc * tc)));
  float cp = cprev ? cprev[idx] : 0.f;
  float dI = dC * gg, dF = dC * cp, dGg = dC * gi;
  dc[idx] = dC * gf;
  d[j] = (dI * gi) * (1.f - gi);
  d[h + j] = (dF * gf) * (1.f - gf);
  d[2 * h + j] = dGg * (1.f - (gg * gg));
  d[3 * h + j] = (dO * go) * (1.f - go);
}

// ---- CTC math: the reference's double-precision polynomials ------------------------------------------------------------
__device__ __forceinline__ double ctc_exp(double x) {
  if (!(x > -700.0)) return 0.0;
  if (x > 700.0) x = 700.0;
  double k = floor((x * 1.4426950408889634) + 0.5);
  double r = (x - (k * 6.93147180369123816490e-01)) - (k * 1.90821492927058770002e-10);
  double p = 1.0 / 6227020800.0;
  p = (p * r) + (1.0 / 479001600.0);
  p = (p * r) + (1.0 / 39916800.0);
  p = (p * r) + (1.0 / 3628800.0);
  p = (p * r) + (1.0 / 362880.0);
  p = (p * r) + (1.0 / 40320.0);
  p = (p * r) + (1.0 / 5040.0);
  p = (p * r) + (1.0 / 720.0);
  p = (p * r) + (1.0 / 120.0);
  p = (p * r) + (1.0 / 24.0);
  p = (p * r) + (1.0 / 6.0);
  p = (p * r) + 0.5;
  p = (p * r) + 1.0;
  p = (p * r) + 1.0;
  return p * __longlong_as_double((long long)((int)k + 1023) << 52);
}

__device__ __forceinline__ double ctc_log(double x) {
  if (x == 0.0) return -INFINITY;
  if (!(x > 0.0) || isinf(x)) return x;
  long long bits = __double_as_longlong(x);
  int e = (int)((bits >> 52) & 0x7FF);
  if (e == 0) {
    bits = __double_as_longlong(x * 18014398509481984.0);
    e = (int)((bits >> 52) & 0x7FF) - 54;
  }
  e -= 1023;
  double m = __longlong_as_double((bits & 0x000FFFFFFFFFFFFFLL) | 0x3FF0000000000000LL);
  if (m > 1.4142135623730951) {
    m *= 0.5;
    e++;
  }
  double s = (m - 1.0) / (m + 1.0);
  double z = s * s;
  double q = 1.0 / 19.0;
  q = (q * z) + (1.0 / 17.0);
  q = (q * z) + (1.0 / 15.0);
  q = (q * z) + (1.0 / 13.0);
  q = (q * z) + (1.0 / 11.0);
  q = (q * z) + (1.0 / 9.0);
  q = (q * z) + (1.0 / 7.0);
  q = (q * z) + (1.0 / 5.0);
  q = (q * z) + (1.0 / 3.0);
  q = (q * z) + 1.0;
  return (e * 0.6931471805599453) + (2.0 * s * q);
}

__device__ __forceinline__ double ctc_logadd(double a, double b) {
  if (a < b) {
    double t = a;
    a = b;
    b = t;
  }
  if (isinf(b) && b < 0) return a;
  double d = b - a;
  return d < -40.0 ? a : a + ctc_log(1.0 + ctc_exp(d));
}

__device__ __forceinline__ int ctc_label(const int32_t* tgt, int blank, int s) { return (s & 1) == 0 ? blank : tgt[s >> 1]; }
__device__ __forceinline__ bool ctc_can_skip(const int32_t* tgt, int s) { return s >= 2 && (s & 1) == 1 && tgt[s >> 1] != tgt[(s >> 1) - 1]; }

constexpr int kCtcThreads = 128;

// alpha for sequence b into alpha[len, ext]; returns the negative log-likelihood (every thread gets it).
// `rows` (2 * ext doubles of shared memory, or null) keeps the last two rows on chip, so that the step-to-step chain does
// not wait on a round trip through L2.
__device__ double ctc_alpha(const float* __restrict__ lp, int batch, int classes, int b, int len, const int32_t* tgt, int tl,
                            int blank, double* __restrict__ alpha, double* sh_nll, double* rows) {
  const int ext = 2 * tl + 1;
  if (len == 0) return tl == 0 ? 0.0 : INFINITY;
  if (tl > len) return INFINITY;  // more labels than frames: no alignment exists (and the scratch is sized for ext <= 2T+1)
  for (int t = 0; t < len; t++) {
    for (int s = threadIdx.x; s < ext; s += kCtcThreads) {
      double a;
      if (t == 0) {
        a = s <= 1 ? 0.0 : -INFINITY;
      } else {
        const double* prev = rows ? rows + ((t - 1) & 1) * ext : alpha + (size_t)(t - 1) * ext;
        a = prev[s];
        if (s >= 1) a = ctc_logadd(a, prev[s - 1]);
        if (ctc_can_skip(tgt, s)) a = ctc_logadd(a, prev[s - 2]);
      }
      double e = (double)lp[((size_t)t * batch + b) * classes + ctc_label(tgt, blank, s)];
      const double v = (isinf(a) && a < 0) ? -INFINITY : a + e;
      alpha[(size_t)t * ext + s] = v;
      if (rows) rows[(t & 1) * ext + s] = v;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    double p = alpha[(size_t)(len - 1) * ext + ext - 1];
    if (ext >= 2) p = ctc_logadd(p, alpha[(size_t)(len - 1) * ext + ext - 2]);
    *sh_nll = (isinf(p) && p < 0) ? INFINITY : -p;
  }
  __syncthreads();
  return *sh_nll;
}

__global__ void __launch_bounds__(kCtcThreads)
ctc_loss_kernel(const float* __restrict__ lp, int steps, int batch, int classes, const int32_t* __restrict__ targets,
                const int32_t* __restrict__ tlen, const int32_t* __restrict__ ilen, int blank, int zero_inf, int max_ext,
                double* __restrict__ alpha_all, float* __restrict__ nll_out, double* __restrict__ per, int32_t* status, int use_rows) {
  __shared__ double sh_nll;
  __shared__ int sh_off;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) {
    int off = 0;
    for (int i = 0; i < b; i++) off += tlen[i];
    sh_off = off;
  }
  __syncthreads();
  const int tl = tlen[b], len = ilen[b];
  const int32_t* tgt = targets + sh_off;
  bool bad = len < 0 || len > steps || tl < 0;
  for (int i = threadIdx.x; i < tl && !bad; i += kCtcThreads)
    if (tgt[i] < 0 || tgt[i] >= classes || tgt[i] == blank) bad = true;
  if (__syncthreads_or(bad)) {
    if (threadIdx.x == 0) {
      if (atomicCAS(status, 0, (int32_t)OM_ERR_INDEX) == 0) status[1] = b;
      if (nll_out) nll_out[b] = 0.f;
      per[b] = 0.0;
    }
    return;
  }
  extern __shared__ double ctc_rows[];
  double nll = ctc_alpha(lp, batch, classes, b, len, tgt, tl, blank, alpha_all + (size_t)b * steps * max_ext, &sh_nll,
                         use_rows ? ctc_rows : nullptr);
  if (threadIdx.x == 0) {
    double v = (isinf(nll) && zero_inf) ? 0.0 : nll;
    per[b] = v;
    if (nll_out) nll_out[b] = (float)v;
  }
}

__global__ void ctc_reduce_kernel(const double* __restrict__ per, const int32_t* __restrict__ tlen, int batch, int reduction,
                                  float* __restrict__ loss) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  double sum = 0;
  for (int b = 0; b < batch; b++) sum += reduction == 1 ? per[b] / (double)max(1, tlen[b]) : per[b];
  loss[0] = (float)(reduction == 1 ? sum / batch : sum);
}

__global__ void __launch_bounds__(kCtcThreads)
ctc_grad_kernel(const float* __restrict__ g, const float* __restrict__ lp, int steps, int batch, int classes,
                const int32_t* __restrict__ targets, const int32_t* __restrict__ tlen, const int32_t* __restrict__ ilen, int blank,
                int reduction, int max_ext, double* __restrict__ alpha_all, double* __restrict__ beta_all, float* __restrict__ grad,
                int use_rows) {
  extern __shared__ double ctc_rows[];
  double* rows = use_rows ? ctc_rows : nullptr;
  __shared__ double sh_nll;
  __shared__ int sh_off;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) {
    int off = 0;
    for (int i = 0; i < b; i++) off += tlen[i];
    sh_off = off;
  }
  __syncthreads();
  const int tl = tlen[b], len = min(max(ilen[b], 0), steps);
  const int32_t* tgt = targets + sh_off;
  const int ext = 2 * tl + 1;
  // The gradient tensor starts at zero.
  for (int t = 0; t < steps; t++)
    for (int c = threadIdx.x; c < classes; c += kCtcThreads) grad[((size_t)t * batch + b) * classes + c] = 0.f;
  double* alpha = alpha_all + (size_t)b * steps * max_ext;
  double* beta = beta_all + (size_t)b * steps * max_ext;
  double nll = ctc_alpha(lp, batch, classes, b, len, tgt, tl, blank, alpha, &sh_nll, rows);
  if (len == 0 || isinf(nll)) return;
  double scale = reduction == 0 ? (double)g[b] : (double)g[0];
  if (reduction == 1) scale = scale / (double)max(1, tl) / (double)batch;
  // beta for all steps first (a chain over t) ...
  for (int t = len - 1; t >= 0; t--) {
    for (int s = threadIdx.x; s < ext; s += kCtcThreads) {
      double v;
      if (t == len - 1) {
        v = s >= ext - 2 ? 0.0 : -INFINITY;
      } else {
        const double* nxt = rows ? rows + ((t + 1) & 1) * ext : beta + (size_t)(t + 1) * ext;
        v = nxt[s];
        if (s + 1 < ext) v = ctc_logadd(v, nxt[s + 1]);
        if (s + 2 < ext && ctc_can_skip(tgt, s + 2)) v = ctc_logadd(v, nxt[s + 2]);
      }
      double e = (double)lp[((size_t)t * batch + b) * classes + ctc_label(tgt, blank, s)];
      const double w = (isinf(v) && v < 0) ? -INFINITY : v + e;
      beta[(size_t)t * ext + s] = w;
      if (rows) rows[(t & 1) * ext + s] = w;
    }
    __syncthreads();
  }
  // ... then the gradient of every (step, class) independently: the walk over the extended labels of one class goes in
  // increasing s (LogAdd is not associative), but nothing orders one (step, class) against another.
  for (int item = threadIdx.x; item < len * classes; item += kCtcThreads) {
    const int t = item / classes, c = item % classes;
    double acc = -INFINITY;
    for (int s = 0; s < ext; s++) {
      if (ctc_label(tgt, blank, s) != c) continue;
      double ab = alpha[(size_t)t * ext + s] + beta[(size_t)t * ext + s];
      if (!(isinf(ab) && ab < 0) && !(ab != ab)) acc = ctc_logadd(acc, ab);
    }
    if (isinf(acc) && acc < 0) continue;
    double l = (double)lp[((size_t)t * batch + b) * classes + c];
    grad[((size_t)t * batch + b) * classes + c] = (float)(-scale * ctc_exp(acc - l + nll));
  }
}

// Greedy decode (Ctc.Greedy, Ctc.cs:89-190): per step the argmax with the reference's rule (`>` so ties go to the lower
// index, a NaN best is replaced by whatever comes next), runs of equal labels merged, blanks dropped; each kept run
// reports its label and its first and last step. One thread per sequence (the work is T*C compares).
__global__ void ctc_greedy_kernel(const float* __restrict__ lp, int steps, int batch, int classes, const int32_t* __restrict__ ilen,
                                  int blank, int32_t* __restrict__ labels, int32_t* __restrict__ first_step,
                                  int32_t* __restrict__ last_step, int32_t* __restrict__ lengths) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  int len = ilen ? min(max(ilen[b], 0), steps) : steps;
  int count = 0, last = blank, first = 0;
  for (int t = 0; t < len; t++) {
    const float* row = lp + ((size_t)t * batch + b) * classes;
    int best = 0;
    float bv = row[0];
    for (int c = 1; c < classes; c++) {
      if (row[c] > bv || bv != bv) {
        bv = row[c];
        best = c;
      }
    }
    if (best != last) {
      if (last != blank) {
        labels[(size_t)b * steps + count] = last;
        if (first_step) first_step[(size_t)b * steps + count] = first;
        if (last_step) last_step[(size_t)b * steps + count] = t - 1;
        count++;
      }
      if (best != blank) first = t;
    }
    last = best;
  }
  if (last != blank && len > 0) {
    labels[(size_t)b * steps + count] = last;
    if (first_step) first_step[(size_t)b * steps + count] = first;
    if (last_step) last_step[(size_t)b * steps + count] = len - 1;
    count++;
  }
  for (int i = count; i < steps; i++) {
    labels[(size_t)b * steps + i] = -1;
    if (first_step) first_step[(size_t)b * steps + i] = -1;
    if (last_step) last_step[(size_t)b * steps + i] = -1;
  }
  lengths[b] = count;
}

}  // namespace om

using namespace om;

extern "C" {

static int32_t lstm_fwd_body(om_ctx* ctx, int32_t reverse, int32_t t, int32_t b, int32_t i, int32_t h, const float* x, const float* w_ih,
                             const float* w_hh, const float* b_ih, const float* b_hh, const float* h0, const float* c0, float* y,
                             float* gates, float* c, float* tanh_c) {
  const int h4 = 4 * h, bh = b * h;
  OM_TRY(gemm_dispatch(ctx, 0, 1, t * b, h4, i, x, i, w_ih, i, gates, h4, 0, nullptr));
  float *bias = nullptr, *rec = nullptr;
  const bool has_bias = b_ih || b_hh;
  if (has_bias) {
    OM_TRY(pool_alloc(ctx, sizeof(float) * h4, false, (void**)&bias));
    lstm_bias_kernel<<<(unsigned)ceil_div(h4, 256), 256, 0, ctx->stream>>>(b_ih, b_hh, h4, bias);
  }
  int32_t st = pool_alloc(ctx, sizeof(float) * (size_t)b * h4, false, (void**)&rec);
  for (int f = 0; f < t && st == OM_OK; f++) {
    int tt = reverse ? t - 1 - f : f;
    int pt = reverse ? tt + 1 : tt - 1;
    bool first = f == 0;
    const float* hp = first ? h0 : y + (size_t)pt * bh;
    const float* cp = first ? c0 : c + (size_t)pt * bh;
    if (hp) {
      st = gemm_dispatch(ctx, 0, 1, b, h4, h, hp, h, w_hh, h, rec, h4, 0, nullptr);
    } else {
      cudaMemsetAsync(rec, 0, sizeof(float) * (size_t)b * h4, ctx->stream);
    }
    if (st != OM_OK) break;
    lstm_cell_fwd_kernel<<<(unsigned)ceil_div(bh, 256), 256, 0, ctx->stream>>>(gates + (size_t)tt * b * h4, rec, bias, cp, b, h,
                                                                             c + (size_t)tt * bh, tanh_c + (size_t)tt * bh, y + (size_t)tt * bh);
  }
  if (bias) pool_free(ctx, bias);
  if (rec) pool_free(ctx, rec);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_lstm_layer_fwd");
  return OM_OK;
}

// All time steps of `dirs` directions in one cooperative launch (om_lstm_seq.cu): the input products and the bias sums
// first, then the sequence kernel. Index k of the pointer tables is the direction; reverse[k] its time order.
static int32_t lstm_fwd_seq(om_ctx* ctx, int dirs, const int32_t* reverse, int32_t t, int32_t b, int32_t i, int32_t h, const float* x,
                            const float* const* w_ih, const float* const* w_hh, const float* const* b_ih, const float* const* b_hh,
                            const float* const* h0, const float* const* c0, float* const* y, float* const* gates, float* const* c,
                            float* const* tanh_c) {
  const int h4 = 4 * h;
  LstmSeqFwdDir d[2];
  float* bias[2] = {nullptr, nullptr};
  int32_t st = OM_OK;
  for (int k = 0; k < dirs && st == OM_OK; k++) {
    st = gemm_dispatch(ctx, 0, 1, t * b, h4, i, x, i, w_ih[k], i, gates[k], h4, 0, nullptr);
    const float* bi = b_ih ? b_ih[k] : nullptr;
    const float* bhh = b_hh ? b_hh[k] : nullptr;
    if (st == OM_OK && (bi || bhh)) {
      st = pool_alloc(ctx, sizeof(float) * h4, false, (void**)&bias[k]);
      if (st == OM_OK) lstm_bias_kernel<<<(unsigned)ceil_div(h4, 256), 256, 0, ctx->stream>>>(bi, bhh, h4, bias[k]);
    }
    d[k].gates = gates[k];
    d[k].w_hh = w_hh[k];
    d[k].bias = bias[k];
    d[k].h0 = h0 ? h0[k] : nullptr;
    d[k].c0 = c0 ? c0[k] : nullptr;
    d[k].y = y[k];
    d[k].c = c[k];
    d[k].tanh_c = tanh_c[k];
    d[k].counter = nullptr;
    d[k].reverse = reverse[k];
  }
  if (st == OM_OK) st = lstm_seq_fwd(ctx, dirs, t, b, h, d);
  for (int k = 0; k < 2; k++)
    if (bias[k]) pool_free(ctx, bias[k]);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_lstm_layer_fwd");
  return OM_OK;
}

int32_t om_lstm_layer_fwd(om_ctx* ctx, int32_t reverse, int32_t t, int32_t b, int32_t i, int32_t h, const float* x,
                          const float* w_ih, const float* w_hh, const float* b_ih, const float* b_hh, const float* h0,
                          const float* c0, float* y, float* gates, float* c, float* tanh_c) {
  OM_CHECK_CTX(ctx);
  if (t < 0 || b < 0 || i < 1 || h < 1) return fail(ctx, OM_ERR_SHAPE, "LstmLayer: T %d B %d I %d H %d", t, b, i, h);
  if (t == 0 || b == 0) return OM_OK;
  ProfileScope prof(ctx, "om_lstm_layer_fwd", 2.0 * t * b * 4.0 * h * (i + h), 4.0 * t * b * (double)(i + 7 * h));
  if (lstm_seq_supported(ctx, 1, t, b, h, false))
    return lstm_fwd_seq(ctx, 1, &reverse, t, b, i, h, x, &w_ih, &w_hh, &b_ih, &b_hh, &h0, &c0, &y, &gates, &c, &tanh_c);
  return lstm_fwd_body(ctx, reverse, t, b, i, h, x, w_ih, w_hh, b_ih, b_hh, h0, c0, y, gates, c, tanh_c);
}

int32_t om_lstm_bilayer_fwd(om_ctx* ctx, int32_t t, int32_t b, int32_t i, int32_t h, const float* x, const float* const* w_ih,
                            const float* const* w_hh, const float* const* b_ih, const float* const* b_hh, float* const* y,
                            float* const* gates, float* const* c, float* const* tanh_c) {
  OM_CHECK_CTX(ctx);
  if (t < 0 || b < 0 || i < 1 || h < 1) return fail(ctx, OM_ERR_SHAPE, "LstmLayer: T %d B %d I %d H %d", t, b, i, h);
  if (t == 0 || b == 0) return OM_OK;
  ProfileScope prof(ctx, "om_lstm_layer_fwd", 2.0 * 2 * t * b * 4.0 * h * (i + h), 2.0 * 4.0 * t * b * (double)(i + 7 * h));
  if (lstm_seq_supported(ctx, 2, t, b, h, false)) {
    const int32_t order[2] = {0, 1};
    return lstm_fwd_seq(ctx, 2, order, t, b, i, h, x, w_ih, w_hh, b_ih, b_hh, nullptr, nullptr, y, gates, c, tanh_c);
  }
  return run_forked(
      ctx, [&] { return lstm_fwd_body(ctx, 0, t, b, i, h, x, w_ih[0], w_hh[0], b_ih ? b_ih[0] : nullptr, b_hh ? b_hh[0] : nullptr, nullptr, nullptr, y[0], gates[0], c[0], tanh_c[0]); },
      [&] { return lstm_fwd_body(ctx, 1, t, b, i, h, x, w_ih[1], w_hh[1], b_ih ? b_ih[1] : nullptr, b_hh ? b_hh[1] : nullptr, nullptr, nullptr, y[1], gates[1], c[1], tanh_c[1]); });
}

// hprev[t] = y[t -/+ 1], and the initial state (or zeros) at the first processed step of the forward pass.
static void lstm_hprev(om_ctx* ctx, int32_t reverse, int32_t t, size_t bh, const float* y, const float* h0, float* hprev) {
  const int first_t = reverse ? t - 1 : 0;
  if (t > 1) {
    if (reverse) cudaMemcpyAsync(hprev, y + bh, sizeof(float) * (size_t)(t - 1) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
    else cudaMemcpyAsync(hprev + bh, y, sizeof(float) * (size_t)(t - 1) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
  }
  if (h0) cudaMemcpyAsync(hprev + (size_t)first_t * bh, h0, sizeof(float) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
  else cudaMemsetAsync(hprev + (size_t)first_t * bh, 0, sizeof(float) * bh, ctx->stream);
}

// The products over all time steps once the gate gradients dG [T*B, 4H] are complete.
static int32_t lstm_bwd_products(om_ctx* ctx, int32_t rows, int32_t i, int32_t h, const float* dG, const float* x, const float* hprev,
                                 const float* w_ih, float* dx, float* dw_ih, float* dw_hh, float* db_ih, float* db_hh) {
  const int h4 = 4 * h;
  if (dx) OM_TRY(gemm_dispatch(ctx, 0, 0, rows, i, h4, dG, h4, w_ih, i, dx, i, 0, nullptr));
  if (dw_ih) OM_TRY(gemm_dispatch(ctx, 1, 0, h4, i, rows, dG, h4, x, i, dw_ih, i, 0, nullptr));
  if (dw_hh) OM_TRY(gemm_dispatch(ctx, 1, 0, h4, h, rows, dG, h4, hprev, h, dw_hh, h, 0, nullptr));
  if (db_ih) OM_TRY(colsum_ld(ctx, dG, rows, h4, h4, db_ih, 0));
  if (db_hh) OM_TRY(colsum_ld(ctx, dG, rows, h4, h4, db_hh, 0));
  return OM_OK;
}

static int32_t lstm_bwd_body(om_ctx* ctx, int32_t reverse, int32_t t, int32_t b, int32_t i, int32_t h, const float* gy, const float* ghn,
                             const float* gcn, const float* x, const float* y, const float* w_ih, const float* w_hh, const float* h0,
                             const float* c0, const float* gates, const float* c, const float* tanh_c, float* dx, float* dw_ih,
                             float* dw_hh, float* db_ih, float* db_hh, float* dh0, float* dc0) {
  const int h4 = 4 * h, bh = b * h, rows = t * b;
  float *dG = nullptr, *dh = nullptr, *dc = nullptr, *hprev = nullptr;
  int32_t st = pool_alloc(ctx, sizeof(float) * (size_t)rows * h4, false, (void**)&dG);
  if (st == OM_OK) st = pool_alloc(ctx, sizeof(float) * bh, true, (void**)&dh);
  if (st == OM_OK) st = pool_alloc(ctx, sizeof(float) * bh, true, (void**)&dc);
  if (st == OM_OK) st = pool_alloc(ctx, sizeof(float) * (size_t)rows * h, false, (void**)&hprev);
  if (st == OM_OK) {
    if (ghn) cudaMemcpyAsync(dh, ghn, sizeof(float) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
    if (gcn) cudaMemcpyAsync(dc, gcn, sizeof(float) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
    lstm_hprev(ctx, reverse, t, (size_t)bh, y, h0, hprev);
  }
  for (int s = 0; s < t && st == OM_OK; s++) {
    int tt = reverse ? s : t - 1 - s;
    int pt = reverse ? tt + 1 : tt - 1;
    bool first = reverse ? tt == t - 1 : tt == 0;
    const float* cp = first ? c0 : c + (size_t)pt * bh;
    lstm_cell_bwd_kernel<<<(unsigned)ceil_div(bh, 256), 256, 0, ctx->stream>>>(gates + (size_t)tt * b * h4, tanh_c + (size_t)tt * bh,
                                                                             gy + (size_t)tt * bh, dh, dc, cp, b, h, dG + (size_t)tt * b * h4);
    if (s < t - 1 || dh0) st = gemm_dispatch(ctx, 0, 0, b, h, h4, dG + (size_t)tt * b * h4, h4, w_hh, h, dh, h, 0, nullptr);
  }
  if (st == OM_OK) st = lstm_bwd_products(ctx, rows, i, h, dG, x, hprev, w_ih, dx, dw_ih, dw_hh, db_ih, db_hh);
  if (st == OM_OK && dh0) cudaMemcpyAsync(dh0, dh, sizeof(float) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
  if (st == OM_OK && dc0) cudaMemcpyAsync(dc0, dc, sizeof(float) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
  if (dG) pool_free(ctx, dG);
  if (dh) pool_free(ctx, dh);
  if (dc) pool_free(ctx, dc);
  if (hprev) pool_free(ctx, hprev);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_lstm_layer_bwd");
  return OM_OK;
}

// The backward sweep of `dirs` directions in one cooperative launch, then each direction's products (on two streams when
// there are two directions).
static int32_t lstm_bwd_seq(om_ctx* ctx, int dirs, const int32_t* reverse, int32_t t, int32_t b, int32_t i, int32_t h,
                            const float* const* gy, const float* const* ghn, const float* const* gcn, const float* x,
                            const float* const* y, const float* const* w_ih, const float* const* w_hh, const float* const* h0,
                            const float* const* c0, const float* const* gates, const float* const* c, const float* const* tanh_c,
                            float* const* dx, float* const* dw_ih, float* const* dw_hh, float* const* db_ih, float* const* db_hh,
                            float* const* dh0, float* const* dc0) {
  const int h4 = 4 * h, rows = t * b;
  const size_t bh = (size_t)b * h;
  float* dG[2] = {nullptr, nullptr};
  float* hprev[2] = {nullptr, nullptr};
  LstmSeqBwdDir d[2];
  int32_t st = OM_OK;
  for (int k = 0; k < dirs && st == OM_OK; k++) {
    st = pool_alloc(ctx, sizeof(float) * (size_t)rows * h4, false, (void**)&dG[k]);
    if (st == OM_OK) st = pool_alloc(ctx, sizeof(float) * (size_t)rows * h, false, (void**)&hprev[k]);
    if (st != OM_OK) break;
    lstm_hprev(ctx, reverse[k], t, bh, y[k], h0 ? h0[k] : nullptr, hprev[k]);
    d[k].gates = gates[k];
    d[k].tanh_c = tanh_c[k];
    d[k].c = c[k];
    d[k].c0 = c0 ? c0[k] : nullptr;
    d[k].gy = gy[k];
    d[k].ghn = ghn ? ghn[k] : nullptr;
    d[k].gcn = gcn ? gcn[k] : nullptr;
    d[k].w_hh = w_hh[k];
    d[k].dG = dG[k];
    d[k].dh0 = dh0 ? dh0[k] : nullptr;
    d[k].dc0 = dc0 ? dc0[k] : nullptr;
    d[k].counter = nullptr;
    d[k].reverse = reverse[k];
  }
  if (st == OM_OK) st = lstm_seq_bwd(ctx, dirs, t, b, h, d);
  auto products = [&](int k) {
    return lstm_bwd_products(ctx, rows, i, h, dG[k], x, hprev[k], w_ih[k], dx ? dx[k] : nullptr, dw_ih ? dw_ih[k] : nullptr,
                             dw_hh ? dw_hh[k] : nullptr, db_ih ? db_ih[k] : nullptr, db_hh ? db_hh[k] : nullptr);
  };
  if (st == OM_OK) st = dirs == 2 ? run_forked(ctx, [&] { return products(0); }, [&] { return products(1); }) : products(0);
  for (int k = 0; k < 2; k++) {
    if (dG[k]) pool_free(ctx, dG[k]);
    if (hprev[k]) pool_free(ctx, hprev[k]);
  }
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_lstm_layer_bwd");
  return OM_OK;
}

int32_t om_lstm_layer_bwd(om_ctx* ctx, int32_t reverse, int32_t t, int32_t b, int32_t i, int32_t h, const float* gy,
                          const float* ghn, const float* gcn, const float* x, const float* y, const float* w_ih,
                          const float* w_hh, const float* h0, const float* c0, const float* gates, const float* c,
                          const float* tanh_c, float* dx, float* dw_ih, float* dw_hh, float* db_ih, float* db_hh, float* dh0,
                          float* dc0) {
  OM_CHECK_CTX(ctx);
  if (t < 0 || b < 0 || i < 1 || h < 1) return fail(ctx, OM_ERR_SHAPE, "LstmBackward: T %d B %d I %d H %d", t, b, i, h);
  if (t == 0 || b == 0) return OM_OK;
  ProfileScope prof(ctx, "om_lstm_layer_bwd", 4.0 * t * b * 4.0 * h * (i + h), 4.0 * t * b * (double)(2 * i + 12 * h));
  if (lstm_seq_supported(ctx, 1, t, b, h, true))
    return lstm_bwd_seq(ctx, 1, &reverse, t, b, i, h, &gy, &ghn, &gcn, x, &y, &w_ih, &w_hh, &h0, &c0, &gates, &c, &tanh_c, &dx, &dw_ih, &dw_hh,
                        &db_ih, &db_hh, &dh0, &dc0);
  return lstm_bwd_body(ctx, reverse, t, b, i, h, gy, ghn, gcn, x, y, w_ih, w_hh, h0, c0, gates, c, tanh_c, dx, dw_ih, dw_hh, db_ih, db_hh,
                       dh0, dc0);
}

int32_t om_lstm_bilayer_bwd(om_ctx* ctx, int32_t t, int32_t b, int32_t i, int32_t h, const float* const* gy, const float* x,
                            const float* const* y, const float* const* w_ih, const float* const* w_hh, const float* const* gates,
                            const float* const* c, const float* const* tanh_c, float* const* dx, float* const* dw_ih,
                            float* const* dw_hh, float* const* db_ih, float* const* db_hh) {
  OM_CHECK_CTX(ctx);
  if (t < 0 || b < 0 || i < 1 || h < 1) return fail(ctx, OM_ERR_SHAPE, "LstmBackward: T %d B %d I %d H %d", t, b, i, h);
  if (t == 0 || b == 0) return OM_OK;
  ProfileScope prof(ctx, "om_lstm_layer_bwd", 2.0 * 4.0 * t * b * 4.0 * h * (i + h), 2.0 * 4.0 * t * b * (double)(2 * i + 12 * h));
  if (lstm_seq_supported(ctx, 2, t, b, h, true)) {
    const int32_t order[2] = {0, 1};
    return lstm_bwd_seq(ctx, 2, order, t, b, i, h, gy, nullptr, nullptr, x, y, w_ih, w_hh, nullptr, nullptr, gates, c, tanh_c, dx, dw_ih, dw_hh,
                        db_ih, db_hh, nullptr, nullptr);
  }
  auto dir = [&](int d) {
    return lstm_bwd_body(ctx, d, t, b, i, h, gy[d], nullptr, nullptr, x, y[d], w_ih[d], w_hh[d], nullptr, nullptr, gates[d], c[d], tanh_c[d],
                         dx ? dx[d] : nullptr, dw_ih ? dw_ih[d] : nullptr, dw_hh ? dw_hh[d] : nullptr, db_ih ? db_ih[d] : nullptr,
                         db_hh ? db_hh[d] : nullptr, nullptr, nullptr);
  };
  return run_forked(ctx, [&] { return dir(0); }, [&] { return dir(1); });
}

static int32_t ctc_check(om_ctx* ctx, const char* who, int t, int b, int c, int blank, int reduction) {
  if (t < 0 || b < 0 || c < 1) return fail(ctx, OM_ERR_SHAPE, "%s needs log-probabilities [T,B,C] (T %d B %d C %d)", who, t, b, c);
  if (blank < 0 || blank >= c) return fail(ctx, OM_ERR_ARG, "The blank index %d is outside [0, %d).", blank, c);
  if (reduction < 0 || reduction > 2) return fail(ctx, OM_ERR_ARG, "%s: reduction %d", who, reduction);
  return OM_OK;
}

int32_t om_ctc_loss(om_ctx* ctx, const float* lp, int32_t t, int32_t b, int32_t c, const int32_t* targets,
                    const int32_t* target_lengths, const int32_t* input_lengths, int32_t blank, int32_t reduction,
                    int32_t zero_infinity, float* nll, float* loss) {
  OM_CHECK_CTX(ctx);
  OM_TRY(ctc_check(ctx, "CtcLoss", t, b, c, blank, reduction));
  if (b == 0) return OM_OK;
  ProfileScope prof(ctx, "om_ctc_loss", 0, 4.0 * t * b * (double)c);
  // The extended target is at most 2*T+1 long for a feasible alignment; longer targets are infeasible but still legal,
  // so size the scratch for the worst case the caller can express: sum of lengths is unknown here, bound by T.
  const int max_ext = 2 * (t > 0 ? t : 1) + 1;
  double *alpha = nullptr, *per = nullptr;
  OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)b * (t > 0 ? t : 1) * max_ext, false, (void**)&alpha));
  int32_t st = pool_alloc(ctx, sizeof(double) * b, false, (void**)&per);
  if (st == OM_OK) {
    const size_t rows_bytes = 2 * sizeof(double) * (size_t)max_ext;   // the last two alpha rows on chip when they fit
    const int use_rows = rows_bytes <= 40 * 1024;
    ctc_loss_kernel<<<b, kCtcThreads, use_rows ? rows_bytes : 0, ctx->stream>>>(lp, t, b, c, targets, target_lengths, input_lengths, blank,
                                                                                zero_infinity, max_ext, alpha, nll, per, ctx->status_dev, use_rows);
    if (reduction != 0 && loss) ctc_reduce_kernel<<<1, 32, 0, ctx->stream>>>(per, target_lengths, b, reduction, loss);
  }
  pool_free(ctx, alpha);
  if (per) pool_free(ctx, per);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_ctc_loss");
  return OM_OK;
}

int32_t om_ctc_grad(om_ctx* ctx, const float* g, const float* lp, int32_t t, int32_t b, int32_t c, const int32_t* targets,
                    const int32_t* target_lengths, const int32_t* input_lengths, const float* nll, int32_t blank,
                    int32_t reduction, int32_t zero_infinity, float* grad) {
  OM_CHECK_CTX(ctx);
  (void)nll;
  (void)zero_infinity;
  OM_TRY(ctc_check(ctx, "CtcBackward", t, b, c, blank, reduction));
  if (b == 0 || t == 0) return OM_OK;
  ProfileScope prof(ctx, "om_ctc_grad", 0, 8.0 * t * b * (double)c);
  const int max_ext = 2 * t + 1;
  double *alpha = nullptr, *beta = nullptr;
  OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)b * t * max_ext, false, (void**)&alpha));
  int32_t st = pool_alloc(ctx, sizeof(double) * (size_t)b * t * max_ext, false, (void**)&beta);
  if (st == OM_OK) {
    const size_t rows_bytes = 2 * sizeof(double) * (size_t)max_ext;
    const int use_rows = rows_bytes <= 40 * 1024;
    ctc_grad_kernel<<<b, kCtcThreads, use_rows ? rows_bytes : 0, ctx->stream>>>(g, lp, t, b, c, targets, target_lengths, input_lengths, blank,
                                                                                reduction, max_ext, alpha, beta, grad, use_rows);
  }
  pool_free(ctx, alpha);
  if (beta) pool_free(ctx, beta);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_ctc_grad");
  return OM_OK;
}

int32_t om_ctc_greedy(om_ctx* ctx, const float* lp, int32_t t, int32_t b, int32_t c, const int32_t* input_lengths, int32_t blank,
                      int32_t* labels, int32_t* first_step, int32_t* last_step, int32_t* lengths) {
  OM_CHECK_CTX(ctx);
  OM_TRY(ctc_check(ctx, "Ctc.Greedy", t, b, c, blank, 0));
  if (b == 0) return OM_OK;
  ProfileScope prof(ctx, "om_ctc_greedy", 0, 4.0 * t * b * (double)c);
  ctc_greedy_kernel<<<(unsigned)ceil_div(b, 64), 64, 0, ctx->stream>>>(lp, t, b, c, input_lengths, blank, labels, first_step, last_step, lengths);
  OM_LAUNCH_CHECK(ctx, "om_ctc_greedy");
  return OM_OK;
}

}  // extern "C"
