/*
 * TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT.
 * CPU restatement of the reference's convolution, pooling, LSTM and CTC training code (see om_oracle_core.c for the
 * rules). Paths are relative to the reference repository.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

void orc_gemm(int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B, int ldb, float* C, int ldc, int accumulate);

typedef struct {
  int n, cin, h, w, cout, kh, kw, sh, sw, pt, pl, pb, pr, dh, dw, groups;
} conv_shape;

static int out_h(const conv_shape* s) { return (s->h + s->pt + s->pb - s->dh * (s->kh - 1) - 1) / s->sh + 1; }
static int out_w(const conv_shape* s) { return (s->w + s->pl + s->pr - s->dw * (s->kw - 1) - 1) / s->sw + 1; }

/* Im2ColPatchMajor (src/OneModel/Tensors/Autograd/BackwardNn.cs:405-428): cols[p, k]. */
static void im2col_patch_major(const conv_shape* s, const float* x, float* cols) {
  int cg = s->cin / s->groups, kk = cg * s->kh * s->kw, ow = out_w(s), oh = out_h(s);
  for (int oy = 0; oy < oh; oy++)
    for (int ox = 0; ox < ow; ox++) {
      float* row = cols + (size_t)(oy * ow + ox) * kk;
      int k = 0;
      for (int c = 0; c < cg; c++)
        for (int ky = 0; ky < s->kh; ky++) {
          int iy = oy * s->sh - s->pt + ky * s->dh;
          for (int kx = 0; kx < s->kw; kx++, k++) {
            int ix = ox * s->sw - s->pl + kx * s->dw;
            row[k] = (iy >= 0 && iy < s->h && ix >= 0 && ix < s->w) ? x[((size_t)c * s->h + iy) * s->w + ix] : 0.0f;
          }
        }
    }
}

/* Col2Im (BackwardNn.cs:431-462): taps added in increasing (row of dcols, p) order. */
static void col2im(const conv_shape* s, const float* dcols, float* dx) {
  int cg = s->cin / s->groups, ow = out_w(s), oh = out_h(s), plane = oh * ow, k = 0;
  for (int c = 0; c < cg; c++)
    for (int ky = 0; ky < s->kh; ky++)
      for (int kx = 0; kx < s->kw; kx++, k++) {
        const float* row = dcols + (size_t)k * plane;
        for (int oy = 0; oy < oh; oy++) {
          int iy = oy * s->sh - s->pt + ky * s->dh;
          if (iy < 0 || iy >= s->h) continue;
          for (int ox = 0; ox < ow; ox++) {
            int ix = ox * s->sw - s->pl + kx * s->dw;
            if (ix >= 0 && ix < s->w) dx[((size_t)c * s->h + iy) * s->w + ix] += row[oy * ow + ox];
          }
        }
      }
}

/* Forward: the definition y[n,co,p] = sum_k w[co,k] cols[p,k] + b[co] with the reference GEMM's per-output order
 * (the reference forward runs Conv.Run, whose fast kernels agree with this sum to fp32 rounding, docs/kernels-conv.md). */
API void orc_conv2d_fwd(const conv_shape* s, const float* x, const float* w, const float* bias, float* y) {
  int cg = s->cin / s->groups, og = s->cout / s->groups, kk = cg * s->kh * s->kw, plane = out_h(s) * out_w(s);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < s->n; n++) {
    float* cols = (float*)malloc(sizeof(float) * (size_t)plane * kk + 4);
    for (int grp = 0; grp < s->groups; grp++) {
      im2col_patch_major(s, x + ((size_t)n * s->cin + (size_t)grp * cg) * s->h * s->w, cols);
      float* yo = y + ((size_t)n * s->cout + (size_t)grp * og) * plane;
      orc_gemm(0, 1, og, plane, kk, w + (size_t)grp * og * kk, kk, cols, kk, yo, plane, 0);
      if (bias)
        for (int co = 0; co < og; co++)
          for (int p = 0; p < plane; p++) yo[(size_t)co * plane + p] += bias[grp * og + co];
    }
    free(cols);
  }
}

/* ConvBackward (BackwardNn.cs:317-402). */
API void orc_conv2d_bwd(const conv_shape* s, const float* g, const float* x, const float* w, float* dx, float* dw, float* dbias) {
  int cg = s->cin / s->groups, og = s->cout / s->groups, kk = cg * s->kh * s->kw, plane = out_h(s) * out_w(s);
  if (dbias) {
    double* a = (double*)calloc((size_t)s->cout, sizeof(double));
    for (int n = 0; n < s->n; n++)
      for (int co = 0; co < s->cout; co++) {
        const float* row = g + ((size_t)n * s->cout + co) * plane;
        double t = 0;
        for (int i = 0; i < plane; i++) t += row[i];
        a[co] += t;
      }
    for (int co = 0; co < s->cout; co++) dbias[co] = (float)a[co];
    free(a);
  }
  if (dw) {
    memset(dw, 0, sizeof(float) * (size_t)s->cout * kk);
    float* cols = (float*)malloc(sizeof(float) * (size_t)plane * kk + 4);
    float* tmp = (float*)malloc(sizeof(float) * (size_t)og * kk + 4);
    for (int n = 0; n < s->n; n++)
      for (int grp = 0; grp < s->groups; grp++) {
        im2col_patch_major(s, x + ((size_t)n * s->cin + (size_t)grp * cg) * s->h * s->w, cols);
        orc_gemm(0, 0, og, kk, plane, g + ((size_t)n * s->cout + (size_t)grp * og) * plane, plane, cols, kk, tmp, kk, 0);
        float* dst = dw + (size_t)grp * og * kk;
        for (int i = 0; i < og * kk; i++) dst[i] += tmp[i];
      }
    free(cols);
    free(tmp);
  }
  if (dx) {
    memset(dx, 0, sizeof(float) * (size_t)s->n * s->cin * s->h * s->w);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < s->n; n++) {
      float* dcols = (float*)malloc(sizeof(float) * (size_t)kk * plane + 4);
      for (int grp = 0; grp < s->groups; grp++) {
        /* dcols[K,P] = W_g^T [K,og] . g[og,P] (the reference transposes W_g once, then a plain product). */
        orc_gemm(1, 0, kk, plane, og, w + (size_t)grp * og * kk, kk, g + ((size_t)n * s->cout + (size_t)grp * og) * plane, plane, dcols, plane, 0);
        col2im(s, dcols, dx + ((size_t)n * s->cin + (size_t)grp * cg) * s->h * s->w);
      }
      free(dcols);
    }
  }
}

/* ReferenceKernels.MaxPool2d (src/OneModel/Tensors/TensorKernels.cs:242-295). */
API void orc_maxpool_fwd(const float* x, int planes, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int oh, int ow,
                         float* y, int32_t* idx) {
  for (int pl = 0; pl < planes; pl++)
    for (int oy = 0; oy < oh; oy++)
      for (int ox = 0; ox < ow; ox++) {
        float best = -INFINITY;
        int bi = -1;
        for (int ky = 0; ky < kh; ky++) {
          int yy = oy * sh - ph + ky;
          if (yy < 0 || yy >= h) continue;
          for (int kx = 0; kx < kw; kx++) {
            int xx = ox * sw - pw + kx;
            if (xx < 0 || xx >= w) continue;
            float v = x[((size_t)pl * h + yy) * w + xx];
            int wins = bi < 0 || (v > best && !isnan(best)) || (isnan(v) && !isnan(best));
            if (wins) {
              best = v;
              bi = (pl * h + yy) * w + xx;
            }
          }
        }
        y[((size_t)pl * oh + oy) * ow + ox] = best;
        idx[((size_t)pl * oh + oy) * ow + ox] = bi;
      }
}
/* MaxPoolBackward (BackwardOps.cs:285-298). */
API void orc_maxpool_bwd(const float* g, const int32_t* idx, int64_t n_out, int64_t n_in, float* dx) {
  memset(dx, 0, sizeof(float) * (size_t)n_in);
  for (int64_t i = 0; i < n_out; i++) dx[idx[i]] += g[i];
}

/* PoolWindow (BackwardNn.cs:490-506). */
static void pool_window(int kh, int kw, int sh, int sw, int ph, int pw, int inc, int h, int w, int oy, int ox, int* y0, int* y1, int* x0,
                        int* x1, int* count) {
  int ys = oy * sh - ph, xs = ox * sw - pw;
  int ye = ys + kh < h + ph ? ys + kh : h + ph, xe = xs + kw < w + pw ? xs + kw : w + pw;
  int padded = (ye - ys) * (xe - xs);
  *y0 = ys > 0 ? ys : 0;
  *x0 = xs > 0 ? xs : 0;
  *y1 = ye < h ? ye : h;
  *x1 = xe < w ? xe : w;
  int inb = (*y1 - *y0) * (*x1 - *x0);
  *count = inc ? padded : (inb > 1 ? inb : 1);
}
/* Ops.AvgPool2d (Ops.Layers.cs:414-461) and AvgPoolBackward (BackwardNn.cs:464-488). */
API void orc_avgpool_fwd(const float* x, int planes, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int inc, int oh, int ow, float* y) {
  for (int pl = 0; pl < planes; pl++)
    for (int oy = 0; oy < oh; oy++)
      for (int ox = 0; ox < ow; ox++) {
        int y0, y1, x0, x1, count;
        pool_window(kh, kw, sh, sw, ph, pw, inc, h, w, oy, ox, &y0, &y1, &x0, &x1, &count);
        float sum = 0.0f;
        for (int yy = y0; yy < y1; yy++)
          for (int xx = x0; xx < x1; xx++) sum += x[((size_t)pl * h + yy) * w + xx];
        y[((size_t)pl * oh + oy) * ow + ox] = sum / count;
      }
}
API void orc_avgpool_bwd(const float* g, int planes, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int inc, int oh, int ow, float* dx) {
  memset(dx, 0, sizeof(float) * (size_t)planes * h * w);
  for (int pl = 0; pl < planes; pl++)
    for (int oy = 0; oy < oh; oy++)
      for (int ox = 0; ox < ow; ox++) {
        int y0, y1, x0, x1, count;
        pool_window(kh, kw, sh, sw, ph, pw, inc, h, w, oy, ox, &y0, &y1, &x0, &x1, &count);
        float share = g[((size_t)pl * oh + oy) * ow + ox] / count;
        for (int yy = y0; yy < y1; yy++)
          for (int xx = x0; xx < x1; xx++) dx[((size_t)pl * h + yy) * w + xx] += share;
      }
}

/* ---- LSTM (Ops.Recurrent.cs:40-146; BackwardRecurrent.cs:10-113,224-246), zero initial state --------------------------- */
static float sigm(float x) { return 1.0f / (1.0f + expf(-x)); }

API void orc_lstm_fwd(int reverse, int steps, int batch, int in_size, int h, const float* x, const float* wih, const float* whh,
                      const float* bih, const float* bhh, float* y, float* gates, float* cseq, float* tanhc) {
  int h4 = 4 * h, bh = batch * h;
  float* rec = (float*)malloc(sizeof(float) * (size_t)batch * h4);
  float* zeros = (float*)calloc((size_t)bh, sizeof(float));
  float* bias = (float*)calloc((size_t)h4, sizeof(float));
  orc_gemm(0, 1, steps * batch, h4, in_size, x, in_size, wih, in_size, gates, h4, 0);
  if (bih) memcpy(bias, bih, sizeof(float) * h4);
  if (bhh) for (int i = 0; i < h4; i++) bias[i] += bhh[i];
  int has_bias = bih || bhh;
  for (int f = 0; f < steps; f++) {
    int t = reverse ? steps - 1 - f : f, pt = reverse ? t + 1 : t - 1;
    const float* hp = f == 0 ? zeros : y + (size_t)pt * bh;
    const float* cp = f == 0 ? zeros : cseq + (size_t)pt * bh;
    orc_gemm(0, 1, batch, h4, h, hp, h, whh, h, rec, h4, 0);   /* h_prev . W_hh^T (the reference multiplies by the transposed copy) */
    for (int b = 0; b < batch; b++) {
      float* g = gates + ((size_t)t * batch + b) * h4;
      const float* rr = rec + (size_t)b * h4;
      for (int i = 0; i < h4; i++) g[i] = g[i] + rr[i];
      if (has_bias) for (int i = 0; i < h4; i++) g[i] = g[i] + bias[i];
      for (int j = 0; j < 2 * h; j++) g[j] = sigm(g[j]);
      for (int j = 2 * h; j < 3 * h; j++) g[j] = tanhf(g[j]);
      for (int j = 3 * h; j < h4; j++) g[j] = sigm(g[j]);
      float* c = cseq + ((size_t)t * batch + b) * h;
      float* tc = tanhc + ((size_t)t * batch + b) * h;
      float* ho = y + ((size_t)t * batch + b) * h;
      for (int j = 0; j < h; j++) {
        float fc = g[h + j] * cp[b * h + j];
        float ig = g[j] * g[2 * h + j];
        c[j] = fc + ig;
        tc[j] = tanhf(c[j]);
        ho[j] = g[3 * h + j] * tc[j];
      }
    }
  }
  free(rec);
  free(zeros);
  free(bias);
}

API void orc_lstm_bwd(int reverse, int steps, int batch, int in_size, int h, const float* gy, const float* x, const float* y,
                      const float* wih, const float* whh, const float* gates, const float* cseq, const float* tanhc, float* dx,
                      float* dwih, float* dwhh, float* dbih, float* dbhh) {
  int h4 = 4 * h, bh = batch * h, rows = steps * batch;
  float* dG = (float*)malloc(sizeof(float) * (size_t)rows * h4);
  float* dh = (float*)calloc((size_t)bh, sizeof(float));
  float* dc = (float*)calloc((size_t)bh, sizeof(float));
  float* zeros = (float*)calloc((size_t)bh, sizeof(float));
  float* hprev = (float*)malloc(sizeof(float) * (size_t)rows * h);
  for (int s = 0; s < steps; s++) {
    int t = reverse ? s : steps - 1 - s, pt = reverse ? t + 1 : t - 1;
    int first = reverse ? t == steps - 1 : t == 0;
    const float* cp = first ? zeros : cseq + (size_t)pt * bh;
    const float* hpv = first ? zeros : y + (size_t)pt * bh;
    memcpy(hprev + (size_t)t * bh, hpv, sizeof(float) * bh);
    for (int b = 0; b < batch; b++) {
      size_t row = (size_t)t * batch + b;
      const float* g = gates + row * h4;
      float* d = dG + row * h4;
      for (int j = 0; j < h; j++) {
        int k = b * h + j;
        float gi = g[j], gf = g[h + j], gg = g[2 * h + j], go = g[3 * h + j];
        float tc = tanhc[row * h + j];
        float dH = gy[row * h + j] + dh[k];
        float dO = dH * tc;
        float dC = dc[k] + ((dH * go) * (1.0f - (tc * tc)));
        float dI = dC * gg, dF = dC * cp[k], dGg = dC * gi;
        dc[k] = dC * gf;
        d[j] = (dI * gi) * (1.0f - gi);
        d[h + j] = (dF * gf) * (1.0f - gf);
        d[2 * h + j] = dGg * (1.0f - (gg * gg));
        d[3 * h + j] = (dO * go) * (1.0f - go);
      }
    }
    if (s < steps - 1) orc_gemm(0, 0, batch, h, h4, dG + (size_t)t * batch * h4, h4, whh, h, dh, h, 0);
  }
  if (dx) orc_gemm(0, 0, rows, in_size, h4, dG, h4, wih, in_size, dx, in_size, 0);
  if (dwih) orc_gemm(1, 0, h4, in_size, rows, dG, h4, x, in_size, dwih, in_size, 0);
  if (dwhh) orc_gemm(1, 0, h4, h, rows, dG, h4, hprev, h, dwhh, h, 0);
  if (dbih || dbhh) {
    double* a = (double*)calloc((size_t)h4, sizeof(double));
    for (int i = 0; i < rows; i++)
      for (int c = 0; c < h4; c++) a[c] += dG[(size_t)i * h4 + c];
    for (int c = 0; c < h4; c++) {
      if (dbih) dbih[c] = (float)a[c];
      if (dbhh) dbhh[c] = (float)a[c];
    }
    free(a);
  }
  free(dG); free(dh); free(dc); free(zeros); free(hprev);
}

/* ---- GRU (Ops.Recurrent.cs:148-260; BackwardRecurrent.cs:115-221), PyTorch's formulation, optional initial state --- */
API void orc_gru_fwd(int reverse, int steps, int batch, int in_size, int h, const float* x, const float* wih, const float* whh,
                     const float* bih, const float* bhh, const float* h0, float* y, float* gates, float* hn) {
  int h3 = 3 * h, bh = batch * h;
  float* rec = (float*)malloc(sizeof(float) * (size_t)batch * h3);
  float* zeros = (float*)calloc((size_t)bh, sizeof(float));
  orc_gemm(0, 1, steps * batch, h3, in_size, x, in_size, wih, in_size, gates, h3, 0);
  for (int f = 0; f < steps; f++) {
    int t = reverse ? steps - 1 - f : f, pt = reverse ? t + 1 : t - 1;
    const float* hp = f == 0 ? (h0 ? h0 : zeros) : y + (size_t)pt * bh;
    orc_gemm(0, 1, batch, h3, h, hp, h, whh, h, rec, h3, 0);
    for (int b = 0; b < batch; b++) {
      float* g = gates + ((size_t)t * batch + b) * h3;
      float* rr = rec + (size_t)b * h3;
      if (bih) for (int i = 0; i < h3; i++) g[i] = g[i] + bih[i];
      if (bhh) for (int i = 0; i < h3; i++) rr[i] = rr[i] + bhh[i];
      for (int i = 0; i < 2 * h; i++) g[i] = sigm(g[i] + rr[i]);
      float* hside = hn + ((size_t)t * batch + b) * h;
      for (int j = 0; j < h; j++) hside[j] = rr[2 * h + j];
      for (int j = 0; j < h; j++) {
        float prod = g[j] * hside[j];
        g[2 * h + j] = tanhf(g[2 * h + j] + prod);
      }
      float* ho = y + ((size_t)t * batch + b) * h;
      for (int j = 0; j < h; j++) {
        float z = g[h + j];
        float keep = (1.0f - z) * g[2 * h + j];
        float carry = z * hp[b * h + j];
        ho[j] = keep + carry;
      }
    }
  }
  free(rec);
  free(zeros);
}

API void orc_gru_bwd(int reverse, int steps, int batch, int in_size, int h, const float* gy, const float* x, const float* y,
                     const float* wih, const float* whh, const float* h0, const float* gates, const float* hn, float* dx,
                     float* dwih, float* dwhh, float* dbih, float* dbhh, float* dh0) {
  int h3 = 3 * h, bh = batch * h, rows = steps * batch;
  float* dX = (float*)malloc(sizeof(float) * (size_t)rows * h3);
  float* dH = (float*)malloc(sizeof(float) * (size_t)rows * h3);
  float* dn = (float*)calloc((size_t)bh, sizeof(float));
  float* direct = (float*)malloc(sizeof(float) * (size_t)bh);
  float* zeros = (float*)calloc((size_t)bh, sizeof(float));
  float* hprev = (float*)malloc(sizeof(float) * (size_t)rows * h);
  for (int s = 0; s < steps; s++) {
    int t = reverse ? s : steps - 1 - s, pt = reverse ? t + 1 : t - 1;
    int first = reverse ? t == steps - 1 : t == 0;
    const float* hpv = first ? (h0 ? h0 : zeros) : y + (size_t)pt * bh;
    memcpy(hprev + (size_t)t * bh, hpv, sizeof(float) * bh);
    for (int b = 0; b < batch; b++) {
      size_t row = (size_t)t * batch + b;
      const float* g = gates + row * h3;
      float* dxr = dX + row * h3;
      float* dhr = dH + row * h3;
      for (int j = 0; j < h; j++) {
        int k = b * h + j;
        float rg = g[j], zg = g[h + j], ng = g[2 * h + j];
        float dHt = gy[row * h + j] + dn[k];
        float dz = dHt * (hpv[k] - ng);
        float dNew = dHt * (1.0f - zg);
        direct[k] = dHt * zg;
        float dan = dNew * (1.0f - (ng * ng));
        float drg = dan * hn[row * h + j];
        float dar = (drg * rg) * (1.0f - rg);
        float daz = (dz * zg) * (1.0f - zg);
        dxr[j] = dar; dxr[h + j] = daz; dxr[2 * h + j] = dan;
        dhr[j] = dar; dhr[h + j] = daz; dhr[2 * h + j] = dan * rg;
      }
    }
    orc_gemm(0, 0, batch, h, h3, dH + (size_t)t * batch * h3, h3, whh, h, dn, h, 0);
    for (int i = 0; i < bh; i++) dn[i] += direct[i];
  }
  if (dx) orc_gemm(0, 0, rows, in_size, h3, dX, h3, wih, in_size, dx, in_size, 0);
  if (dwih) orc_gemm(1, 0, h3, in_size, rows, dX, h3, x, in_size, dwih, in_size, 0);
  if (dwhh) orc_gemm(1, 0, h3, h, rows, dH, h3, hprev, h, dwhh, h, 0);
  for (int which = 0; which < 2; which++) {
    float* out = which ? dbhh : dbih;
    const float* src = which ? dH : dX;
    if (!out) continue;
    double* a = (double*)calloc((size_t)h3, sizeof(double));
    for (int i = 0; i < rows; i++)
      for (int c = 0; c < h3; c++) a[c] += src[(size_t)i * h3 + c];
    for (int c = 0; c < h3; c++) out[c] = (float)a[c];
    free(a);
  }
  if (dh0) memcpy(dh0, dn, sizeof(float) * bh);
  free(dX); free(dH); free(dn); free(direct); free(zeros); free(hprev);
}

/* ---- CTC (src/OneModel/Tensors/CtcLoss.cs:170-281; Ctc.cs:515-616) ----------------------------------------------------- */
static double ctc_exp(double x) {
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
  int64_t bits = (int64_t)((int)k + 1023) << 52;
  double scale;
  memcpy(&scale, &bits, 8);
  return p * scale;
}
static double ctc_log(double x) {
  if (x == 0.0) return -INFINITY;
  if (!(x > 0.0) || isinf(x)) return x;
  int64_t bits;
  memcpy(&bits, &x, 8);
  int e = (int)((bits >> 52) & 0x7FF);
  if (e == 0) {
    double xs = x * 18014398509481984.0;
    memcpy(&bits, &xs, 8);
    e = (int)((bits >> 52) & 0x7FF) - 54;
  }
  e -= 1023;
  int64_t mb = (bits & 0x000FFFFFFFFFFFFFLL) | 0x3FF0000000000000LL;
  double m;
  memcpy(&m, &mb, 8);
  if (m > 1.4142135623730951) {
    m *= 0.5;
    e++;
  }
  double s = (m - 1.0) / (m + 1.0), z = s * s, q = 1.0 / 19.0;
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
static double logadd(double a, double b) {
  if (a < b) { double t = a; a = b; b = t; }
  if (isinf(b) && b < 0) return a;
  double d = b - a;
  return d < -40.0 ? a : a + ctc_log(1.0 + ctc_exp(d));
}
static int label_at(const int32_t* tgt, int blank, int s) { return (s & 1) == 0 ? blank : tgt[s >> 1]; }
static int can_skip(const int32_t* tgt, int s) { return s >= 2 && (s & 1) == 1 && tgt[s >> 1] != tgt[(s >> 1) - 1]; }

static double ctc_alpha(const float* lp, int batch, int classes, int b, int len, const int32_t* tgt, int tl, int blank, double* alpha) {
  int ext = 2 * tl + 1;
  if (len == 0) return tl == 0 ? 0.0 : INFINITY;
  for (int t = 0; t < len; t++)
    for (int s = 0; s < ext; s++) {
      double a;
      if (t == 0) a = s <= 1 ? 0.0 : -INFINITY;
      else {
        a = alpha[(size_t)(t - 1) * ext + s];
        if (s >= 1) a = logadd(a, alpha[(size_t)(t - 1) * ext + s - 1]);
        if (can_skip(tgt, s)) a = logadd(a, alpha[(size_t)(t - 1) * ext + s - 2]);
      }
      alpha[(size_t)t * ext + s] = (isinf(a) && a < 0) ? -INFINITY : a + lp[((size_t)t * batch + b) * classes + label_at(tgt, blank, s)];
    }
  double p = alpha[(size_t)(len - 1) * ext + ext - 1];
  if (ext >= 2) p = logadd(p, alpha[(size_t)(len - 1) * ext + ext - 2]);
  return (isinf(p) && p < 0) ? INFINITY : -p;
}

/* Ops.CtcLoss: per-sequence nll (double out) and the reduced loss. reduction 0 none, 1 mean, 2 sum. */
API void orc_ctc_loss(const float* lp, int steps, int batch, int classes, const int32_t* targets, const int32_t* tlen, const int32_t* ilen,
                      int blank, int reduction, int zero_inf, float* nll_out, float* loss) {
  int max_s = 1;
  for (int b = 0; b < batch; b++) if (2 * tlen[b] + 1 > max_s) max_s = 2 * tlen[b] + 1;
  double* alpha = (double*)malloc(sizeof(double) * (size_t)(steps > 0 ? steps : 1) * max_s);
  double sum = 0;
  int off = 0;
  for (int b = 0; b < batch; b++) {
    double nll = ctc_alpha(lp, batch, classes, b, ilen[b], targets + off, tlen[b], blank, alpha);
    off += tlen[b];
    double per = (isinf(nll) && zero_inf) ? 0.0 : nll;
    nll_out[b] = (float)per;
    sum += reduction == 1 ? per / (tlen[b] > 1 ? tlen[b] : 1) : per;
  }
  if (loss) *loss = (float)(reduction == 1 ? sum / batch : sum);
  free(alpha);
}

/* CtcBackward + CtcLossMath.Gradient. g is [B] for reduction none, one value otherwise. */
API void orc_ctc_grad(const float* g, const float* lp, int steps, int batch, int classes, const int32_t* targets, const int32_t* tlen,
                      const int32_t* ilen, int blank, int reduction, float* grad) {
  int max_s = 1;
  for (int b = 0; b < batch; b++) if (2 * tlen[b] + 1 > max_s) max_s = 2 * tlen[b] + 1;
  size_t an = (size_t)(steps > 0 ? steps : 1) * max_s;
  double* alpha = (double*)malloc(sizeof(double) * an);
  double* beta = (double*)malloc(sizeof(double) * an);
  double* acc = (double*)malloc(sizeof(double) * (size_t)classes);
  memset(grad, 0, sizeof(float) * (size_t)steps * batch * classes);
  int off = 0;
  for (int b = 0; b < batch; b++) {
    const int32_t* tgt = targets + off;
    int tl = tlen[b], len = ilen[b], ext = 2 * tl + 1;
    off += tl;
    double scale = reduction == 0 ? g[b] : g[0];
    if (reduction == 1) scale = scale / (tl > 1 ? tl : 1) / batch;
    double nll = ctc_alpha(lp, batch, classes, b, len, tgt, tl, blank, alpha);
    if (len == 0 || isinf(nll)) continue;
    for (int t = len - 1; t >= 0; t--) {
      for (int s = ext - 1; s >= 0; s--) {
        double v;
        if (t == len - 1) v = s >= ext - 2 ? 0.0 : -INFINITY;
        else {
          v = beta[(size_t)(t + 1) * ext + s];
          if (s + 1 < ext) v = logadd(v, beta[(size_t)(t + 1) * ext + s + 1]);
          if (s + 2 < ext && can_skip(tgt, s + 2)) v = logadd(v, beta[(size_t)(t + 1) * ext + s + 2]);
        }
        beta[(size_t)t * ext + s] = (isinf(v) && v < 0) ? -INFINITY : v + lp[((size_t)t * batch + b) * classes + label_at(tgt, blank, s)];
      }
      for (int c = 0; c < classes; c++) acc[c] = -INFINITY;
      for (int s = 0; s < ext; s++) {
        double ab = alpha[(size_t)t * ext + s] + beta[(size_t)t * ext + s];
        if (!(isinf(ab) && ab < 0) && !isnan(ab)) {
          int cls = label_at(tgt, blank, s);
          acc[cls] = logadd(acc[cls], ab);
        }
      }
      for (int c = 0; c < classes; c++) {
        if (isinf(acc[c]) && acc[c] < 0) continue;
        double l = lp[((size_t)t * batch + b) * classes + c];
        grad[((size_t)t * batch + b) * classes + c] += (float)(-scale * ctc_exp(acc[c] - l + nll));
      }
    }
  }
  free(alpha); free(beta); free(acc);
}

/* Ctc.Greedy (src/OneModel/Tensors/Ctc.cs:89-190): argmax per step with `>` (ties to the lower index; a NaN best is
 * replaced by the next value), runs merged, blanks dropped; label, first and last step of every kept run.
 * labels/first/last are [B, T] padded with -1. */
API void orc_ctc_greedy(const float* lp, int steps, int batch, int classes, const int32_t* ilen, int blank, int32_t* labels,
                        int32_t* first_step, int32_t* last_step, int32_t* lengths) {
  for (int b = 0; b < batch; b++) {
    int len = ilen ? ilen[b] : steps, count = 0, last = blank, first = 0;
    for (int t = 0; t < len; t++) {
      const float* row = lp + ((size_t)t * batch + b) * classes;
      int best = 0;
      float bv = row[0];
      for (int c = 1; c < classes; c++)
        if (row[c] > bv || isnan(bv)) { bv = row[c]; best = c; }
      if (best != last) {
        if (last != blank) {
          labels[(size_t)b * steps + count] = last;
          first_step[(size_t)b * steps + count] = first;
          last_step[(size_t)b * steps + count] = t - 1;
          count++;
        }
        if (best != blank) first = t;
      }
      last = best;
    }
    if (last != blank && len > 0) {
      labels[(size_t)b * steps + count] = last;
      first_step[(size_t)b * steps + count] = first;
      last_step[(size_t)b * steps + count] = len - 1;
      count++;
    }
    for (int i = count; i < steps; i++) labels[(size_t)b * steps + i] = first_step[(size_t)b * steps + i] = last_step[(size_t)b * steps + i] = -1;
    lengths[b] = count;
  }
}
