// Layer normalisation (rows) and batch normalisation (NCHW channels), forward and backward. Bandwidth-bound:
// every kernel streams its operands once with coalesced 128-byte warp accesses. Statistics that the reference
// accumulates in double (BackwardNn.cs:170-307, Ops.Layers.cs:185-219) are accumulated in double here too, over a
// partition that depends only on the shape and is combined in a fixed order.
#include "om_common.cuh"

namespace om {

__device__ __forceinline__ double wsum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float wsum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- layer norm forward: one warp per row -------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
layernorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                     int32_t rows, int32_t cols, float eps, float* __restrict__ y, float* __restrict__ mean_out,
                     float* __restrict__ inv_out) {
  pdl_enter();
  int lane = threadIdx.x & 31;
  int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  int64_t warps = (int64_t)gridDim.x * 8;
  float n = (float)cols;
  for (int64_t r = warp; r < rows; r += warps) {
    const float* xr = x + r * cols;
    float s = 0.f;
    for (int j = lane; j < cols; j += 32) s += xr[j];
    float mean = wsum_f(s) / n;
    float q = 0.f;
    for (int j = lane; j < cols; j += 32) {
      float d = xr[j] - mean;
      q += d * d;
    }
    float inv = 1.0f / sqrtf((wsum_f(q) / n) + eps);
    if (lane == 0) {
      if (mean_out) mean_out[r] = mean;
      if (inv_out) inv_out[r] = inv;
    }
    float* yr = y + r * cols;
    for (int j = lane; j < cols; j += 32) yr[j] = (((xr[j] - mean) * inv) * gamma[j]) + beta[j];
  }
}

// ---- layer norm backward -------------------------------------------------------------------------------------------
// dx: a warp per row, the row in registers (NC columns per lane), the two row sums in double
// (LayerNormBackward, BackwardNn.cs:170-242 of the reference). CTA = 8 warps owns kLnRowsPerCta consecutive rows.
constexpr int kLnRowsPerCta = 16;   // two rows per warp: 512 CTAs for 8192 rows keep enough loads in flight

template <int NC>
__global__ void __launch_bounds__(256)
layernorm_bwd_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ gamma,
                     const float* __restrict__ mean, const float* __restrict__ inv, int32_t rows, int32_t cols,
                     float* __restrict__ dx) {
  pdl_enter();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int r0 = blockIdx.x * kLnRowsPerCta;
  const int r1 = min(rows, r0 + kLnRowsPerCta);
  float gam[NC];
#pragma unroll
  for (int i = 0; i < NC; i++) {
    int j = lane + 32 * i;
    gam[i] = j < cols ? gamma[j] : 0.f;
  }
  for (int r = r0 + w; r < r1; r += 8) {
    const float* xr = x + (int64_t)r * cols;
    const float* gr = g + (int64_t)r * cols;
    const float m = mean[r], s = inv[r];
    float xh[NC], dh[NC];
#pragma unroll
    for (int i = 0; i < NC; i++) {
      int j = lane + 32 * i;
      const bool in = j < cols;
      const float gv = in ? gr[j] : 0.f;
      const float xv = in ? xr[j] : m;
      xh[i] = (xv - m) * s;
      dh[i] = gv * gam[i];
    }
    double sum1 = 0.0, sum2 = 0.0;
#pragma unroll
    for (int i = 0; i < NC; i++) {
      if (lane + 32 * i < cols) {
        sum1 += (double)dh[i];
        sum2 += (double)(dh[i] * xh[i]);
      }
    }
    sum1 = wsum_d(sum1);
    sum2 = wsum_d(sum2);
    const float m1 = (float)(sum1 / cols), m2 = (float)(sum2 / cols);
    float* dr = dx + (int64_t)r * cols;
#pragma unroll
    for (int i = 0; i < NC; i++) {
      int j = lane + 32 * i;
      if (j < cols) dr[j] = s * ((dh[i] - m1) - (xh[i] * m2));
    }
  }
}

// Column partials of the layer-norm parameter gradients: dgamma[j] = sum_r g[r,j] * xhat[r,j], dbeta[j] = sum_r g[r,j].
// CTA (bx, by) owns 32 columns and one chunk of 512 rows: 8 column groups x 32 row lanes, a thread holds four adjacent
// columns (16-byte loads) and 16 rows, all loads of a row pair in flight together; lanes are combined in lane order.
constexpr int kLnParamRows = 512;
__global__ void __launch_bounds__(256)
layernorm_param_partials_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ mean,
                                const float* __restrict__ inv, int32_t rows, int32_t cols, double* __restrict__ part_gamma,
                                double* __restrict__ part_beta) {
  pdl_enter();
  __shared__ double sg[32][33], sb[32][33];
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  const int col = blockIdx.x * 32 + tx * 4;
  const int r0 = blockIdx.y * kLnParamRows, r1 = min(rows, r0 + kLnParamRows);
  double ag[4] = {0.0, 0.0, 0.0, 0.0}, ab[4] = {0.0, 0.0, 0.0, 0.0};
  const bool vec = (cols & 3) == 0 && col + 3 < cols;
  for (int r = r0 + ty; r < r1; r += 64) {
    const int r2 = r + 32;
    float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), xa = ga, gb = ga, xb = ga;
    float ma = 0.f, sa = 0.f, mb = 0.f, sbv = 0.f;
    if (vec) {
      ga = __ldg(reinterpret_cast<const float4*>(g + (int64_t)r * cols + col));
      xa = __ldg(reinterpret_cast<const float4*>(x + (int64_t)r * cols + col));
      ma = mean[r]; sa = inv[r];
      if (r2 < r1) {
        gb = __ldg(reinterpret_cast<const float4*>(g + (int64_t)r2 * cols + col));
        xb = __ldg(reinterpret_cast<const float4*>(x + (int64_t)r2 * cols + col));
        mb = mean[r2]; sbv = inv[r2];
      }
    } else {
      float* gp[2] = {&ga.x, &gb.x};
      float* xp[2] = {&xa.x, &xb.x};
      for (int q = 0; q < 2; q++) {
        const int rr = q ? r2 : r;
        if (rr >= r1) continue;
        for (int c = 0; c < 4; c++)
          if (col + c < cols) {
            gp[q][c] = g[(int64_t)rr * cols + col + c];
            xp[q][c] = x[(int64_t)rr * cols + col + c];
          }
        if (q) { mb = mean[rr]; sbv = inv[rr]; } else { ma = mean[rr]; sa = inv[rr]; }
      }
    }
    ag[0] += (double)(ga.x * ((xa.x - ma) * sa)); ab[0] += (double)ga.x;
    ag[1] += (double)(ga.y * ((xa.y - ma) * sa)); ab[1] += (double)ga.y;
    ag[2] += (double)(ga.z * ((xa.z - ma) * sa)); ab[2] += (double)ga.z;
    ag[3] += (double)(ga.w * ((xa.w - ma) * sa)); ab[3] += (double)ga.w;
    if (r2 < r1) {
      ag[0] += (double)(gb.x * ((xb.x - mb) * sbv)); ab[0] += (double)gb.x;
      ag[1] += (double)(gb.y * ((xb.y - mb) * sbv)); ab[1] += (double)gb.y;
      ag[2] += (double)(gb.z * ((xb.z - mb) * sbv)); ab[2] += (double)gb.z;
      ag[3] += (double)(gb.w * ((xb.w - mb) * sbv)); ab[3] += (double)gb.w;
    }
  }
#pragma unroll
  for (int c = 0; c < 4; c++) {
    sg[ty][tx * 4 + c] = ag[c];
    sb[ty][tx * 4 + c] = ab[c];
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int c = blockIdx.x * 32 + threadIdx.x;
    if (c < cols) {
      double tg = 0.0, tb = 0.0;
#pragma unroll
      for (int l = 0; l < 32; l++) {
        tg += sg[l][threadIdx.x];
        tb += sb[l][threadIdx.x];
      }
      if (part_gamma) part_gamma[(int64_t)blockIdx.y * cols + c] = tg;
      if (part_beta) part_beta[(int64_t)blockIdx.y * cols + c] = tb;
    }
  }
}

// out[j] = sum over chunks of partial[chunk, j] for one or two tables of double partials. A CTA owns 32 columns; 16
// chunk lanes each add chunks lane, lane + 16, ... in increasing order, then the lane sums are added in lane order: a
// fixed order, so the result does not depend on the launch.
__global__ void __launch_bounds__(512)
column_partials_finish_kernel(const double* __restrict__ pa, const double* __restrict__ pb, int chunks, int32_t cols,
                              float* __restrict__ oa, float* __restrict__ ob, int accumulate) {
  pdl_enter();
  __shared__ double sa[16][33], sb[16][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + tx;
  double ta = 0.0, tb = 0.0;
  if (j < cols) {
    // Eight loads are issued before the first add: the adds stay in increasing chunk order.
    if (pa && oa) {
#pragma unroll 8
      for (int c = ty; c < chunks; c += 16) ta += pa[(int64_t)c * cols + j];
    }
    if (pb && ob) {
#pragma unroll 8
      for (int c = ty; c < chunks; c += 16) tb += pb[(int64_t)c * cols + j];
    }
  }
  sa[ty][tx] = ta;
  sb[ty][tx] = tb;
  __syncthreads();
  if (ty == 0 && j < cols) {
    if (pa && oa) {
      double t = 0.0;
#pragma unroll
      for (int l = 0; l < 16; l++) t += sa[l][tx];
      oa[j] = accumulate ? oa[j] + (float)t : (float)t;
    }
    if (pb && ob) {
      double t = 0.0;
#pragma unroll
      for (int l = 0; l < 16; l++) t += sb[l][tx];
      ob[j] = accumulate ? ob[j] + (float)t : (float)t;
    }
  }
}

// ---- batch norm ------------------------------------------------------------------------------------------------------
// Channel statistics: CTA (ch, slice) sums the planes of images [slice*ipc, (slice+1)*ipc) of channel ch. MODE 0: sum x.
// MODE 1: sum (x - mu64)^2. MODE 2 (backward): sum g*xhat and sum g.
constexpr int kBnThreads = 256;

template <int MODE>
__global__ void __launch_bounds__(kBnThreads)
bn_partial_kernel(const float* __restrict__ x, const float* __restrict__ g, const double* __restrict__ mu64,
                  const float* __restrict__ mean, const float* __restrict__ inv, int32_t n, int32_t c, int32_t plane,
                  int32_t ipc, double* __restrict__ pa, double* __restrict__ pb) {
  __shared__ double sa[kBnThreads / 32], sb[kBnThreads / 32];
  const int ch = blockIdx.x, slice = blockIdx.y;
  const int i0 = slice * ipc, i1 = min(n, i0 + ipc);
  double a = 0.0, b = 0.0;
  double mu = MODE == 1 ? mu64[ch] : 0.0;
  float mm = MODE == 2 ? mean[ch] : 0.f, s = MODE == 2 ? inv[ch] : 0.f;
  // The slice's planes as one index space; with a plane that is a multiple of four a thread reads 16 bytes at a time.
  const int64_t span = (int64_t)(i1 - i0) * plane;
  auto term = [&](float xv, float gv) {
    if (MODE == 0) {
      a += (double)xv;
    } else if (MODE == 1) {
      double d = (double)xv - mu;
      a += d * d;
    } else {
      a += (double)(gv * ((xv - mm) * s));
      b += (double)gv;
    }
  };
  if ((plane & 3) == 0) {
    for (int64_t e = (int64_t)threadIdx.x * 4; e < span; e += kBnThreads * 4) {
      const int i = i0 + (int)(e / plane);
      const int64_t o = ((int64_t)i * c + ch) * plane + (e % plane);
      const float4 xv = __ldg(reinterpret_cast<const float4*>(x + o));
      float4 gv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (MODE == 2) gv = __ldg(reinterpret_cast<const float4*>(g + o));
      term(xv.x, gv.x); term(xv.y, gv.y); term(xv.z, gv.z); term(xv.w, gv.w);
    }
  } else {
    for (int64_t e = threadIdx.x; e < span; e += kBnThreads) {
      const int i = i0 + (int)(e / plane);
      const int64_t o = ((int64_t)i * c + ch) * plane + (e % plane);
      term(x[o], MODE == 2 ? g[o] : 0.f);
    }
  }
  a = wsum_d(a);
  if (MODE == 2) b = wsum_d(b);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) {
    sa[w] = a;
    sb[w] = b;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double ta = 0.0, tb = 0.0;
#pragma unroll
    for (int k = 0; k < kBnThreads / 32; k++) {
      ta += sa[k];
      tb += sb[k];
    }
    pa[(int64_t)slice * c + ch] = ta;
    if (MODE == 2) pb[(int64_t)slice * c + ch] = tb;
  }
}

__global__ void bn_mean_kernel(const double* __restrict__ pa, int slices, int32_t c, double m, double* __restrict__ mu64) {
  int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  double t = 0.0;
  for (int s = 0; s < slices; s++) t += pa[(int64_t)s * c + ch];
  mu64[ch] = t / m;
}

__global__ void bn_finish_stats_kernel(const double* __restrict__ pa, const double* __restrict__ mu64, int slices,
                                       int32_t c, double m, float momentum, float eps, float* __restrict__ mean,
                                       float* __restrict__ inv, float* __restrict__ rm, float* __restrict__ rv) {
  int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  double ss = 0.0;
  for (int s = 0; s < slices; s++) ss += pa[(int64_t)s * c + ch];
  double var = ss / m;
  double mu = mu64[ch];
  mean[ch] = (float)mu;
  inv[ch] = 1.0f / sqrtf((float)var + eps);
  double unbiased = m > 1 ? var * m / (m - 1) : var;
  // (1 - momentum) is float arithmetic promoted to double in the reference: ((1 - momentum) * rm) + (momentum * mu64).
  float keep = 1 - momentum;
  rm[ch] = (float)(((double)(keep * rm[ch])) + ((double)momentum * mu));
  rv[ch] = (float)(((double)(keep * rv[ch])) + ((double)momentum * unbiased));
}

__global__ void bn_eval_stats_kernel(const float* __restrict__ rm, const float* __restrict__ rv, int32_t c, float eps,
                                     float* __restrict__ mean, float* __restrict__ inv) {
  int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  mean[ch] = rm[ch];
  inv[ch] = 1.0f / sqrtf(rv[ch] + eps);
}

// Element-wise over the whole tensor, VEC consecutive elements of one plane per thread (VEC == 4: plane % 4 == 0).
template <int VEC>
__global__ void __launch_bounds__(256)
bn_apply_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                const float* __restrict__ mean, const float* __restrict__ inv, int64_t total, int32_t c, int32_t plane,
                float* __restrict__ y) {
  int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * VEC;
  int64_t stride = (int64_t)gridDim.x * blockDim.x * VEC;
  for (int64_t e = i; e < total; e += stride) {
    const int ch = (int)((e / plane) % c);
    const float mm = mean[ch], s = inv[ch], gg = gamma[ch], bb = beta[ch];
    if (VEC == 4) {
      float4 v = __ldg(reinterpret_cast<const float4*>(x + e));
      v.x = (((v.x - mm) * s) * gg) + bb; v.y = (((v.y - mm) * s) * gg) + bb;
      v.z = (((v.z - mm) * s) * gg) + bb; v.w = (((v.w - mm) * s) * gg) + bb;
      *reinterpret_cast<float4*>(y + e) = v;
    } else {
      y[e] = (((x[e] - mm) * s) * gg) + bb;
    }
  }
}

// Per-channel scalars of the backward: k = gamma * inv, cb = mean(g), cg = mean(g * xhat), from the slice partials.
__global__ void bn_bwd_coef_kernel(const float* __restrict__ gamma, const float* __restrict__ inv, const double* __restrict__ pa,
                                   const double* __restrict__ pb, int slices, double m, int32_t c, float* __restrict__ coef) {
  int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  double sg = 0.0, sb = 0.0;
  for (int s = 0; s < slices; s++) {
    sg += pa[(int64_t)s * c + ch];
    sb += pb[(int64_t)s * c + ch];
  }
  coef[ch] = gamma[ch] * inv[ch];
  coef[c + ch] = (float)(sb / m);
  coef[2 * c + ch] = (float)(sg / m);
}

template <int VEC>
__global__ void __launch_bounds__(256)
bn_bwd_apply_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ mean,
                    const float* __restrict__ inv, const float* __restrict__ coef, int64_t total, int32_t c, int32_t plane,
                    int training, float* __restrict__ dx) {
  int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * VEC;
  int64_t stride = (int64_t)gridDim.x * blockDim.x * VEC;
  for (int64_t e = i; e < total; e += stride) {
    const int ch = (int)((e / plane) % c);
    const float mm = mean[ch], s = inv[ch], k = coef[ch], cb = coef[c + ch], cg = coef[2 * c + ch];
    if (VEC == 4) {
      const float4 gv = __ldg(reinterpret_cast<const float4*>(g + e));
      const float4 xv = __ldg(reinterpret_cast<const float4*>(x + e));
      float4 o;
      if (training) {
        o.x = k * ((gv.x - cb) - (((xv.x - mm) * s) * cg)); o.y = k * ((gv.y - cb) - (((xv.y - mm) * s) * cg));
        o.z = k * ((gv.z - cb) - (((xv.z - mm) * s) * cg)); o.w = k * ((gv.w - cb) - (((xv.w - mm) * s) * cg));
      } else {
        o.x = k * gv.x; o.y = k * gv.y; o.z = k * gv.z; o.w = k * gv.w;
      }
      *reinterpret_cast<float4*>(dx + e) = o;
    } else {
      dx[e] = training ? k * ((g[e] - cb) - (((x[e] - mm) * s) * cg)) : k * g[e];
    }
  }
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_layernorm_fwd(om_ctx* ctx, const float* x, const float* gamma, const float* beta, int32_t rows, int32_t cols,
                         float eps, float* y, float* mean, float* inv) {
  OM_CHECK_CTX(ctx);
  if (rows < 0 || cols < 0) return fail(ctx, OM_ERR_SHAPE, "om_layernorm_fwd: [%d,%d]", rows, cols);
  if (rows == 0 || cols == 0) return OM_OK;
  ProfileScope prof(ctx, "om_layernorm_fwd", 0, 8.0 * rows * (double)cols);
  int grid = (int)std::min<int64_t>(ceil_div(rows, 8), (int64_t)ctx->sm_count * 8);
  launch_chained(ctx, layernorm_fwd_kernel, grid, 256, 0, x, gamma, beta, rows, cols, eps, y, mean, inv);
  OM_LAUNCH_CHECK(ctx, "om_layernorm_fwd");
  return OM_OK;
}

int32_t om_layernorm_bwd(om_ctx* ctx, const float* g, const float* x, const float* gamma, const float* mean,
                         const float* inv, int32_t rows, int32_t cols, float* dx, float* dgamma, float* dbeta,
                         int32_t accumulate_params) {
  OM_CHECK_CTX(ctx);
  if (rows < 0 || cols < 0) return fail(ctx, OM_ERR_SHAPE, "om_layernorm_bwd: [%d,%d]", rows, cols);
  if (cols == 0) return OM_OK;
  if (cols > 1024) return fail(ctx, OM_ERR_UNSUPPORTED, "om_layernorm_bwd: rows wider than 1024 (%d) are not implemented", cols);
  ProfileScope prof(ctx, "om_layernorm_bwd", 0, 12.0 * rows * (double)cols);
  // dx: a warp per row, the row in registers. The parameter gradients are column sums and run as their own pass over
  // (g, x) with the column-sum blocking: for wide rows that beats carrying per-lane column partials through the row loop.
  const int row_ctas = (int)ceil_div(rows > 0 ? rows : 1, kLnRowsPerCta);
  int nc = (int)ceil_div(cols, 32);
  if (dx && rows > 0) {
#define OM_LN_BWD(NC) launch_chained(ctx, layernorm_bwd_kernel<NC>, row_ctas, 256, 0, g, x, gamma, mean, inv, rows, cols, dx)
    if (nc <= 4) OM_LN_BWD(4);
    else if (nc <= 8) OM_LN_BWD(8);
    else if (nc <= 12) OM_LN_BWD(12);
    else if (nc <= 16) OM_LN_BWD(16);
    else if (nc <= 24) OM_LN_BWD(24);
    else OM_LN_BWD(32);
#undef OM_LN_BWD
  }
  double *pg = nullptr, *pb = nullptr;
  if (dgamma || dbeta) {
    const int chunks = (int)ceil_div(rows > 0 ? rows : 1, kLnParamRows);
    if (dgamma) OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)chunks * cols, false, (void**)&pg));
    if (dbeta) OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)chunks * cols, false, (void**)&pb));
    launch_chained(ctx, layernorm_param_partials_kernel, dim3((unsigned)ceil_div(cols, 32), (unsigned)chunks), 256, 0, g, x, mean, inv, rows, cols, pg, pb);
    launch_chained(ctx, column_partials_finish_kernel, (unsigned)ceil_div(cols, 32), 512, 0, pg, pb, chunks, cols, dgamma, dbeta, accumulate_params);
  }
  if (pg) pool_free(ctx, pg);
  if (pb) pool_free(ctx, pb);
  OM_LAUNCH_CHECK(ctx, "om_layernorm_bwd");
  return OM_OK;
}

static int bn_slices(int n) { return n < 16 ? (n > 0 ? n : 1) : 16; }

int32_t om_batchnorm_fwd(om_ctx* ctx, const float* x, const float* gamma, const float* beta, float* running_mean,
                         float* running_var, int32_t n, int32_t c, int32_t plane, int32_t training, float momentum,
                         float eps, float* y, float* mean, float* inv) {
  OM_CHECK_CTX(ctx);
  if (n < 0 || c < 0 || plane < 0) return fail(ctx, OM_ERR_SHAPE, "om_batchnorm_fwd: n %d c %d plane %d", n, c, plane);
  if (training && (int64_t)n * plane < 1) return fail(ctx, OM_ERR_SHAPE, "BatchNorm2d in training needs at least one value per channel.");
  if (c == 0) return OM_OK;
  double total = (double)n * c * plane;
  ProfileScope prof(ctx, "om_batchnorm_fwd", 0, (training ? 16.0 : 8.0) * total);
  if (training) {
    int slices = bn_slices(n), ipc = (int)ceil_div(n, slices);
    double *pa = nullptr, *mu64 = nullptr;
    OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)slices * c, false, (void**)&pa));
    OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)c, false, (void**)&mu64));
    double m = (double)n * plane;
    dim3 grid(c, slices);
    bn_partial_kernel<0><<<grid, kBnThreads, 0, ctx->stream>>>(x, nullptr, nullptr, nullptr, nullptr, n, c, plane, ipc, pa, nullptr);
    bn_mean_kernel<<<(unsigned)ceil_div(c, 128), 128, 0, ctx->stream>>>(pa, slices, c, m, mu64);
    bn_partial_kernel<1><<<grid, kBnThreads, 0, ctx->stream>>>(x, nullptr, mu64, nullptr, nullptr, n, c, plane, ipc, pa, nullptr);
    bn_finish_stats_kernel<<<(unsigned)ceil_div(c, 128), 128, 0, ctx->stream>>>(pa, mu64, slices, c, m, momentum, eps, mean, inv, running_mean, running_var);
    pool_free(ctx, pa);
    pool_free(ctx, mu64);
  } else {
    bn_eval_stats_kernel<<<(unsigned)ceil_div(c, 128), 128, 0, ctx->stream>>>(running_mean, running_var, c, eps, mean, inv);
  }
  int64_t planes = (int64_t)n * c;
  if (planes > 0 && plane > 0) {
    const int64_t total = planes * plane;
    if ((plane & 3) == 0) bn_apply_kernel<4><<<grid_for(ctx, total / 4, 256), 256, 0, ctx->stream>>>(x, gamma, beta, mean, inv, total, c, plane, y);
    else bn_apply_kernel<1><<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(x, gamma, beta, mean, inv, total, c, plane, y);
  }
  OM_LAUNCH_CHECK(ctx, "om_batchnorm_fwd");
  return OM_OK;
}

int32_t om_batchnorm_bwd(om_ctx* ctx, const float* g, const float* x, const float* gamma, const float* mean,
                         const float* inv, int32_t n, int32_t c, int32_t plane, int32_t training, float* dx,
                         float* dgamma, float* dbeta, int32_t accumulate_params) {
  OM_CHECK_CTX(ctx);
  if (n < 0 || c < 0 || plane < 0) return fail(ctx, OM_ERR_SHAPE, "om_batchnorm_bwd: n %d c %d plane %d", n, c, plane);
  if (c == 0) return OM_OK;
  double total = (double)n * c * plane;
  ProfileScope prof(ctx, "om_batchnorm_bwd", 0, 20.0 * total);
  int slices = bn_slices(n), ipc = (int)ceil_div(n > 0 ? n : 1, slices);
  double *pa = nullptr, *pb = nullptr;
  OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)slices * c, false, (void**)&pa));
  OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)slices * c, false, (void**)&pb));
  bn_partial_kernel<2><<<dim3(c, slices), kBnThreads, 0, ctx->stream>>>(x, g, nullptr, mean, inv, n, c, plane, ipc, pa, pb);
  int64_t planes = (int64_t)n * c;
  if (dx && planes > 0 && plane > 0) {
    float* coef = nullptr;
    OM_TRY(pool_alloc(ctx, sizeof(float) * 3 * (size_t)c, false, (void**)&coef));
    bn_bwd_coef_kernel<<<(unsigned)ceil_div(c, 128), 128, 0, ctx->stream>>>(gamma, inv, pa, pb, slices, (double)n * plane, c, coef);
    const int64_t total = planes * plane;
    if ((plane & 3) == 0) bn_bwd_apply_kernel<4><<<grid_for(ctx, total / 4, 256), 256, 0, ctx->stream>>>(g, x, mean, inv, coef, total, c, plane, training, dx);
    else bn_bwd_apply_kernel<1><<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(g, x, mean, inv, coef, total, c, plane, training, dx);
    pool_free(ctx, coef);
  }
  if (dgamma || dbeta)
    launch_chained(ctx, column_partials_finish_kernel, (unsigned)ceil_div(c, 32), 512, 0, pa, pb, slices, c, dgamma, dbeta, accumulate_params);
  pool_free(ctx, pa);
  pool_free(ctx, pb);
  OM_LAUNCH_CHECK(ctx, "om_batchnorm_bwd");
  return OM_OK;
}

}  // extern "C"
