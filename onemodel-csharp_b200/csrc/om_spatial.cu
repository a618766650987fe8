// Convolution and pooling, forward and backward, on NCHW tensors.
//
// Convolution follows the data flow of the reference's ConvBackward (BackwardNn.cs:317-462): the input is unfolded
// (im2col) once per call for all images, the products run as strided-batched GEMMs over the images (one launch per
// group, the weight matrix shared by all images), and the input gradient is folded back (col2im) as a GATHER: every
// input element adds the taps that touch it in increasing (ky, kx) order, which is the order of the reference's
// scatter loop, so no atomics are needed. The weight gradient sums over images inside the kernel (fixed chunks of
// images per CTA, partials combined in chunk order).
//
// With OM_TF32 set (and one group, TMA-describable pitches) the three products instead run on the tensor pipe as ONE
// product each over all images: the unfolded input is laid out [K, N*P] (K = Cin*KH*KW taps, P = OH*OW pixels), the
// output gradient is brought from [N, Cout, P] to [Cout, N*P], and
//   forward  y_t [Cout, N*P] = W [Cout, K] * cols [K, N*P]          (then back to NCHW with the bias in the same pass)
//   dgrad    dcols [K, N*P]  = W^T * g_t [Cout, N*P]                 (then the same col2im gather)
//   wgrad    dW [Cout, K]    = g_t [Cout, N*P] * cols^T              (one product with k = N*P, fixed split of k)
#include "om_common.cuh"

namespace om {

int32_t gemm_simt(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, int64_t sA,
                  const float* B, int ldb, int64_t sB, float* C, int ldc, int64_t sC, int batch, int acc);
int32_t gemm_simt_batch_reduce(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, int64_t sA,
                               const float* B, int ldb, int64_t sB, float* partial, int64_t chunk_stride, int batch,
                               int batch_per_chunk);

bool gemm_tc_supported(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B,
                       int ldb, const float* C, int ldc);
int32_t gemm_tc(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B, int ldb,
                float* C, int ldc, int acc, const float* bias);

struct ConvGeom {
  int n, cin, h, w, cout, kh, kw, sh, sw, pt, pl, dh, dw, groups, oh, ow;
};

static bool conv_geom(const om_conv_shape* s, ConvGeom* g) {
  g->n = s->n; g->cin = s->cin; g->h = s->h; g->w = s->w; g->cout = s->cout; g->kh = s->kh; g->kw = s->kw;
  g->sh = s->stride_h; g->sw = s->stride_w; g->pt = s->pad_top; g->pl = s->pad_left; g->dh = s->dil_h; g->dw = s->dil_w;
  g->groups = s->groups;
  if (g->n < 0 || g->cin < 1 || g->cout < 1 || g->kh < 1 || g->kw < 1 || g->sh < 1 || g->sw < 1 || g->dh < 1 || g->dw < 1 ||
      g->groups < 1 || g->cin % g->groups || g->cout % g->groups || g->pt < 0 || g->pl < 0 || s->pad_bottom < 0 || s->pad_right < 0)
    return false;
  g->oh = (g->h + g->pt + s->pad_bottom - g->dh * (g->kh - 1) - 1) / g->sh + 1;
  g->ow = (g->w + g->pl + s->pad_right - g->dw * (g->kw - 1) - 1) / g->sw + 1;
  return g->oh >= 1 && g->ow >= 1;
}

// cols[(c*KH+ky)*KW+kx][n][oy*OW+ox] = x[n][c][oy*sh-pt+ky*dh][ox*sw-pl+kx*dw], zero outside the image.
// The element of tap row k, image n, pixel p sits at k * k_stride + n * n_stride + p: (P, K*P) is the per-image layout
// [N][K][P], (N*P, P) the all-images layout [K][N*P]. blockIdx.y is the tap row; a thread owns VEC consecutive pixels
// of one image (VEC == 4 needs P, the strides and the base to be multiples of four: one 16-byte store).
// IDX is the type of the pixel counter: int when N * P fits 31 bits (the 64-bit divisions are most of the kernel otherwise).
template <int VEC, typename IDX>
__global__ void __launch_bounds__(256)
im2col_kernel(ConvGeom g, const float* __restrict__ x, float* __restrict__ cols, int64_t pixels_all, int64_t k_stride, int64_t n_stride) {
  const int plane = g.oh * g.ow;
  const int kidx = blockIdx.y;
  const int kx = kidx % g.kw, ky = (kidx / g.kw) % g.kh, c = kidx / (g.kw * g.kh);
  IDX q0 = (IDX)((blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * VEC);
  const int64_t qstride = (int64_t)gridDim.x * blockDim.x * VEC;
  for (int64_t q64 = q0; q64 < pixels_all; q64 += qstride) {
    const IDX q = (IDX)q64;
    const int n = (int)(q / (IDX)plane);
    const int p = (int)(q - (IDX)n * (IDX)plane);
    const float* xc = x + ((int64_t)n * g.cin + c) * g.h * g.w;
    float v[VEC];
    if (VEC == 4 && (g.ow & 3) == 0) {
      // The four pixels lie in one output row: one division, one input row, four input columns sw apart.
      const int oy = p / g.ow, ox = p - oy * g.ow;
      const int iy = oy * g.sh - g.pt + ky * g.dh;
      const bool row_ok = (unsigned)iy < (unsigned)g.h;
      const float* xr = xc + iy * g.w;
      const int ix0 = ox * g.sw - g.pl + kx * g.dw;
#pragma unroll
      for (int j = 0; j < VEC; j++) {
        const int ix = ix0 + j * g.sw;
        v[j] = (row_ok && (unsigned)ix < (unsigned)g.w) ? __ldg(xr + ix) : 0.f;
      }
    } else {
#pragma unroll
      for (int j = 0; j < VEC; j++) {
        const int pj = p + j;
        const int oy = pj / g.ow, ox = pj - oy * g.ow;
        const int iy = oy * g.sh - g.pt + ky * g.dh, ix = ox * g.sw - g.pl + kx * g.dw;
        v[j] = ((unsigned)iy < (unsigned)g.h && (unsigned)ix < (unsigned)g.w) ? __ldg(xc + iy * g.w + ix) : 0.f;
      }
    }
    float* dst = cols + (int64_t)kidx * k_stride + (int64_t)n * n_stride + p;
    if (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    else dst[0] = v[0];
  }
}

// dx[n][c][iy][ix] = sum over (ky, kx) in increasing order of dcols[(c,ky,kx)][n][oy*OW+ox] where the tap lands on (iy, ix).
// S is the stride when both strides equal it (1 or 2: the divisions become shifts), 0 for the general case.
// PLANES: blockIdx.y = channel, blockIdx.z = image, threads over the input plane (no per-element plane arithmetic: the
// layout for planes of hundreds of elements and more). Otherwise one thread per input element over all images and
// channels: the planes of a deep layer are a few dozen elements, and a CTA per plane would idle most of its threads.
template <int S, bool PLANES>
__global__ void __launch_bounds__(256)
col2im_gather_kernel(ConvGeom g, const float* __restrict__ dcols, float* __restrict__ dx, int64_t k_stride, int64_t n_stride, int total) {
  const int sh = S ? S : g.sh, sw = S ? S : g.sw;
  const int hw = g.h * g.w;
  const int limit = PLANES ? hw : total;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < limit; t += gridDim.x * blockDim.x) {
    int e, n, c;
    if (PLANES) {
      e = t; c = blockIdx.y; n = blockIdx.z;
    } else {
      // Planes in (channel, image) order: for one channel and tap the unfolded matrix holds all images' output pixels
      // next to one another, so the planes a CTA covers read neighbouring segments of the same rows.
      const int pl = t / hw;
      e = t - pl * hw;
      c = pl / g.n;
      n = pl - c * g.n;
    }
    const float* base = dcols + (int64_t)n * n_stride + (int64_t)c * g.kh * g.kw * k_stride;
    const int iy = e / g.w, ix = e - iy * g.w;
    float acc = 0.f;
    for (int ky = 0; ky < g.kh; ky++) {
      int ty = iy + g.pt - ky * g.dh;
      if (ty < 0 || ty % sh) continue;
      int oy = ty / sh;
      if (oy >= g.oh) continue;
      for (int kx = 0; kx < g.kw; kx++) {
        int tx = ix + g.pl - kx * g.dw;
        if (tx < 0 || tx % sw) continue;
        int ox = tx / sw;
        if (ox >= g.ow) continue;
        acc += base[(int64_t)(ky * g.kw + kx) * k_stride + oy * g.ow + ox];
      }
    }
    dx[((int64_t)n * g.cin + c) * hw + e] = acc;
  }
}

template <bool PLANES>
static void launch_col2im_as(om_ctx* ctx, dim3 grid, const ConvGeom& g, const float* dcols, float* dx, int64_t k_stride, int64_t n_stride, int total) {
  if (g.sh == 1 && g.sw == 1) col2im_gather_kernel<1, PLANES><<<grid, 256, 0, ctx->stream>>>(g, dcols, dx, k_stride, n_stride, total);
  else if (g.sh == 2 && g.sw == 2) col2im_gather_kernel<2, PLANES><<<grid, 256, 0, ctx->stream>>>(g, dcols, dx, k_stride, n_stride, total);
  else col2im_gather_kernel<0, PLANES><<<grid, 256, 0, ctx->stream>>>(g, dcols, dx, k_stride, n_stride, total);
}

static void launch_col2im(om_ctx* ctx, const ConvGeom& g, const float* dcols, float* dx, int64_t k_stride, int64_t n_stride) {
  const int hw = g.h * g.w;
  const int64_t total = (int64_t)g.n * g.cin * hw;
  if (hw < 256 && total < (int64_t)INT32_MAX) {
    launch_col2im_as<false>(ctx, dim3((unsigned)grid_for(ctx, total, 256)), g, dcols, dx, k_stride, n_stride, (int)total);
  } else {
    dim3 grid((unsigned)std::min<int64_t>(ceil_div(hw, 256), 64), (unsigned)g.cin, (unsigned)g.n);
    launch_col2im_as<true>(ctx, grid, g, dcols, dx, k_stride, n_stride, 0);
  }
}

__global__ void add_plane_bias_kernel(float* __restrict__ y, const float* __restrict__ bias, int cout, int plane, int64_t total) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = i; e < total; e += stride) y[e] += bias[(e / plane) % cout];
}

// t[c][n*plane + p] = g[n][c][p]. A thread moves VEC consecutive pixels of one plane (VEC == 4: plane a multiple of four).
template <int VEC>
__global__ void __launch_bounds__(256)
nchw_to_cnhw_kernel(const float* __restrict__ g, float* __restrict__ t, int n, int c, int plane, int64_t total) {
  int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * VEC;
  int64_t stride = (int64_t)gridDim.x * blockDim.x * VEC;
  const int64_t np = (int64_t)n * plane;
  for (int64_t e = i; e < total; e += stride) {
    const int64_t r = e / plane;
    const int p = (int)(e - r * plane);
    const int img = (int)(r / c), ch = (int)(r - (int64_t)img * c);
    float* dst = t + (int64_t)ch * np + (int64_t)img * plane + p;
    if (VEC == 4) *reinterpret_cast<float4*>(dst) = __ldg(reinterpret_cast<const float4*>(g + e));
    else *dst = g[e];
  }
}
// y[n][c][p] = t[c][n*plane + p] + bias[c]
template <int VEC>
__global__ void __launch_bounds__(256)
cnhw_to_nchw_bias_kernel(const float* __restrict__ t, const float* __restrict__ bias, float* __restrict__ y, int n, int c, int plane,
                         int64_t total) {
  int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * VEC;
  int64_t stride = (int64_t)gridDim.x * blockDim.x * VEC;
  const int64_t np = (int64_t)n * plane;
  for (int64_t e = i; e < total; e += stride) {
    const int64_t r = e / plane;
    const int p = (int)(e - r * plane);
    const int img = (int)(r / c), ch = (int)(r - (int64_t)img * c);
    const float* src = t + (int64_t)ch * np + (int64_t)img * plane + p;
    const float bv = bias ? bias[ch] : 0.f;
    if (VEC == 4) {
      float4 v = __ldg(reinterpret_cast<const float4*>(src));
      if (bias) { v.x += bv; v.y += bv; v.z += bv; v.w += bv; }
      *reinterpret_cast<float4*>(y + e) = v;
    } else {
      y[e] = bias ? *src + bv : *src;
    }
  }
}

// dbias[co] = sum over images of the plane sums of g[n][co][:], in double. Stage 1: CTA (co, slice) sums the planes of a
// fixed slice of images (thread partials in a fixed tree); stage 2 adds the slices in order.
constexpr int kDbiasSlices = 16;
__global__ void __launch_bounds__(256)
conv_dbias_partial_kernel(const float* __restrict__ g, int n, int cout, int plane, int per_slice, double* __restrict__ partial) {
  __shared__ double sm[256];
  const int co = blockIdx.x, slice = blockIdx.y;
  const int i0 = slice * per_slice, i1 = min(n, i0 + per_slice);
  double acc = 0.0;
  const int64_t span = (int64_t)(i1 - i0) * plane;
  for (int64_t e = threadIdx.x; e < span; e += 256) {
    const int i = i0 + (int)(e / plane);
    const int p = (int)(e % plane);
    acc += (double)g[((int64_t)i * cout + co) * plane + p];
  }
  sm[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) sm[threadIdx.x] += sm[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[(int64_t)slice * cout + co] = sm[0];
}
__global__ void conv_dbias_finish_kernel(const double* __restrict__ partial, int slices, int cout, float* __restrict__ dbias, int accumulate) {
  int co = blockIdx.x * blockDim.x + threadIdx.x;
  if (co >= cout) return;
  double t = 0.0;
  for (int s = 0; s < slices; s++) t += partial[(int64_t)s * cout + co];
  dbias[co] = accumulate ? dbias[co] + (float)t : (float)t;
}

__global__ void chunk_reduce_kernel(const float* __restrict__ part, int chunks, int64_t len, float* __restrict__ out, int accumulate) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < len; j += stride) {
    float acc = part[j];
    for (int c = 1; c < chunks; c++) acc += part[(int64_t)c * len + j];
    out[j] = accumulate ? out[j] + acc : acc;
  }
}

// ---- pooling --------------------------------------------------------------------------------------------------------------
struct PoolGeom {
  int h, w, oh, ow, kh, kw, sh, sw, ph, pw;
};

static bool pool_out(int size, int kernel, int stride, int pad, int* out) {
  if (kernel < 1 || stride < 1 || pad < 0 || pad >= kernel) return false;
  int64_t span = (int64_t)size + 2 * pad - kernel;
  if (span < 0) return false;
  *out = (int)(span / stride) + 1;
  return true;
}

// First maximum wins ties, NaN wins over numbers (ReferenceKernels.MaxPool2d, TensorKernels.cs:242-295).
// IDX: int when the input has fewer than 2^31 elements (32-bit divisions).
template <typename IDX>
__global__ void maxpool_fwd_kernel(PoolGeom g, const float* __restrict__ x, int64_t total, float* __restrict__ y, int32_t* __restrict__ idx) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = i; e < total; e += stride) {
    const IDX e32 = (IDX)e;
    const IDX row = e32 / (IDX)g.ow;
    int ox = (int)(e32 - row * (IDX)g.ow);
    const IDX pl = row / (IDX)g.oh;
    int oy = (int)(row - pl * (IDX)g.oh);
    const float* xp = x + (int64_t)pl * g.h * g.w;
    float best = -INFINITY;
    int bestIdx = -1;
    for (int ky = 0; ky < g.kh; ky++) {
      int yy = oy * g.sh - g.ph + ky;
      if ((unsigned)yy >= (unsigned)g.h) continue;
      for (int kx = 0; kx < g.kw; kx++) {
        int xx = ox * g.sw - g.pw + kx;
        if ((unsigned)xx >= (unsigned)g.w) continue;
        float v = xp[yy * g.w + xx];
        bool wins = bestIdx < 0 || (v > best && !(best != best)) || ((v != v) && !(best != best));
        if (wins) {
          best = v;
          bestIdx = (int)(pl * g.h * g.w) + yy * g.w + xx;
        }
      }
    }
    y[e] = best;
    if (idx) idx[e] = bestIdx;
  }
}

// dx[j] = sum of g[i] over the outputs i (in increasing i) whose saved index is j.
__global__ void maxpool_bwd_kernel(PoolGeom g, const float* __restrict__ gr, const int32_t* __restrict__ idx, int64_t total,
                                   float* __restrict__ dx) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = i; e < total; e += stride) {
    int ix = (int)(e % g.w), iy = (int)((e / g.w) % g.h);
    int64_t pl = e / ((int64_t)g.w * g.h);
    int oy0 = max(0, (iy + g.ph - g.kh + g.sh) / g.sh), oy1 = min(g.oh - 1, (iy + g.ph) / g.sh);
    int ox0 = max(0, (ix + g.pw - g.kw + g.sw) / g.sw), ox1 = min(g.ow - 1, (ix + g.pw) / g.sw);
    float acc = 0.f;
    for (int oy = oy0; oy <= oy1; oy++)
      for (int ox = ox0; ox <= ox1; ox++) {
        int64_t o = (pl * g.oh + oy) * g.ow + ox;
        if (idx[o] == (int32_t)e) acc += gr[o];
      }
    dx[e] = acc;
  }
}

// Windows that tile the plane (stride equal to the kernel, no padding): every input belongs to at most one window, so
// dx[e] is g of that window when its saved index is e, else zero. 32-bit index arithmetic; a thread owns VEC adjacent
// inputs of a row (one 16-byte store when VEC is 4: w a multiple of 4 and dx 16-byte aligned).
template <int VEC>
__global__ void maxpool_bwd_tiled_kernel(int h, int w, int oh, int ow, int kh, int kw, const float* __restrict__ gr,
                                         const int32_t* __restrict__ idx, int groups, float* __restrict__ dx) {
  const int stride = gridDim.x * blockDim.x;
  const int wg = w / VEC;
  for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < groups; q += stride) {
    const int xg = q % wg, t = q / wg;
    const int iy = t % h, pl = t / h;
    const int oy = iy / kh;
    const int e0 = (pl * h + iy) * w + xg * VEC;
    float v[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) v[j] = 0.f;
    if (oy < oh) {
      const int obase = (pl * oh + oy) * ow;
      int last_ox = -1, last_idx = 0;
      float last_g = 0.f;
#pragma unroll
      for (int j = 0; j < VEC; j++) {
        const int ox = (xg * VEC + j) / kw;
        if (ox < ow) {
          if (ox != last_ox) {
            last_ox = ox;
            last_idx = __ldg(idx + obase + ox);
            last_g = __ldg(gr + obase + ox);
          }
          if (last_idx == e0 + j) v[j] = last_g;
        }
      }
    }
    if (VEC == 4) {
      *reinterpret_cast<float4*>(dx + e0) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
      for (int j = 0; j < VEC; j++) dx[e0 + j] = v[j];
    }
  }
}

// The in-bounds window of output (oy, ox) and its divisor (PoolWindow, BackwardNn.cs:490-506).
__device__ __forceinline__ void pool_window(const PoolGeom& g, int include_pad, int oy, int ox, int* y0, int* y1, int* x0, int* x1, int* count) {
  int ys = oy * g.sh - g.ph, xs = ox * g.sw - g.pw;
  int ye = min(ys + g.kh, g.h + g.ph), xe = min(xs + g.kw, g.w + g.pw);
  int padded = (ye - ys) * (xe - xs);
  *y0 = max(ys, 0);
  *x0 = max(xs, 0);
  *y1 = min(ye, g.h);
  *x1 = min(xe, g.w);
  *count = include_pad ? padded : max(1, (*y1 - *y0) * (*x1 - *x0));
}

__global__ void avgpool_fwd_kernel(PoolGeom g, int include_pad, const float* __restrict__ x, int64_t total, float* __restrict__ y) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = i; e < total; e += stride) {
    int ox = (int)(e % g.ow), oy = (int)((e / g.ow) % g.oh);
    int64_t pl = e / ((int64_t)g.ow * g.oh);
    int y0, y1, x0, x1, count;
    pool_window(g, include_pad, oy, ox, &y0, &y1, &x0, &x1, &count);
    const float* xp = x + pl * g.h * g.w;
    float sum = 0.f;
    for (int yy = y0; yy < y1; yy++)
      for (int xx = x0; xx < x1; xx++) sum += xp[yy * g.w + xx];
    y[e] = sum / (float)count;
  }
}

__global__ void avgpool_bwd_kernel(PoolGeom g, int include_pad, const float* __restrict__ gr, int64_t total, float* __restrict__ dx) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = i; e < total; e += stride) {
    int ix = (int)(e % g.w), iy = (int)((e / g.w) % g.h);
    int64_t pl = e / ((int64_t)g.w * g.h);
    int oy0 = max(0, (iy + g.ph - g.kh + g.sh) / g.sh), oy1 = min(g.oh - 1, (iy + g.ph) / g.sh);
    int ox0 = max(0, (ix + g.pw - g.kw + g.sw) / g.sw), ox1 = min(g.ow - 1, (ix + g.pw) / g.sw);
    float acc = 0.f;
    for (int oy = oy0; oy <= oy1; oy++)
      for (int ox = ox0; ox <= ox1; ox++) {
        int y0, y1, x0, x1, count;
        pool_window(g, include_pad, oy, ox, &y0, &y1, &x0, &x1, &count);
        if (iy >= y0 && iy < y1 && ix >= x0 && ix < x1) acc += gr[(pl * g.oh + oy) * g.ow + ox] / (float)count;
      }
    dx[e] = acc;
  }
}

// ---- resize ---------------------------------------------------------------------------------------------------------------
// Source coordinate of one output index (Ops.SourceCoord, Ops.Spatial.cs:200-235 of the reference). mode 0 nearest, 1 bilinear.
__device__ __forceinline__ void source_coord(int mode, int align, int dst, int in_size, int out_size, int* i0, int* i1, float* lambda) {
  if (mode == 0) {
    float scale = (float)in_size / (float)out_size;
    int v = (int)floorf((float)dst * scale);
    *i0 = v < in_size - 1 ? v : in_size - 1;
    *i1 = *i0;
    *lambda = 0.f;
    return;
  }
  float src;
  if (align) {
    float scale = out_size > 1 ? (float)(in_size - 1) / (float)(out_size - 1) : 0.f;
    src = scale * (float)dst;
  } else {
    float scale = (float)in_size / (float)out_size;
    src = (scale * ((float)dst + 0.5f)) - 0.5f;
    if (src < 0.f) src = 0.f;
  }
  int a = (int)src;
  if (a > in_size - 1) a = in_size - 1;
  *i0 = a;
  *i1 = a + (a < in_size - 1 ? 1 : 0);
  *lambda = src - (float)a;
}

__global__ void resize_fwd_kernel(const float* __restrict__ x, int64_t planes, int h, int w, int oh, int ow, int mode, int align,
                                  float* __restrict__ y) {
  int64_t total = planes * oh * ow;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    int ox = (int)(i % ow), oy = (int)((i / ow) % oh);
    int64_t pl = i / ((int64_t)ow * oh);
    const float* sp = x + pl * h * w;
    int y0, y1, x0, x1;
    float ly, lx;
    source_coord(mode, align, oy, h, oh, &y0, &y1, &ly);
    source_coord(mode, align, ox, w, ow, &x0, &x1, &lx);
    float v;
    if (mode == 0) {
      v = sp[y0 * w + x0];
    } else {
      float top = ((1.f - lx) * sp[y0 * w + x0]) + (lx * sp[y0 * w + x1]);
      float bottom = ((1.f - lx) * sp[y1 * w + x0]) + (lx * sp[y1 * w + x1]);
      v = ((1.f - ly) * top) + (ly * bottom);
    }
    y[i] = v;
  }
}

// dx[pl][iy][ix]: the reference scatters every output pixel's four weighted terms in output order (ResizeBackward,
// BackwardRecurrent.cs:371-412); here every input pixel gathers the same terms in the same order, so no atomics are needed.
__global__ void resize_bwd_kernel(const float* __restrict__ g, int64_t planes, int h, int w, int oh, int ow, int mode, int align,
                                  float* __restrict__ dx) {
  int64_t total = planes * h * w;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    int ix = (int)(i % w), iy = (int)((i / w) % h);
    int64_t pl = i / ((int64_t)w * h);
    const float* gp = g + pl * oh * ow;
    float acc = 0.f;
    for (int oy = 0; oy < oh; oy++) {
      int y0, y1;
      float ly;
      source_coord(mode, align, oy, h, oh, &y0, &y1, &ly);
      if (y0 != iy && y1 != iy) continue;
      for (int ox = 0; ox < ow; ox++) {
        int x0, x1;
        float lx;
        source_coord(mode, align, ox, w, ow, &x0, &x1, &lx);
        if (x0 != ix && x1 != ix) continue;
        float gg = gp[oy * ow + ox];
        if (mode == 0) {
          acc += gg;
        } else {
          float t = (1.f - ly) * gg, b = ly * gg;
          if (y0 == iy && x0 == ix) acc += (1.f - lx) * t;
          if (y0 == iy && x1 == ix) acc += lx * t;
          if (y1 == iy && x0 == ix) acc += (1.f - lx) * b;
          if (y1 == iy && x1 == ix) acc += lx * b;
        }
      }
    }
    dx[i] = acc;
  }
}

static int32_t unfold(om_ctx* ctx, const ConvGeom& g, const float* x, float** cols, bool all_images = false) {
  int64_t total = (int64_t)g.n * g.cin * g.kh * g.kw * g.oh * g.ow;
  const int64_t plane = (int64_t)g.oh * g.ow, kk_all = (int64_t)g.cin * g.kh * g.kw;
  if (kk_all > 65535 || g.cin > 65535 || g.n > 65535)
    return fail(ctx, OM_ERR_UNSUPPORTED, "convolution: more than 65535 images, input channels or taps per output in one call");
  OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)(total > 0 ? total : 1), false, (void**)cols));
  if (total > 0) {
    const int64_t pixels_all = (int64_t)g.n * plane;
    const bool vec = (plane & 3) == 0;
    dim3 grid((unsigned)std::min<int64_t>(ceil_div(pixels_all, vec ? 1024 : 256), 65535), (unsigned)kk_all);
    const int64_t ks = all_images ? pixels_all : plane, ns = all_images ? plane : kk_all * plane;
    const bool small = pixels_all + 4 < (int64_t)INT32_MAX;
    if (vec && small) im2col_kernel<4, int><<<grid, 256, 0, ctx->stream>>>(g, x, *cols, pixels_all, ks, ns);
    else if (vec) im2col_kernel<4, int64_t><<<grid, 256, 0, ctx->stream>>>(g, x, *cols, pixels_all, ks, ns);
    else if (small) im2col_kernel<1, int><<<grid, 256, 0, ctx->stream>>>(g, x, *cols, pixels_all, ks, ns);
    else im2col_kernel<1, int64_t><<<grid, 256, 0, ctx->stream>>>(g, x, *cols, pixels_all, ks, ns);
  }
  return OM_OK;
}

// The all-images tensor-pipe formulation applies: TF32 asked for, one group, every pitch a multiple of four floats.
static bool conv_on_tensor_pipe(om_ctx* ctx, const ConvGeom& g, bool need_w_kmajor) {
  if (!(ctx->flags & OM_TF32) || g.groups != 1) return false;
  const int64_t np = (int64_t)g.n * g.oh * g.ow;
  const int kk = g.cin * g.kh * g.kw;
  if (np > INT32_MAX || (np & 3)) return false;
  if (need_w_kmajor && (kk & 3)) return false;          // W [Cout, K] is read with row pitch K
  return (double)g.cout * kk * (double)np >= 32.0 * 32 * 32;
}

static int32_t to_cnhw(om_ctx* ctx, const ConvGeom& g, const float* gr, float** out) {
  const int plane = g.oh * g.ow;
  int64_t total = (int64_t)g.n * g.cout * plane;
  OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)total, false, (void**)out));
  if ((plane & 3) == 0) nchw_to_cnhw_kernel<4><<<grid_for(ctx, total / 4, 256), 256, 0, ctx->stream>>>(gr, *out, g.n, g.cout, plane, total);
  else nchw_to_cnhw_kernel<1><<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(gr, *out, g.n, g.cout, plane, total);
  return OM_OK;
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_conv2d_fwd(om_ctx* ctx, const om_conv_shape* s, const float* x, const float* w, const float* bias, float* y) {
  OM_CHECK_CTX(ctx);
  ConvGeom g;
  if (!s || !conv_geom(s, &g)) return fail(ctx, OM_ERR_SHAPE, "Invalid convolution geometry.");
  if (g.n == 0) return OM_OK;
  const int cg = g.cin / g.groups, og = g.cout / g.groups, kk = cg * g.kh * g.kw, plane = g.oh * g.ow;
  if (g.n > 65535) return fail(ctx, OM_ERR_UNSUPPORTED, "om_conv2d_fwd: more than 65535 images in one call");
  ProfileScope prof(ctx, "om_conv2d_fwd", 2.0 * g.n * g.cout * (double)kk * plane, 4.0 * ((double)g.n * g.cin * g.h * g.w + (double)g.n * g.cout * plane));
  if (conv_on_tensor_pipe(ctx, g, true)) {
    const int np = g.n * plane;
    float *cols = nullptr, *yt = nullptr;
    OM_TRY(unfold(ctx, g, x, &cols, true));
    int32_t st = pool_alloc(ctx, sizeof(float) * (size_t)g.cout * np, false, (void**)&yt);
    if (st == OM_OK) st = gemm_tc(ctx, 0, 0, g.cout, np, kk, w, kk, cols, np, yt, np, 0, nullptr);
    if (st == OM_OK) {
      int64_t total = (int64_t)g.cout * np;
      if ((plane & 3) == 0) cnhw_to_nchw_bias_kernel<4><<<grid_for(ctx, total / 4, 256), 256, 0, ctx->stream>>>(yt, bias, y, g.n, g.cout, plane, total);
      else cnhw_to_nchw_bias_kernel<1><<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(yt, bias, y, g.n, g.cout, plane, total);
    }
    pool_free(ctx, cols);
    if (yt) pool_free(ctx, yt);
    OM_TRY(st);
    OM_LAUNCH_CHECK(ctx, "om_conv2d_fwd");
    return OM_OK;
  }
  float* cols = nullptr;
  OM_TRY(unfold(ctx, g, x, &cols));
  int32_t st = OM_OK;
  for (int grp = 0; grp < g.groups && st == OM_OK; grp++) {
    // y_n[og, P] = W_g[og, kk] * cols_n[kk, P]
    st = gemm_simt(ctx, 0, 0, og, plane, kk, w + (size_t)grp * og * kk, kk, 0, cols + (size_t)grp * kk * plane, plane,
                   (int64_t)g.groups * kk * plane, y + (size_t)grp * og * plane, plane, (int64_t)g.cout * plane, g.n, 0);
  }
  pool_free(ctx, cols);
  OM_TRY(st);
  if (bias) {
    int64_t total = (int64_t)g.n * g.cout * plane;
    add_plane_bias_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(y, bias, g.cout, plane, total);
  }
  OM_LAUNCH_CHECK(ctx, "om_conv2d_fwd");
  return OM_OK;
}

int32_t om_conv2d_dgrad(om_ctx* ctx, const om_conv_shape* s, const float* gr, const float* w, float* dx) {
  OM_CHECK_CTX(ctx);
  ConvGeom g;
  if (!s || !conv_geom(s, &g)) return fail(ctx, OM_ERR_SHAPE, "Invalid convolution geometry.");
  if (g.n == 0) return OM_OK;
  if (g.n > 65535) return fail(ctx, OM_ERR_UNSUPPORTED, "om_conv2d_dgrad: more than 65535 images in one call");
  const int cg = g.cin / g.groups, og = g.cout / g.groups, kk = cg * g.kh * g.kw, plane = g.oh * g.ow;
  ProfileScope prof(ctx, "om_conv2d_dgrad", 2.0 * g.n * g.cout * (double)kk * plane, 4.0 * ((double)g.n * g.cin * g.h * g.w + (double)g.n * g.cout * plane));
  float* dcols = nullptr;
  int64_t total_cols = (int64_t)g.n * g.groups * kk * plane;
  OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)total_cols, false, (void**)&dcols));
  if (conv_on_tensor_pipe(ctx, g, true)) {
    const int np = g.n * plane;
    float* gt = nullptr;
    int32_t st = to_cnhw(ctx, g, gr, &gt);
    // dcols [K, N*P] = W^T [K, Cout] * g_t [Cout, N*P]
    if (st == OM_OK) st = gemm_tc(ctx, 1, 0, kk, np, g.cout, w, kk, gt, np, dcols, np, 0, nullptr);
    if (st == OM_OK) {
      launch_col2im(ctx, g, dcols, dx, np, plane);
    }
    if (gt) pool_free(ctx, gt);
    pool_free(ctx, dcols);
    OM_TRY(st);
    OM_LAUNCH_CHECK(ctx, "om_conv2d_dgrad");
    return OM_OK;
  }
  int32_t st = OM_OK;
  for (int grp = 0; grp < g.groups && st == OM_OK; grp++) {
    // dcols_n[kk, P] = W_g^T[kk, og] * g_n[og, P]
    st = gemm_simt(ctx, 1, 0, kk, plane, og, w + (size_t)grp * og * kk, kk, 0, gr + (size_t)grp * og * plane, plane,
                   (int64_t)g.cout * plane, dcols + (size_t)grp * kk * plane, plane, (int64_t)g.groups * kk * plane, g.n, 0);
  }
  if (st == OM_OK) {
    launch_col2im(ctx, g, dcols, dx, plane, (int64_t)g.cin * g.kh * g.kw * plane);
  }
  pool_free(ctx, dcols);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_conv2d_dgrad");
  return OM_OK;
}

int32_t om_conv2d_wgrad(om_ctx* ctx, const om_conv_shape* s, const float* gr, const float* x, float* dw, int32_t accumulate) {
  OM_CHECK_CTX(ctx);
  ConvGeom g;
  if (!s || !conv_geom(s, &g)) return fail(ctx, OM_ERR_SHAPE, "Invalid convolution geometry.");
  const int cg = g.cin / g.groups, og = g.cout / g.groups, kk = cg * g.kh * g.kw, plane = g.oh * g.ow;
  const int64_t wlen = (int64_t)g.cout * kk;
  if (g.n == 0) {
    if (!accumulate) OM_CUDA(ctx, cudaMemsetAsync(dw, 0, sizeof(float) * (size_t)wlen, ctx->stream));
    return OM_OK;
  }
  ProfileScope prof(ctx, "om_conv2d_wgrad", 2.0 * g.n * g.cout * (double)kk * plane, 4.0 * ((double)g.n * g.cin * g.h * g.w + (double)g.n * g.cout * plane));
  if (conv_on_tensor_pipe(ctx, g, false)) {
    const int np = g.n * plane;
    float *cols = nullptr, *gt = nullptr;
    OM_TRY(unfold(ctx, g, x, &cols, true));
    int32_t st = to_cnhw(ctx, g, gr, &gt);
    // dW [Cout, K] = g_t [Cout, N*P] * cols^T [N*P, K]: both operands k-contiguous, k = N*P split in fixed slices.
    if (st == OM_OK) st = gemm_tc(ctx, 0, 1, g.cout, kk, np, gt, np, cols, np, dw, kk, accumulate, nullptr);
    pool_free(ctx, cols);
    if (gt) pool_free(ctx, gt);
    OM_TRY(st);
    OM_LAUNCH_CHECK(ctx, "om_conv2d_wgrad");
    return OM_OK;
  }
  float* cols = nullptr;
  OM_TRY(unfold(ctx, g, x, &cols));
  // Images are summed inside the kernel in fixed chunks; the chunk size depends on the shape only.
  const int tiles = (int)(ceil_div(og, 64) * ceil_div(kk, 64)) * g.groups;
  int chunks = (int)std::min<int64_t>(g.n, std::max<int64_t>(1, ceil_div(2 * 148, tiles)));
  const int per_chunk = (int)ceil_div(g.n, chunks);
  chunks = (int)ceil_div(g.n, per_chunk);
  float* partial = nullptr;
  int32_t st = pool_alloc(ctx, sizeof(float) * (size_t)chunks * wlen, false, (void**)&partial);
  for (int grp = 0; grp < g.groups && st == OM_OK; grp++) {
    // dW_g[og, kk] = sum_n g_n[og, P] * cols_n[kk, P]^T ; partial chunk c lives at partial + c*wlen
    st = gemm_simt_batch_reduce(ctx, 0, 1, og, kk, plane, gr + (size_t)grp * og * plane, plane, (int64_t)g.cout * plane,
                                cols + (size_t)grp * kk * plane, plane, (int64_t)g.groups * kk * plane,
                                partial + (size_t)grp * og * kk, wlen, g.n, per_chunk);
  }
  if (st == OM_OK) chunk_reduce_kernel<<<grid_for(ctx, wlen, 256), 256, 0, ctx->stream>>>(partial, chunks, wlen, dw, accumulate);
  pool_free(ctx, cols);
  if (partial) pool_free(ctx, partial);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_conv2d_wgrad");
  return OM_OK;
}

int32_t om_conv2d_dbias(om_ctx* ctx, const om_conv_shape* s, const float* gr, float* dbias, int32_t accumulate) {
  OM_CHECK_CTX(ctx);
  ConvGeom g;
  if (!s || !conv_geom(s, &g)) return fail(ctx, OM_ERR_SHAPE, "Invalid convolution geometry.");
  ProfileScope prof(ctx, "om_conv2d_dbias", 0, 4.0 * g.n * g.cout * (double)g.oh * g.ow);
  if (g.n == 0) {
    if (!accumulate) OM_CUDA(ctx, cudaMemsetAsync(dbias, 0, sizeof(float) * (size_t)g.cout, ctx->stream));
    return OM_OK;
  }
  const int slices = g.n < kDbiasSlices ? g.n : kDbiasSlices, per_slice = (int)ceil_div(g.n, slices);
  double* partial = nullptr;
  OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)slices * g.cout, false, (void**)&partial));
  conv_dbias_partial_kernel<<<dim3(g.cout, slices), 256, 0, ctx->stream>>>(gr, g.n, g.cout, g.oh * g.ow, per_slice, partial);
  conv_dbias_finish_kernel<<<(unsigned)ceil_div(g.cout, 128), 128, 0, ctx->stream>>>(partial, slices, g.cout, dbias, accumulate);
  pool_free(ctx, partial);
  OM_LAUNCH_CHECK(ctx, "om_conv2d_dbias");
  return OM_OK;
}

int32_t om_resize2d_fwd(om_ctx* ctx, const float* x, int64_t planes, int32_t h, int32_t w, int32_t out_h, int32_t out_w, int32_t mode,
                        int32_t align_corners, float* y) {
  OM_CHECK_CTX(ctx);
  if (planes < 0 || h < 1 || w < 1 || out_h < 1 || out_w < 1 || mode < 0 || mode > 1)
    return fail(ctx, OM_ERR_SHAPE, "Resize2d needs an (N,C,H,W) input and a positive output size (planes %lld, %dx%d -> %dx%d, mode %d)",
                (long long)planes, h, w, out_h, out_w, mode);
  int64_t total = planes * out_h * out_w;
  if (total == 0) return OM_OK;
  ProfileScope prof(ctx, "om_resize2d_fwd", 0, 4.0 * (planes * (double)h * w + total));
  resize_fwd_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(x, planes, h, w, out_h, out_w, mode, align_corners && mode == 1, y);
  OM_LAUNCH_CHECK(ctx, "om_resize2d_fwd");
  return OM_OK;
}

int32_t om_resize2d_bwd(om_ctx* ctx, const float* g, int64_t planes, int32_t h, int32_t w, int32_t out_h, int32_t out_w, int32_t mode,
                        int32_t align_corners, float* dx) {
  OM_CHECK_CTX(ctx);
  if (planes < 0 || h < 1 || w < 1 || out_h < 1 || out_w < 1 || mode < 0 || mode > 1)
    return fail(ctx, OM_ERR_SHAPE, "Resize2d backward: planes %lld, %dx%d -> %dx%d, mode %d", (long long)planes, h, w, out_h, out_w, mode);
  int64_t total = planes * h * w;
  if (total == 0) return OM_OK;
  ProfileScope prof(ctx, "om_resize2d_bwd", 0, 4.0 * (planes * (double)out_h * out_w + total));
  resize_bwd_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(g, planes, h, w, out_h, out_w, mode, align_corners && mode == 1, dx);
  OM_LAUNCH_CHECK(ctx, "om_resize2d_bwd");
  return OM_OK;
}

static int32_t pool_geom(om_ctx* ctx, const char* who, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, PoolGeom* g) {
  g->h = h; g->w = w; g->kh = kh; g->kw = kw; g->sh = sh; g->sw = sw; g->ph = ph; g->pw = pw;
  if (h < 0 || w < 0 || !pool_out(h, kh, sh, ph, &g->oh) || !pool_out(w, kw, sw, pw, &g->ow))
    return fail(ctx, OM_ERR_SHAPE, "%s: Invalid pooling window (kernel %dx%d, stride %dx%d, pad %dx%d) for %dx%d.", who, kh, kw, sh, sw, ph, pw, h, w);
  return OM_OK;
}

int32_t om_maxpool_fwd(om_ctx* ctx, const float* x, int32_t planes, int32_t h, int32_t w, int32_t kh, int32_t kw, int32_t sh,
                       int32_t sw, int32_t ph, int32_t pw, float* y, int32_t* idx) {
  OM_CHECK_CTX(ctx);
  PoolGeom g;
  OM_TRY(pool_geom(ctx, "om_maxpool_fwd", h, w, kh, kw, sh, sw, ph, pw, &g));
  if ((int64_t)planes * h * w > INT32_MAX) return fail(ctx, OM_ERR_SHAPE, "om_maxpool_fwd: more than 2^31-1 input elements");
  int64_t total = (int64_t)planes * g.oh * g.ow;
  if (total <= 0) return OM_OK;
  ProfileScope prof(ctx, "om_maxpool_fwd", 0, 4.0 * planes * ((double)h * w + 2.0 * g.oh * g.ow));
  if ((int64_t)planes * h * w < (int64_t)INT32_MAX) maxpool_fwd_kernel<int><<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(g, x, total, y, idx);
  else maxpool_fwd_kernel<int64_t><<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(g, x, total, y, idx);
  OM_LAUNCH_CHECK(ctx, "om_maxpool_fwd");
  return OM_OK;
}

int32_t om_maxpool_bwd(om_ctx* ctx, const float* gr, const int32_t* idx, int32_t planes, int32_t h, int32_t w, int32_t oh,
                       int32_t ow, int32_t kh, int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw, float* dx) {
  OM_CHECK_CTX(ctx);
  PoolGeom g;
  OM_TRY(pool_geom(ctx, "om_maxpool_bwd", h, w, kh, kw, sh, sw, ph, pw, &g));
  if (g.oh != oh || g.ow != ow) return fail(ctx, OM_ERR_SHAPE, "om_maxpool_bwd: output %dx%d does not match the window", oh, ow);
  int64_t total = (int64_t)planes * h * w;
  if (total <= 0) return OM_OK;
  ProfileScope prof(ctx, "om_maxpool_bwd", 0, 4.0 * planes * ((double)h * w + 2.0 * oh * ow));
  if (kh == sh && kw == sw && ph == 0 && pw == 0 && total < (int64_t)1 << 30) {
    if ((w & 3) == 0 && (reinterpret_cast<uintptr_t>(dx) & 15) == 0)
      maxpool_bwd_tiled_kernel<4><<<grid_for(ctx, total / 4, 256), 256, 0, ctx->stream>>>(h, w, oh, ow, kh, kw, gr, idx, (int)(total / 4), dx);
    else
      maxpool_bwd_tiled_kernel<1><<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(h, w, oh, ow, kh, kw, gr, idx, (int)total, dx);
  } else
    maxpool_bwd_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(g, gr, idx, total, dx);
  OM_LAUNCH_CHECK(ctx, "om_maxpool_bwd");
  return OM_OK;
}

int32_t om_avgpool_fwd(om_ctx* ctx, const float* x, int32_t planes, int32_t h, int32_t w, int32_t kh, int32_t kw, int32_t sh,
                       int32_t sw, int32_t ph, int32_t pw, int32_t count_include_pad, float* y) {
  OM_CHECK_CTX(ctx);
  PoolGeom g;
  OM_TRY(pool_geom(ctx, "om_avgpool_fwd", h, w, kh, kw, sh, sw, ph, pw, &g));
  int64_t total = (int64_t)planes * g.oh * g.ow;
  if (total <= 0) return OM_OK;
  ProfileScope prof(ctx, "om_avgpool_fwd", 0, 4.0 * planes * ((double)h * w + g.oh * g.ow));
  avgpool_fwd_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(g, count_include_pad, x, total, y);
  OM_LAUNCH_CHECK(ctx, "om_avgpool_fwd");
  return OM_OK;
}

int32_t om_avgpool_bwd(om_ctx* ctx, const float* gr, int32_t planes, int32_t h, int32_t w, int32_t kh, int32_t kw, int32_t sh,
                       int32_t sw, int32_t ph, int32_t pw, int32_t count_include_pad, float* dx) {
  OM_CHECK_CTX(ctx);
  PoolGeom g;
  OM_TRY(pool_geom(ctx, "om_avgpool_bwd", h, w, kh, kw, sh, sw, ph, pw, &g));
  int64_t total = (int64_t)planes * h * w;
  if (total <= 0) return OM_OK;
  ProfileScope prof(ctx, "om_avgpool_bwd", 0, 4.0 * planes * ((double)h * w + g.oh * g.ow));
  avgpool_bwd_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(g, count_include_pad, gr, total, dx);
  OM_LAUNCH_CHECK(ctx, "om_avgpool_bwd");
  return OM_OK;
}

}  // extern "C"
