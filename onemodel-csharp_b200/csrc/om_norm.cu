// Layer normalisation (rows) and batch normalisation (NCHW channels), forward and backward. Bandwidth-bound:
// every kernel streams its operands once with coalesced 128-byte warp accesses. Statistics that the reference
// accumulates in double (BackwardNn.cs:170-307, Ops.Layers.cs:185-219) are accumulated in double here too, over a
// partition that depends only on the shape and is combined in a fixed order.
#include <cuda_bf16.h>

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

// out[j] = sum over chunks of partial[chunk, j] for one or two tables of double partials. A CTA owns 32 columns; 32
// chunk lanes each add chunks lane, lane + 32, ... in increasing order (five chunks of each table on their way at a time:
// the kernel is a chain of memory round trips and nothing else), then the lane sums are added in lane order: a fixed
// order, so the result does not depend on the launch.
__global__ void __launch_bounds__(1024)
column_partials_finish_kernel(const double* __restrict__ pa, const double* __restrict__ pb, int chunks, int32_t cols,
                              float* __restrict__ oa, float* __restrict__ ob, int accumulate) {
  pdl_enter();
  __shared__ double sa[32][33], sb[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + tx;
  const bool wa = pa && oa, wb = pb && ob;
  double ta = 0.0, tb = 0.0;
  if (j < cols) {
    for (int c0 = ty; c0 < chunks; c0 += 32 * 5) {
      double va[5], vb[5];
#pragma unroll
      for (int u = 0; u < 5; u++) {
        const int c = c0 + 32 * u;
        va[u] = (wa && c < chunks) ? pa[(int64_t)c * cols + j] : 0.0;
        vb[u] = (wb && c < chunks) ? pb[(int64_t)c * cols + j] : 0.0;
      }
#pragma unroll
      for (int u = 0; u < 5; u++) {
        if (c0 + 32 * u < chunks) {
          ta += va[u];
          tb += vb[u];
        }
      }
    }
  }
  sa[ty][tx] = ta;
  sb[ty][tx] = tb;
  __syncthreads();
  if (ty == 0 && j < cols) {
    if (wa) {
      double t = 0.0;
#pragma unroll
      for (int l = 0; l < 32; l++) t += sa[l][tx];
      oa[j] = accumulate ? oa[j] + (float)t : (float)t;
    }
    if (wb) {
      double t = 0.0;
#pragma unroll
      for (int l = 0; l < 32; l++) t += sb[l][tx];
      ob[j] = accumulate ? ob[j] + (float)t : (float)t;
    }
  }
}

// ---- layer norm with the row in registers ---------------------------------------------------------------------------
// Forward: one read of x per row (the kernel above reads it three times through L1), the same sums in the same order
// (lane l owns columns l, l + 32, ...), and optionally the bfloat16 copy of y that the next product reads.
__device__ __forceinline__ uint16_t bf16_bits(float v) {
  __nv_bfloat16 h = __float2bfloat16_rn(v);
  return *reinterpret_cast<uint16_t*>(&h);
}

template <int NC>
__global__ void __launch_bounds__(256)
layernorm_fwd_reg_kernel(const float* __restrict__ x, const float* __restrict__ addend, float* __restrict__ sum_out,
                         const float* __restrict__ gamma, const float* __restrict__ beta, int32_t rows, int32_t cols, float eps,
                         float* __restrict__ y, uint16_t* __restrict__ y16, float* __restrict__ mean_out, float* __restrict__ inv_out) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), warps = (int64_t)gridDim.x * 8;
  const float n = (float)cols;
  float gam[NC], bet[NC];
#pragma unroll
  for (int i = 0; i < NC; i++) {
    const int j = lane + 32 * i;
    gam[i] = j < cols ? gamma[j] : 0.f;
    bet[i] = j < cols ? beta[j] : 0.f;
  }
  for (int64_t r = warp; r < rows; r += warps) {
    const float* xr = x + r * cols;
    float v[NC];
#pragma unroll
    for (int i = 0; i < NC; i++) {
      const int j = lane + 32 * i;
      v[i] = j < cols ? xr[j] : 0.f;
    }
    if (addend) {
      // The residual sum x + addend is formed here (and written out: the backward pass normalises it again).
      const float* ar = addend + r * cols;
      float* sr = sum_out + r * cols;
#pragma unroll
      for (int i = 0; i < NC; i++) {
        const int j = lane + 32 * i;
        if (j < cols) {
          v[i] = v[i] + ar[j];
          sr[j] = v[i];
        }
      }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NC; i++)
      if (lane + 32 * i < cols) s += v[i];
    const float mean = wsum_f(s) / n;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NC; i++)
      if (lane + 32 * i < cols) {
        const float d = v[i] - mean;
        q += d * d;
      }
    const float inv = 1.0f / sqrtf((wsum_f(q) / n) + eps);
    if (lane == 0) {
      if (mean_out) mean_out[r] = mean;
      if (inv_out) inv_out[r] = inv;
    }
    float* yr = y + r * cols;
#pragma unroll
    for (int i = 0; i < NC; i++) {
      const int j = lane + 32 * i;
      if (j < cols) {
        const float o = (((v[i] - mean) * inv) * gam[i]) + bet[i];
        yr[j] = o;
        if (y16) y16[r * cols + j] = bf16_bits(o);
      }
    }
  }
}

// Backward in one pass over (g, x): a CTA owns kLnFusedRows consecutive rows, a warp takes every eighth of them with the
// row in registers, writes dx (and optionally its bfloat16 copy) and keeps, per lane and column, the sums of g * xhat and
// of g over its eight rows (fp32: eight terms). The eight warps' sums are added in warp order in double through shared
// memory and written as the CTA's row of two double partial tables; column_partials_finish_kernel adds the CTAs' rows in
// CTA order. The partition depends on the shape only, so the sums are the same from run to run.
constexpr int kLnFusedRows = 64;
template <int NC>
__global__ void __launch_bounds__(256, 2)
layernorm_bwd_fused_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ gamma,
                           const float* __restrict__ mean, const float* __restrict__ inv, int32_t rows, int32_t cols,
                           float* __restrict__ dx, uint16_t* __restrict__ dx16, double* __restrict__ part_gamma,
                           double* __restrict__ part_beta) {
  pdl_enter();
  extern __shared__ double ln_smem[];            // [8][cols]
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int r0 = blockIdx.x * kLnFusedRows;
  const int r1 = min(rows, r0 + kLnFusedRows);
  float ag[NC], ab[NC];
#pragma unroll
  for (int i = 0; i < NC; i++) {
    ag[i] = 0.f;
    ab[i] = 0.f;
  }
  for (int r = r0 + w; r < r1; r += 8) {
    const float* xr = x + (int64_t)r * cols;
    const float* gr = g + (int64_t)r * cols;
    const float m = mean[r], s = inv[r];
    float xh[NC], dh[NC];
#pragma unroll
    for (int i = 0; i < NC; i++) {
      const int j = lane + 32 * i;
      const bool in = j < cols;
      const float gv = in ? gr[j] : 0.f;
      const float xv = in ? xr[j] : m;
      xh[i] = (xv - m) * s;
      dh[i] = gv * (in ? __ldg(gamma + j) : 0.f);   // gamma stays in L1: keeping it in registers would not fit two CTAs per SM
      ag[i] += gv * xh[i];
      ab[i] += gv;
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
    if (dx) {
      float* dr = dx + (int64_t)r * cols;
#pragma unroll
      for (int i = 0; i < NC; i++) {
        const int j = lane + 32 * i;
        if (j < cols) {
          const float o = s * ((dh[i] - m1) - (xh[i] * m2));
          dr[j] = o;
          if (dx16) dx16[(int64_t)r * cols + j] = bf16_bits(o);
        }
      }
    }
  }
  // The CTA's column sums: warps in order, one table after the other through the same shared memory.
#pragma unroll 1
  for (int table = 0; table < 2; table++) {
    double* out = table == 0 ? part_gamma : part_beta;
    if (!out) continue;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NC; i++) {
      const int j = lane + 32 * i;
      if (j < cols) ln_smem[w * cols + j] = (double)(table == 0 ? ag[i] : ab[i]);
    }
    __syncthreads();
    for (int j = threadIdx.x; j < cols; j += 256) {
      double t = 0.0;
#pragma unroll
      for (int k = 0; k < 8; k++) t += ln_smem[k * cols + j];
      out[(int64_t)blockIdx.x * cols + j] = t;
    }
  }
}

// ---- layer norm, rows of 16-byte groups ------------------------------------------------------------------------------
// The same two kernels for rows whose width is a multiple of four and whose tensors are 16-byte aligned: a lane owns the
// groups of four columns lane, lane + 32, ... (one 16-byte access each, a warp's access 512 contiguous bytes), so a row of 768
// columns is six loads per tensor instead of twenty-four. Row sums add a lane's columns in increasing order and combine the
// lanes in the same butterfly as before; the partition is by shape alone, so results are the same from run to run.
__device__ __forceinline__ uint2 bf16x4_bits(float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  return make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

template <int NV>
__global__ void __launch_bounds__(256)
layernorm_fwd_vec_kernel(const float* __restrict__ x, const float* __restrict__ addend, float* __restrict__ sum_out,
                         const float* __restrict__ gamma, const float* __restrict__ beta, int32_t rows, int32_t cols, float eps,
                         float* __restrict__ y, uint16_t* __restrict__ y16, float* __restrict__ mean_out, float* __restrict__ inv_out) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), warps = (int64_t)gridDim.x * 8;
  const float n = (float)cols;
  const int nv = cols >> 2;
  float4 gam[NV], bet[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const int j = lane + 32 * i;
    gam[i] = j < nv ? __ldg(reinterpret_cast<const float4*>(gamma) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    bet[i] = j < nv ? __ldg(reinterpret_cast<const float4*>(beta) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int64_t r = warp; r < rows; r += warps) {
    const float4* xr = reinterpret_cast<const float4*>(x + r * cols);
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int j = lane + 32 * i;
      v[i] = j < nv ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (addend) {
      // The residual sum x + addend is formed here (and written out: the backward pass normalises it again).
      const float4* ar = reinterpret_cast<const float4*>(addend + r * cols);
      float4 a[NV];
#pragma unroll
      for (int i = 0; i < NV; i++) {
        const int j = lane + 32 * i;
        a[i] = j < nv ? ar[j] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float4* sr = reinterpret_cast<float4*>(sum_out + r * cols);
#pragma unroll
      for (int i = 0; i < NV; i++) {
        const int j = lane + 32 * i;
        v[i].x += a[i].x; v[i].y += a[i].y; v[i].z += a[i].z; v[i].w += a[i].w;
        if (j < nv) sr[j] = v[i];
      }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++)
      if (lane + 32 * i < nv) s += ((v[i].x + v[i].y) + v[i].z) + v[i].w;
    const float mean = wsum_f(s) / n;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++)
      if (lane + 32 * i < nv) {
        const float d0 = v[i].x - mean, d1 = v[i].y - mean, d2 = v[i].z - mean, d3 = v[i].w - mean;
        q += ((d0 * d0 + d1 * d1) + d2 * d2) + d3 * d3;
      }
    const float inv = 1.0f / sqrtf((wsum_f(q) / n) + eps);
    if (lane == 0) {
      if (mean_out) mean_out[r] = mean;
      if (inv_out) inv_out[r] = inv;
    }
    float4* yr = reinterpret_cast<float4*>(y + r * cols);
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int j = lane + 32 * i;
      if (j < nv) {
        float4 o;
        o.x = (((v[i].x - mean) * inv) * gam[i].x) + bet[i].x;
        o.y = (((v[i].y - mean) * inv) * gam[i].y) + bet[i].y;
        o.z = (((v[i].z - mean) * inv) * gam[i].z) + bet[i].z;
        o.w = (((v[i].w - mean) * inv) * gam[i].w) + bet[i].w;
        yr[j] = o;
        if (y16) reinterpret_cast<uint2*>(y16 + r * cols)[j] = bf16x4_bits(o);
      }
    }
  }
}

// Backward: a CTA owns kLnVecRows consecutive rows, a warp takes every eighth of them; otherwise as layernorm_bwd_fused_kernel.
constexpr int kLnVecRows = 56;
template <int NV>
__global__ void __launch_bounds__(256, 2)
layernorm_bwd_vec_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ gamma,
                         const float* __restrict__ mean, const float* __restrict__ inv, int32_t rows, int32_t cols,
                         float* __restrict__ dx, uint16_t* __restrict__ dx16, double* __restrict__ part_gamma, double* __restrict__ part_beta) {
  pdl_enter();
  extern __shared__ double ln_smem[];            // [8][cols]
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int nv = cols >> 2;
  const int r0 = blockIdx.x * kLnVecRows;
  const int r1 = min(rows, r0 + kLnVecRows);
  float4 ag[NV], ab[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) ag[i] = ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = r0 + w; r < r1; r += 8) {
    const float4* xr = reinterpret_cast<const float4*>(x + (int64_t)r * cols);
    const float4* gr = reinterpret_cast<const float4*>(g + (int64_t)r * cols);
    float4 xh[NV], dh[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int j = lane + 32 * i;
      xh[i] = j < nv ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
      dh[i] = j < nv ? gr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float m = mean[r], s = inv[r];
    double sum1 = 0.0, sum2 = 0.0;
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int j = lane + 32 * i;
      if (j < nv) {
        const float4 gm = __ldg(reinterpret_cast<const float4*>(gamma) + j);   // gamma stays in L1: registers would not fit two CTAs per SM
        const float4 gv = dh[i];
        xh[i].x = (xh[i].x - m) * s; xh[i].y = (xh[i].y - m) * s; xh[i].z = (xh[i].z - m) * s; xh[i].w = (xh[i].w - m) * s;
        dh[i].x = gv.x * gm.x; dh[i].y = gv.y * gm.y; dh[i].z = gv.z * gm.z; dh[i].w = gv.w * gm.w;
        ag[i].x += gv.x * xh[i].x; ag[i].y += gv.y * xh[i].y; ag[i].z += gv.z * xh[i].z; ag[i].w += gv.w * xh[i].w;
        ab[i].x += gv.x; ab[i].y += gv.y; ab[i].z += gv.z; ab[i].w += gv.w;
        sum1 += (double)dh[i].x; sum1 += (double)dh[i].y; sum1 += (double)dh[i].z; sum1 += (double)dh[i].w;
        sum2 += (double)(dh[i].x * xh[i].x); sum2 += (double)(dh[i].y * xh[i].y); sum2 += (double)(dh[i].z * xh[i].z);
        sum2 += (double)(dh[i].w * xh[i].w);
      }
    }
    sum1 = wsum_d(sum1);
    sum2 = wsum_d(sum2);
    const float m1 = (float)(sum1 / cols), m2 = (float)(sum2 / cols);
    if (dx) {
      float4* dr = reinterpret_cast<float4*>(dx + (int64_t)r * cols);
#pragma unroll
      for (int i = 0; i < NV; i++) {
        const int j = lane + 32 * i;
        if (j < nv) {
          float4 o;
          o.x = s * ((dh[i].x - m1) - (xh[i].x * m2));
          o.y = s * ((dh[i].y - m1) - (xh[i].y * m2));
          o.z = s * ((dh[i].z - m1) - (xh[i].z * m2));
          o.w = s * ((dh[i].w - m1) - (xh[i].w * m2));
          dr[j] = o;
          if (dx16) reinterpret_cast<uint2*>(dx16 + (int64_t)r * cols)[j] = bf16x4_bits(o);
        }
      }
    }
  }
  // The CTA's column sums: warps in order, one table after the other through the same shared memory.
#pragma unroll 1
  for (int table = 0; table < 2; table++) {
    double* out = table == 0 ? part_gamma : part_beta;
    if (!out) continue;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int j = lane + 32 * i;
      if (j < nv) {
        const float4 a = table == 0 ? ag[i] : ab[i];
        double* dst = ln_smem + (size_t)w * cols + 4 * j;
        dst[0] = (double)a.x; dst[1] = (double)a.y; dst[2] = (double)a.z; dst[3] = (double)a.w;
      }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < cols; j += 256) {
      double t = 0.0;
#pragma unroll
      for (int k = 0; k < 8; k++) t += ln_smem[k * cols + j];
      out[(int64_t)blockIdx.x * cols + j] = t;
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

int32_t om_layernorm_fwd_b16(om_ctx* ctx, const float* x, const float* gamma, const float* beta, int32_t rows, int32_t cols,
                             float eps, float* y, uint16_t* y16, float* mean, float* inv) {
  return om_add_layernorm_fwd_b16(ctx, x, nullptr, nullptr, gamma, beta, rows, cols, eps, y, y16, mean, inv);
}

int32_t om_add_layernorm_fwd_b16(om_ctx* ctx, const float* x, const float* addend, float* sum, const float* gamma, const float* beta,
                                 int32_t rows, int32_t cols, float eps, float* y, uint16_t* y16, float* mean, float* inv) {
  OM_CHECK_CTX(ctx);
  if (rows < 0 || cols < 0) return fail(ctx, OM_ERR_SHAPE, "om_layernorm_fwd: [%d,%d]", rows, cols);
  if (rows == 0 || cols == 0) return OM_OK;
  if ((addend != nullptr) != (sum != nullptr)) return fail(ctx, OM_ERR_ARG, "om_add_layernorm_fwd_b16: the addend and the sum go together");
  if (addend && cols > 1024) return fail(ctx, OM_ERR_UNSUPPORTED, "om_add_layernorm_fwd_b16: rows wider than 1024 (%d): add first, then om_layernorm_fwd", cols);
  ProfileScope prof(ctx, "om_layernorm_fwd", 0, ((y16 ? 10.0 : 8.0) + (addend ? 8.0 : 0.0)) * rows * (double)cols);
  int grid = (int)std::min<int64_t>(ceil_div(rows, 8), (int64_t)ctx->sm_count * 8);
  const int nc = (int)ceil_div(cols, 32);
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec = (cols & 3) == 0 && cols <= 1024 && al16(x) && al16(y) && al16(gamma) && al16(beta) && (!addend || (al16(addend) && al16(sum))) &&
                   (!y16 || (reinterpret_cast<uintptr_t>(y16) & 7) == 0);
  if (vec) {
    const int nvec = (int)ceil_div(cols, 128);
#define OM_LN_FWDV(NV) launch_chained(ctx, layernorm_fwd_vec_kernel<NV>, grid, 256, 0, x, addend, sum, gamma, beta, rows, cols, eps, y, y16, mean, inv)
    if (nvec <= 1) OM_LN_FWDV(1);
    else if (nvec <= 2) OM_LN_FWDV(2);
    else if (nvec <= 3) OM_LN_FWDV(3);
    else if (nvec <= 4) OM_LN_FWDV(4);
    else if (nvec <= 6) OM_LN_FWDV(6);
    else OM_LN_FWDV(8);
#undef OM_LN_FWDV
  } else if (nc <= 32) {
#define OM_LN_FWD(NC) launch_chained(ctx, layernorm_fwd_reg_kernel<NC>, grid, 256, 0, x, addend, sum, gamma, beta, rows, cols, eps, y, y16, mean, inv)
    if (nc <= 4) OM_LN_FWD(4);
    else if (nc <= 8) OM_LN_FWD(8);
    else if (nc <= 12) OM_LN_FWD(12);
    else if (nc <= 16) OM_LN_FWD(16);
    else if (nc <= 24) OM_LN_FWD(24);
    else OM_LN_FWD(32);
#undef OM_LN_FWD
  } else {
    if (y16) return fail(ctx, OM_ERR_UNSUPPORTED, "om_layernorm_fwd_b16: rows wider than 1024 (%d) have no fused bfloat16 copy", cols);
    launch_chained(ctx, layernorm_fwd_kernel, grid, 256, 0, x, gamma, beta, rows, cols, eps, y, mean, inv);
  }
  OM_LAUNCH_CHECK(ctx, "om_layernorm_fwd");
  return OM_OK;
}

int32_t om_layernorm_fwd(om_ctx* ctx, const float* x, const float* gamma, const float* beta, int32_t rows, int32_t cols,
                         float eps, float* y, float* mean, float* inv) {
  return om_layernorm_fwd_b16(ctx, x, gamma, beta, rows, cols, eps, y, nullptr, mean, inv);
}

int32_t om_layernorm_bwd_b16(om_ctx* ctx, const float* g, const float* x, const float* gamma, const float* mean,
                             const float* inv, int32_t rows, int32_t cols, float* dx, uint16_t* dx16, float* dgamma, float* dbeta,
                             int32_t accumulate_params) {
  OM_CHECK_CTX(ctx);
  if (rows < 0 || cols < 0) return fail(ctx, OM_ERR_SHAPE, "om_layernorm_bwd: [%d,%d]", rows, cols);
  if (cols == 0) return OM_OK;
  if (cols > 1024) return fail(ctx, OM_ERR_UNSUPPORTED, "om_layernorm_bwd: rows wider than 1024 (%d) are not implemented", cols);
  if (dx16 && !dx) return fail(ctx, OM_ERR_ARG, "om_layernorm_bwd_b16: the bfloat16 copy needs dx");
  ProfileScope prof(ctx, "om_layernorm_bwd", 0, (dx16 ? 14.0 : 12.0) * rows * (double)cols);
  const int nc = (int)ceil_div(cols, 32);
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec = (cols & 3) == 0 && al16(g) && al16(x) && al16(gamma) && (!dx || al16(dx)) && (!dx16 || (reinterpret_cast<uintptr_t>(dx16) & 7) == 0);
  // One pass: dx and the CTAs' column partials together; the partials are then added in CTA order.
  const int used = (int)ceil_div(rows > 0 ? rows : 1, vec ? kLnVecRows : kLnFusedRows);
  double *pg = nullptr, *pb = nullptr;
  if (dgamma) OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)used * cols, false, (void**)&pg));
  if (dbeta) OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)used * cols, false, (void**)&pb));
  const size_t smem = sizeof(double) * 8 * (size_t)cols;
#define OM_LN_BWD(NC)                                                                                                            \
  do {                                                                                                                           \
    static bool attr_set = false;                                                                                                \
    if (!attr_set) {                                                                                                             \
      OM_CUDA(ctx, cudaFuncSetAttribute(layernorm_bwd_fused_kernel<NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 1024 * 8)); \
      attr_set = true;                                                                                                           \
    }                                                                                                                            \
    launch_chained(ctx, layernorm_bwd_fused_kernel<NC>, used, 256, smem, g, x, gamma, mean, inv, rows, cols, dx, dx16, pg, pb); \
  } while (0)
#define OM_LN_BWDV(NV)                                                                                                           \
  do {                                                                                                                           \
    static bool attr_set = false;                                                                                                \
    if (!attr_set) {                                                                                                             \
      OM_CUDA(ctx, cudaFuncSetAttribute(layernorm_bwd_vec_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 1024 * 8)); \
      attr_set = true;                                                                                                           \
    }                                                                                                                            \
    launch_chained(ctx, layernorm_bwd_vec_kernel<NV>, used, 256, smem, g, x, gamma, mean, inv, rows, cols, dx, dx16, pg, pb);   \
  } while (0)
  const int nvec = (int)ceil_div(cols, 128);
  if (vec && nvec <= 1) OM_LN_BWDV(1);
  else if (vec && nvec <= 2) OM_LN_BWDV(2);
  else if (vec && nvec <= 3) OM_LN_BWDV(3);
  else if (vec && nvec <= 4) OM_LN_BWDV(4);
  else if (vec && nvec <= 6) OM_LN_BWDV(6);
  else if (vec) OM_LN_BWDV(8);
  else if (nc <= 4) OM_LN_BWD(4);
  else if (nc <= 8) OM_LN_BWD(8);
  else if (nc <= 12) OM_LN_BWD(12);
  else if (nc <= 16) OM_LN_BWD(16);
  else if (nc <= 24) OM_LN_BWD(24);
  else OM_LN_BWD(32);
#undef OM_LN_BWD
#undef OM_LN_BWDV
  if (dgamma || dbeta)
    launch_chained(ctx, column_partials_finish_kernel, (unsigned)ceil_div(cols, 32), 1024, 0, pg, pb, used, cols, dgamma, dbeta, accumulate_params);
  if (pg) pool_free(ctx, pg);
  if (pb) pool_free(ctx, pb);
  OM_LAUNCH_CHECK(ctx, "om_layernorm_bwd");
  return OM_OK;
}

int32_t om_layernorm_bwd(om_ctx* ctx, const float* g, const float* x, const float* gamma, const float* mean,
                         const float* inv, int32_t rows, int32_t cols, float* dx, float* dgamma, float* dbeta,
                         int32_t accumulate_params) {
  return om_layernorm_bwd_b16(ctx, g, x, gamma, mean, inv, rows, cols, dx, nullptr, dgamma, dbeta, accumulate_params);
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
    launch_chained(ctx, column_partials_finish_kernel, (unsigned)ceil_div(c, 32), 1024, 0, pa, pb, slices, c, dgamma, dbeta, accumulate_params);
  pool_free(ctx, pa);
  pool_free(ctx, pb);
  OM_LAUNCH_CHECK(ctx, "om_batchnorm_bwd");
  return OM_OK;
}

}  // extern "C"
