// Bandwidth-bound elementwise, copy and broadcast-sum kernels. All are grid-stride, 128-bit vectorised where the
// layout allows, and free of floating-point atomics. The library is compiled with --fmad=false so that a*b+c
// written here rounds twice exactly as the reference's managed code does; fused multiply-adds are explicit fmaf.
#include <cuda_bf16.h>

#include "om_act.cuh"
#include "om_common.cuh"

namespace om {

constexpr int kMaxRank = 8;

struct Strided2 {
  int32_t rank;
  int32_t shape[kMaxRank];
  int64_t sa[kMaxRank];
  int64_t sb[kMaxRank];
};

__device__ __forceinline__ float binary_apply(int op, float a, float b) {
  switch (op) {
    case OM_ADD: return a + b;
    case OM_SUB: return a - b;
    case OM_MUL: return a * b;
    default: return a / b;
  }
}

template <int OP>
__global__ void binary_same_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                   int64_t n4, int64_t n) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float4* a4 = reinterpret_cast<const float4*>(a);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  float4* o4 = reinterpret_cast<float4*>(out);
  for (int64_t j = i; j < n4; j += stride) {
    float4 x = a4[j], y = b4[j], r;
    r.x = binary_apply(OP, x.x, y.x);
    r.y = binary_apply(OP, x.y, y.y);
    r.z = binary_apply(OP, x.z, y.z);
    r.w = binary_apply(OP, x.w, y.w);
    o4[j] = r;
  }
  for (int64_t j = n4 * 4 + i; j < n; j += stride) out[j] = binary_apply(OP, a[j], b[j]);
}

// out[r, c] = a[r, c] (op) b[c]: the bias-add pattern; also a b that spans several trailing axes (a position table added to
// every batch element), the trailing axes then counting as one row of `cols` elements.
template <int OP>
__global__ void binary_rowb_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                   int64_t rows, int32_t cols) {
  pdl_enter();
  int64_t total = rows * cols;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if ((cols & 3) == 0) {
    int64_t n4 = total >> 2;
    int32_t c4 = cols >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    float4* o4 = reinterpret_cast<float4*>(out);
    if (n4 < (int64_t(1) << 31)) {
      // 32-bit index arithmetic: the 64-bit remainder costs more than the memory access it addresses.
      const uint32_t un4 = (uint32_t)n4, uc4 = (uint32_t)c4, ustride = (uint32_t)stride;
      for (uint32_t j = (uint32_t)i; j < un4; j += ustride) {
        float4 x = a4[j], y = b4[j % uc4], r;
        r.x = binary_apply(OP, x.x, y.x);
        r.y = binary_apply(OP, x.y, y.y);
        r.z = binary_apply(OP, x.z, y.z);
        r.w = binary_apply(OP, x.w, y.w);
        o4[j] = r;
        if (j + ustride < j) break;   // the next index would wrap
      }
    } else {
      for (int64_t j = i; j < n4; j += stride) {
        float4 x = a4[j], y = b4[j % c4], r;
        r.x = binary_apply(OP, x.x, y.x);
        r.y = binary_apply(OP, x.y, y.y);
        r.z = binary_apply(OP, x.z, y.z);
        r.w = binary_apply(OP, x.w, y.w);
        o4[j] = r;
      }
    }
  } else {
    for (int64_t j = i; j < total; j += stride) out[j] = binary_apply(OP, a[j], b[j % cols]);
  }
}

__global__ void binary_strided_kernel(int op, Strided2 s, const float* __restrict__ a, const float* __restrict__ b,
                                      float* __restrict__ out, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < n; j += stride) {
    int64_t rem = j, oa = 0, ob = 0;
    for (int ax = s.rank - 1; ax >= 0; ax--) {
      int64_t idx = rem % s.shape[ax];
      rem /= s.shape[ax];
      oa += idx * s.sa[ax];
      ob += idx * s.sb[ax];
    }
    out[j] = binary_apply(op, a[oa], b[ob]);
  }
}

// ---- unary forward / backward ---------------------------------------------------------------------------------

// Four bfloat16 values (round to nearest even) as one 8-byte word.
__device__ __forceinline__ uint2 pack_bf16x4(float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  return make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}
__device__ __forceinline__ uint16_t bf16_of(float v) {
  __nv_bfloat16 h = __float2bfloat16_rn(v);
  return *reinterpret_cast<uint16_t*>(&h);
}

// y16 (may be null): the bfloat16 copy of y, written in the same pass for the product that reads y next.
template <int OP>
__global__ void unary_kernel(const float* __restrict__ x, float* __restrict__ y, uint16_t* __restrict__ y16, int64_t n4, int64_t n) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  float4* y4 = reinterpret_cast<float4*>(y);
  for (int64_t j = i; j < n4; j += stride) {
    float4 v = x4[j], r;
    r.x = unary_apply<OP>(v.x);
    r.y = unary_apply<OP>(v.y);
    r.z = unary_apply<OP>(v.z);
    r.w = unary_apply<OP>(v.w);
    y4[j] = r;
    if (y16) reinterpret_cast<uint2*>(y16)[j] = pack_bf16x4(r);
  }
  for (int64_t j = n4 * 4 + i; j < n; j += stride) {
    const float r = unary_apply<OP>(x[j]);
    y[j] = r;
    if (y16) y16[j] = bf16_of(r);
  }
}

template <int OP>
__global__ void unary_bwd_kernel(const float* __restrict__ g, const float* __restrict__ s, float* __restrict__ dx,
                                 uint16_t* __restrict__ dx16, int64_t n4, int64_t n) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  const float4* s4 = reinterpret_cast<const float4*>(s);
  float4* d4 = reinterpret_cast<float4*>(dx);
  for (int64_t j = i; j < n4; j += stride) {
    float4 a = g4[j], b = s4[j], r;
    r.x = unary_grad<OP>(a.x, b.x);
    r.y = unary_grad<OP>(a.y, b.y);
    r.z = unary_grad<OP>(a.z, b.z);
    r.w = unary_grad<OP>(a.w, b.w);
    d4[j] = r;
    if (dx16) reinterpret_cast<uint2*>(dx16)[j] = pack_bf16x4(r);
  }
  for (int64_t j = n4 * 4 + i; j < n; j += stride) {
    const float r = unary_grad<OP>(g[j], s[j]);
    dx[j] = r;
    if (dx16) dx16[j] = bf16_of(r);
  }
}

__global__ void add_into_kernel(float* dst, const float* __restrict__ src, int64_t n4, int64_t n) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  float4* d4 = reinterpret_cast<float4*>(dst);
  const float4* s4 = reinterpret_cast<const float4*>(src);
  for (int64_t j = i; j < n4; j += stride) {
    float4 a = d4[j], b = s4[j];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    d4[j] = a;
  }
  for (int64_t j = n4 * 4 + i; j < n; j += stride) dst[j] += src[j];
}

__global__ void div_scalar_kernel(const float* __restrict__ x, float d, float* __restrict__ y, int64_t n) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < n; j += stride) y[j] = x[j] / d;
}

__global__ void fill_kernel(float* __restrict__ dst, float v, int64_t n) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < n; j += stride) dst[j] = v;
}

constexpr int kZeroTensors = 64;
struct ZeroTable {
  float* p[kZeroTensors];
  int64_t len[kZeroTensors];
  int32_t count;
};

// blockIdx.y selects the tensor; each tensor is zeroed by gridDim.x CTAs.
__global__ void multi_zero_kernel(ZeroTable t) {
  pdl_enter();
  float* p = t.p[blockIdx.y];
  int64_t n = t.len[blockIdx.y];
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    float4* p4 = reinterpret_cast<float4*>(p);
    int64_t n4 = n >> 2;
    float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t j = i; j < n4; j += stride) p4[j] = z;
    for (int64_t j = n4 * 4 + i; j < n; j += stride) p[j] = 0.f;
  } else {
    for (int64_t j = i; j < n; j += stride) p[j] = 0.f;
  }
}

// ---- strided copy -------------------------------------------------------------------------------------------------

__global__ void strided_copy_kernel(Strided2 s, const float* __restrict__ src, float* __restrict__ dst, int64_t n) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < n; j += stride) {
    int64_t rem = j, oa = 0, ob = 0;
    for (int ax = s.rank - 1; ax >= 0; ax--) {
      int64_t idx = rem % s.shape[ax];
      rem /= s.shape[ax];
      oa += idx * s.sa[ax];
      ob += idx * s.sb[ax];
    }
    dst[ob] = src[oa];
  }
}

// Same with the innermost axis contiguous on both sides and a multiple of 4 elements, 16-byte aligned: one float4
// per thread-iteration.
__global__ void strided_copy_vec4_kernel(Strided2 s, const float* __restrict__ src, float* __restrict__ dst,
                                         int64_t n4) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int32_t inner4 = s.shape[s.rank - 1] >> 2;
  for (int64_t j = i; j < n4; j += stride) {
    int64_t rem = j / inner4;
    int64_t in = (j % inner4) * 4;
    int64_t oa = in, ob = in;
    for (int ax = s.rank - 2; ax >= 0; ax--) {
      int64_t idx = rem % s.shape[ax];
      rem /= s.shape[ax];
      oa += idx * s.sa[ax];
      ob += idx * s.sb[ax];
    }
    *reinterpret_cast<float4*>(dst + ob) = *reinterpret_cast<const float4*>(src + oa);
  }
}

// 2-D transpose through a padded shared tile: dst[c, r] = src[r, c].
__global__ void transpose2d_kernel(const float* __restrict__ src, float* __restrict__ dst, int32_t rows, int32_t cols,
                                   int64_t src_ld, int64_t dst_ld) {
  pdl_enter();
  __shared__ float tile[32][33];
  int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int rr = by + r, cc = bx + threadIdx.x;
    if (rr < rows && cc < cols) tile[r][threadIdx.x] = src[(int64_t)rr * src_ld + cc];
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int cc = bx + r, rr = by + threadIdx.x;
    if (rr < rows && cc < cols) dst[(int64_t)cc * dst_ld + rr] = tile[threadIdx.x][r];
  }
}

// ---- broadcast sums ---------------------------------------------------------------------------------------------

constexpr int kColsumRowsPerChunk = 512;

constexpr int kColsumLanes = 32;

// Stage 2 inside stage 1: the CTA that arrives last for its 32 columns (all chunks' partial sums are then in memory)
// adds them in increasing chunk order, exactly as colsum_stage2_kernel does, and resets the arrival counter for the next
// launch. Which CTA arrives last does not matter for the result. `tid` is the thread's linear index in the CTA.
template <int COLS = 32>
__device__ __forceinline__ void colsum_finish(const double* __restrict__ partial, unsigned* __restrict__ arrival, float* __restrict__ out,
                                              int accumulate, int32_t cols, int tid, int* is_last) {
  __syncthreads();
  if (tid == 0) *is_last = atomicAdd(&arrival[blockIdx.x], 1u) == gridDim.y - 1;
  __syncthreads();
  if (!*is_last) return;
  __threadfence();
  if (tid < COLS) {
    const int c = blockIdx.x * COLS + tid;
    if (c < cols) {
      // Sixteen loads are on their way before the first add; the adds stay in increasing chunk order.
      double t = 0.0;
      unsigned ch = 0;
      for (; ch + 16 <= gridDim.y; ch += 16) {
        double v[16];
#pragma unroll
        for (int u = 0; u < 16; u++) v[u] = __ldcg(partial + (int64_t)(ch + u) * cols + c);
#pragma unroll
        for (int u = 0; u < 16; u++) t += v[u];
      }
      for (; ch < gridDim.y; ch++) t += __ldcg(partial + (int64_t)ch * cols + c);
      const float r = (float)t;
      out[c] = accumulate ? out[c] + r : r;
    }
  }
  if (tid == 0) arrival[blockIdx.x] = 0u;
}

// Stage 1 of a column sum over g[rows, cols]: CTA (bx, by) owns 32 columns and one chunk of kColsumRowsPerChunk rows.
// 32 row-lanes per column accumulate in double over rows lane, lane+32, ...; the 32 lane sums are combined in lane
// order. partial[chunk, col] is written in double.
__global__ void __launch_bounds__(1024)
colsum_stage1_kernel(const float* __restrict__ g, int32_t rows, int32_t cols, int64_t ld, double* __restrict__ partial,
                     unsigned* __restrict__ arrival, float* __restrict__ out, int accumulate) {
  pdl_enter();
  __shared__ double sm[kColsumLanes][33];
  __shared__ int is_last;
  int col = blockIdx.x * 32 + threadIdx.x;
  int r0 = blockIdx.y * kColsumRowsPerChunk;
  int r1 = min(rows, r0 + kColsumRowsPerChunk);
  double acc = 0.0;
  if (col < cols) {
    for (int r = r0 + threadIdx.y; r < r1; r += kColsumLanes) acc += (double)g[(int64_t)r * ld + col];
  }
  sm[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < cols) {
    double t = 0.0;
#pragma unroll
    for (int l = 0; l < kColsumLanes; l++) t += sm[l][threadIdx.x];
    partial[(int64_t)blockIdx.y * cols + col] = t;
    __threadfence();
  }
  if (arrival != nullptr) colsum_finish(partial, arrival, out, accumulate, cols, threadIdx.y * 32 + threadIdx.x, &is_last);
}

// Stage 1 for rows that are 16-byte aligned (ld a multiple of four, aligned base): the same sums in the same order as
// colsum_stage1_kernel, but each thread owns four adjacent columns (one 16-byte load per row) and has all of its 16
// rows in flight at once. A CTA is 8 column groups x 32 row lanes and covers 32 columns of one chunk.
__global__ void __launch_bounds__(256)
colsum_stage1_vec4_kernel(const float* __restrict__ g, int32_t rows, int32_t cols, int64_t ld, double* __restrict__ partial,
                          unsigned* __restrict__ arrival, float* __restrict__ out, int accumulate) {
  pdl_enter();
  __shared__ double sm[kColsumLanes][33];
  __shared__ int is_last;
  constexpr int PER_LANE = kColsumRowsPerChunk / kColsumLanes;
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  const int col = blockIdx.x * 32 + tx * 4;
  const int r0 = blockIdx.y * kColsumRowsPerChunk;
  const int r1 = min(rows, r0 + kColsumRowsPerChunk);
  double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
  if (col + 3 < cols) {
    float4 v[PER_LANE];
#pragma unroll
    for (int u = 0; u < PER_LANE; u++) {
      const int r = r0 + ty + kColsumLanes * u;
      v[u] = r < r1 ? __ldg(reinterpret_cast<const float4*>(g + (int64_t)r * ld + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < PER_LANE; u++) {
      if (r0 + ty + kColsumLanes * u < r1) {
        a0 += (double)v[u].x; a1 += (double)v[u].y; a2 += (double)v[u].z; a3 += (double)v[u].w;
      }
    }
  } else if (col < cols) {
    for (int r = r0 + ty; r < r1; r += kColsumLanes) {
      const float* row = g + (int64_t)r * ld + col;
      a0 += (double)row[0];
      if (col + 1 < cols) a1 += (double)row[1];
      if (col + 2 < cols) a2 += (double)row[2];
    }
  }
  sm[ty][tx * 4 + 0] = a0; sm[ty][tx * 4 + 1] = a1; sm[ty][tx * 4 + 2] = a2; sm[ty][tx * 4 + 3] = a3;
  __syncthreads();
  if (threadIdx.x < 32) {
    const int c = blockIdx.x * 32 + threadIdx.x;
    if (c < cols) {
      double t = 0.0;
#pragma unroll
      for (int l = 0; l < kColsumLanes; l++) t += sm[l][threadIdx.x];
      partial[(int64_t)blockIdx.y * cols + c] = t;
      __threadfence();
    }
  }
  if (arrival != nullptr) colsum_finish(partial, arrival, out, accumulate, cols, threadIdx.x, &is_last);
}

// The column sums of a bfloat16 matrix (the copy of an output gradient that the products read): the same partition as above
// (chunks of 512 rows, 32 row lanes), a thread owning eight adjacent columns (one 16-byte load per row) with its 16 rows in
// flight at once; a CTA covers 64 columns of a chunk. A thread adds its 16 rows in fp32, in increasing row order (the
// conversion of every element to double made the kernel arithmetic-bound at 3 TB/s); the 32 lane sums of a chunk and then
// the chunks are combined in double, in increasing order. The order is fixed, so the same input gives the same bits.
__device__ __forceinline__ void add_bf16x8(float (&a)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int q = 0; q < 4; q++) {
    a[2 * q] += __uint_as_float(w[q] << 16);
    a[2 * q + 1] += __uint_as_float(w[q] & 0xFFFF0000u);
  }
}
__global__ void __launch_bounds__(256, 3)
colsum16_stage1_kernel(const uint16_t* __restrict__ g, int32_t rows, int32_t cols, int64_t ld, double* __restrict__ partial,
                       unsigned* __restrict__ arrival, float* __restrict__ out, int accumulate) {
  pdl_enter();
  __shared__ float sm[kColsumLanes][65];
  __shared__ int is_last;
  constexpr int PER_LANE = kColsumRowsPerChunk / kColsumLanes;
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  const int col = blockIdx.x * 64 + tx * 8;
  const int r0 = blockIdx.y * kColsumRowsPerChunk;
  const int r1 = min(rows, r0 + kColsumRowsPerChunk);
  float a[8];
#pragma unroll
  for (int q = 0; q < 8; q++) a[q] = 0.f;
  if (col + 7 < cols) {
    uint4 v[PER_LANE];
#pragma unroll
    for (int u = 0; u < PER_LANE; u++) {
      const int r = r0 + ty + kColsumLanes * u;
      v[u] = r < r1 ? __ldg(reinterpret_cast<const uint4*>(g + (int64_t)r * ld + col)) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < PER_LANE; u++)
      if (r0 + ty + kColsumLanes * u < r1) add_bf16x8(a, v[u]);
  } else if (col < cols) {
    for (int r = r0 + ty; r < r1; r += kColsumLanes)
      for (int q = 0; q < 8 && col + q < cols; q++) a[q] += __uint_as_float((uint32_t)g[(int64_t)r * ld + col + q] << 16);
  }
#pragma unroll
  for (int q = 0; q < 8; q++) sm[ty][tx * 8 + q] = a[q];
  __syncthreads();
  if (threadIdx.x < 64) {
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < cols) {
      double t = 0.0;
#pragma unroll
      for (int l = 0; l < kColsumLanes; l++) t += (double)sm[l][threadIdx.x];
      partial[(int64_t)blockIdx.y * cols + c] = t;
      __threadfence();
    }
  }
  if (arrival != nullptr) colsum_finish<64>(partial, arrival, out, accumulate, cols, threadIdx.x, &is_last);
}

__global__ void colsum_stage2_kernel(const double* __restrict__ partial, int32_t chunks, int32_t cols,
                                     float* __restrict__ out, int accumulate) {
  pdl_enter();
  int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  double t = 0.0;
  for (int c = 0; c < chunks; c++) t += partial[(int64_t)c * cols + col];
  float r = (float)t;
  out[col] = accumulate ? out[col] + r : r;
}

// Row sums: out[r] = sum_c g[r, c]; one warp per row, lanes stride the row, lane sums combined by a fixed
// butterfly (xor shuffle) so every lane ends with the same bits.
__global__ void rowsum_kernel(const float* __restrict__ g, int64_t rows, int32_t cols, float* __restrict__ out) {
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  int warps = (gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp; r < rows; r += warps) {
    double acc = 0.0;
    for (int c = lane; c < cols; c += 32) acc += (double)g[r * cols + c];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[r] = (float)acc;
  }
}

struct SumToShape {
  int32_t rank;
  int32_t shape[kMaxRank];
  int64_t ts[kMaxRank];   // target stride per axis of g (0 on reduced axes)
  int64_t gs[kMaxRank];   // contiguous strides of g
};

// Generic fallback: one thread per output element walks every source element that maps to it in increasing source
// order (the reference's order) with a double accumulator.
__global__ void sum_to_generic_kernel(SumToShape s, const float* __restrict__ g, float* __restrict__ out,
                                      int64_t out_len) {
  int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (o >= out_len) return;
  // Decompose o over the kept axes (those with ts != 0), ordered by decreasing target stride = increasing axis.
  int64_t base = 0, rem = o;
  int32_t red_shape[kMaxRank];
  int64_t red_stride[kMaxRank];
  int nred = 0;
  int64_t count = 1;
  for (int ax = 0; ax < s.rank; ax++) {
    if (s.ts[ax] != 0) {
      int64_t idx = rem / s.ts[ax];
      rem -= idx * s.ts[ax];
      base += idx * s.gs[ax];
    } else {
      red_shape[nred] = s.shape[ax];
      red_stride[nred] = s.gs[ax];
      count *= s.shape[ax];
      nred++;
    }
  }
  double acc = 0.0;
  for (int64_t j = 0; j < count; j++) {
    int64_t r = j, off = base;
    for (int a = nred - 1; a >= 0; a--) {
      off += (r % red_shape[a]) * red_stride[a];
      r /= red_shape[a];
    }
    acc += (double)g[off];
  }
  out[o] = (float)acc;
}

// Sum/Mean over the middle axis of [outer, n, inner] with a double accumulator in increasing order.
__global__ void reduce_fwd_kernel(const float* __restrict__ x, int64_t outer, int64_t n, int64_t inner, int mean,
                                  float* __restrict__ y) {
  int64_t total = outer * inner;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < total; j += stride) {
    int64_t o = j / inner, in = j % inner;
    double acc = 0.0;
    for (int64_t k = 0; k < n; k++) acc += (double)x[(o * n + k) * inner + in];
    y[j] = mean ? (float)(acc / (double)n) : (float)acc;
  }
}

// Whole-tensor sum with one CTA (used for rank-0 results): fixed partition over 1024 threads, fixed tree.
__global__ void reduce_all_kernel(const float* __restrict__ x, int64_t n, int mean, float* __restrict__ y) {
  __shared__ double sm[1024];
  double acc = 0.0;
  for (int64_t j = threadIdx.x; j < n; j += 1024) acc += (double)x[j];
  sm[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) sm[threadIdx.x] += sm[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) y[0] = mean ? (float)(sm[0] / (double)n) : (float)sm[0];
}

__global__ void reduce_bwd_kernel(const float* __restrict__ g, int64_t outer, int64_t n, int64_t inner, int mean,
                                  float* __restrict__ dx) {
  int64_t total = outer * n * inner;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  float fn = (float)n;
  for (int64_t j = i; j < total; j += stride) {
    int64_t in = j % inner;
    int64_t o = j / (inner * n);
    float v = g[o * inner + in];
    dx[j] = mean ? v / fn : v;
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Column sums of g[rows, cols] whose rows are ld elements apart.
int32_t colsum_ld(om_ctx* ctx, const float* g, int32_t rows, int32_t cols, int64_t ld, float* out, int32_t accumulate) {
  if (rows < 0 || cols < 0) return fail(ctx, OM_ERR_SHAPE, "om_colsum: [%d,%d]", rows, cols);
  if (cols == 0) return OM_OK;
  ProfileScope prof(ctx, "om_colsum", 0, 4.0 * rows * cols + 4.0 * cols);
  int chunks = (int)ceil_div(rows > 0 ? rows : 1, kColsumRowsPerChunk);
  double* partial = nullptr;
  OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)chunks * cols, false, (void**)&partial));
  dim3 grid((unsigned)ceil_div(cols, 32), (unsigned)chunks);
  // One launch when the context's arrival counters cover the column blocks: the last CTA of each block of 32 columns
  // does stage 2. Wider matrices take the two launches.
  unsigned* arrival = grid.x <= (unsigned)kArrivalSlots ? ctx->arrival[ctx->aux_active ? 1 : 0] : nullptr;
  if ((ld & 3) == 0 && aligned16(g))
    launch_chained(ctx, colsum_stage1_vec4_kernel, grid, 256, 0, g, rows, cols, ld, partial, arrival, out, accumulate);
  else
    launch_chained(ctx, colsum_stage1_kernel, grid, dim3(32, kColsumLanes), 0, g, rows, cols, ld, partial, arrival, out, accumulate);
  if (arrival == nullptr)
    launch_chained(ctx, colsum_stage2_kernel, (unsigned)ceil_div(cols, 128), 128, 0, partial, chunks, cols, out, accumulate);
  pool_free(ctx, partial);
  OM_LAUNCH_CHECK(ctx, "om_colsum");
  return OM_OK;
}

// out[c] (+)= sum over rows of the bfloat16 matrix g16[rows, cols] with pitch ld (a multiple of 8, 16-byte aligned base).
int32_t colsum16_ld(om_ctx* ctx, const uint16_t* g16, int32_t rows, int32_t cols, int64_t ld, float* out, int32_t accumulate) {
  if (rows < 0 || cols < 0) return fail(ctx, OM_ERR_SHAPE, "om_colsum_bf16: [%d,%d]", rows, cols);
  if (cols == 0) return OM_OK;
  if ((ld & 7) || (reinterpret_cast<uintptr_t>(g16) & 15)) return fail(ctx, OM_ERR_UNSUPPORTED, "om_colsum_bf16: the pitch must be a multiple of 8 and the base 16-byte aligned");
  ProfileScope prof(ctx, "om_colsum", 0, 2.0 * rows * cols + 4.0 * cols);
  int chunks = (int)ceil_div(rows > 0 ? rows : 1, kColsumRowsPerChunk);
  double* partial = nullptr;
  OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)chunks * cols, false, (void**)&partial));
  dim3 grid((unsigned)ceil_div(cols, 64), (unsigned)chunks);
  unsigned* arrival = grid.x <= (unsigned)kArrivalSlots ? ctx->arrival[ctx->aux_active ? 1 : 0] : nullptr;
  launch_chained(ctx, colsum16_stage1_kernel, grid, 256, 0, g16, rows, cols, ld, partial, arrival, out, accumulate);
  if (arrival == nullptr)
    launch_chained(ctx, colsum_stage2_kernel, (unsigned)ceil_div(cols, 128), 128, 0, partial, chunks, cols, out, accumulate);
  pool_free(ctx, partial);
  OM_LAUNCH_CHECK(ctx, "om_colsum_bf16");
  return OM_OK;
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_colsum_bf16(om_ctx* ctx, const uint16_t* g16, int32_t rows, int32_t cols, int32_t ld, float* out, int32_t accumulate) {
  OM_CHECK_CTX(ctx);
  if (ld < cols) return fail(ctx, OM_ERR_SHAPE, "om_colsum_bf16: pitch %d below %d columns", ld, cols);
  return colsum16_ld(ctx, g16, rows, cols, ld, out, accumulate);
}

int32_t om_binary(om_ctx* ctx, int32_t op, int32_t rank, const int32_t* shape, const float* a,
                  const int64_t* a_strides, const float* b, const int64_t* b_strides, float* out) {
  OM_CHECK_CTX(ctx);
  if (rank < 0 || rank > kMaxRank || op < 0 || op > OM_DIV) return fail(ctx, OM_ERR_ARG, "om_binary: rank %d op %d", rank, op);
  int64_t n = 1;
  for (int i = 0; i < rank; i++) {
    if (shape[i] < 0) return fail(ctx, OM_ERR_SHAPE, "om_binary: negative extent");
    n *= shape[i];
  }
  if (n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_binary", 0, 12.0 * n);
  // Classify: both contiguous at the full shape, or a contiguous and b contiguous over some trailing axes and broadcast
  // (stride 0) over all the axes in front of them: a row vector, or a table added to every batch element.
  bool a_contig = true, b_contig = true, b_row = rank >= 1;
  int64_t acc = 1, b_period = 1;
  bool in_tail = true;
  for (int ax = rank - 1; ax >= 0; ax--) {
    if (shape[ax] != 1) {
      if (a_strides[ax] != acc) a_contig = false;
      if (b_strides[ax] != acc) b_contig = false;
      if (in_tail && b_strides[ax] == acc && (ax == rank - 1 || b_strides[ax] != 0)) b_period = acc * shape[ax];
      else {
        in_tail = false;
        if (b_strides[ax] != 0) b_row = false;
      }
    }
    acc *= shape[ax];
  }
  if (b_period <= 1 || b_period > INT32_MAX) b_row = false;
  const int threads = 256;
  if (a_contig && b_contig) {
    bool vec = aligned16(a) && aligned16(b) && aligned16(out);
    int64_t n4 = vec ? n / 4 : 0;
    int grid = grid_for(ctx, vec ? (n + 3) / 4 : n, threads);
    switch (op) {
      case OM_ADD: launch_chained(ctx, binary_same_kernel<OM_ADD>, grid, threads, 0, a, b, out, n4, n); break;
      case OM_SUB: launch_chained(ctx, binary_same_kernel<OM_SUB>, grid, threads, 0, a, b, out, n4, n); break;
      case OM_MUL: launch_chained(ctx, binary_same_kernel<OM_MUL>, grid, threads, 0, a, b, out, n4, n); break;
      default: launch_chained(ctx, binary_same_kernel<OM_DIV>, grid, threads, 0, a, b, out, n4, n); break;
    }
  } else if (a_contig && b_row && aligned16(a) && aligned16(b) && aligned16(out)) {
    int32_t cols = (int32_t)b_period;
    int64_t rows = n / cols;
    int grid = grid_for(ctx, (n + 3) / 4, threads);
    switch (op) {
      case OM_ADD: launch_chained(ctx, binary_rowb_kernel<OM_ADD>, grid, threads, 0, a, b, out, rows, cols); break;
      case OM_SUB: launch_chained(ctx, binary_rowb_kernel<OM_SUB>, grid, threads, 0, a, b, out, rows, cols); break;
      case OM_MUL: launch_chained(ctx, binary_rowb_kernel<OM_MUL>, grid, threads, 0, a, b, out, rows, cols); break;
      default: launch_chained(ctx, binary_rowb_kernel<OM_DIV>, grid, threads, 0, a, b, out, rows, cols); break;
    }
  } else {
    Strided2 s;
    s.rank = rank;
    for (int i = 0; i < rank; i++) {
      s.shape[i] = shape[i];
      s.sa[i] = a_strides[i];
      s.sb[i] = b_strides[i];
    }
    binary_strided_kernel<<<grid_for(ctx, n, threads), threads, 0, ctx->stream>>>(op, s, a, b, out, n);
  }
  OM_LAUNCH_CHECK(ctx, "om_binary");
  return OM_OK;
}

#define OM_UNARY_DISPATCH(KERNEL, ...)                                                             \
  switch (op) {                                                                                    \
    case OM_UNARY_NONE: launch_chained(ctx, KERNEL<OM_UNARY_NONE>, grid, threads, 0, __VA_ARGS__); break; \
    case OM_RELU: launch_chained(ctx, KERNEL<OM_RELU>, grid, threads, 0, __VA_ARGS__); break;          \
    case OM_GELU_ERF: launch_chained(ctx, KERNEL<OM_GELU_ERF>, grid, threads, 0, __VA_ARGS__); break;  \
    case OM_GELU_TANH: launch_chained(ctx, KERNEL<OM_GELU_TANH>, grid, threads, 0, __VA_ARGS__); break; \
    case OM_SIGMOID: launch_chained(ctx, KERNEL<OM_SIGMOID>, grid, threads, 0, __VA_ARGS__); break;    \
    case OM_TANH: launch_chained(ctx, KERNEL<OM_TANH>, grid, threads, 0, __VA_ARGS__); break;          \
    case OM_NEG: launch_chained(ctx, KERNEL<OM_NEG>, grid, threads, 0, __VA_ARGS__); break;            \
    case OM_EXP: launch_chained(ctx, KERNEL<OM_EXP>, grid, threads, 0, __VA_ARGS__); break;            \
    case OM_SQRT: launch_chained(ctx, KERNEL<OM_SQRT>, grid, threads, 0, __VA_ARGS__); break;          \
    case OM_ERF: launch_chained(ctx, KERNEL<OM_ERF>, grid, threads, 0, __VA_ARGS__); break;            \
    default: return fail(ctx, OM_ERR_ARG, "unknown unary op %d", op);                              \
  }

int32_t om_unary_b16(om_ctx* ctx, int32_t op, const float* x, float* y, uint16_t* y16, int64_t n) {
  OM_CHECK_CTX(ctx);
  if (n < 0) return fail(ctx, OM_ERR_SHAPE, "om_unary: n %lld", (long long)n);
  if (n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_unary", 0, (y16 ? 10.0 : 8.0) * n);
  bool vec = aligned16(x) && aligned16(y) && (!y16 || (reinterpret_cast<uintptr_t>(y16) & 7) == 0);
  int64_t n4 = vec ? n / 4 : 0;
  const int threads = 256;
  int grid = grid_for(ctx, vec ? (n + 3) / 4 : n, threads);
  // With a bfloat16 copy to write (the bfloat16-operand tier) the erf GELU takes its short form (om_act.cuh), the same that
  // the product epilogues apply.
  if (op == OM_GELU_ERF && y16) launch_chained(ctx, unary_kernel<OM_GELU_ERF_FAST>, grid, threads, 0, x, y, y16, n4, n);
  else OM_UNARY_DISPATCH(unary_kernel, x, y, y16, n4, n)
  OM_LAUNCH_CHECK(ctx, "om_unary");
  return OM_OK;
}

int32_t om_unary(om_ctx* ctx, int32_t op, const float* x, float* y, int64_t n) { return om_unary_b16(ctx, op, x, y, nullptr, n); }

int32_t om_unary_bwd_b16(om_ctx* ctx, int32_t op, const float* g, const float* saved, float* dx, uint16_t* dx16, int64_t n) {
  OM_CHECK_CTX(ctx);
  if (n < 0) return fail(ctx, OM_ERR_SHAPE, "om_unary_bwd: n %lld", (long long)n);
  if (n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_unary_bwd", 0, (dx16 ? 14.0 : 12.0) * n);
  bool vec = aligned16(g) && aligned16(saved) && aligned16(dx) && (!dx16 || (reinterpret_cast<uintptr_t>(dx16) & 7) == 0);
  int64_t n4 = vec ? n / 4 : 0;
  const int threads = 256;
  int grid = grid_for(ctx, vec ? (n + 3) / 4 : n, threads);
  if (op == OM_GELU_ERF && dx16) launch_chained(ctx, unary_bwd_kernel<OM_GELU_ERF_FAST>, grid, threads, 0, g, saved, dx, dx16, n4, n);
  else OM_UNARY_DISPATCH(unary_bwd_kernel, g, saved, dx, dx16, n4, n)
  OM_LAUNCH_CHECK(ctx, "om_unary_bwd");
  return OM_OK;
}

int32_t om_unary_bwd(om_ctx* ctx, int32_t op, const float* g, const float* saved, float* dx, int64_t n) {
  return om_unary_bwd_b16(ctx, op, g, saved, dx, nullptr, n);
}

int32_t om_add_into(om_ctx* ctx, float* dst, const float* src, int64_t n) {
  OM_CHECK_CTX(ctx);
  if (n <= 0) return n == 0 ? OM_OK : fail(ctx, OM_ERR_SHAPE, "om_add_into: n < 0");
  ProfileScope prof(ctx, "om_add_into", 0, 12.0 * n);
  bool vec = aligned16(dst) && aligned16(src);
  int64_t n4 = vec ? n / 4 : 0;
  const int threads = 256;
  launch_chained(ctx, add_into_kernel, grid_for(ctx, vec ? (n + 3) / 4 : n, threads), threads, 0, dst, src, n4, n);
  OM_LAUNCH_CHECK(ctx, "om_add_into");
  return OM_OK;
}

int32_t om_div_scalar(om_ctx* ctx, const float* x, float d, float* y, int64_t n) {
  OM_CHECK_CTX(ctx);
  if (n <= 0) return OM_OK;
  ProfileScope prof(ctx, "om_div_scalar", 0, 8.0 * n);
  launch_chained(ctx, div_scalar_kernel, grid_for(ctx, n, 256), 256, 0, x, d, y, n);
  OM_LAUNCH_CHECK(ctx, "om_div_scalar");
  return OM_OK;
}

int32_t om_fill(om_ctx* ctx, float* dst, float value, int64_t n) {
  OM_CHECK_CTX(ctx);
  if (n <= 0) return OM_OK;
  ProfileScope prof(ctx, "om_fill", 0, 4.0 * n);
  launch_chained(ctx, fill_kernel, grid_for(ctx, n, 256), 256, 0, dst, value, n);
  OM_LAUNCH_CHECK(ctx, "om_fill");
  return OM_OK;
}

int32_t om_zero(om_ctx* ctx, int32_t count, float* const* ptrs, const int64_t* len) {
  OM_CHECK_CTX(ctx);
  if (count < 0) return fail(ctx, OM_ERR_ARG, "om_zero: count < 0");
  double bytes = 0;
  for (int i = 0; i < count; i++) bytes += 4.0 * len[i];
  ProfileScope prof(ctx, "om_zero", 0, bytes);
  for (int base = 0; base < count; base += kZeroTensors) {
    ZeroTable t;
    int c = 0;
    int64_t longest = 0;
    for (int i = base; i < count && c < kZeroTensors; i++) {
      if (len[i] <= 0) continue;
      t.p[c] = ptrs[i];
      t.len[c] = len[i];
      if (len[i] > longest) longest = len[i];
      c++;
    }
    if (c == 0) continue;
    t.count = c;
    int gx = (int)std::min<int64_t>(ceil_div(longest, 256 * 4 * 4), 4 * ctx->sm_count);
    if (gx < 1) gx = 1;
    launch_chained(ctx, multi_zero_kernel, dim3(gx, c), 256, 0, t);
    OM_LAUNCH_CHECK(ctx, "om_zero");
  }
  return OM_OK;
}

int32_t om_strided_copy(om_ctx* ctx, int32_t rank, const int32_t* shape, const float* src,
                        const int64_t* src_strides, float* dst, const int64_t* dst_strides) {
  OM_CHECK_CTX(ctx);
  if (rank < 0 || rank > kMaxRank) return fail(ctx, OM_ERR_ARG, "om_strided_copy: rank %d", rank);
  // Drop extent-1 axes and merge axes that are contiguous on both sides.
  Strided2 s;
  s.rank = 0;
  int64_t n = 1;
  for (int i = 0; i < rank; i++) {
    if (shape[i] < 0) return fail(ctx, OM_ERR_SHAPE, "om_strided_copy: negative extent");
    n *= shape[i];
    if (shape[i] == 1) continue;
    if (s.rank > 0 && s.sa[s.rank - 1] == src_strides[i] * shape[i] && s.sb[s.rank - 1] == dst_strides[i] * shape[i]) {
      s.shape[s.rank - 1] *= shape[i];
      s.sa[s.rank - 1] = src_strides[i];
      s.sb[s.rank - 1] = dst_strides[i];
    } else {
      s.shape[s.rank] = shape[i];
      s.sa[s.rank] = src_strides[i];
      s.sb[s.rank] = dst_strides[i];
      s.rank++;
    }
  }
  if (n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_strided_copy", 0, 8.0 * n);
  if (s.rank == 0) {
    s.rank = 1;
    s.shape[0] = 1;
    s.sa[0] = s.sb[0] = 1;
  }
  const int threads = 256;
  if (s.rank == 1 && s.sa[0] == 1 && s.sb[0] == 1) {
    OM_CUDA(ctx, cudaMemcpyAsync(dst, src, n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    return OM_OK;
  }
  if (s.rank == 2 && s.sa[1] != 1 && s.sa[0] == 1 && s.sb[1] == 1) {
    // dst[r, c] = src[c * ld + r]: a plain 2-D transpose.
    dim3 grid((unsigned)ceil_div(s.shape[0], 32), (unsigned)ceil_div(s.shape[1], 32));
    if (grid.y <= 65535) {
      launch_chained(ctx, transpose2d_kernel, grid, dim3(32, 8), 0, src, dst, s.shape[1], s.shape[0], s.sa[1], s.sb[0]);
      OM_LAUNCH_CHECK(ctx, "om_strided_copy(transpose)");
      return OM_OK;
    }
  }
  bool vec = s.sa[s.rank - 1] == 1 && s.sb[s.rank - 1] == 1 && (s.shape[s.rank - 1] & 3) == 0 && aligned16(src) &&
             aligned16(dst);
  if (vec)
    for (int i = 0; i < s.rank - 1; i++)
      if ((s.sa[i] & 3) || (s.sb[i] & 3)) vec = false;
  if (vec) {
    launch_chained(ctx, strided_copy_vec4_kernel, grid_for(ctx, n / 4, threads), threads, 0, s, src, dst, n / 4);
  } else {
    launch_chained(ctx, strided_copy_kernel, grid_for(ctx, n, threads), threads, 0, s, src, dst, n);
  }
  OM_LAUNCH_CHECK(ctx, "om_strided_copy");
  return OM_OK;
}

int32_t om_colsum(om_ctx* ctx, const float* g, int32_t rows, int32_t cols, float* out, int32_t accumulate) {
  OM_CHECK_CTX(ctx);
  return colsum_ld(ctx, g, rows, cols, cols, out, accumulate);
}

int32_t om_sum_to(om_ctx* ctx, int32_t rank, const int32_t* shape, const float* g, const int64_t* t_strides,
                  float* out, int64_t out_len) {
  OM_CHECK_CTX(ctx);
  if (rank < 0 || rank > kMaxRank) return fail(ctx, OM_ERR_ARG, "om_sum_to: rank %d", rank);
  int64_t n = 1;
  for (int i = 0; i < rank; i++) n *= shape[i];
  if (out_len == 0) return OM_OK;
  if (n == 0) return om_fill(ctx, out, 0.f, out_len);
  // Leading axes reduced, trailing axes kept and contiguous: column sums.
  int split = 0;
  while (split < rank && (t_strides[split] == 0 || shape[split] == 1)) split++;
  bool tail_kept = true;
  int64_t acc = 1;
  for (int ax = rank - 1; ax >= split; ax--) {
    if (shape[ax] != 1 && t_strides[ax] != acc) tail_kept = false;
    acc *= shape[ax];
  }
  if (tail_kept && acc == out_len && n / acc <= INT32_MAX && acc <= INT32_MAX)
    return om_colsum(ctx, g, (int32_t)(n / acc), (int32_t)acc, out, 0);
  // Leading axes kept and contiguous, trailing axes reduced: row sums.
  int tsplit = rank;
  while (tsplit > 0 && (t_strides[tsplit - 1] == 0 || shape[tsplit - 1] == 1)) tsplit--;
  int64_t inner = 1;
  for (int ax = tsplit; ax < rank; ax++) inner *= shape[ax];
  bool head_kept = true;
  acc = 1;
  for (int ax = tsplit - 1; ax >= 0; ax--) {
    if (shape[ax] != 1 && t_strides[ax] != acc) head_kept = false;
    acc *= shape[ax];
  }
  ProfileScope prof(ctx, "om_sum_to", 0, 4.0 * n + 4.0 * out_len);
  if (head_kept && acc == out_len && inner <= INT32_MAX) {
    int threads = 256;
    rowsum_kernel<<<grid_for(ctx, out_len * 32, threads), threads, 0, ctx->stream>>>(g, out_len, (int32_t)inner, out);
    OM_LAUNCH_CHECK(ctx, "om_sum_to(rows)");
    return OM_OK;
  }
  SumToShape s;
  s.rank = rank;
  int64_t gs = 1;
  for (int ax = rank - 1; ax >= 0; ax--) {
    s.shape[ax] = shape[ax];
    s.ts[ax] = shape[ax] == 1 ? 0 : t_strides[ax];
    s.gs[ax] = gs;
    gs *= shape[ax];
  }
  sum_to_generic_kernel<<<(unsigned)ceil_div(out_len, 128), 128, 0, ctx->stream>>>(s, g, out, out_len);
  OM_LAUNCH_CHECK(ctx, "om_sum_to");
  return OM_OK;
}

int32_t om_reduce_fwd(om_ctx* ctx, const float* x, int64_t outer, int64_t n, int64_t inner, int32_t mean, float* y) {
  OM_CHECK_CTX(ctx);
  if (outer < 0 || n < 0 || inner < 0) return fail(ctx, OM_ERR_SHAPE, "om_reduce_fwd: negative extent");
  if (outer * inner == 0) return OM_OK;
  ProfileScope prof(ctx, "om_reduce_fwd", 0, 4.0 * outer * n * inner);
  if (outer * inner == 1 && n > 4096) {
    reduce_all_kernel<<<1, 1024, 0, ctx->stream>>>(x, n, mean, y);
  } else {
    reduce_fwd_kernel<<<grid_for(ctx, outer * inner, 128), 128, 0, ctx->stream>>>(x, outer, n, inner, mean, y);
  }
  OM_LAUNCH_CHECK(ctx, "om_reduce_fwd");
  return OM_OK;
}

int32_t om_reduce_bwd(om_ctx* ctx, const float* g, int64_t outer, int64_t n, int64_t inner, int32_t mean, float* dx) {
  OM_CHECK_CTX(ctx);
  if (outer < 0 || n < 0 || inner < 0) return fail(ctx, OM_ERR_SHAPE, "om_reduce_bwd: negative extent");
  int64_t total = outer * n * inner;
  if (total == 0) return OM_OK;
  ProfileScope prof(ctx, "om_reduce_bwd", 0, 4.0 * total);
  reduce_bwd_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(g, outer, n, inner, mean, dx);
  OM_LAUNCH_CHECK(ctx, "om_reduce_bwd");
  return OM_OK;
}

}  // extern "C"
