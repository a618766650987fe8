// Fused multi-tensor optimizer step, gradient-norm clipping and value clipping. One launch covers up to
// kMaxTensors parameters: the pointer table travels in the kernel arguments (so a captured graph replays it
// unchanged) and every CTA finds its tensor by a search over a prefix of chunk counts. HBM-bound: AdamW moves
// 28 bytes per parameter (read p, g, m, v; write p, m, v), SGD with momentum 20.
//
// The per-element arithmetic is written with explicit round-to-nearest intrinsics, one rounding per operation and no
// fused multiply-add, in exactly the order of Adam.UpdateRange / Sgd.Update of the reference
// (src/OneModel.Training/Optimizers.cs:335-373,554-589), so the updated parameters are bit-identical to the
// reference's given the same gradients.
#include <cuda_bf16.h>

#include "om_common.cuh"

namespace om {

constexpr int kMaxTensors = 40;
constexpr int kChunk = 16384;  // elements per CTA visit

struct TensorTable {
  float* p[kMaxTensors];
  const float* g[kMaxTensors];
  float* a[kMaxTensors];  // m (Adam) or momentum buffer (SGD)
  float* b[kMaxTensors];  // v
  float* c[kMaxTensors];  // vmax
  uint16_t* p16[kMaxTensors];  // Adam: the bfloat16 copy of the parameter to refresh in the same pass (may be null)
  int64_t len[kMaxTensors];
  int32_t chunk_prefix[kMaxTensors + 1];
  int32_t first[kMaxTensors];
  int32_t n;
};

__device__ __forceinline__ int find_tensor(const TensorTable& t, int chunk) {
  int lo = 0, hi = t.n;  // chunk_prefix[lo] <= chunk < chunk_prefix[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (t.chunk_prefix[mid] <= chunk) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ float adam_element(float& p, float g, float& m, float& v, float* vmax, const om_adam_hyper& h,
                                              float omb1, float omb2, float decay) {
  if (h.grad_scale != 1.0f) g = __fmul_rn(g, h.grad_scale);
  float pi = p;
  if (h.weight_decay != 0.0f) {
    if (h.decoupled) pi = __fmul_rn(pi, decay);
    else g = __fadd_rn(g, __fmul_rn(h.weight_decay, pi));
  }
  float mi = __fadd_rn(__fmul_rn(h.beta1, m), __fmul_rn(omb1, g));
  float vi = __fadd_rn(__fmul_rn(h.beta2, v), __fmul_rn(__fmul_rn(omb2, g), g));
  m = mi;
  v = vi;
  float vd = vi;
  if (h.amsgrad) {
    float vm = *vmax;
    vd = vm > vi ? vm : vi;
    *vmax = vd;
  }
  float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(vd), h.sqrt_bc2), h.eps);
  p = __fsub_rn(pi, __fdiv_rn(__fmul_rn(h.step_size, mi), denom));
  return p;
}

__global__ void __launch_bounds__(256)
adam_kernel(TensorTable t, om_adam_hyper hv, const om_adam_hyper* __restrict__ hd) {
  pdl_enter();
  const om_adam_hyper h = hd ? *hd : hv;
  const float omb1 = __fsub_rn(1.0f, h.beta1), omb2 = __fsub_rn(1.0f, h.beta2);
  const float decay = __fsub_rn(1.0f, __fmul_rn(h.lr, h.weight_decay));
  const int total = t.chunk_prefix[t.n];
  for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
    int ti = find_tensor(t, chunk);
    int64_t start = (int64_t)(chunk - t.chunk_prefix[ti]) * kChunk;
    int64_t end = min(t.len[ti], start + kChunk);
    float* p = t.p[ti];
    const float* g = t.g[ti];
    float* m = t.a[ti];
    float* v = t.b[ti];
    float* vm = t.c[ti];
    uint16_t* p16 = t.p16[ti];
    bool vec = !h.amsgrad && (((uintptr_t)p16) & 7) == 0 && (((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0;
    if (vec) {
      int64_t e4 = start + ((end - start) & ~(int64_t)3);
      for (int64_t i = start + threadIdx.x * 4; i < e4; i += 256 * 4) {
        float4 pp = *reinterpret_cast<float4*>(p + i), gg = *reinterpret_cast<const float4*>(g + i);
        float4 mm = *reinterpret_cast<float4*>(m + i), vv = *reinterpret_cast<float4*>(v + i);
        adam_element(pp.x, gg.x, mm.x, vv.x, nullptr, h, omb1, omb2, decay);
        adam_element(pp.y, gg.y, mm.y, vv.y, nullptr, h, omb1, omb2, decay);
        adam_element(pp.z, gg.z, mm.z, vv.z, nullptr, h, omb1, omb2, decay);
        adam_element(pp.w, gg.w, mm.w, vv.w, nullptr, h, omb1, omb2, decay);
        *reinterpret_cast<float4*>(p + i) = pp;
        *reinterpret_cast<float4*>(m + i) = mm;
        *reinterpret_cast<float4*>(v + i) = vv;
        if (p16) {
          __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
          *reinterpret_cast<uint2*>(p16 + i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
      }
      for (int64_t i = e4 + threadIdx.x; i < end; i += 256) {
        adam_element(p[i], g[i], m[i], v[i], nullptr, h, omb1, omb2, decay);
        if (p16) {
          __nv_bfloat16 hv16 = __float2bfloat16_rn(p[i]);
          p16[i] = *reinterpret_cast<uint16_t*>(&hv16);
        }
      }
    } else {
      for (int64_t i = start + threadIdx.x; i < end; i += 256) {
        adam_element(p[i], g[i], m[i], v[i], h.amsgrad ? vm + i : nullptr, h, omb1, omb2, decay);
        if (p16) {
          __nv_bfloat16 hv16 = __float2bfloat16_rn(p[i]);
          p16[i] = *reinterpret_cast<uint16_t*>(&hv16);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(256)
sgd_kernel(TensorTable t, om_sgd_hyper hv, const om_sgd_hyper* __restrict__ hd) {
  const om_sgd_hyper h = hd ? *hd : hv;
  const float keep = __fsub_rn(1.0f, h.dampening);
  const int total = t.chunk_prefix[t.n];
  for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
    int ti = find_tensor(t, chunk);
    int64_t start = (int64_t)(chunk - t.chunk_prefix[ti]) * kChunk;
    int64_t end = min(t.len[ti], start + kChunk);
    float* p = t.p[ti];
    const float* gr = t.g[ti];
    float* buf = t.a[ti];
    const bool first = t.first[ti] != 0;
    for (int64_t i = start + threadIdx.x; i < end; i += 256) {
      float g = gr[i];
      if (h.grad_scale != 1.0f) g = __fmul_rn(g, h.grad_scale);
      float pi = p[i];
      if (h.weight_decay != 0.0f) g = __fadd_rn(g, __fmul_rn(h.weight_decay, pi));
      if (h.has_momentum) {
        float bv = first ? g : __fadd_rn(__fmul_rn(h.momentum, buf[i]), __fmul_rn(keep, g));
        buf[i] = bv;
        g = h.nesterov ? __fadd_rn(g, __fmul_rn(h.momentum, bv)) : bv;
      }
      p[i] = __fsub_rn(pi, __fmul_rn(h.lr, g));
    }
  }
}

// ---- gradient norm --------------------------------------------------------------------------------------------------
// Stage 1: one double partial per chunk (256 threads, each summing its strided elements in order, fixed tree).
__global__ void __launch_bounds__(256)
sumsq_kernel(TensorTable t, int infinity, double* __restrict__ partial, int chunk_base) {
  pdl_enter();
  __shared__ double sm[256];
  const int total = t.chunk_prefix[t.n];
  for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
    int ti = find_tensor(t, chunk);
    int64_t start = (int64_t)(chunk - t.chunk_prefix[ti]) * kChunk;
    int64_t end = min(t.len[ti], start + kChunk);
    const float* g = t.g[ti];
    double acc = 0.0;
    for (int64_t i = start + threadIdx.x; i < end; i += 256) {
      double v = (double)g[i];
      if (infinity) {
        double a = fabs(v);
        if (a > acc || a != a) acc = a;
      } else {
        acc += v * v;
      }
    }
    sm[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
      if ((int)threadIdx.x < o) {
        double x = sm[threadIdx.x], y = sm[threadIdx.x + o];
        sm[threadIdx.x] = infinity ? ((y > x || y != y) ? y : x) : x + y;
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) partial[chunk_base + chunk] = sm[0];
    __syncthreads();
  }
}

// Stage 2: one CTA combines the chunk partials in chunk order and writes {norm, coef}.
__global__ void norm_finish_kernel(const double* __restrict__ partial, int chunks, int infinity, float max_norm,
                                   float* __restrict__ total_norm, float* __restrict__ coef_out) {
  pdl_enter();
  __shared__ double sm[1024];
  double acc = 0.0;
  // Thread i owns the contiguous span [i*span, (i+1)*span) so that the combine order is the chunk order.
  int span = (chunks + 1023) / 1024;
  int lo = threadIdx.x * span, hi = min(chunks, lo + span);
  for (int i = lo; i < hi; i++) {
    double y = partial[i];
    acc = infinity ? ((y > acc || y != y) ? y : acc) : acc + y;
  }
  sm[threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < 1024; i++) {
      double y = sm[i];
      t = infinity ? ((y > t || y != y) ? y : t) : t + y;
    }
    double norm = infinity ? t : sqrt(t);
    if (total_norm) total_norm[0] = (float)norm;
    float coef = 1.0f;
    if (isfinite(norm)) coef = (float)((double)max_norm / (norm + 1e-6));
    coef_out[0] = coef;
  }
}

__global__ void __launch_bounds__(256)
scale_by_coef_kernel(TensorTable t, const float* __restrict__ coef_ptr) {
  pdl_enter();
  const float coef = coef_ptr[0];
  if (!(coef < 1.0f)) return;
  const int total = t.chunk_prefix[t.n];
  for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
    int ti = find_tensor(t, chunk);
    int64_t start = (int64_t)(chunk - t.chunk_prefix[ti]) * kChunk;
    int64_t end = min(t.len[ti], start + kChunk);
    float* g = t.p[ti];
    for (int64_t i = start + threadIdx.x; i < end; i += 256) g[i] = __fmul_rn(g[i], coef);
  }
}

__global__ void __launch_bounds__(256)
clip_value_kernel(TensorTable t, float clip) {
  const int total = t.chunk_prefix[t.n];
  for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
    int ti = find_tensor(t, chunk);
    int64_t start = (int64_t)(chunk - t.chunk_prefix[ti]) * kChunk;
    int64_t end = min(t.len[ti], start + kChunk);
    float* g = t.p[ti];
    for (int64_t i = start + threadIdx.x; i < end; i += 256) {
      float v = g[i];
      g[i] = v > clip ? clip : (v < -clip ? -clip : v);
    }
  }
}

// Fills one table with tensors [base, base + count) and returns the number of chunks.
static int fill_table(TensorTable& t, int base, int count, float* const* p, const float* const* g, float* const* a,
                      float* const* b, float* const* c, const int32_t* first, const int64_t* len) {
  t.n = count;
  int chunks = 0;
  for (int i = 0; i < count; i++) {
    int s = base + i;
    t.p[i] = p ? p[s] : nullptr;
    t.g[i] = g ? g[s] : nullptr;
    t.a[i] = a ? a[s] : nullptr;
    t.b[i] = b ? b[s] : nullptr;
    t.c[i] = c ? c[s] : nullptr;
    t.p16[i] = nullptr;
    t.first[i] = first ? first[s] : 0;
    t.len[i] = len[s];
    t.chunk_prefix[i] = chunks;
    chunks += (int)ceil_div(len[s] > 0 ? len[s] : 0, kChunk);
  }
  t.chunk_prefix[count] = chunks;
  return chunks;
}

static int grid_chunks(om_ctx* ctx, int chunks) {
  int cap = ctx->sm_count * 8;
  return chunks < cap ? (chunks > 0 ? chunks : 1) : cap;
}

// ---- row-sparse updates (SparseAdam, sparse Sgd): only the table rows that a step touched are updated ------------------
// touched[row] = how many positions of this step's id list name the row (0 = untouched, its parameters AND moments stay
// as they are: SparseAdam does not decay the moments of absent rows). grad is the dense-format table gradient of
// om_embedding_bwd, whose touched rows hold the coalesced sums the reference's RowSparseGradient holds.
__global__ void rows_touched_kernel(const void* __restrict__ ids, int dtype, int64_t n, int32_t rows, int64_t pad,
                                    int32_t* __restrict__ touched, int32_t* status) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    long long id = dtype == OM_I64 ? ((const long long*)ids)[i] : (long long)((const int32_t*)ids)[i];
    if (id == pad) continue;
    if (id < 0 || id >= rows) {
      atomicCAS(status, 0, (int32_t)OM_ERR_INDEX);
      continue;
    }
    atomicAdd(&touched[id], 1);
  }
}

// One warp per row. SparseAdam.UpdateSparse (Optimizers.cs:696-722), this rounding sequence, no fused multiply-add:
//   m = b1*m + (1-b1)*g;  v = b2*v + ((1-b2)*g)*g;  p -= (stepSize*m) / (sqrt(v) + eps)
__global__ void sparse_adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                                   const int32_t* __restrict__ touched, int32_t rows, int32_t width, float b1, float b2, float eps,
                                   float step_size) {
  const int lane = threadIdx.x & 31;
  const float omb1 = __fsub_rn(1.f, b1), omb2 = __fsub_rn(1.f, b2);
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp; r < rows; r += warps) {
    if (touched[r] == 0) continue;
    const int64_t o = r * width;
    for (int j = lane; j < width; j += 32) {
      float gi = g[o + j];
      float mi = __fadd_rn(__fmul_rn(b1, m[o + j]), __fmul_rn(omb1, gi));
      float vi = __fadd_rn(__fmul_rn(b2, v[o + j]), __fmul_rn(__fmul_rn(omb2, gi), gi));
      m[o + j] = mi;
      v[o + j] = vi;
      p[o + j] = __fsub_rn(p[o + j], __fdiv_rn(__fmul_rn(step_size, mi), __fadd_rn(__fsqrt_rn(vi), eps)));
    }
  }
}

// Sgd.UpdateSparse (Optimizers.cs:377-397): p -= lr * g on the touched rows; no momentum, no weight decay.
__global__ void sparse_sgd_kernel(float* __restrict__ p, const float* __restrict__ g, const int32_t* __restrict__ touched, int32_t rows,
                                  int32_t width, float lr) {
  const int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp; r < rows; r += warps) {
    if (touched[r] == 0) continue;
    const int64_t o = r * width;
    for (int j = lane; j < width; j += 32) p[o + j] = __fsub_rn(p[o + j], __fmul_rn(lr, g[o + j]));
  }
}

// The same two updates from a row list (the row-sparse gradient of om_embedding_bwd_sparse: rows[k] ascending, values[k, :],
// the count on the device): one warp per listed row, the same rounding sequence as above, so a table updated from the row
// list has the bits of one updated from the dense-format gradient.
__global__ void sparse_adam_rows_kernel(float* __restrict__ p, const int32_t* __restrict__ rows, const float* __restrict__ g,
                                        const int32_t* __restrict__ row_count, int32_t capacity, float* __restrict__ m, float* __restrict__ v,
                                        int32_t table_rows, int32_t width, float b1, float b2, float eps, float step_size, int32_t* status) {
  const int lane = threadIdx.x & 31;
  const float omb1 = __fsub_rn(1.f, b1), omb2 = __fsub_rn(1.f, b2);
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int n = min(*row_count, capacity);
  for (int64_t k = warp; k < n; k += warps) {
    const int r = rows[k];
    if (r < 0 || r >= table_rows) {
      if (lane == 0 && atomicCAS(status, 0, (int32_t)OM_ERR_INDEX) == 0) status[1] = (int32_t)k;
      continue;
    }
    const int64_t o = (int64_t)r * width, s = k * width;
    for (int j = lane; j < width; j += 32) {
      float gi = g[s + j];
      float mi = __fadd_rn(__fmul_rn(b1, m[o + j]), __fmul_rn(omb1, gi));
      float vi = __fadd_rn(__fmul_rn(b2, v[o + j]), __fmul_rn(__fmul_rn(omb2, gi), gi));
      m[o + j] = mi;
      v[o + j] = vi;
      p[o + j] = __fsub_rn(p[o + j], __fdiv_rn(__fmul_rn(step_size, mi), __fadd_rn(__fsqrt_rn(vi), eps)));
    }
  }
}

__global__ void sparse_sgd_rows_kernel(float* __restrict__ p, const int32_t* __restrict__ rows, const float* __restrict__ g,
                                       const int32_t* __restrict__ row_count, int32_t capacity, int32_t table_rows, int32_t width, float lr,
                                       int32_t* status) {
  const int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int n = min(*row_count, capacity);
  for (int64_t k = warp; k < n; k += warps) {
    const int r = rows[k];
    if (r < 0 || r >= table_rows) {
      if (lane == 0 && atomicCAS(status, 0, (int32_t)OM_ERR_INDEX) == 0) status[1] = (int32_t)k;
      continue;
    }
    const int64_t o = (int64_t)r * width, s = k * width;
    for (int j = lane; j < width; j += 32) p[o + j] = __fsub_rn(p[o + j], __fmul_rn(lr, g[s + j]));
  }
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_optim_adam_step(om_ctx* ctx, int32_t n_tensors, float* const* p, const float* const* g, float* const* m,
                           float* const* v, float* const* vmax, const int64_t* len, const om_adam_hyper* hyper_host,
                           const om_adam_hyper* hyper_dev) {
  return om_optim_adam_step_b16(ctx, n_tensors, p, g, m, v, vmax, nullptr, len, hyper_host, hyper_dev);
}

int32_t om_optim_adam_step_b16(om_ctx* ctx, int32_t n_tensors, float* const* p, const float* const* g, float* const* m,
                               float* const* v, float* const* vmax, uint16_t* const* p16, const int64_t* len,
                               const om_adam_hyper* hyper_host, const om_adam_hyper* hyper_dev) {
  OM_CHECK_CTX(ctx);
  if (n_tensors < 0 || !hyper_host) return fail(ctx, OM_ERR_ARG, "om_optim_adam_step: bad arguments");
  if (hyper_host->amsgrad && !vmax) return fail(ctx, OM_ERR_ARG, "om_optim_adam_step: amsgrad needs vmax");
  double elems = 0;
  for (int i = 0; i < n_tensors; i++) elems += (double)len[i];
  ProfileScope prof(ctx, "om_optim_adam_step", 0, 28.0 * elems);
  for (int base = 0; base < n_tensors; base += kMaxTensors) {
    TensorTable t;
    int count = std::min(kMaxTensors, n_tensors - base);
    int chunks = fill_table(t, base, count, p, g, m, v, vmax, nullptr, len);
    if (chunks == 0) continue;
    if (p16)
      for (int i = 0; i < count; i++) t.p16[i] = p16[base + i];
    launch_chained(ctx, adam_kernel, grid_chunks(ctx, chunks), 256, 0, t, *hyper_host, hyper_dev);
    OM_LAUNCH_CHECK(ctx, "om_optim_adam_step");
  }
  return OM_OK;
}

int32_t om_optim_sgd_step(om_ctx* ctx, int32_t n_tensors, float* const* p, const float* const* g, float* const* buf,
                          const int32_t* first, const int64_t* len, const om_sgd_hyper* hyper_host,
                          const om_sgd_hyper* hyper_dev) {
  OM_CHECK_CTX(ctx);
  if (n_tensors < 0 || !hyper_host) return fail(ctx, OM_ERR_ARG, "om_optim_sgd_step: bad arguments");
  if (hyper_host->has_momentum && !buf) return fail(ctx, OM_ERR_ARG, "om_optim_sgd_step: momentum needs buffers");
  double elems = 0;
  for (int i = 0; i < n_tensors; i++) elems += (double)len[i];
  ProfileScope prof(ctx, "om_optim_sgd_step", 0, (hyper_host->has_momentum ? 20.0 : 12.0) * elems);
  for (int base = 0; base < n_tensors; base += kMaxTensors) {
    TensorTable t;
    int count = std::min(kMaxTensors, n_tensors - base);
    int chunks = fill_table(t, base, count, p, g, buf, nullptr, nullptr, first, len);
    if (chunks == 0) continue;
    sgd_kernel<<<grid_chunks(ctx, chunks), 256, 0, ctx->stream>>>(t, *hyper_host, hyper_dev);
    OM_LAUNCH_CHECK(ctx, "om_optim_sgd_step");
  }
  return OM_OK;
}

int32_t om_grad_norm_clip(om_ctx* ctx, int32_t n_tensors, float* const* g, const int64_t* len, float max_norm,
                          int32_t infinity_norm, float* total_norm) {
  OM_CHECK_CTX(ctx);
  if (n_tensors < 0) return fail(ctx, OM_ERR_ARG, "om_grad_norm_clip: n_tensors < 0");
  if (!(max_norm > 0.f)) return fail(ctx, OM_ERR_ARG, "The maximum norm must be positive.");
  double elems = 0;
  int total_chunks = 0;
  for (int i = 0; i < n_tensors; i++) {
    elems += (double)len[i];
    total_chunks += (int)ceil_div(len[i] > 0 ? len[i] : 0, kChunk);
  }
  ProfileScope prof(ctx, "om_grad_norm_clip", 0, 12.0 * elems);
  double* partial = nullptr;
  float* coef = nullptr;
  OM_TRY(pool_alloc(ctx, sizeof(double) * (size_t)(total_chunks > 0 ? total_chunks : 1), false, (void**)&partial));
  OM_TRY(pool_alloc(ctx, 256, false, (void**)&coef));
  int chunk_base = 0;
  for (int base = 0; base < n_tensors; base += kMaxTensors) {
    TensorTable t;
    int count = std::min(kMaxTensors, n_tensors - base);
    int chunks = fill_table(t, base, count, nullptr, (const float* const*)g, nullptr, nullptr, nullptr, nullptr, len);
    if (chunks == 0) continue;
    launch_chained(ctx, sumsq_kernel, grid_chunks(ctx, chunks), 256, 0, t, infinity_norm, partial, chunk_base);
    chunk_base += chunks;
  }
  launch_chained(ctx, norm_finish_kernel, 1, 1024, 0, partial, total_chunks, infinity_norm, max_norm, total_norm, coef);
  for (int base = 0; base < n_tensors; base += kMaxTensors) {
    TensorTable t;
    int count = std::min(kMaxTensors, n_tensors - base);
    int chunks = fill_table(t, base, count, g, nullptr, nullptr, nullptr, nullptr, nullptr, len);
    if (chunks == 0) continue;
    launch_chained(ctx, scale_by_coef_kernel, grid_chunks(ctx, chunks), 256, 0, t, coef);
  }
  pool_free(ctx, partial);
  pool_free(ctx, coef);
  OM_LAUNCH_CHECK(ctx, "om_grad_norm_clip");
  return OM_OK;
}

int32_t om_grad_clip_value(om_ctx* ctx, int32_t n_tensors, float* const* g, const int64_t* len, float clip) {
  OM_CHECK_CTX(ctx);
  if (n_tensors < 0) return fail(ctx, OM_ERR_ARG, "om_grad_clip_value: n_tensors < 0");
  if (!(clip >= 0.f)) return fail(ctx, OM_ERR_ARG, "The bound must not be negative.");
  for (int base = 0; base < n_tensors; base += kMaxTensors) {
    TensorTable t;
    int count = std::min(kMaxTensors, n_tensors - base);
    int chunks = fill_table(t, base, count, g, nullptr, nullptr, nullptr, nullptr, nullptr, len);
    if (chunks == 0) continue;
    clip_value_kernel<<<grid_chunks(ctx, chunks), 256, 0, ctx->stream>>>(t, clip);
    OM_LAUNCH_CHECK(ctx, "om_grad_clip_value");
  }
  return OM_OK;
}

int32_t om_rows_touched(om_ctx* ctx, const void* ids, int32_t id_dtype, int64_t n, int32_t rows, int64_t padding_index, int32_t* touched) {
  OM_CHECK_CTX(ctx);
  if (n < 0 || rows < 0 || (id_dtype != OM_I32 && id_dtype != OM_I64)) return fail(ctx, OM_ERR_SHAPE, "om_rows_touched: n %lld rows %d", (long long)n, rows);
  if (rows == 0) return OM_OK;
  OM_CUDA(ctx, cudaMemsetAsync(touched, 0, sizeof(int32_t) * (size_t)rows, ctx->stream));
  if (n > 0) rows_touched_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(ids, id_dtype, n, rows, padding_index, touched, ctx->status_dev);
  OM_LAUNCH_CHECK(ctx, "om_rows_touched");
  return OM_OK;
}

int32_t om_optim_sparse_adam_step(om_ctx* ctx, float* p, const float* g, float* m, float* v, const int32_t* touched, int32_t rows,
                                  int32_t width, float beta1, float beta2, float eps, float step_size) {
  OM_CHECK_CTX(ctx);
  if (rows < 0 || width < 0) return fail(ctx, OM_ERR_SHAPE, "SparseAdam parameters must be rank 2 ([rows, width]) tables.");
  if (rows == 0 || width == 0) return OM_OK;
  ProfileScope prof(ctx, "om_optim_sparse_adam_step", 0, 4.0 * rows);
  sparse_adam_kernel<<<grid_for(ctx, (int64_t)rows * 32, 256), 256, 0, ctx->stream>>>(p, g, m, v, touched, rows, width, beta1, beta2, eps, step_size);
  OM_LAUNCH_CHECK(ctx, "om_optim_sparse_adam_step");
  return OM_OK;
}

int32_t om_optim_sparse_sgd_step(om_ctx* ctx, float* p, const float* g, const int32_t* touched, int32_t rows, int32_t width, float lr) {
  OM_CHECK_CTX(ctx);
  if (rows < 0 || width < 0) return fail(ctx, OM_ERR_SHAPE, "Sparse Sgd parameters must be rank 2 ([rows, width]) tables.");
  if (rows == 0 || width == 0) return OM_OK;
  ProfileScope prof(ctx, "om_optim_sparse_sgd_step", 0, 4.0 * rows);
  sparse_sgd_kernel<<<grid_for(ctx, (int64_t)rows * 32, 256), 256, 0, ctx->stream>>>(p, g, touched, rows, width, lr);
  OM_LAUNCH_CHECK(ctx, "om_optim_sparse_sgd_step");
  return OM_OK;
}

int32_t om_optim_sparse_adam_step_rows(om_ctx* ctx, float* p, const int32_t* rows, const float* values, const int32_t* row_count,
                                       int32_t capacity, float* m, float* v, int32_t table_rows, int32_t width, float beta1, float beta2,
                                       float eps, float step_size) {
  OM_CHECK_CTX(ctx);
  if (table_rows < 0 || width < 0 || capacity < 0) return fail(ctx, OM_ERR_SHAPE, "SparseAdam parameters must be rank 2 ([rows, width]) tables.");
  if (!rows || !values || !row_count) return fail(ctx, OM_ERR_ARG, "om_optim_sparse_adam_step_rows: the row list is needed");
  if (table_rows == 0 || width == 0 || capacity == 0) return OM_OK;
  ProfileScope prof(ctx, "om_optim_sparse_adam_step", 0, 28.0 * capacity * width);
  sparse_adam_rows_kernel<<<grid_for(ctx, (int64_t)capacity * 32, 256), 256, 0, ctx->stream>>>(p, rows, values, row_count, capacity, m, v, table_rows,
                                                                                              width, beta1, beta2, eps, step_size, ctx->status_dev);
  OM_LAUNCH_CHECK(ctx, "om_optim_sparse_adam_step_rows");
  return OM_OK;
}

int32_t om_optim_sparse_sgd_step_rows(om_ctx* ctx, float* p, const int32_t* rows, const float* values, const int32_t* row_count, int32_t capacity,
                                      int32_t table_rows, int32_t width, float lr) {
  OM_CHECK_CTX(ctx);
  if (table_rows < 0 || width < 0 || capacity < 0) return fail(ctx, OM_ERR_SHAPE, "Sparse Sgd parameters must be rank 2 ([rows, width]) tables.");
  if (!rows || !values || !row_count) return fail(ctx, OM_ERR_ARG, "om_optim_sparse_sgd_step_rows: the row list is needed");
  if (table_rows == 0 || width == 0 || capacity == 0) return OM_OK;
  ProfileScope prof(ctx, "om_optim_sparse_sgd_step", 0, 12.0 * capacity * width);
  sparse_sgd_rows_kernel<<<grid_for(ctx, (int64_t)capacity * 32, 256), 256, 0, ctx->stream>>>(p, rows, values, row_count, capacity, table_rows, width, lr,
                                                                                             ctx->status_dev);
  OM_LAUNCH_CHECK(ctx, "om_optim_sparse_sgd_step_rows");
  return OM_OK;
}

}  // extern "C"
