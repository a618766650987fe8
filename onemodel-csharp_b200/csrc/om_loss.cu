// Softmax family and the negative-log-likelihood / cross-entropy losses. Rows are independent: a warp owns a
// narrow row, a CTA owns a wide one (the 30522-wide vocabulary rows of the masked-LM head). Row sums are
// accumulated in double as the reference does (BackwardNn.cs:26-80, Ops.Layers.cs:47-96) and combined by a fixed
// butterfly, so results do not depend on the launch geometry.
#include "om_common.cuh"

namespace om {

constexpr int kRowThreads = 256;
constexpr int kWideRow = 1024;

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Reduction helper for a group of G threads (32 = one warp, kRowThreads = one CTA).
template <int G>
struct RowGroup {
  __device__ static double sum(double v, double* sm) {
    v = warp_sum_d(v);
    if (G == 32) return v;
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) sm[w] = v;
    __syncthreads();
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < G / 32; i++) t += sm[i];
    return t;
  }
  __device__ static float max(float v, double* sm) {
    v = warp_max_f(v);
    if (G == 32) return v;
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    float* smf = reinterpret_cast<float*>(sm);
    __syncthreads();
    if (l == 0) smf[w] = v;
    __syncthreads();
    float t = smf[0];
#pragma unroll
    for (int i = 1; i < G / 32; i++) t = fmaxf(t, smf[i]);
    return t;
  }
};

enum RowOp { SOFTMAX_FWD, LOGSOFTMAX_FWD, SOFTMAX_BWD, LOGSOFTMAX_BWD };

// a = x (fwd) or g (bwd); b = y (bwd only).
template <int G, int OP>
__global__ void __launch_bounds__(kRowThreads)
row_kernel(const float* __restrict__ a, const float* __restrict__ b, int32_t rows, int32_t cols, int64_t ld, float* __restrict__ out) {
  pdl_enter();
  __shared__ double sm[kRowThreads / 32];
  const int lane = G == 32 ? (threadIdx.x & 31) : threadIdx.x;
  const int64_t group = G == 32 ? ((int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5)) : blockIdx.x;
  const int64_t groups = G == 32 ? (int64_t)gridDim.x * (kRowThreads / 32) : gridDim.x;
  // Uniform trip count per CTA keeps __syncthreads legal for G == kRowThreads (the whole CTA shares `row`).
  for (int64_t row = group; row < rows; row += groups) {
    const float* ar = a + row * ld;
    const float* br = b ? b + row * ld : nullptr;
    float* orow = out + row * ld;
    if (OP == SOFTMAX_FWD || OP == LOGSOFTMAX_FWD) {
      float mx = -INFINITY;
      for (int j = lane; j < cols; j += G) mx = fmaxf(mx, ar[j]);
      mx = RowGroup<G>::max(mx, sm);
      double s = 0.0;
      for (int j = lane; j < cols; j += G) s += (double)expf(ar[j] - mx);
      s = RowGroup<G>::sum(s, sm);
      if (OP == LOGSOFTMAX_FWD) {
        float lse = mx + logf((float)s);
        for (int j = lane; j < cols; j += G) orow[j] = ar[j] - lse;
      } else {
        float fs = (float)s;
        for (int j = lane; j < cols; j += G) orow[j] = expf(ar[j] - mx) / fs;
      }
    } else if (OP == SOFTMAX_BWD) {
      double dot = 0.0;
      for (int j = lane; j < cols; j += G) dot += (double)(ar[j] * br[j]);
      float df = (float)RowGroup<G>::sum(dot, sm);
      for (int j = lane; j < cols; j += G) orow[j] = br[j] * (ar[j] - df);
    } else {
      double s = 0.0;
      for (int j = lane; j < cols; j += G) s += (double)ar[j];
      float sf = (float)RowGroup<G>::sum(s, sm);
      for (int j = lane; j < cols; j += G) orow[j] = ar[j] - (expf(br[j]) * sf);
    }
  }
}

template <int OP>
static int32_t launch_rows(om_ctx* ctx, const char* name, const float* a, const float* b, int32_t rows, int32_t cols, float* out, int64_t ld = 0) {
  if (ld == 0) ld = cols;
  if (rows < 0 || cols < 0) return fail(ctx, OM_ERR_SHAPE, "%s: [%d,%d]", name, rows, cols);
  if (rows == 0 || cols == 0) return OM_OK;
  double bytes = (b ? 12.0 : 8.0) * rows * (double)cols;
  ProfileScope prof(ctx, name, 0, bytes);
  if (cols >= kWideRow) {
    int grid = (int)std::min<int64_t>(rows, (int64_t)ctx->sm_count * 8);
    launch_chained(ctx, row_kernel<kRowThreads, OP>, grid, kRowThreads, 0, a, b, rows, cols, ld, out);
  } else {
    int grid = (int)std::min<int64_t>(ceil_div(rows, kRowThreads / 32), (int64_t)ctx->sm_count * 8);
    launch_chained(ctx, row_kernel<32, OP>, grid, kRowThreads, 0, a, b, rows, cols, ld, out);
  }
  OM_LAUNCH_CHECK(ctx, name);
  return OM_OK;
}

__device__ __forceinline__ int64_t target_at(const void* t, int dtype, int64_t i) {
  return dtype == OM_I32 ? (int64_t)reinterpret_cast<const int32_t*>(t)[i] : reinterpret_cast<const int64_t*>(t)[i];
}

__device__ __forceinline__ void report(int32_t* status, int32_t code, int32_t detail) {
  if (atomicCAS(status, 0, code) == 0) status[1] = detail;
}

// One CTA of 1024 threads: loss = -(sum of logp[i, t_i]) over counted rows (double, fixed tree), count of counted rows.
__global__ void nll_fwd_kernel(const float* __restrict__ logp, const void* __restrict__ targets, int dtype, int32_t rows,
                               int32_t cols, int64_t ld, int mean, int64_t ignore, float denominator, float* __restrict__ loss,
                               int32_t* __restrict__ count_out, int32_t* status) {
  pdl_enter();
  __shared__ double ssum[1024];
  __shared__ int scount[1024];
  double s = 0.0;
  int c = 0;
  for (int i = threadIdx.x; i < rows; i += 1024) {
    int64_t t = target_at(targets, dtype, i);
    if (t == ignore) continue;
    if (t < 0 || t >= cols) {
      report(status, OM_ERR_INDEX, i);
      continue;
    }
    s -= (double)logp[(int64_t)i * ld + t];
    c++;
  }
  ssum[threadIdx.x] = s;
  scount[threadIdx.x] = c;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) {
      ssum[threadIdx.x] += ssum[threadIdx.x + o];
      scount[threadIdx.x] += scount[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int cnt = scount[0];
    double div = denominator > 0.f ? (double)denominator : (double)(cnt > 1 ? cnt : 1);
    if (loss) loss[0] = (float)(mean ? ssum[0] / div : ssum[0]);
    if (count_out) count_out[0] = cnt;
  }
}

__global__ void count_targets_kernel(const void* __restrict__ targets, int dtype, int32_t rows, int64_t ignore,
                                     int32_t* __restrict__ count_out) {
  pdl_enter();
  __shared__ int scount[1024];
  int c = 0;
  for (int i = threadIdx.x; i < rows; i += 1024) c += target_at(targets, dtype, i) != ignore;
  scount[threadIdx.x] = c;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) scount[threadIdx.x] += scount[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) count_out[0] = scount[0];
}

__global__ void target_mask_kernel(const void* __restrict__ targets, int dtype, int32_t rows, int64_t ignore, float* __restrict__ mask) {
  pdl_enter();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += gridDim.x * blockDim.x)
    mask[i] = target_at(targets, dtype, i) != ignore ? 1.f : 0.f;
}

__device__ __forceinline__ float nll_scale(const float* g, int mean, const int32_t* count, float denominator) {
  float gv = g[0];
  if (!mean) return gv;
  float div = denominator > 0.f ? denominator : (float)(count[0] > 1 ? count[0] : 1);
  return gv / div;
}

__global__ void nll_bwd_kernel(const float* __restrict__ g, const void* __restrict__ targets, int dtype, int32_t rows,
                               int32_t cols, int mean, int64_t ignore, const int32_t* __restrict__ count,
                               float* __restrict__ dx) {
  float scale = nll_scale(g, mean, count, 0.f);
  int64_t total = (int64_t)rows * cols;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < total; j += stride) {
    int64_t r = j / cols;
    int64_t c = j - r * cols;
    int64_t t = target_at(targets, dtype, r);
    dx[j] = (t != ignore && c == t) ? -scale : 0.f;
  }
}

// One CTA per row: dlogits = onehot-term - exp(logp) * s with s = -scale for counted rows (the LogSoftmax backward
// applied to the NLL gradient, which has a single non-zero per row).
__global__ void __launch_bounds__(kRowThreads)
cross_entropy_bwd_kernel(const float* __restrict__ g, const float* __restrict__ logp, const void* __restrict__ targets,
                         int dtype, int32_t rows, int32_t cols, int64_t ld, int mean, int64_t ignore, float denominator,
                         const int32_t* __restrict__ count, float* __restrict__ dx) {
  pdl_enter();
  float scale = nll_scale(g, mean, count, denominator);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    int64_t t = target_at(targets, dtype, row);
    bool counted = t != ignore;
    float s = counted ? -scale : 0.f;
    const float* y = logp + row * ld;
    float* d = dx + row * ld;
    for (int j = threadIdx.x; j < cols; j += kRowThreads) {
      float gv = (counted && j == t) ? -scale : 0.f;
      d[j] = gv - (expf(y[j]) * s);
    }
  }
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_softmax_fwd(om_ctx* ctx, const float* x, int32_t rows, int32_t cols, float* y) {
  OM_CHECK_CTX(ctx);
  return launch_rows<SOFTMAX_FWD>(ctx, "om_softmax_fwd", x, nullptr, rows, cols, y);
}
int32_t om_softmax_bwd(om_ctx* ctx, const float* g, const float* y, int32_t rows, int32_t cols, float* dx) {
  OM_CHECK_CTX(ctx);
  return launch_rows<SOFTMAX_BWD>(ctx, "om_softmax_bwd", g, y, rows, cols, dx);
}
int32_t om_logsoftmax_fwd(om_ctx* ctx, const float* x, int32_t rows, int32_t cols, float* y) {
  OM_CHECK_CTX(ctx);
  return launch_rows<LOGSOFTMAX_FWD>(ctx, "om_logsoftmax_fwd", x, nullptr, rows, cols, y);
}
int32_t om_logsoftmax_bwd(om_ctx* ctx, const float* g, const float* y, int32_t rows, int32_t cols, float* dx) {
  OM_CHECK_CTX(ctx);
  return launch_rows<LOGSOFTMAX_BWD>(ctx, "om_logsoftmax_bwd", g, y, rows, cols, dx);
}

static int32_t check_targets(om_ctx* ctx, const char* who, int32_t dtype, int32_t rows, int32_t cols) {
  if (dtype != OM_I32 && dtype != OM_I64) return fail(ctx, OM_ERR_SHAPE, "%s: targets must be Int32 or Int64", who);
  if (rows < 0 || cols < 0) return fail(ctx, OM_ERR_SHAPE, "%s: [%d,%d]", who, rows, cols);
  return OM_OK;
}

int32_t om_target_mask(om_ctx* ctx, const void* targets, int32_t target_dtype, int32_t rows, int64_t ignore_index, float* mask) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check_targets(ctx, "om_target_mask", target_dtype, rows, 0));
  if (rows == 0) return OM_OK;
  ProfileScope prof(ctx, "om_target_mask", 0, 12.0 * rows);
  launch_chained(ctx, target_mask_kernel, grid_for(ctx, rows, 256), 256, 0, targets, (int)target_dtype, rows, ignore_index, mask);
  OM_LAUNCH_CHECK(ctx, "om_target_mask");
  return OM_OK;
}

int32_t om_nll_fwd(om_ctx* ctx, const float* logp, const void* targets, int32_t target_dtype, int32_t rows, int32_t cols,
                   int32_t mean, int64_t ignore_index, float* loss, int32_t* count) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check_targets(ctx, "om_nll_fwd", target_dtype, rows, cols));
  ProfileScope prof(ctx, "om_nll_fwd", 0, 12.0 * rows);
  launch_chained(ctx, nll_fwd_kernel, 1, 1024, 0, logp, targets, target_dtype, rows, cols, cols, mean, ignore_index, 0.f, loss, count, ctx->status_dev);
  OM_LAUNCH_CHECK(ctx, "om_nll_fwd");
  return OM_OK;
}

int32_t om_nll_bwd(om_ctx* ctx, const float* g, const void* targets, int32_t target_dtype, int32_t rows, int32_t cols,
                   int32_t mean, int64_t ignore_index, float* dx) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check_targets(ctx, "om_nll_bwd", target_dtype, rows, cols));
  if ((int64_t)rows * cols == 0) return OM_OK;
  ProfileScope prof(ctx, "om_nll_bwd", 0, 4.0 * rows * (double)cols);
  int32_t* count = nullptr;
  OM_TRY(pool_alloc(ctx, 256, false, (void**)&count));
  launch_chained(ctx, count_targets_kernel, 1, 1024, 0, targets, target_dtype, rows, ignore_index, count);
  nll_bwd_kernel<<<grid_for(ctx, (int64_t)rows * cols, 256), 256, 0, ctx->stream>>>(g, targets, target_dtype, rows, cols, mean, ignore_index, count, dx);
  pool_free(ctx, count);
  OM_LAUNCH_CHECK(ctx, "om_nll_bwd");
  return OM_OK;
}

int32_t om_cross_entropy_fwd_ld(om_ctx* ctx, const float* logits, const void* targets, int32_t target_dtype, int32_t rows,
                                int32_t cols, int32_t ld, int32_t mean, int64_t ignore_index, float denominator, float* logp,
                                float* loss, int32_t* count) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check_targets(ctx, "om_cross_entropy_fwd", target_dtype, rows, cols));
  if (ld < cols) return fail(ctx, OM_ERR_SHAPE, "om_cross_entropy_fwd: row pitch %d < %d", ld, cols);
  if (!logp) return fail(ctx, OM_ERR_ARG, "om_cross_entropy_fwd: logp is required (the backward reads it)");
  OM_TRY(launch_rows<LOGSOFTMAX_FWD>(ctx, "om_cross_entropy_fwd.logsoftmax", logits, nullptr, rows, cols, logp, ld));
  ProfileScope prof(ctx, "om_cross_entropy_fwd.nll", 0, 12.0 * rows);
  launch_chained(ctx, nll_fwd_kernel, 1, 1024, 0, logp, targets, target_dtype, rows, cols, ld, mean, ignore_index, denominator, loss, count, ctx->status_dev);
  OM_LAUNCH_CHECK(ctx, "om_cross_entropy_fwd");
  return OM_OK;
}

int32_t om_cross_entropy_fwd(om_ctx* ctx, const float* logits, const void* targets, int32_t target_dtype, int32_t rows,
                             int32_t cols, int32_t mean, int64_t ignore_index, float denominator, float* logp,
                             float* loss, int32_t* count) {
  return om_cross_entropy_fwd_ld(ctx, logits, targets, target_dtype, rows, cols, cols, mean, ignore_index, denominator, logp, loss, count);
}

int32_t om_cross_entropy_bwd_ld(om_ctx* ctx, const float* g, const float* logp, const void* targets, int32_t target_dtype,
                                int32_t rows, int32_t cols, int32_t ld, int32_t mean, int64_t ignore_index, float denominator,
                                float* dlogits) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check_targets(ctx, "om_cross_entropy_bwd", target_dtype, rows, cols));
  if (ld < cols) return fail(ctx, OM_ERR_SHAPE, "om_cross_entropy_bwd: row pitch %d < %d", ld, cols);
  if ((int64_t)rows * cols == 0) return OM_OK;
  ProfileScope prof(ctx, "om_cross_entropy_bwd", 0, 8.0 * rows * (double)cols);
  int32_t* count = nullptr;
  OM_TRY(pool_alloc(ctx, 256, false, (void**)&count));
  launch_chained(ctx, count_targets_kernel, 1, 1024, 0, targets, target_dtype, rows, ignore_index, count);
  int grid = (int)std::min<int64_t>(rows, (int64_t)ctx->sm_count * 8);
  launch_chained(ctx, cross_entropy_bwd_kernel, grid, kRowThreads, 0, g, logp, targets, target_dtype, rows, cols, ld, mean, ignore_index, denominator, count, dlogits);
  pool_free(ctx, count);
  OM_LAUNCH_CHECK(ctx, "om_cross_entropy_bwd");
  return OM_OK;
}

int32_t om_cross_entropy_bwd(om_ctx* ctx, const float* g, const float* logp, const void* targets, int32_t target_dtype,
                             int32_t rows, int32_t cols, int32_t mean, int64_t ignore_index, float denominator,
                             float* dlogits) {
  return om_cross_entropy_bwd_ld(ctx, g, logp, targets, target_dtype, rows, cols, cols, mean, ignore_index, denominator, dlogits);
}

}  // extern "C"
