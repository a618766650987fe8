// Element-wise and indexing operations of the reference's graph-op family and their backward functions
// (Ops.GraphOps.cs:175-394; BackwardGraphOps.cs:44-139): Pow, Where, Gather. All bandwidth-bound; the gather backward
// adds the gradient slices that share a destination in increasing source order (the order of the reference's loop), by
// letting every destination element walk the index list, so no floating-point atomics are needed.
#include "om_common.cuh"

namespace om {

// x^p with the reference's exact cases (PowScalar, Ops.GraphOps.cs:199-206).
__device__ __forceinline__ float pow_scalar(float x, float p) {
  if (p == 1.f) return x;
  if (p == 2.f) return x * x;
  if (p == 0.5f) return sqrtf(x);
  if (p == -1.f) return 1.f / x;
  return powf(x, p);
}
// d/dx x^p (PowDerivative, BackwardGraphOps.cs:69-76).
__device__ __forceinline__ float pow_derivative(float x, float p) {
  if (p == 1.f) return 1.f;
  if (p == 2.f) return x + x;
  if (p == 0.5f) return 1.f / (sqrtf(x) + sqrtf(x));
  if (p == -1.f) return -1.f / (x * x);
  return p * powf(x, p - 1.f);
}

__global__ void pow_kernel(const float* __restrict__ x, float p, float* __restrict__ y, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) y[i] = pow_scalar(x[i], p);
}
__global__ void pow_bwd_kernel(const float* __restrict__ g, const float* __restrict__ x, float p, float* __restrict__ dx, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dx[i] = g[i] * pow_derivative(x[i], p);
}
__global__ void where_kernel(const int32_t* __restrict__ c, const float* __restrict__ a, const float* __restrict__ b,
                             float* __restrict__ out, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = c[i] != 0 ? a[i] : b[i];
}
__global__ void where_bwd_kernel(const int32_t* __restrict__ c, const float* __restrict__ g, int wanted, float* __restrict__ out, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = ((c[i] != 0) == (wanted != 0)) ? g[i] : 0.f;
}

__device__ __forceinline__ long long index_at(const void* ids, int dtype, int64_t j) {
  return dtype == OM_I64 ? ((const long long*)ids)[j] : (long long)((const int32_t*)ids)[j];
}

// out[o][j][k] = data[o][id_j][k]; negative ids count from the end; an id outside the axis raises OM_ERR_INDEX.
__global__ void gather_fwd_kernel(const float* __restrict__ data, const void* __restrict__ ids, int dtype, int64_t outer, int64_t count,
                                  int64_t n, int64_t inner, float* __restrict__ out, int32_t* __restrict__ status) {
  int64_t total = outer * count * inner;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    int64_t k = i % inner, j = (i / inner) % count, o = i / (inner * count);
    long long id = index_at(ids, dtype, j);
    if (id < 0) id += n;
    if (id < 0 || id >= n) {
      atomicCAS(status, 0, OM_ERR_INDEX);
      out[i] = 0.f;
    } else {
      out[i] = data[(o * n + id) * inner + k];
    }
  }
}
// dx[o][id][k] = sum over j with id_j == id, in increasing j, of g[o][j][k].
__global__ void gather_bwd_kernel(const float* __restrict__ g, const void* __restrict__ ids, int dtype, int64_t outer, int64_t count,
                                  int64_t n, int64_t inner, float* __restrict__ dx) {
  int64_t total = outer * n * inner;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    int64_t k = i % inner, row = (i / inner) % n, o = i / (inner * n);
    float acc = 0.f;
    for (int64_t j = 0; j < count; j++) {
      long long id = index_at(ids, dtype, j);
      if (id < 0) id += n;
      if (id == row) acc += g[(o * count + j) * inner + k];
    }
    dx[i] = acc;
  }
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_pow(om_ctx* ctx, const float* x, float exponent, float* y, int64_t n) {
  OM_CHECK_CTX(ctx);
  if (n < 0) return fail(ctx, OM_ERR_SHAPE, "om_pow: n %lld", (long long)n);
  if (n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_pow", 0, 8.0 * n);
  pow_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(x, exponent, y, n);
  OM_LAUNCH_CHECK(ctx, "om_pow");
  return OM_OK;
}

int32_t om_pow_bwd(om_ctx* ctx, const float* g, const float* x, float exponent, float* dx, int64_t n) {
  OM_CHECK_CTX(ctx);
  if (n < 0) return fail(ctx, OM_ERR_SHAPE, "om_pow_bwd: n %lld", (long long)n);
  if (n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_pow_bwd", 0, 12.0 * n);
  pow_bwd_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(g, x, exponent, dx, n);
  OM_LAUNCH_CHECK(ctx, "om_pow_bwd");
  return OM_OK;
}

int32_t om_where(om_ctx* ctx, const int32_t* condition, const float* a, const float* b, float* out, int64_t n) {
  OM_CHECK_CTX(ctx);
  if (n < 0) return fail(ctx, OM_ERR_SHAPE, "om_where: n %lld", (long long)n);
  if (n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_where", 0, 16.0 * n);
  where_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(condition, a, b, out, n);
  OM_LAUNCH_CHECK(ctx, "om_where");
  return OM_OK;
}

int32_t om_where_bwd(om_ctx* ctx, const int32_t* condition, const float* g, int32_t wanted, float* out, int64_t n) {
  OM_CHECK_CTX(ctx);
  if (n < 0) return fail(ctx, OM_ERR_SHAPE, "om_where_bwd: n %lld", (long long)n);
  if (n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_where_bwd", 0, 12.0 * n);
  where_bwd_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(condition, g, wanted, out, n);
  OM_LAUNCH_CHECK(ctx, "om_where_bwd");
  return OM_OK;
}

static int32_t gather_check(om_ctx* ctx, const char* who, int32_t dtype, int64_t outer, int64_t count, int64_t n, int64_t inner) {
  if (dtype != OM_I32 && dtype != OM_I64) return fail(ctx, OM_ERR_ARG, "%s needs Int32 or Int64 indices.", who);
  if (outer < 0 || count < 0 || n < 0 || inner < 0) return fail(ctx, OM_ERR_SHAPE, "%s: outer %lld count %lld axis %lld inner %lld", who,
                                                                 (long long)outer, (long long)count, (long long)n, (long long)inner);
  return OM_OK;
}

int32_t om_gather_fwd(om_ctx* ctx, const float* data, const void* ids, int32_t id_dtype, int64_t outer, int64_t count, int64_t n,
                      int64_t inner, float* out) {
  OM_CHECK_CTX(ctx);
  OM_TRY(gather_check(ctx, "Gather", id_dtype, outer, count, n, inner));
  int64_t total = outer * count * inner;
  if (total == 0) return OM_OK;
  ProfileScope prof(ctx, "om_gather_fwd", 0, 8.0 * total);
  gather_fwd_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(data, ids, id_dtype, outer, count, n, inner, out, ctx->status_dev);
  OM_LAUNCH_CHECK(ctx, "om_gather_fwd");
  return OM_OK;
}

int32_t om_gather_bwd(om_ctx* ctx, const float* g, const void* ids, int32_t id_dtype, int64_t outer, int64_t count, int64_t n,
                      int64_t inner, float* dx) {
  OM_CHECK_CTX(ctx);
  OM_TRY(gather_check(ctx, "Gather backward", id_dtype, outer, count, n, inner));
  int64_t total = outer * n * inner;
  if (total == 0) return OM_OK;
  ProfileScope prof(ctx, "om_gather_bwd", 0, 4.0 * total + 4.0 * outer * count * inner);
  gather_bwd_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(g, ids, id_dtype, outer, count, n, inner, dx);
  OM_LAUNCH_CHECK(ctx, "om_gather_bwd");
  return OM_OK;
}

}  // extern "C"
