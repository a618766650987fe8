// Embedding lookup and its table gradient. The gradient is built without floating-point atomics: positions are
// bucketed by id with integer counters (exact, order-free), each bucket is put back into increasing position order,
// and one warp per table row adds the gradient rows of its bucket in that order starting from zero - the order of
// EmbeddingBackward in the reference (BackwardNn.cs:508-546), so duplicate ids sum to the same bits. The same pass
// writes the zeros of untouched rows, so no separate zero-fill of the [V, dim] gradient is needed.
#include "om_common.cuh"

namespace om {

__device__ __forceinline__ int64_t id_at(const void* ids, int dtype, int64_t i) {
  return dtype == OM_I32 ? (int64_t)reinterpret_cast<const int32_t*>(ids)[i] : reinterpret_cast<const int64_t*>(ids)[i];
}

__device__ __forceinline__ void report_index(int32_t* status, int32_t detail) {
  if (atomicCAS(status, 0, (int32_t)OM_ERR_INDEX) == 0) status[1] = detail;
}

__global__ void embedding_fwd_kernel(const float* __restrict__ table, int32_t v, int32_t dim, const void* __restrict__ ids,
                                     int dtype, int64_t n, float* __restrict__ out, int32_t* status) {
  pdl_enter();
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  bool vec = (dim & 3) == 0 && ((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  for (int64_t i = warp; i < n; i += warps) {
    int64_t id = id_at(ids, dtype, i);
    float* o = out + i * dim;
    if (id < 0 || id >= v) {
      if (lane == 0) report_index(status, (int32_t)i);
      for (int j = lane; j < dim; j += 32) o[j] = 0.f;
      continue;
    }
    const float* row = table + id * dim;
    if (vec) {
      const float4* r4 = reinterpret_cast<const float4*>(row);
      float4* o4 = reinterpret_cast<float4*>(o);
      for (int j = lane; j < (dim >> 2); j += 32) o4[j] = r4[j];
    } else {
      for (int j = lane; j < dim; j += 32) o[j] = row[j];
    }
  }
}

__global__ void embedding_count_kernel(const void* __restrict__ ids, int dtype, int64_t n, int32_t v, int64_t pad,
                                       int32_t* __restrict__ count, int32_t* status) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < n; j += stride) {
    int64_t id = id_at(ids, dtype, j);
    if (id == pad) continue;
    if (id < 0 || id >= v) {
      report_index(status, (int32_t)j);
      continue;
    }
    atomicAdd(&count[id], 1);
  }
}

// Exclusive prefix sum of count[0..v) by one CTA of 1024 threads (each thread scans a contiguous span).
__global__ void embedding_scan_kernel(const int32_t* __restrict__ count, int32_t v, int32_t* __restrict__ offset) {
  pdl_enter();
  __shared__ int32_t totals[1024];
  int span = (v + 1023) / 1024;
  int lo = threadIdx.x * span, hi = min(v, lo + span);
  int32_t s = 0;
  for (int i = lo; i < hi; i++) s += count[i];
  totals[threadIdx.x] = s;
  __syncthreads();
  // Hillis-Steele inclusive scan over 1024 totals.
  for (int o = 1; o < 1024; o <<= 1) {
    int32_t t = (int)threadIdx.x >= o ? totals[threadIdx.x - o] : 0;
    __syncthreads();
    totals[threadIdx.x] += t;
    __syncthreads();
  }
  int32_t base = threadIdx.x == 0 ? 0 : totals[threadIdx.x - 1];
  for (int i = lo; i < hi; i++) {
    offset[i] = base;
    base += count[i];
  }
}

__global__ void embedding_fill_kernel(const void* __restrict__ ids, int dtype, int64_t n, int32_t v, int64_t pad,
                                      const int32_t* __restrict__ offset, int32_t* __restrict__ cursor,
                                      int32_t* __restrict__ bucket) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < n; j += stride) {
    int64_t id = id_at(ids, dtype, j);
    if (id == pad || id < 0 || id >= v) continue;
    int slot = atomicAdd(&cursor[id], 1);
    bucket[offset[id] + slot] = (int32_t)j;
  }
}

// One warp per table row: order the row's bucket by position (rank = number of smaller entries; positions are unique),
// then add g rows in that order.
__global__ void embedding_bwd_rows_kernel(const float* __restrict__ g, int32_t v, int32_t dim,
                                          const int32_t* __restrict__ count, const int32_t* __restrict__ offset,
                                          const int32_t* __restrict__ bucket, int32_t* __restrict__ sorted,
                                          float* __restrict__ dtable, int accumulate) {
  pdl_enter();
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp; row < v; row += warps) {
    int b = count[row];
    float* d = dtable + row * dim;
    if (b == 0) {
      if (!accumulate)
        for (int j = lane; j < dim; j += 32) d[j] = 0.f;
      continue;
    }
    const int32_t* bk = bucket + offset[row];
    int32_t* so = sorted + offset[row];
    for (int e = lane; e < b; e += 32) {
      int32_t p = bk[e];
      int rank = 0;
      for (int f = 0; f < b; f++) rank += bk[f] < p;
      so[rank] = p;
    }
    __syncwarp();
    for (int j = lane; j < dim; j += 32) {
      float acc = accumulate ? d[j] : 0.f;
      for (int e = 0; e < b; e++) acc += g[(int64_t)so[e] * dim + j];
      d[j] = acc;
    }
    __syncwarp();
  }
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_embedding_fwd(om_ctx* ctx, const float* table, int32_t v, int32_t dim, const void* ids, int32_t id_dtype,
                         int64_t n, float* out) {
  OM_CHECK_CTX(ctx);
  if (v < 0 || dim < 0 || n < 0 || (id_dtype != OM_I32 && id_dtype != OM_I64))
    return fail(ctx, OM_ERR_SHAPE, "Embedding needs a [V, D] float32 table and Int32 or Int64 ids.");
  if (n == 0 || dim == 0) return OM_OK;
  ProfileScope prof(ctx, "om_embedding_fwd", 0, 8.0 * n * dim);
  launch_chained(ctx, embedding_fwd_kernel, grid_for(ctx, n * 32, 256), 256, 0, table, v, dim, ids, id_dtype, n, out, ctx->status_dev);
  OM_LAUNCH_CHECK(ctx, "om_embedding_fwd");
  return OM_OK;
}

int32_t om_embedding_bwd(om_ctx* ctx, const float* g, const void* ids, int32_t id_dtype, int64_t n, int32_t v,
                         int32_t dim, int64_t padding_index, float* dtable, int32_t accumulate) {
  OM_CHECK_CTX(ctx);
  if (v < 0 || dim < 0 || n < 0 || n > INT32_MAX || (id_dtype != OM_I32 && id_dtype != OM_I64))
    return fail(ctx, OM_ERR_SHAPE, "om_embedding_bwd: v %d dim %d n %lld", v, dim, (long long)n);
  if (v == 0 || dim == 0) return OM_OK;
  ProfileScope prof(ctx, "om_embedding_bwd", 0, 4.0 * n * dim + 4.0 * (double)v * dim);
  // scratch: count[v], cursor[v], offset[v], bucket[n], sorted[n]
  size_t ints = 3 * (size_t)v + 2 * (size_t)(n > 0 ? n : 1);
  int32_t* scratch = nullptr;
  OM_TRY(pool_alloc(ctx, ints * sizeof(int32_t), false, (void**)&scratch));
  int32_t *count = scratch, *cursor = scratch + v, *offset = scratch + 2 * (size_t)v;
  int32_t *bucket = scratch + 3 * (size_t)v, *sorted = bucket + (n > 0 ? n : 1);
  OM_CUDA(ctx, cudaMemsetAsync(count, 0, 2 * (size_t)v * sizeof(int32_t), ctx->stream));
  if (n > 0) {
    launch_chained(ctx, embedding_count_kernel, grid_for(ctx, n, 256), 256, 0, ids, id_dtype, n, v, padding_index, count, ctx->status_dev);
    launch_chained(ctx, embedding_scan_kernel, 1, 1024, 0, count, v, offset);
    launch_chained(ctx, embedding_fill_kernel, grid_for(ctx, n, 256), 256, 0, ids, id_dtype, n, v, padding_index, offset, cursor, bucket);
  }
  launch_chained(ctx, embedding_bwd_rows_kernel, grid_for(ctx, (int64_t)v * 32, 256), 256, 0, g, v, dim, count, offset, bucket, sorted, dtable, accumulate);
  pool_free(ctx, scratch);
  OM_LAUNCH_CHECK(ctx, "om_embedding_bwd");
  return OM_OK;
}

}  // extern "C"
