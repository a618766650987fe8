// Embedding lookup and its table gradient. The gradient is built without floating-point atomics: positions are
// bucketed by id with integer counters (exact, order-free), each bucket is put back into increasing position order,
// and one warp per table row adds the gradient rows of its bucket in that order starting from zero - the order of
// EmbeddingBackward in the reference (BackwardNn.cs:508-546), so duplicate ids sum to the same bits. The same pass
// writes the zeros of untouched rows, so no separate zero-fill of the [V, dim] gradient is needed.
#include <algorithm>

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
  // Rows of 16-byte multiples (every table of the configurations): four columns per lane and access. Each column's sum is
  // formed in the same order either way.
  const bool vec = (dim & 3) == 0 && ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(dtable)) & 15) == 0;
  for (int64_t row = warp; row < v; row += warps) {
    int b = count[row];
    float* d = dtable + row * dim;
    if (b == 0) {
      if (!accumulate) {
        if (vec) {
          float4* d4 = reinterpret_cast<float4*>(d);
          for (int j = lane; j < (dim >> 2); j += 32) d4[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
          for (int j = lane; j < dim; j += 32) d[j] = 0.f;
        }
      }
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
    if (vec) {
      float4* d4 = reinterpret_cast<float4*>(d);
      for (int j = lane; j < (dim >> 2); j += 32) {
        float4 acc = accumulate ? d4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int e = 0; e < b; e++) {
          const float4 t = reinterpret_cast<const float4*>(g + (int64_t)so[e] * dim)[j];
          acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
        }
        d4[j] = acc;
      }
    } else {
      for (int j = lane; j < dim; j += 32) {
        float acc = accumulate ? d[j] : 0.f;
        for (int e = 0; e < b; e++) acc += g[(int64_t)so[e] * dim + j];
        d[j] = acc;
      }
    }
    __syncwarp();
  }
}

// ---- the row-sparse form of the table gradient ---------------------------------------------------------------------------
// RowSparseGradient of the reference (RowSparseGradient.cs:14-120): the touched row numbers in ascending order, each once,
// and a [row count, width] tensor of their gradients, each the sum of the output gradients of the row's lookups in
// increasing position order starting from zero (EmbeddingSparseBackward, BackwardNn.cs:548-600: the dense gradient's rows
// bit for bit). Here the row count lives on the device, the two arrays have a fixed capacity, and the entries behind the
// row count are row -1 with zero values: nothing has to read the count back, and the value array can be scaled or
// normed as a plain [capacity, width] tensor.

// slot[i] = number of rows below i with flag[i] != 0 (the position of row i among the touched rows); *total = their count.
__global__ void rowsparse_slot_scan_kernel(const int32_t* __restrict__ flag, int32_t v, int32_t* __restrict__ slot, int32_t* __restrict__ total) {
  pdl_enter();
  __shared__ int32_t totals[1024];
  int span = (v + 1023) / 1024;
  int lo = min(v, (int)threadIdx.x * span), hi = min(v, lo + span);
  int32_t s = 0;
  for (int i = lo; i < hi; i++) s += flag[i] != 0;
  totals[threadIdx.x] = s;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    int32_t t = (int)threadIdx.x >= o ? totals[threadIdx.x - o] : 0;
    __syncthreads();
    totals[threadIdx.x] += t;
    __syncthreads();
  }
  int32_t base = threadIdx.x == 0 ? 0 : totals[threadIdx.x - 1];
  for (int i = lo; i < hi; i++) {
    slot[i] = base;
    base += flag[i] != 0;
  }
  if (threadIdx.x == 1023) *total = totals[1023];
}

// One warp per table row that was looked up: its bucket put into position order, its sum written to values[slot[row]].
__global__ void embedding_bwd_sparse_rows_kernel(const float* __restrict__ g, int32_t v, int32_t dim, const int32_t* __restrict__ count,
                                                 const int32_t* __restrict__ offset, const int32_t* __restrict__ bucket,
                                                 int32_t* __restrict__ sorted, const int32_t* __restrict__ slot,
                                                 int32_t* __restrict__ rows_out, float* __restrict__ values) {
  pdl_enter();
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp; row < v; row += warps) {
    int b = count[row];
    if (b == 0) continue;
    const int k = slot[row];
    if (lane == 0) rows_out[k] = (int32_t)row;
    const int32_t* bk = bucket + offset[row];
    int32_t* so = sorted + offset[row];
    for (int e = lane; e < b; e += 32) {
      int32_t p = bk[e];
      int rank = 0;
      for (int f = 0; f < b; f++) rank += bk[f] < p;
      so[rank] = p;
    }
    __syncwarp();
    float* d = values + (int64_t)k * dim;
    for (int j = lane; j < dim; j += 32) {
      float acc = 0.f;
      for (int e = 0; e < b; e++) acc += g[(int64_t)so[e] * dim + j];
      d[j] = acc;
    }
    __syncwarp();
  }
}

// Entries behind the row count: row -1, zero values.
__global__ void rowsparse_tail_kernel(int32_t* __restrict__ rows, float* __restrict__ values, const int32_t* __restrict__ row_count,
                                      int32_t capacity, int32_t dim) {
  pdl_enter();
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int n = *row_count;
  for (int64_t k = n + warp; k < capacity; k += warps) {
    if (lane == 0) rows[k] = -1;
    for (int j = lane; j < dim; j += 32) values[k * dim + j] = 0.f;
  }
}

// dense[rows[k]] += values[k] (RowSparseGradient.AddTo): the rows are distinct, so no two warps meet.
__global__ void rowsparse_add_to_kernel(const int32_t* __restrict__ rows, const float* __restrict__ values, const int32_t* __restrict__ row_count,
                                        int32_t capacity, int32_t dim, float* __restrict__ dense, int32_t v, int32_t* status) {
  pdl_enter();
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int n = min(*row_count, capacity);
  for (int64_t k = warp; k < n; k += warps) {
    const int row = rows[k];
    if (row < 0 || row >= v) {
      if (lane == 0) report_index(status, (int32_t)k);
      continue;
    }
    float* d = dense + (int64_t)row * dim;
    const float* s = values + k * dim;
    for (int j = lane; j < dim; j += 32) d[j] += s[j];
  }
}

// Merge, step one: where[row] = k + 1 for the k-th entry of a list, present[row] = 1.
__global__ void rowsparse_mark_kernel(const int32_t* __restrict__ rows, const int32_t* __restrict__ row_count, int32_t capacity, int32_t v,
                                      int32_t* __restrict__ where, int32_t* __restrict__ present, int32_t* status) {
  pdl_enter();
  const int n = min(*row_count, capacity);
  for (int64_t k = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; k < n; k += (int64_t)gridDim.x * blockDim.x) {
    const int row = rows[k];
    if (row < 0 || row >= v) {
      report_index(status, (int32_t)k);
      continue;
    }
    where[row] = (int32_t)k + 1;
    present[row] = 1;
  }
}

// Merge, step two: one warp per table row in either list; a's values (or zero), then b's added (RowSparseGradient.Merge: a first).
__global__ void rowsparse_merge_rows_kernel(const int32_t* __restrict__ where_a, const float* __restrict__ values_a,
                                            const int32_t* __restrict__ where_b, const float* __restrict__ values_b,
                                            const int32_t* __restrict__ present, const int32_t* __restrict__ slot, int32_t v, int32_t dim,
                                            int32_t* __restrict__ rows_out, float* __restrict__ values_out) {
  pdl_enter();
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp; row < v; row += warps) {
    if (!present[row]) continue;
    const int k = slot[row], ka = where_a[row], kb = where_b[row];
    if (lane == 0) rows_out[k] = (int32_t)row;
    float* d = values_out + (int64_t)k * dim;
    for (int j = lane; j < dim; j += 32) {
      float acc = ka ? values_a[(int64_t)(ka - 1) * dim + j] : 0.f;
      if (kb) acc += values_b[(int64_t)(kb - 1) * dim + j];
      d[j] = acc;
    }
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

int32_t om_embedding_bwd_sparse(om_ctx* ctx, const float* g, const void* ids, int32_t id_dtype, int64_t n, int32_t v, int32_t dim,
                                int64_t padding_index, int32_t* rows, float* values, int32_t capacity, int32_t* row_count) {
  OM_CHECK_CTX(ctx);
  if (v < 1 || dim < 1 || n < 0 || n > INT32_MAX || (id_dtype != OM_I32 && id_dtype != OM_I64))
    return fail(ctx, OM_ERR_SHAPE, "om_embedding_bwd_sparse: v %d dim %d n %lld", v, dim, (long long)n);
  if (!rows || !values || !row_count || capacity < 1 || (int64_t)capacity < std::min<int64_t>(n, v))
    return fail(ctx, OM_ERR_ARG, "om_embedding_bwd_sparse: rows, values and row_count are needed, with capacity (%d) at least min(n, v) = %lld", capacity,
                (long long)std::min<int64_t>(n, v));
  ProfileScope prof(ctx, "om_embedding_bwd", 0, 8.0 * n * dim);
  // scratch: count[v], cursor[v], offset[v], slot[v], bucket[n], sorted[n]
  const size_t nn = (size_t)(n > 0 ? n : 1);
  int32_t* scratch = nullptr;
  OM_TRY(pool_alloc(ctx, (4 * (size_t)v + 2 * nn) * sizeof(int32_t), false, (void**)&scratch));
  int32_t *count = scratch, *cursor = scratch + v, *offset = scratch + 2 * (size_t)v, *slot = scratch + 3 * (size_t)v;
  int32_t *bucket = scratch + 4 * (size_t)v, *sorted = bucket + nn;
  OM_CUDA(ctx, cudaMemsetAsync(count, 0, 2 * (size_t)v * sizeof(int32_t), ctx->stream));
  if (n > 0) {
    launch_chained(ctx, embedding_count_kernel, grid_for(ctx, n, 256), 256, 0, ids, id_dtype, n, v, padding_index, count, ctx->status_dev);
    launch_chained(ctx, embedding_scan_kernel, 1, 1024, 0, (const int32_t*)count, v, offset);
    launch_chained(ctx, embedding_fill_kernel, grid_for(ctx, n, 256), 256, 0, ids, id_dtype, n, v, padding_index, (const int32_t*)offset, cursor, bucket);
  }
  launch_chained(ctx, rowsparse_slot_scan_kernel, 1, 1024, 0, (const int32_t*)count, v, slot, row_count);
  if (n > 0)
    launch_chained(ctx, embedding_bwd_sparse_rows_kernel, grid_for(ctx, (int64_t)v * 32, 256), 256, 0, g, v, dim, (const int32_t*)count,
                   (const int32_t*)offset, (const int32_t*)bucket, sorted, (const int32_t*)slot, rows, values);
  launch_chained(ctx, rowsparse_tail_kernel, grid_for(ctx, (int64_t)capacity * 32, 256), 256, 0, rows, values, (const int32_t*)row_count, capacity, dim);
  pool_free(ctx, scratch);
  OM_LAUNCH_CHECK(ctx, "om_embedding_bwd_sparse");
  return OM_OK;
}

int32_t om_rowsparse_add_to(om_ctx* ctx, const int32_t* rows, const float* values, const int32_t* row_count, int32_t capacity, int32_t dim,
                            float* dense, int32_t v) {
  OM_CHECK_CTX(ctx);
  if (capacity < 0 || dim < 1 || v < 1) return fail(ctx, OM_ERR_SHAPE, "om_rowsparse_add_to: capacity %d dim %d v %d", capacity, dim, v);
  if (!rows || !values || !row_count || !dense) return fail(ctx, OM_ERR_ARG, "om_rowsparse_add_to: null argument");
  if (capacity == 0) return OM_OK;
  ProfileScope prof(ctx, "om_rowsparse_add_to", 0, 12.0 * capacity * dim);
  launch_chained(ctx, rowsparse_add_to_kernel, grid_for(ctx, (int64_t)capacity * 32, 256), 256, 0, rows, values, row_count, capacity, dim, dense, v,
                 ctx->status_dev);
  OM_LAUNCH_CHECK(ctx, "om_rowsparse_add_to");
  return OM_OK;
}

int32_t om_rowsparse_merge(om_ctx* ctx, const int32_t* rows_a, const float* values_a, const int32_t* count_a, int32_t capacity_a,
                           const int32_t* rows_b, const float* values_b, const int32_t* count_b, int32_t capacity_b, int32_t v, int32_t dim,
                           int32_t* rows_out, float* values_out, int32_t capacity_out, int32_t* count_out) {
  OM_CHECK_CTX(ctx);
  if (capacity_a < 1 || capacity_b < 1 || v < 1 || dim < 1)
    return fail(ctx, OM_ERR_SHAPE, "om_rowsparse_merge: capacities %d %d v %d dim %d", capacity_a, capacity_b, v, dim);
  if (!rows_a || !values_a || !count_a || !rows_b || !values_b || !count_b || !rows_out || !values_out || !count_out)
    return fail(ctx, OM_ERR_ARG, "om_rowsparse_merge: null argument");
  if ((int64_t)capacity_out < std::min<int64_t>((int64_t)capacity_a + capacity_b, v))
    return fail(ctx, OM_ERR_ARG, "om_rowsparse_merge: the result needs capacity min(capacity_a + capacity_b, v) = %lld, not %d",
                (long long)std::min<int64_t>((int64_t)capacity_a + capacity_b, v), capacity_out);
  ProfileScope prof(ctx, "om_rowsparse_merge", 0, 8.0 * ((double)capacity_a + capacity_b) * dim);
  int32_t* scratch = nullptr;   // where_a[v], where_b[v], present[v], slot[v]
  OM_TRY(pool_alloc(ctx, 4 * (size_t)v * sizeof(int32_t), false, (void**)&scratch));
  int32_t *where_a = scratch, *where_b = scratch + v, *present = scratch + 2 * (size_t)v, *slot = scratch + 3 * (size_t)v;
  OM_CUDA(ctx, cudaMemsetAsync(scratch, 0, 3 * (size_t)v * sizeof(int32_t), ctx->stream));
  launch_chained(ctx, rowsparse_mark_kernel, grid_for(ctx, capacity_a, 256), 256, 0, rows_a, count_a, capacity_a, v, where_a, present, ctx->status_dev);
  launch_chained(ctx, rowsparse_mark_kernel, grid_for(ctx, capacity_b, 256), 256, 0, rows_b, count_b, capacity_b, v, where_b, present, ctx->status_dev);
  launch_chained(ctx, rowsparse_slot_scan_kernel, 1, 1024, 0, (const int32_t*)present, v, slot, count_out);
  launch_chained(ctx, rowsparse_merge_rows_kernel, grid_for(ctx, (int64_t)v * 32, 256), 256, 0, (const int32_t*)where_a, values_a, (const int32_t*)where_b,
                 values_b, (const int32_t*)present, (const int32_t*)slot, v, dim, rows_out, values_out);
  launch_chained(ctx, rowsparse_tail_kernel, grid_for(ctx, (int64_t)capacity_out * 32, 256), 256, 0, rows_out, values_out, (const int32_t*)count_out,
                 capacity_out, dim);
  pool_free(ctx, scratch);
  OM_LAUNCH_CHECK(ctx, "om_rowsparse_merge");
  return OM_OK;
}

}  // extern "C"
