// Column sums (the bias gradient) without any device allocation: om_colsum_static.
//
// om_colsum takes its table of per-chunk partial sums from the context's memory pool, which may have to go to the
// driver for a new block. This variant keeps the table in a fixed array that is part of the loaded module, so the call
// never asks the pool or the driver for memory: a host that has handed its whole device budget out at start-up, or
// that must not risk the device-wide synchronisation and the late out-of-memory failure of a driver allocation in the
// middle of a run, can still take a bias gradient. The arithmetic (row chunks of 512, 32 row lanes per column
// summed in double, lanes then chunks combined in increasing order) is that of om_colsum, so the two entry points
// give the same bits.
//
// The array is one per device and shared by every call on that device. It keeps whatever the last call left in it;
// nothing in it has to start at zero, because stage 1 writes every slot that stage 2 of the same call reads. Two calls
// that overlap on one device (two streams, two contexts, two threads) race on it: callers serialise them.
//
// The first call on a device looks the array's device address up (cudaGetSymbolAddress, with that device current)
// and keeps it; that look-up is set-up work and should come before any stream capture.
#include "om_common.cuh"

#include <mutex>

namespace om {

constexpr int kStaticRowsPerChunk = 512;
constexpr int kStaticLanes = 32;   // row lanes per column, as in om_colsum
// 131072 doubles = 1 MiB. A call needs ceil(rows / 512) * cols slots.
constexpr long long kStaticSlots = 131072;
constexpr int kStaticMaxDevices = 64;

static __device__ __align__(256) double g_colsum_scratch[kStaticSlots];

static std::mutex g_scratch_mutex;
static double* g_scratch_addr[kStaticMaxDevices] = {nullptr};

__global__ void __launch_bounds__(1024)
colsum_static_stage1_kernel(const float* __restrict__ g, int32_t rows, int32_t cols, int64_t ld,
                                            double* __restrict__ partial) {
  __shared__ double sm[kStaticLanes][33];
  int col = blockIdx.x * 32 + threadIdx.x;
  int r0 = blockIdx.y * kStaticRowsPerChunk;
  int r1 = min(rows, r0 + kStaticRowsPerChunk);
  double acc = 0.0;
  if (col < cols) {
    for (int r = r0 + threadIdx.y; r < r1; r += kStaticLanes) acc += (double)g[(int64_t)r * ld + col];
  }
  sm[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < cols) {
    double t = 0.0;
#pragma unroll
    for (int l = 0; l < kStaticLanes; l++) t += sm[l][threadIdx.x];
    partial[(int64_t)blockIdx.y * cols + col] = t;
  }
}

__global__ void colsum_static_stage2_kernel(const double* __restrict__ partial, int32_t chunks, int32_t cols,
                                            float* __restrict__ out, int accumulate) {
  int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  double t = 0.0;
  for (int c = 0; c < chunks; c++) t += partial[(int64_t)c * cols + col];
  float r = (float)t;
  out[col] = accumulate ? out[col] + r : r;
}

// Device address of the scratch array on the context's device (which the caller has made current). Looked up once
// per device; host code never uses the array's name as an address.
static int32_t scratch_for(om_ctx* ctx, double** out) {
  if (ctx->device < 0 || ctx->device >= kStaticMaxDevices)
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_colsum_static: device ordinal %d beyond %d", ctx->device, kStaticMaxDevices - 1);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[ctx->device] == nullptr) {
    double* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_colsum_scratch);
    if (e != cudaSuccess) return check_cuda(ctx, e, "cudaGetSymbolAddress(colsum scratch)");
    if (ptr == nullptr) return fail(ctx, OM_ERR_CUDA, "om_colsum_static: the scratch array has no device address");
    g_scratch_addr[ctx->device] = ptr;
  }
  *out = g_scratch_addr[ctx->device];
  return OM_OK;
}

}  // namespace om

using namespace om;

extern "C" int32_t om_colsum_static(om_ctx* ctx, const float* g, int32_t rows, int32_t cols, float* out, int32_t accumulate) {
  OM_CHECK_CTX(ctx);
  if (rows < 0 || cols < 0) return fail(ctx, OM_ERR_SHAPE, "om_colsum_static: [%d,%d]", rows, cols);
  if (cols == 0) return OM_OK;
  if (g == nullptr || out == nullptr) return fail(ctx, OM_ERR_ARG, "om_colsum_static: null pointer");
  const long long chunks = ceil_div(rows > 0 ? rows : 1, kStaticRowsPerChunk);
  if (chunks * (long long)cols > kStaticSlots)
    return fail(ctx, OM_ERR_UNSUPPORTED,
                "om_colsum_static: [%d,%d] needs %lld scratch slots (ceil(rows/512) * cols), the fixed array holds %lld; "
                "use om_colsum",
                rows, cols, chunks * (long long)cols, kStaticSlots);
  // The chunks ride on the grid's y dimension, which ends at 65535: a very tall, very narrow table (more than 33.5 million
  // rows of one or two columns) fits the array but not the launch, and is refused the same way.
  if (chunks > 65535)
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_colsum_static: [%d,%d] needs %lld row chunks of 512, the launch holds 65535; use om_colsum", rows,
                cols, chunks);
  double* partial = nullptr;
  OM_TRY(scratch_for(ctx, &partial));
  dim3 grid((unsigned)ceil_div(cols, 32), (unsigned)chunks);
  colsum_static_stage1_kernel<<<grid, dim3(32, kStaticLanes), 0, ctx->stream>>>(g, rows, cols, cols, partial);
  colsum_static_stage2_kernel<<<(unsigned)ceil_div(cols, 128), 128, 0, ctx->stream>>>(partial, (int)chunks, cols, out, accumulate);
  OM_LAUNCH_CHECK(ctx, "om_colsum_static");
  return OM_OK;
}
