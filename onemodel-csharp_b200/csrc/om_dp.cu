// Data-parallel gradient exchange: one rank per process and GPU, NCCL over NVLink/NVSwitch. The reference is a
// single process, so this has no counterpart there. NCCL is bound at run time (dlopen) so that the library loads and
// every other entry point works without it.
//
// Each bucket is a contiguous range of gradient memory. om_dp_allreduce_bucket orders the reduction after the work
// already queued on the context stream (an event) and runs it on a separate communication stream, so the rest of the
// backward pass overlaps it; om_dp_wait joins the communication stream back and checks the communicator for
// asynchronous errors under a host deadline instead of blocking without bound.
#include <dlfcn.h>
#include <stdlib.h>
#include <nccl.h>

#include <chrono>
#include <thread>

#include "om_common.cuh"

namespace om {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi g_nccl;

static int32_t load_nccl(om_ctx* ctx) {
  if (g_nccl.handle) return OM_OK;
  // OM_NCCL_LIBRARY names another library with the same seven entry points (a host whose NCCL lives elsewhere; the tests'
  // stand-in communicator that reports errors and delays on demand).
  const char* named = getenv("OM_NCCL_LIBRARY");
  void* h = nullptr;
  if (named && *named) {
    h = dlopen(named, RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(ctx, OM_ERR_NCCL, "cannot load %s (OM_NCCL_LIBRARY): %s", named, dlerror());
  } else {
    h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(ctx, OM_ERR_NCCL, "cannot load libnccl.so.2: %s", dlerror());
  }
#define OM_SYM(field, name)                                                        \
  g_nccl.field = (decltype(g_nccl.field))dlsym(h, name);                           \
  if (!g_nccl.field) return fail(ctx, OM_ERR_NCCL, "libnccl has no symbol %s", name);
  OM_SYM(GetUniqueId, "ncclGetUniqueId")
  OM_SYM(CommInitRank, "ncclCommInitRank")
  OM_SYM(CommDestroy, "ncclCommDestroy")
  OM_SYM(CommAbort, "ncclCommAbort")
  OM_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
  OM_SYM(AllReduce, "ncclAllReduce")
  OM_SYM(GetErrorString, "ncclGetErrorString")
#undef OM_SYM
  g_nccl.handle = h;
  return OM_OK;
}

struct Bucket {
  float* base = nullptr;
  int64_t count = 0;
  cudaEvent_t done = nullptr;
  bool in_flight = false;
};

struct DpState {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ready = nullptr;
  std::vector<Bucket> buckets;
};

static int32_t nccl_fail(om_ctx* ctx, ncclResult_t r, const char* what) {
  return fail(ctx, OM_ERR_NCCL, "%s: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "nccl error");
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_dp_unique_id(om_ctx* ctx, uint8_t id128[128]) {
  OM_CHECK_CTX(ctx);
  OM_TRY(load_nccl(ctx));
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  ncclResult_t r = g_nccl.GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(ctx, r, "ncclGetUniqueId");
  memcpy(id128, &id, 128);
  return OM_OK;
}

int32_t om_dp_init(om_ctx* ctx, const uint8_t id128[128], int32_t rank, int32_t world) {
  OM_CHECK_CTX(ctx);
  if (ctx->dp) return fail(ctx, OM_ERR_ARG, "om_dp_init: already initialised");
  if (world < 1 || rank < 0 || rank >= world) return fail(ctx, OM_ERR_ARG, "om_dp_init: rank %d of %d", rank, world);
  OM_TRY(load_nccl(ctx));
  DpState* dp = new DpState();
  dp->rank = rank;
  dp->world = world;
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  ncclResult_t r = g_nccl.CommInitRank(&dp->comm, world, id, rank);
  if (r != ncclSuccess) {
    delete dp;
    return nccl_fail(ctx, r, "ncclCommInitRank");
  }
  cudaError_t e = cudaStreamCreateWithFlags(&dp->comm_stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&dp->ready, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    g_nccl.CommAbort(dp->comm);
    delete dp;
    return check_cuda(ctx, e, "om_dp_init");
  }
  ctx->dp = dp;
  return OM_OK;
}

int32_t om_dp_register_bucket(om_ctx* ctx, int32_t bucket_id, float* base, int64_t count) {
  OM_CHECK_CTX(ctx);
  if (!ctx->dp) return fail(ctx, OM_ERR_ARG, "om_dp_register_bucket: om_dp_init has not run");
  if (bucket_id < 0 || bucket_id > 4096 || count < 0 || (!base && count > 0))
    return fail(ctx, OM_ERR_ARG, "om_dp_register_bucket: id %d count %lld", bucket_id, (long long)count);
  DpState* dp = ctx->dp;
  if ((size_t)bucket_id >= dp->buckets.size()) dp->buckets.resize(bucket_id + 1);
  Bucket& b = dp->buckets[bucket_id];
  b.base = base;
  b.count = count;
  if (!b.done) OM_CUDA(ctx, cudaEventCreateWithFlags(&b.done, cudaEventDisableTiming));
  return OM_OK;
}

int32_t om_dp_allreduce_bucket(om_ctx* ctx, int32_t bucket_id) {
  OM_CHECK_CTX(ctx);
  DpState* dp = ctx->dp;
  if (!dp || bucket_id < 0 || (size_t)bucket_id >= dp->buckets.size() || !dp->buckets[bucket_id].done)
    return fail(ctx, OM_ERR_ARG, "om_dp_allreduce_bucket: unknown bucket %d", bucket_id);
  Bucket& b = dp->buckets[bucket_id];
  if (b.count == 0) return OM_OK;
  if (!dp->comm) return fail(ctx, OM_ERR_NCCL, "om_dp_allreduce_bucket: the communicator was aborted after an error; create a new group");
  ProfileScope prof(ctx, "om_dp_allreduce_bucket", 0, 4.0 * b.count);
  OM_CUDA(ctx, cudaEventRecord(dp->ready, ctx->stream));
  OM_CUDA(ctx, cudaStreamWaitEvent(dp->comm_stream, dp->ready, 0));
  ncclResult_t r = g_nccl.AllReduce(b.base, b.base, (size_t)b.count, ncclFloat32, ncclSum, dp->comm, dp->comm_stream);
  if (r != ncclSuccess) return nccl_fail(ctx, r, "ncclAllReduce");
  OM_CUDA(ctx, cudaEventRecord(b.done, dp->comm_stream));
  b.in_flight = true;
  return OM_OK;
}

int32_t om_dp_allreduce(om_ctx* ctx, void* buf, int64_t count, int32_t dtype) {
  OM_CHECK_CTX(ctx);
  DpState* dp = ctx->dp;
  if (!dp) return fail(ctx, OM_ERR_ARG, "om_dp_allreduce: om_dp_init has not run");
  if (!dp->comm) return fail(ctx, OM_ERR_NCCL, "om_dp_allreduce: the communicator was aborted after an error; create a new group");
  ncclDataType_t t = dtype == OM_F32 ? ncclFloat32 : dtype == OM_I32 ? ncclInt32 : ncclInt64;
  ncclResult_t r = g_nccl.AllReduce(buf, buf, (size_t)count, t, ncclSum, dp->comm, ctx->stream);
  if (r != ncclSuccess) return nccl_fail(ctx, r, "ncclAllReduce");
  return OM_OK;
}

int32_t om_dp_wait_bucket(om_ctx* ctx, int32_t bucket_id) {
  OM_CHECK_CTX(ctx);
  DpState* dp = ctx->dp;
  if (!dp) return OM_OK;
  if (bucket_id < 0 || (size_t)bucket_id >= dp->buckets.size()) return fail(ctx, OM_ERR_ARG, "om_dp_wait_bucket: unknown bucket %d", bucket_id);
  Bucket& b = dp->buckets[bucket_id];
  if (!b.in_flight) return OM_OK;
  OM_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, b.done, 0));
  b.in_flight = false;
  return OM_OK;
}

int32_t om_dp_wait(om_ctx* ctx, int32_t timeout_ms) {
  OM_CHECK_CTX(ctx);
  DpState* dp = ctx->dp;
  if (!dp) return OM_OK;
  for (Bucket& b : dp->buckets) {
    if (!b.in_flight) continue;
    OM_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, b.done, 0));
    b.in_flight = false;
  }
  if (!dp->comm) return fail(ctx, OM_ERR_NCCL, "om_dp_wait: the communicator was aborted after an error; create a new group");
  ncclResult_t async = ncclSuccess;
  ncclResult_t r = g_nccl.CommGetAsyncError(dp->comm, &async);
  if (r != ncclSuccess) return nccl_fail(ctx, r, "ncclCommGetAsyncError");
  if (async != ncclSuccess && async != ncclInProgress) {
    g_nccl.CommAbort(dp->comm);
    dp->comm = nullptr;
    return nccl_fail(ctx, async, "asynchronous NCCL error (communicator aborted)");
  }
  if (timeout_ms > 0 && !ctx->capturing) {
    // Host deadline: wait for the joined stream, polling instead of blocking so a dead peer cannot hang the caller.
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {
      cudaError_t q = cudaStreamQuery(ctx->stream);
      if (q == cudaSuccess) break;
      if (q != cudaErrorNotReady) return check_cuda(ctx, q, "om_dp_wait");
      auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
      if (ms > timeout_ms) {
        if (dp->comm) g_nccl.CommAbort(dp->comm);
        dp->comm = nullptr;
        return fail(ctx, OM_ERR_TIMEOUT, "om_dp_wait: gradient exchange not finished after %d ms; communicator aborted", timeout_ms);
      }
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
  return OM_OK;
}

int32_t om_dp_finalize(om_ctx* ctx) {
  if (!ctx || !ctx->dp) return OM_OK;
  cudaSetDevice(ctx->device);
  DpState* dp = ctx->dp;
  cudaStreamSynchronize(ctx->stream);
  if (dp->comm_stream) cudaStreamSynchronize(dp->comm_stream);
  if (dp->comm) g_nccl.CommDestroy(dp->comm);
  for (Bucket& b : dp->buckets)
    if (b.done) cudaEventDestroy(b.done);
  if (dp->ready) cudaEventDestroy(dp->ready);
  if (dp->comm_stream) cudaStreamDestroy(dp->comm_stream);
  delete dp;
  ctx->dp = nullptr;
  return OM_OK;
}

}  // extern "C"
