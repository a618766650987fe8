// Context, pooled device memory, copies, graph capture and the per-entry-point profiler.
#include <stdarg.h>

#include <algorithm>
#include <mutex>
#include <set>

#include "om_common.cuh"

namespace om {

thread_local std::string g_create_error;

int32_t fail(om_ctx* ctx, int32_t code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->last_error = buf; else g_create_error = buf;
  return code;
}

int32_t check_cuda(om_ctx* ctx, cudaError_t e, const char* what) {
  if (e == cudaSuccess) return OM_OK;
  int32_t code = (e == cudaErrorMemoryAllocation) ? OM_ERR_OOM : OM_ERR_CUDA;
  return fail(ctx, code, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

size_t Pool::size_class(size_t bytes) {
  if (bytes <= 256) return 256;
  size_t b = 256;
  while ((b << 1) < bytes) b <<= 1;  // b < bytes <= 2b
  size_t q = b >> 2;
  for (int i = 1; i <= 4; i++) {
    size_t c = b + q * i;
    if (c >= bytes) return c;
  }
  return b << 1;
}

constexpr size_t kGuardBytes = 64;

// One thread per guard byte; the first mismatch is reported through the context's status word.
__global__ void guard_check_kernel(const uint8_t* guard, int32_t* status) {
  if (guard[threadIdx.x] != 0xA5 && atomicCAS(status, 0, (int32_t)OM_ERR_CANARY) == 0) status[1] = (int32_t)threadIdx.x;
}

static int32_t pool_alloc_block(om_ctx* ctx, size_t bytes, bool zero, void** out);

int32_t pool_alloc(om_ctx* ctx, size_t bytes, bool zero, void** out) {
  if (!(ctx->flags & OM_CHECKED)) return pool_alloc_block(ctx, bytes, zero, out);
  // CHECKED: poison (or zero) the caller's bytes and lay 64 guard bytes behind them.
  const size_t len = ((bytes == 0 ? 1 : bytes) + 15) & ~(size_t)15;
  OM_TRY(pool_alloc_block(ctx, len + kGuardBytes, false, out));
  uint8_t* base = (uint8_t*)*out;
  OM_CUDA(ctx, cudaMemsetAsync(base, zero ? 0 : 0xFF, len, ctx->stream));
  OM_CUDA(ctx, cudaMemsetAsync(base + len, 0xA5, kGuardBytes, ctx->stream));
  (ctx->aux_active ? ctx->pool_aux : ctx->pool).guarded[*out] = len;
  return OM_OK;
}

static int32_t pool_alloc_block(om_ctx* ctx, size_t bytes, bool zero, void** out) {
  *out = nullptr;
  size_t cls = Pool::size_class(bytes == 0 ? 1 : bytes);
  Pool& p = ctx->aux_active ? ctx->pool_aux : ctx->pool;
  void* ptr = nullptr;
  if (ctx->capturing) {
    // First choice while capturing: a block this capture has already used and freed.
    auto gc = p.graph_cache.find(ctx->capture_id);
    if (gc != p.graph_cache.end()) {
      auto git = gc->second.find(cls);
      if (git != gc->second.end() && !git->second.empty()) {
        ptr = git->second.back();
        git->second.pop_back();
        p.live[ptr] = cls;
        p.bytes_in_use += cls;
        *out = ptr;
        if (zero) {
          cudaError_t e = cudaMemsetAsync(ptr, 0, bytes, ctx->stream);
          if (e != cudaSuccess) return check_cuda(ctx, e, "cudaMemsetAsync");
        }
        return OM_OK;
      }
    }
  }
  auto it = p.cache.find(cls);
  if (it != p.cache.end() && !it->second.empty()) {
    ptr = it->second.back();
    it->second.pop_back();
    p.bytes_cached -= cls;
  } else {
    // During graph capture (relaxed mode) a driver allocation is still legal; the block stays owned by the pool, so the
    // captured address remains valid for every replay.
    cudaError_t e = cudaMalloc(&ptr, cls);
    if (e == cudaErrorMemoryAllocation) {
      cudaGetLastError();
      // Give cached blocks back to the driver and retry once.
      if (ctx->capturing) return check_cuda(ctx, e, "cudaMalloc during graph capture");
      cudaStreamSynchronize(ctx->stream);
      for (auto& kv : p.cache) {
        for (void* q : kv.second) cudaFree(q);
        kv.second.clear();
      }
      p.bytes_cached = 0;
      e = cudaMalloc(&ptr, cls);
    }
    if (e != cudaSuccess) return check_cuda(ctx, e, "cudaMalloc");
    p.driver_allocs++;
  }
  p.live[ptr] = cls;
  p.bytes_in_use += cls;
  if (ctx->capturing) p.reserved[ptr] = ctx->capture_id;
  if (zero) {
    cudaError_t e = cudaMemsetAsync(ptr, 0, bytes, ctx->stream);
    if (e != cudaSuccess) return check_cuda(ctx, e, "cudaMemsetAsync");
  }
  *out = ptr;
  return OM_OK;
}

int32_t pool_free(om_ctx* ctx, void* ptr) {
  if (!ptr) return OM_OK;
  // A block goes back to the pool it came from (main or auxiliary stream), whichever stream is current now.
  Pool* pp = &ctx->pool;
  auto it = pp->live.find(ptr);
  if (it == pp->live.end()) {
    pp = &ctx->pool_aux;
    it = pp->live.find(ptr);
    if (it == pp->live.end()) return fail(ctx, OM_ERR_ARG, "om_free: %p was not allocated by this context", ptr);
  }
  Pool& p = *pp;
  size_t cls = it->second;
  auto gd = p.guarded.find(ptr);
  if (gd != p.guarded.end()) {
    // CHECKED: verify the guard bytes, then poison what is returned (in stream order, behind every kernel that used it).
    guard_check_kernel<<<1, (unsigned)kGuardBytes, 0, ctx->stream>>>((const uint8_t*)ptr + gd->second, ctx->status_dev);
    cudaMemsetAsync(ptr, 0xFF, gd->second, ctx->stream);
    p.guarded.erase(gd);
  }
  p.live.erase(it);
  p.bytes_in_use -= cls;
  auto rv = p.reserved.find(ptr);
  if (rv != p.reserved.end()) {
    p.graph_cache[rv->second][cls].push_back(ptr);   // stays with its graph
    return OM_OK;
  }
  p.cache[cls].push_back(ptr);
  p.bytes_cached += cls;
  return OM_OK;
}

// The graph is gone: its blocks are ordinary blocks again.
static void release_graph_blocks(Pool& p, int id) {
  auto gc = p.graph_cache.find(id);
  if (gc != p.graph_cache.end()) {
    for (auto& kv : gc->second)
      for (void* q : kv.second) {
        p.cache[kv.first].push_back(q);
        p.bytes_cached += kv.first;
      }
    p.graph_cache.erase(gc);
  }
  for (auto it = p.reserved.begin(); it != p.reserved.end();)
    it = it->second == id ? p.reserved.erase(it) : std::next(it);
}

int32_t run_forked(om_ctx* ctx, const std::function<int32_t()>& first, const std::function<int32_t()>& second) {
  if (!ctx->aux_stream) {
    cudaError_t e = cudaStreamCreateWithFlags(&ctx->aux_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->fork_event, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->join_event, cudaEventDisableTiming);
    if (e != cudaSuccess) return check_cuda(ctx, e, "auxiliary stream");
  }
  cudaError_t e = cudaEventRecord(ctx->fork_event, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->aux_stream, ctx->fork_event, 0);
  if (e != cudaSuccess) return check_cuda(ctx, e, "fork to the auxiliary stream");
  const int32_t s0 = first();
  cudaStream_t main_stream = ctx->stream;
  ctx->stream = ctx->aux_stream;
  ctx->aux_active = true;
  const int32_t s1 = second();
  ctx->stream = main_stream;
  ctx->aux_active = false;
  e = cudaEventRecord(ctx->join_event, ctx->aux_stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->stream, ctx->join_event, 0);
  if (e != cudaSuccess) return check_cuda(ctx, e, "join from the auxiliary stream");
  return s0 != OM_OK ? s0 : s1;
}

static cudaEvent_t get_event(om_ctx* ctx) {
  if (!ctx->event_pool.empty()) {
    cudaEvent_t e = ctx->event_pool.back();
    ctx->event_pool.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}

ProfileScope::ProfileScope(om_ctx* c, const char* name, double flops, double bytes) : ctx(c) {
  if (!c->profiling || c->capturing) return;
  e = &c->profile[name];
  e->calls++;
  e->flops += flops;
  e->bytes += bytes;
  start = get_event(c);
  cudaEventRecord(start, c->stream);
}

ProfileScope::~ProfileScope() {
  if (!e) return;
  cudaEvent_t stop = get_event(ctx);
  cudaEventRecord(stop, ctx->stream);
  e->pending.emplace_back(start, stop);
}

static void profile_drain(om_ctx* ctx) {
  cudaStreamSynchronize(ctx->stream);
  for (auto& kv : ctx->profile) {
    for (auto& pr : kv.second.pending) {
      float ms = 0;
      if (cudaEventElapsedTime(&ms, pr.first, pr.second) == cudaSuccess) kv.second.ms += ms;
      ctx->event_pool.push_back(pr.first);
      ctx->event_pool.push_back(pr.second);
    }
    kv.second.pending.clear();
  }
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_version(void) { return 100; }

// The contexts that exist: om_free on a context that was destroyed (a caller that releases its buffers after the context,
// as a garbage-collected host may) returns OM_ERR_ARG instead of touching freed memory; the destroyed context has given
// its blocks back to the driver already.
static std::mutex g_live_mutex;
static std::set<om_ctx*> g_live;

int32_t om_ctx_create(int32_t device, uint32_t flags, om_ctx** out) {
  if (!out) return OM_ERR_ARG;
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    return fail(nullptr, OM_ERR_CUDA, "no CUDA device is visible (%s): this library has no CPU path",
                e == cudaSuccess ? "device count 0" : cudaGetErrorString(e));
  }
  if (device < 0 || device >= count) return fail(nullptr, OM_ERR_ARG, "device %d of %d", device, count);
  if ((e = cudaSetDevice(device)) != cudaSuccess) return check_cuda(nullptr, e, "cudaSetDevice");
  cudaDeviceProp prop;
  if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return check_cuda(nullptr, e, "cudaGetDeviceProperties");
  if (prop.major != 10) {
    return fail(nullptr, OM_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                prop.major, prop.minor);
  }
  om_ctx* ctx = new om_ctx();
  ctx->device = device;
  ctx->flags = flags;
  ctx->sm_count = prop.multiProcessorCount;
  if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess) {
    delete ctx;
    return check_cuda(nullptr, e, "cudaStreamCreate");
  }
  if ((e = cudaHostAlloc((void**)&ctx->status_host, 64, cudaHostAllocMapped)) != cudaSuccess) {
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return check_cuda(nullptr, e, "cudaHostAlloc");
  }
  memset(ctx->status_host, 0, 64);
  cudaHostGetDevicePointer((void**)&ctx->status_dev, ctx->status_host, 0);
  for (int k = 0; k < 2; k++) {
    if ((e = cudaMalloc((void**)&ctx->arrival[k], kArrivalSlots * sizeof(unsigned))) == cudaSuccess)
      e = cudaMemset(ctx->arrival[k], 0, kArrivalSlots * sizeof(unsigned));
    if (e != cudaSuccess) {
      om_ctx_destroy(ctx);
      return check_cuda(nullptr, e, "arrival counters");
    }
  }
  {
    std::lock_guard<std::mutex> lock(g_live_mutex);
    g_live.insert(ctx);
  }
  *out = ctx;
  return OM_OK;
}

int32_t om_dp_finalize(om_ctx* ctx);

int32_t om_ctx_destroy(om_ctx* ctx) {
  if (!ctx) return OM_OK;
  {
    std::lock_guard<std::mutex> lock(g_live_mutex);
    if (!g_live.erase(ctx)) return OM_ERR_ARG;   // not a context of this library (or destroyed twice)
  }
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->dp) om_dp_finalize(ctx);
  for (auto& kv : ctx->pool.cache)
    for (void* p : kv.second) cudaFree(p);
  for (auto& kv : ctx->pool.live) cudaFree(kv.first);
  for (auto& kv : ctx->pool_aux.cache)
    for (void* p : kv.second) cudaFree(p);
  for (auto& kv : ctx->pool_aux.live) cudaFree(kv.first);
  for (Pool* pp : {&ctx->pool, &ctx->pool_aux})
    for (auto& g : pp->graph_cache)
      for (auto& kv : g.second)
        for (void* p : kv.second) cudaFree(p);
  if (ctx->copy_stream) {
    cudaStreamSynchronize(ctx->copy_stream);
    cudaStreamDestroy(ctx->copy_stream);
    for (int i = 0; i < om_ctx::kStageSlots; i++) {
      if (ctx->stage_ready[i]) cudaEventDestroy(ctx->stage_ready[i]);
      if (ctx->stage_taken[i]) cudaEventDestroy(ctx->stage_taken[i]);
    }
  }
  if (ctx->aux_stream) {
    cudaStreamSynchronize(ctx->aux_stream);
    cudaStreamDestroy(ctx->aux_stream);
    cudaEventDestroy(ctx->fork_event);
    cudaEventDestroy(ctx->join_event);
  }
  for (auto& kv : ctx->profile)
    for (auto& pr : kv.second.pending) {
      cudaEventDestroy(pr.first);
      cudaEventDestroy(pr.second);
    }
  for (cudaEvent_t e : ctx->event_pool) cudaEventDestroy(e);
  for (int k = 0; k < 2; k++)
    if (ctx->arrival[k]) cudaFree(ctx->arrival[k]);
  if (ctx->status_host) cudaFreeHost(ctx->status_host);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return OM_OK;
}

int32_t om_ctx_set_flags(om_ctx* ctx, uint32_t flags) {
  if (!ctx) return OM_ERR_ARG;
  ctx->flags = flags;
  return OM_OK;
}

int32_t om_ctx_set_wait_budget_us(om_ctx* ctx, int64_t microseconds) {
  OM_CHECK_CTX(ctx);
  if (microseconds < 0) return fail(ctx, OM_ERR_ARG, "om_ctx_set_wait_budget_us: %lld", (long long)microseconds);
  int khz = 0;
  OM_CUDA(ctx, cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device));
  // Kernels already queued keep reading the word: finish them first so that one kernel sees one budget.
  OM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  long long units = microseconds == 0 ? 0 : ((long long)microseconds * khz / 1000) >> 10;
  if (microseconds > 0 && units < 1) units = 1;
  if (units > INT32_MAX) units = INT32_MAX;
  ((volatile int32_t*)ctx->status_host)[2] = (int32_t)units;
  return OM_OK;
}

int32_t om_ctx_get_flags(om_ctx* ctx, uint32_t* flags) {
  if (!ctx || !flags) return OM_ERR_ARG;
  *flags = ctx->flags;
  return OM_OK;
}

int32_t om_last_error(om_ctx* ctx, char* buf, size_t n) {
  if (!buf || n == 0) return OM_ERR_ARG;
  const std::string& s = ctx ? ctx->last_error : g_create_error;
  size_t len = std::min(n - 1, s.size());
  memcpy(buf, s.data(), len);
  buf[len] = 0;
  return OM_OK;
}

int32_t om_ctx_stream(om_ctx* ctx, void** stream) {
  if (!ctx || !stream) return OM_ERR_ARG;
  *stream = (void*)ctx->stream;
  return OM_OK;
}

int32_t om_alloc(om_ctx* ctx, size_t bytes, int32_t zero, void** dptr) {
  OM_CHECK_CTX(ctx);
  if (!dptr) return OM_ERR_ARG;
  return pool_alloc(ctx, bytes, zero != 0, dptr);
}

int32_t om_free(om_ctx* ctx, void* dptr) {
  if (!ctx) return OM_ERR_ARG;
  {
    std::lock_guard<std::mutex> lock(g_live_mutex);
    if (!g_live.count(ctx)) return OM_ERR_ARG;
  }
  return pool_free(ctx, dptr);
}

int32_t om_pool_trim(om_ctx* ctx) {
  OM_CHECK_CTX(ctx);
  OM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (auto& kv : ctx->pool.cache) {
    for (void* p : kv.second) cudaFree(p);
    kv.second.clear();
  }
  ctx->pool.bytes_cached = 0;
  return OM_OK;
}

int32_t om_pool_stats(om_ctx* ctx, uint64_t* in_use, uint64_t* cached, uint64_t* driver_allocs) {
  if (!ctx) return OM_ERR_ARG;
  if (in_use) *in_use = ctx->pool.bytes_in_use;
  if (cached) *cached = ctx->pool.bytes_cached;
  if (driver_allocs) *driver_allocs = ctx->pool.driver_allocs;
  return OM_OK;
}

int32_t om_memcpy_h2d(om_ctx* ctx, void* dst, const void* src, size_t bytes) {
  OM_CHECK_CTX(ctx);
  if (bytes == 0) return OM_OK;
  OM_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return OM_OK;
}

static int32_t stage_setup(om_ctx* ctx, int32_t slot) {
  if (slot < 0 || slot >= om_ctx::kStageSlots) return fail(ctx, OM_ERR_ARG, "staging slot %d outside [0, %d)", slot, om_ctx::kStageSlots);
  if (!ctx->copy_stream) OM_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
  if (!ctx->stage_ready[slot]) {
    OM_CUDA(ctx, cudaEventCreateWithFlags(&ctx->stage_ready[slot], cudaEventDisableTiming));
    OM_CUDA(ctx, cudaEventCreateWithFlags(&ctx->stage_taken[slot], cudaEventDisableTiming));
  }
  return OM_OK;
}

int32_t om_stage_h2d(om_ctx* ctx, int32_t slot, void* dst, const void* src_pinned, size_t bytes) {
  OM_CHECK_CTX(ctx);
  OM_TRY(stage_setup(ctx, slot));
  // The slot's previous batch must have been taken by its step before the copy overwrites it.
  if (ctx->stage_has_taken[slot]) OM_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->stage_taken[slot], 0));
  if (bytes != 0) OM_CUDA(ctx, cudaMemcpyAsync(dst, src_pinned, bytes, cudaMemcpyHostToDevice, ctx->copy_stream));
  return OM_OK;
}

int32_t om_stage_commit(om_ctx* ctx, int32_t slot) {
  OM_CHECK_CTX(ctx);
  OM_TRY(stage_setup(ctx, slot));
  OM_CUDA(ctx, cudaEventRecord(ctx->stage_ready[slot], ctx->copy_stream));
  return OM_OK;
}

int32_t om_stage_acquire(om_ctx* ctx, int32_t slot) {
  OM_CHECK_CTX(ctx);
  OM_TRY(stage_setup(ctx, slot));
  OM_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->stage_ready[slot], 0));
  return OM_OK;
}

int32_t om_stage_wait_taken(om_ctx* ctx, int32_t slot) {
  OM_CHECK_CTX(ctx);
  OM_TRY(stage_setup(ctx, slot));
  if (ctx->stage_has_taken[slot]) OM_CUDA(ctx, cudaEventSynchronize(ctx->stage_taken[slot]));
  return OM_OK;
}

int32_t om_stage_release(om_ctx* ctx, int32_t slot) {
  OM_CHECK_CTX(ctx);
  OM_TRY(stage_setup(ctx, slot));
  OM_CUDA(ctx, cudaEventRecord(ctx->stage_taken[slot], ctx->stream));
  ctx->stage_has_taken[slot] = true;
  return OM_OK;
}

int32_t om_memcpy_d2h(om_ctx* ctx, void* dst, const void* src, size_t bytes) {
  OM_CHECK_CTX(ctx);
  if (bytes != 0) OM_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  OM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return OM_OK;
}

int32_t om_memcpy_d2d(om_ctx* ctx, void* dst, const void* src, size_t bytes) {
  OM_CHECK_CTX(ctx);
  if (bytes == 0) return OM_OK;
  OM_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return OM_OK;
}

int32_t om_memset(om_ctx* ctx, void* dst, int32_t byte, size_t bytes) {
  OM_CHECK_CTX(ctx);
  if (bytes == 0) return OM_OK;
  OM_CUDA(ctx, cudaMemsetAsync(dst, byte, bytes, ctx->stream));
  return OM_OK;
}

int32_t om_host_alloc_pinned(om_ctx* ctx, size_t bytes, void** hptr) {
  OM_CHECK_CTX(ctx);
  if (!hptr) return OM_ERR_ARG;
  OM_CUDA(ctx, cudaHostAlloc(hptr, bytes == 0 ? 1 : bytes, cudaHostAllocDefault));
  return OM_OK;
}

int32_t om_host_free_pinned(om_ctx* ctx, void* hptr) {
  OM_CHECK_CTX(ctx);
  OM_CUDA(ctx, cudaFreeHost(hptr));
  return OM_OK;
}

int32_t om_sync(om_ctx* ctx) {
  OM_CHECK_CTX(ctx);
  OM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  int32_t s = *(volatile int32_t*)ctx->status_host;
  if (s != 0) {
    int32_t detail = ((volatile int32_t*)ctx->status_host)[1];
    *(volatile int32_t*)ctx->status_host = 0;
    ((volatile int32_t*)ctx->status_host)[1] = 0;
    const char* what = s == OM_ERR_INDEX ? "an index operand was out of range"
                       : s == OM_ERR_CANARY ? "the guard bytes behind a released buffer were overwritten (a kernel wrote past its end)"
                       : s == OM_ERR_TIMEOUT ? "a bounded device-side wait expired"
                                             : "a kernel reported an error";
    return fail(ctx, s, "device status %d: %s (detail %d)", s, what, detail);
  }
  return OM_OK;
}

int32_t om_graph_begin(om_ctx* ctx) {
  OM_CHECK_CTX(ctx);
  if (ctx->capturing) return fail(ctx, OM_ERR_ARG, "om_graph_begin: already capturing");
  OM_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
  ctx->capturing = true;
  ctx->capture_id = ctx->next_graph_id++;
  return OM_OK;
}

int32_t om_graph_end(om_ctx* ctx, void** graph_exec) {
  OM_CHECK_CTX(ctx);
  if (!ctx->capturing) return fail(ctx, OM_ERR_ARG, "om_graph_end: not capturing");
  ctx->capturing = false;
  const int id = ctx->capture_id;
  ctx->capture_id = 0;
  cudaGraph_t graph = nullptr;
  cudaError_t ce = cudaStreamEndCapture(ctx->stream, &graph);
  if (ce != cudaSuccess) {
    release_graph_blocks(ctx->pool, id);
    release_graph_blocks(ctx->pool_aux, id);
    return check_cuda(ctx, ce, "cudaStreamEndCapture");
  }
  {
    size_t n = 0;
    ctx->last_graph_kernel_nodes = 0;
    if (cudaGraphGetNodes(graph, nullptr, &n) == cudaSuccess && n > 0) {
      std::vector<cudaGraphNode_t> nodes(n);
      if (cudaGraphGetNodes(graph, nodes.data(), &n) == cudaSuccess) {
        for (size_t i = 0; i < n; i++) {
          cudaGraphNodeType type;
          if (cudaGraphNodeGetType(nodes[i], &type) == cudaSuccess && type == cudaGraphNodeTypeKernel)
            ctx->last_graph_kernel_nodes++;
        }
      }
    }
  }
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    release_graph_blocks(ctx->pool, id);
    release_graph_blocks(ctx->pool_aux, id);
    return check_cuda(ctx, e, "cudaGraphInstantiate");
  }
  ctx->graph_ids[(void*)exec] = id;
  *graph_exec = (void*)exec;
  return OM_OK;
}

int32_t om_graph_last_kernel_nodes(om_ctx* ctx, int32_t* n) {
  if (!ctx || !n) return OM_ERR_ARG;
  *n = ctx->last_graph_kernel_nodes;
  return OM_OK;
}

int32_t om_graph_launch(om_ctx* ctx, void* graph_exec) {
  OM_CHECK_CTX(ctx);
  OM_CUDA(ctx, cudaGraphLaunch((cudaGraphExec_t)graph_exec, ctx->stream));
  return OM_OK;
}

int32_t om_graph_destroy(om_ctx* ctx, void* graph_exec) {
  OM_CHECK_CTX(ctx);
  if (!graph_exec) return OM_OK;
  // Replays in flight still write to the graph's blocks: let them finish before the blocks become ordinary again.
  OM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  OM_CUDA(ctx, cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
  auto it = ctx->graph_ids.find(graph_exec);
  if (it != ctx->graph_ids.end()) {
    release_graph_blocks(ctx->pool, it->second);
    release_graph_blocks(ctx->pool_aux, it->second);
    ctx->graph_ids.erase(it);
  }
  return OM_OK;
}

int32_t om_profile_enable(om_ctx* ctx, int32_t on) {
  if (!ctx) return OM_ERR_ARG;
  if (!on && ctx->profiling) {
    cudaSetDevice(ctx->device);
    profile_drain(ctx);
  }
  ctx->profiling = on != 0;
  return OM_OK;
}

int32_t om_profile_reset(om_ctx* ctx) {
  OM_CHECK_CTX(ctx);
  profile_drain(ctx);
  ctx->profile.clear();
  return OM_OK;
}

int32_t om_profile_read(om_ctx* ctx, om_profile_row* rows, int32_t cap, int32_t* n) {
  OM_CHECK_CTX(ctx);
  profile_drain(ctx);
  int32_t i = 0;
  for (auto& kv : ctx->profile) {
    if (i < cap && rows) {
      memset(&rows[i], 0, sizeof rows[i]);
      strncpy(rows[i].name, kv.first.c_str(), sizeof rows[i].name - 1);
      rows[i].calls = kv.second.calls;
      rows[i].ms = kv.second.ms;
      rows[i].flops = kv.second.flops;
      rows[i].bytes = kv.second.bytes;
    }
    i++;
  }
  if (n) *n = i;
  return OM_OK;
}

}  // extern "C"
