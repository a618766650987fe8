// Shared internals of libonemodel_b200: the context object, error plumbing, the device memory pool and
// the per-entry-point profiler. Nothing here is visible through the C ABI except the opaque om_ctx.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <functional>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/onemodel_b200.h"

namespace om {

// Device pool with the reference pool's size classes: for the power of two b below the request, the next of
// b*{1.25,1.5,1.75,2} (docs/tensors.md:93-118 of the reference). Blocks are cached per class and reused in
// stream order (single stream per context).
struct Pool {
  std::unordered_map<void*, size_t> live;              // ptr -> class bytes
  std::map<size_t, std::vector<void*>> cache;          // class bytes -> free blocks
  uint64_t bytes_in_use = 0, bytes_cached = 0, driver_allocs = 0;
  // Blocks handed out while a step was being captured belong to that graph: a replay writes to their addresses, so they
  // must never back an unrelated allocation while the graph exists. Freed, they wait in the graph's own cache (where later
  // allocations of the same capture find them again) and return to the general cache when the graph is destroyed.
  std::unordered_map<void*, int> reserved;                          // ptr -> owning graph
  std::map<int, std::map<size_t, std::vector<void*>>> graph_cache;  // graph -> class bytes -> free blocks
  std::unordered_map<void*, size_t> guarded;                        // OM_CHECKED: ptr -> offset of its 64 guard bytes
  static size_t size_class(size_t bytes);
};

struct ProfileEntry {
  uint64_t calls = 0;
  double flops = 0, bytes = 0;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending;
  double ms = 0;
};

struct DpState;  // om_dp.cu

}  // namespace om

struct om_ctx {
  int device = 0;
  uint32_t flags = 0;
  cudaStream_t stream = nullptr;
  std::string last_error;
  int32_t* status_host = nullptr;  // pinned, device-visible status word
  int32_t* status_dev = nullptr;
  int sm_count = 148;
  om::Pool pool;
  // A second stream for work that forks off the main one inside an entry point (the two directions of a bidirectional
  // recurrent layer). While it is current, scratch comes from its own pool so that blocks never change streams.
  cudaStream_t aux_stream = nullptr;
  cudaEvent_t fork_event = nullptr, join_event = nullptr;
  om::Pool pool_aux;
  // Arrival counters of kernels whose last CTA finishes a reduction (column sums): one array per stream of the context,
  // zero between launches (the finishing CTA resets its counter).
  unsigned* arrival[2] = {nullptr, nullptr};
  bool aux_active = false;
  bool profiling = false;
  bool capturing = false;
  int capture_id = 0;                       // the graph being captured (0 when none)
  int next_graph_id = 1;
  std::map<void*, int> graph_ids;           // instantiated graph -> its id in the pools
  int32_t last_graph_kernel_nodes = 0;
  std::map<std::string, om::ProfileEntry> profile;
  std::vector<cudaEvent_t> event_pool;
  om::DpState* dp = nullptr;
  // Staging of input batches ahead of the step that uses them: a copy stream of its own and, per ring slot, an event the
  // copy stream records when the slot's batch has landed and one the compute stream records when the step has taken it.
  cudaStream_t copy_stream = nullptr;
  static constexpr int kStageSlots = 16;
  cudaEvent_t stage_ready[kStageSlots] = {}, stage_taken[kStageSlots] = {};
  bool stage_has_taken[kStageSlots] = {};
};

namespace om {

extern thread_local std::string g_create_error;

int32_t fail(om_ctx* ctx, int32_t code, const char* fmt, ...);
int32_t check_cuda(om_ctx* ctx, cudaError_t e, const char* what);
int32_t pool_alloc(om_ctx* ctx, size_t bytes, bool zero, void** out);
int32_t pool_free(om_ctx* ctx, void* p);
// Runs `second` on the context's auxiliary stream concurrently with `first` on the main stream (fork / join by events;
// inside a stream capture both become branches of the captured graph). Both are synchronous host functions that enqueue
// work on ctx->stream. Returns the first non-zero status.
int32_t run_forked(om_ctx* ctx, const std::function<int32_t()>& first, const std::function<int32_t()>& second);

struct ProfileScope {
  om_ctx* ctx;
  ProfileEntry* e = nullptr;
  cudaEvent_t start = nullptr;
  ProfileScope(om_ctx* c, const char* name, double flops, double bytes);
  ~ProfileScope();
};

#define OM_CHECK_CTX(ctx)                              \
  do {                                                 \
    if ((ctx) == nullptr) return OM_ERR_ARG;           \
    cudaError_t _e = cudaSetDevice((ctx)->device);     \
    if (_e != cudaSuccess) return om::check_cuda((ctx), _e, "cudaSetDevice"); \
  } while (0)

#define OM_CUDA(ctx, call)                                       \
  do {                                                           \
    cudaError_t _e = (call);                                     \
    if (_e != cudaSuccess) return om::check_cuda((ctx), _e, #call); \
  } while (0)

#define OM_LAUNCH_CHECK(ctx, what)                                \
  do {                                                            \
    cudaError_t _e = cudaGetLastError();                          \
    if (_e != cudaSuccess) return om::check_cuda((ctx), _e, what); \
  } while (0)

#define OM_TRY(expr)                 \
  do {                               \
    int32_t _s = (expr);             \
    if (_s != OM_OK) return _s;      \
  } while (0)

constexpr int kArrivalSlots = 4096;

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- overlapped launches (programmatic dependent launch) ------------------------------------------------------------
// A kernel that begins with pdl_enter() may be launched through launch_chained(): with OM_OVERLAP_LAUNCHES its CTAs
// become resident while the previous kernel of the stream is still draining, and hold at the wait until that kernel
// has completed and its writes are visible; launch latency and the prologue then overlap the predecessor's tail.
// The trigger comes first so that the chain is not held up by this kernel's own wait; a kernel that allocates a scarce
// resource its predecessor's CTAs might still need (tensor memory) triggers only after it holds the resource.
// Without the launch attribute both instructions do nothing.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
  pdl_trigger();
  pdl_wait();
}

template <typename... KArgs, typename... Args>
static inline void launch_chained(om_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (ctx->flags & OM_OVERLAP_LAUNCHES) ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// Grid size for a grid-stride kernel: enough CTAs to fill the machine a few times over, never more than the work.
static inline int grid_for(om_ctx* ctx, int64_t work_items, int per_block, int waves = 8) {
  int64_t need = ceil_div(work_items, per_block);
  int64_t cap = (int64_t)ctx->sm_count * waves;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

}  // namespace om
