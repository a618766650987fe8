// A wait that nothing satisfies, with the context's wait budget: the way to see the timeout path of the tensor-pipe
// kernels' bounded waits work (status word, host read-back, context still usable) without a kernel that hangs.
#include "om_tc.cuh"

namespace om {

__global__ void bounded_wait_probe_kernel(int32_t* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // No thread and no copy ever arrives on the barrier: the wait can only end by running out.
    mbar_wait(&bar, 0, &abort_flag, status, 99);
  }
}

}  // namespace om

using namespace om;

extern "C" int32_t om_selftest_bounded_wait(om_ctx* ctx) {
  OM_CHECK_CTX(ctx);
  bounded_wait_probe_kernel<<<1, 32, 0, ctx->stream>>>(ctx->status_dev);
  OM_LAUNCH_CHECK(ctx, "om_selftest_bounded_wait");
  return OM_OK;
}
