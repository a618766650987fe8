// Tensor-pipe matrix product (tcgen05 + TMEM + TMA). Placeholder until the kernel lands: reports "not supported"
// so that every product runs on the fp32 FMA kernel.
#include "om_common.cuh"
namespace om {
bool gemm_tc_supported(om_ctx*, int, int, int, int, int, const float*, int, const float*, int, const float*, int) { return false; }
int32_t gemm_tc(om_ctx* ctx, int, int, int, int, int, const float*, int, const float*, int, float*, int, int, const float*) {
  return fail(ctx, OM_ERR_UNSUPPORTED, "tensor-pipe GEMM not built");
}
}  // namespace om
