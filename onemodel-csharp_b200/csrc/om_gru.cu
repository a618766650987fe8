// GRU layer, forward and backward through time, in PyTorch's formulation as the reference has it (Ops.GruLayer,
// Ops.Recurrent.cs:148-260; GruBackward, BackwardRecurrent.cs:115-221):
//   r = sigmoid(W_ir x + b_ir + W_hr h' + b_hr), z likewise, n = tanh(W_in x + b_in + r * (W_hn h' + b_hn)),
//   h = (1 - z) * n + z * h'.
// The input projection of all steps is one product; each step is one small recurrent product plus one fused cell
// kernel; the backward runs the cell gradients step by step (one small product each for dh') and finishes with three
// large products and two double-precision column sums. Every element is computed with the reference's operation order.
#include "om_common.cuh"

namespace om {

int32_t gemm_dispatch(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B,
                      int ldb, float* C, int ldc, int acc, const float* bias);
int32_t colsum_ld(om_ctx* ctx, const float* g, int32_t rows, int32_t cols, int64_t ld, float* out, int32_t accumulate);

__device__ __forceinline__ float gru_sigm(float x) { return 1.0f / (1.0f + expf(-x)); }

// One step for all batch rows. gates_t [B,3H] holds the input side on entry and the activated r, z, n on exit;
// rec [B,3H] is h' W_hh^T; hn_t [B,H] receives the hidden side of n (W_hn h' + b_hn).
__global__ void gru_cell_fwd_kernel(float* __restrict__ gates_t, const float* __restrict__ rec, const float* __restrict__ b_ih,
                                    const float* __restrict__ b_hh, const float* __restrict__ hprev, int batch, int h,
                                    float* __restrict__ hn_t, float* __restrict__ y_t) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= batch * h) return;
  int b = idx / h, j = idx % h;
  float* g = gates_t + (size_t)b * 3 * h;
  const float* rr = rec + (size_t)b * 3 * h;
  float gi[3], gh[3];
#pragma unroll
  for (int q = 0; q < 3; q++) {
    gi[q] = g[q * h + j];
    if (b_ih) gi[q] = gi[q] + b_ih[q * h + j];
    gh[q] = rr[q * h + j];
    if (b_hh) gh[q] = gh[q] + b_hh[q * h + j];
  }
  float r = gru_sigm(gi[0] + gh[0]);
  float z = gru_sigm(gi[1] + gh[1]);
  float prod = r * gh[2];
  float n = tanhf(gi[2] + prod);
  g[j] = r;
  g[h + j] = z;
  g[2 * h + j] = n;
  hn_t[idx] = gh[2];
  float keep = (1.0f - z) * n;
  float carry = z * (hprev ? hprev[idx] : 0.f);
  y_t[idx] = keep + carry;
}

// Gate gradients of one step. dn_in [B,H] is the gradient that flowed back from the later step; direct [B,H] receives
// dH * z (the part of dh' that bypasses the gates); dx_t and dh_t are rows of the two [rows, 3H] gradient tables.
__global__ void gru_cell_bwd_kernel(const float* __restrict__ gates_t, const float* __restrict__ hn_t, const float* __restrict__ gy_t,
                                    const float* __restrict__ dn_in, const float* __restrict__ hprev, int batch, int h,
                                    float* __restrict__ direct, float* __restrict__ dx_t, float* __restrict__ dh_t) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= batch * h) return;
  int b = idx / h, j = idx % h;
  const float* g = gates_t + (size_t)b * 3 * h;
  float rg = g[j], zg = g[h + j], ng = g[2 * h + j];
  float dHt = gy_t[idx] + dn_in[idx];
  float hp = hprev ? hprev[idx] : 0.f;
  float dz = dHt * (hp - ng);
  float dNew = dHt * (1.0f - zg);
  direct[idx] = dHt * zg;
  float dan = dNew * (1.0f - (ng * ng));
  float drg = dan * hn_t[idx];
  float dar = (drg * rg) * (1.0f - rg);
  float daz = (dz * zg) * (1.0f - zg);
  float* dx = dx_t + (size_t)b * 3 * h;
  float* dh = dh_t + (size_t)b * 3 * h;
  dx[j] = dar;
  dx[h + j] = daz;
  dx[2 * h + j] = dan;
  dh[j] = dar;
  dh[h + j] = daz;
  dh[2 * h + j] = dan * rg;
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_gru_layer_fwd(om_ctx* ctx, int32_t reverse, int32_t t, int32_t b, int32_t i, int32_t h, const float* x,
                         const float* w_ih, const float* w_hh, const float* b_ih, const float* b_hh, const float* h0, float* y,
                         float* gates, float* hn) {
  OM_CHECK_CTX(ctx);
  if (t < 0 || b < 0 || i < 1 || h < 1) return fail(ctx, OM_ERR_SHAPE, "GruLayer: T %d B %d I %d H %d", t, b, i, h);
  if (t == 0 || b == 0) return OM_OK;
  const int h3 = 3 * h, bh = b * h;
  ProfileScope prof(ctx, "om_gru_layer_fwd", 2.0 * t * b * (double)h3 * (i + h), 4.0 * t * b * (double)(i + 6 * h));
  OM_TRY(gemm_dispatch(ctx, 0, 1, t * b, h3, i, x, i, w_ih, i, gates, h3, 0, nullptr));
  float* rec = nullptr;
  int32_t st = pool_alloc(ctx, sizeof(float) * (size_t)b * h3, false, (void**)&rec);
  for (int f = 0; f < t && st == OM_OK; f++) {
    int tt = reverse ? t - 1 - f : f;
    int pt = reverse ? tt + 1 : tt - 1;
    const float* hp = f == 0 ? h0 : y + (size_t)pt * bh;
    if (hp) {
      st = gemm_dispatch(ctx, 0, 1, b, h3, h, hp, h, w_hh, h, rec, h3, 0, nullptr);
    } else {
      cudaMemsetAsync(rec, 0, sizeof(float) * (size_t)b * h3, ctx->stream);
    }
    if (st != OM_OK) break;
    gru_cell_fwd_kernel<<<(unsigned)ceil_div(bh, 256), 256, 0, ctx->stream>>>(gates + (size_t)tt * b * h3, rec, b_ih, b_hh, hp, b, h,
                                                                            hn + (size_t)tt * bh, y + (size_t)tt * bh);
  }
  if (rec) pool_free(ctx, rec);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_gru_layer_fwd");
  return OM_OK;
}

int32_t om_gru_layer_bwd(om_ctx* ctx, int32_t reverse, int32_t t, int32_t b, int32_t i, int32_t h, const float* gy, const float* x,
                         const float* y, const float* w_ih, const float* w_hh, const float* h0, const float* gates,
                         const float* hn, float* dx, float* dw_ih, float* dw_hh, float* db_ih, float* db_hh, float* dh0) {
  OM_CHECK_CTX(ctx);
  if (t < 0 || b < 0 || i < 1 || h < 1) return fail(ctx, OM_ERR_SHAPE, "GruBackward: T %d B %d I %d H %d", t, b, i, h);
  if (t == 0 || b == 0) return OM_OK;
  const int h3 = 3 * h, bh = b * h, rows = t * b;
  ProfileScope prof(ctx, "om_gru_layer_bwd", 4.0 * t * b * (double)h3 * (i + h), 4.0 * t * b * (double)(2 * i + 12 * h));
  float *dX = nullptr, *dH = nullptr, *dn[2] = {nullptr, nullptr}, *hprev = nullptr;
  int32_t st = pool_alloc(ctx, sizeof(float) * (size_t)rows * h3, false, (void**)&dX);
  if (st == OM_OK) st = pool_alloc(ctx, sizeof(float) * (size_t)rows * h3, false, (void**)&dH);
  if (st == OM_OK) st = pool_alloc(ctx, sizeof(float) * bh, true, (void**)&dn[0]);
  if (st == OM_OK) st = pool_alloc(ctx, sizeof(float) * bh, false, (void**)&dn[1]);
  if (st == OM_OK) st = pool_alloc(ctx, sizeof(float) * (size_t)rows * h, false, (void**)&hprev);
  if (st == OM_OK) {
    // hprev[t] = y[t -/+ 1], and the initial state (or zeros) at the first processed step of the forward pass.
    int first_t = reverse ? t - 1 : 0;
    if (t > 1) {
      if (reverse) cudaMemcpyAsync(hprev, y + bh, sizeof(float) * (size_t)(t - 1) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
      else cudaMemcpyAsync(hprev + bh, y, sizeof(float) * (size_t)(t - 1) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
    }
    if (h0) cudaMemcpyAsync(hprev + (size_t)first_t * bh, h0, sizeof(float) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
    else cudaMemsetAsync(hprev + (size_t)first_t * bh, 0, sizeof(float) * bh, ctx->stream);
  }
  int cur = 0;
  for (int s = 0; s < t && st == OM_OK; s++) {
    int tt = reverse ? s : t - 1 - s;
    // The cell kernel leaves dH * z in the other buffer; the product then adds dH_t W_hh to it: dh' = dH_t W_hh + dH z.
    gru_cell_bwd_kernel<<<(unsigned)ceil_div(bh, 256), 256, 0, ctx->stream>>>(gates + (size_t)tt * b * h3, hn + (size_t)tt * bh,
                                                                            gy + (size_t)tt * bh, dn[cur], hprev + (size_t)tt * bh, b, h,
                                                                            dn[cur ^ 1], dX + (size_t)tt * b * h3, dH + (size_t)tt * b * h3);
    if (s < t - 1 || dh0) st = gemm_dispatch(ctx, 0, 0, b, h, h3, dH + (size_t)tt * b * h3, h3, w_hh, h, dn[cur ^ 1], h, 1, nullptr);
    cur ^= 1;
  }
  if (st == OM_OK && dx) st = gemm_dispatch(ctx, 0, 0, rows, i, h3, dX, h3, w_ih, i, dx, i, 0, nullptr);
  if (st == OM_OK && dw_ih) st = gemm_dispatch(ctx, 1, 0, h3, i, rows, dX, h3, x, i, dw_ih, i, 0, nullptr);
  if (st == OM_OK && dw_hh) st = gemm_dispatch(ctx, 1, 0, h3, h, rows, dH, h3, hprev, h, dw_hh, h, 0, nullptr);
  if (st == OM_OK && db_ih) st = colsum_ld(ctx, dX, rows, h3, h3, db_ih, 0);
  if (st == OM_OK && db_hh) st = colsum_ld(ctx, dH, rows, h3, h3, db_hh, 0);
  if (st == OM_OK && dh0) cudaMemcpyAsync(dh0, dn[cur], sizeof(float) * bh, cudaMemcpyDeviceToDevice, ctx->stream);
  if (dX) pool_free(ctx, dX);
  if (dH) pool_free(ctx, dH);
  if (dn[0]) pool_free(ctx, dn[0]);
  if (dn[1]) pool_free(ctx, dn[1]);
  if (hprev) pool_free(ctx, hprev);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "om_gru_layer_bwd");
  return OM_OK;
}

}  // extern "C"
