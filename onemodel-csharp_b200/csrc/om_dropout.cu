// Dropout with a counter-based mask. The reference's Dropout module (Layers.cs:308-371) draws element i of call number
// `draw` as u = (Mix(stream + (i+1)*gamma) >> 40) * 2^-24 with stream = Mix(seed + draw*gamma), Mix the SplitMix64 finaliser
// and gamma its increment (Generator.cs:10-48); the element is kept (and scaled by 1/(1-p)) when u >= p. Every element is
// a pure function of (seed, draw, i): integer work with no state, so each thread forms its own mask bits and the results
// are the reference's bit for bit. The call counter lives in device memory: the forward reads it, notes the value it used
// for the backward, and a one-thread kernel advances it afterwards in stream order, so a captured step draws a fresh mask
// on every replay. The backward forms the same bits again from the noted value instead of reading a stored mask: it moves
// 8 B per element (g in, dx out) instead of 12.
#include "om_common.cuh"

namespace om {

constexpr unsigned long long kGamma = 0x9E3779B97F4A7C15ULL;

__host__ __device__ __forceinline__ unsigned long long splitmix_finish(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}

__device__ __forceinline__ float keep_factor(unsigned long long stream, int64_t i, float p, float scale) {
  unsigned long long bits = splitmix_finish(stream + (unsigned long long)(i + 1) * kGamma);
  float u = (float)(bits >> 40) * (1.0f / 16777216.0f);
  return u >= p ? scale : 0.f;
}

// MODE 0: mask only; 1: y = x * mask (mask also stored when `mask` is not null); 2: backward, dx = g * mask.
template <int MODE>
__global__ void __launch_bounds__(256)
dropout_kernel(const float* __restrict__ x, int64_t n, float p, float scale, unsigned long long seed,
               const int64_t* __restrict__ draw_src, int64_t* __restrict__ draw_used, float* __restrict__ y,
               float* __restrict__ mask) {
  pdl_enter();
  const unsigned long long draw = (unsigned long long)draw_src[0];
  const unsigned long long stream = splitmix_finish(seed + draw * kGamma);
  if (MODE != 2 && draw_used && blockIdx.x == 0 && threadIdx.x == 0) draw_used[0] = (int64_t)draw;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool vec = (n & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(mask)) & 15) == 0;
  if (vec) {
    for (int64_t q = tid; q < (n >> 2); q += stride) {
      const int64_t i = q << 2;
      float4 m = make_float4(keep_factor(stream, i, p, scale), keep_factor(stream, i + 1, p, scale),
                             keep_factor(stream, i + 2, p, scale), keep_factor(stream, i + 3, p, scale));
      if (MODE != 0) {
        float4 v = reinterpret_cast<const float4*>(x)[q];
        reinterpret_cast<float4*>(y)[q] = make_float4(v.x * m.x, v.y * m.y, v.z * m.z, v.w * m.w);
      }
      if (MODE != 2 && mask) reinterpret_cast<float4*>(mask)[q] = m;
    }
  } else {
    for (int64_t i = tid; i < n; i += stride) {
      float m = keep_factor(stream, i, p, scale);
      if (MODE != 0) y[i] = x[i] * m;
      if (MODE != 2 && mask) mask[i] = m;
    }
  }
}

__global__ void counter_advance_kernel(int64_t* counter, int64_t by) {
  pdl_enter();
  counter[0] += by;
}

static int32_t check(om_ctx* ctx, const char* who, int64_t n, float p, const void* counter) {
  if (n < 0) return fail(ctx, OM_ERR_SHAPE, "%s: n %lld", who, (long long)n);
  if (!(p >= 0.f && p < 1.f)) return fail(ctx, OM_ERR_ARG, "%s: the probability must be in [0, 1), not %g", who, (double)p);
  if (!counter) return fail(ctx, OM_ERR_ARG, "%s: the draw counter is null", who);
  return OM_OK;
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_dropout_mask(om_ctx* ctx, uint64_t seed, const int64_t* draw, float p, int64_t n, float* mask) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check(ctx, "om_dropout_mask", n, p, draw));
  if (n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_dropout_mask", 0, 4.0 * n);
  int grid = grid_for(ctx, (n + 3) / 4, 256);
  launch_chained(ctx, dropout_kernel<0>, grid, 256, 0, (const float*)nullptr, n, p, 1.0f / (1.0f - p), (unsigned long long)seed,
                 draw, (int64_t*)nullptr, (float*)nullptr, mask);
  OM_LAUNCH_CHECK(ctx, "om_dropout_mask");
  return OM_OK;
}

int32_t om_dropout_fwd(om_ctx* ctx, const float* x, int64_t n, float p, uint64_t seed, int64_t* draws, int64_t* draw_used,
                       float* y, float* mask) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check(ctx, "om_dropout_fwd", n, p, draws));
  ProfileScope prof(ctx, "om_dropout_fwd", 0, (mask ? 12.0 : 8.0) * n);
  int grid = n ? grid_for(ctx, (n + 3) / 4, 256) : 1;
  launch_chained(ctx, dropout_kernel<1>, grid, 256, 0, x, n, p, 1.0f / (1.0f - p), (unsigned long long)seed,
                 (const int64_t*)draws, draw_used, y, mask);
  launch_chained(ctx, counter_advance_kernel, 1, 1, 0, draws, (int64_t)1);
  OM_LAUNCH_CHECK(ctx, "om_dropout_fwd");
  return OM_OK;
}

int32_t om_dropout_bwd(om_ctx* ctx, const float* g, int64_t n, float p, uint64_t seed, const int64_t* draw_used, float* dx) {
  OM_CHECK_CTX(ctx);
  OM_TRY(check(ctx, "om_dropout_bwd", n, p, draw_used));
  if (n == 0) return OM_OK;
  ProfileScope prof(ctx, "om_dropout_bwd", 0, 8.0 * n);
  int grid = grid_for(ctx, (n + 3) / 4, 256);
  launch_chained(ctx, dropout_kernel<2>, grid, 256, 0, g, n, p, 1.0f / (1.0f - p), (unsigned long long)seed, draw_used,
                 (int64_t*)nullptr, dx, (float*)nullptr);
  OM_LAUNCH_CHECK(ctx, "om_dropout_bwd");
  return OM_OK;
}

}  // extern "C"
