// Attention forward for sequences of several tiles with bfloat16 product operands (the OM_BF16_OPERANDS tier).
//
// Ops.Attention of the reference (Ops.Layers.cs attention forward; softmax(scale Q K^T + mask) V per (batch, head)), here
// one CTA per (128 queries, batch, head) that walks the key tiles twice:
//   pass 1   S_j = Q K_j^T (tcgen05.mma kind::f16, bfloat16 tiles brought in by TMA, fp32 accumulator in tensor memory);
//            the row threads keep the running maximum of scale S + mask. No exponential is taken.
//   pass 2   S_j again; P_j = exp(scale S_j + mask - max) is summed per row in fp32, rounded to bfloat16 into shared memory
//            and O += P_j V_j accumulates in tensor memory. Nothing is rescaled on the way; the result is O / sum at the
//            end, with the row log-sum-exp max + log(sum) that the backward needs, and optionally O as bfloat16 (the next
//            Linear layer's operand).
// ONE pass where a bound on the scores is at hand: without a mask, scale |q_i| max_j |k_j| bounds every scaled score of row i
// (Cauchy-Schwarz), so it can stand in for the row maximum: exp(score - bound) <= 1 never overflows, and while the bound is
// at most 40 it is at least e^-80, far inside fp32 and bfloat16 range; sum, O / sum and the log-sum-exp bound + log(sum) are
// the same quantities, rounded as before. max_j |k_j|^2 per (batch, head) comes from a small kernel in front
// (attention_kmax_kernel); a CTA one of whose rows has a larger bound, or that has a mask, walks the key tiles twice as
// described. The first pass is a third of the two-pass kernel's products and read-backs.
// The second Q K^T costs tensor-pipe time that the kernel does not lack. A CTA keeps its steps in sequence (product,
// read-back, exponentials, staging, product) and is sized so that TWO CTAs share an SM (112 KB of shared memory, 256 columns
// of tensor memory, at most 113 registers per thread): one CTA's products run under the other's exponentials.
// Sums are fp32 in a fixed order; every wait is bounded (om_tc.cuh).
#include <cuda_bf16.h>

#include "om_tc.cuh"

namespace om {

constexpr int AF_TILE = 128;
constexpr int AF_D = 64;
constexpr int AF_BLOCK = AF_TILE * 128;          // [128 rows x 128 bytes]: 64 bfloat16 per row
constexpr int AF_THREADS = 288;                  // warps 0-7: half a score row per thread; warp 8: TMA and MMA issue
constexpr uint32_t AF_COL_S = 0, AF_COL_O = 128, AF_TMEM_COLS = 256;
constexpr uint32_t AF_DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // stride offset 1024 bytes, version 1, 128-byte swizzle
constexpr uint32_t AF_LBO_K = (16u >> 4) << 16;
constexpr uint32_t AF_LBO_MN = ((uint32_t)AF_BLOCK >> 4) << 16;

struct AttFwd16Params {
  int lq, lk, heads;
  float scale;
  const float* mask;
  long long mask_batch_stride;
  float* lse;                                    // [B*H, lq] (may be null)
  const float* kmax2;                            // [B*H] max over the keys of |k|^2, or null: always two passes
  int want16;
  int32_t* status;
};

__device__ __forceinline__ void af_arrive(uint64_t* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory"); }
__device__ __forceinline__ void af_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float af_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t af_pack(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// The lower word of a shared-memory descriptor is (address >> 4) | leading-offset field; the upper word is the same for all.
__device__ __forceinline__ void af_mma(uint32_t tmem_c, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, {%6, %6, %6, %6}, p;\n\t}"
      ::"r"(tmem_c), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(AF_DESC_HI), "r"(0u)
      : "memory");
}
// kind::f16, bfloat16 A and B, fp32 accumulator, M = 128.
__device__ __forceinline__ uint32_t af_idesc(int n, bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(AF_TILE >> 4) << 24);
}
__device__ __forceinline__ void af_tma_store_4d(const CUtensorMap* map, const uint8_t* slot, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2),
               "r"(c3), "r"(smem_u32(slot))
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

constexpr float AF_BOUND_LIMIT = 40.f;

// kmax2[b, h] = max over the keys of |k|^2 (fp32 sum of the squares of the bfloat16 values). One CTA per (batch, head).
__global__ void __launch_bounds__(256)
attention_kmax_kernel(const uint16_t* __restrict__ k16, long long s_batch, long long s_head, long long s_row, int heads, int lk,
                      float* __restrict__ kmax2) {
  pdl_enter();
  __shared__ float wmax[8];
  const int bh = blockIdx.x, bi = bh / heads, hi = bh - bi * heads;
  const uint16_t* base = k16 + bi * s_batch + hi * s_head;
  float best = 0.f;
  for (int key = threadIdx.x; key < lk; key += 256) {
    const uint4* rowp = reinterpret_cast<const uint4*>(base + (long long)key * s_row);
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < AF_D / 8; c++) {
      const uint4 v = __ldg(rowp + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const float lo = __uint_as_float(w[q] << 16), hi2 = __uint_as_float(w[q] & 0xFFFF0000u);
        ss = fmaf(lo, lo, ss);
        ss = fmaf(hi2, hi2, ss);
      }
    }
    best = fmaxf(best, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = wmax[0];
#pragma unroll
    for (int w = 1; w < 8; w++) t = fmaxf(t, wmax[w]);
    kmax2[bh] = t;
  }
}

__global__ void __launch_bounds__(AF_THREADS, 2)
attention_fwd16_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                       const __grid_constant__ CUtensorMap map_o16, AttFwd16Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* slot_q = smem;                               // Q_i: S (K-major A)
  uint8_t* slot_k = smem + AF_BLOCK;                    // K_j, two buffers: S (K-major B, 128 rows)
  uint8_t* slot_v = smem + 3 * AF_BLOCK;                // V_j, two buffers: O (MN-major B)
  uint8_t* stage_p = smem + 5 * AF_BLOCK;               // P: two blocks of [128 queries x 64 keys]; O (K-major A)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * AF_BLOCK);
  uint64_t *bar_q = bars, *bar_k = bars + 1 /* [2] */, *bar_v = bars + 3 /* [2] */, *bar_s = bars + 5, *bar_staged = bars + 6, *bar_done = bars + 7,
           *bar_x = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* two_pass_flag = abort_flag + 1;         // set by a row thread whose bound is too large for the one-pass form
  float* xch = reinterpret_cast<float*>(stage_p);       // [2][128]: the two threads of a row exchange their maximum, later their sum

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x, bh = blockIdx.y, bi = bh / p.heads, hi = bh % p.heads;
  const int nk = (p.lk + AF_TILE - 1) / AF_TILE;
  const bool bound_known = p.kmax2 != nullptr && p.mask == nullptr && nk >= 2;   // the same for every thread of the CTA

  if ((smem_u32(smem) & 1023u) != 0) {
    // The swizzled tiles need 1024-byte alignment; a base that is not would give wrong products, so refuse.
    if (threadIdx.x == 0 && atomicCAS(p.status, 0, (int32_t)OM_ERR_UNSUPPORTED) == 0) p.status[1] = 60;
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int a = 0; a < 2; a++) {
      mbar_init(&bar_k[a], 1);
      mbar_init(&bar_v[a], 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_staged, 256);
    mbar_init(bar_done, 1);
    mbar_init(bar_x, 256);
    *abort_flag = 0;
    *two_pass_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, AF_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  pdl_wait();

  if (warp == 8) {
    // ---- one thread loads the tiles and issues the products; step g = pass * nk + key tile ----
    if (lane == 0) {
      const uint32_t idesc_s = af_idesc(128, false, false), idesc_o = af_idesc(64, false, true);
      const uint32_t q_k = (smem_u32(slot_q) >> 4) | AF_LBO_K, k_k0 = (smem_u32(slot_k) >> 4) | AF_LBO_K;
      const uint32_t v_mn0 = (smem_u32(slot_v) >> 4) | AF_LBO_MN, p_k = (smem_u32(stage_p) >> 4) | AF_LBO_K;
      constexpr uint32_t BLK = (uint32_t)AF_BLOCK >> 4;
      auto load_k = [&](int g) {
        mbar_expect_tx(&bar_k[g & 1], AF_BLOCK);
        tma_load_4d(slot_k + (g & 1) * AF_BLOCK, &map_k, 0, (g % nk) * AF_TILE, hi, bi, &bar_k[g & 1]);
      };
      auto load_v = [&](int j) {
        mbar_expect_tx(&bar_v[j & 1], AF_BLOCK);
        tma_load_4d(slot_v + (j & 1) * AF_BLOCK, &map_v, 0, j * AF_TILE, hi, bi, &bar_v[j & 1]);
      };
      // S = Q K^T for step g into the score columns: four products of 16 head-dimension elements, 128 keys wide.
      auto issue_s = [&](int g) {
        const uint32_t kk = k_k0 + (uint32_t)(g & 1) * BLK;
#pragma unroll
        for (int ks = 0; ks < AF_D / 16; ks++) af_mma(tmem_base + AF_COL_S, q_k + ks * 2, kk + ks * 2, idesc_s, ks > 0 ? 1u : 0u);
        umma_commit(bar_s);
      };
      mbar_expect_tx(bar_q, AF_BLOCK);
      tma_load_4d(slot_q, &map_q, 0, i * AF_TILE, hi, bi, bar_q);
      int steps = 2 * nk;                     // nk when the row threads settle on one pass (known after step 0 is staged)
      bool one_pass = false;
      load_k(0);
      load_k(1);                              // 2 * nk >= 2 steps, or nk >= 2 of them
      load_v(0);
      if (nk > 1) load_v(1);
      bool ok = mbar_wait(bar_q, 0, abort_flag, p.status, 61) && mbar_wait(&bar_k[0], 0, abort_flag, p.status, 62);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int g = 0; g < steps && ok; g++) {
        const int j = g % nk;
        // The row threads have read S of step g out of tensor memory (and, in the second pass, staged P_j).
        ok = mbar_wait(bar_staged, (uint32_t)g & 1, abort_flag, p.status, 63);
        if (!ok) break;
        tc_fence_after();
        if (g == 0 && bound_known && *two_pass_flag == 0) {
          one_pass = true;
          steps = nk;
        }
        const bool second = one_pass || g >= nk;
        if (second) {
          ok = mbar_wait(&bar_v[j & 1], (uint32_t)(j >> 1) & 1, abort_flag, p.status, 64);
          if (!ok) break;
          tc_fence_after();
          // O += P_j V_j: A = P (K-major: m = queries, k = keys, 64 keys per block), B = V_j (MN-major: k = keys, n = d).
          const uint32_t vmn = v_mn0 + (uint32_t)(j & 1) * BLK;
#pragma unroll
          for (int ks = 0; ks < AF_TILE / 16; ks++)
            af_mma(tmem_base + AF_COL_O, p_k + (ks / 4) * BLK + (ks % 4) * 2, vmn + ks * 128, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
          if (g + 1 == steps) umma_commit(bar_done);
          // The staged arrival of this step came after the row threads saw S of this step, which was committed after the
          // product of tile j - 1: that product is complete and its V buffer takes tile j + 1.
          if (j >= 1 && j + 1 < nk) load_v(j + 1);
        }
        if (g + 1 < steps) {
          ok = mbar_wait(&bar_k[(g + 1) & 1], (uint32_t)((g + 1) >> 1) & 1, abort_flag, p.status, 62);
          if (!ok) break;
          tc_fence_after();
          issue_s(g + 1);
          // S of step g is complete (the row threads read it): its K buffer takes the tile of step g + 2.
          if (g + 2 < steps) load_k(g + 2);
        }
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ---- row threads: row = 32 * (warp % 4) + lane of the tile, columns 64 * (warp / 4) .. + 63 of the key tile ----
    const int quad = warp & 3, hh = warp >> 2;
    const int row = quad * 32 + lane;
    const int qrow = i * AF_TILE + row;
    const bool row_ok = qrow < p.lq;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    const float sl2 = p.scale * LOG2E;
    const float* mrow = (p.mask && row_ok) ? p.mask + (long long)bi * p.mask_batch_stride + (long long)qrow * p.lk : nullptr;
    float m = -INFINITY, m2 = 0.f, l = 0.f;
    bool ok = true;
    // The 256 row threads meet on a barrier of their own (bounded like every other wait, where bar.sync is not).
    uint32_t n_meet = 0;
    auto meet = [&]() {
      af_arrive(bar_x);
      const bool got = mbar_wait(bar_x, n_meet & 1, abort_flag, p.status, 67);
      n_meet++;
      return got;
    };
    // One pass if every row of the tile has a bound on its scores that exponentials can be taken against.
    bool one_pass = false;
    if (bound_known) {
      ok = mbar_wait(bar_q, 0, abort_flag, p.status, 68);
      if (ok) {
        // |q|^2 of this row from the swizzled tile (the order of the eight 16-byte chunks does not matter for a sum).
        const uint8_t* qr = slot_q + (size_t)row * 128;
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < 8; c++) {
          const uint4 v = *reinterpret_cast<const uint4*>(qr + (((c ^ lane) & 7) << 4));
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const float lo = __uint_as_float(w[q] << 16), hi2 = __uint_as_float(w[q] & 0xFFFF0000u);
            ss = fmaf(lo, lo, ss);
            ss = fmaf(hi2, hi2, ss);
          }
        }
        const float bound = p.scale * sqrtf(ss * p.kmax2[bh]);
        if (!(bound <= AF_BOUND_LIMIT)) *two_pass_flag = 1;       // also a bound that is not a number
        ok = meet();
        if (ok && *two_pass_flag == 0) {
          one_pass = true;
          m = bound;
          m2 = m * LOG2E;
        }
      }
    }
    const int steps = one_pass ? nk : 2 * nk;
    for (int g = 0; g < steps && ok; g++) {
      const int j = g % nk;
      const bool second = one_pass || g >= nk;
      const bool edge = (j + 1) * AF_TILE > p.lk || p.mask != nullptr;
      ok = mbar_wait(bar_s, (uint32_t)g & 1, abort_flag, p.status, 65);
      if (!ok) break;
      tc_fence_after();
      const uint32_t prow = smem_u32(stage_p + hh * AF_BLOCK) + (uint32_t)row * 128u;
#pragma unroll 1
      for (int c2 = 0; c2 < 2; c2++) {
        uint32_t rs[32];
        tmem_ld_32x32b_x32(lane_base + AF_COL_S + (uint32_t)(hh * 64 + c2 * 32), rs);
        tmem_ld_wait();
        const int key0 = j * AF_TILE + hh * 64 + c2 * 32;
        if (!second) {
          if (edge) {
#pragma unroll
            for (int c = 0; c < 32; c++) {
              float sc = __uint_as_float(rs[c]) * p.scale;
              if (mrow && key0 + c < p.lk) sc = sc + mrow[key0 + c];
              if (key0 + c < p.lk) m = fmaxf(m, sc);
            }
          } else {
            float mm = __uint_as_float(rs[0]);
#pragma unroll
            for (int c = 1; c < 32; c++) mm = fmaxf(mm, __uint_as_float(rs[c]));
            // scale > 0 keeps the order: the maximum of the scaled scores is the scaled maximum (scale <= 0 takes the edge path)
            m = fmaxf(m, mm * p.scale);
          }
        } else {
          uint32_t pw[16];
#pragma unroll
          for (int c = 0; c < 16; c++) {
            float e2[2];
#pragma unroll
            for (int u = 0; u < 2; u++) {
              const int cc = 2 * c + u;
              float e;
              if (edge) {
                float sc = __uint_as_float(rs[cc]) * p.scale;
                if (mrow && key0 + cc < p.lk) sc = sc + mrow[key0 + cc];
                e = af_ex2(fmaf(sc, LOG2E, -m2));
                if (key0 + cc >= p.lk) e = 0.f;
              } else {
                e = af_ex2(fmaf(__uint_as_float(rs[cc]), sl2, -m2));
              }
              l += e;
              e2[u] = e;
            }
            pw[c] = af_pack(e2[0], e2[1]);
          }
          // 32 keys = 64 bytes = four 16-byte chunks of this row in block hh; chunk c of a row sits at c ^ (row & 7).
#pragma unroll
          for (int c4 = 0; c4 < 4; c4++) {
            const uint32_t off = (uint32_t)(((c2 * 4 + c4) ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + off), "r"(pw[4 * c4]), "r"(pw[4 * c4 + 1]), "r"(pw[4 * c4 + 2]),
                         "r"(pw[4 * c4 + 3])
                         : "memory");
          }
        }
      }
      if (!one_pass && g == nk - 1) {
        // End of the first pass: the two threads of a row combine their maxima (the staging block is not in use yet).
        xch[hh * AF_TILE + row] = m;
        if (!(ok = meet())) break;
        m = fmaxf(xch[row], xch[AF_TILE + row]);
        if (!(m > -INFINITY)) m = 0.f;      // a row with every key masked out: all exponentials are zero
        m2 = m * LOG2E;
        if (!(ok = meet())) break;          // both have read before P is staged over the exchange area
      }
      tc_fence_before();
      if (second) af_fence_async();
      af_arrive(bar_staged);
    }
    if (ok) ok = mbar_wait(bar_done, 0, abort_flag, p.status, 66);
    // Every product has completed: the staging block is free. Row sums of the two threads, in a fixed order.
    float sum = 0.f;
    if (ok) {
      tc_fence_after();
      xch[hh * AF_TILE + row] = l;
      ok = meet();
    }
    if (ok) {
      sum = xch[row] + xch[AF_TILE + row];
      ok = meet();                          // everyone has read before the slots below overwrite the exchange area
    }
    // Warp-uniform from here: the stores below synchronise the warp.
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const float inv = sum > 0.f ? 1.0f / sum : 0.f;
      if (p.lse && hh == 0 && row_ok) p.lse[(long long)bh * p.lq + qrow] = m + logf(sum);
      // O: this thread's 32 of the 64 columns, scaled, through a 4 KB slot of the staging area to a TMA store (fp32, then
      // bfloat16); rows beyond lq are clipped by the tensor map.
      uint32_t r[32];
      tmem_ld_32x32b_x32(lane_base + AF_COL_O + (uint32_t)(hh * 32), r);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 32; c++) r[c] = __float_as_uint(__uint_as_float(r[c]) * inv);
      uint8_t* slot = stage_p + warp * 4096;
      const bool live = i * AF_TILE + quad * 32 < p.lq;
      const uint32_t row_addr = smem_u32(slot) + (uint32_t)lane * 128u;
#pragma unroll
      for (int c4 = 0; c4 < 8; c4++)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (uint32_t)((c4 ^ (lane & 7)) << 4)), "r"(r[4 * c4]), "r"(r[4 * c4 + 1]),
                     "r"(r[4 * c4 + 2]), "r"(r[4 * c4 + 3])
                     : "memory");
      af_fence_async();
      __syncwarp();
      if (lane == 0 && live) af_tma_store_4d(&map_o, slot, hh * 32, i * AF_TILE + quad * 32, hi, bi);
      if (p.want16) {
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
        const uint32_t row16 = smem_u32(slot) + (uint32_t)lane * 64u;
#pragma unroll
        for (int c8 = 0; c8 < 4; c8++)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row16 + (uint32_t)((c8 ^ ((lane >> 1) & 3)) << 4)),
                       "r"(af_pack(__uint_as_float(r[8 * c8]), __uint_as_float(r[8 * c8 + 1]))),
                       "r"(af_pack(__uint_as_float(r[8 * c8 + 2]), __uint_as_float(r[8 * c8 + 3]))),
                       "r"(af_pack(__uint_as_float(r[8 * c8 + 4]), __uint_as_float(r[8 * c8 + 5]))),
                       "r"(af_pack(__uint_as_float(r[8 * c8 + 6]), __uint_as_float(r[8 * c8 + 7])))
                       : "memory");
        af_fence_async();
        __syncwarp();
        if (lane == 0 && live) af_tma_store_4d(&map_o16, slot, hh * 32, i * AF_TILE + quad * 32, hi, bi);
      }
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      __syncwarp();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, AF_TMEM_COLS);
  }
}

// Rank-4 map over a bfloat16 activation seen as [B, H, L, 64] through element strides; box = [64, 128 rows, 1, 1].
static bool fwd16_operand_map(CUtensorMap* map, const uint16_t* base, int l, int heads, int batch, long long s_row, long long s_head, long long s_batch) {
  cuuint64_t dims[4] = {(cuuint64_t)AF_D, (cuuint64_t)l, (cuuint64_t)heads, (cuuint64_t)batch};
  const cuuint64_t filler = ((cuuint64_t)s_row * 2 * (cuuint64_t)l + 15) & ~(cuuint64_t)15;
  cuuint64_t strides[3] = {(cuuint64_t)s_row * 2, heads > 1 ? (cuuint64_t)s_head * 2 : filler, batch > 1 ? (cuuint64_t)s_batch * 2 : filler};
  cuuint32_t box[4] = {(cuuint32_t)AF_D, (cuuint32_t)AF_TILE, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<uint16_t*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// Rank-4 store map over the result seen as [B, H, L, 64]; box = [32 columns, 32 rows, 1, 1]; fp32 with the 128-byte swizzle,
// bfloat16 with the 64-byte one.
static bool fwd16_store_map(CUtensorMap* map, void* base, bool half, int l, int heads, int batch, long long s_row, long long s_head, long long s_batch) {
  const cuuint64_t es = half ? 2 : 4;
  cuuint64_t dims[4] = {(cuuint64_t)AF_D, (cuuint64_t)l, (cuuint64_t)heads, (cuuint64_t)batch};
  const cuuint64_t filler = ((cuuint64_t)s_row * es * (cuuint64_t)l + 15) & ~(cuuint64_t)15;
  cuuint64_t strides[3] = {(cuuint64_t)s_row * es, heads > 1 ? (cuuint64_t)s_head * es : filler, batch > 1 ? (cuuint64_t)s_batch * es : filler};
  cuuint32_t box[4] = {32, 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_fn()(map, half ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, half ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool strides_ok(const om_head_strides* s, int heads, int batch, int mult) {
  if ((s->row % mult) || s->row <= 0) return false;
  if (heads > 1 && ((s->head % mult) || s->head <= 0)) return false;
  if (batch > 1 && ((s->batch % mult) || s->batch <= 0)) return false;
  return true;
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_attention_fwd_bf16_supported(om_ctx* ctx, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d, float scale) {
  if (!ctx || !encode_fn()) return 0;
  return (d == AF_D && lq >= 1 && lk >= 1 && b >= 1 && h >= 1 && (long long)b * h <= 65535 && scale > 0.f) ? 1 : 0;
}

int32_t om_attention_fwd_bf16(om_ctx* ctx, const uint16_t* q16, const om_head_strides* qs, const uint16_t* k16, const om_head_strides* ks,
                              const uint16_t* v16, const om_head_strides* vs, const float* mask, int64_t mask_batch_stride, int32_t b, int32_t h,
                              int32_t lq, int32_t lk, int32_t d, float scale, float* out, uint16_t* out16, const om_head_strides* os, float* lse) {
  OM_CHECK_CTX(ctx);
  if (b < 0 || h < 0 || lq < 0 || lk < 0) return fail(ctx, OM_ERR_SHAPE, "om_attention_fwd_bf16: b %d h %d lq %d lk %d", b, h, lq, lk);
  if ((long long)b * h == 0 || lq == 0) return OM_OK;
  if (lk == 0) return fail(ctx, OM_ERR_SHAPE, "om_attention_fwd_bf16: no keys");
  if (!om_attention_fwd_bf16_supported(ctx, b, h, lq, lk, d, scale))
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_fwd_bf16: head dimension %d (64 is built), %lld (batch, head) pairs (at most 65535) or scale %g (positive)",
                d, (long long)b * h, (double)scale);
  if (!q16 || !k16 || !v16 || !out) return fail(ctx, OM_ERR_ARG, "om_attention_fwd_bf16: q, k, v and the result are required");
  auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!aligned16(q16) || !aligned16(k16) || !aligned16(v16) || !strides_ok(qs, h, b, 8) || !strides_ok(ks, h, b, 8) || !strides_ok(vs, h, b, 8))
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_fwd_bf16: bfloat16 operands need 16-byte aligned bases and strides that are multiples of 8");
  if (!aligned16(out) || !strides_ok(os, h, b, 4) || (out16 && (!aligned16(out16) || !strides_ok(os, h, b, 8))))
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_fwd_bf16: the result needs a 16-byte aligned base and strides that are multiples of 4 (8 with a bfloat16 copy)");
  ProfileScope prof(ctx, "om_attention_fwd", 4.0 * b * h * (double)lq * lk * d, 2.0 * b * h * ((double)lq * d + 2.0 * (double)lk * d) + (out16 ? 6.0 : 4.0) * b * h * (double)lq * d);
  CUtensorMap mq, mk, mv, mo, mo16;
  bool ok = fwd16_operand_map(&mq, q16, lq, h, b, qs->row, qs->head, qs->batch) && fwd16_operand_map(&mk, k16, lk, h, b, ks->row, ks->head, ks->batch) &&
            fwd16_operand_map(&mv, v16, lk, h, b, vs->row, vs->head, vs->batch) && fwd16_store_map(&mo, out, false, lq, h, b, os->row, os->head, os->batch);
  mo16 = mo;
  if (ok && out16) ok = fwd16_store_map(&mo16, out16, true, lq, h, b, os->row, os->head, os->batch);
  if (!ok) return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed for the attention forward");
  AttFwd16Params p;
  p.lq = lq; p.lk = lk; p.heads = h; p.scale = scale; p.mask = mask; p.mask_batch_stride = mask_batch_stride; p.lse = lse;
  // Without a mask and with several key tiles: the largest key norm per (batch, head), for the one-pass form.
  float* kmax2 = nullptr;
  if (!mask && lk > AF_TILE) {
    OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)b * h, false, (void**)&kmax2));
    launch_chained(ctx, attention_kmax_kernel, dim3((unsigned)(b * h)), 256, 0, k16, (long long)ks->batch, (long long)ks->head, (long long)ks->row, (int)h,
                   (int)lk, kmax2);
  }
  p.kmax2 = kmax2;
  p.want16 = out16 ? 1 : 0;
  p.status = ctx->status_dev;
  const size_t smem = (size_t)7 * AF_BLOCK + 128;
  static bool set = false;
  if (!set) {
    OM_CUDA(ctx, cudaFuncSetAttribute(attention_fwd16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    OM_CUDA(ctx, cudaFuncSetAttribute(attention_fwd16_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    set = true;
  }
  const int nq = (lq + AF_TILE - 1) / AF_TILE;
  launch_chained(ctx, attention_fwd16_kernel, dim3((unsigned)nq, (unsigned)(b * h)), AF_THREADS, smem, mq, mk, mv, mo, mo16, p);
  if (kmax2) pool_free(ctx, kmax2);
  OM_LAUNCH_CHECK(ctx, "om_attention_fwd_bf16");
  return OM_OK;
}

}  // extern "C"
