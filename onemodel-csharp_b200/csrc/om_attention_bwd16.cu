// Attention backward for sequences of several tiles, fully fused, with bfloat16 product operands (the OM_BF16_OPERANDS
// tier): one CTA per (batch, head, key tile) walks the query tiles and nothing of size Lq x Lk ever reaches HBM.
//
// AttentionBackward of the reference (BackwardNn.cs:636-701), per (batch, head):
//   S = Q K^T, dP = dO V^T, P = exp(scale S + mask - lse), dot = rowsum(dO o O), dS = P (dP - dot) scale,
//   dV = P^T dO, dK = dS^T Q, dQ = dS K.
// Three launches:
//   attention_dots_kernel     dot[b, h, q] = rowsum(dO o O) from the fp32 tensors, once for all key tiles;
//   attention_bwd16_kernel    for key tile j (128 keys) and every query tile i (128 queries), in two halves of 64 keys:
//       S_h, dP_h [128 x 64]  tcgen05.mma kind::f16 (bfloat16 Q, K, V, dO tiles brought in by TMA), accumulators in tensor memory
//       P_h, dS_h             256 threads, two per score row: tcgen05.ld, exp2, rounded to bfloat16 into shared memory
//       dV_j += P^T dO_i, dK_j += dS^T Q_i   accumulated in tensor memory over i, written at the end
//       dQ_ij = dS K_j                        this key tile's part of dQ_i, written as fp32 to a workspace [key tile][b, h, q, 64]
//   attention_dq_reduce_kernel  dQ = sum over key tiles in increasing order, with its bfloat16 copy.
// The halves alternate between two accumulator buffers, so the tensor pipe computes the next half's S and dP (and the
// previous query tile's dV, dK, dQ products) while the row threads turn the current half into P and dS: the chain
// MMA -> tcgen05.ld -> exp -> shared memory -> MMA that a single buffer serialises runs two deep. With 2-byte elements one
// shared-memory tile serves a product as the K-major operand and another as the MN-major one (same 128-byte swizzle), so
// Q, K, V, dO, P and dS are each staged once. Sums are fp32 in a fixed order (the split of dQ over key tiles is by shape
// alone); every wait is bounded (om_tc.cuh).
#include <cuda_bf16.h>

#include "om_tc.cuh"

namespace om {

constexpr int AB_TILE = 128;
constexpr int AB_D = 64;
constexpr int AB_BLOCK = AB_TILE * 128;          // [128 rows x 128 bytes]: 64 bfloat16 per row
constexpr int AB_THREADS = 320;                  // warps 0-7: half a score row per thread; warp 8: MMA issue; warp 9: TMA
// Tensor-memory columns: two buffers of S_h | dP_h (64 columns each), then dV, dK and the current dQ part.
constexpr uint32_t AB_COL_SDP = 0, AB_COL_DV = 256, AB_COL_DK = 320, AB_COL_DQ = 384;

struct AttBwd16Params {
  int lq, lk, heads, bh;
  float scale;
  const float* mask;
  long long mask_batch_stride;
  const float* lse;                              // [B*H, lq]
  const float* dots;                             // [B*H, lq] rowsum(dO o O)
  const float *dk, *dv;                          // only whether they are wanted: the stores go through tensor maps
  const uint16_t *dk16, *dv16;                   // bfloat16 copies of the results (may be null)
  int32_t* status;
};

__device__ __forceinline__ void ab_arrive(uint64_t* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory"); }
__device__ __forceinline__ void ab_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float ab_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The products are issued by one thread, about forty per (key tile, query tile) pair, so what that thread executes per
// product counts: every shared-memory descriptor here has the same upper word (stride offset 1024 bytes, version 1, 128-byte
// swizzle), and its lower word is (address >> 4) | (leading offset >> 4) << 16, which steps along a tile by adding a constant.
constexpr uint32_t AB_DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t AB_LBO_K = (16u >> 4) << 16;             // K-major operand
constexpr uint32_t AB_LBO_MN = ((uint32_t)AB_BLOCK >> 4) << 16;   // MN-major operand: 64-element chunks one block apart
__device__ __forceinline__ void ab_mma(uint32_t tmem_c, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, {%6, %6, %6, %6}, p;\n\t}"
      ::"r"(tmem_c), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(AB_DESC_HI), "r"(0u)
      : "memory");
}
// kind::f16, bfloat16 A and B, fp32 accumulator, M = 128, N = 64.
__device__ __forceinline__ uint32_t ab_idesc(bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(64 >> 3) << 17) |
         ((uint32_t)(AB_TILE >> 4) << 24);
}
__device__ __forceinline__ uint32_t ab_pack(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// A 32 x 32 block of an accumulator (lane l holds row l) into a 4 KB staging slot in the layout of a TMA store with the
// 128-byte swizzle (fp32: 16-byte chunk c of row r at c ^ (r & 7)) or the 64-byte swizzle (bfloat16: chunk c at
// c ^ ((r >> 1) & 3)); one lane then hands the slot to the TMA unit, which clips rows beyond the tensor's extent.
__device__ __forceinline__ void ab_stage_f32(uint8_t* slot, int lane, const uint32_t (&r)[32]) {
  const uint32_t row_addr = smem_u32(slot) + (uint32_t)lane * 128u;
#pragma unroll
  for (int c4 = 0; c4 < 8; c4++)
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (uint32_t)((c4 ^ (lane & 7)) << 4)), "r"(r[4 * c4]), "r"(r[4 * c4 + 1]),
                 "r"(r[4 * c4 + 2]), "r"(r[4 * c4 + 3])
                 : "memory");
}
__device__ __forceinline__ void ab_stage_bf16(uint8_t* slot, int lane, const uint32_t (&r)[32]) {
  const uint32_t row16 = smem_u32(slot) + (uint32_t)lane * 64u;
#pragma unroll
  for (int c8 = 0; c8 < 4; c8++)
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row16 + (uint32_t)((c8 ^ ((lane >> 1) & 3)) << 4)),
                 "r"(ab_pack(__uint_as_float(r[8 * c8]), __uint_as_float(r[8 * c8 + 1]))),
                 "r"(ab_pack(__uint_as_float(r[8 * c8 + 2]), __uint_as_float(r[8 * c8 + 3]))),
                 "r"(ab_pack(__uint_as_float(r[8 * c8 + 4]), __uint_as_float(r[8 * c8 + 5]))),
                 "r"(ab_pack(__uint_as_float(r[8 * c8 + 6]), __uint_as_float(r[8 * c8 + 7])))
                 : "memory");
}
__device__ __forceinline__ void ab_tma_store_3d(const CUtensorMap* map, const uint8_t* slot, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2),
               "r"(smem_u32(slot))
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void ab_tma_store_4d(const CUtensorMap* map, const uint8_t* slot, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2),
               "r"(c3), "r"(smem_u32(slot))
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// The slot's previous store has read it (lane 0 issued it), so the warp may overwrite the slot.
__device__ __forceinline__ void ab_slot_free(int lane) {
  if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  __syncwarp();
}

// dot[bh, q] = sum_d dO[b, q, h, d] * O[b, q, h, d]: a warp per row, two elements per lane, lanes combined in a butterfly.
// Rows are taken in the order (batch, query, head), the order of memory for activations stored [batch, query, head * 64], so
// that the warps of a CTA read one contiguous stretch.
__global__ void __launch_bounds__(256)
attention_dots_kernel(const float* __restrict__ g, const float* __restrict__ out, long long g_batch, long long g_head, long long g_row,
                      long long o_batch, long long o_head, long long o_row, int heads, int lq, long long rows, float* __restrict__ dots) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), warps = (long long)gridDim.x * (blockDim.x >> 5);
  // Row indices fit 31 bits (the host checks); 32-bit arithmetic keeps the index computation off the critical path.
  const unsigned nrows = (unsigned)rows, uh = (unsigned)heads, ulq = (unsigned)lq;
  for (unsigned r0 = (unsigned)warp * 8u; r0 < nrows; r0 += (unsigned)warps * 8u) {
    float2 a[8], b[8];
    int slot[8];
    unsigned hi = r0 % uh, t = r0 / uh, q = t % ulq, bi = t / ulq;
#pragma unroll
    for (int u = 0; u < 8; u++) {
      a[u] = b[u] = make_float2(0.f, 0.f);
      slot[u] = -1;
      if (r0 + u < nrows) {
        a[u] = *reinterpret_cast<const float2*>(g + (long long)bi * g_batch + (long long)hi * g_head + (long long)q * g_row + 2 * lane);
        b[u] = *reinterpret_cast<const float2*>(out + (long long)bi * o_batch + (long long)hi * o_head + (long long)q * o_row + 2 * lane);
        slot[u] = (int)((bi * uh + hi) * ulq + q);
      }
      if (++hi == uh) {
        hi = 0;
        if (++q == ulq) {
          q = 0;
          bi++;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; u++) {
      float acc = a[u].x * b[u].x + a[u].y * b[u].y;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0 && slot[u] >= 0) dots[slot[u]] = acc;
    }
  }
}

// dQ[b, q, h, :] = sum over key tiles of the parts, in increasing order. CTA (x, bh) takes 512 groups of four columns of
// one (batch, head); a thread owns two of them and has four parts of each in flight. No division per element: the head
// is the CTA's y index and a row of 64 columns is 16 groups.
__global__ void __launch_bounds__(256)
attention_dq_reduce_kernel(const float* __restrict__ parts, int nk, long long part_stride, int heads, int lq, float* __restrict__ dq,
                           uint16_t* __restrict__ dq16, long long dq_batch, long long dq_head, long long dq_row) {
  pdl_enter();
  const int bh = blockIdx.y, bi = bh / heads, hi = bh - bi * heads;
  const int per_head = lq * (AB_D / 4);
  const float4* src = reinterpret_cast<const float4*>(parts) + (long long)bh * per_head;
  const long long part4 = part_stride / 4;
  const long long obase = bi * dq_batch + hi * dq_head;
  int t[2];
  t[0] = blockIdx.x * 512 + threadIdx.x;
  t[1] = t[0] + 256;
  float4 acc[2];
  acc[0] = acc[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j0 = 0; j0 < nk; j0 += 4) {
    float4 v[2][4];
#pragma unroll
    for (int e = 0; e < 2; e++)
#pragma unroll
      for (int u = 0; u < 4; u++)
        if (t[e] < per_head && j0 + u < nk) v[e][u] = __ldcs(src + (long long)(j0 + u) * part4 + t[e]);
#pragma unroll
    for (int e = 0; e < 2; e++)
#pragma unroll
      for (int u = 0; u < 4; u++)
        if (t[e] < per_head && j0 + u < nk) {
          if (j0 + u == 0) acc[e] = v[e][u];
          else { acc[e].x += v[e][u].x; acc[e].y += v[e][u].y; acc[e].z += v[e][u].z; acc[e].w += v[e][u].w; }
        }
  }
#pragma unroll
  for (int e = 0; e < 2; e++) {
    if (t[e] >= per_head) continue;
    const long long o = obase + (long long)(t[e] >> 4) * dq_row + (t[e] & 15) * 4;
    if (dq) *reinterpret_cast<float4*>(dq + o) = acc[e];
    if (dq16) *reinterpret_cast<uint2*>(dq16 + o) = make_uint2(ab_pack(acc[e].x, acc[e].y), ab_pack(acc[e].z, acc[e].w));
  }
}

// One half-step of a row thread: 32 scores and 32 values of dP out of registers into P and dS as packed bfloat16. EDGE: the
// tile holds rows beyond lq or keys beyond lk, or a mask is added.
template <bool EDGE>
__device__ __forceinline__ void ab_scores(const uint32_t (&rs)[32], const uint32_t (&rd)[32], uint32_t (&pw)[16], uint32_t (&sw)[16], float scale,
                                          float dot, float lse_l, bool row_ok, const float* mrow, int key0, int lk) {
  const float LOG2E = 1.4426950408889634f;
  const float sl2 = scale * LOG2E;
#pragma unroll
  for (int c = 0; c < 16; c++) {
    float e2[2], d2[2];
#pragma unroll
    for (int u = 0; u < 2; u++) {
      const int jj = 2 * c + u;
      float e;
      if (EDGE) {
        float sc = __uint_as_float(rs[jj]) * scale;
        if (mrow && key0 + jj < lk) sc = sc + mrow[key0 + jj];
        e = ab_ex2(fmaf(sc, LOG2E, -lse_l));
        if (!row_ok || key0 + jj >= lk) e = 0.f;
      } else {
        e = ab_ex2(fmaf(__uint_as_float(rs[jj]), sl2, -lse_l));
      }
      e2[u] = e;
      d2[u] = (e * (__uint_as_float(rd[jj]) - dot)) * scale;
    }
    pw[c] = ab_pack(e2[0], e2[1]);
    sw[c] = ab_pack(d2[0], d2[1]);
  }
}

__global__ void __launch_bounds__(AB_THREADS, 1)
attention_bwd16_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_g,
                       const __grid_constant__ CUtensorMap map_parts, const __grid_constant__ CUtensorMap map_dk,
                       const __grid_constant__ CUtensorMap map_dk16, const __grid_constant__ CUtensorMap map_dv,
                       const __grid_constant__ CUtensorMap map_dv16, AttBwd16Params p) {
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* slot_k = smem;                               // K_j: S (K-major B), dQ (MN-major B)
  uint8_t* slot_v = smem + AB_BLOCK;                    // V_j: dP (K-major B)
  uint8_t* slot_q = smem + 2 * AB_BLOCK;                // Q_i, two buffers: S (K-major A), dK (MN-major B)
  uint8_t* slot_g = smem + 4 * AB_BLOCK;                // dO_i, two buffers: dP (K-major A), dV (MN-major B)
  uint8_t* stage_p = smem + 6 * AB_BLOCK;               // P: two blocks of [128 queries x 64 keys]; dV (MN-major A)
  uint8_t* stage_s = smem + 8 * AB_BLOCK;               // dS: the same shape; dQ (K-major A), dK (MN-major A)
  uint8_t* slots = smem + 10 * AB_BLOCK;                // a 4 KB staging slot per row warp for the TMA stores of results
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 10 * AB_BLOCK + 8 * 4096);
  uint64_t *bar_kv = bars, *bar_qg = bars + 1 /* [2] */, *bar_sdp = bars + 3 /* [2] */, *bar_staged = bars + 5 /* [2] */, *bar_out = bars + 7 /* [2] */,
           *bar_dqread = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x, bh = blockIdx.y, bi = bh / p.heads, hi = bh % p.heads;
  const int nq = (p.lq + AB_TILE - 1) / AB_TILE;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int a = 0; a < 2; a++) {
      mbar_init(&bar_qg[a], 1);
      mbar_init(&bar_sdp[a], 1);
      mbar_init(&bar_staged[a], 256);
      mbar_init(&bar_out[a], 1);
    }
    mbar_init(bar_dqread, 256);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  pdl_wait();

  if (warp == 9) {
    // ---- TMA producer: K_j and V_j once, then Q_i and dO_i into the buffer that query tile i - 2 has left ----
    if (lane == 0) {
      mbar_expect_tx(bar_kv, 2 * AB_BLOCK);
      tma_load_4d(slot_k, &map_k, 0, j * AB_TILE, hi, bi, bar_kv);
      tma_load_4d(slot_v, &map_v, 0, j * AB_TILE, hi, bi, bar_kv);
      for (int i = 0; i < nq; i++) {
        const int buf = i & 1;
        // The products of query tile i - 2 (the last readers of this buffer) are complete.
        if (i >= 2 && !mbar_wait(&bar_out[buf], (uint32_t)((i - 2) >> 1) & 1, abort_flag, p.status, 51)) break;
        mbar_expect_tx(&bar_qg[buf], 2 * AB_BLOCK);
        tma_load_4d(slot_q + buf * AB_BLOCK, &map_q, 0, i * AB_TILE, hi, bi, &bar_qg[buf]);
        tma_load_4d(slot_g + buf * AB_BLOCK, &map_g, 0, i * AB_TILE, hi, bi, &bar_qg[buf]);
      }
    }
  } else if (warp == 8) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const uint32_t idesc_kk = ab_idesc(false, false), idesc_mm = ab_idesc(true, true), idesc_km = ab_idesc(false, true);
      // Lower descriptor words of every operand tile (>> 4: 16-byte units).
      const uint32_t p_mn = (smem_u32(stage_p) >> 4) | AB_LBO_MN, s_mn = (smem_u32(stage_s) >> 4) | AB_LBO_MN, s_k = (smem_u32(stage_s) >> 4) | AB_LBO_K;
      const uint32_t k_k = (smem_u32(slot_k) >> 4) | AB_LBO_K, k_mn = (smem_u32(slot_k) >> 4) | AB_LBO_MN, v_k = (smem_u32(slot_v) >> 4) | AB_LBO_K;
      const uint32_t q_k0 = (smem_u32(slot_q) >> 4) | AB_LBO_K, q_mn0 = (smem_u32(slot_q) >> 4) | AB_LBO_MN;
      const uint32_t g_k0 = (smem_u32(slot_g) >> 4) | AB_LBO_K, g_mn0 = (smem_u32(slot_g) >> 4) | AB_LBO_MN;
      constexpr uint32_t BLK = (uint32_t)AB_BLOCK >> 4, HALF = (64u * 128u) >> 4;
      // S_h = Q_i K_j[h]^T and dP_h = dO_i V_j[h]^T into accumulator buffer h: 128 queries x 64 keys each, contraction
      // over the head dimension (a step of 16 elements is 32 bytes along the swizzled row).
      auto issue_sdp = [&](int i, int h) {
        const uint32_t qk = q_k0 + (uint32_t)(i & 1) * BLK, gk = g_k0 + (uint32_t)(i & 1) * BLK;
        const uint32_t kk = k_k + (uint32_t)h * HALF, vk = v_k + (uint32_t)h * HALF;
        const uint32_t col = tmem_base + AB_COL_SDP + (uint32_t)h * 128u;
#pragma unroll
        for (int ks = 0; ks < AB_D / 16; ks++) ab_mma(col, qk + ks * 2, kk + ks * 2, idesc_kk, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < AB_D / 16; ks++) ab_mma(col + 64u, gk + ks * 2, vk + ks * 2, idesc_kk, ks > 0 ? 1u : 0u);
        umma_commit(&bar_sdp[h]);
      };
      bool ok = mbar_wait(bar_kv, 0, abort_flag, p.status, 52) && mbar_wait(&bar_qg[0], 0, abort_flag, p.status, 53);
      if (ok) {
        tc_fence_after();
        issue_sdp(0, 0);
        issue_sdp(0, 1);
      }
      for (int i = 0; i < nq && ok; i++) {
        for (int h = 0; h < 2 && ok; h++) {
          // The row threads have read S_h and dP_h of query tile i out of buffer h and staged P_h and dS_h.
          ok = mbar_wait(&bar_staged[h], (uint32_t)i & 1, abort_flag, p.status, 55);
          if (!ok) break;
          tc_fence_after();
          if (h == 1) {
            // The previous tile's part of dQ has been read out of tensor memory.
            if (i > 0 && !(ok = mbar_wait(bar_dqread, (uint32_t)(i - 1) & 1, abort_flag, p.status, 56))) break;
            tc_fence_after();
            const uint32_t qmn = q_mn0 + (uint32_t)(i & 1) * BLK, gmn = g_mn0 + (uint32_t)(i & 1) * BLK;
            const uint32_t first = i > 0 ? 1u : 0u;
            // dV_j += P^T dO_i: A = P^T (MN-major: m = keys, k = queries), B = dO_i (MN-major: k = queries, n = d); a step of
            // 16 queries is 16 rows of 128 bytes.
#pragma unroll
            for (int ks = 0; ks < AB_TILE / 16; ks++) ab_mma(tmem_base + AB_COL_DV, p_mn + ks * 128, gmn + ks * 128, idesc_mm, ks > 0 ? 1u : first);
            // dK_j += dS^T Q_i.
#pragma unroll
            for (int ks = 0; ks < AB_TILE / 16; ks++) ab_mma(tmem_base + AB_COL_DK, s_mn + ks * 128, qmn + ks * 128, idesc_mm, ks > 0 ? 1u : first);
            // dQ_ij = dS K_j: A = dS (K-major: m = queries, k = keys, 64 keys per block), B = K_j (MN-major: k = keys, n = d).
#pragma unroll
            for (int ks = 0; ks < AB_TILE / 16; ks++)
              ab_mma(tmem_base + AB_COL_DQ, s_k + (ks / 4) * BLK + (ks % 4) * 2, k_mn + ks * 128, idesc_km, ks > 0 ? 1u : 0u);
            umma_commit(&bar_out[i & 1]);
          }
          if (i + 1 < nq) {
            if (h == 0 && !(ok = mbar_wait(&bar_qg[(i + 1) & 1], (uint32_t)((i + 1) >> 1) & 1, abort_flag, p.status, 53))) break;
            tc_fence_after();
            issue_sdp(i + 1, h);
          }
        }
      }
      if (!ok) *abort_flag = 1;     // let the row threads out of whatever they wait for
    }
  } else {
    // ---- row threads: row = 32 * (warp % 4) + lane of the tile, columns 32 * (warp / 4) .. + 31 of each 64-key half ----
    const int quad = warp & 3, hh = warp >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    uint8_t* slot = slots + warp * 4096;
    bool ok = true;
    // This warp's 32 x 32 block of the part of dQ for query tile i: out of tensor memory, through the slot, to the workspace
    // [key tile * (batch, head)][query][64] by a TMA store (rows beyond lq are clipped).
    auto drain_dq = [&](int i) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(lane_base + AB_COL_DQ + (uint32_t)(hh * 32), r);
      tmem_ld_wait();
      ab_slot_free(lane);
      ab_stage_f32(slot, lane, r);
      ab_fence_async();
      __syncwarp();
      if (lane == 0 && i * AB_TILE + quad * 32 < p.lq) ab_tma_store_3d(&map_parts, slot, hh * 32, i * AB_TILE + quad * 32, j * p.bh + bh);
    };
    const bool key_edge = (j + 1) * AB_TILE > p.lk || p.mask != nullptr;
    for (int i = 0; i < nq && ok; i++) {
      const int qrow = i * AB_TILE + row;
      const bool row_ok = qrow < p.lq;
      const bool edge = key_edge || (i + 1) * AB_TILE > p.lq;
      const float dot = row_ok ? __ldg(p.dots + (long long)bh * p.lq + qrow) : 0.f;
      const float lse_l = row_ok ? __ldg(p.lse + (long long)bh * p.lq + qrow) * LOG2E : 0.f;
      const float* mrow = (p.mask && row_ok) ? p.mask + (long long)bi * p.mask_batch_stride + (long long)qrow * p.lk : nullptr;
      for (int h = 0; h < 2 && ok; h++) {
        ok = mbar_wait(&bar_sdp[h], (uint32_t)i & 1, abort_flag, p.status, 57);
        if (!ok) break;
        tc_fence_after();
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(lane_base + AB_COL_SDP + (uint32_t)(h * 128 + hh * 32), rs);
        tmem_ld_32x32b_x32(lane_base + AB_COL_SDP + (uint32_t)(h * 128 + 64 + hh * 32), rd);
        tmem_ld_wait();
        const int key0 = j * AB_TILE + h * 64 + hh * 32;
        uint32_t pw[16], sw[16];
        if (edge) ab_scores<true>(rs, rd, pw, sw, p.scale, dot, lse_l, row_ok, mrow, key0, p.lk);
        else ab_scores<false>(rs, rd, pw, sw, p.scale, dot, lse_l, true, nullptr, key0, p.lk);
        // The staging blocks are free once the previous query tile's products have read them (which also completes that
        // tile's part of dQ).
        if (h == 0 && i > 0) {
          ok = mbar_wait(&bar_out[(i - 1) & 1], (uint32_t)((i - 1) >> 1) & 1, abort_flag, p.status, 58);
          if (!ok) break;
          tc_fence_after();
        }
        // 32 keys = 64 bytes = four 16-byte chunks of row `row` in block h; chunk c of a row sits at c ^ (row & 7).
        const uint32_t prow = smem_u32(stage_p + h * AB_BLOCK) + (uint32_t)row * 128u;
        const uint32_t srow = smem_u32(stage_s + h * AB_BLOCK) + (uint32_t)row * 128u;
#pragma unroll
        for (int c4 = 0; c4 < 4; c4++) {
          const uint32_t off = (uint32_t)(((hh * 4 + c4) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + off), "r"(pw[4 * c4]), "r"(pw[4 * c4 + 1]), "r"(pw[4 * c4 + 2]),
                       "r"(pw[4 * c4 + 3])
                       : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + off), "r"(sw[4 * c4]), "r"(sw[4 * c4 + 1]), "r"(sw[4 * c4 + 2]),
                       "r"(sw[4 * c4 + 3])
                       : "memory");
        }
        tc_fence_before();
        ab_fence_async();
        ab_arrive(&bar_staged[h]);
        if (h == 0 && i > 0) {
          drain_dq(i - 1);
          tc_fence_before();
          ab_arrive(bar_dqread);
        }
      }
    }
    if (ok) ok = mbar_wait(&bar_out[(nq - 1) & 1], (uint32_t)((nq - 1) >> 1) & 1, abort_flag, p.status, 59);
    if (ok) {
      tc_fence_after();
      drain_dq(nq - 1);
      // dV_j (warps 0-3) and dK_j (warps 4-7): 32 key rows per warp, 64 columns as two blocks, fp32 and bfloat16.
      const bool want32 = hh == 0 ? p.dv != nullptr : p.dk != nullptr;
      const bool want16 = hh == 0 ? p.dv16 != nullptr : p.dk16 != nullptr;
      const bool want = want32 || want16;
      const CUtensorMap* m32 = hh == 0 ? &map_dv : &map_dk;
      const CUtensorMap* m16 = hh == 0 ? &map_dv16 : &map_dk16;
      if (want && j * AB_TILE + quad * 32 < p.lk) {
        // P and dS are dead (every product has completed): each warp takes 8 KB of their space, so that with its own slot no
        // store has to wait for an earlier one to leave shared memory.
        uint8_t* big = stage_p + warp * 8192;
#pragma unroll 1
        for (int cb = 0; cb < 2; cb++) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(lane_base + (hh == 0 ? AB_COL_DV : AB_COL_DK) + (uint32_t)(cb * 32), r);
          tmem_ld_wait();
          uint8_t* f32_slot = cb == 0 ? slot : big;
          uint8_t* b16_slot = big + 4096 + cb * 2048;
          if (cb == 0) ab_slot_free(lane);
          if (want32) ab_stage_f32(f32_slot, lane, r);
          if (want16) ab_stage_bf16(b16_slot, lane, r);
          ab_fence_async();
          __syncwarp();
          if (lane == 0) {
            if (want32) ab_tma_store_4d(m32, f32_slot, cb * 32, j * AB_TILE + quad * 32, hi, bi);
            if (want16) ab_tma_store_4d(m16, b16_slot, cb * 32, j * AB_TILE + quad * 32, hi, bi);
          }
        }
      }
    }
    ab_slot_free(lane);      // the TMA unit has read the slot: shared memory may go
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Rank-4 map over a bfloat16 activation seen as [B, H, L, 64] through element strides; box = [64, 128 rows, 1, 1].
static bool att16_map(CUtensorMap* map, const uint16_t* base, int l, int heads, int batch, long long s_row, long long s_head, long long s_batch) {
  cuuint64_t dims[4] = {(cuuint64_t)AB_D, (cuuint64_t)l, (cuuint64_t)heads, (cuuint64_t)batch};
  const cuuint64_t filler = ((cuuint64_t)s_row * 2 * (cuuint64_t)l + 15) & ~(cuuint64_t)15;
  cuuint64_t strides[3] = {(cuuint64_t)s_row * 2, heads > 1 ? (cuuint64_t)s_head * 2 : filler, batch > 1 ? (cuuint64_t)s_batch * 2 : filler};
  cuuint32_t box[4] = {(cuuint32_t)AB_D, (cuuint32_t)AB_TILE, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<uint16_t*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Rank-4 store map over a result seen as [B, H, L, 64] through element strides; box = [32 columns, 32 rows, 1, 1]. fp32 takes
// the 128-byte swizzle, bfloat16 (64 bytes per row of the box) the 64-byte one.
static bool att16_store_map(CUtensorMap* map, void* base, bool half, int l, int heads, int batch, long long s_row, long long s_head, long long s_batch) {
  const cuuint64_t es = half ? 2 : 4;
  cuuint64_t dims[4] = {(cuuint64_t)AB_D, (cuuint64_t)l, (cuuint64_t)heads, (cuuint64_t)batch};
  const cuuint64_t filler = ((cuuint64_t)s_row * es * (cuuint64_t)l + 15) & ~(cuuint64_t)15;
  cuuint64_t strides[3] = {(cuuint64_t)s_row * es, heads > 1 ? (cuuint64_t)s_head * es : filler, batch > 1 ? (cuuint64_t)s_batch * es : filler};
  cuuint32_t box[4] = {32, 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_fn()(map, half ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, half ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// The workspace of the parts of dQ: [key tiles * (batch, head)][lq][64] fp32, box [32 columns, 32 rows, 1].
static bool att16_parts_map(CUtensorMap* map, float* base, int lq, long long groups) {
  cuuint64_t dims[3] = {(cuuint64_t)AB_D, (cuuint64_t)lq, (cuuint64_t)groups};
  cuuint64_t strides[2] = {(cuuint64_t)AB_D * 4, (cuuint64_t)lq * AB_D * 4};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool operand16_ok(const uint16_t* p, const om_head_strides* s, int heads, int batch) {
  if ((reinterpret_cast<uintptr_t>(p) & 15) || (s->row & 7) || s->row <= 0) return false;
  if (heads > 1 && ((s->head & 7) || s->head <= 0)) return false;
  if (batch > 1 && ((s->batch & 7) || s->batch <= 0)) return false;
  return true;
}
static bool result_ok(const float* p, const om_head_strides* s) {
  return p == nullptr || (((reinterpret_cast<uintptr_t>(p) & 15) == 0) && (s->row & 3) == 0 && (s->head & 3) == 0 && (s->batch & 3) == 0);
}

}  // namespace om

using namespace om;

extern "C" {

int32_t om_attention_bwd_bf16_supported(om_ctx* ctx, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d) {
  if (!ctx || !encode_fn()) return 0;
  return (d == AB_D && lq >= 1 && lk >= 1 && b >= 1 && h >= 1 && (long long)b * h <= 65535 && (long long)b * h * lq < (1ll << 31)) ? 1 : 0;
}

int32_t om_attention_bwd_bf16(om_ctx* ctx, const uint16_t* g16, const float* g, const om_head_strides* gs, const uint16_t* q16,
                              const om_head_strides* qs, const uint16_t* k16, const om_head_strides* ks, const uint16_t* v16,
                              const om_head_strides* vs, const float* out, const om_head_strides* os, const float* mask,
                              int64_t mask_batch_stride, const float* lse, int32_t b, int32_t h, int32_t lq, int32_t lk, int32_t d, float scale,
                              float* dq, uint16_t* dq16, const om_head_strides* dqs, float* dk, uint16_t* dk16, const om_head_strides* dks,
                              float* dv, uint16_t* dv16, const om_head_strides* dvs) {
  OM_CHECK_CTX(ctx);
  if (b < 0 || h < 0 || lq < 0 || lk < 0) return fail(ctx, OM_ERR_SHAPE, "om_attention_bwd_bf16: b %d h %d lq %d lk %d", b, h, lq, lk);
  if ((long long)b * h == 0 || lq == 0 || lk == 0) return OM_OK;
  if (!om_attention_bwd_bf16_supported(ctx, b, h, lq, lk, d))
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_bwd_bf16: head dimension %d (64 is built) or %lld (batch, head) pairs (at most 65535)", d,
                (long long)b * h);
  if (!g16 || !g || !q16 || !k16 || !v16 || !out || !lse)
    return fail(ctx, OM_ERR_ARG, "om_attention_bwd_bf16: the gradient (both forms), q, k, v, the forward's output and its log-sum-exp are required");
  if (!operand16_ok(g16, gs, h, b) || !operand16_ok(q16, qs, h, b) || !operand16_ok(k16, ks, h, b) || !operand16_ok(v16, vs, h, b))
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_bwd_bf16: bfloat16 operands need 16-byte aligned bases and strides that are multiples of 8");
  if (!result_ok(dq, dqs) || !result_ok(dk, dks) || !result_ok(dv, dvs) || (gs->row & 1) || (os->row & 1) || (reinterpret_cast<uintptr_t>(g) & 7) ||
      (reinterpret_cast<uintptr_t>(out) & 7) || (gs->head & 1) || (gs->batch & 1) || (os->head & 1) || (os->batch & 1))
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_bwd_bf16: results need 16-byte aligned bases and strides that are multiples of 4");
  // Each of dq, dk, dv may be asked for as fp32, as bfloat16, or both (bfloat16 alone is all that a following product reads).
  if ((dq16 && !dq && !result_ok(reinterpret_cast<const float*>(dq16), dqs)) || (dk16 && !dk && !result_ok(reinterpret_cast<const float*>(dk16), dks)) ||
      (dv16 && !dv && !result_ok(reinterpret_cast<const float*>(dv16), dvs)))
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_bwd_bf16: results need 16-byte aligned bases and strides that are multiples of 4");
  auto copy_ok = [](const uint16_t* c, const om_head_strides* st) {
    return c == nullptr || (((reinterpret_cast<uintptr_t>(c) & 15) == 0) && (st->row & 7) == 0 && (st->head & 7) == 0 && (st->batch & 7) == 0);
  };
  if (!copy_ok(dk16, dks) || !copy_ok(dv16, dvs) || (dq16 && (reinterpret_cast<uintptr_t>(dq16) & 7)))
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_bwd_bf16: the bfloat16 copies of dk and dv need 16-byte aligned bases and strides that are multiples of 8");
  ProfileScope prof(ctx, "om_attention_bwd", 8.0 * b * h * (double)lq * lk * d, 2.0 * b * h * ((double)lq * d * 2 + (double)lk * d * 2) + 4.0 * b * h * ((double)lq * d * 3 + (double)lk * d * 2));
  CUtensorMap mq, mk, mv, mg;
  if (!att16_map(&mq, q16, lq, h, b, qs->row, qs->head, qs->batch) || !att16_map(&mk, k16, lk, h, b, ks->row, ks->head, ks->batch) ||
      !att16_map(&mv, v16, lk, h, b, vs->row, vs->head, vs->batch) || !att16_map(&mg, g16, lq, h, b, gs->row, gs->head, gs->batch))
    return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed for the attention operands");
  const int bh = b * h, nk = (lk + AB_TILE - 1) / AB_TILE;
  const long long rows = (long long)bh * lq;
  float *dots = nullptr, *parts = nullptr;
  OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)rows, false, (void**)&dots));
  int32_t st = pool_alloc(ctx, sizeof(float) * (size_t)nk * rows * AB_D, false, (void**)&parts);
  if (st != OM_OK) {
    pool_free(ctx, dots);
    return st;
  }
  launch_chained(ctx, attention_dots_kernel, grid_for(ctx, (rows + 7) / 8 * 32, 256, 16), 256, 0, g, out, (long long)gs->batch, (long long)gs->head,
                 (long long)gs->row, (long long)os->batch, (long long)os->head, (long long)os->row, (int)h, (int)lq, rows, dots);
  AttBwd16Params p;
  p.lq = lq; p.lk = lk; p.heads = h; p.bh = bh; p.scale = scale; p.mask = mask; p.mask_batch_stride = mask_batch_stride; p.lse = lse;
  p.dots = dots;
  p.dk = dk; p.dv = dv; p.dk16 = dk16; p.dv16 = dv16;
  p.status = ctx->status_dev;
  CUtensorMap mparts, mdk, mdk16, mdv, mdv16;
  bool maps = att16_parts_map(&mparts, parts, lq, (long long)nk * bh);
  mdk = mdk16 = mdv = mdv16 = mparts;     // a parameter must hold a valid map even when its result is not wanted
  if (dk) maps = maps && att16_store_map(&mdk, dk, false, lk, h, b, dks->row, dks->head, dks->batch);
  if (dk16) maps = maps && att16_store_map(&mdk16, dk16, true, lk, h, b, dks->row, dks->head, dks->batch);
  if (dv) maps = maps && att16_store_map(&mdv, dv, false, lk, h, b, dvs->row, dvs->head, dvs->batch);
  if (dv16) maps = maps && att16_store_map(&mdv16, dv16, true, lk, h, b, dvs->row, dvs->head, dvs->batch);
  if (!maps) {
    pool_free(ctx, parts);
    pool_free(ctx, dots);
    return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed for the attention results");
  }
  const size_t smem = (size_t)10 * AB_BLOCK + 8 * 4096 + 128 + 1024;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(attention_bwd16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      pool_free(ctx, parts);
      pool_free(ctx, dots);
      return check_cuda(ctx, e, "om_attention_bwd_bf16");
    }
    set = true;
  }
  launch_chained(ctx, attention_bwd16_kernel, dim3((unsigned)nk, (unsigned)bh), AB_THREADS, smem, mq, mk, mv, mg, mparts, mdk, mdk16, mdv, mdv16, p);
  if (dq || dq16) {
    const dim3 grid((unsigned)ceil_div((long long)lq * (AB_D / 4), 512), (unsigned)bh);
    launch_chained(ctx, attention_dq_reduce_kernel, grid, 256, 0, (const float*)parts, nk, rows * AB_D, (int)h, (int)lq, dq, dq16,
                   (long long)dqs->batch, (long long)dqs->head, (long long)dqs->row);
  }
  pool_free(ctx, parts);
  pool_free(ctx, dots);
  OM_LAUNCH_CHECK(ctx, "om_attention_bwd_bf16");
  return OM_OK;
}

}  // extern "C"
