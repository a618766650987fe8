// Attention backward for sequences of several tiles, fully fused, with bfloat16 product operands (the OM_BF16_OPERANDS
// tier): one CTA per (batch, head) walks all (key tile, query tile) pairs and nothing of size Lq x Lk ever reaches HBM.
//
// AttentionBackward of the reference (BackwardNn.cs:636-701), per (batch, head):
//   S = Q K^T, dP = dO V^T, P = exp(scale S + mask - lse), dot = rowsum(dO o O), dS = P (dP - dot) scale,
//   dV = P^T dO, dK = dS^T Q, dQ = dS K.
// Here, for key tile j (128 keys) and query tile i (128 queries), in two halves of 64 keys:
//   S_h, dP_h [128 x 64]  tcgen05.mma kind::f16 (bfloat16 Q, K, V, dO tiles brought in by TMA), accumulators in tensor memory
//   P_h, dS_h             256 threads, two per score row: tcgen05.ld, exp2, rounded to bfloat16 into shared memory
//   dV_j += P^T dO_i, dK_j += dS^T Q_i, dQ_i += dS K_j      accumulated in tensor memory over i (dV, dK) and over j (dQ)
// dV_j and dK_j are written when the query tiles of key tile j are done; the dQ tiles (at most four: Lq <= 512, head
// dimension 64) stay in tensor memory until the end. With 2-byte elements one shared-memory tile serves a product as the
// K-major operand and another as the MN-major one (same 128-byte swizzle), so Q, K, V, dO, P and dS are each staged once.
// Sums are fp32 in a fixed order; every wait is bounded (om_tc.cuh).
#include <cuda_bf16.h>

#include "om_tc.cuh"

namespace om {

constexpr int AB_TILE = 128;
constexpr int AB_D = 64;
constexpr int AB_BLOCK = AB_TILE * 128;          // [128 rows x 128 bytes]: 64 bfloat16 per row
constexpr int AB_THREADS = 288;                  // warps 0-7: half a score row per thread; warp 8: TMA + MMA issue
constexpr int AB_MAX_Q_TILES = 4;
constexpr uint32_t AB_COL_S = 0, AB_COL_DP = 64, AB_COL_DV = 128, AB_COL_DK = 192, AB_COL_DQ = 256;

struct AttBwd16Params {
  int lq, lk, heads;
  float scale;
  const float* mask;
  long long mask_batch_stride;
  const float* lse;                              // [B*H, lq]
  const float *g, *out;                          // fp32 dO and O for the row dots
  long long g_batch, g_head, g_row, o_batch, o_head, o_row;
  float *dq, *dk, *dv;
  uint16_t *dq16, *dk16, *dv16;                  // bfloat16 copies of the results (may be null)
  long long dq_batch, dq_head, dq_row, dk_batch, dk_head, dk_row, dv_batch, dv_head, dv_row;
  int32_t* status;
};

__device__ __forceinline__ void ab_arrive(uint64_t* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory"); }
__device__ __forceinline__ void ab_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float ab_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void ab_mma(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
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

// One 32 x 32 block of an accumulator (lane l holds row l) to global memory as fp32 and, optionally, bfloat16: turned
// through shared memory so that eight lanes write one 128-byte row segment.
__device__ __forceinline__ void ab_store_block(float* stg, int lane, const uint32_t (&r)[32], float* dst, uint16_t* dst16, long long row_stride,
                                               int row0, int rows_valid, int col0) {
#pragma unroll
  for (int j = 0; j < 32; j += 4)
    *reinterpret_cast<float4*>(stg + lane * 36 + j) =
        make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int rr = i * 4 + (lane >> 3);
    if (row0 + rr < rows_valid) {
      const float4 v = *reinterpret_cast<const float4*>(stg + rr * 36 + (lane & 7) * 4);
      const long long o = (long long)(row0 + rr) * row_stride + col0 + (lane & 7) * 4;
      *reinterpret_cast<float4*>(dst + o) = v;
      if (dst16) *reinterpret_cast<uint2*>(dst16 + o) = make_uint2(ab_pack(v.x, v.y), ab_pack(v.z, v.w));
    }
  }
  __syncwarp();
}

__global__ void __launch_bounds__(AB_THREADS, 1)
attention_bwd16_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_g, AttBwd16Params p) {
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* slot_k = smem;                               // K_j, two buffers: S (K-major B), dQ (MN-major B)
  uint8_t* slot_v = smem + 2 * AB_BLOCK;                // V_j, two buffers: dP (K-major B)
  uint8_t* slot_q = smem + 4 * AB_BLOCK;                // Q_i, two buffers: S (K-major A), dK (MN-major B)
  uint8_t* slot_g = smem + 6 * AB_BLOCK;                // dO_i, two buffers: dP (K-major A), dV (MN-major B)
  uint8_t* stage_p = smem + 8 * AB_BLOCK;               // P: two blocks of [128 queries x 64 keys]; dV (MN-major A)
  uint8_t* stage_s = smem + 10 * AB_BLOCK;              // dS: the same shape; dQ (K-major A), dK (MN-major A)
  float* dots = reinterpret_cast<float*>(smem + 12 * AB_BLOCK);          // [512] rowsum(dO o O)
  float* lses = dots + AB_MAX_Q_TILES * AB_TILE;                         // [512] log-sum-exp times log2(e)
  uint64_t* bars = reinterpret_cast<uint64_t*>(lses + AB_MAX_Q_TILES * AB_TILE);
  uint64_t *bar_kv = bars /* [2] */, *bar_qg = bars + 2 /* [2] */, *bar_sdp = bars + 4, *bar_staged = bars + 5, *bar_jdone = bars + 6, *bar_epi = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, bi = bh / p.heads, hi = bh % p.heads;
  const int nq = (p.lq + AB_TILE - 1) / AB_TILE, nk = (p.lk + AB_TILE - 1) / AB_TILE;

  if (threadIdx.x == 0) {
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
    mbar_init(&bar_qg[0], 1);
    mbar_init(&bar_qg[1], 1);
    mbar_init(bar_sdp, 1);
    mbar_init(bar_staged, 256);
    mbar_init(bar_jdone, 1);
    mbar_init(bar_epi, 256);
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

  if (warp == 8) {
    if (lane == 0) {
      const uint32_t idesc_kk = ab_idesc(false, false), idesc_mm = ab_idesc(true, true), idesc_km = ab_idesc(false, true);
      const uint32_t pa = smem_u32(stage_p), sa = smem_u32(stage_s);
      uint32_t n_sdp = 0, n_staged = 0, n_qg[2] = {0, 0};
      bool ok = true;
      const int total = nk * nq;
      auto load_kv = [&](int j) {
        const int kb = j & 1;
        mbar_expect_tx(&bar_kv[kb], 2 * AB_BLOCK);
        tma_load_4d(slot_k + kb * AB_BLOCK, &map_k, 0, j * AB_TILE, hi, bi, &bar_kv[kb]);
        tma_load_4d(slot_v + kb * AB_BLOCK, &map_v, 0, j * AB_TILE, hi, bi, &bar_kv[kb]);
      };
      // First query tile, first two key tiles.
      mbar_expect_tx(&bar_qg[0], 2 * AB_BLOCK);
      tma_load_4d(slot_q, &map_q, 0, 0, hi, bi, &bar_qg[0]);
      tma_load_4d(slot_g, &map_g, 0, 0, hi, bi, &bar_qg[0]);
      load_kv(0);
      if (nk > 1) load_kv(1);
      for (int j = 0; j < nk && ok; j++) {
        const uint32_t ka = smem_u32(slot_k + (j & 1) * AB_BLOCK), va = smem_u32(slot_v + (j & 1) * AB_BLOCK);
        ok = mbar_wait(&bar_kv[j & 1], (uint32_t)(j >> 1) & 1, abort_flag, p.status, 52);
        for (int i = 0; i < nq && ok; i++) {
          const int blk = j * nq + i, buf = blk & 1;
          ok = mbar_wait(&bar_qg[buf], n_qg[buf] & 1, abort_flag, p.status, 53);
          if (!ok) break;
          n_qg[buf]++;
          tc_fence_after();
          const uint32_t qa = smem_u32(slot_q + buf * AB_BLOCK), ga = smem_u32(slot_g + buf * AB_BLOCK);
          for (int h = 0; h < 2 && ok; h++) {
            // S_h = Q_i K_j[h]^T and dP_h = dO_i V_j[h]^T: 128 queries x 64 keys each, contraction over the head dimension.
#pragma unroll
            for (int ks = 0; ks < AB_D / 16; ks++)
              ab_mma(tmem_base + AB_COL_S, make_desc(qa + ks * 32, 16, 1024, 2), make_desc(ka + h * (64 * 128) + ks * 32, 16, 1024, 2), idesc_kk,
                     ks > 0 ? 1u : 0u);
#pragma unroll
            for (int ks = 0; ks < AB_D / 16; ks++)
              ab_mma(tmem_base + AB_COL_DP, make_desc(ga + ks * 32, 16, 1024, 2), make_desc(va + h * (64 * 128) + ks * 32, 16, 1024, 2), idesc_kk,
                     ks > 0 ? 1u : 0u);
            umma_commit(bar_sdp);
            if (h == 0 && blk + 1 < total) {
              // Everything issued before these two products has completed once they have: the other Q / dO buffer is
              // free for the next query tile.
              ok = mbar_wait(bar_sdp, n_sdp & 1, abort_flag, p.status, 54);
              if (!ok) break;
              const int ni = (i + 1) % nq, nb = buf ^ 1;
              mbar_expect_tx(&bar_qg[nb], 2 * AB_BLOCK);
              tma_load_4d(slot_q + nb * AB_BLOCK, &map_q, 0, ni * AB_TILE, hi, bi, &bar_qg[nb]);
              tma_load_4d(slot_g + nb * AB_BLOCK, &map_g, 0, ni * AB_TILE, hi, bi, &bar_qg[nb]);
            }
            n_sdp++;
            // The 256 row threads have read S_h and dP_h out of tensor memory and staged P_h and dS_h.
            ok = mbar_wait(bar_staged, n_staged & 1, abort_flag, p.status, 55);
            n_staged++;
          }
          if (!ok) break;
          if (i == 0 && j > 0) {
            // The results of the previous key tile have been read out of tensor memory (bar_epi), and with them its products
            // are complete: its accumulators may be overwritten, and its K / V buffer takes the key tile after this one.
            ok = mbar_wait(bar_epi, (uint32_t)(j - 1) & 1, abort_flag, p.status, 51);
            if (!ok) break;
            if (j + 1 < nk) load_kv(j + 1);
          }
          tc_fence_after();
          // dV_j += P^T dO_i: A = P^T (MN-major: m = keys, k = queries), B = dO_i (MN-major: k = queries, n = d).
#pragma unroll
          for (int ks = 0; ks < AB_TILE / 16; ks++)
            ab_mma(tmem_base + AB_COL_DV, make_desc(pa + ks * 2048, AB_BLOCK, 1024, 2), make_desc(ga + ks * 2048, AB_BLOCK, 1024, 2), idesc_mm,
                   (i > 0 || ks > 0) ? 1u : 0u);
          // dK_j += dS^T Q_i.
#pragma unroll
          for (int ks = 0; ks < AB_TILE / 16; ks++)
            ab_mma(tmem_base + AB_COL_DK, make_desc(sa + ks * 2048, AB_BLOCK, 1024, 2), make_desc(qa + ks * 2048, AB_BLOCK, 1024, 2), idesc_mm,
                   (i > 0 || ks > 0) ? 1u : 0u);
          // dQ_i += dS K_j: A = dS (K-major: m = queries, k = keys, 64 keys per block), B = K_j (MN-major: k = keys, n = d).
#pragma unroll
          for (int ks = 0; ks < AB_TILE / 16; ks++)
            ab_mma(tmem_base + AB_COL_DQ + (uint32_t)i * AB_D, make_desc(sa + (ks / 4) * AB_BLOCK + (ks % 4) * 32, 16, 1024, 2),
                   make_desc(ka + ks * 2048, AB_BLOCK, 1024, 2), idesc_km, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(bar_jdone);     // key tile j is complete (or nothing is outstanding after an abort)
      }
      if (!ok) {
        // Let the row threads out of whatever they wait for.
        *abort_flag = 1;
      }
    }
  } else {
    // ---- row threads: row = 32 * (warp % 4) + lane of the tile, columns 32 * (warp / 4) .. + 31 of each 64-key half ----
    const int quad = warp & 3, hh = warp >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    // Row dots and log-sum-exp of all queries: a warp per row, two elements per lane.
    {
      const float* gp = p.g + (long long)bi * p.g_batch + (long long)hi * p.g_head;
      const float* op = p.out + (long long)bi * p.o_batch + (long long)hi * p.o_head;
      for (int r0 = warp * 8; r0 < nq * AB_TILE; r0 += 64) {
        float acc[8];
        float2 a[8], b[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {      // sixteen loads in flight before the first use
          const int r = r0 + u;
          a[u] = b[u] = make_float2(0.f, 0.f);
          if (r < p.lq) {
            a[u] = *reinterpret_cast<const float2*>(gp + (long long)r * p.g_row + 2 * lane);
            b[u] = *reinterpret_cast<const float2*>(op + (long long)r * p.o_row + 2 * lane);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
          acc[u] = a[u].x * b[u].x + a[u].y * b[u].y;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
        }
        if (lane < 8) {
          const int r = r0 + lane;
          float mine = acc[0];
#pragma unroll
          for (int u = 1; u < 8; u++) mine = lane == u ? acc[u] : mine;
          dots[r] = mine;
          lses[r] = r < p.lq ? p.lse[(long long)bh * p.lq + r] * LOG2E : 0.f;
        }
      }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    uint32_t n_sdp = 0;
    bool ok = true;
    float* stg = reinterpret_cast<float*>(stage_p) + warp * 32 * 36;     // output staging: P and dS are dead by then
    for (int j = 0; j < nk && ok; j++) {
      for (int i = 0; i < nq && ok; i++) {
        const int qrow = i * AB_TILE + row;
        const bool row_ok = qrow < p.lq;
        const float dot = dots[qrow], lse_l = lses[qrow];
        const float* mrow = (p.mask && row_ok) ? p.mask + (long long)bi * p.mask_batch_stride + (long long)qrow * p.lk : nullptr;
        for (int h = 0; h < 2 && ok; h++) {
          ok = mbar_wait(bar_sdp, n_sdp & 1, abort_flag, p.status, 56);
          n_sdp++;
          if (!ok) break;
          tc_fence_after();
          uint32_t rs[32], rd[32];
          tmem_ld_32x32b_x32(lane_base + AB_COL_S + (uint32_t)(hh * 32), rs);
          tmem_ld_32x32b_x32(lane_base + AB_COL_DP + (uint32_t)(hh * 32), rd);
          tmem_ld_wait();
          const int key0 = j * AB_TILE + h * 64 + hh * 32;
          uint32_t pw[16], sw[16];
#pragma unroll
          for (int c = 0; c < 16; c++) {
            float e2[2], d2[2];
#pragma unroll
            for (int u = 0; u < 2; u++) {
              const int jj = 2 * c + u;
              float s = __uint_as_float(rs[jj]) * p.scale;
              if (mrow && key0 + jj < p.lk) s = s + mrow[key0 + jj];
              float e = ab_ex2(fmaf(s, LOG2E, -lse_l));
              if (!row_ok || key0 + jj >= p.lk) e = 0.f;
              e2[u] = e;
              d2[u] = (e * (__uint_as_float(rd[jj]) - dot)) * p.scale;
            }
            pw[c] = ab_pack(e2[0], e2[1]);
            sw[c] = ab_pack(d2[0], d2[1]);
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
          ab_arrive(bar_staged);
        }
      }
      if (!ok) break;
      // dV_j (warps 0-3) and dK_j (warps 4-7): 32 key rows per warp, 64 columns as two blocks.
      ok = mbar_wait(bar_jdone, (uint32_t)j & 1, abort_flag, p.status, 57);
      if (!ok) break;
      tc_fence_after();
      {
        float* dst = hh == 0 ? p.dv : p.dk;
        uint16_t* dst16 = hh == 0 ? p.dv16 : p.dk16;
        const long long base = hh == 0 ? (long long)bi * p.dv_batch + (long long)hi * p.dv_head : (long long)bi * p.dk_batch + (long long)hi * p.dk_head;
        const long long rs_ = hh == 0 ? p.dv_row : p.dk_row;
        if (dst) {
#pragma unroll 1
          for (int cb = 0; cb < 2; cb++) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(lane_base + (hh == 0 ? AB_COL_DV : AB_COL_DK) + (uint32_t)(cb * 32), r);
            tmem_ld_wait();
            ab_store_block(stg, lane, r, dst + base, dst16 ? dst16 + base : nullptr, rs_, j * AB_TILE + quad * 32, p.lk, cb * 32);
          }
        }
      }
      tc_fence_before();
      ab_arrive(bar_epi);
    }
    if (ok && p.dq) {
      // dQ: query tile i, rows of this warp's quadrant, its 32 of the 64 columns.
      const long long base = (long long)bi * p.dq_batch + (long long)hi * p.dq_head;
#pragma unroll 1
      for (int i = 0; i < nq; i++) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_base + AB_COL_DQ + (uint32_t)(i * AB_D + hh * 32), r);
        tmem_ld_wait();
        ab_store_block(stg, lane, r, p.dq + base, p.dq16 ? p.dq16 + base : nullptr, p.dq_row, i * AB_TILE + quad * 32, p.lq, hh * 32);
      }
    }
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
  return (d == AB_D && lq >= 1 && lk >= 1 && lq <= AB_MAX_Q_TILES * AB_TILE && b >= 1 && h >= 1) ? 1 : 0;
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
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_bwd_bf16: head dimension %d (64 is built) or %d queries (at most 512)", d, lq);
  if (!g16 || !g || !q16 || !k16 || !v16 || !out || !lse)
    return fail(ctx, OM_ERR_ARG, "om_attention_bwd_bf16: the gradient (both forms), q, k, v, the forward's output and its log-sum-exp are required");
  if (!operand16_ok(g16, gs, h, b) || !operand16_ok(q16, qs, h, b) || !operand16_ok(k16, ks, h, b) || !operand16_ok(v16, vs, h, b))
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_bwd_bf16: bfloat16 operands need 16-byte aligned bases and strides that are multiples of 8");
  if (!result_ok(dq, dqs) || !result_ok(dk, dks) || !result_ok(dv, dvs) || (gs->row & 1) || (os->row & 1) || (reinterpret_cast<uintptr_t>(g) & 7) ||
      (reinterpret_cast<uintptr_t>(out) & 7) || (gs->head & 1) || (gs->batch & 1) || (os->head & 1) || (os->batch & 1))
    return fail(ctx, OM_ERR_UNSUPPORTED, "om_attention_bwd_bf16: results need 16-byte aligned bases and strides that are multiples of 4");
  if ((dq16 && !dq) || (dk16 && !dk) || (dv16 && !dv)) return fail(ctx, OM_ERR_ARG, "om_attention_bwd_bf16: a bfloat16 copy needs its fp32 result");
  ProfileScope prof(ctx, "om_attention_bwd", 8.0 * b * h * (double)lq * lk * d, 2.0 * b * h * ((double)lq * d * 2 + (double)lk * d * 2) + 4.0 * b * h * ((double)lq * d * 3 + (double)lk * d * 2));
  CUtensorMap mq, mk, mv, mg;
  if (!att16_map(&mq, q16, lq, h, b, qs->row, qs->head, qs->batch) || !att16_map(&mk, k16, lk, h, b, ks->row, ks->head, ks->batch) ||
      !att16_map(&mv, v16, lk, h, b, vs->row, vs->head, vs->batch) || !att16_map(&mg, g16, lq, h, b, gs->row, gs->head, gs->batch))
    return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed for the attention operands");
  AttBwd16Params p;
  p.lq = lq; p.lk = lk; p.heads = h; p.scale = scale; p.mask = mask; p.mask_batch_stride = mask_batch_stride; p.lse = lse;
  p.g = g; p.out = out;
  p.g_batch = gs->batch; p.g_head = gs->head; p.g_row = gs->row; p.o_batch = os->batch; p.o_head = os->head; p.o_row = os->row;
  p.dq = dq; p.dk = dk; p.dv = dv; p.dq16 = dq16; p.dk16 = dk16; p.dv16 = dv16;
  p.dq_batch = dq ? dqs->batch : 0; p.dq_head = dq ? dqs->head : 0; p.dq_row = dq ? dqs->row : 0;
  p.dk_batch = dk ? dks->batch : 0; p.dk_head = dk ? dks->head : 0; p.dk_row = dk ? dks->row : 0;
  p.dv_batch = dv ? dvs->batch : 0; p.dv_head = dv ? dvs->head : 0; p.dv_row = dv ? dvs->row : 0;
  p.status = ctx->status_dev;
  const size_t smem = (size_t)12 * AB_BLOCK + 2 * AB_MAX_Q_TILES * AB_TILE * sizeof(float) + 128 + 1024;
  static bool set = false;
  if (!set) {
    OM_CUDA(ctx, cudaFuncSetAttribute(attention_bwd16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    set = true;
  }
  launch_chained(ctx, attention_bwd16_kernel, dim3((unsigned)(b * h)), AB_THREADS, smem, mq, mk, mv, mg, p);
  OM_LAUNCH_CHECK(ctx, "om_attention_bwd_bf16");
  return OM_OK;
}

}  // extern "C"
