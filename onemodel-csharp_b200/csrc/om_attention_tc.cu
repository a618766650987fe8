// Fused attention on the tensor pipe for sequences that fit one tile (Lq, Lk <= 128): one CTA per (batch, head) keeps the
// score matrix in tensor memory from the first product to the last, so the [B*H, Lq, Lk] scores and probabilities never
// travel through HBM.
//
// Forward (AttentionDriver.Run in the reference, Kernels/AttentionDriver.cs:29; Ops.Attention, Ops.Layers.cs:746-807):
//   S = Q K^T            tcgen05.mma, Q and K tiles K-major, accumulator 128 x 128 in TMEM
//   P = softmax(scale S + mask)   each of 128 threads owns one row (tcgen05.ld gives a thread its whole row), max and
//                                 sum are thread-local (fp32: this kernel only serves the TF32 tier)
//   O = P V              P goes to shared memory in the K-major swizzled operand layout, V is an MN-major tile
// and the row log-sum-exp is kept for the backward.
//
// Every mbarrier wait is bounded (om_tc.cuh): on expiry the kernel raises OM_ERR_TIMEOUT in the status word, all roles
// leave, TMEM is released.
#include "om_tc.cuh"

namespace om {

constexpr int ATT_TILE = 128;                 // queries and keys per CTA
constexpr int ATT_THREADS = 160;              // warps 0-3: one accumulator row per thread; warp 4: TMA + MMA issue
constexpr int ATT_BLOCK_BYTES = ATT_TILE * 128;   // one [128 rows x 128 bytes] operand block: 16 KiB

struct AttFwdParams {
  int lq, lk, d, heads;
  float scale;
  const float* mask;
  long long mask_batch_stride;
  float* out;
  long long o_batch, o_head, o_row;
  float* lse;            // [B*H, lq] or null
  int32_t* status;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// 2^x on the special-function unit, one instruction (inputs here are at most 0, or -inf for masked columns: 2^-inf = 0).
__device__ __forceinline__ float fast_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Instruction descriptor for kind::tf32 with an fp32 accumulator: M = 128, N = n, operand major bits.
__device__ __forceinline__ uint32_t att_idesc(int n, bool a_mn, bool b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(ATT_TILE >> 4) << 24);
}

// Writes one accumulator row (values v[0..127], already TF32) into a K-major operand tile of 4 blocks [128 rows x 128 B]
// with the 128-byte swizzle on 16-byte units: chunk c of row r sits at chunk c ^ (r & 7).
__device__ __forceinline__ void store_row_kmajor(uint8_t* tile, int row, const float* v) {
#pragma unroll
  for (int kb = 0; kb < 4; kb++) {
    uint8_t* base = tile + kb * ATT_BLOCK_BYTES + row * 128;
#pragma unroll
    for (int c = 0; c < 8; c++) {
      const int j = kb * 32 + c * 4;
      *reinterpret_cast<float4*>(base + ((c ^ (row & 7)) << 4)) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
  }
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attention_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, AttFwdParams p) {
  constexpr int DB = D / 32;                            // 128-byte blocks along the head dimension
  constexpr uint32_t TMEM_COLS = 256;                   // S: 128 columns, O: D columns
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  // P (4 blocks, a K-major operand of 128 keys) is written over the Q and K tiles, which are dead once S is complete;
  // the same region stages the output rows at the end. V follows it.
  uint8_t* p_s = smem;
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + DB * ATT_BLOCK_BYTES;
  uint8_t* v_s = smem + 4 * ATT_BLOCK_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + DB * ATT_BLOCK_BYTES);
  uint64_t *bar_load = bars, *bar_s = bars + 1, *bar_p = bars + 2, *bar_o = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, bi = bh / p.heads, hi = bh % p.heads;

  if (threadIdx.x == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, ATT_TILE);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();   // tensor memory is held: later kernels may become resident
  pdl_wait();      // everything below may depend on the previous kernel

  if (warp == 4) {
    if (lane == 0) {
      // ---- loads ----
      mbar_expect_tx(bar_load, 3 * DB * ATT_BLOCK_BYTES);
#pragma unroll
      for (int kb = 0; kb < DB; kb++) {
        tma_load_4d(q_s + kb * ATT_BLOCK_BYTES, &map_q, 32 * kb, 0, hi, bi, bar_load);
        tma_load_4d(k_s + kb * ATT_BLOCK_BYTES, &map_k, 32 * kb, 0, hi, bi, bar_load);
        tma_load_4d(v_s + kb * ATT_BLOCK_BYTES, &map_v, 32 * kb, 0, hi, bi, bar_load);
      }
      bool ok = mbar_wait(bar_load, 0, abort_flag, p.status, 11);
      if (ok) {
        tc_fence_after();
        // ---- S = Q K^T: both operands K-major, k = D ----
        const uint32_t idesc = att_idesc(ATT_TILE, false, false);
        const uint32_t qa = smem_u32(q_s), ka = smem_u32(k_s);
#pragma unroll
        for (int ks = 0; ks < D / 8; ks++) {
          const uint32_t off = (ks / 4) * ATT_BLOCK_BYTES + (ks % 4) * 32;
          umma_tf32(tmem_base, make_desc(qa + off, 16, 1024, 2), make_desc(ka + off, 16, 1024, 2), idesc, ks > 0 ? 1u : 0u);
        }
      }
      umma_commit(bar_s);
      // ---- O = P V: P K-major from shared memory (k = 128 keys), V MN-major (n = D) ----
      if (ok) ok = mbar_wait(bar_p, 0, abort_flag, p.status, 12);
      if (ok) {
        tc_fence_after();
        const uint32_t idesc = att_idesc(D, false, true);
        const uint32_t pa = smem_u32(p_s), va = smem_u32(v_s);
#pragma unroll
        for (int ks = 0; ks < ATT_TILE / 8; ks++) {
          const uint64_t adesc = make_desc(pa + (ks / 4) * ATT_BLOCK_BYTES + (ks % 4) * 32, 16, 1024, 2);
          const uint64_t bdesc = make_desc(va + ks * 1024, ATT_BLOCK_BYTES, 512, 1);
          umma_tf32(tmem_base + ATT_TILE, adesc, bdesc, idesc, ks > 0 ? 1u : 0u);
        }
      }
      umma_commit(bar_o);
    }
  } else {
    // ---- one row per thread ----
    const int row = warp * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    bool ok = mbar_wait(bar_s, 0, abort_flag, p.status, 13);
    tc_fence_after();
    float v[ATT_TILE];
    if (ok) {
#pragma unroll
      for (int c = 0; c < 4; c++) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_base + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j++) v[c * 32 + j] = __uint_as_float(r[j]);
      }
      // scale * s + mask, row maximum, exponentials and their sum; four independent chains keep the pipes busy. The
      // exponential is 2^(x * log2 e) on the special-function unit; the sum runs in fp32 (128 terms).
      const float* mrow = nullptr;
      if (p.mask && row < p.lq) mrow = p.mask + (long long)bi * p.mask_batch_stride + (long long)row * p.lk;
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (mrow == nullptr && p.lk == ATT_TILE) {
#pragma unroll
        for (int j = 0; j < ATT_TILE; j++) {
          v[j] = v[j] * p.scale;
          m4[j & 3] = fmaxf(m4[j & 3], v[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < ATT_TILE; j++) {
          float s = -INFINITY;
          if (j < p.lk) s = (v[j] * p.scale) + (mrow ? mrow[j] : 0.f);
          v[j] = s;
          m4[j & 3] = fmaxf(m4[j & 3], s);
        }
      }
      const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      const float mxl = mx * 1.4426950408889634f;
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < ATT_TILE; j++) {
        float e = exp2f(fmaf(v[j], 1.4426950408889634f, -mxl));     // exp(-inf) = 0 for the columns past lk
        v[j] = e;
        s4[j & 3] += e;
      }
      const float fs = (s4[0] + s4[1]) + (s4[2] + s4[3]);
      const float inv = 1.0f / fs;
#pragma unroll
      for (int j = 0; j < ATT_TILE; j++) v[j] = to_tf32(v[j] * inv);
      if (p.lse && row < p.lq) p.lse[(long long)bh * p.lq + row] = mx + logf(fs);
      store_row_kmajor(p_s, row, v);
      fence_async_smem();
    }
    mbar_arrive(bar_p);
    // ---- output ----
    if (ok) ok = mbar_wait(bar_o, 0, abort_flag, p.status, 14);
    tc_fence_after();
    if (ok) {
      constexpr int STG_LD = D + 4;
      float* stg = reinterpret_cast<float*>(p_s) + warp * 32 * STG_LD;   // the PV products have consumed P
      float* outp = p.out + (long long)bi * p.o_batch + (long long)hi * p.o_head;
#pragma unroll
      for (int c = 0; c < DB; c++) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_base + ATT_TILE + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(stg + lane * STG_LD + c * 32 + j) =
              make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      }
      __syncwarp();
      // D / 4 lanes cover one output row (D floats, contiguous in memory); a warp store writes 32 / (D / 4) rows.
      constexpr int LPR = D / 4, RPI = 32 / LPR;
#pragma unroll
      for (int i = 0; i < 32 / RPI; i++) {
        const int rr = i * RPI + lane / LPR;
        const int orow = warp * 32 + rr;
        if (orow < p.lq) {
          const float4 val = *reinterpret_cast<const float4*>(stg + rr * STG_LD + (lane % LPR) * 4);
          *reinterpret_cast<float4*>(outp + (long long)orow * p.o_row + (lane % LPR) * 4) = val;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- backward -------------------------------------------------------------------------------------------------------------
// AttentionBackward of the reference (BackwardNn.cs:636-701) for one (batch, head) per CTA, head dimension 32:
//   S = Q K^T, dP = dO V^T                      (K-major tiles, accumulators in TMEM columns 0-127 and 128-255)
//   P = exp(scale S + mask - lse)               (lse saved by the forward), dot = rowsum(P dP), dS = P (dP - dot) scale
//   dV = P^T dO, dQ = dS K, dK = dS^T Q         (P and dS go to shared memory as MN-major / K-major operands; the second
//                                                operands are MN-major tiles fetched again by TMA over the dead K-major ones)
// Rows are split over two threads (columns 0-63 and 64-127) so that eight warps share the exponentials.
constexpr int ATT_BWD_THREADS = 288;          // warps 0-7: half an accumulator row per thread; warp 8: TMA + MMA issue

struct AttBwdParams {
  int lq, lk, heads;
  float scale;
  const float* mask;
  long long mask_batch_stride;
  const float* lse;
  float *dq, *dk, *dv;
  long long dq_batch, dq_head, dq_row, dk_batch, dk_head, dk_row, dv_batch, dv_head, dv_row;
  int32_t* status;
};

// 32 consecutive floats (one 128-byte row segment) of a K-major operand block: chunk c of row r sits at c ^ (r & 7).
__device__ __forceinline__ void store_seg_kmajor(uint8_t* block, int row, const float* v) {
  uint8_t* base = block + row * 128;
#pragma unroll
  for (int c = 0; c < 8; c++)
    *reinterpret_cast<float4*>(base + ((c ^ (row & 7)) << 4)) = make_float4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
}
// The same 32 floats as row `krow` of an MN-major chunk [128 k-rows x 128 bytes]: 128-byte swizzle on 32-byte units,
// address bits 5-6 ^= bits 7-8 (the k-row's low two bits).
__device__ __forceinline__ void store_seg_mnmajor(uint8_t* chunk, int krow, const float* v) {
  uint8_t* base = chunk + krow * 128;
  const int x = (krow & 3) << 5;
#pragma unroll
  for (int c = 0; c < 8; c++)
    *reinterpret_cast<float4*>(base + ((c << 4) ^ x)) = make_float4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
}

__device__ __forceinline__ void store_rows_32(float* stg, int lane, const uint32_t (&r)[32], float* dst, long long row_stride, int row0,
                                              int rows_valid) {
  // stg: 32 x 36 floats of this warp. Turn the 32 x 32 block so that eight lanes write one 128-byte row.
#pragma unroll
  for (int j = 0; j < 32; j += 4)
    *reinterpret_cast<float4*>(stg + lane * 36 + j) =
        make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int rr = i * 4 + (lane >> 3);
    if (row0 + rr < rows_valid)
      *reinterpret_cast<float4*>(dst + (long long)(row0 + rr) * row_stride + (lane & 7) * 4) =
          *reinterpret_cast<const float4*>(stg + rr * 36 + (lane & 7) * 4);
  }
  __syncwarp();
}

__global__ void __launch_bounds__(ATT_BWD_THREADS, 1)
attention_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_qk, const __grid_constant__ CUtensorMap map_kk,
                        const __grid_constant__ CUtensorMap map_vk, const __grid_constant__ CUtensorMap map_gk,
                        const __grid_constant__ CUtensorMap map_qm, const __grid_constant__ CUtensorMap map_km,
                        const __grid_constant__ CUtensorMap map_gm, AttBwdParams p) {
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DQ = 288, COL_DK = 320;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* slot_q = smem;                               // Q K-major, later Q MN-major
  uint8_t* slot_k = smem + 1 * ATT_BLOCK_BYTES;         // K K-major, later K MN-major
  uint8_t* slot_v = smem + 2 * ATT_BLOCK_BYTES;         // V K-major
  uint8_t* slot_g = smem + 3 * ATT_BLOCK_BYTES;         // dO K-major, later dO MN-major
  uint8_t* stage_a = smem + 4 * ATT_BLOCK_BYTES;        // P^T, later dS^T: MN-major operand, 4 chunks of [128 q-rows x 128 B of keys]
  uint8_t* stage_b = smem + 8 * ATT_BLOCK_BYTES;        // dS: K-major operand, 4 blocks of [128 q-rows x 128 B of keys]; later output staging
  float* dots = reinterpret_cast<float*>(smem + 12 * ATT_BLOCK_BYTES);   // [2][128] partial row dots
  uint64_t* bars = reinterpret_cast<uint64_t*>(dots + 2 * ATT_TILE);
  uint64_t *bar_load = bars, *bar_sdp = bars + 1, *bar_mn = bars + 2, *bar_pt = bars + 3, *bar_dv = bars + 4, *bar_ds = bars + 5,
           *bar_dqk = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, bi = bh / p.heads, hi = bh % p.heads;

  if (threadIdx.x == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_sdp, 1);
    mbar_init(bar_mn, 1);
    mbar_init(bar_pt, 256);
    mbar_init(bar_dv, 1);
    mbar_init(bar_ds, 256);
    mbar_init(bar_dqk, 1);
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
  pdl_trigger();   // tensor memory is held: later kernels may become resident
  pdl_wait();      // everything below may depend on the previous kernel

  if (warp == 8) {
    if (lane == 0) {
      mbar_expect_tx(bar_load, 4 * ATT_BLOCK_BYTES);
      tma_load_4d(slot_q, &map_qk, 0, 0, hi, bi, bar_load);
      tma_load_4d(slot_k, &map_kk, 0, 0, hi, bi, bar_load);
      tma_load_4d(slot_v, &map_vk, 0, 0, hi, bi, bar_load);
      tma_load_4d(slot_g, &map_gk, 0, 0, hi, bi, bar_load);
      bool ok = mbar_wait(bar_load, 0, abort_flag, p.status, 21);
      if (ok) {
        tc_fence_after();
        const uint32_t idesc = att_idesc(ATT_TILE, false, false);
        const uint32_t qa = smem_u32(slot_q), ka = smem_u32(slot_k), va = smem_u32(slot_v), ga = smem_u32(slot_g);
#pragma unroll
        for (int ks = 0; ks < 4; ks++)      // S = Q K^T
          umma_tf32(tmem_base + COL_S, make_desc(qa + ks * 32, 16, 1024, 2), make_desc(ka + ks * 32, 16, 1024, 2), idesc, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 4; ks++)      // dP = dO V^T
          umma_tf32(tmem_base + COL_DP, make_desc(ga + ks * 32, 16, 1024, 2), make_desc(va + ks * 32, 16, 1024, 2), idesc, ks > 0 ? 1u : 0u);
      }
      umma_commit(bar_sdp);
      // The K-major tiles are dead once both products are complete: fetch the MN-major forms over them.
      if (ok) ok = mbar_wait(bar_sdp, 0, abort_flag, p.status, 22);
      if (ok) {
        mbar_expect_tx(bar_mn, 3 * ATT_BLOCK_BYTES);
        tma_load_4d(slot_q, &map_qm, 0, 0, hi, bi, bar_mn);
        tma_load_4d(slot_k, &map_km, 0, 0, hi, bi, bar_mn);
        tma_load_4d(slot_g, &map_gm, 0, 0, hi, bi, bar_mn);
        ok = mbar_wait(bar_mn, 0, abort_flag, p.status, 23);
      }
      if (ok) ok = mbar_wait(bar_pt, 0, abort_flag, p.status, 24);
      if (ok) {
        tc_fence_after();
        // dV = P^T dO: A = P^T MN-major (m = keys, k = queries), B = dO MN-major (n = 32)
        const uint32_t idesc = att_idesc(32, true, true);
        const uint32_t aa = smem_u32(stage_a), ga = smem_u32(slot_g);
#pragma unroll
        for (int ks = 0; ks < ATT_TILE / 8; ks++)
          umma_tf32(tmem_base + COL_DV, make_desc(aa + ks * 1024, ATT_BLOCK_BYTES, 512, 1), make_desc(ga + ks * 1024, ATT_BLOCK_BYTES, 512, 1),
                    idesc, ks > 0 ? 1u : 0u);
      }
      umma_commit(bar_dv);
      if (ok) ok = mbar_wait(bar_ds, 0, abort_flag, p.status, 25);
      if (ok) {
        tc_fence_after();
        const uint32_t aa = smem_u32(stage_a), ba = smem_u32(stage_b), qa = smem_u32(slot_q), ka = smem_u32(slot_k);
        // dQ = dS K: A = dS K-major (k = keys), B = K MN-major
        const uint32_t idesc_q = att_idesc(32, false, true);
#pragma unroll
        for (int ks = 0; ks < ATT_TILE / 8; ks++)
          umma_tf32(tmem_base + COL_DQ, make_desc(ba + (ks / 4) * ATT_BLOCK_BYTES + (ks % 4) * 32, 16, 1024, 2),
                    make_desc(ka + ks * 1024, ATT_BLOCK_BYTES, 512, 1), idesc_q, ks > 0 ? 1u : 0u);
        // dK = dS^T Q: A = dS^T MN-major (m = keys, k = queries), B = Q MN-major
        const uint32_t idesc_k = att_idesc(32, true, true);
#pragma unroll
        for (int ks = 0; ks < ATT_TILE / 8; ks++)
          umma_tf32(tmem_base + COL_DK, make_desc(aa + ks * 1024, ATT_BLOCK_BYTES, 512, 1), make_desc(qa + ks * 1024, ATT_BLOCK_BYTES, 512, 1),
                    idesc_k, ks > 0 ? 1u : 0u);
      }
      umma_commit(bar_dqk);
    }
  } else {
    // ---- half a row per thread: row = 32 * (warp % 4) + lane, columns 64 * (warp / 4) .. + 63 ----
    const int quad = warp & 3, half = warp >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    bool ok = mbar_wait(bar_sdp, 0, abort_flag, p.status, 26);
    tc_fence_after();
    float pv[64], dp[64];
    float dot = 0.f;
    if (ok) {
      const float lse_l = (row < p.lq ? p.lse[(long long)bh * p.lq + row] : 0.f) * LOG2E;
      const float* mrow = nullptr;
      if (p.mask && row < p.lq) mrow = p.mask + (long long)bi * p.mask_batch_stride + (long long)row * p.lk;
      float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 2; c++) {
        const int col0 = half * 64 + c * 32;
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(lane_base + COL_S + col0, rs);
        tmem_ld_32x32b_x32(lane_base + COL_DP + col0, rd);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j++) {
          float s = __uint_as_float(rs[j]) * p.scale;
          if (mrow && col0 + j < p.lk) s = s + mrow[col0 + j];
          float e = exp2f(fmaf(s, LOG2E, -lse_l));
          if (col0 + j >= p.lk) e = 0.f;
          const float d = __uint_as_float(rd[j]);
          pv[c * 32 + j] = e;
          dp[c * 32 + j] = d;
          d4[j & 3] = fmaf(e, d, d4[j & 3]);
        }
      }
      dots[half * ATT_TILE + row] = (d4[0] + d4[1]) + (d4[2] + d4[3]);
      // P^T for dV: this thread's 64 keys of query `row` are two 128-byte segments of k-row `row` in chunks 2*half, 2*half+1.
#pragma unroll
      for (int c = 0; c < 2; c++) {
        float t[32];
#pragma unroll
        for (int j = 0; j < 32; j++) t[j] = to_tf32(pv[c * 32 + j]);
        store_seg_mnmajor(stage_a + (half * 2 + c) * ATT_BLOCK_BYTES, row, t);
      }
      fence_async_smem();
    }
    mbar_arrive(bar_pt);
    asm volatile("bar.sync 1, 256;" ::: "memory");      // both halves of every row have published their partial dots
    if (ok) {
      dot = dots[row] + dots[ATT_TILE + row];
#pragma unroll
      for (int j = 0; j < 64; j++) pv[j] = to_tf32((pv[j] * (dp[j] - dot)) * p.scale);   // dS in place
#pragma unroll
      for (int c = 0; c < 2; c++) store_seg_kmajor(stage_b + (half * 2 + c) * ATT_BLOCK_BYTES, row, pv + c * 32);
      // dS^T goes where P^T was: wait until the dV product has read it.
      ok = mbar_wait(bar_dv, 0, abort_flag, p.status, 27);
    }
    if (ok) {
#pragma unroll
      for (int c = 0; c < 2; c++) store_seg_mnmajor(stage_a + (half * 2 + c) * ATT_BLOCK_BYTES, row, pv + c * 32);
      fence_async_smem();
    }
    mbar_arrive(bar_ds);
    if (ok) ok = mbar_wait(bar_dqk, 0, abort_flag, p.status, 28);
    tc_fence_after();
    if (ok) {
      // Warps 0-3 write dQ and dV, warps 4-7 write dK; each warp owns the 32 rows of its TMEM lane quadrant.
      float* stg = reinterpret_cast<float*>(stage_b) + warp * 32 * 36;   // the dQ product has consumed dS
      uint32_t r[32];
      if (half == 0) {
        if (p.dq) {
          tmem_ld_32x32b_x32(lane_base + COL_DQ, r);
          tmem_ld_wait();
          store_rows_32(stg, lane, r, p.dq + (long long)bi * p.dq_batch + (long long)hi * p.dq_head, p.dq_row, quad * 32, p.lq);
        }
        if (p.dv) {
          tmem_ld_32x32b_x32(lane_base + COL_DV, r);
          tmem_ld_wait();
          store_rows_32(stg, lane, r, p.dv + (long long)bi * p.dv_batch + (long long)hi * p.dv_head, p.dv_row, quad * 32, p.lk);
        }
      } else if (p.dk) {
        tmem_ld_32x32b_x32(lane_base + COL_DK, r);
        tmem_ld_wait();
        store_rows_32(stg, lane, r, p.dk + (long long)bi * p.dk_batch + (long long)hi * p.dk_head, p.dk_row, quad * 32, p.lk);
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

// ---- forward, sequences of several tiles ---------------------------------------------------------------------------------
// One CTA per (128 queries, batch, head) walks the key tiles twice. Pass 1 forms S_j = Q K_j^T for every key tile and keeps,
// per row, the running maximum and the sum of exponentials (online softmax statistics: no output yet). Pass 2 forms S_j
// again, turns it into the final probabilities P_j = exp(s - max) / sum with the statistics of pass 1, stages P_j as the
// K-major operand and accumulates O += P_j V_j in tensor memory: nothing is ever rescaled. The second Q K^T costs tensor
// pipe time that the kernel does not lack (its pace is set by the exponentials). S is double-buffered in tensor memory
// and K in shared memory, so the product of the next tile and its load run under the current tile's row pass.
// The row warps' waits are made warp-uniform (__all_sync): a warp leaves its loop together, so its __syncwarp points hold even
// when a wait ran out. Steps g = 0 .. 2 nk - 1 number the (pass, tile) pairs; S buffer and K buffer of step g are g & 1. A score row is
// shared by four threads (32 columns of the tile each): each keeps its own running maximum and sum through pass 1 and the
// four are combined once, in a fixed order, before pass 2.
constexpr int ATT_MT_PARTS = 4;              // threads per score row: each owns 32 of the tile's 128 columns
constexpr int ATT_MT_ISSUE_WARP = 4 * ATT_MT_PARTS;
constexpr int ATT_MT_THREADS = 32 * (ATT_MT_ISSUE_WARP + 1);   // 16 row warps (enough of them to hide each other's latencies) + TMA / MMA issue

template <int D>
__global__ void __launch_bounds__(ATT_MT_THREADS, 1)
attention_fwd_mt_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, AttFwdParams p) {
  constexpr int DB = D / 32;
  constexpr uint32_t TMEM_COLS = 512;                   // S0: 0-127, S1: 128-255, O: 256 .. 256 + D
  constexpr uint32_t COL_O = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;                                   // DB blocks
  uint8_t* k_s[2] = {q_s + DB * ATT_BLOCK_BYTES, q_s + 2 * DB * ATT_BLOCK_BYTES};
  uint8_t* v_s[2] = {q_s + 3 * DB * ATT_BLOCK_BYTES, q_s + 4 * DB * ATT_BLOCK_BYTES};   // DB blocks each (MN-major)
  uint8_t* p_s = q_s + 5 * DB * ATT_BLOCK_BYTES;         // 4 blocks; the output staging at the end
  float* stats = reinterpret_cast<float*>(p_s);          // [parts][128 rows][max, sum]: used once, before the first P is staged
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 4 * ATT_BLOCK_BYTES);
  uint64_t* bar_q = bars;
  uint64_t* bar_k = bars + 1;       // [2] K tile landed
  uint64_t* bar_v = bars + 3;       // [2] V tile landed
  uint64_t* bar_s = bars + 5;       // [2] S product complete (and its K buffer free)
  uint64_t* bar_sr = bars + 7;      // [2] S buffer read by all rows
  uint64_t* bar_p = bars + 9;       // P staged by all rows
  uint64_t* bar_pv = bars + 10;     // P V product complete (P buffer and that tile's V buffer free)
  uint64_t* bar_x = bars + 11;      // all parts of every row have published their pass-1 statistics
  uint64_t* bar_x2 = bars + 12;     // ... and have read them: the statistics share their memory with the first P
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * ATT_TILE;
  const int bh = blockIdx.y, bi = bh / p.heads, hi = bh % p.heads;
  const int nk = (p.lk + ATT_TILE - 1) / ATT_TILE, steps = 2 * nk;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int i = 0; i < 2; i++) {
      mbar_init(&bar_k[i], 1);
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_sr[i], ATT_MT_ISSUE_WARP);   // one arrival per row warp
    }
    mbar_init(&bar_v[0], 1);
    mbar_init(&bar_v[1], 1);
    mbar_init(bar_p, ATT_MT_ISSUE_WARP);
    mbar_init(bar_pv, 1);
    mbar_init(bar_x, ATT_MT_PARTS * ATT_TILE);
    mbar_init(bar_x2, ATT_MT_PARTS * ATT_TILE);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == ATT_MT_ISSUE_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  pdl_wait();

  if (warp == ATT_MT_ISSUE_WARP) {
    if (lane == 0) {
      const uint32_t idesc_s = att_idesc(ATT_TILE, false, false), idesc_o = att_idesc(D, false, true);
      const uint32_t qa = smem_u32(q_s), pa = smem_u32(p_s);
      auto load_v = [&](int t) {          // value tile t into buffer t & 1
        mbar_expect_tx(&bar_v[t & 1], DB * ATT_BLOCK_BYTES);
        for (int kb = 0; kb < DB; kb++) tma_load_4d(v_s[t & 1] + kb * ATT_BLOCK_BYTES, &map_v, 32 * kb, t * ATT_TILE, hi, bi, &bar_v[t & 1]);
      };
      auto load_k = [&](int g) {          // key tile of step g into its buffer
        const int i = g & 1, j = g % nk;
        mbar_expect_tx(&bar_k[i], DB * ATT_BLOCK_BYTES);
        for (int kb = 0; kb < DB; kb++) tma_load_4d(k_s[i] + kb * ATT_BLOCK_BYTES, &map_k, 32 * kb, j * ATT_TILE, hi, bi, &bar_k[i]);
      };
      auto issue_s = [&](int g) {         // S[g & 1] = Q K^T for the key tile in buffer g & 1
        const int i = g & 1;
        const uint32_t ka = smem_u32(k_s[i]);
#pragma unroll
        for (int ks = 0; ks < D / 8; ks++) {
          const uint32_t off = (ks / 4) * ATT_BLOCK_BYTES + (ks % 4) * 32;
          umma_tf32(tmem_base + (uint32_t)(i * ATT_TILE), make_desc(qa + off, 16, 1024, 2), make_desc(ka + off, 16, 1024, 2), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(&bar_s[i]);
      };
      mbar_expect_tx(bar_q, DB * ATT_BLOCK_BYTES);
      for (int kb = 0; kb < DB; kb++) tma_load_4d(q_s + kb * ATT_BLOCK_BYTES, &map_q, 32 * kb, q0, hi, bi, bar_q);
      load_k(0);
      if (steps > 1) load_k(1);
      load_v(0);                          // both value buffers are free: the first two tiles come in during pass 1
      if (nk > 1) load_v(1);
      bool ok = mbar_wait(bar_q, 0, abort_flag, p.status, 41);
      if (ok) ok = mbar_wait(&bar_k[0], 0, abort_flag, p.status, 42);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int g = 0; g < steps && ok; g++) {
        const int i = g & 1;
        // 1. the product of the next step, as soon as its key tile has landed and its S buffer has been read (step g - 1)
        if (g + 1 < steps) {
          const int n = (g + 1) & 1;
          ok = mbar_wait(&bar_k[n], (uint32_t)((g + 1) >> 1) & 1, abort_flag, p.status, 43);
          if (ok && g >= 1) ok = mbar_wait(&bar_sr[n], (uint32_t)(((g + 1) >> 1) - 1) & 1, abort_flag, p.status, 44);
          if (!ok) break;
          tc_fence_after();
          issue_s(g + 1);
        }
        // 2. the key tile of step g + 2 into this step's buffer, once this step's product has read it
        if (g + 2 < steps) {
          ok = mbar_wait(&bar_s[i], (uint32_t)(g >> 1) & 1, abort_flag, p.status, 45);
          if (!ok) break;
          load_k(g + 2);
        }
        // 3. second pass: O += P V
        if (g >= nk) {
          const int t = g - nk;
          if (t >= 1) {
            // P V of tile t - 1 is complete: its value buffer takes tile t + 1 while this tile's row pass runs
            ok = mbar_wait(bar_pv, (uint32_t)(t - 1) & 1, abort_flag, p.status, 46);
            if (!ok) break;
            if (t + 1 < nk) load_v(t + 1);
          }
          ok = mbar_wait(&bar_v[t & 1], (uint32_t)(t >> 1) & 1, abort_flag, p.status, 47);
          if (ok) ok = mbar_wait(bar_p, (uint32_t)t & 1, abort_flag, p.status, 48);
          if (!ok) break;
          tc_fence_after();
          const uint32_t va = smem_u32(v_s[t & 1]);
#pragma unroll
          for (int ks = 0; ks < ATT_TILE / 8; ks++) {
            const uint64_t adesc = make_desc(pa + (ks / 4) * ATT_BLOCK_BYTES + (ks % 4) * 32, 16, 1024, 2);
            const uint64_t bdesc = make_desc(va + ks * 1024, ATT_BLOCK_BYTES, 512, 1);
            umma_tf32(tmem_base + COL_O, adesc, bdesc, idesc_o, (t > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(bar_pv);
        }
      }
    }
  } else {
    // ---- a quarter of a score row per thread: row = 32 * (warp % 4) + lane, columns 32 * (warp / 4) .. + 31 of each tile ----
    const int quad = warp & 3, part = warp >> 2;
    const int row = quad * 32 + lane, qrow = q0 + row;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    const float sl2 = p.scale * LOG2E;
    const float* mrow = nullptr;
    if (p.mask && qrow < p.lq) mrow = p.mask + (long long)bi * p.mask_batch_stride + (long long)qrow * p.lk;
    float run_max = -INFINITY, run_sum = 0.f, inv_sum = 0.f, max_l2 = 0.f;
    bool ok = true;
    float v[32];
    for (int g = 0; g < steps && ok; g++) {
      const int i = g & 1, j = g % nk, col0 = j * ATT_TILE + part * 32;
      ok = __all_sync(0xffffffffu, mbar_wait(&bar_s[i], (uint32_t)(g >> 1) & 1, abort_flag, p.status, 49));
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_base + (uint32_t)(i * ATT_TILE + part * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < 32; jj++) v[jj] = __uint_as_float(r[jj]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_sr[i]);       // the next product may overwrite this S buffer (one arrival per warp:
                                                    // hundreds of arrivals on one barrier word would serialise)
      // Scores in the base-2 domain from here on: t = (scale s + mask) log2 e, so that an exponential is one ex2.
      const bool full = mrow == nullptr && col0 + 32 <= p.lk;
      if (full) {
#pragma unroll
        for (int jj = 0; jj < 32; jj++) v[jj] = v[jj] * sl2;
      } else {
#pragma unroll
        for (int jj = 0; jj < 32; jj++) {
          float sv = -INFINITY;
          if (col0 + jj < p.lk) sv = fmaf(v[jj], sl2, mrow ? mrow[col0 + jj] * LOG2E : 0.f);
          v[jj] = sv;
        }
      }
      if (g < nk) {
        // pass 1: running maximum and sum of exponentials of this thread's columns
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int jj = 0; jj < 32; jj++) m4[jj & 3] = fmaxf(m4[jj & 3], v[jj]);
        const float tile_max = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        const float new_max = fmaxf(run_max, tile_max);
        if (new_max > -INFINITY) {
          float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int jj = 0; jj < 32; jj++) s4[jj & 3] += fast_ex2(v[jj] - new_max);
          const float carry = run_max > -INFINITY ? run_sum * fast_ex2(run_max - new_max) : 0.f;
          run_sum = carry + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
          run_max = new_max;
        }
        if (g == nk - 1) {
          // the threads of a row exchange their statistics once and combine them in the order of the column ranges, so that
          // all of them hold the same bits
          stats[(part * ATT_TILE + row) * 2] = run_max;
          stats[(part * ATT_TILE + row) * 2 + 1] = run_sum;
          mbar_arrive(bar_x);                       // a bounded wait, not a named barrier: a thread that gave up never arrives
          ok = __all_sync(0xffffffffu, mbar_wait(bar_x, 0, abort_flag, p.status, 52));
          if (!ok) break;
          float mx = -INFINITY;
#pragma unroll
          for (int q = 0; q < ATT_MT_PARTS; q++) mx = fmaxf(mx, stats[(q * ATT_TILE + row) * 2]);
          float total = 0.f;
#pragma unroll
          for (int q = 0; q < ATT_MT_PARTS; q++) {
            const float mq = stats[(q * ATT_TILE + row) * 2], sq = stats[(q * ATT_TILE + row) * 2 + 1];
            total += mq > -INFINITY ? sq * fast_ex2(mq - mx) : 0.f;
          }
          mbar_arrive(bar_x2);
          inv_sum = 1.0f / total;
          max_l2 = mx;
          if (part == 0 && p.lse && qrow < p.lq) p.lse[(long long)bh * p.lq + qrow] = mx * 0.6931471805599453f + logf(total);
        }
      } else {
        // pass 2: the final probabilities of this thread's columns, staged as the K-major operand of P V
        const int t = g - nk;
#pragma unroll
        for (int jj = 0; jj < 32; jj++) v[jj] = to_tf32(fast_ex2(v[jj] - max_l2) * inv_sum);
        if (t >= 1) ok = __all_sync(0xffffffffu, mbar_wait(bar_pv, (uint32_t)(t - 1) & 1, abort_flag, p.status, 50));   // the previous P has been consumed
        else ok = __all_sync(0xffffffffu, mbar_wait(bar_x2, 0, abort_flag, p.status, 53));                               // everyone has read the statistics
        if (ok) {
          store_seg_kmajor(p_s + part * ATT_BLOCK_BYTES, row, v);
          fence_async_smem();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p);
      }
    }
    // ---- output: warps 0-3 write columns 0-31, warps 4-7 columns 32-63 (D = 64) ----
    if (ok) ok = mbar_wait(bar_pv, (uint32_t)(nk - 1) & 1, abort_flag, p.status, 51);
    tc_fence_after();
    if (ok && part < DB) {
      float* stg = reinterpret_cast<float*>(p_s) + warp * 32 * 36;          // the last P V product has consumed P
      float* outp = p.out + (long long)bi * p.o_batch + (long long)hi * p.o_head + part * 32;
      uint32_t r[32];
      tmem_ld_32x32b_x32(lane_base + COL_O + part * 32, r);
      tmem_ld_wait();
      store_rows_32(stg, lane, r, outp, p.o_row, q0 + quad * 32, p.lq);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == ATT_MT_ISSUE_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- backward, sequences of several tiles: the probabilities and the score gradients --------------------------------------
// The first half of AttentionBackward (BackwardNn.cs:636-701) as one kernel per 128 queries: S = Q K_j^T and dP = dO V_j^T in
// tensor memory for every key tile j, P = exp(scale S + mask - lse) with the forward's log-sum-exp, dS = P (dP - dot) scale,
// both written to the [B*H, Lq, Lk] matrices that the three output products (dV = P^T dO, dQ = dS K, dK = dS^T Q) read. It
// replaces two products and two passes over those matrices. dot = rowsum(P dP) needs the whole row: when the forward's
// output O is at hand it is rowsum(dO O) (the same number, O = P V), taken from the two rows before the first tile and the
// key tiles are walked once (ONE_PASS); without O a first pass over the key tiles accumulates it and a second pass forms
// the products again. S and dP are double-buffered in tensor memory (the products of the next tile run under this tile's row
// pass); each thread owns a quarter of a score row of the tile, and a warp turns its 32 x 32 block through shared memory so
// that the stores to P and dS are whole 128-byte row segments.
struct AttFrontParams {
  int lq, lk, heads, d;
  float scale;
  const float* mask;
  long long mask_batch_stride;
  const float* lse;      // [B*H, lq]
  const float* g;        // dO and O as strided [B, H, L, D] views (ONE_PASS)
  const float* o;
  long long g_batch, g_head, g_row, o_batch, o_head, o_row;
  float* p_out;          // [B*H, lq, lk]
  float* ds_out;         // [B*H, lq, lk]
  int32_t* status;
};

constexpr int ATT_STG_LD = 36;          // floats per staged row of 32: 16-byte aligned, rows spread over the banks

// Writes a warp's 32 x 32 block (lane l holds row l in v[0..31]) to dst rows row0 + l, columns col0 .. col0 + 31.
__device__ __forceinline__ void store_block_32(float* stg, int lane, const float* v, float* dst, long long ld, int row0, int rows_valid, int col0,
                                               int cols_valid, bool vec_ok) {
#pragma unroll
  for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(stg + lane * ATT_STG_LD + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
  __syncwarp();
  if (vec_ok && col0 + 32 <= cols_valid) {
    const int c4 = (lane & 7) * 4;
#pragma unroll
    for (int it = 0; it < 8; it++) {
      const int r = it * 4 + (lane >> 3);
      if (row0 + r < rows_valid)
        *reinterpret_cast<float4*>(dst + (long long)(row0 + r) * ld + col0 + c4) = *reinterpret_cast<const float4*>(stg + r * ATT_STG_LD + c4);
    }
  } else {
    for (int r = 0; r < 32; r++) {
      if (row0 + r >= rows_valid) break;
      if (col0 + lane < cols_valid) dst[(long long)(row0 + r) * ld + col0 + lane] = stg[r * ATT_STG_LD + lane];
    }
  }
  __syncwarp();
}

template <int D, bool ONE_PASS>
__global__ void __launch_bounds__(ATT_MT_THREADS, 1)
attention_bwd_front_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_g,
                           const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, AttFrontParams p) {
  constexpr int DB = D / 32;
  constexpr uint32_t TMEM_COLS = 512;                   // S0: 0, S1: 128, dP0: 256, dP1: 384
  constexpr uint32_t COL_DP = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;
  uint8_t* g_s = q_s + DB * ATT_BLOCK_BYTES;
  uint8_t* k_s = q_s + 2 * DB * ATT_BLOCK_BYTES;
  uint8_t* v_s = q_s + 3 * DB * ATT_BLOCK_BYTES;
  float* stage = reinterpret_cast<float*>(q_s + 4 * DB * ATT_BLOCK_BYTES);       // [row warps][32][ATT_STG_LD]
  float* stats = stage + ATT_MT_ISSUE_WARP * 32 * ATT_STG_LD;                     // [parts][128 rows] partial dots
  uint64_t* bars = reinterpret_cast<uint64_t*>(stats + ATT_MT_PARTS * ATT_TILE);
  uint64_t* bar_qg = bars;          // Q and dO landed
  uint64_t* bar_kv = bars + 1;      // K and V tile landed
  uint64_t* bar_s = bars + 2;       // [2] both products complete (and the K, V buffer free)
  uint64_t* bar_sr = bars + 4;      // [2] S and dP buffers read by all rows
  uint64_t* bar_x = bars + 6;       // both halves of every row have published their partial dot
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * ATT_TILE;
  const int bh = blockIdx.y, bi = bh / p.heads, hi = bh % p.heads;
  const int nk = (p.lk + ATT_TILE - 1) / ATT_TILE, steps = ONE_PASS ? nk : 2 * nk;

  if (threadIdx.x == 0) {
    mbar_init(bar_qg, 1);
    mbar_init(bar_kv, 1);
    for (int i = 0; i < 2; i++) {
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_sr[i], ATT_MT_ISSUE_WARP);   // one arrival per row warp
    }
    mbar_init(bar_x, ATT_MT_PARTS * ATT_TILE);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == ATT_MT_ISSUE_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  pdl_wait();

  if (warp == ATT_MT_ISSUE_WARP) {
    if (lane == 0) {
      const uint32_t idesc = att_idesc(ATT_TILE, false, false);
      const uint32_t qa = smem_u32(q_s), ga = smem_u32(g_s), ka = smem_u32(k_s), va = smem_u32(v_s);
      auto load_kv = [&](int g) {
        const int j = g % nk;
        mbar_expect_tx(bar_kv, 2 * DB * ATT_BLOCK_BYTES);
        for (int kb = 0; kb < DB; kb++) {
          tma_load_4d(k_s + kb * ATT_BLOCK_BYTES, &map_k, 32 * kb, j * ATT_TILE, hi, bi, bar_kv);
          tma_load_4d(v_s + kb * ATT_BLOCK_BYTES, &map_v, 32 * kb, j * ATT_TILE, hi, bi, bar_kv);
        }
      };
      auto issue = [&](int g) {           // S[g & 1] = Q K^T, dP[g & 1] = dO V^T
        const int i = g & 1;
#pragma unroll
        for (int ks = 0; ks < D / 8; ks++) {
          const uint32_t off = (ks / 4) * ATT_BLOCK_BYTES + (ks % 4) * 32;
          umma_tf32(tmem_base + (uint32_t)(i * ATT_TILE), make_desc(qa + off, 16, 1024, 2), make_desc(ka + off, 16, 1024, 2), idesc, ks > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < D / 8; ks++) {
          const uint32_t off = (ks / 4) * ATT_BLOCK_BYTES + (ks % 4) * 32;
          umma_tf32(tmem_base + COL_DP + (uint32_t)(i * ATT_TILE), make_desc(ga + off, 16, 1024, 2), make_desc(va + off, 16, 1024, 2), idesc,
                    ks > 0 ? 1u : 0u);
        }
        umma_commit(&bar_s[i]);
      };
      mbar_expect_tx(bar_qg, 2 * DB * ATT_BLOCK_BYTES);
      for (int kb = 0; kb < DB; kb++) {
        tma_load_4d(q_s + kb * ATT_BLOCK_BYTES, &map_q, 32 * kb, q0, hi, bi, bar_qg);
        tma_load_4d(g_s + kb * ATT_BLOCK_BYTES, &map_g, 32 * kb, q0, hi, bi, bar_qg);
      }
      load_kv(0);
      bool ok = mbar_wait(bar_qg, 0, abort_flag, p.status, 61);
      if (ok) ok = mbar_wait(bar_kv, 0, abort_flag, p.status, 62);
      if (ok) {
        tc_fence_after();
        issue(0);
      }
      for (int g = 0; g + 1 < steps && ok; g++) {
        // The single K, V buffer is free once this step's products have read it; the next tile's load and products then run
        // under this step's row pass.
        ok = mbar_wait(&bar_s[g & 1], (uint32_t)(g >> 1) & 1, abort_flag, p.status, 63);
        if (!ok) break;
        load_kv(g + 1);
        ok = mbar_wait(bar_kv, (uint32_t)(g + 1) & 1, abort_flag, p.status, 64);
        if (ok && g >= 1) ok = mbar_wait(&bar_sr[(g + 1) & 1], (uint32_t)(((g + 1) >> 1) - 1) & 1, abort_flag, p.status, 65);
        if (!ok) break;
        tc_fence_after();
        issue(g + 1);
      }
    }
  } else {
    const int quad = warp & 3, part = warp >> 2;
    const int row = quad * 32 + lane, qrow = q0 + row;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    const float sl2 = p.scale * LOG2E;
    const float* mrow = nullptr;
    if (p.mask && qrow < p.lq) mrow = p.mask + (long long)bi * p.mask_batch_stride + (long long)qrow * p.lk;
    const float lse_l = (qrow < p.lq ? p.lse[(long long)bh * p.lq + qrow] : 0.f) * LOG2E;
    const bool vec_ok = (p.lk & 3) == 0 && ((reinterpret_cast<uintptr_t>(p.p_out) | reinterpret_cast<uintptr_t>(p.ds_out)) & 15) == 0;
    float* stg = stage + warp * 32 * ATT_STG_LD;
    float* p_mat = p.p_out + (long long)bh * p.lq * p.lk;
    float* ds_mat = p.ds_out + (long long)bh * p.lq * p.lk;
    float dot = 0.f;
    float d4[4] = {0.f, 0.f, 0.f, 0.f};
    bool ok = true;
    auto combine = [&](float mine) -> bool {      // the row's parts added in the order of their column (or head-dimension) ranges
      stats[part * ATT_TILE + row] = mine;
      mbar_arrive(bar_x);
      if (!__all_sync(0xffffffffu, mbar_wait(bar_x, 0, abort_flag, p.status, 67))) return false;
      float t = stats[row];
#pragma unroll
      for (int q = 1; q < ATT_MT_PARTS; q++) t += stats[q * ATT_TILE + row];
      dot = t;
      return true;
    };
    if (ONE_PASS) {
      // dot = rowsum(dO O): this thread's quarter of the head dimension
      constexpr int DW = D / ATT_MT_PARTS;
      float mine = 0.f;
      if (qrow < p.lq) {
        const float* gr = p.g + (long long)bi * p.g_batch + (long long)hi * p.g_head + (long long)qrow * p.g_row + part * DW;
        const float* orow = p.o + (long long)bi * p.o_batch + (long long)hi * p.o_head + (long long)qrow * p.o_row + part * DW;
#pragma unroll
        for (int j = 0; j < DW; j += 4) {
          const float4 a = *reinterpret_cast<const float4*>(gr + j), b = *reinterpret_cast<const float4*>(orow + j);
          d4[0] = fmaf(a.x, b.x, d4[0]); d4[1] = fmaf(a.y, b.y, d4[1]); d4[2] = fmaf(a.z, b.z, d4[2]); d4[3] = fmaf(a.w, b.w, d4[3]);
        }
        mine = (d4[0] + d4[1]) + (d4[2] + d4[3]);
      }
      ok = combine(mine);
    }
    float pv[32], dp[32];
    for (int g = 0; g < steps && ok; g++) {
      const int i = g & 1, j = g % nk, col0 = j * ATT_TILE + part * 32;
      ok = __all_sync(0xffffffffu, mbar_wait(&bar_s[i], (uint32_t)(g >> 1) & 1, abort_flag, p.status, 66));
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(lane_base + (uint32_t)(i * ATT_TILE + part * 32), rs);
        tmem_ld_32x32b_x32(lane_base + COL_DP + (uint32_t)(i * ATT_TILE + part * 32), rd);
        tmem_ld_wait();
        if (mrow == nullptr && col0 + 32 <= p.lk) {
#pragma unroll
          for (int jj = 0; jj < 32; jj++) {
            pv[jj] = fast_ex2(fmaf(__uint_as_float(rs[jj]), sl2, -lse_l));
            dp[jj] = __uint_as_float(rd[jj]);
          }
        } else {
#pragma unroll
          for (int jj = 0; jj < 32; jj++) {
            const int col = col0 + jj;
            float e = 0.f;
            if (col < p.lk) e = fast_ex2(fmaf(__uint_as_float(rs[jj]), sl2, (mrow ? mrow[col] * LOG2E : 0.f) - lse_l));
            pv[jj] = e;
            dp[jj] = __uint_as_float(rd[jj]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_sr[i]);
      if (!ONE_PASS && g < nk) {
#pragma unroll
        for (int jj = 0; jj < 32; jj++) d4[jj & 3] = fmaf(pv[jj], dp[jj], d4[jj & 3]);
        if (g == nk - 1) {
          ok = combine((d4[0] + d4[1]) + (d4[2] + d4[3]));
          if (!ok) break;
        }
      } else {
        store_block_32(stg, lane, pv, p_mat, p.lk, q0 + quad * 32, p.lq, col0, p.lk, vec_ok);
#pragma unroll
        for (int jj = 0; jj < 32; jj++) dp[jj] = (pv[jj] * (dp[jj] - dot)) * p.scale;      // dS
        store_block_32(stg, lane, dp, ds_mat, p.lk, q0 + quad * 32, p.lq, col0, p.lk, vec_ok);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == ATT_MT_ISSUE_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Rank-4 map over an activation seen as [B, H, L, D] through element strides; box = [32 floats, 128 rows, 1, 1].
static bool att_map(CUtensorMap* map, const float* base, int d, int l, int heads, int batch, long long s_row, long long s_head,
                    long long s_batch, bool mn_major) {
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)l, (cuuint64_t)heads, (cuuint64_t)batch};
  const cuuint64_t filler = ((cuuint64_t)s_row * 4 * (cuuint64_t)l + 15) & ~(cuuint64_t)15;
  cuuint64_t strides[3] = {(cuuint64_t)s_row * 4, heads > 1 ? (cuuint64_t)s_head * 4 : filler, batch > 1 ? (cuuint64_t)s_batch * 4 : filler};
  cuuint32_t box[4] = {32, (cuuint32_t)ATT_TILE, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool att_operand_ok(const float* p, const om_head_strides* s, int heads, int batch) {
  if ((reinterpret_cast<uintptr_t>(p) & 15) || (s->row & 3) || s->row <= 0) return false;
  if (heads > 1 && ((s->head & 3) || s->head <= 0)) return false;
  if (batch > 1 && ((s->batch & 3) || s->batch <= 0)) return false;
  return true;
}

bool attention_tc_fwd_supported(om_ctx* ctx, const float* q, const om_head_strides* qs, const float* k, const om_head_strides* ks,
                                const float* v, const om_head_strides* vs, const float* out, const om_head_strides* os, int b, int h,
                                int lq, int lk, int d) {
  if (!(ctx->flags & OM_TF32) || !encode_fn()) return false;
  if (lq < 1 || lk < 1 || (d != 32 && d != 64) || b < 1 || h < 1) return false;
  if ((lq > ATT_TILE || lk > ATT_TILE) && (long long)b * h > 65535) return false;   // the several-tile kernel puts (batch, head) on grid.y
  if (!att_operand_ok(q, qs, h, b) || !att_operand_ok(k, ks, h, b) || !att_operand_ok(v, vs, h, b)) return false;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (os->row & 3) || (os->head & 3) || (os->batch & 3)) return false;
  return true;
}

int32_t attention_tc_fwd(om_ctx* ctx, const float* q, const om_head_strides* qs, const float* k, const om_head_strides* ks, const float* v,
                         const om_head_strides* vs, const float* mask, long long mask_batch_stride, int b, int h, int lq, int lk, int d,
                         float scale, float* out, const om_head_strides* os, float* lse) {
  CUtensorMap mq, mk, mv;
  if (!att_map(&mq, q, d, lq, h, b, qs->row, qs->head, qs->batch, false) || !att_map(&mk, k, d, lk, h, b, ks->row, ks->head, ks->batch, false) ||
      !att_map(&mv, v, d, lk, h, b, vs->row, vs->head, vs->batch, true))
    return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed for the attention operands");
  AttFwdParams p;
  p.lq = lq; p.lk = lk; p.d = d; p.heads = h; p.scale = scale; p.mask = mask; p.mask_batch_stride = mask_batch_stride;
  p.out = out; p.o_batch = os->batch; p.o_head = os->head; p.o_row = os->row; p.lse = lse; p.status = ctx->status_dev;
  if (lq > ATT_TILE || lk > ATT_TILE) {
    // Several tiles: one CTA per 128 queries walks the key tiles (two passes, see attention_fwd_mt_kernel).
    const size_t smem_mt = (size_t)(5 * (d / 32) + 4) * ATT_BLOCK_BYTES + 1024 + 256;
    const dim3 grid_mt((unsigned)((lq + ATT_TILE - 1) / ATT_TILE), (unsigned)(b * h));
    if (d == 32) {
      static bool set = false;
      if (!set) {
        OM_CUDA(ctx, cudaFuncSetAttribute(attention_fwd_mt_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mt));
        set = true;
      }
      launch_chained(ctx, attention_fwd_mt_kernel<32>, grid_mt, ATT_MT_THREADS, smem_mt, mq, mk, mv, p);
    } else {
      static bool set = false;
      if (!set) {
        OM_CUDA(ctx, cudaFuncSetAttribute(attention_fwd_mt_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mt));
        set = true;
      }
      launch_chained(ctx, attention_fwd_mt_kernel<64>, grid_mt, ATT_MT_THREADS, smem_mt, mq, mk, mv, p);
    }
    OM_LAUNCH_CHECK(ctx, "attention_fwd_mt");
    return OM_OK;
  }
  const size_t smem = (size_t)((d / 32) + 4) * ATT_BLOCK_BYTES + 1024 + 256;
  const unsigned grid = (unsigned)(b * h);
  if (d == 32) {
    static bool set32 = false;
    if (!set32) {
      OM_CUDA(ctx, cudaFuncSetAttribute(attention_fwd_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      set32 = true;
    }
    launch_chained(ctx, attention_fwd_tc_kernel<32>, grid, ATT_THREADS, smem, mq, mk, mv, p);
  } else {
    static bool set64 = false;
    if (!set64) {
      OM_CUDA(ctx, cudaFuncSetAttribute(attention_fwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      set64 = true;
    }
    launch_chained(ctx, attention_fwd_tc_kernel<64>, grid, ATT_THREADS, smem, mq, mk, mv, p);
  }
  OM_LAUNCH_CHECK(ctx, "attention_fwd_tc");
  return OM_OK;
}

bool attention_tc_bwd_supported(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q, const om_head_strides* qs,
                                const float* k, const om_head_strides* ks, const float* v, const om_head_strides* vs, const float* lse,
                                int b, int h, int lq, int lk, int d, const float* dq, const om_head_strides* dqs, const float* dk,
                                const om_head_strides* dks, const float* dv, const om_head_strides* dvs) {
  if (!(ctx->flags & OM_TF32) || !encode_fn() || lse == nullptr) return false;
  if (lq < 1 || lk < 1 || lq > ATT_TILE || lk > ATT_TILE || d != 32 || b < 1 || h < 1) return false;
  if (!att_operand_ok(g, gs, h, b) || !att_operand_ok(q, qs, h, b) || !att_operand_ok(k, ks, h, b) || !att_operand_ok(v, vs, h, b)) return false;
  const float* outs[3] = {dq, dk, dv};
  const om_head_strides* os[3] = {dqs, dks, dvs};
  for (int i = 0; i < 3; i++)
    if (outs[i] && ((reinterpret_cast<uintptr_t>(outs[i]) & 15) || (os[i]->row & 3) || (os[i]->head & 3) || (os[i]->batch & 3))) return false;
  return true;
}

int32_t attention_tc_bwd(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q, const om_head_strides* qs, const float* k,
                         const om_head_strides* ks, const float* v, const om_head_strides* vs, const float* mask, long long mask_batch_stride,
                         const float* lse, int b, int h, int lq, int lk, float scale, float* dq, const om_head_strides* dqs, float* dk,
                         const om_head_strides* dks, float* dv, const om_head_strides* dvs) {
  CUtensorMap qk, kk, vk, gk, qm, km, gm;
  bool okm = att_map(&qk, q, 32, lq, h, b, qs->row, qs->head, qs->batch, false) && att_map(&kk, k, 32, lk, h, b, ks->row, ks->head, ks->batch, false) &&
             att_map(&vk, v, 32, lk, h, b, vs->row, vs->head, vs->batch, false) && att_map(&gk, g, 32, lq, h, b, gs->row, gs->head, gs->batch, false) &&
             att_map(&qm, q, 32, lq, h, b, qs->row, qs->head, qs->batch, true) && att_map(&km, k, 32, lk, h, b, ks->row, ks->head, ks->batch, true) &&
             att_map(&gm, g, 32, lq, h, b, gs->row, gs->head, gs->batch, true);
  if (!okm) return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed for the attention backward operands");
  AttBwdParams p;
  p.lq = lq; p.lk = lk; p.heads = h; p.scale = scale; p.mask = mask; p.mask_batch_stride = mask_batch_stride; p.lse = lse;
  p.dq = dq; p.dk = dk; p.dv = dv;
  p.dq_batch = dq ? dqs->batch : 0; p.dq_head = dq ? dqs->head : 0; p.dq_row = dq ? dqs->row : 0;
  p.dk_batch = dk ? dks->batch : 0; p.dk_head = dk ? dks->head : 0; p.dk_row = dk ? dks->row : 0;
  p.dv_batch = dv ? dvs->batch : 0; p.dv_head = dv ? dvs->head : 0; p.dv_row = dv ? dvs->row : 0;
  p.status = ctx->status_dev;
  const size_t smem = (size_t)12 * ATT_BLOCK_BYTES + 2 * ATT_TILE * sizeof(float) + 1024 + 256;
  static bool set = false;
  if (!set) {
    OM_CUDA(ctx, cudaFuncSetAttribute(attention_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    set = true;
  }
  launch_chained(ctx, attention_bwd_tc_kernel, (unsigned)(b * h), ATT_BWD_THREADS, smem, qk, kk, vk, gk, qm, km, gm, p);
  OM_LAUNCH_CHECK(ctx, "attention_bwd_tc");
  return OM_OK;
}

// The several-tile backward front: P and dS for the whole [B*H, Lq, Lk] score space from one kernel.
bool attention_bwd_front_supported(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q, const om_head_strides* qs,
                                   const float* k, const om_head_strides* ks, const float* v, const om_head_strides* vs, const float* lse,
                                   int b, int h, int lq, int lk, int d) {
  if (!(ctx->flags & OM_TF32) || !encode_fn() || lse == nullptr) return false;
  if (lq < 1 || lk < 1 || (d != 32 && d != 64) || b < 1 || h < 1 || (long long)b * h > 65535) return false;
  return att_operand_ok(g, gs, h, b) && att_operand_ok(q, qs, h, b) && att_operand_ok(k, ks, h, b) && att_operand_ok(v, vs, h, b);
}

template <int D, bool ONE_PASS>
static int32_t launch_front(om_ctx* ctx, dim3 grid, size_t smem, const CUtensorMap& mq, const CUtensorMap& mg, const CUtensorMap& mk,
                            const CUtensorMap& mv, const AttFrontParams& p) {
  static bool set = false;
  if (!set) {
    OM_CUDA(ctx, cudaFuncSetAttribute(attention_bwd_front_kernel<D, ONE_PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    set = true;
  }
  launch_chained(ctx, attention_bwd_front_kernel<D, ONE_PASS>, grid, ATT_MT_THREADS, smem, mq, mg, mk, mv, p);
  return OM_OK;
}

// o (the forward's output, with its strides) may be null: the kernel then takes a first pass over the key tiles for the row dots.
int32_t attention_bwd_front(om_ctx* ctx, const float* g, const om_head_strides* gs, const float* q, const om_head_strides* qs, const float* k,
                            const om_head_strides* ks, const float* v, const om_head_strides* vs, const float* o, const om_head_strides* os,
                            const float* mask, long long mask_batch_stride, const float* lse, int b, int h, int lq, int lk, int d, float scale,
                            float* p_out, float* ds_out) {
  CUtensorMap mq, mg, mk, mv;
  if (!att_map(&mq, q, d, lq, h, b, qs->row, qs->head, qs->batch, false) || !att_map(&mg, g, d, lq, h, b, gs->row, gs->head, gs->batch, false) ||
      !att_map(&mk, k, d, lk, h, b, ks->row, ks->head, ks->batch, false) || !att_map(&mv, v, d, lk, h, b, vs->row, vs->head, vs->batch, false))
    return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed for the attention backward operands");
  const bool one_pass = o != nullptr && os != nullptr && (reinterpret_cast<uintptr_t>(o) & 15) == 0 && (os->row & 3) == 0 &&
                        (os->head & 3) == 0 && (os->batch & 3) == 0;
  AttFrontParams p;
  p.lq = lq; p.lk = lk; p.heads = h; p.d = d; p.scale = scale; p.mask = mask; p.mask_batch_stride = mask_batch_stride; p.lse = lse;
  p.g = g; p.g_batch = gs->batch; p.g_head = gs->head; p.g_row = gs->row;
  p.o = one_pass ? o : nullptr; p.o_batch = one_pass ? os->batch : 0; p.o_head = one_pass ? os->head : 0; p.o_row = one_pass ? os->row : 0;
  p.p_out = p_out; p.ds_out = ds_out; p.status = ctx->status_dev;
  const size_t smem = (size_t)(4 * (d / 32)) * ATT_BLOCK_BYTES + 1024 + (ATT_MT_ISSUE_WARP * 32 * ATT_STG_LD + ATT_MT_PARTS * ATT_TILE) * sizeof(float) + 256;
  const dim3 grid((unsigned)((lq + ATT_TILE - 1) / ATT_TILE), (unsigned)(b * h));
  int32_t st;
  if (d == 32) st = one_pass ? launch_front<32, true>(ctx, grid, smem, mq, mg, mk, mv, p) : launch_front<32, false>(ctx, grid, smem, mq, mg, mk, mv, p);
  else st = one_pass ? launch_front<64, true>(ctx, grid, smem, mq, mg, mk, mv, p) : launch_front<64, false>(ctx, grid, smem, mq, mg, mk, mv, p);
  OM_TRY(st);
  OM_LAUNCH_CHECK(ctx, "attention_bwd_front");
  return OM_OK;
}

}  // namespace om
