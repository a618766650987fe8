// Persistent matrix product on the tensor pipe with CTA pairs and two accumulator buffers in tensor memory.
//
// One cluster of two CTAs (tcgen05.mma.cta_group::2) stays on its pair of SMs and walks a fixed list of 256 x BN tiles
// of C (cluster c takes tiles c, c + clusters, ...). Per CTA: warp 0 issues TMA loads into a ring of operand stages,
// warp 1 of the pair's leader issues the MMAs into one of TWO accumulator buffers in tensor memory, and four epilogue
// warps read the other buffer back (tcgen05.ld), add the bias and hand 32 x 32 blocks to the TMA unit
// (cp.async.bulk.tensor store, or cp.reduce .add when the product accumulates into C), optionally together with the same
// block rounded to bfloat16 for a second tensor (the copy that a following bfloat16 product or attention kernel reads).
// A tile's read-back and its stores therefore run under the next tile's MMAs; with one tile per CTA they were as long as
// the main loop of a k = 384 ... 768 product.
//
// Operand element types: TF32 (fp32 in memory, rounded to nearest even by the TMA load) or BF16 (bfloat16 in memory:
// half the bytes through L2 and shared memory per MMA, which is what bounds the fp32-operand tile). Accumulation is fp32
// in both. All four operand orientations run in place (K-major and MN-major shared-memory tiles).
//
// No multicast loads: each CTA fetches its own 128 rows of A and its own half of the B tile. Every wait is bounded
// (om_tc.cuh): on a timeout the kernel raises OM_ERR_TIMEOUT in the context's status word, all roles leave their loops,
// tensor memory is released and the kernel returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "om_act.cuh"
#include "om_tc.cuh"

namespace om {

constexpr int W_BM = 128;                 // rows of C per CTA; a pair computes 256
#ifndef OM_WS_STAGES
#define OM_WS_STAGES 6
#endif
#ifndef OM_WS_EPI_WARPS
#define OM_WS_EPI_WARPS 4
#endif
#ifndef OM_WS_RING
#define OM_WS_RING 1
#endif
constexpr int W_STAGES = OM_WS_STAGES;
constexpr int W_EPI_WARPS = OM_WS_EPI_WARPS;   // a multiple of four: the warps of a TMEM lane quadrant share the tile's columns
// With arithmetic or an extra operand in the epilogue: four warps per lane quadrant, so that their loads and dependent
// arithmetic hide one another, and one operand stage less to make room for their staging slots.
constexpr int W_ACT_EPI_WARPS = 16;
constexpr int W_ACT_STAGES = 5;
constexpr int W_RING = OM_WS_RING;        // staging slots per epilogue warp
#ifndef OM_WS_SLOT
#define OM_WS_SLOT 4096
#endif
constexpr int W_SLOT = OM_WS_SLOT;        // 4096: a 32 x 32 fp32 block (its bfloat16 copy follows through the same slot); 6144: both side by side
constexpr int kWsClusters = 74;           // pairs of one round on a 148-SM device: the k-split target (a constant of the shape rule)

template <int ELEM> struct WsElem;
// TF32: 32 fp32 per 128-byte row, one MMA consumes 8 of them (32 bytes). MN-major tiles use the 32-byte-unit swizzle.
template <> struct WsElem<0> {
  static constexpr int BYTES = 4, BK = 32, UMMA_K = 8;
  static constexpr uint32_t FORMAT = 2, MN_LAYOUT = 1, MN_SBO = 512;
};
// BF16: 64 per 128-byte row, one MMA consumes 16. MN-major tiles use the ordinary 128-byte swizzle: 8 k-rows per atom.
template <> struct WsElem<1> {
  static constexpr int BYTES = 2, BK = 64, UMMA_K = 16;
  static constexpr uint32_t FORMAT = 1, MN_LAYOUT = 2, MN_SBO = 1024;
};

struct WsParams {
  int m, n, k;
  int tiles_m, tiles_n, splits;   // tiles_m counts 256-row pairs
  int kb_per_split;               // k blocks per slice
  const float* bias;
  int accumulate;
  int shared_c;                   // both k-slices add (cp.reduce .add) into the one zeroed C instead of a workspace slice each
  int c16;                        // also store the bfloat16 copy of every block through map_c16 (never with accumulate)
  int store32;                    // store the fp32 result (0: only the bfloat16 copy leaves the kernel)
  int32_t* status;
  const float* aux;               // ACT 2: the activation's saved input; ACT 3: the tensor to add; [m, n] fp32 with pitch ld_aux
  long long ld_aux;
};

__device__ __forceinline__ uint32_t ws_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void ws_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the mbarrier at the same shared-memory offset in CTA `cta` of the cluster.
__device__ __forceinline__ void ws_arrive_remote(uint64_t* bar, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(cta));
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
__device__ __forceinline__ void ws_tma_load(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* leader_bar) {
  // The completion goes to the barrier at this offset in the pair's leader (the local address with the peer bit cleared).
  const uint32_t bar_addr = smem_u32(leader_bar) & 0xFEFFFFFFu;
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_addr)
      : "memory");
}
template <int ELEM>
__device__ __forceinline__ void ws_mma(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (ELEM == 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
  }
}
__device__ __forceinline__ void ws_commit(uint64_t* bar) {
  const uint16_t mask = 3;   // the barrier at this offset in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "h"(mask)
               : "memory");
}

// fp32 accumulator, A and B of the element format, major bits, N >> 3, M = 256 >> 4.
template <int ELEM>
__host__ __device__ constexpr uint32_t ws_idesc(int bn, bool a_mn, bool b_mn) {
  return (1u << 4) | (WsElem<ELEM>::FORMAT << 7) | (WsElem<ELEM>::FORMAT << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <int BN, int EW, int ST>
constexpr size_t ws_smem_bytes() {
  return (size_t)ST * (W_BM * 128 + (BN / 2) * 128) + (size_t)EW * W_RING * W_SLOT + 1024 + 256;
}

// Shared-memory tiles. K-major: rows (m or n) of 128 bytes of k, 8-row swizzle atoms 1024 bytes apart. MN-major: chunks of
// [BK k-rows x 128 bytes of m/n], BK * 128 bytes apart (leading offset); groups of k-rows MN_SBO bytes apart.
//
// ACT (with the unary operator OP) puts an activation between two Linear layers into the epilogue:
//   1: C receives the product (+ bias) as before, the bfloat16 tensor receives OP(C) rounded: the next layer's operand,
//      without the activation's own pass over C;
//   2: C and its bfloat16 copy receive d/dx OP(aux) * product, aux being the activation's saved input: the input
//      gradient of the layer after the activation, already multiplied by the activation's derivative;
//   3: C (and its copy) receive aux + product: a gradient that joins another branch's (a residual connection) without
//      a read-modify-write of that branch's tensor, which may then stay shared with its other readers;
//   4: C (and its copy) receive aux * product: the input gradient through an activation whose derivative was left behind by
//      the forward pass (5), with no transcendental arithmetic in this epilogue;
//   5: as 1, but C receives OP'(product + bias), the derivative that 4 multiplies by, instead of the product itself.
// EW epilogue warps (four, or eight when the epilogue has this arithmetic to do).
template <int ELEM, int BN, bool A_MN, bool B_MN, int ACT = 0, int OP = 0, int EW = W_EPI_WARPS, int ST = W_STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(32 * (2 + EW), 1)
gemm_ws_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_c16, WsParams p) {
  using E = WsElem<ELEM>;
  constexpr int BK = E::BK;
  constexpr int HB = BN / 2;                                   // rows of the B tile this CTA loads
  constexpr int A_BYTES = W_BM * 128, B_BYTES = HB * 128, STAGE = A_BYTES + B_BYTES;
  constexpr int MN_CHUNK = 128 / E::BYTES;                     // m/n elements per 128-byte row of an MN-major chunk
  constexpr int MN_CHUNK_BYTES = BK * 128;
  constexpr int MN_KSTEP_BYTES = E::UMMA_K * 128;              // one MMA's k-rows in an MN-major chunk
  constexpr uint32_t TMEM_COLS = 2 * BN;                       // two accumulator buffers
  constexpr int NB = BN / 32;                                  // 32-column blocks per tile

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + (size_t)ST * STAGE;
  constexpr int PARTS = EW / 4, CB_PER = NB / PARTS;            // the warps of a lane quadrant split the tile's column blocks
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + (size_t)EW * W_RING * W_SLOT);
  uint64_t* empty = full + ST;
  uint64_t* acc_full = empty + ST;           // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2], used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ws_cluster_ctarank();                  // 0 = leader
  const int cluster_id = (int)(blockIdx.x >> 1), clusters = (int)(gridDim.x >> 1);
  const int tiles = p.tiles_m * p.tiles_n, units = tiles * p.splits;
  const int k_blocks_total = (p.k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * EW);                        // every epilogue warp of both CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  ws_cluster_sync();                                           // both CTAs' barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  pdl_wait();

  if (warp == 0) {
    // ---- TMA producer (each CTA loads its own rows of A and its half of B) ----
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int u = cluster_id; u < units && ok; u += clusters) {
        const int split = u / tiles, t = u % tiles;
        const int m0 = (2 * (t / p.tiles_n) + (int)rank) * W_BM;
        const int nb = (t % p.tiles_n) * BN + (int)rank * HB;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(k_blocks_total, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = (int)(it % ST);
          const uint32_t round = it / ST;
          if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, abort_flag, p.status, 41)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + (size_t)s * STAGE;
          uint8_t* b_dst = a_dst + A_BYTES;
          const int k0 = kb * BK;
          if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE);  // the bytes of both CTAs land on the leader's barrier
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < W_BM / MN_CHUNK; j++) ws_tma_load(a_dst + j * MN_CHUNK_BYTES, &map_a, m0 + MN_CHUNK * j, k0, &full[s]);
          } else {
            ws_tma_load(a_dst, &map_a, k0, m0, &full[s]);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < HB / MN_CHUNK; j++) ws_tma_load(b_dst + j * MN_CHUNK_BYTES, &map_b, nb + MN_CHUNK * j, k0, &full[s]);
          } else {
            ws_tma_load(b_dst, &map_b, k0, nb, &full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (one thread of the leader CTA) ----
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = ws_idesc<ELEM>(BN, A_MN, B_MN);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int u = cluster_id; u < units && ok; u += clusters, tile_i++) {
        const int split = u / tiles;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(k_blocks_total, kb0 + p.kb_per_split);
        const uint32_t a = tile_i & 1, use = tile_i >> 1;
        // The epilogue warps of both CTAs must have read this buffer's previous tile out of tensor memory.
        if (use > 0 && !mbar_wait(&acc_empty[a], (use - 1) & 1, abort_flag, p.status, 42)) break;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + a * BN;
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = (int)(it % ST);
          const uint32_t round = it / ST;
          ok = mbar_wait(&full[s], round & 1, abort_flag, p.status, 43);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int ks = 0; ks < BK / E::UMMA_K; ks++) {
            // K-major: step 32 bytes along the swizzled row. MN-major: step one MMA's k-rows.
            const uint64_t adesc = A_MN ? make_desc(a_addr + ks * MN_KSTEP_BYTES, MN_CHUNK_BYTES, E::MN_SBO, E::MN_LAYOUT)
                                        : make_desc(a_addr + ks * 32, 16, 1024, 2);
            const uint64_t bdesc = B_MN ? make_desc(b_addr + ks * MN_KSTEP_BYTES, MN_CHUNK_BYTES, E::MN_SBO, E::MN_LAYOUT)
                                        : make_desc(b_addr + ks * 32, 16, 1024, 2);
            ws_mma<ELEM>(tmem_acc, adesc, bdesc, idesc, (kb > kb0 || ks > 0) ? 1u : 0u);
          }
          ws_commit(&empty[s]);          // frees the stage in both CTAs when these MMAs have read it
        }
        ws_commit(&acc_full[a]);         // the tile's accumulator is complete (or nothing is outstanding after an abort)
      }
    }
  } else {
    // ---- epilogue: warps 2..9; warp % 4 is the TMEM lane quadrant a warp may read, the two warps of a quadrant split
    //      the tile's 32-column blocks between them ----
    const int e = warp - 2;
    const int quad = warp & 3;
    const int part = e >> 2;
    uint8_t* ring = staging + (size_t)e * W_RING * W_SLOT;
    uint32_t tile_i = 0, stored = 0;
    bool ok = true;
    for (int u = cluster_id; u < units && ok; u += clusters, tile_i++) {
      const int split = p.shared_c ? 0 : u / tiles, t = u % tiles;
      const int m0 = (2 * (t / p.tiles_n) + (int)rank) * W_BM;
      const int n0 = (t % p.tiles_n) * BN;
      const uint32_t a = tile_i & 1, use = tile_i >> 1;
      const int row_base = m0 + quad * 32;
      // ACT 2, 3: this lane's 32 values of the extra operand for a column block (n is a multiple of four, so that a 16-byte
      // load never straddles the last column), asked for before the accumulator block is read back; the other warps of
      // the quadrant work while they are on their way.
      // With eight epilogue warps (two per lane quadrant) the next block's values are asked for a block ahead, into a second
      // set of registers; with sixteen the other warps of the quadrant cover the wait.
      // The factor of ACT 4 is stored as IEEE half (32 values in four 16-byte loads; n is then a multiple of eight).
      constexpr bool AHEAD = (ACT >= 2 && ACT <= 4) && EW == 8;
      constexpr int AUXN = ACT == 4 ? 4 : 8, AUX_PER = 32 / AUXN;
      float4 aux[AUXN], nxt[AHEAD ? AUXN : 1];
      auto load_aux = [&](float4 (&dst)[AUXN], int cb) {
        const int c0 = n0 + cb * 32, row = row_base + lane;
        const bool in = row < p.m && c0 < p.n;
        const int64_t at = (int64_t)(in ? row : 0) * p.ld_aux + (in ? c0 : 0);
        const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const char*>(p.aux) + at * (ACT == 4 ? 2 : 4));
#pragma unroll
        for (int c4 = 0; c4 < AUXN; c4++) dst[c4] = (in && c0 + AUX_PER * c4 < p.n) ? __ldg(src + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
      };
      if (AHEAD) load_aux(aux, part * CB_PER);
      ok = mbar_wait(&acc_full[a], use & 1, abort_flag, p.status, 44);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tmem_acc = tmem_base + a * BN + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int cb = part * CB_PER; cb < (part + 1) * CB_PER; cb++) {
        const int col0 = n0 + cb * 32;
        const bool live = row_base < p.m && col0 < p.n;
        uint32_t r[32];
        if (AHEAD) {
          if (cb + 1 < (part + 1) * CB_PER) load_aux(reinterpret_cast<float4(&)[AUXN]>(nxt), cb + 1);
        } else if (ACT >= 2 && ACT <= 4) {
          load_aux(aux, cb);
        }
        if (live) {
          tmem_ld_32x32b_x32(tmem_acc + (uint32_t)(cb * 32), r);
          tmem_ld_wait();
        }
        if (cb == (part + 1) * CB_PER - 1) {
          // This warp has everything it needs out of the buffer: the next tile but one may overwrite it.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) ws_arrive_remote(&acc_empty[a], 0);
        }
        if (!live) continue;
        if (p.bias) add_bias32(r, p.bias, col0, p.n);
        if constexpr (ACT == 2) {
#pragma unroll
          for (int c4 = 0; c4 < 8; c4++) {
            r[4 * c4 + 0] = __float_as_uint(unary_grad<OP>(__uint_as_float(r[4 * c4 + 0]), aux[c4].x));
            r[4 * c4 + 1] = __float_as_uint(unary_grad<OP>(__uint_as_float(r[4 * c4 + 1]), aux[c4].y));
            r[4 * c4 + 2] = __float_as_uint(unary_grad<OP>(__uint_as_float(r[4 * c4 + 2]), aux[c4].z));
            r[4 * c4 + 3] = __float_as_uint(unary_grad<OP>(__uint_as_float(r[4 * c4 + 3]), aux[c4].w));
          }
        }
        if constexpr (ACT == 4) {
#pragma unroll
          for (int c4 = 0; c4 < 4; c4++) {
            const __half2* h = reinterpret_cast<const __half2*>(&aux[c4]);
#pragma unroll
            for (int q = 0; q < 4; q++) {
              const float2 f = __half22float2(h[q]);
              r[8 * c4 + 2 * q] = __float_as_uint(__uint_as_float(r[8 * c4 + 2 * q]) * f.x);
              r[8 * c4 + 2 * q + 1] = __float_as_uint(__uint_as_float(r[8 * c4 + 2 * q + 1]) * f.y);
            }
          }
        }
        if constexpr (ACT == 5) {
          // The activation as packed bfloat16 (map_c16) and its derivative as packed IEEE half (map_c, a second 16-bit map of
          // the same shape): two 2 KB blocks in the 64-byte swizzle, side by side in the slot, stored together.
          if (stored >= W_RING) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(W_RING - 1) : "memory");
            __syncwarp();
          }
          uint8_t* blk5 = ring + (size_t)(stored % W_RING) * W_SLOT;
          const uint32_t row16 = smem_u32(blk5) + (uint32_t)lane * 64u;
#pragma unroll
          for (int c8 = 0; c8 < 4; c8++) {
            uint32_t wa[4], wd[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
              float a0, a1, d0, d1;
              unary_both<OP>(__uint_as_float(r[8 * c8 + 2 * q]), &a0, &d0);
              unary_both<OP>(__uint_as_float(r[8 * c8 + 2 * q + 1]), &a1, &d1);
              __nv_bfloat162 ha = __floats2bfloat162_rn(a0, a1);
              __half2 hd = __floats2half2_rn(d0, d1);
              wa[q] = *reinterpret_cast<uint32_t*>(&ha);
              wd[q] = *reinterpret_cast<uint32_t*>(&hd);
            }
            const uint32_t at = row16 + (uint32_t)((c8 ^ ((lane >> 1) & 3)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(at), "r"(wa[0]), "r"(wa[1]), "r"(wa[2]), "r"(wa[3]) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(at + 2048u), "r"(wd[0]), "r"(wd[1]), "r"(wd[2]), "r"(wd[3]) : "memory");
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&map_c16), "r"(col0),
                         "r"(row_base), "r"(smem_u32(blk5))
                         : "memory");
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&map_c), "r"(col0),
                         "r"(row_base), "r"(smem_u32(blk5 + 2048))
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          stored++;
          continue;
        }
        if constexpr (ACT == 3) {
#pragma unroll
          for (int c4 = 0; c4 < 8; c4++) {
            r[4 * c4 + 0] = __float_as_uint(aux[c4].x + __uint_as_float(r[4 * c4 + 0]));
            r[4 * c4 + 1] = __float_as_uint(aux[c4].y + __uint_as_float(r[4 * c4 + 1]));
            r[4 * c4 + 2] = __float_as_uint(aux[c4].z + __uint_as_float(r[4 * c4 + 2]));
            r[4 * c4 + 3] = __float_as_uint(aux[c4].w + __uint_as_float(r[4 * c4 + 3]));
          }
        }
        if (AHEAD) {
#pragma unroll
          for (int c4 = 0; c4 < AUXN; c4++) aux[c4] = nxt[AHEAD ? c4 : 0];
        }
        if (stored >= W_RING) {
          // The block about to be overwritten was handed to the TMA unit W_RING stores ago.
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(W_RING - 1) : "memory");   // all but the newest W_RING - 1
          __syncwarp();
        }
        uint8_t* blk = ring + (size_t)(stored % W_RING) * W_SLOT;
        // The block as bfloat16: 64 bytes per row in the 64-byte swizzle of map_c16 (16-byte chunk c of row r at
        // c ^ ((r >> 1) & 3)). With a slot of 6144 bytes it lies behind the fp32 block and both stores go out together;
        // with a slot of 4096 it takes the slot's place once the fp32 store has read it.
        auto stage_bf16 = [&](uint8_t* dst16) {
          const uint32_t row16 = smem_u32(dst16) + (uint32_t)lane * 64u;
#pragma unroll
          for (int c8 = 0; c8 < 4; c8++) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * c8 + 2 * q]), __uint_as_float(r[8 * c8 + 2 * q + 1]));
              w[q] = *reinterpret_cast<uint32_t*>(&h);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row16 + (uint32_t)((c8 ^ ((lane >> 1) & 3)) << 4)), "r"(w[0]), "r"(w[1]),
                         "r"(w[2]), "r"(w[3])
                         : "memory");
          }
        };
        const bool both_at_once = W_SLOT >= 6144 && ACT != 1;
        if (p.store32) {
          const uint32_t row_addr = smem_u32(blk) + (uint32_t)lane * 128u;
#pragma unroll
          for (int c4 = 0; c4 < 8; c4++)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (uint32_t)((c4 ^ (lane & 7)) << 4)), "r"(r[4 * c4]),
                         "r"(r[4 * c4 + 1]), "r"(r[4 * c4 + 2]), "r"(r[4 * c4 + 3])
                         : "memory");
          if (p.c16 && both_at_once) stage_bf16(blk + 4096);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (p.c16 && both_at_once)
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&map_c16), "r"(col0),
                           "r"(row_base), "r"(smem_u32(blk + 4096))
                           : "memory");
            if (p.accumulate)
              asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(&map_c),
                           "r"(col0), "r"(row_base), "r"(split), "r"(smem_u32(blk))
                           : "memory");
            else
              asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(&map_c), "r"(col0),
                           "r"(row_base), "r"(split), "r"(smem_u32(blk))
                           : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        if (p.c16 && !(p.store32 && both_at_once)) {
          if (ACT == 1) {
            // The activation's arithmetic runs while the TMA unit reads the fp32 block out of the slot.
#pragma unroll
            for (int i = 0; i < 32; i++) r[i] = __float_as_uint(unary_apply<OP>(__uint_as_float(r[i])));
          }
          if (p.store32) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
          }
          stage_bf16(blk);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&map_c16), "r"(col0),
                         "r"(row_base), "r"(smem_u32(blk))
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        stored++;
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  ws_cluster_sync();                                           // neither CTA leaves (or frees tensor memory) while its partner still works
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

void splitk_reduce_launch(om_ctx* ctx, const float* part, int splits, int64_t mn, int n, int64_t ldc, const float* bias, float* out, int accumulate);

// Rank-2 operand map over a row-major matrix [outer, inner] with leading dimension ld (elements). K-major tiles take the
// 128-byte swizzle; MN-major tiles the 32-byte-unit one for 4-byte elements and the ordinary one for 2-byte elements.
static bool ws_operand_map(CUtensorMap* map, int elem, const void* base, int inner, int outer, long long ld, int box_outer, bool mn_major) {
  const int bytes = elem == 0 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * bytes};
  cuuint32_t box[2] = {(cuuint32_t)(128 / bytes), (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = (mn_major && elem == 0) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  return encode_fn()(map, elem == 0 ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The map the epilogue stores through: C as [splits, m, n] fp32, box [1, 32 rows, 32 columns], 128-byte swizzle.
static bool ws_store_map(CUtensorMap* map, float* base, int n, int m, long long ld, int splits, long long split_stride) {
  cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)splits};
  cuuint64_t filler = (((cuuint64_t)ld * m * 4) + 15) & ~(cuuint64_t)15;
  cuuint64_t strides[2] = {(cuuint64_t)ld * 4, splits > 1 ? (cuuint64_t)split_stride * 4 : filler};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The map of the bfloat16 copy of C: [m, n] with the same pitch in elements, box [32 rows, 32 columns], 64-byte swizzle.
static bool ws_store_map16(CUtensorMap* map, uint16_t* base, int n, int m, long long ld) {
  cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)m};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// What the kernel can take: operand and C pitches and base addresses that TMA can describe (16-byte multiples), any m, n, k.
bool gemm_ws_supported(om_ctx* ctx, int elem, int m, int n, int k, const void* A, long long lda, const void* B, long long ldb, const float* C,
                       long long ldc) {
  (void)ctx;
  if (!encode_fn()) return false;
  if (m < 1 || n < 1 || k < 1) return false;
  const int per16 = elem == 0 ? 4 : 8;
  if ((lda % per16) || (ldb % per16) || (ldc & 3)) return false;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15)) return false;
  return true;
}

template <int ELEM, int BN>
static int32_t ws_launch(om_ctx* ctx, bool a_mn, bool b_mn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                         const CUtensorMap& mc16, const WsParams& p, int units) {
  constexpr size_t smem = ws_smem_bytes<BN, W_EPI_WARPS, W_STAGES>();
  constexpr int W_THREADS = 32 * (2 + W_EPI_WARPS);
#define OM_WS(AMN, BMN)                                                                                                          \
  do {                                                                                                                           \
    static int max_clusters = 0;                                                                                                 \
    if (max_clusters == 0) {                                                                                                     \
      OM_CUDA(ctx, cudaFuncSetAttribute(gemm_ws_kernel<ELEM, BN, AMN, BMN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      cudaLaunchConfig_t q = {};                                                                                                 \
      q.gridDim = dim3(2 * (unsigned)ctx->sm_count);                                                                             \
      q.blockDim = dim3(W_THREADS);                                                                                              \
      q.dynamicSmemBytes = smem;                                                                                                 \
      int nc = 0;                                                                                                                \
      if (cudaOccupancyMaxActiveClusters(&nc, gemm_ws_kernel<ELEM, BN, AMN, BMN>, &q) != cudaSuccess || nc < 1) {                 \
        cudaGetLastError();                                                                                                      \
        nc = ctx->sm_count / 2;                                                                                                  \
      }                                                                                                                          \
      max_clusters = nc;                                                                                                         \
    }                                                                                                                            \
    const int clusters = units < max_clusters ? units : max_clusters;                                                            \
    launch_chained(ctx, gemm_ws_kernel<ELEM, BN, AMN, BMN>, dim3(2 * (unsigned)clusters), W_THREADS, smem, ma, mb, mc, mc16, p);  \
  } while (0)
  if (!a_mn && !b_mn) OM_WS(false, false);
  else if (!a_mn && b_mn) OM_WS(false, true);
  else if (a_mn && !b_mn) OM_WS(true, false);
  else OM_WS(true, true);
#undef OM_WS
  OM_LAUNCH_CHECK(ctx, "gemm_ws");
  return OM_OK;
}

// The variants with an activation in the epilogue: bfloat16 operands, 256-wide tiles, A row-major [m, k]; B is [n, k]
// for ACT 1 (a Linear forward) and [k, n] for ACT 2 (a Linear input gradient).
template <int ACT, int OP>
static int32_t ws_launch_act(om_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const CUtensorMap& mc16,
                             const WsParams& p, int units) {
  // The plain sum (ACT 3) has next to no arithmetic and joins long products: eight warps and the full operand ring.
  constexpr bool light = ACT == 3 || ACT == 4;
  constexpr int EW = light ? 8 : W_ACT_EPI_WARPS, ST = light ? W_STAGES : W_ACT_STAGES;
  constexpr size_t smem = ws_smem_bytes<256, EW, ST>();
  constexpr int threads = 32 * (2 + EW);
  auto kernel = gemm_ws_kernel<1, 256, false, (ACT >= 2 && ACT <= 4), ACT, OP, EW, ST>;
  static int max_clusters = 0;
  if (max_clusters == 0) {
    OM_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(2 * (unsigned)ctx->sm_count);
    q.blockDim = dim3(threads);
    q.dynamicSmemBytes = smem;
    int nc = 0;
    if (cudaOccupancyMaxActiveClusters(&nc, kernel, &q) != cudaSuccess || nc < 1) {
      cudaGetLastError();
      nc = ctx->sm_count / 2;
    }
    max_clusters = nc;
  }
  const int clusters = units < max_clusters ? units : max_clusters;
  launch_chained(ctx, kernel, dim3(2 * (unsigned)clusters), threads, smem, ma, mb, mc, mc16, p);
  OM_LAUNCH_CHECK(ctx, "gemm_ws (activation epilogue)");
  return OM_OK;
}

// C[m, n] (+)= op(A)[m, k] op(B)[k, n] + bias. elem 0: A and B are fp32 (TF32 products); elem 1: A and B are bfloat16.
// ta != 0: A is stored [k, m]; tb != 0: B is stored [n, k]. Leading dimensions in elements of the operand's own type.
// C16 (may be null): also receives C rounded to bfloat16, element i of C16 being element i of C (same pitch). Needs a
// pitch that is a multiple of 8, a 16-byte aligned C16 and no accumulation; gemm_ws_c16_ok tells.
bool gemm_ws_c16_ok(const uint16_t* C16, long long ldc, int acc) {
  return C16 && !acc && (ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C16) & 15) == 0;
}

int32_t cast_bf16_rows(om_ctx* ctx, const float* src, uint16_t* dst, int rows, int cols, long long ld);

// act 0: none. act 1 with op: C16 receives op(C) instead of C. act 2 with op: C and C16 receive op'(aux) * C. act 3: aux + C.
// act 4: aux * C, aux holding IEEE half values (pitch ld_aux in those). act 5 with op: C16 receives op(C) and the memory at C
// receives op'(C) as IEEE half with C16's pitch (the pointer is typed float* for the other variants' sake).
// gemm_ws_act_ok tells whether a product can take the activation (no split of k, the layouts above).
static int ws_splits(int tiles, int k_blocks) {
  // Fixed split of k by shape alone: enough slices for one round of pairs, each at least 8 k-blocks deep.
  int splits = 1;
  if (tiles < kWsClusters && k_blocks >= 16) {
    splits = (int)std::min<int64_t>(kWsClusters / tiles, k_blocks / 8);
    if (splits < 1) splits = 1;
    if (splits > 32) splits = 32;
  }
  return splits;
}

bool gemm_ws_act_ok(int act, int op, int m, int n, int k, const float* C, long long ldc, const uint16_t* C16, const float* aux, long long ld_aux) {
  if (act < 1 || act > 5) return false;
  const bool fwd = act == 1 || act == 5, with_aux = act >= 2 && act <= 4;
  if (act != 3 && act != 4 && op != OM_GELU_ERF && op != OM_GELU_TANH) return false;
  if (m < 1 || n < 256 || (n & 3)) return false;
  const int tiles = (int)(ceil_div(m, 2 * W_BM) * ceil_div(n, 256));
  if (ws_splits(tiles, (int)ceil_div(k, 64)) != 1) return false;
  if (fwd && !gemm_ws_c16_ok(C16, ldc, 0)) return false;
  if (with_aux && (C16 != nullptr) && !gemm_ws_c16_ok(C16, ldc, 0)) return false;
  if (with_aux && (!aux || (ld_aux & 3) || (reinterpret_cast<uintptr_t>(aux) & 15))) return false;
  if (act == 4 && ((ld_aux & 7) || (n & 7))) return false;
  if (act == 5 && (!C || (reinterpret_cast<uintptr_t>(C) & 15))) return false;
  (void)C;
  return true;
}

int32_t gemm_ws_act(om_ctx* ctx, int elem, int ta, int tb, int m, int n, int k, const void* A, long long lda, const void* B, long long ldb, float* C,
                    long long ldc, int acc, const float* bias, uint16_t* C16, int act, int op, const float* aux, long long ld_aux);

int32_t gemm_ws(om_ctx* ctx, int elem, int ta, int tb, int m, int n, int k, const void* A, long long lda, const void* B, long long ldb, float* C,
                long long ldc, int acc, const float* bias, uint16_t* C16) {
  return gemm_ws_act(ctx, elem, ta, tb, m, n, k, A, lda, B, ldb, C, ldc, acc, bias, C16, 0, 0, nullptr, 0);
}

int32_t gemm_ws_act(om_ctx* ctx, int elem, int ta, int tb, int m, int n, int k, const void* A, long long lda, const void* B, long long ldb, float* C,
                    long long ldc, int acc, const float* bias, uint16_t* C16, int act, int op, const float* aux, long long ld_aux) {
  const bool a_mn = ta != 0, b_mn = tb == 0;
  const bool store32 = C != nullptr;
  if (!store32 && (!C16 || acc || elem != 1))
    return fail(ctx, OM_ERR_ARG, "persistent product: without an fp32 result the bfloat16 one is required (bfloat16 operands, no accumulation)");
  if (act != 0) {
    if (elem != 1 || acc || a_mn || b_mn != (act >= 2 && act <= 4) || !gemm_ws_act_ok(act, op, m, n, k, C, ldc, C16, aux, ld_aux))
      return fail(ctx, OM_ERR_UNSUPPORTED, "persistent product: this shape or layout cannot take the activation in its epilogue (m %d n %d k %d)", m, n, k);
  }
  const int bk = elem == 0 ? 32 : 64, mn_chunk = elem == 0 ? 32 : 64;
  // Tile width: 256 unless the last 256-wide tile would be less than half used.
  const int rem = n % 256;
  const int bn = act != 0 ? 256 : (n <= 128 || (rem > 0 && rem <= 128 && n < 1024)) ? 128 : 256;
  CUtensorMap map_a, map_b, map_c, map_c16;
  bool ok = a_mn ? ws_operand_map(&map_a, elem, A, m, k, lda, bk, true) : ws_operand_map(&map_a, elem, A, k, m, lda, W_BM, false);
  ok = ok && (b_mn ? ws_operand_map(&map_b, elem, B, n, k, ldb, bk, true) : ws_operand_map(&map_b, elem, B, k, n, ldb, bn / 2, false));
  (void)mn_chunk;
  if (!ok) return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed (persistent product, m %d n %d k %d lda %lld ldb %lld)", m, n, k, lda, ldb);
  WsParams p;
  p.m = m; p.n = n; p.k = k;
  p.tiles_m = (int)ceil_div(m, 2 * W_BM);
  p.tiles_n = (int)ceil_div(n, bn);
  const int tiles = p.tiles_m * p.tiles_n, k_blocks = (int)ceil_div(k, bk);
  int splits = ws_splits(tiles, k_blocks);
  p.kb_per_split = (int)ceil_div(k_blocks, splits);
  splits = (int)ceil_div(k_blocks, p.kb_per_split);
  p.splits = splits;
  p.status = ctx->status_dev;
  p.store32 = store32 ? 1 : 0;
  p.shared_c = 0;
  if (!store32 && splits > 1) return fail(ctx, OM_ERR_UNSUPPORTED, "persistent product: a product whose k is split needs its fp32 result (m %d n %d k %d)", m, n, k);
  p.aux = aux;
  p.ld_aux = ld_aux;
  float* workspace = nullptr;
  // Two slices of k and nothing else to fold in (a weight gradient that overwrites): C is zeroed and both slices add their
  // tiles into it with the TMA unit's reduction. (0 + a) + b and (0 + b) + a are the same fp32 value, so the result does not
  // depend on which slice arrives first, and it is the a + b that the slice sum gives; more than two slices would.
  const bool two_in_place = splits == 2 && !acc && !bias && !C16 && store32 && act == 0;
  if (two_in_place) {
    OM_CUDA(ctx, cudaMemset2DAsync(C, (size_t)ldc * 4, 0, (size_t)n * 4, (size_t)m, ctx->stream));
    p.bias = nullptr; p.accumulate = 1; p.shared_c = 1;
    ok = ws_store_map(&map_c, C, n, m, ldc, 1, 0);
  } else if (splits > 1) {
    OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)splits * m * n, false, (void**)&workspace));
    p.bias = nullptr; p.accumulate = 0;
    ok = ws_store_map(&map_c, workspace, n, m, n, splits, (long long)m * n);
  } else {
    p.bias = bias; p.accumulate = acc;
    ok = !store32 || ws_store_map(&map_c, C, n, m, ldc, 1, 0);
  }
  // The bfloat16 copy rides in the epilogue of an unsplit product; after a split of k it is cast from the finished C.
  p.c16 = (C16 && splits == 1 && gemm_ws_c16_ok(C16, ldc, acc)) ? 1 : 0;
  if (!store32 && !p.c16) return fail(ctx, OM_ERR_UNSUPPORTED, "persistent product: the bfloat16 result needs a pitch that is a multiple of 8 and a 16-byte aligned base");
  if (p.c16) ok = ok && ws_store_map16(&map_c16, C16, n, m, ldc);
  else map_c16 = map_c;   // never used, but the parameter must hold a valid map
  if (!store32) map_c = map_c16;
  if (act == 5) ok = ok && ws_store_map16(&map_c, reinterpret_cast<uint16_t*>(C), n, m, ldc);
  if (!ok) {
    if (workspace) pool_free(ctx, workspace);
    return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed for C (persistent product, m %d n %d ldc %lld)", m, n, ldc);
  }
  const int units = tiles * splits;
  int32_t st;
  if (act == 1) st = op == OM_GELU_ERF ? ws_launch_act<1, OM_GELU_ERF_FAST>(ctx, map_a, map_b, map_c, map_c16, p, units)
                                       : ws_launch_act<1, OM_GELU_TANH>(ctx, map_a, map_b, map_c, map_c16, p, units);
  else if (act == 2) st = op == OM_GELU_ERF ? ws_launch_act<2, OM_GELU_ERF_FAST>(ctx, map_a, map_b, map_c, map_c16, p, units)
                                            : ws_launch_act<2, OM_GELU_TANH>(ctx, map_a, map_b, map_c, map_c16, p, units);
  else if (act == 3) st = ws_launch_act<3, 0>(ctx, map_a, map_b, map_c, map_c16, p, units);
  else if (act == 4) st = ws_launch_act<4, 0>(ctx, map_a, map_b, map_c, map_c16, p, units);
  else if (act == 5) st = op == OM_GELU_ERF ? ws_launch_act<5, OM_GELU_ERF_FAST>(ctx, map_a, map_b, map_c, map_c16, p, units)
                                            : ws_launch_act<5, OM_GELU_TANH>(ctx, map_a, map_b, map_c, map_c16, p, units);
  else if (elem == 0) st = bn == 256 ? ws_launch<0, 256>(ctx, a_mn, b_mn, map_a, map_b, map_c, map_c16, p, units) : ws_launch<0, 128>(ctx, a_mn, b_mn, map_a, map_b, map_c, map_c16, p, units);
  else st = bn == 256 ? ws_launch<1, 256>(ctx, a_mn, b_mn, map_a, map_b, map_c, map_c16, p, units) : ws_launch<1, 128>(ctx, a_mn, b_mn, map_a, map_b, map_c, map_c16, p, units);
  if (st == OM_OK && splits > 1 && !two_in_place) splitk_reduce_launch(ctx, workspace, splits, (int64_t)m * n, n, ldc, bias, C, acc);
  if (workspace) pool_free(ctx, workspace);
  if (st == OM_OK && C16 && !p.c16) st = cast_bf16_rows(ctx, C, C16, m, n, ldc);
  return st;
}

}  // namespace om
