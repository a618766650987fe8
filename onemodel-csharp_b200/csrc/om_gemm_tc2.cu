// Matrix product on the tensor pipe with CTA pairs (tcgen05.mma.cta_group::2): two CTAs on neighbouring SMs compute one
// 256 x BN tile of C together. Each CTA loads its own 128 rows of A and HALF of the B tile, the pair's MMA reads both
// halves, so per 128 x BN outputs a CTA brings in (128 + BN / 2) operand rows instead of (128 + BN): with fp32 operands
// (4 bytes per element) the operand delivery from L2, not the MMA rate, bounds the one-CTA kernel (om_gemm_tc.cu), and
// this halves it. No multicast loads are involved: every CTA fetches exactly the bytes it keeps.
//
// Roles per CTA as in the one-CTA kernel: warp 0 lane 0 issues TMA loads (completing on the LEADER's full barrier), warp
// 1 owns the TMEM allocation (both CTAs allocate with cta_group::2) and, in the leader CTA only, one thread issues the
// MMAs and commits to the barriers of both CTAs; warps 2-5 read the CTA's own accumulator rows back and store them.
// Waits are bounded as everywhere (om_tc.cuh).
#include "om_tc.cuh"

namespace om {

constexpr int P_BM = 128, P_BK = 32, P_STAGES = 3, P_UMMA_K = 8;
constexpr int P_THREADS = 192;

struct PairParams {
  int m, n, k;
  int k_per_split, splits;
  float* c;
  int ldc;
  int accumulate;
  const float* bias;
  int32_t* status;
  int tma_store;        // the epilogue writes C through map_c
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// TMA tile load of a CTA of a pair; the completion goes to the mbarrier at the same offset in the pair's leader CTA
// (the leader's shared-window address is the local one with the peer bit cleared).
__device__ __forceinline__ void tma_load_4d_pair(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
  const uint32_t bar_addr = smem_u32(bar) & 0xFEFFFFFFu;
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar_addr)
      : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs of the pair when the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "h"(mask)
               : "memory");
}

// Instruction descriptor: fp32 accumulator, TF32 operands, M = 256 (the pair), N = BN.
__host__ __device__ constexpr uint32_t pair_idesc(int bn, bool a_mn, bool b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(bn >> 3) << 17) |
         ((uint32_t)(256 >> 4) << 24);
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, PairParams p) {
  constexpr int HB = BN / 2;                              // rows of the B tile this CTA loads
  constexpr int A_BYTES = P_BM * P_BK * 4, B_BYTES = HB * P_BK * 4, STAGE = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = BN <= 128 ? 128 : 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)P_STAGES * STAGE);
  uint64_t* empty = full + P_STAGES;
  uint64_t* acc_full = empty + P_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                // 0 = leader
  // blockIdx.x = 2 * column tile + rank, blockIdx.y = pair of row blocks: the column tiles of one pair of row blocks are
  // launched next to one another, so their common A rows are read from HBM once and then found in L2.
  const int m0 = (2 * (int)blockIdx.y + (int)rank) * P_BM;
  const int n0 = (int)(blockIdx.x >> 1) * BN;
  const int split = blockIdx.z;
  const int k_begin = split * p.k_per_split;
  const int k_end = min(p.k, k_begin + p.k_per_split);
  const int k_blocks = (k_end - k_begin + P_BK - 1) / P_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                     // both CTAs' barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < k_blocks; kb++) {
        const int s = kb % P_STAGES;
        const uint32_t round = kb / P_STAGES;
        if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, abort_flag, p.status, 31)) break;
        uint8_t* a_dst = smem + (size_t)s * STAGE;
        uint8_t* b_dst = a_dst + A_BYTES;
        const int k0 = k_begin + kb * P_BK;
        if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE);     // the bytes of both CTAs land on the leader's barrier
        if (A_MN) {
#pragma unroll
          for (int j = 0; j < P_BM / 32; j++) tma_load_4d_pair(a_dst + j * (P_BK * 128), &map_a, m0 + 32 * j, k0, 0, 0, &full[s]);
        } else {
          tma_load_4d_pair(a_dst, &map_a, k0, m0, 0, 0, &full[s]);
        }
        const int nb = n0 + (int)rank * HB;                    // this CTA's half of the B tile
        if (B_MN) {
#pragma unroll
          for (int j = 0; j < HB / 32; j++) tma_load_4d_pair(b_dst + j * (P_BK * 128), &map_b, nb + 32 * j, k0, 0, 0, &full[s]);
        } else {
          tma_load_4d_pair(b_dst, &map_b, k0, nb, 0, 0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = pair_idesc(BN, A_MN, B_MN);
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; kb++) {
        const int s = kb % P_STAGES;
        const uint32_t round = kb / P_STAGES;
        ok = mbar_wait(&full[s], round & 1, abort_flag, p.status, 32);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE);
        const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
        for (int ks = 0; ks < P_BK / P_UMMA_K; ks++) {
          const uint64_t adesc = A_MN ? make_desc(a_addr + ks * 1024, P_BK * 128, 512, 1) : make_desc(a_addr + ks * (P_UMMA_K * 4), 16, 1024, 2);
          const uint64_t bdesc = B_MN ? make_desc(b_addr + ks * 1024, P_BK * 128, 512, 1) : make_desc(b_addr + ks * (P_UMMA_K * 4), 16, 1024, 2);
          umma_tf32_pair(tmem_base, adesc, bdesc, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit_pair(&empty[s]);
      }
      umma_commit_pair(acc_full);
    }
  } else {
    // ---- epilogue: this CTA's 128 accumulator rows, as in the one-CTA kernel ----
    const int quad = warp & 3;
    bool ok = true;
    if (k_blocks > 0) ok = mbar_wait(acc_full, 0, abort_flag, p.status, 33);
    tc_fence_after();
    float* c = p.c + (size_t)split * p.m * p.ldc;
    constexpr int STG_LD = 36;
    float* stg = reinterpret_cast<float*>(smem) + quad * 32 * STG_LD;
    const int row_base = m0 + quad * 32;
    const bool aligned = ((reinterpret_cast<uintptr_t>(c) & 15) == 0) && ((p.ldc & 3) == 0);
    if (ok && row_base < p.m && p.tma_store) {
      // Bulk stores as in the one-CTA kernel: 32 x 32 blocks staged in the swizzled layout of the C map and handed to the
      // TMA unit. A warp cycles through four 4 KB staging blocks; before it overwrites one it waits until the bulk copy
      // that read it (three copies back) has finished reading.
      constexpr int RING = 4;
#pragma unroll 1
      for (int cb = 0; cb < BN / 32; cb++) {
        const int col0 = n0 + cb * 32;
        if (col0 >= p.n) break;
        uint32_t r[32];
        if (k_blocks > 0) {
          tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(cb * 32), r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++) r[j] = 0u;
        }
        if (p.bias) add_bias32(r, p.bias, col0, p.n);
        if (cb >= RING) {
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
          __syncwarp();
        }
        uint8_t* blk = smem + (size_t)(quad * RING + (cb % RING)) * 4096;
        const uint32_t row_addr = smem_u32(blk) + (uint32_t)lane * 128u;
#pragma unroll
        for (int c4 = 0; c4 < 8; c4++)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (uint32_t)((c4 ^ (lane & 7)) << 4)), "r"(r[4 * c4]),
                       "r"(r[4 * c4 + 1]), "r"(r[4 * c4 + 2]), "r"(r[4 * c4 + 3])
                       : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          if (p.accumulate)
            asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(&map_c),
                         "r"(col0), "r"(row_base), "r"(split), "r"(0), "r"(smem_u32(blk))
                         : "memory");
          else
            asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(&map_c), "r"(col0),
                         "r"(row_base), "r"(split), "r"(0), "r"(smem_u32(blk))
                         : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      __syncwarp();
    } else if (ok && row_base < p.m) {
#pragma unroll 1
      for (int cb = 0; cb < BN / 32; cb++) {
        const int col0 = n0 + cb * 32;
        if (col0 >= p.n) break;
        uint32_t r[32];
        if (k_blocks > 0) {
          tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(cb * 32), r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++) r[j] = 0u;
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(stg + lane * STG_LD + j) =
              make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        __syncwarp();
        if (aligned && col0 + 32 <= p.n) {
          const int cc = (lane & 7) * 4;
          float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
          if (p.bias) bv = *reinterpret_cast<const float4*>(p.bias + col0 + cc);
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int rr = i * 4 + (lane >> 3);
            const int row = row_base + rr;
            if (row < p.m) {
              float4 v = *reinterpret_cast<const float4*>(stg + rr * STG_LD + cc);
              if (p.bias) { v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w; }
              float4* dst = reinterpret_cast<float4*>(c + (size_t)row * p.ldc + col0 + cc);
              if (p.accumulate) {
                float4 o = *dst;
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
              }
              *dst = v;
            }
          }
        } else {
          const int col = col0 + lane;
          if (col < p.n) {
            const float bvs = p.bias ? p.bias[col] : 0.f;
            for (int rr = 0; rr < 32; rr++) {
              const int row = row_base + rr;
              if (row >= p.m) break;
              float v = stg[rr * STG_LD + lane];
              if (p.bias) v += bvs;
              float* dst = c + (size_t)row * p.ldc + col;
              if (p.accumulate) v += *dst;
              *dst = v;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                     // neither CTA leaves (or frees TMEM) while its partner still works
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

bool make_store_map(CUtensorMap* map, float* base, int n, int m, long long ld, int inner_count, long long inner_stride, int outer_count,
                    long long outer_stride);
void splitk_reduce_launch(om_ctx* ctx, const float* part, int splits, int64_t mn, int n, int64_t ldc, const float* bias, float* out, int accumulate);

// Rank-4 map with unit batch dimensions (the pair kernel serves plain products only).
static bool pair_map(CUtensorMap* map, const float* base, int inner, int outer, int ld, int box_outer, bool mn_major) {
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)outer, 1, 1};
  cuuint64_t filler = (((cuuint64_t)ld * outer * 4) + 15) & ~(cuuint64_t)15;
  if (filler < 16) filler = 16;
  cuuint64_t strides[3] = {(cuuint64_t)ld * 4, filler, filler};
  cuuint32_t box[4] = {32, (cuuint32_t)box_outer, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The pair kernel needs rows for pairs and a width of at least one 128-column tile. By default it takes the products
// with several rounds of tiles over the device and no split of k (measured: 3 to 10 % faster on the widest products of a
// 768-wide encoder, 1.44x at 4096^3, slower on products of one or two rounds, where the larger tile leaves SMs idle);
// OM_PAIR_TILES sends every product it can take to it.
bool gemm_pair_supported(om_ctx* ctx, int m, int n, int k) {
  if (m < 256 || n < 128 || k < 64 || m > 65535 * 256) return false;
  if (ctx->flags & OM_PAIR_TILES) return true;
  const int64_t tiles = ceil_div(m, P_BM) * ceil_div(n, 128);
  if (tiles >= 4 * (int64_t)148 && m >= 1024 && n >= 256) return true;
  // Deep-k products with few tiles (the weight gradients of a wide layer): measured 1.3-1.4x at 768-wide layers, about
  // even at 384.
  return tiles < 148 && k >= 128 * P_BK && m >= 512 && m % 256 == 0 && n >= 512 && n % 256 == 0;
}

template <int BN>
static int32_t launch_pair(om_ctx* ctx, bool a_mn, bool b_mn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                           const PairParams& p, dim3 grid) {
  constexpr size_t smem = (size_t)P_STAGES * (P_BM * P_BK * 4 + (BN / 2) * P_BK * 4) + 1024 + 256;
#define OM_PAIR(AMN, BMN)                                                                                                   \
  do {                                                                                                                      \
    static bool attr_set = false;                                                                                           \
    if (!attr_set) {                                                                                                        \
      OM_CUDA(ctx, cudaFuncSetAttribute(gemm_pair_kernel<BN, AMN, BMN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      attr_set = true;                                                                                                      \
    }                                                                                                                       \
    launch_chained(ctx, gemm_pair_kernel<BN, AMN, BMN>, grid, P_THREADS, smem, ma, mb, mc, p);                              \
  } while (0)
  if (!a_mn && !b_mn) OM_PAIR(false, false);
  else if (!a_mn && b_mn) OM_PAIR(false, true);
  else if (a_mn && !b_mn) OM_PAIR(true, false);
  else OM_PAIR(true, true);
#undef OM_PAIR
  OM_LAUNCH_CHECK(ctx, "gemm_pair");
  return OM_OK;
}

int32_t gemm_pair(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B, int ldb, float* C, int ldc,
                  int acc, const float* bias) {
  const bool a_mn = ta != 0, b_mn = tb == 0;
  // Tile width 128, 192 or 256: the one with the shortest estimated time, counted as rounds of CTAs over the device (two
  // CTAs per SM) times the work of a CTA (its tile width plus a fixed part for prologue and epilogue). Wide tiles bring in
  // fewer operand bytes per output but leave small products with too few CTAs.
  int bn = 128;
  {
    const int64_t slots = kSplitSlots;
    int64_t best = 0;
    for (int cand : {128, 192, 256}) {
      const int64_t ctas_c = 2 * ceil_div(m, 2 * P_BM) * ceil_div(n, cand);
      const int64_t cost = ceil_div(ctas_c, slots) * (cand + 64);
      if (best == 0 || cost < best || (cost == best && cand > bn)) {
        best = cost;
        bn = cand;
      }
    }
    // Few tiles and a deep k (weight gradients): k is split to fill the round anyway, so take the widest tile that
    // divides the width (fewest operand bytes per output).
    if (2 * ceil_div(m, 2 * P_BM) * ceil_div(n, 128) < 148 && k >= 64 * P_BK) bn = n % 256 == 0 ? 256 : n % 192 == 0 ? 192 : 128;
  }
  CUtensorMap map_a, map_b;
  bool ok = a_mn ? pair_map(&map_a, A, m, k, lda, P_BK, true) : pair_map(&map_a, A, k, m, lda, P_BM, false);
  ok = ok && (b_mn ? pair_map(&map_b, B, n, k, ldb, P_BK, true) : pair_map(&map_b, B, k, n, ldb, bn / 2, false));
  if (!ok) return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed (pair kernel, m %d n %d k %d)", m, n, k);
  const int pairs = (int)ceil_div(m, 2 * P_BM), n_tiles = (int)ceil_div(n, bn);
  const int ctas = 2 * pairs * n_tiles, k_blocks = (int)ceil_div(k, P_BK);
  int splits = 1;
  if (ctas < 148 && k_blocks >= 16) {
    splits = (int)std::min<int64_t>(kSplitSlots / ctas, k_blocks / 8);
    if (splits < 1) splits = 1;
    if (splits > 32) splits = 32;
  }
  const int kb_per_split = (int)ceil_div(k_blocks, splits);
  splits = (int)ceil_div(k_blocks, kb_per_split);
  PairParams p;
  p.m = m; p.n = n; p.k = k; p.k_per_split = kb_per_split * P_BK; p.splits = splits; p.status = ctx->status_dev;
  float* workspace = nullptr;
  if (splits > 1) {
    OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)splits * m * n, false, (void**)&workspace));
    p.c = workspace; p.ldc = n; p.accumulate = 0; p.bias = nullptr;
  } else {
    p.c = C; p.ldc = ldc; p.accumulate = acc; p.bias = bias;
  }
  CUtensorMap map_c;
  p.tma_store = splits > 1 ? make_store_map(&map_c, workspace, n, m, n, splits, (long long)m * n, 1, 0)
                           : make_store_map(&map_c, C, n, m, ldc, 1, 0, 1, 0);
  if (!p.tma_store) map_c = map_a;
  dim3 grid((unsigned)(2 * n_tiles), (unsigned)pairs, (unsigned)splits);
  int32_t st = bn == 256   ? launch_pair<256>(ctx, a_mn, b_mn, map_a, map_b, map_c, p, grid)
               : bn == 192 ? launch_pair<192>(ctx, a_mn, b_mn, map_a, map_b, map_c, p, grid)
                           : launch_pair<128>(ctx, a_mn, b_mn, map_a, map_b, map_c, p, grid);
  if (st == OM_OK && splits > 1) splitk_reduce_launch(ctx, workspace, splits, (int64_t)m * n, n, ldc, bias, C, acc);
  if (workspace) pool_free(ctx, workspace);
  return st;
}

}  // namespace om
