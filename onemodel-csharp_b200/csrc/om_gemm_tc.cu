// Matrix product on the Blackwell tensor pipe: tcgen05.mma with TF32 operands read from shared memory, fp32
// accumulators in tensor memory (TMEM), operand tiles brought in by TMA (cp.async.bulk.tensor, 128-byte swizzle, no
// multicast) through a ring of mbarrier-guarded stages.
//
// One CTA computes one 128 x 128 tile of C (optionally one k-slice of it: fixed split-k with an ordered second pass,
// no floating-point atomics). Warp roles: warp 0 issues TMA loads, warp 1 owns the TMEM allocation and issues the
// MMAs (one elected thread), warps 2-5 read the accumulator back (tcgen05.ld) and write C.
//
// All four operand orientations run without a transposed copy: an operand whose contraction index k is contiguous in
// memory is a "K-major" tile, one whose m (or n) index is contiguous is an "MN-major" tile; the shared-memory matrix
// descriptor and the instruction descriptor's major bits tell the tensor core which one it is reading.
//   forward  y = x W^T      : A K-major,  B K-major
//   dgrad    dx = g W       : A K-major,  B MN-major
//   wgrad    dW = g^T x     : A MN-major, B MN-major
//
// Every wait on an mbarrier is bounded: when the bound is hit the kernel raises OM_ERR_TIMEOUT in the context's status
// word, every role leaves its loop, TMEM is released and the kernel returns.
#include "om_tc.cuh"

namespace om {

constexpr int BM = 128, BN = 128, BK = 32;       // BK fp32 elements = one 128-byte swizzle row
constexpr int STAGES = 3;                        // 96 KiB of operand tiles: two CTAs per SM, one's epilogue under the other's MMAs
constexpr int UMMA_K = 8;                        // tf32: 32 bytes of k per instruction
constexpr int A_TILE_BYTES = BM * BK * 4;        // 16 KiB
constexpr int B_TILE_BYTES = BN * BK * 4;
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int TC_THREADS = 192;
constexpr int TMEM_COLS = 128;
constexpr size_t TC_SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;

struct TcParams {
  int tma_store;        // the epilogue writes C through map_c (C and its pitches are 16-byte aligned)
  int m, n, k;
  int k_per_split;      // multiple of BK
  int splits;
  float* c;             // C (splits == 1) or the partial workspace [splits][m][n]
  int ldc;
  int accumulate;       // only when splits == 1
  const float* bias;    // only when splits == 1
  int32_t* status;
  int batched;          // blockIdx.z is a matrix of a strided batch (then splits == 1)
  int inner;            // matrix z sits at outer index z / inner, inner index z % inner (1 = plain strided batch)
  long long stride_c;   // elements between the C matrices of consecutive outer indices
  long long inner_c;    // ... and of consecutive inner indices
};

// Instruction descriptor for kind::tf32: fp32 accumulator, TF32 A and B, major bits, N >> 3, M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_tf32(bool a_mn, bool b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}

// ---- the kernel -------------------------------------------------------------------------------------------------------
// A_MN / B_MN: the operand tile is MN-major (its m / n index is contiguous in global memory).
// K-major tile in shared memory : 128 rows (m or n) x 128 bytes of k, 8-row swizzle atoms 1024 bytes apart.
// MN-major tile in shared memory: 4 chunks of [BK k-rows x 128 bytes of m/n]; chunks BK*128 bytes apart (leading
//                                 offset), 4-row k groups (the 32-byte-unit swizzle atom) 512 bytes apart (stride
//                                 offset); one MMA consumes 8 k-rows = 1024 bytes.
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(TC_THREADS, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int split = p.batched ? 0 : blockIdx.z;
  const int zb = p.batched ? blockIdx.z : 0;
  const int zo = zb / p.inner, zi = zb % p.inner;
  const int k_begin = split * p.k_per_split;
  const int k_end = min(p.k, k_begin + p.k_per_split);
  const int k_blocks = (k_end - k_begin + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // The CTA holds its tensor memory: later kernels of the stream may become resident now, and everything from here on
  // (operand loads, bias, C) may depend on the previous kernel.
  pdl_trigger();
  pdl_wait();

  if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      for (int kb = 0; kb < k_blocks; kb++) {
        const int s = kb % STAGES;
        const uint32_t round = kb / STAGES;
        if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, abort_flag, p.status, 1)) break;
        uint8_t* a_dst = smem + (size_t)s * STAGE_BYTES;
        uint8_t* b_dst = a_dst + A_TILE_BYTES;
        const int k0 = k_begin + kb * BK;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        if (A_MN) {
#pragma unroll
          for (int j = 0; j < BM / 32; j++) tma_load_4d(a_dst + j * (BK * 128), &map_a, m0 + 32 * j, k0, zi, zo, &full[s]);
        } else {
          tma_load_4d(a_dst, &map_a, k0, m0, zi, zo, &full[s]);
        }
        if (B_MN) {
#pragma unroll
          for (int j = 0; j < BN / 32; j++) tma_load_4d(b_dst + j * (BK * 128), &map_b, n0 + 32 * j, k0, zi, zo, &full[s]);
        } else {
          tma_load_4d(b_dst, &map_b, k0, n0, zi, zo, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_tf32(A_MN, B_MN);
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; kb++) {
        const int s = kb % STAGES;
        const uint32_t round = kb / STAGES;
        ok = mbar_wait(&full[s], round & 1, abort_flag, p.status, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
        const uint32_t b_addr = a_addr + A_TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < BK / UMMA_K; ks++) {
          // K-major: step 32 bytes along the swizzled row. MN-major: step one 8-row k group (1024 bytes).
          const uint64_t adesc = A_MN ? make_desc(a_addr + ks * 1024, BK * 128, 512, 1) : make_desc(a_addr + ks * (UMMA_K * 4), 16, 1024, 2);
          const uint64_t bdesc = B_MN ? make_desc(b_addr + ks * 1024, BK * 128, 512, 1) : make_desc(b_addr + ks * (UMMA_K * 4), 16, 1024, 2);
          umma_tf32(tmem_base, adesc, bdesc, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);   // frees the stage when these MMAs have read it
      }
      umma_commit(acc_full);      // accumulator complete (or nothing outstanding after an abort)
    }
  } else {
    // ---- epilogue: warps 2..5 own TMEM lane quadrants (warp % 4) ----
    // tcgen05.ld hands lane l the 32 columns of accumulator row l. Storing from there would make every warp store touch
    // 32 different rows (16 bytes each); instead each 32 x 32 block is turned through shared memory (the operand stages are
    // dead once acc_full has fired) so that eight lanes cover one 128-byte row segment and a warp store writes four full
    // row segments.
    const int quad = warp & 3;
    bool ok = true;
    if (k_blocks > 0) ok = mbar_wait(acc_full, 0, abort_flag, p.status, 3);
    tc_fence_after();
    float* c = p.c + (size_t)split * p.m * p.ldc + (size_t)zo * p.stride_c + (size_t)zi * p.inner_c;
    constexpr int STG_LD = 36;                                   // floats per staged row: 144 bytes keeps float4 alignment and
    float* stg = reinterpret_cast<float*>(smem) + quad * 32 * STG_LD;   // spreads the eight rows of a phase over all banks
    const int row_base = m0 + quad * 32;
    const bool aligned = ((reinterpret_cast<uintptr_t>(c) & 15) == 0) && ((p.ldc & 3) == 0);
    if (ok && row_base < p.m && p.tma_store) {
      // Bulk stores: each 32 x 32 block goes to its own 4 KB of the (dead) operand stages in the 128-byte-swizzled layout
      // of the C tensor map (16-byte chunk c of row r at chunk c ^ (r & 7): a quarter warp writes 128 distinct bytes),
      // and one lane hands it to the TMA unit, which writes full rows, clips the ragged edges of C and, when the product
      // accumulates, adds in place of storing. The warp does not wait for a block before it reads the next one from TMEM.
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
        uint8_t* blk = smem + (size_t)(quad * (BN / 32) + cb) * 4096;
        const uint32_t row_addr = smem_u32(blk) + (uint32_t)lane * 128u;
#pragma unroll
        for (int c4 = 0; c4 < 8; c4++)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (uint32_t)((c4 ^ (lane & 7)) << 4)), "r"(r[4 * c4]),
                       "r"(r[4 * c4 + 1]), "r"(r[4 * c4 + 2]), "r"(r[4 * c4 + 3])
                       : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          const int z2 = p.batched ? zi : split, z3 = p.batched ? zo : 0;
          if (p.accumulate)
            asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(&map_c),
                         "r"(col0), "r"(row_base), "r"(z2), "r"(z3), "r"(smem_u32(blk))
                         : "memory");
          else
            asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(&map_c), "r"(col0),
                         "r"(row_base), "r"(z2), "r"(z3), "r"(smem_u32(blk))
                         : "memory");
        }
      }
      if (lane == 0) {
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory may go once the copies have read it
      }
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
          const int cc = (lane & 7) * 4;                         // this lane's four columns of the block
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
          // Ragged right edge or an unaligned C: lane l owns column l of the block, one row per step.
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// out = (accumulate ? out : 0) + part[0] + part[1] + ... in increasing split order.
// The split sums are formed first, then bias and the previous contents are added, as the unsplit epilogue does.
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int splits, int64_t mn, int n, int64_t ldc,
                                     const float* __restrict__ bias, float* __restrict__ out, int accumulate) {
  pdl_enter();
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < mn; j += stride) {
    float acc = part[j];
    for (int s = 1; s < splits; s++) acc += part[(int64_t)s * mn + j];
    int64_t o = (j / n) * ldc + (j % n);
    if (bias) acc += bias[j % n];
    if (accumulate) acc += out[o];
    out[o] = acc;
  }
}

// ---- host side -----------------------------------------------------------------------------------------------------------
// A rank-4 fp32 tensor map over row-major matrices [outer, inner] with leading dimension ld, box [box_outer, 32]:
// dimension 2 walks the `inner_count` matrices that lie inner_stride elements apart, dimension 3 the `outer_count`
// groups outer_stride apart (a plain matrix has both counts 1; a strided batch has inner_count 1; activations laid out
// [batch, length, heads, d] are addressed per (batch, head) with inner = heads). Strides need not be ordered.
// K-major tiles use the 16-byte-unit 128B swizzle, MN-major tiles the 32-byte-unit one. The TFLOAT32 element type makes
// TMA round each value to TF32 (nearest even) on the way in; the tensor core would otherwise truncate the low 13 bits.
static bool make_map(CUtensorMap* map, const float* base, int inner, int outer, int ld, int box_outer, bool mn_major,
                     int outer_count = 1, long long outer_stride = 0, int inner_count = 1, long long inner_stride = 0) {
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)inner_count, (cuuint64_t)outer_count};
  // Strides of dimensions of extent 1 are never used for addressing but must still be multiples of 16 bytes.
  cuuint64_t fallback = (((cuuint64_t)ld * outer * 4) + 15) & ~(cuuint64_t)15;
  if (fallback < 16) fallback = 16;
  cuuint64_t strides[3] = {(cuuint64_t)ld * 4, inner_count > 1 ? (cuuint64_t)inner_stride * 4 : fallback,
                           outer_count > 1 ? (cuuint64_t)outer_stride * 4 : fallback};
  cuuint32_t box[4] = {32, (cuuint32_t)box_outer, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The map the epilogue stores through: C as [outer_count, inner_count, m, n] fp32 with box [32 rows, 32 columns] in the
// 16-byte-unit 128B swizzle. Fails (and the kernel then stores with ordinary instructions) when C or a pitch is not a
// multiple of 16 bytes.
bool make_store_map(CUtensorMap* map, float* base, int n, int m, long long ld, int inner_count, long long inner_stride,
                           int outer_count, long long outer_stride) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld & 3) || ld < n) return false;
  if (inner_count > 1 && ((inner_stride & 3) || inner_stride <= 0)) return false;
  if (outer_count > 1 && ((outer_stride & 3) || outer_stride <= 0)) return false;
  cuuint64_t dims[4] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)inner_count, (cuuint64_t)outer_count};
  cuuint64_t fallback = (((cuuint64_t)ld * m * 4) + 15) & ~(cuuint64_t)15;
  if (fallback < 16) fallback = 16;
  cuuint64_t strides[3] = {(cuuint64_t)ld * 4, inner_count > 1 ? (cuuint64_t)inner_stride * 4 : fallback,
                           outer_count > 1 ? (cuuint64_t)outer_stride * 4 : fallback};
  cuuint32_t box[4] = {32, 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool gemm_tc_supported(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B, int ldb,
                       const float* C, int ldc) {
  (void)ctx; (void)ta; (void)tb; (void)C; (void)ldc;
  if (!(ctx->flags & OM_TF32)) return false;
  if (!encode_fn()) return false;
  if (m < 1 || n < 1 || k < 1) return false;
  if ((lda & 3) || (ldb & 3)) return false;                                    // TMA: row pitch multiple of 16 bytes
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return false;
  if ((double)m * n * k < 32.0 * 32 * 32) return false;                        // tiny products stay on the FMA kernel
  return true;
}

int32_t gemm_tc_batched(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA, const float* B,
                        int ldb, long long sB, float* C, int ldc, long long sC, int batch, int acc, const float* bias);

int32_t gemm_tc(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B, int ldb, float* C,
                int ldc, int acc, const float* bias) {
  return gemm_tc_batched(ctx, ta, tb, m, n, k, A, lda, 0, B, ldb, 0, C, ldc, 0, 1, acc, bias);
}

// Batched products. Matrix z of an operand starts (z / inner) * s + (z % inner) * i elements in: inner == 1 is the
// plain strided batch (stride s), inner == heads addresses [batch, length, heads, d] activations per (batch, head)
// in place. The batch rides on blockIdx.z, so a batched product never splits k.
bool gemm_tc_heads_supported(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA, long long iA,
                             const float* B, int ldb, long long sB, long long iB, int batch, int inner) {
  if (!gemm_tc_supported(ctx, ta, tb, m, n, k, A, lda, B, ldb, nullptr, 0)) return false;
  if (batch < 1 || batch > 65535 || inner < 1 || batch % inner != 0) return false;
  if (batch / inner > 1 && ((sA & 3) || (sB & 3) || sA <= 0 || sB <= 0)) return false;
  if (inner > 1 && ((iA & 3) || (iB & 3) || iA <= 0 || iB <= 0)) return false;
  return true;
}

bool gemm_tc_batched_supported(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA,
                               const float* B, int ldb, long long sB, int batch) {
  return gemm_tc_heads_supported(ctx, ta, tb, m, n, k, A, lda, sA, 0, B, ldb, sB, 0, batch, 1);
}

int32_t gemm_tc_heads(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA, long long iA,
                      const float* B, int ldb, long long sB, long long iB, float* C, int ldc, long long sC, long long iC, int batch,
                      int inner, int acc, const float* bias);

int32_t gemm_tc_batched(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA, const float* B,
                        int ldb, long long sB, float* C, int ldc, long long sC, int batch, int acc, const float* bias) {
  return gemm_tc_heads(ctx, ta, tb, m, n, k, A, lda, sA, 0, B, ldb, sB, 0, C, ldc, sC, 0, batch, 1, acc, bias);
}

bool gemm_pair_supported(om_ctx* ctx, int m, int n, int k);
bool gemm_ws_supported(om_ctx* ctx, int elem, int m, int n, int k, const void* A, long long lda, const void* B, long long ldb, const float* C,
                       long long ldc);
int32_t gemm_ws(om_ctx* ctx, int elem, int ta, int tb, int m, int n, int k, const void* A, long long lda, const void* B, long long ldb, float* C,
                long long ldc, int acc, const float* bias, uint16_t* C16);
int32_t gemm_pair(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, const float* B, int ldb, float* C, int ldc,
                  int acc, const float* bias);

void splitk_reduce_launch(om_ctx* ctx, const float* part, int splits, int64_t mn, int n, int64_t ldc, const float* bias, float* out, int accumulate) {
  launch_chained(ctx, splitk_reduce_kernel, grid_for(ctx, mn, 256), 256, 0, part, splits, mn, n, ldc, bias, out, accumulate);
}

int32_t gemm_tc_heads(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, long long sA, long long iA,
                      const float* B, int ldb, long long sB, long long iB, float* C, int ldc, long long sC, long long iC, int batch,
                      int inner, int acc, const float* bias) {
  if (batch == 1 && (ctx->flags & OM_PERSISTENT_TILES) && m >= 256 && n >= 64 && gemm_ws_supported(ctx, 0, m, n, k, A, lda, B, ldb, C, ldc))
    return gemm_ws(ctx, 0, ta, tb, m, n, k, A, lda, B, ldb, C, ldc, acc, bias, nullptr);
  if (batch == 1 && gemm_pair_supported(ctx, m, n, k)) return gemm_pair(ctx, ta, tb, m, n, k, A, lda, B, ldb, C, ldc, acc, bias);
  // op(A) is [m, k]. ta == 0: stored [m, k] (K-major tile, map inner = k). ta != 0: stored [k, m] (MN-major, inner = m).
  // op(B) is [k, n]. tb != 0: stored [n, k] (K-major, inner = k). tb == 0: stored [k, n] (MN-major, inner = n).
  const bool a_mn = ta != 0, b_mn = tb == 0;
  const int outer = batch / inner;
  CUtensorMap map_a, map_b;
  bool ok = a_mn ? make_map(&map_a, A, m, k, lda, BK, true, outer, sA, inner, iA) : make_map(&map_a, A, k, m, lda, BM, false, outer, sA, inner, iA);
  ok = ok && (b_mn ? make_map(&map_b, B, n, k, ldb, BK, true, outer, sB, inner, iB) : make_map(&map_b, B, k, n, ldb, BN, false, outer, sB, inner, iB));
  if (!ok) return fail(ctx, OM_ERR_CUDA, "cuTensorMapEncodeTiled failed (m %d n %d k %d lda %d ldb %d)", m, n, k, lda, ldb);

  const int tiles = (int)(ceil_div(m, BM) * ceil_div(n, BN));
  const int k_blocks = (int)ceil_div(k, BK);
  // Fixed split of k: slices for one full round of CTAs, each slice at least 8 k-blocks deep. The split count is
  // a function of the shape only, so results do not depend on the device or on timing.
  int splits = 1;
  if (batch == 1 && tiles < 148 && k_blocks >= 16) {
    // As many slices as still run in one round of two CTAs per SM on a 148-SM device (a constant, not the device's count).
    splits = (int)std::min<int64_t>(kSplitSlots / tiles, k_blocks / 8);
    if (splits < 1) splits = 1;
    if (splits > 32) splits = 32;
  }
  const int kb_per_split = (int)ceil_div(k_blocks, splits);
  splits = (int)ceil_div(k_blocks, kb_per_split);

  TcParams p;
  p.m = m; p.n = n; p.k = k;
  p.k_per_split = kb_per_split * BK;
  p.splits = splits;
  p.status = ctx->status_dev;
  p.batched = batch > 1;
  p.inner = inner;
  p.stride_c = sC;
  p.inner_c = iC;
  float* workspace = nullptr;
  if (splits > 1) {
    OM_TRY(pool_alloc(ctx, sizeof(float) * (size_t)splits * m * n, false, (void**)&workspace));
    p.c = workspace; p.ldc = n; p.accumulate = 0; p.bias = nullptr;
  } else {
    p.c = C; p.ldc = ldc; p.accumulate = acc; p.bias = bias;
  }
  CUtensorMap map_c;
  p.tma_store = splits > 1 ? make_store_map(&map_c, workspace, n, m, n, splits, (long long)m * n, 1, 0)
                           : make_store_map(&map_c, C, n, m, ldc, inner, iC, outer, sC);
  if (!p.tma_store) map_c = map_a;   // never used, but the parameter must hold a valid map
  dim3 grid((unsigned)ceil_div(n, BN), (unsigned)ceil_div(m, BM), (unsigned)(batch > 1 ? batch : splits));
#define OM_TC_LAUNCH(AMN, BMN)                                                                                         \
  do {                                                                                                                 \
    static bool attr_set = false;                                                                                      \
    if (!attr_set) {                                                                                                   \
      OM_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<AMN, BMN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM)); \
      attr_set = true;                                                                                                 \
    }                                                                                                                  \
    launch_chained(ctx, gemm_tc_kernel<AMN, BMN>, grid, TC_THREADS, TC_SMEM, map_a, map_b, map_c, p);                    \
  } while (0)
  if (!a_mn && !b_mn) OM_TC_LAUNCH(false, false);
  else if (!a_mn && b_mn) OM_TC_LAUNCH(false, true);
  else if (a_mn && !b_mn) OM_TC_LAUNCH(true, false);
  else OM_TC_LAUNCH(true, true);
#undef OM_TC_LAUNCH
  OM_LAUNCH_CHECK(ctx, "gemm_tc");
  if (splits > 1) {
    int64_t mn = (int64_t)m * n;
    launch_chained(ctx, splitk_reduce_kernel, grid_for(ctx, mn, 256), 256, 0, workspace, splits, mn, n, ldc, bias, C, acc);
    pool_free(ctx, workspace);
    OM_LAUNCH_CHECK(ctx, "splitk_reduce");
  }
  return OM_OK;
}

}  // namespace om
