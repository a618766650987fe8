// fp32 matrix product on the FMA pipe. Each output element has ONE accumulator that starts at +0 and takes
// fmaf(a[i,k], b[k,j], acc) for k = 0, 1, 2, ... in increasing order: the arithmetic of the reference's blocked
// GEMM (docs/kernels-gemm.md:73-79 and docs/exact-mode.md:28-46 of the reference), so results do not depend on
// the tile shape and are bit-identical to a scalar loop with fused multiply-add. This is the path used when
// the context runs without OM_TF32; the tensor-pipe path lives in om_gemm_tc.cu.
#include "om_common.cuh"

namespace om {

template <int BM, int BN, int BK, int TM, int TN, bool TA, bool TB>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(int m, int n, int k, const float* __restrict__ A, int lda, int64_t strideA,
                 const float* __restrict__ B, int ldb, int64_t strideB, float* __restrict__ C, int ldc,
                 int64_t strideC, int accumulate, int batch, int batch_per_z, int inner, int64_t innerA, int64_t innerB,
                 int64_t innerC) {
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  // batch_per_z == 0: blockIdx.z is the matrix of a batch. Otherwise this CTA sums the products of matrices
  // [z0, z1) into one accumulator (in increasing matrix order) and writes output chunk blockIdx.z.
  const int z0 = batch_per_z ? blockIdx.z * batch_per_z : blockIdx.z;
  const int z1 = batch_per_z ? min(batch, z0 + batch_per_z) : z0 + 1;
  const float* A0 = A;
  const float* B0 = B;
  // Matrix z of an operand starts (z / inner) * stride + (z % inner) * innerStride elements in: inner == 1 is the plain
  // strided batch, inner == heads addresses [batch, length, heads, d] activations per (batch, head) without a copy.
  C += (blockIdx.z / inner) * strideC + (blockIdx.z % inner) * innerC;
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

  for (int z = z0; z < z1; z++) {
  A = A0 + (z / inner) * strideA + (z % inner) * innerA;
  B = B0 + (z / inner) * strideB + (z % inner) * innerB;
  for (int k0 = 0; k0 < k; k0 += BK) {
    // A tile -> As[kk][mm]
    if (TA) {
      // A stored [k, m]: consecutive threads walk m (contiguous).
      for (int e = tid; e < BK * BM; e += THREADS) {
        int kk = e / BM, mm = e % BM;
        int gk = k0 + kk, gm = m0 + mm;
        As[kk][mm] = (gk < k && gm < m) ? A[(int64_t)gk * lda + gm] : 0.f;
      }
    } else {
      // A stored [m, k]: consecutive threads walk k (contiguous).
      for (int e = tid; e < BK * BM; e += THREADS) {
        int mm = e / BK, kk = e % BK;
        int gk = k0 + kk, gm = m0 + mm;
        As[kk][mm] = (gk < k && gm < m) ? A[(int64_t)gm * lda + gk] : 0.f;
      }
    }
    if (TB) {
      // B stored [n, k].
      for (int e = tid; e < BK * BN; e += THREADS) {
        int nn = e / BK, kk = e % BK;
        int gk = k0 + kk, gn = n0 + nn;
        Bs[kk][nn] = (gk < k && gn < n) ? B[(int64_t)gn * ldb + gk] : 0.f;
      }
    } else {
      // B stored [k, n].
      for (int e = tid; e < BK * BN; e += THREADS) {
        int kk = e / BN, nn = e % BN;
        int gk = k0 + kk, gn = n0 + nn;
        Bs[kk][nn] = (gk < k && gn < n) ? B[(int64_t)gk * ldb + gn] : 0.f;
      }
    }
    __syncthreads();
    const int kmax = min(BK, k - k0);
    if (kmax == BK) {
#pragma unroll
      for (int kk = 0; kk < BK; kk++) {
        float a[TM], b[TN];
#pragma unroll
        for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
#pragma unroll
        for (int j = 0; j < TN; j++) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; i++)
#pragma unroll
          for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
    } else {
      // The zero padding of a partial k tile must not enter the sum as fmaf(0, 0, acc): harmless for finite
      // values, but -0 + 0 and NaN/Inf operands would differ from the scalar loop. Stop at the true k.
      for (int kk = 0; kk < kmax; kk++) {
        float a[TM], b[TN];
#pragma unroll
        for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
#pragma unroll
        for (int j = 0; j < TN; j++) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; i++)
#pragma unroll
          for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
    }
    __syncthreads();
  }
  }
#pragma unroll
  for (int i = 0; i < TM; i++) {
    int gm = m0 + ty * TM + i;
    if (gm >= m) continue;
#pragma unroll
    for (int j = 0; j < TN; j++) {
      int gn = n0 + tx * TN + j;
      if (gn >= n) continue;
      float* c = C + (int64_t)gm * ldc + gn;
      *c = accumulate ? *c + acc[i][j] : acc[i][j];
    }
  }
}

template <int BM, int BN, int BK, int TM, int TN>
static void launch_simt(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, int64_t sA,
                        const float* B, int ldb, int64_t sB, float* C, int ldc, int64_t sC, int batch, int acc, int bpz = 0,
                        int inner = 1, int64_t iA = 0, int64_t iB = 0, int64_t iC = 0) {
  dim3 grid((unsigned)ceil_div(n, BN), (unsigned)ceil_div(m, BM), (unsigned)(bpz ? ceil_div(batch, bpz) : batch));
  constexpr int T = (BM / TM) * (BN / TN);
  if (!ta && !tb) gemm_simt_kernel<BM, BN, BK, TM, TN, false, false><<<grid, T, 0, ctx->stream>>>(m, n, k, A, lda, sA, B, ldb, sB, C, ldc, sC, acc, batch, bpz, inner, iA, iB, iC);
  else if (!ta && tb) gemm_simt_kernel<BM, BN, BK, TM, TN, false, true><<<grid, T, 0, ctx->stream>>>(m, n, k, A, lda, sA, B, ldb, sB, C, ldc, sC, acc, batch, bpz, inner, iA, iB, iC);
  else if (ta && !tb) gemm_simt_kernel<BM, BN, BK, TM, TN, true, false><<<grid, T, 0, ctx->stream>>>(m, n, k, A, lda, sA, B, ldb, sB, C, ldc, sC, acc, batch, bpz, inner, iA, iB, iC);
  else gemm_simt_kernel<BM, BN, BK, TM, TN, true, true><<<grid, T, 0, ctx->stream>>>(m, n, k, A, lda, sA, B, ldb, sB, C, ldc, sC, acc, batch, bpz, inner, iA, iB, iC);
}

int32_t gemm_simt_heads(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, int64_t sA, int64_t iA,
                        const float* B, int ldb, int64_t sB, int64_t iB, float* C, int ldc, int64_t sC, int64_t iC, int batch,
                        int inner, int acc) {
  if (m == 0 || n == 0 || batch == 0) return OM_OK;
  if (inner < 1) inner = 1;
  int64_t tiles128 = ceil_div(m, 128) * ceil_div(n, 128) * batch;
  if (tiles128 >= ctx->sm_count) {
    launch_simt<128, 128, 16, 8, 8>(ctx, ta, tb, m, n, k, A, lda, sA, B, ldb, sB, C, ldc, sC, batch, acc, 0, inner, iA, iB, iC);
  } else {
    launch_simt<64, 64, 16, 4, 4>(ctx, ta, tb, m, n, k, A, lda, sA, B, ldb, sB, C, ldc, sC, batch, acc, 0, inner, iA, iB, iC);
  }
  OM_LAUNCH_CHECK(ctx, "gemm_simt");
  return OM_OK;
}

int32_t gemm_simt(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, int64_t sA,
                  const float* B, int ldb, int64_t sB, float* C, int ldc, int64_t sC, int batch, int acc) {
  return gemm_simt_heads(ctx, ta, tb, m, n, k, A, lda, sA, 0, B, ldb, sB, 0, C, ldc, sC, 0, batch, 1, acc);
}

// Sums the products of `batch` matrix pairs in chunks of batch_per_chunk: partial[c] = sum over the chunk's matrices
// of op(A_z) op(B_z), each partial dense [m, n], chunk c at partial + c * chunk_stride.
int32_t gemm_simt_batch_reduce(om_ctx* ctx, int ta, int tb, int m, int n, int k, const float* A, int lda, int64_t sA,
                               const float* B, int ldb, int64_t sB, float* partial, int64_t chunk_stride, int batch,
                               int batch_per_chunk) {
  if (m == 0 || n == 0 || batch == 0) return OM_OK;
  launch_simt<64, 64, 16, 4, 4>(ctx, ta, tb, m, n, k, A, lda, sA, B, ldb, sB, partial, n, chunk_stride, batch, 0, batch_per_chunk);
  OM_LAUNCH_CHECK(ctx, "gemm_simt_batch_reduce");
  return OM_OK;
}

}  // namespace om
