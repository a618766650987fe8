// Whole-sequence LSTM kernels: all T time steps of one or two directions in ONE cooperative launch.
//
// The step-by-step path (om_recurrent.cu) launches a recurrent product and a gate kernel per time step: at the sizes
// of a text-line recogniser (batch 64, hidden 256, 64 frames) each of those ~1000 launches per training step does a
// few microseconds of work and the sequence is bound by launch and dependency latency. Here a CTA owns JU hidden units
// (their four gate rows of W_hh stay in shared memory for the whole sequence), computes for every batch row the
// recurrent dot products of its units with fp32 FMAs, applies the cell, and meets the other CTAs of its direction at
// a grid barrier once per time step. The backward kernel owns the same units: it turns (gy_t + dh, dc) into the gate
// gradients of its units, and after the barrier computes its units' slice of dh = dG_t * W_hh from the complete
// gate-gradient row.
//
// Arithmetic: fp32 throughout (more accurate than the TF32 product of the step-by-step fast path). A dot product is
// split in four k ranges summed in a fixed order, so results do not depend on scheduling; they are not the
// one-accumulator order of the reference's exact tier, which stays on the step-by-step path.
//
// The CTAs of a direction wait on one another, so the launch is cooperative (all CTAs resident at once; the host checks
// the occupancy first) and every wait at the barrier is bounded: after about a second a CTA raises OM_ERR_TIMEOUT in the
// context's status word and returns, and the others follow at their own bound.
#include "om_lstm_seq.cuh"

namespace om {

constexpr int kSeqThreads = 256;
constexpr int kSeqRows = 64;          // batch rows per pass; kSeqThreads = kSeqRows * kSeqSplit
constexpr int kSeqSplit = 4;          // k ranges of one dot product
constexpr int kSeqUnits = 4;          // hidden units per CTA
constexpr int kSeqDepth = 16;         // float4 loads of the previous state in flight per thread
constexpr int kSeqMaxBatch = 256;     // backward keeps dh and dc of its units for all rows in shared memory
constexpr long long kSeqWaitCycles = 2000000000LL;

__device__ __forceinline__ float seq_sigm(float x) { return 1.0f / (1.0f + expf(-x)); }

// Grid barrier of one direction: arrival number `target` completes it. Returns false when the wait ran out.
__device__ __forceinline__ bool seq_barrier(unsigned* counter, unsigned target, int32_t* status, int* failed, int where) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    const long long t0 = clock64();
    for (;;) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
      if (v >= target) break;
      if (clock64() - t0 > kSeqWaitCycles) {
        *failed = 1;
        if (atomicCAS(status, 0, (int32_t)OM_ERR_TIMEOUT) == 0) status[1] = where;
        break;
      }
    }
  }
  __syncthreads();
  return *failed == 0;
}

__global__ void __launch_bounds__(kSeqThreads) lstm_seq_fwd_kernel(const LstmSeqFwdParams p) {
  constexpr int JU = kSeqUnits, NC = 4 * JU;
  extern __shared__ __align__(16) float seq_smem[];
  __shared__ int failed;
  const LstmSeqFwdDir& D = p.d[blockIdx.y];
  const int H = p.h, B = p.b, T = p.t, H4 = 4 * p.h;
  const int j0 = blockIdx.x * JU, tid = threadIdx.x;
  float* ws = seq_smem;                       // [NC][H]: row q*JU + j = W_hh[q*H + j0 + j, :]
  float* red = ws + (size_t)NC * H;           // [kSeqSplit][NC][kSeqRows]
  const int hq = H / 4;
  for (int idx = tid; idx < NC * hq; idx += kSeqThreads) {
    int row = idx / hq, k4 = idx % hq, q = row / JU, j = row % JU;
    reinterpret_cast<float4*>(ws)[idx] = __ldg(reinterpret_cast<const float4*>(D.w_hh + (size_t)(q * H + j0 + j) * H) + k4);
  }
  if (tid == 0) failed = 0;
  __syncthreads();
  const int r = tid % kSeqRows, kq = tid / kSeqRows;   // a warp shares kq: its reads of W are broadcasts
  const int kspan4 = hq / kSeqSplit;                   // float4 per k range
  const size_t bh = (size_t)B * H;
  for (int f = 0; f < T; f++) {
    const int tt = D.reverse ? T - 1 - f : f;
    const int pt = D.reverse ? tt + 1 : tt - 1;
    const float* hp = f == 0 ? D.h0 : D.y + (size_t)pt * bh;
    const float* cp = f == 0 ? D.c0 : D.c + (size_t)pt * bh;
    float* gates_t = D.gates + (size_t)tt * B * H4;
    for (int r0 = 0; r0 < B; r0 += kSeqRows) {
      float acc[NC];
#pragma unroll
      for (int c = 0; c < NC; c++) acc[c] = 0.f;
      const int b = r0 + r;
      if (hp != nullptr && b < B) {
        // h of the previous step was written by other CTAs of this launch: read it past L1.
        const float4* hrow = reinterpret_cast<const float4*>(hp + (size_t)b * H) + kq * kspan4;
        const float4* w4 = reinterpret_cast<const float4*>(ws) + kq * kspan4;
        // All loads of a chunk are issued before the first use: one L2 round trip per 16 float4, not one per float4.
        for (int kc = 0; kc < kspan4; kc += kSeqDepth) {
          float4 hv[kSeqDepth];
#pragma unroll
          for (int u = 0; u < kSeqDepth; u++) hv[u] = kc + u < kspan4 ? __ldcg(hrow + kc + u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < kSeqDepth; u++) {
            if (kc + u < kspan4) {
#pragma unroll
              for (int c = 0; c < NC; c++) {
                const float4 wv = w4[c * hq + kc + u];
                acc[c] = fmaf(hv[u].x, wv.x, acc[c]);
                acc[c] = fmaf(hv[u].y, wv.y, acc[c]);
                acc[c] = fmaf(hv[u].z, wv.z, acc[c]);
                acc[c] = fmaf(hv[u].w, wv.w, acc[c]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int c = 0; c < NC; c++) red[(kq * NC + c) * kSeqRows + r] = acc[c];
      __syncthreads();
      for (int e = tid; e < kSeqRows * JU; e += kSeqThreads) {
        const int rr = e / JU, j = e % JU, bb = r0 + rr;
        if (bb >= B) continue;
        const int jg = j0 + j;
        float* g = gates_t + (size_t)bb * H4;
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const float* rp = red + (q * JU + j) * kSeqRows + rr;
          const float rec = ((rp[0] + rp[NC * kSeqRows]) + rp[2 * NC * kSeqRows]) + rp[3 * NC * kSeqRows];
          float tv = g[q * H + jg] + rec;
          if (D.bias) tv = tv + D.bias[q * H + jg];
          v[q] = tv;
        }
        const float gi = seq_sigm(v[0]), gf = seq_sigm(v[1]), gg = tanhf(v[2]), go = seq_sigm(v[3]);
        g[jg] = gi;
        g[H + jg] = gf;
        g[2 * H + jg] = gg;
        g[3 * H + jg] = go;
        const size_t idx = (size_t)bb * H + jg;
        const float fc = gf * (cp ? __ldcg(cp + idx) : 0.f);
        const float ig = gi * gg;
        const float cn = fc + ig;
        D.c[(size_t)tt * bh + idx] = cn;
        const float tc = tanhf(cn);
        D.tanh_c[(size_t)tt * bh + idx] = tc;
        D.y[(size_t)tt * bh + idx] = go * tc;
      }
      __syncthreads();
    }
    if (f + 1 < T && !seq_barrier(D.counter, (unsigned)(f + 1) * gridDim.x, p.status, &failed, 9100 + (int)blockIdx.y)) return;
  }
}

__global__ void __launch_bounds__(kSeqThreads) lstm_seq_bwd_kernel(const LstmSeqBwdParams p) {
  constexpr int JU = kSeqUnits;
  extern __shared__ __align__(16) float seq_smem[];
  __shared__ int failed;
  const LstmSeqBwdDir& D = p.d[blockIdx.y];
  const int H = p.h, B = p.b, T = p.t, H4 = 4 * p.h;
  const int j0 = blockIdx.x * JU, tid = threadIdx.x;
  float* wcol = seq_smem;                          // [4H][JU]: W_hh[c, j0 + j]
  float* dh_s = wcol + (size_t)H4 * JU;            // [B][JU]
  float* dc_s = dh_s + (size_t)B * JU;             // [B][JU]
  float* red = dc_s + (size_t)B * JU;              // [kSeqSplit][JU][kSeqRows]
  for (int c = tid; c < H4; c += kSeqThreads)
    reinterpret_cast<float4*>(wcol)[c] = __ldg(reinterpret_cast<const float4*>(D.w_hh + (size_t)c * H + j0));
  for (int e = tid; e < B * JU; e += kSeqThreads) {
    const size_t idx = (size_t)(e / JU) * H + j0 + e % JU;
    dh_s[e] = D.ghn ? D.ghn[idx] : 0.f;
    dc_s[e] = D.gcn ? D.gcn[idx] : 0.f;
  }
  if (tid == 0) failed = 0;
  __syncthreads();
  const int r = tid % kSeqRows, kq = tid / kSeqRows;
  const int kspan4 = H4 / 4 / kSeqSplit;           // float4 of the gate-gradient row per k range
  const size_t bh = (size_t)B * H;
  for (int s = 0; s < T; s++) {
    const int tt = D.reverse ? s : T - 1 - s;
    const int pt = D.reverse ? tt + 1 : tt - 1;
    const bool first = D.reverse ? tt == T - 1 : tt == 0;
    const float* cp = first ? D.c0 : D.c + (size_t)pt * bh;
    const float* gates_t = D.gates + (size_t)tt * B * H4;
    float* dg_t = D.dG + (size_t)tt * B * H4;
    // Gate gradients of this CTA's units (BackwardRecurrent.cs:37-57 of the reference, the same operation order).
    for (int e = tid; e < B * JU; e += kSeqThreads) {
      const int bb = e / JU, jg = j0 + e % JU;
      const size_t idx = (size_t)bb * H + jg;
      const float* g = gates_t + (size_t)bb * H4;
      float* d = dg_t + (size_t)bb * H4;
      const float gi = g[jg], gf = g[H + jg], gg = g[2 * H + jg], go = g[3 * H + jg];
      const float tc = D.tanh_c[(size_t)tt * bh + idx];
      const float dH = D.gy[(size_t)tt * bh + idx] + dh_s[e];
      const float dO = dH * tc;
      const float dC = dc_s[e] + ((dH * go) * (1.f - (tc * tc)));
      const float cpv = cp ? cp[idx] : 0.f;
      const float dI = dC * gg, dF = dC * cpv, dGg = dC * gi;
      dc_s[e] = dC * gf;
      d[jg] = (dI * gi) * (1.f - gi);
      d[H + jg] = (dF * gf) * (1.f - gf);
      d[2 * H + jg] = dGg * (1.f - (gg * gg));
      d[3 * H + jg] = (dO * go) * (1.f - go);
    }
    if (s == T - 1 && D.dh0 == nullptr) break;
    if (!seq_barrier(D.counter, (unsigned)(s + 1) * gridDim.x, p.status, &failed, 9200 + (int)blockIdx.y)) return;
    // dh of the next processed step, this CTA's units: dG_t[b, :] . W_hh[:, j]
    for (int r0 = 0; r0 < B; r0 += kSeqRows) {
      float acc[JU];
#pragma unroll
      for (int j = 0; j < JU; j++) acc[j] = 0.f;
      const int b = r0 + r;
      if (b < B) {
        const float4* drow = reinterpret_cast<const float4*>(dg_t + (size_t)b * H4) + kq * kspan4;
        const float4* w4 = reinterpret_cast<const float4*>(wcol) + (size_t)kq * kspan4 * 4;
        for (int kc = 0; kc < kspan4; kc += kSeqDepth) {
          float4 dvs[kSeqDepth];
#pragma unroll
          for (int u = 0; u < kSeqDepth; u++) dvs[u] = kc + u < kspan4 ? __ldcg(drow + kc + u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < kSeqDepth; u++) {
            if (kc + u < kspan4) {
              const int k4 = kc + u;
              const float4 dv = dvs[u];
              const float4 w0 = w4[4 * k4], w1 = w4[4 * k4 + 1], w2 = w4[4 * k4 + 2], w3 = w4[4 * k4 + 3];
              acc[0] = fmaf(dv.x, w0.x, acc[0]); acc[1] = fmaf(dv.x, w0.y, acc[1]); acc[2] = fmaf(dv.x, w0.z, acc[2]); acc[3] = fmaf(dv.x, w0.w, acc[3]);
              acc[0] = fmaf(dv.y, w1.x, acc[0]); acc[1] = fmaf(dv.y, w1.y, acc[1]); acc[2] = fmaf(dv.y, w1.z, acc[2]); acc[3] = fmaf(dv.y, w1.w, acc[3]);
              acc[0] = fmaf(dv.z, w2.x, acc[0]); acc[1] = fmaf(dv.z, w2.y, acc[1]); acc[2] = fmaf(dv.z, w2.z, acc[2]); acc[3] = fmaf(dv.z, w2.w, acc[3]);
              acc[0] = fmaf(dv.w, w3.x, acc[0]); acc[1] = fmaf(dv.w, w3.y, acc[1]); acc[2] = fmaf(dv.w, w3.z, acc[2]); acc[3] = fmaf(dv.w, w3.w, acc[3]);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < JU; j++) red[(kq * JU + j) * kSeqRows + r] = acc[j];
      __syncthreads();
      for (int e = tid; e < kSeqRows * JU; e += kSeqThreads) {
        const int rr = e / JU, j = e % JU, bb = r0 + rr;
        if (bb >= B) continue;
        const float* rp = red + j * kSeqRows + rr;
        dh_s[bb * JU + j] = ((rp[0] + rp[JU * kSeqRows]) + rp[2 * JU * kSeqRows]) + rp[3 * JU * kSeqRows];
      }
      __syncthreads();
    }
  }
  __syncthreads();
  for (int e = tid; e < B * JU; e += kSeqThreads) {
    const size_t idx = (size_t)(e / JU) * H + j0 + e % JU;
    if (D.dh0) D.dh0[idx] = dh_s[e];
    if (D.dc0) D.dc0[idx] = dc_s[e];
  }
}

static_assert(kSeqUnits == 4, "the backward inner loop is written for four units per CTA");
static_assert(kSeqThreads == kSeqRows * kSeqSplit, "thread layout");

static size_t seq_fwd_smem(int h) { return sizeof(float) * ((size_t)4 * kSeqUnits * h + (size_t)kSeqSplit * 4 * kSeqUnits * kSeqRows); }
static size_t seq_bwd_smem(int b, int h) {
  return sizeof(float) * ((size_t)4 * h * kSeqUnits + 2 * (size_t)b * kSeqUnits + (size_t)kSeqSplit * kSeqUnits * kSeqRows);
}

// Shapes the kernels take, and room for all CTAs of `dirs` directions to be resident at once.
bool lstm_seq_supported(om_ctx* ctx, int dirs, int t, int b, int h, bool backward) {
  if (!(ctx->flags & OM_SEQ_KERNELS) || t < 2 || b < 1 || h < 16 || h % 16 != 0) return false;
  if (backward && b > kSeqMaxBatch) return false;
  const size_t smem = backward ? seq_bwd_smem(b, h) : seq_fwd_smem(h);
  if (smem > 200 * 1024) return false;
  const void* fn = backward ? (const void*)lstm_seq_bwd_kernel : (const void*)lstm_seq_fwd_kernel;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kSeqThreads, smem) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return (long long)per_sm * ctx->sm_count >= (long long)dirs * (h / kSeqUnits);
}

static int32_t seq_counters(om_ctx* ctx, unsigned** out) {
  OM_TRY(pool_alloc(ctx, 2 * sizeof(unsigned), true, (void**)out));
  return OM_OK;
}

int32_t lstm_seq_fwd(om_ctx* ctx, int dirs, int t, int b, int h, const LstmSeqFwdDir* d) {
  LstmSeqFwdParams p;
  unsigned* counters = nullptr;
  OM_TRY(seq_counters(ctx, &counters));
  for (int k = 0; k < 2; k++) {
    p.d[k] = d[k < dirs ? k : 0];
    p.d[k].counter = counters + k;
  }
  p.t = t;
  p.b = b;
  p.h = h;
  p.status = ctx->status_dev;
  void* args[] = {&p};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)lstm_seq_fwd_kernel, dim3((unsigned)(h / kSeqUnits), (unsigned)dirs), dim3(kSeqThreads), args,
                                              seq_fwd_smem(h), ctx->stream);
  pool_free(ctx, counters);
  if (e != cudaSuccess) return check_cuda(ctx, e, "lstm_seq_fwd");
  return OM_OK;
}

int32_t lstm_seq_bwd(om_ctx* ctx, int dirs, int t, int b, int h, const LstmSeqBwdDir* d) {
  LstmSeqBwdParams p;
  unsigned* counters = nullptr;
  OM_TRY(seq_counters(ctx, &counters));
  for (int k = 0; k < 2; k++) {
    p.d[k] = d[k < dirs ? k : 0];
    p.d[k].counter = counters + k;
  }
  p.t = t;
  p.b = b;
  p.h = h;
  p.status = ctx->status_dev;
  void* args[] = {&p};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)lstm_seq_bwd_kernel, dim3((unsigned)(h / kSeqUnits), (unsigned)dirs), dim3(kSeqThreads), args,
                                              seq_bwd_smem(b, h), ctx->stream);
  pool_free(ctx, counters);
  if (e != cudaSuccess) return check_cuda(ctx, e, "lstm_seq_bwd");
  return OM_OK;
}

}  // namespace om
