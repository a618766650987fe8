// Whole-sequence LSTM kernels: all T time steps of one or two directions in ONE cooperative launch.
//
// The step-by-step path (om_recurrent.cu) launches a recurrent product and a gate kernel per time step: at the sizes
// of a text-line recogniser (batch 64, hidden 256, 64 frames) each of those ~1000 launches per training step does a
// few microseconds of work and the sequence is bound by launch and dependency latency. Here the work of a step is
// tiled over CTAs as (16 hidden units) x (a group of batch rows): a CTA keeps the rows (forward) or columns (backward)
// of W_hh that belong to its units in shared memory for the whole sequence, and per step brings in only the previous
// state (forward: h, 16 rows x H) or the gate gradients (backward: 16 rows x 4H) of its own batch rows, computes with
// fp32 FMAs from shared memory, applies the cell, and meets the CTAs that share its batch rows (the other unit slices)
// at a barrier, once per time step. CTAs of different row groups and directions never wait for one another.
//
// Arithmetic: fp32 throughout (more accurate than the TF32 product of the step-by-step fast path). A dot product is
// split in two (forward) or eight (backward) k ranges summed in a fixed order, so results do not depend on scheduling;
// they are not the one-accumulator order of the reference's exact tier, which stays on the step-by-step path.
//
// CTAs wait on one another, so the launch is cooperative (all CTAs resident at once; the host checks the occupancy
// first) and every wait at the barrier is bounded: after about a second a CTA raises OM_ERR_TIMEOUT in the context's
// status word and returns, and the others follow at their own bound.
#include "om_lstm_seq.cuh"

namespace om {

constexpr int kSeqThreads = 256;
constexpr int kSeqRows = 16;          // batch rows per pass
constexpr int kSeqUnits = 16;         // hidden units per CTA
constexpr int kSeqMaxGroups = 16;     // row groups (barrier counters) per direction
constexpr int kSeqPad = 4;            // floats of padding per shared-memory row: rows land on different banks
constexpr long long kSeqWaitCycles = 2000000000LL;

__device__ __forceinline__ float seq_sigm(float x) { return 1.0f / (1.0f + expf(-x)); }

// Barrier of one (direction, row group): arrival number `target` completes it. Returns false when the wait ran out.
__device__ __forceinline__ bool seq_barrier(unsigned* counter, unsigned target, int32_t* status, int* failed, int where) {
  __syncthreads();
  if (threadIdx.x == 0) {
    // Release at device scope: the CTA's writes (ordered before this thread by the barrier above) are visible to whoever
    // observes the count.
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
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

// Forward. Grid (H / 16, row groups, directions). Shared memory: ws [64][H + 4] (row q * 16 + j = W_hh[q * H + j0 + j, :]),
// hs [16][H + 4] (previous h of the pass's rows), red [128][8] (the upper k half's partial sums).
// Threads: k half = tid / 128; within a half, row pair = (tid % 128) / 16, unit = tid % 16: a thread forms the four gate
// dot products of one unit for two batch rows over its half of k; the lower half then adds the upper half's sums and
// applies the cell to its two (row, unit) elements.
__global__ void __launch_bounds__(kSeqThreads) lstm_seq_fwd_kernel(const LstmSeqFwdParams p) {
  extern __shared__ __align__(16) float seq_smem[];
  __shared__ int failed;
  const LstmSeqFwdDir& D = p.d[blockIdx.z];
  const int H = p.h, B = p.b, T = p.t, H4 = 4 * p.h, ldw = p.h + kSeqPad;
  const int j0 = blockIdx.x * kSeqUnits, tid = threadIdx.x;
  const int group_rows = p.passes * kSeqRows, row_base = blockIdx.y * group_rows;
  float* ws = seq_smem;
  float* hs = ws + (size_t)64 * ldw;
  float* red = hs + (size_t)kSeqRows * ldw;
  const int hq = H / 4;
  for (int idx = tid; idx < 64 * hq; idx += kSeqThreads) {
    const int row = idx / hq, k4 = idx % hq, q = row / kSeqUnits, j = row % kSeqUnits;
    *reinterpret_cast<float4*>(ws + (size_t)row * ldw + 4 * k4) = __ldg(reinterpret_cast<const float4*>(D.w_hh + (size_t)(q * H + j0 + j) * H) + k4);
  }
  if (tid == 0) failed = 0;
  __syncthreads();
  const int half = tid >> 7, rp = (tid & 127) >> 4, cg = tid & 15;
  const int kspan4 = hq / 2;
  const size_t bh = (size_t)B * H;
  unsigned* counter = D.counter + blockIdx.y;
  const int jg = j0 + cg;
  float bias[4] = {0.f, 0.f, 0.f, 0.f};
  if (D.bias != nullptr)
    for (int q = 0; q < 4; q++) bias[q] = D.bias[q * H + jg];
  for (int f = 0; f < T; f++) {
    const int tt = D.reverse ? T - 1 - f : f;
    const int pt = D.reverse ? tt + 1 : tt - 1;
    const float* hp = f == 0 ? D.h0 : D.y + (size_t)pt * bh;
    const float* cp = f == 0 ? D.c0 : D.c + (size_t)pt * bh;
    float* gates_t = D.gates + (size_t)tt * B * H4;
    for (int pass = 0; pass < p.passes; pass++) {
      const int r0 = row_base + pass * kSeqRows;
      if (r0 >= B) break;
      // The cell's own inputs do not depend on the other CTAs: issue their loads before the dot products.
      float pre[2][4], cprev[2];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        cprev[u] = 0.f;
#pragma unroll
        for (int q = 0; q < 4; q++) pre[u][q] = 0.f;
      }
      if (half == 0) {
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int b = r0 + 2 * rp + u;
          if (b < B) {
#pragma unroll
            for (int q = 0; q < 4; q++) pre[u][q] = gates_t[(size_t)b * H4 + q * H + jg];
            if (cp != nullptr) cprev[u] = __ldcg(cp + (size_t)b * H + jg);
          }
        }
      }
      float acc[2][4];
#pragma unroll
      for (int u = 0; u < 2; u++)
#pragma unroll
        for (int q = 0; q < 4; q++) acc[u][q] = 0.f;
      if (hp != nullptr) {
        // h of the previous step was written by other CTAs of this launch: read it past L1, into shared memory.
        for (int idx = tid; idx < kSeqRows * hq; idx += kSeqThreads) {
          const int r = idx / hq, k4 = idx % hq, b = r0 + r;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (b < B) v = __ldcg(reinterpret_cast<const float4*>(hp + (size_t)b * H) + k4);
          *reinterpret_cast<float4*>(hs + (size_t)r * ldw + 4 * k4) = v;
        }
        __syncthreads();
        const float4* h0p = reinterpret_cast<const float4*>(hs + (size_t)(2 * rp) * ldw) + half * kspan4;
        const float4* h1p = reinterpret_cast<const float4*>(hs + (size_t)(2 * rp + 1) * ldw) + half * kspan4;
        const float4* w0p = reinterpret_cast<const float4*>(ws + (size_t)(0 * kSeqUnits + cg) * ldw) + half * kspan4;
        const float4* w1p = reinterpret_cast<const float4*>(ws + (size_t)(1 * kSeqUnits + cg) * ldw) + half * kspan4;
        const float4* w2p = reinterpret_cast<const float4*>(ws + (size_t)(2 * kSeqUnits + cg) * ldw) + half * kspan4;
        const float4* w3p = reinterpret_cast<const float4*>(ws + (size_t)(3 * kSeqUnits + cg) * ldw) + half * kspan4;
#pragma unroll 4
        for (int k4 = 0; k4 < kspan4; k4++) {
          const float4 a0 = h0p[k4], a1 = h1p[k4];
          float4 w = w0p[k4];
          acc[0][0] = fmaf(a0.x, w.x, acc[0][0]); acc[0][0] = fmaf(a0.y, w.y, acc[0][0]); acc[0][0] = fmaf(a0.z, w.z, acc[0][0]); acc[0][0] = fmaf(a0.w, w.w, acc[0][0]);
          acc[1][0] = fmaf(a1.x, w.x, acc[1][0]); acc[1][0] = fmaf(a1.y, w.y, acc[1][0]); acc[1][0] = fmaf(a1.z, w.z, acc[1][0]); acc[1][0] = fmaf(a1.w, w.w, acc[1][0]);
          w = w1p[k4];
          acc[0][1] = fmaf(a0.x, w.x, acc[0][1]); acc[0][1] = fmaf(a0.y, w.y, acc[0][1]); acc[0][1] = fmaf(a0.z, w.z, acc[0][1]); acc[0][1] = fmaf(a0.w, w.w, acc[0][1]);
          acc[1][1] = fmaf(a1.x, w.x, acc[1][1]); acc[1][1] = fmaf(a1.y, w.y, acc[1][1]); acc[1][1] = fmaf(a1.z, w.z, acc[1][1]); acc[1][1] = fmaf(a1.w, w.w, acc[1][1]);
          w = w2p[k4];
          acc[0][2] = fmaf(a0.x, w.x, acc[0][2]); acc[0][2] = fmaf(a0.y, w.y, acc[0][2]); acc[0][2] = fmaf(a0.z, w.z, acc[0][2]); acc[0][2] = fmaf(a0.w, w.w, acc[0][2]);
          acc[1][2] = fmaf(a1.x, w.x, acc[1][2]); acc[1][2] = fmaf(a1.y, w.y, acc[1][2]); acc[1][2] = fmaf(a1.z, w.z, acc[1][2]); acc[1][2] = fmaf(a1.w, w.w, acc[1][2]);
          w = w3p[k4];
          acc[0][3] = fmaf(a0.x, w.x, acc[0][3]); acc[0][3] = fmaf(a0.y, w.y, acc[0][3]); acc[0][3] = fmaf(a0.z, w.z, acc[0][3]); acc[0][3] = fmaf(a0.w, w.w, acc[0][3]);
          acc[1][3] = fmaf(a1.x, w.x, acc[1][3]); acc[1][3] = fmaf(a1.y, w.y, acc[1][3]); acc[1][3] = fmaf(a1.z, w.z, acc[1][3]); acc[1][3] = fmaf(a1.w, w.w, acc[1][3]);
        }
      }
      if (half == 1) {
        float* dst = red + (size_t)(tid & 127) * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(acc[0][0], acc[0][1], acc[0][2], acc[0][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[1][0], acc[1][1], acc[1][2], acc[1][3]);
      }
      __syncthreads();
      if (half == 0) {
        const float* src = red + (size_t)tid * 8;
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int b = r0 + 2 * rp + u;
          if (b >= B) continue;
          float v[4];
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const float rec = acc[u][q] + src[u * 4 + q];
            float tv = pre[u][q] + rec;
            if (D.bias != nullptr) tv = tv + bias[q];
            v[q] = tv;
          }
          const float gi = seq_sigm(v[0]), gf = seq_sigm(v[1]), gg = tanhf(v[2]), go = seq_sigm(v[3]);
          float* g = gates_t + (size_t)b * H4;
          g[jg] = gi;
          g[H + jg] = gf;
          g[2 * H + jg] = gg;
          g[3 * H + jg] = go;
          const size_t idx = (size_t)b * H + jg;
          const float fc = gf * cprev[u];
          const float ig = gi * gg;
          const float cn = fc + ig;
          D.c[(size_t)tt * bh + idx] = cn;
          const float tc = tanhf(cn);
          D.tanh_c[(size_t)tt * bh + idx] = tc;
          D.y[(size_t)tt * bh + idx] = go * tc;
        }
      }
      __syncthreads();   // hs and red are reused by the next pass
    }
    if (f + 1 < T && !seq_barrier(counter, (unsigned)(f + 1) * gridDim.x, p.status, &failed, 9100 + (int)blockIdx.z)) return;
  }
}

// Backward. Grid as forward. Shared memory: wcol [4H][16] (W_hh[c, j0 .. j0 + 15]), ds [16][4H + 4] (the gate gradients
// of the pass's rows), red [8][16][16], dh_s and dc_s [group rows][16] (the state gradients of this CTA's units).
// Threads for the product: k eighth = tid / 32; within it row pair = (tid % 32) / 4, unit quad = tid % 4: two rows x four
// units over an eighth of the 4H gate columns. Threads for the cell: row = tid / 16, unit = tid % 16.
__global__ void __launch_bounds__(kSeqThreads) lstm_seq_bwd_kernel(const LstmSeqBwdParams p) {
  extern __shared__ __align__(16) float seq_smem[];
  __shared__ int failed;
  const LstmSeqBwdDir& D = p.d[blockIdx.z];
  const int H = p.h, B = p.b, T = p.t, H4 = 4 * p.h, ldd = 4 * p.h + kSeqPad;
  const int j0 = blockIdx.x * kSeqUnits, tid = threadIdx.x;
  const int group_rows = p.passes * kSeqRows, row_base = blockIdx.y * group_rows;
  float* wcol = seq_smem;
  float* ds = wcol + (size_t)H4 * kSeqUnits;
  float* red = ds + (size_t)kSeqRows * ldd;
  float* dh_s = red + 8 * kSeqRows * kSeqUnits;
  float* dc_s = dh_s + (size_t)group_rows * kSeqUnits;
  for (int idx = tid; idx < H4 * 4; idx += kSeqThreads) {
    const int c = idx >> 2, part = idx & 3;
    *reinterpret_cast<float4*>(wcol + (size_t)c * kSeqUnits + 4 * part) = __ldg(reinterpret_cast<const float4*>(D.w_hh + (size_t)c * H + j0) + part);
  }
  for (int e = tid; e < group_rows * kSeqUnits; e += kSeqThreads) {
    const int b = row_base + e / kSeqUnits;
    const size_t idx = (size_t)b * H + j0 + e % kSeqUnits;
    dh_s[e] = (b < B && D.ghn) ? D.ghn[idx] : 0.f;
    dc_s[e] = (b < B && D.gcn) ? D.gcn[idx] : 0.f;
  }
  if (tid == 0) failed = 0;
  __syncthreads();
  const int eighth = tid >> 5, rp = (tid & 31) >> 2, uq = tid & 3;
  const int cr = tid >> 4, cj = tid & 15;            // the cell's (row, unit) of this thread
  const int kspan4 = H4 / 4 / 8;
  const size_t bh = (size_t)B * H;
  unsigned* counter = D.counter + blockIdx.y;
  float pre[7] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < T; s++) {
    const int tt = D.reverse ? s : T - 1 - s;
    const int pt = D.reverse ? tt + 1 : tt - 1;
    const bool first = D.reverse ? tt == T - 1 : tt == 0;
    const float* cp = first ? D.c0 : D.c + (size_t)pt * bh;
    const float* gates_t = D.gates + (size_t)tt * B * H4;
    float* dg_t = D.dG + (size_t)tt * B * H4;
    // Gate gradients of this CTA's units (BackwardRecurrent.cs:37-57 of the reference, the same operation order). With one
    // pass per CTA the step's saved values were fetched ahead (they do not depend on dh), under the previous step's product.
    for (int pass = 0; pass < p.passes; pass++) {
      const int b = row_base + pass * kSeqRows + cr;
      if (b >= B) continue;
      const int e = (pass * kSeqRows + cr) * kSeqUnits + cj, jg = j0 + cj;
      const size_t idx = (size_t)b * H + jg;
      float* d = dg_t + (size_t)b * H4;
      float gi, gf, gg, go, tc, gyv, cpv;
      if (p.passes == 1 && s > 0) {
        gi = pre[0]; gf = pre[1]; gg = pre[2]; go = pre[3]; tc = pre[4]; gyv = pre[5]; cpv = pre[6];
      } else {
        const float* g = gates_t + (size_t)b * H4;
        gi = g[jg]; gf = g[H + jg]; gg = g[2 * H + jg]; go = g[3 * H + jg];
        tc = D.tanh_c[(size_t)tt * bh + idx];
        gyv = D.gy[(size_t)tt * bh + idx];
        cpv = cp ? cp[idx] : 0.f;
      }
      const float dH = gyv + dh_s[e];
      const float dO = dH * tc;
      const float dC = dc_s[e] + ((dH * go) * (1.f - (tc * tc)));
      const float dI = dC * gg, dF = dC * cpv, dGg = dC * gi;
      dc_s[e] = dC * gf;
      d[jg] = (dI * gi) * (1.f - gi);
      d[H + jg] = (dF * gf) * (1.f - gf);
      d[2 * H + jg] = dGg * (1.f - (gg * gg));
      d[3 * H + jg] = (dO * go) * (1.f - go);
    }
    if (s == T - 1 && D.dh0 == nullptr) break;
    if (!seq_barrier(counter, (unsigned)(s + 1) * gridDim.x, p.status, &failed, 9200 + (int)blockIdx.z)) return;
    if (p.passes == 1 && s + 1 < T) {
      // the next step's saved values: issued now, used after the product below
      const int b = row_base + cr;
      if (b < B) {
        const int tn = D.reverse ? s + 1 : T - 2 - s;
        const int pn = D.reverse ? tn + 1 : tn - 1;
        const bool first_n = D.reverse ? tn == T - 1 : tn == 0;
        const size_t idx = (size_t)b * H + j0 + cj;
        const float* g = D.gates + ((size_t)tn * B + b) * H4;
        pre[0] = g[j0 + cj]; pre[1] = g[H + j0 + cj]; pre[2] = g[2 * H + j0 + cj]; pre[3] = g[3 * H + j0 + cj];
        pre[4] = D.tanh_c[(size_t)tn * bh + idx];
        pre[5] = D.gy[(size_t)tn * bh + idx];
        const float* cpn = first_n ? D.c0 : D.c + (size_t)pn * bh;
        pre[6] = cpn ? cpn[idx] : 0.f;
      }
    }
    // dh of the next processed step, this CTA's units: dG_t[b, :] . W_hh[:, j]
    for (int pass = 0; pass < p.passes; pass++) {
      const int r0 = row_base + pass * kSeqRows;
      if (r0 >= B) break;
      for (int idx = tid; idx < kSeqRows * (H4 / 4); idx += kSeqThreads) {
        const int r = idx / (H4 / 4), k4 = idx % (H4 / 4), b = r0 + r;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < B) v = __ldcg(reinterpret_cast<const float4*>(dg_t + (size_t)b * H4) + k4);
        *reinterpret_cast<float4*>(ds + (size_t)r * ldd + 4 * k4) = v;
      }
      __syncthreads();
      float acc[2][4];
#pragma unroll
      for (int u = 0; u < 2; u++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[u][j] = 0.f;
      const float4* d0p = reinterpret_cast<const float4*>(ds + (size_t)(2 * rp) * ldd) + eighth * kspan4;
      const float4* d1p = reinterpret_cast<const float4*>(ds + (size_t)(2 * rp + 1) * ldd) + eighth * kspan4;
      const float* wbase = wcol + (size_t)(eighth * kspan4 * 4) * kSeqUnits + 4 * uq;
#pragma unroll 2
      for (int k4 = 0; k4 < kspan4; k4++) {
        const float4 a0 = d0p[k4], a1 = d1p[k4];
        const float4 w0 = *reinterpret_cast<const float4*>(wbase + (size_t)(4 * k4) * kSeqUnits);
        const float4 w1 = *reinterpret_cast<const float4*>(wbase + (size_t)(4 * k4 + 1) * kSeqUnits);
        const float4 w2 = *reinterpret_cast<const float4*>(wbase + (size_t)(4 * k4 + 2) * kSeqUnits);
        const float4 w3 = *reinterpret_cast<const float4*>(wbase + (size_t)(4 * k4 + 3) * kSeqUnits);
        acc[0][0] = fmaf(a0.x, w0.x, acc[0][0]); acc[0][1] = fmaf(a0.x, w0.y, acc[0][1]); acc[0][2] = fmaf(a0.x, w0.z, acc[0][2]); acc[0][3] = fmaf(a0.x, w0.w, acc[0][3]);
        acc[1][0] = fmaf(a1.x, w0.x, acc[1][0]); acc[1][1] = fmaf(a1.x, w0.y, acc[1][1]); acc[1][2] = fmaf(a1.x, w0.z, acc[1][2]); acc[1][3] = fmaf(a1.x, w0.w, acc[1][3]);
        acc[0][0] = fmaf(a0.y, w1.x, acc[0][0]); acc[0][1] = fmaf(a0.y, w1.y, acc[0][1]); acc[0][2] = fmaf(a0.y, w1.z, acc[0][2]); acc[0][3] = fmaf(a0.y, w1.w, acc[0][3]);
        acc[1][0] = fmaf(a1.y, w1.x, acc[1][0]); acc[1][1] = fmaf(a1.y, w1.y, acc[1][1]); acc[1][2] = fmaf(a1.y, w1.z, acc[1][2]); acc[1][3] = fmaf(a1.y, w1.w, acc[1][3]);
        acc[0][0] = fmaf(a0.z, w2.x, acc[0][0]); acc[0][1] = fmaf(a0.z, w2.y, acc[0][1]); acc[0][2] = fmaf(a0.z, w2.z, acc[0][2]); acc[0][3] = fmaf(a0.z, w2.w, acc[0][3]);
        acc[1][0] = fmaf(a1.z, w2.x, acc[1][0]); acc[1][1] = fmaf(a1.z, w2.y, acc[1][1]); acc[1][2] = fmaf(a1.z, w2.z, acc[1][2]); acc[1][3] = fmaf(a1.z, w2.w, acc[1][3]);
        acc[0][0] = fmaf(a0.w, w3.x, acc[0][0]); acc[0][1] = fmaf(a0.w, w3.y, acc[0][1]); acc[0][2] = fmaf(a0.w, w3.z, acc[0][2]); acc[0][3] = fmaf(a0.w, w3.w, acc[0][3]);
        acc[1][0] = fmaf(a1.w, w3.x, acc[1][0]); acc[1][1] = fmaf(a1.w, w3.y, acc[1][1]); acc[1][2] = fmaf(a1.w, w3.z, acc[1][2]); acc[1][3] = fmaf(a1.w, w3.w, acc[1][3]);
      }
      // red[eighth][row][unit]
#pragma unroll
      for (int u = 0; u < 2; u++)
        *reinterpret_cast<float4*>(red + ((size_t)eighth * kSeqRows + 2 * rp + u) * kSeqUnits + 4 * uq) =
            make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
      __syncthreads();
      {
        const float* rpn = red + (size_t)cr * kSeqUnits + cj;
        float t = rpn[0];
#pragma unroll
        for (int k = 1; k < 8; k++) t += rpn[(size_t)k * kSeqRows * kSeqUnits];
        dh_s[(pass * kSeqRows + cr) * kSeqUnits + cj] = t;
      }
      __syncthreads();
    }
  }
  __syncthreads();
  for (int e = tid; e < group_rows * kSeqUnits; e += kSeqThreads) {
    const int b = row_base + e / kSeqUnits;
    if (b >= B) continue;
    const size_t idx = (size_t)b * H + j0 + e % kSeqUnits;
    if (D.dh0) D.dh0[idx] = dh_s[e];
    if (D.dc0) D.dc0[idx] = dc_s[e];
  }
}

static_assert(kSeqThreads == kSeqRows * kSeqUnits, "the cell phases map one thread to one (row, unit)");

static size_t seq_fwd_smem(int h) { return sizeof(float) * ((size_t)(64 + kSeqRows) * (h + kSeqPad) + 128 * 8); }
static size_t seq_bwd_smem(int h, int passes) {
  return sizeof(float) * ((size_t)4 * h * kSeqUnits + (size_t)kSeqRows * (4 * h + kSeqPad) + 8 * kSeqRows * kSeqUnits +
                          2 * (size_t)passes * kSeqRows * kSeqUnits);
}

// The launch shape: row groups of `passes` x 16 rows, as few passes as lets all CTAs of `dirs` directions be resident at
// once. Returns false when the shape does not fit the kernels.
static bool seq_plan(om_ctx* ctx, int dirs, int b, int h, bool backward, int* passes_out, int* groups_out) {
  if (h < 16 || h % 16 != 0 || b < 1) return false;
  const void* fn = backward ? (const void*)lstm_seq_bwd_kernel : (const void*)lstm_seq_fwd_kernel;
  const int tiles = (int)ceil_div(b, kSeqRows);
  for (int passes = 1;; passes *= 2) {
    const int groups = (int)ceil_div(tiles, passes);
    if (groups <= kSeqMaxGroups) {
      const size_t smem = backward ? seq_bwd_smem(h, passes) : seq_fwd_smem(h);
      if (smem > 200 * 1024) return false;
      if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return false;
      }
      int per_sm = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kSeqThreads, smem) != cudaSuccess) {
        cudaGetLastError();
        return false;
      }
      if ((long long)per_sm * ctx->sm_count >= (long long)dirs * groups * (h / kSeqUnits)) {
        *passes_out = passes;
        *groups_out = groups;
        return true;
      }
    }
    if (passes >= tiles) return false;
  }
}

bool lstm_seq_supported(om_ctx* ctx, int dirs, int t, int b, int h, bool backward) {
  if (!(ctx->flags & OM_SEQ_KERNELS) || t < 2) return false;
  int passes = 0, groups = 0;
  return seq_plan(ctx, dirs, b, h, backward, &passes, &groups);
}

int32_t lstm_seq_fwd(om_ctx* ctx, int dirs, int t, int b, int h, const LstmSeqFwdDir* d) {
  LstmSeqFwdParams p;
  if (!seq_plan(ctx, dirs, b, h, false, &p.passes, &p.groups)) return fail(ctx, OM_ERR_UNSUPPORTED, "lstm_seq_fwd: B %d H %d", b, h);
  unsigned* counters = nullptr;
  OM_TRY(pool_alloc(ctx, 2 * kSeqMaxGroups * sizeof(unsigned), true, (void**)&counters));
  for (int k = 0; k < 2; k++) {
    p.d[k] = d[k < dirs ? k : 0];
    p.d[k].counter = counters + k * kSeqMaxGroups;
  }
  p.t = t;
  p.b = b;
  p.h = h;
  p.status = ctx->status_dev;
  void* args[] = {&p};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)lstm_seq_fwd_kernel, dim3((unsigned)(h / kSeqUnits), (unsigned)p.groups, (unsigned)dirs),
                                              dim3(kSeqThreads), args, seq_fwd_smem(h), ctx->stream);
  pool_free(ctx, counters);
  if (e != cudaSuccess) return check_cuda(ctx, e, "lstm_seq_fwd");
  return OM_OK;
}

int32_t lstm_seq_bwd(om_ctx* ctx, int dirs, int t, int b, int h, const LstmSeqBwdDir* d) {
  LstmSeqBwdParams p;
  if (!seq_plan(ctx, dirs, b, h, true, &p.passes, &p.groups)) return fail(ctx, OM_ERR_UNSUPPORTED, "lstm_seq_bwd: B %d H %d", b, h);
  unsigned* counters = nullptr;
  OM_TRY(pool_alloc(ctx, 2 * kSeqMaxGroups * sizeof(unsigned), true, (void**)&counters));
  for (int k = 0; k < 2; k++) {
    p.d[k] = d[k < dirs ? k : 0];
    p.d[k].counter = counters + k * kSeqMaxGroups;
  }
  p.t = t;
  p.b = b;
  p.h = h;
  p.status = ctx->status_dev;
  void* args[] = {&p};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)lstm_seq_bwd_kernel, dim3((unsigned)(h / kSeqUnits), (unsigned)p.groups, (unsigned)dirs),
                                              dim3(kSeqThreads), args, seq_bwd_smem(h, p.passes), ctx->stream);
  pool_free(ctx, counters);
  if (e != cudaSuccess) return check_cuda(ctx, e, "lstm_seq_bwd");
  return OM_OK;
}

}  // namespace om
