// Dense part of the emission / prediction gradients on the SIMT pipes.
//
// The reference forms these with torch ops (transducer/torch_binding.py:85-89):
//   Wn = occupancy / expLN;  egrads += expE * bmm(Wn, expP);
//   pgrads += expP * bmm(Wn^T, expE);  both scaled by deltas[b].
// Here W[t,u] = occupancy * exp(rowRef[t] + maxP[u] - LN[t,u]) is the same weight
// (expLN = exp(LN - rowRef - maxP)), expE is recomputed from E on the fly (never
// stored), and every element of egrads/pgrads is written exactly once: no memset,
// no read-modify-write of the dense buffers except the label-arc scatter.
//
// These fp32 FMA kernels take any vocabulary size and alignment; the tensor-core
// kernels replace them for shapes TMA can address.
#include "kernels.h"
#include "profile.h"

namespace tb200 {
namespace {

constexpr int BM = 64, BN = 64, BK = 16;

// egrads tile: rows t0..t0+63 of utterance b, columns v0..v0+63.
__global__ void __launch_bounds__(256) egrad_simt_kernel(
    const float* __restrict__ E, const float* __restrict__ rowRef,
    const float* __restrict__ W, int ldW, const float* __restrict__ expP,
    const float* __restrict__ eBlank, const float* __restrict__ deltas,
    float* __restrict__ egrads, const int* __restrict__ inLens,
    const int* __restrict__ labLens, int maxT, int maxU, int V, int blank) {
  __shared__ __align__(16) float Ws[BK][BM + 4];
  __shared__ __align__(16) float Ps[BK][BN];
  const int b = blockIdx.z, t0 = blockIdx.y * BM, v0 = blockIdx.x * BN;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  float* out = egrads + (i64)b * maxT * V;

  if (t0 >= T || U <= 0) {  // padded frames: exact zeros, inputs not read
    for (int m = ty * 4; m < ty * 4 + 4; ++m)
      for (int n = tx * 4; n < tx * 4 + 4; ++n)
        if (t0 + m < maxT && v0 + n < V) out[(i64)(t0 + m) * V + v0 + n] = 0.0f;
    return;
  }
  const float* w = W + (i64)b * maxT * ldW;
  const float* xp = expP + (i64)b * maxU * V;
  float acc[4][4] = {};
  for (int u0 = 0; u0 < U; u0 += BK) {
    {  // W tile, transposed into [k][m]
      const int m = tid >> 2, k4 = (tid & 3) * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = t0 + m, u = u0 + k4 + j;
        Ws[k4 + j][m] = (t < T && u < U) ? w[(i64)t * ldW + u] : 0.0f;
      }
    }
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int k = pass * 4 + (tid >> 6), n = tid & 63;
      const int u = u0 + k, v = v0 + n;
      Ps[k][n] = (u < U && v < V) ? xp[(i64)u * V + v] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&Ws[k][ty * 4]);
      const float4 c = *reinterpret_cast<const float4*>(&Ps[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, cv[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int m = 0; m < 4; ++m)
#pragma unroll
        for (int n = 0; n < 4; ++n) acc[m][n] = fmaf(av[m], cv[n], acc[m][n]);
    }
    __syncthreads();
  }
  const float delta = deltas ? deltas[b] : 1.0f;
  const float* e = E + (i64)b * maxT * V;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const int t = t0 + ty * 4 + m;
    if (t >= maxT) continue;
    const bool live = t < T;
    const float ref = live ? rowRef[(i64)b * maxT + t] : 0.0f;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int v = v0 + tx * 4 + n;
      if (v >= V) continue;
      float val = 0.0f;
      if (live) {
        val = expf(e[(i64)t * V + v] - ref) * acc[m][n];
        if (v == blank) val -= eBlank[(i64)b * maxT + t];
        val *= delta;
      }
      out[(i64)t * V + v] = val;
    }
  }
}

// egrads[t, label_u] -= delta * em[t,u]; one thread per frame walks u in order, so
// repeated labels on a frame are combined deterministically.
__global__ void __launch_bounds__(128) egrad_label_scatter_kernel(
    const float* __restrict__ em, const int* __restrict__ labels,
    const float* __restrict__ deltas, float* __restrict__ egrads,
    const int* __restrict__ inLens, const int* __restrict__ labLens, int maxT, int maxU,
    int V) {
  const int b = blockIdx.y, t = blockIdx.x * blockDim.x + threadIdx.x;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  if (t >= T || U <= 1) return;
  const float delta = deltas ? deltas[b] : 1.0f;
  const float* m = em + ((i64)b * maxT + t) * maxU;
  const int* lab = labels + (i64)b * (maxU - 1);
  float* row = egrads + ((i64)b * maxT + t) * V;
  for (int u = 0; u < U - 1; ++u) row[lab[u]] -= delta * m[u];
}

// pgrads tile: rows u0..u0+63 of utterance b, columns v0..v0+63; K runs over frames.
__global__ void __launch_bounds__(256) pgrad_simt_kernel(
    const float* __restrict__ E, const float* __restrict__ rowRef,
    const float* __restrict__ W, int ldW, const float* __restrict__ expP,
    const float* __restrict__ pBlank, const float* __restrict__ pLabel,
    const int* __restrict__ labels, const float* __restrict__ deltas,
    float* __restrict__ pgrads, const int* __restrict__ inLens,
    const int* __restrict__ labLens, int maxT, int maxU, int V, int blank) {
  __shared__ __align__(16) float Ws[BK][BM];
  __shared__ __align__(16) float Es[BK][BN];
  const int b = blockIdx.z, u0 = blockIdx.y * BM, v0 = blockIdx.x * BN;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  float* out = pgrads + (i64)b * maxU * V;

  if (u0 >= U || T <= 0) {
    for (int m = ty * 4; m < ty * 4 + 4; ++m)
      for (int n = tx * 4; n < tx * 4 + 4; ++n)
        if (u0 + m < maxU && v0 + n < V) out[(i64)(u0 + m) * V + v0 + n] = 0.0f;
    return;
  }
  const float* w = W + (i64)b * maxT * ldW;
  const float* e = E + (i64)b * maxT * V;
  const float* ref = rowRef + (i64)b * maxT;
  float acc[4][4] = {};
  for (int t0 = 0; t0 < T; t0 += BK) {
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int k = pass * 4 + (tid >> 6), c = tid & 63;
      const int t = t0 + k;
      const int u = u0 + c, v = v0 + c;
      Ws[k][c] = (t < T && u < U) ? w[(i64)t * ldW + u] : 0.0f;
      Es[k][c] = (t < T && v < V) ? expf(e[(i64)t * V + v] - ref[t]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&Ws[k][ty * 4]);
      const float4 c = *reinterpret_cast<const float4*>(&Es[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, cv[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int m = 0; m < 4; ++m)
#pragma unroll
        for (int n = 0; n < 4; ++n) acc[m][n] = fmaf(av[m], cv[n], acc[m][n]);
    }
    __syncthreads();
  }
  const float delta = deltas ? deltas[b] : 1.0f;
  const float* xp = expP + (i64)b * maxU * V;
  const int* lab = labels + (i64)b * (maxU - 1);
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const int u = u0 + ty * 4 + m;
    if (u >= maxU) continue;
    const bool live = u < U;
    const int myLab = (live && u < U - 1) ? lab[u] : -1;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int v = v0 + tx * 4 + n;
      if (v >= V) continue;
      float val = 0.0f;
      if (live) {
        val = xp[(i64)u * V + v] * acc[m][n];
        if (v == blank) val -= pBlank[(i64)b * maxU + u];
        if (v == myLab) val -= pLabel[(i64)b * maxU + u];
        val *= delta;
      }
      out[(i64)u * V + v] = val;
    }
  }
}

}  // namespace

void launch_egrad_simt(const float* E, const float* rowRef, const float* W, int ldW,
                       const float* expP, const float* eBlank, const float* em,
                       const int* labels, const float* deltas, float* egrads,
                       const int* inLens, const int* labLens, Dims d,
                       cudaStream_t stream) {
  if (d.B <= 0 || d.maxT <= 0 || d.V <= 0) return;
  dim3 grid(div_up(d.V, BN), div_up(d.maxT, BM), d.B);
  {
  ScopedKernel sk("egrad_simt", stream);
  egrad_simt_kernel<<<grid, 256, 0, stream>>>(E, rowRef, W, ldW, expP, eBlank, deltas,
                                              egrads, inLens, labLens, d.maxT, d.maxU, d.V,
                                              d.blank);
  }
  TB200_CHECK_LAUNCH();
  if (d.maxU > 1) {
    ScopedKernel sk("egrad_label_scatter", stream);
    dim3 g2(div_up(d.maxT, 128), d.B);
    egrad_label_scatter_kernel<<<g2, 128, 0, stream>>>(em, labels, deltas, egrads, inLens,
                                                       labLens, d.maxT, d.maxU, d.V);
    TB200_CHECK_LAUNCH();
  }
}

void launch_pgrad_simt(const float* E, const float* rowRef, const float* W, int ldW,
                       const float* expP, const float* pBlank, const float* pLabel,
                       const int* labels, const float* deltas, float* pgrads,
                       const int* inLens, const int* labLens, Dims d,
                       cudaStream_t stream) {
  if (d.B <= 0 || d.maxU <= 0 || d.V <= 0) return;
  dim3 grid(div_up(d.V, BN), div_up(d.maxU, BM), d.B);
  ScopedKernel sk("pgrad_simt", stream);
  pgrad_simt_kernel<<<grid, 256, 0, stream>>>(E, rowRef, W, ldW, expP, pBlank, pLabel,
                                              labels, deltas, pgrads, inLens, labLens,
                                              d.maxT, d.maxU, d.V, d.blank);
  TB200_CHECK_LAUNCH();
}

}  // namespace tb200
