// best[b,t,u] = max over v != blank of (E[b,t,v] + P[b,u,v]): the label-arc score the
// Viterbi sweep needs at every lattice node (transducer/transducer_cpu.cpp:156-169
// evaluates it inside the sweep; transducer_cuda.cu:233-242 inside the wavefront).
// fp32 add followed by max is exact and order-independent, so a tiled evaluation is
// bit-identical to the reference's serial loop.  Which v attains the maximum is only
// needed on the final path and is resolved after the backtrack.
//
// (max,+) has no tensor-core form; this is a register-tiled SIMT kernel: 2 issue
// slots (FADD, FMNMX) per (t,u,v).
#include "kernels.h"
#include "profile.h"

namespace tb200 {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256) maxplus_kernel(
    const float* __restrict__ E, const float* __restrict__ P, float* __restrict__ best,
    const int* __restrict__ inLens, const int* __restrict__ labLens, int maxT, int maxU,
    int V, int blank) {
  __shared__ __align__(16) float Es[TK][TM + 4];
  __shared__ __align__(16) float Ps[TK][TN + 4];
  const int b = blockIdx.z, t0 = blockIdx.y * TM, u0 = blockIdx.x * TN;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  if (t0 >= T || u0 >= U - 1) return;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const float* e = E + (i64)b * maxT * V;
  const float* p = P + (i64)b * maxU * V;
  const float ninf = neg_inf();
  float acc[4][4];
#pragma unroll
  for (int m = 0; m < 4; ++m)
#pragma unroll
    for (int n = 0; n < 4; ++n) acc[m][n] = ninf;

  const int lm = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < V; k0 += TK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int v = k0 + lk + j;
      const int t = t0 + lm, u = u0 + lm;
      const bool ok = v < V && v != blank;
      Es[lk + j][lm] = (ok && t < T) ? e[(i64)t * V + v] : ninf;
      Ps[lk + j][lm] = (ok && u < U - 1) ? p[(i64)u * V + v] : ninf;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&Es[k][ty * 4]);
      const float4 c = *reinterpret_cast<const float4*>(&Ps[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, cv[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int m = 0; m < 4; ++m)
#pragma unroll
        for (int n = 0; n < 4; ++n) acc[m][n] = fmaxf(acc[m][n], av[m] + cv[n]);
    }
    __syncthreads();
  }
  float* o = best + (i64)b * maxT * maxU;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const int t = t0 + ty * 4 + m;
    if (t >= T) continue;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int u = u0 + tx * 4 + n;
      if (u < U - 1) o[(i64)t * maxU + u] = acc[m][n];
    }
  }
}

}  // namespace

void launch_maxplus(const float* E, const float* P, float* best, const int* inLens,
                    const int* labLens, Dims d, cudaStream_t stream) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 1) return;
  dim3 grid(div_up(d.maxU - 1, TN), div_up(d.maxT, TM), d.B);
  ScopedKernel sk("maxplus", stream);
  maxplus_kernel<<<grid, 256, 0, stream>>>(E, P, best, inLens, labLens, d.maxT, d.maxU, d.V,
                                           d.blank);
  TB200_CHECK_LAUNCH();
}

}  // namespace tb200
