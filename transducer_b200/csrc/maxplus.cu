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
    int V, int blank, const int* __restrict__ guard, int guardCap) {
  if (guard != nullptr && *guard <= guardCap) return;
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

// Larger register tile for vocabularies that are a multiple of 4 (float4 loads along v):
// 128 frames x 16*NT label positions per CTA, 8 x NT outputs per thread, K tiles of 16
// double-buffered in shared memory with the next tile's global loads in flight during the
// arithmetic.  NT is picked so that the label axis fills its tiles (U-1 = 149 -> NT = 5, two
// tiles of 80).
constexpr int BM = 128, BK = 16;

// max of three floats in one instruction (exact, like two nested fmaxf)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

template <int NT>
__global__ void __launch_bounds__(256) maxplus_tiled_kernel(
    const float* __restrict__ E, const float* __restrict__ P, float* __restrict__ best,
    const int* __restrict__ inLens, const int* __restrict__ labLens, int maxT, int maxU,
    int V, int blank, const int* __restrict__ guard, int guardCap) {
  if (guard != nullptr && *guard <= guardCap) return;
  constexpr int BN = 16 * NT;
  constexpr int kPLoads = (BN * 4 + 255) / 256;  // float4 loads of the P tile per thread
  __shared__ __align__(16) float Es[2][BK][BM + 4];
  __shared__ __align__(16) float Ps[2][BK][BN + 4];
  const int b = blockIdx.z, t0 = blockIdx.y * BM, u0 = blockIdx.x * BN;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  if (t0 >= T || u0 >= U - 1) return;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const float* e = E + (i64)b * maxT * V;
  const float* p = P + (i64)b * maxU * V;
  const float ninf = neg_inf();
  float acc[8][NT];
#pragma unroll
  for (int m = 0; m < 8; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n) acc[m][n] = ninf;

  // global -> registers: rows clamped into the lattice (their results are never stored),
  // columns beyond V and the blank column become -inf
  float4 eReg[2], pReg[kPLoads];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + 256 * i, row = idx >> 2, v = k0 + (idx & 3) * 4;
      const int t = min(t0 + row, T - 1);
      eReg[i] = (v < V) ? *reinterpret_cast<const float4*>(e + (i64)t * V + v)
                        : make_float4(ninf, ninf, ninf, ninf);
    }
#pragma unroll
    for (int i = 0; i < kPLoads; ++i) {
      const int idx = tid + 256 * i, row = idx >> 2, v = k0 + (idx & 3) * 4;
      const int u = min(u0 + row, U - 1);
      pReg[i] = (v < V && idx < BN * 4) ? *reinterpret_cast<const float4*>(p + (i64)u * V + v)
                                        : make_float4(ninf, ninf, ninf, ninf);
    }
  };
  auto stash = [&](int buf, int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + 256 * i, row = idx >> 2, kq = (idx & 3) * 4, v = k0 + kq;
      float x[4] = {eReg[i].x, eReg[i].y, eReg[i].z, eReg[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) Es[buf][kq + j][row] = (v + j == blank) ? ninf : x[j];
    }
#pragma unroll
    for (int i = 0; i < kPLoads; ++i) {
      const int idx = tid + 256 * i, row = idx >> 2, kq = (idx & 3) * 4;
      if (idx < BN * 4) {
        const float x[4] = {pReg[i].x, pReg[i].y, pReg[i].z, pReg[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) Ps[buf][kq + j][row] = x[j];
      }
    }
  };

  const int nK = (V + BK - 1) / BK;
  fetch(0);
  stash(0, 0);
  __syncthreads();
  for (int kt = 0; kt < nK; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < nK) fetch((kt + 1) * BK);
    // two vocabulary entries per step: the three-input max of sm_100 takes both sums at once,
    // which halves the max instructions (they issue at half the rate of the adds)
#pragma unroll
    for (int k = 0; k < BK; k += 2) {
      float av[2][8], cv[2][NT];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float4 a0 = *reinterpret_cast<const float4*>(&Es[buf][k + h][ty * 8]);
        const float4 a1 = *reinterpret_cast<const float4*>(&Es[buf][k + h][ty * 8 + 4]);
        av[h][0] = a0.x; av[h][1] = a0.y; av[h][2] = a0.z; av[h][3] = a0.w;
        av[h][4] = a1.x; av[h][5] = a1.y; av[h][6] = a1.z; av[h][7] = a1.w;
#pragma unroll
        for (int n = 0; n < NT; ++n) cv[h][n] = Ps[buf][k + h][tx * NT + n];
      }
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
          acc[m][n] = max3(acc[m][n], av[0][m] + cv[0][n], av[1][m] + cv[1][n]);
    }
    if (kt + 1 < nK) stash(buf ^ 1, (kt + 1) * BK);
    __syncthreads();
  }
  float* o = best + (i64)b * maxT * maxU;
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const int t = t0 + ty * 8 + m;
    if (t >= T) continue;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int u = u0 + tx * NT + n;
      if (u < U - 1) o[(i64)t * maxU + u] = acc[m][n];
    }
  }
}

}  // namespace

void launch_maxplus(const float* E, const float* P, float* best, const int* inLens,
                    const int* labLens, Dims d, cudaStream_t stream, const int* guard,
                    int guardCap) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 1) return;
  ScopedKernel sk(guard ? "maxplus_if_unsettled" : "maxplus", stream);
  const bool vec = d.V % 4 == 0 && (reinterpret_cast<uintptr_t>(E) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(P) & 15) == 0;
  if (vec) {
    // label positions per thread: the tile width 16*NT that wastes the least of the label axis
    const int n = d.maxU - 1;
    int bestNT = 8;
    long bestWaste = -1;
    for (int NT : {8, 6, 5, 4}) {
      const long waste = (long)div_up(n, 16 * NT) * 16 * NT - n;
      if (bestWaste < 0 || waste < bestWaste) {
        bestWaste = waste;
        bestNT = NT;
      }
    }
#define CALL(NT)                                                                         \
  maxplus_tiled_kernel<NT><<<dim3(div_up(n, 16 * NT), div_up(d.maxT, BM), d.B), 256, 0,  \
                             stream>>>(E, P, best, inLens, labLens, d.maxT, d.maxU, d.V, d.blank,   \
                                       guard, guardCap)
    switch (bestNT) {
      case 4: CALL(4); break;
      case 5: CALL(5); break;
      case 6: CALL(6); break;
      default: CALL(8); break;
    }
#undef CALL
  } else {
    dim3 grid(div_up(d.maxU - 1, TN), div_up(d.maxT, TM), d.B);
    maxplus_kernel<<<grid, 256, 0, stream>>>(E, P, best, inLens, labLens, d.maxT, d.maxU, d.V,
                                             d.blank, guard, guardCap);
  }
  TB200_CHECK_LAUNCH();
}

}  // namespace tb200
