// Exact fp32 log-normalisers and the row statistics the factored kernels need.
//
// lognorm_exact: logsumexp_v(E[t,v]+P[u,v]) per lattice node with the maximum
// subtracted before exponentiation -- the brute-force definition the reference's
// tests use (transducer/test.h:51-80).  One warp per node, lanes stride over the
// vocabulary, warp-shuffle reductions.  It serves as (i) the recompute path for
// nodes whose exp-factored sum under- or overflowed, (ii) the only log-normaliser
// for shapes the TMA-fed tensor-core kernel cannot take (vocabulary not a multiple
// of 4 floats, unaligned base pointers).
#include "kernels.h"
#include "profile.h"

namespace tb200 {
namespace {

__device__ __forceinline__ float node_logsumexp(const float* __restrict__ er,
                                                const float* __restrict__ pr, int V,
                                                int lane) {
  float m = neg_inf();
  for (int v = lane; v < V; v += 32) m = fmaxf(m, er[v] + pr[v]);
  m = warp_max(m);
  float s = 0.0f;
  if (m != neg_inf() && m != pos_inf()) {
    for (int v = lane; v < V; v += 32) s += expf((er[v] + pr[v]) - m);
  }
  s = warp_sum(s);
  return logf(s) + m;
}

constexpr int kWarpsPerCta = 8;

// grid = (ceil(maxU / 8), maxT, B); warp w of CTA (x,t,b) owns node (t, x*8+w).
__global__ void __launch_bounds__(kWarpsPerCta * 32) lognorm_exact_kernel(
    const float* __restrict__ E, const float* __restrict__ P, float* __restrict__ LN,
    const int* __restrict__ inLens, const int* __restrict__ labLens, int maxT, int maxU,
    int V) {
  const int b = blockIdx.z, t = blockIdx.y;
  const int u = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  if (t >= T || u >= U) return;
  const int lane = threadIdx.x & 31;
  const float r = node_logsumexp(E + ((i64)b * maxT + t) * V, P + ((i64)b * maxU + u) * V,
                                 V, lane);
  if (lane == 0) LN[((i64)b * maxT + t) * maxU + u] = r;
}

__global__ void __launch_bounds__(kWarpsPerCta * 32) lognorm_exact_list_kernel(
    const float* __restrict__ E, const float* __restrict__ P, float* __restrict__ LN,
    const int* __restrict__ cells, const int* __restrict__ count, int maxCount, int maxT,
    int maxU, int V) {
  const int n = min(*count, maxCount);
  const int lane = threadIdx.x & 31;
  const int warpsTotal = gridDim.x * kWarpsPerCta;
  for (int k = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5); k < n; k += warpsTotal) {
    const int b = cells[3 * k], t = cells[3 * k + 1], u = cells[3 * k + 2];
    const float r = node_logsumexp(E + ((i64)b * maxT + t) * V,
                                   P + ((i64)b * maxU + u) * V, V, lane);
    if (lane == 0) LN[((i64)b * maxT + t) * maxU + u] = r;
  }
}

// One warp per row: rowMax = max_v X[row, v]; rows at or beyond the utterance's
// length get 0.  `lens[b] + lenOffset` is the number of valid rows.
__global__ void __launch_bounds__(256) row_max_kernel(
    const float* __restrict__ X, float* __restrict__ rowMax, const int* __restrict__ lens,
    int lenOffset, int maxRows, int V) {
  const int b = blockIdx.y;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= maxRows) return;
  const int lane = threadIdx.x & 31;
  const int n = min(lens[b] + lenOffset, maxRows);
  float m = 0.0f;
  if (row < n) {
    const float* x = X + ((i64)b * maxRows + row) * V;
    m = neg_inf();
    for (int v = lane; v < V; v += 32) m = fmaxf(m, x[v]);
    m = warp_max(m);
  }
  if (lane == 0) rowMax[(i64)b * maxRows + row] = m;
}

// One CTA per prediction row: maxP and expP = exp(P - maxP); zeros for padded rows.
__global__ void __launch_bounds__(256) exp_rows_kernel(
    const float* __restrict__ P, float* __restrict__ expP, float* __restrict__ maxP,
    const int* __restrict__ labLens, int maxU, int V) {
  __shared__ float red[8];
  const int b = blockIdx.y, u = blockIdx.x;
  const int U = min(labLens[b] + 1, maxU);
  const float* p = P + ((i64)b * maxU + u) * V;
  float* o = expP + ((i64)b * maxU + u) * V;
  if (u >= U) {
    for (int v = threadIdx.x; v < V; v += blockDim.x) o[v] = 0.0f;
    if (threadIdx.x == 0) maxP[(i64)b * maxU + u] = 0.0f;
    return;
  }
  float m = neg_inf();
  for (int v = threadIdx.x; v < V; v += blockDim.x) m = fmaxf(m, p[v]);
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) m = fmaxf(m, red[k]);
  for (int v = threadIdx.x; v < V; v += blockDim.x) o[v] = expf(p[v] - m);
  if (threadIdx.x == 0) maxP[(i64)b * maxU + u] = m;
}

}  // namespace

void launch_lognorm_exact(const float* E, const float* P, float* LN, const int* inLens,
                          const int* labLens, Dims d, cudaStream_t stream) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 0) return;
  if (d.maxT > 65535 || d.B > 65535)
    throw std::invalid_argument("exact log-normaliser: batch or frame count above 65535");
  dim3 grid(div_up(d.maxU, kWarpsPerCta), d.maxT, d.B);
  ScopedKernel sk("lognorm_exact", stream);
  lognorm_exact_kernel<<<grid, kWarpsPerCta * 32, 0, stream>>>(E, P, LN, inLens, labLens,
                                                               d.maxT, d.maxU, d.V);
  TB200_CHECK_LAUNCH();
}

void launch_lognorm_exact_list(const float* E, const float* P, float* LN,
                               const int* cells, const int* count, int maxCount,
                               Dims d, cudaStream_t stream) {
  if (maxCount <= 0) return;
  const int ctas = 148 * 4;
  ScopedKernel sk("lognorm_exact_list", stream);
  lognorm_exact_list_kernel<<<ctas, kWarpsPerCta * 32, 0, stream>>>(
      E, P, LN, cells, count, maxCount, d.maxT, d.maxU, d.V);
  TB200_CHECK_LAUNCH();
}

void launch_row_max(const float* X, float* rowMax, const int* lens, int lenOffset, int B,
                    int maxRows, int V, cudaStream_t stream) {
  if (B <= 0 || maxRows <= 0) return;
  dim3 grid(div_up(maxRows, 8), B);
  ScopedKernel sk("row_max", stream);
  row_max_kernel<<<grid, 256, 0, stream>>>(X, rowMax, lens, lenOffset, maxRows, V);
  TB200_CHECK_LAUNCH();
}

void launch_exp_rows(const float* P, float* expP, float* maxP, const int* labLens, int B,
                     int maxU, int V, cudaStream_t stream) {
  if (B <= 0 || maxU <= 0) return;
  dim3 grid(maxU, B);
  ScopedKernel sk("exp_rows", stream);
  exp_rows_kernel<<<grid, 256, 0, stream>>>(P, expP, maxP, labLens, maxU, V);
  TB200_CHECK_LAUNCH();
}

}  // namespace tb200
