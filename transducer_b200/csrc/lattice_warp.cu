// Lattice sweeps for label axes of at most 128 positions: the recursion runs in ONE warp.
//
// The wavefront kernels of lattice.cu spend a block barrier and a shared-memory exchange on
// every anti-diagonal.  Here lane l of a single warp owns the label positions u = 4l .. 4l+3;
// all nodes of a diagonal are independent, the one value per lane that crosses from the
// neighbouring lane arrives by a warp shuffle, and nothing else sits on the dependent chain:
//   * the arc log-probabilities of every node were combined once by lattice_prep_kernel into
//     the skewed array arcs[d][u] = (blank arc, label arc) in log2 units, a large negative
//     finite number where the arc or the node does not exist -- so the recursion needs no
//     validity logic and no -inf special cases;
//   * in the skewed layout (node (t,u) at (t+u)*ld + u, see lattice.cu) a block of 16
//     diagonals is one contiguous range of memory: it is fetched by one bulk asynchronous
//     copy into a shared-memory ring, several blocks ahead of its use.
// alpha: a single warp per utterance does everything.  reverse sweep: the exponentials of the
// arc terms do not depend on the recursion, so four helper warps prepare them for the block
// ahead and write the results of the block behind, while the recursion warp is left with two
// multiplies and an add per node.
//
//   alpha   transducer/transducer_cpu.cpp:30-79   (transducer_cuda.cu:32-97)
//   reverse transducer/transducer_cpu.cpp:81-143  (transducer_cuda.cu:99-176)
#include "kernels.h"
#include "profile.h"
#include "sm100.cuh"

namespace tb200 {
namespace {

using namespace sm100;

constexpr int kDiag = 16;   // diagonals per block
constexpr int kRing = 4;    // blocks in flight
constexpr float kLn2F = 0.6931471805599453f;

__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void finish_cost_w(float* costs, int b, float cost, int B,
                                              float* lossSum, unsigned* ticket) {
  costs[b] = cost;
  if (lossSum == nullptr) return;
  __threadfence();
  const unsigned done = atomicAdd(ticket, 1u);
  if (done == (unsigned)(B - 1)) {  // last utterance: add the costs in index order
    __threadfence();
    float s = 0.0f;
    for (int k = 0; k < B; ++k) s += ((volatile float*)costs)[k];
    *lossSum = s;
    *ticket = 0u;
  }
}

// ---------------------------------------------------------------------------
// alpha
// ---------------------------------------------------------------------------
// One warp per utterance.  The recursion runs in log2 units,
//   a(t,u) = log2( 2^(a(t-1,u) + blank arc) + 2^(a(t,u-1) + label arc) ),
// so that the two transcendental steps are the bare ex2 / lg2 instructions, and the alphas are
// stored in log2 units too: the reverse sweep must form a(t,u) + arc with the very same
// rounding as here, or the occupancies stop being a conserved flow (the rounding of an alpha
// of magnitude 1e4 is 1e-3, and such errors would compound along the 2000 steps of a path).
__global__ void __launch_bounds__(32) alpha_warp_kernel(
    const float2* __restrict__ arcs, float* __restrict__ costs, float* __restrict__ alphas, int ld,
    i64 latStride, int nDiag, const int* __restrict__ inLens, const int* __restrict__ labLens,
    int B, int maxT, int maxU, float* lossSum, unsigned* ticket, int* status) {
  extern __shared__ __align__(128) uint8_t smemA[];
  float2* ring = reinterpret_cast<float2*>(smemA);  // [kRing][kDiag * ld]
  __shared__ uint64_t bar[kRing];
  __shared__ int abortFlag;
  const int b = blockIdx.x, lane = threadIdx.x;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  if (T <= 0 || U <= 0) {
    if (lane == 0) finish_cost_w(costs, b, pos_inf(), B, lossSum, ticket);
    return;
  }
  const float2* ar = arcs + (i64)b * latStride;
  float* al = alphas + (i64)b * latStride;
  const int S = T + U - 1;
  const int nBlocks = (S + kDiag - 1) / kDiag;
  const int slot = kDiag * ld;  // float2 elements per ring slot

  if (lane == 0) {
    for (int s = 0; s < kRing; ++s) mbar_init(&bar[s], 1);
    abortFlag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  auto issue = [&](int k) {  // lane 0: rows [16k, 16k+16) of arcs -> ring slot k % kRing
    if (k < nBlocks) {
      const int rows = min(kDiag, nDiag - k * kDiag);
      const uint32_t bytes = (uint32_t)(rows * ld) * 8u;
      mbar_arrive_expect_tx(&bar[k % kRing], bytes);
      bulk_load_1d(ring + (size_t)(k % kRing) * slot, ar + (size_t)k * slot, bytes, &bar[k % kRing]);
    }
  };
  if (lane == 0)
    for (int k = 0; k < kRing - 1; ++k) issue(k);

  // large negative and finite: the identity of the recursion without -inf arithmetic
  const float kNone = __uint_as_float(kNoArcBits);
  // Lane l owns the label positions u = 4l + r, r = 0..3: the value crossing from u-1 is the
  // lane's own for r > 0 and comes from lane l-1 by ONE shuffle per diagonal for r = 0; the
  // four arc pairs and the four alphas of a lane are contiguous (two 16-byte loads, one store).
  const int u0 = 4 * lane;
  const bool act = u0 < ld;  // rows are ld <= 128 wide
  float stayIn[4], stepOut[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) stayIn[r] = stepOut[r] = kNone;
  if (lane == 0) stayIn[0] = 0.0f;  // alpha(0,0) = 0
  float cost = 0.0f;
  bool owner = false, ok = true;

  int kFail = 0;
  for (int k = 0; k < nBlocks; ++k) {
    if (lane == 0) {
      fence_proxy_async_smem();  // the slot refilled next was read by this warp one block ago
      issue(k + kRing - 1);
    }
    ok = mbar_wait(&bar[k % kRing], (k / kRing) & 1, &abortFlag, status, kStatusTimeoutTma);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      kFail = k;
      break;
    }
    const float2* blk = ring + (size_t)(k % kRing) * slot;
    const int nd = min(kDiag, S - k * kDiag);
#pragma unroll 2
    for (int dd = 0; dd < nd; ++dd) {
      const int d = k * kDiag + dd;
      float4 f01 = make_float4(kNone, kNone, kNone, kNone), f23 = f01;
      if (act) {
        const float4* src = reinterpret_cast<const float4*>(blk + dd * ld + u0);
        f01 = src[0];
        f23 = src[1];
      }
      const float fx[4] = {f01.x, f01.z, f23.x, f23.z}, fy[4] = {f01.y, f01.w, f23.y, f23.w};
      const float up = __shfl_up_sync(0xffffffffu, stepOut[3], 1);
      float left[4], m[4], e[4], a[4];
      left[0] = lane ? up : kNone;
#pragma unroll
      for (int r = 1; r < 4; ++r) left[r] = stepOut[r - 1];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        m[r] = fmaxf(left[r], stayIn[r]);
        e[r] = ex2_approx(-fabsf(left[r] - stayIn[r]));
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) a[r] = m[r] + lg2_approx(1.0f + e[r]);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        stayIn[r] = a[r] + fx[r];
        stepOut[r] = a[r] + fy[r];
      }
      if (act) *reinterpret_cast<float4*>(al + d * ld + u0) = make_float4(a[0], a[1], a[2], a[3]);
      if (d == S - 1) {
#pragma unroll
        for (int r = 0; r < 4; ++r)
          if (u0 + r == U - 1) {
            cost = -stayIn[r] * kLn2F;
            owner = true;
          }
      }
    }
  }
  if (!ok) {  // a copy never landed: make the failure visible in the result
    if (lane == 0) {  // give the copies still in flight a bounded time to land
      for (int j = kFail; j < min(kFail + kRing, nBlocks); ++j) {
        const unsigned long long t1 = global_timer_ns();
        while (!mbar_try_wait(&bar[j % kRing], (j / kRing) & 1) &&
               global_timer_ns() - t1 < 50000000ull) {
        }
      }
    }
    cost = __int_as_float(0x7fc00000);
    owner = (lane == 0);
  }
  if (owner) finish_cost_w(costs, b, cost, B, lossSum, ticket);
}

// ---------------------------------------------------------------------------
// reverse occupancy sweep
// ---------------------------------------------------------------------------
// With g(t,u) the occupancy of node (t,u) (the reference's dalphas, sign dropped):
//   stay(t,u) = g(t+1,u) * FB(t,u),  FB = 2^((alpha(t,u) + blank arc) - alpha(t+1,u))
//   step(t,u) = g(t,u+1) * FL(t,u),  FL = 2^((alpha(t,u) + label arc) - alpha(t,u+1))
//   (alphas and arcs in log2 units; the parenthesised sums are rounded exactly as in the alpha
//   kernel, so FB and FL of the arcs entering a node add up to 1 to within the error of ex2/lg2)
//   g(t,u) = stay + step,            g(T-1,U-1) = 1 (the terminating blank, booked as stay)
// Warp 0 runs the recursion on (FB, FL) pairs staged in shared memory and hands (stay, step)
// back the same way.  The helper warps (kHelperGroups groups of four, thread <-> label position
// u, the diagonals of a block dealt round-robin to the groups): one thread issues the bulk
// copies of the arc terms and the alphas, kRing-1 blocks ahead; all of them turn the block
// after the current one into (FB, FL), write the (stay, step) of the block before it to the
// skewed lattices stayS / stepS, and accumulate per label position sum_t stay -> pBlank[u],
// sum_t step -> pLabel[u] in a fixed order (per group, the groups' partial sums added in
// group order at the end).
// Block k holds the diagonals dTop(k) = S-1-16k down to dLo(k) = max(dTop-15, 0).
constexpr int kHelperGroups = 4;  // helper group j takes the diagonals dd = j (mod 4) of a block
constexpr int kGammaThreads = 32 + 128 * kHelperGroups;

__global__ void __launch_bounds__(kGammaThreads) gamma_warp_kernel(
    const float2* __restrict__ arcs, const float* __restrict__ alphas, int ld, i64 latStride,
    const int* __restrict__ inLens, const int* __restrict__ labLens, float* __restrict__ stayS,
    float* __restrict__ stepS, float* __restrict__ pBlank, float* __restrict__ pLabel, int maxT,
    int maxU, int* status) {
  extern __shared__ __align__(128) uint8_t smemG[];
  // ring slot: arcs of kDiag diagonals, then alphas of kDiag+1 diagonals (+ one spare row)
  const int arcBytes = kDiag * ld * 8, slotBytes = arcBytes + (kDiag + 2) * ld * 4;
  float2 (*F)[kDiag][128] = reinterpret_cast<float2 (*)[kDiag][128]>(smemG + kRing * slotBytes);
  float2 (*G)[kDiag][128] = F + 2;
  __shared__ uint64_t bar[kRing];
  __shared__ int abortFlag;
  __shared__ float sAcc[kHelperGroups][2][128];
  const int b = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  const bool empty = (T <= 0 || U <= 0);
  // padded tails of the per-position outputs are defined (zero)
  for (int u = (empty ? 0 : U) + tid; u < maxU; u += kGammaThreads) {
    pBlank[(i64)b * maxU + u] = 0.0f;
    pLabel[(i64)b * maxU + u] = 0.0f;
  }
  if (empty) return;
  const float2* ar = arcs + (i64)b * latStride;
  const float* al = alphas + (i64)b * latStride;
  float* sS = stayS + (i64)b * latStride;
  float* pS = stepS + (i64)b * latStride;
  const int S = T + U - 1;
  const int nBlocks = (S + kDiag - 1) / kDiag;

  if (tid == 0) {
    for (int s = 0; s < kRing; ++s) mbar_init(&bar[s], 1);
    abortFlag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  auto issue = [&](int k) {  // one thread
    if (k < nBlocks) {
      const int dTop = S - 1 - k * kDiag, dLo = max(dTop - (kDiag - 1), 0), nd = dTop - dLo + 1;
      uint8_t* dst = smemG + (size_t)(k % kRing) * slotBytes;
      const uint32_t b1 = (uint32_t)(nd * ld) * 8u, b2 = (uint32_t)((nd + 1) * ld) * 4u;
      mbar_arrive_expect_tx(&bar[k % kRing], b1 + b2);
      bulk_load_1d(dst, ar + (size_t)dLo * ld, b1, &bar[k % kRing]);
      bulk_load_1d(dst + arcBytes, al + (size_t)dLo * ld, b2, &bar[k % kRing]);
    }
  };
  const int hu = (tid - 32) & 127;   // helper threads: label position
  const int hg = (tid - 32) >> 7;    //                 group
  float accB = 0.0f, accL = 0.0f;
  auto stage = [&](int k) -> bool {  // helpers: (FB, FL) of block k -> F[k & 1]
    bool ok = mbar_wait(&bar[k % kRing], (k / kRing) & 1, &abortFlag, status, kStatusTimeoutTma);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return ok;
    const int dTop = S - 1 - k * kDiag, dLo = max(dTop - (kDiag - 1), 0), nd = dTop - dLo + 1;
    if (hu >= ld) {  // beyond the row: no node
      for (int dd = hg; dd < nd; dd += kHelperGroups) F[k & 1][dd][hu] = make_float2(0.0f, 0.0f);
      return ok;
    }
    const uint8_t* src = smemG + (size_t)(k % kRing) * slotBytes;
    const float2* tb = reinterpret_cast<const float2*>(src);
    const float* aa = reinterpret_cast<const float*>(src + arcBytes);
#pragma unroll 4
    for (int dd = hg; dd < nd; dd += kHelperGroups) {
      const int row = dTop - dd - dLo, t = dTop - dd - hu;
      const float2 arc = tb[row * ld + hu];
      const float a = aa[row * ld + hu], adn = aa[(row + 1) * ld + hu];
      const float art = aa[(row + 1) * ld + hu + 1];
      const bool valid = hu < U && t >= 0 && t < T;
      float2 f;
      f.x = (valid && t < T - 1) ? ex2_approx((a + arc.x) - adn) : 0.0f;
      if (t == T - 1 && hu == U - 1) f.x = 1.0f;  // terminating blank, fed by g(T,U-1) := 1
      f.y = (valid && hu < U - 1) ? ex2_approx((a + arc.y) - art) : 0.0f;
      F[k & 1][dd][hu] = f;
    }
    return ok;
  };
  auto post = [&](int k) {  // helpers: (stay, step) of block k -> global, running sums
    if (hu >= U) return;
    const int dTop = S - 1 - k * kDiag, nd = min(kDiag, dTop + 1);
#pragma unroll 4
    for (int dd = hg; dd < nd; dd += kHelperGroups) {
      const int d = dTop - dd, t = d - hu;
      if (t >= 0 && t < T) {
        const float2 g = G[k & 1][dd][hu];
        sS[d * ld + hu] = g.x;
        pS[d * ld + hu] = g.y;
        accB += g.x;
        accL += g.y;
      }
    }
  };

  int issuedN = 0;  // thread 32: blocks whose copies were issued
  if (tid == 32)
    for (; issuedN < kRing - 1; ++issuedN) issue(issuedN);
  if (warp > 0) stage(0);
  __syncthreads();

  // recursion warp: lane l owns u = 4l + r; the value crossing from u+1 is the lane's own
  // for r < 3 and comes from lane l+1 by one shuffle per diagonal for r = 3
  const int u0 = 4 * lane;
  float g[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) g[r] = (u0 + r == U - 1) ? 1.0f : 0.0f;

  bool ok = true;
  for (int k = 0; k < nBlocks && ok; ++k) {
    if (warp > 0) {
      if (tid == 32) {
        fence_proxy_async_smem();  // the slot refilled next was read two blocks ago
        issue(issuedN++);
      }
      if (k > 0) post(k - 1);
      if (k + 1 < nBlocks) stage(k + 1);
    } else {
      const int nd = min(kDiag, S - k * kDiag);
#pragma unroll 4
      for (int dd = 0; dd < nd; ++dd) {
        const float4* src = reinterpret_cast<const float4*>(&F[k & 1][dd][u0]);
        const float4 f01 = src[0], f23 = src[1];
        const float dn = __shfl_down_sync(0xffffffffu, g[0], 1);
        const float right3 = (lane < 31) ? dn : 0.0f;
        float4 o01, o23;
        o01.x = g[0] * f01.x;  o01.y = g[1] * f01.y;       // u0:   stay, step
        o01.z = g[1] * f01.z;  o01.w = g[2] * f01.w;       // u0+1
        o23.x = g[2] * f23.x;  o23.y = g[3] * f23.y;       // u0+2
        o23.z = g[3] * f23.z;  o23.w = right3 * f23.w;     // u0+3
        g[0] = o01.x + o01.y;
        g[1] = o01.z + o01.w;
        g[2] = o23.x + o23.y;
        g[3] = o23.z + o23.w;
        float4* dst = reinterpret_cast<float4*>(&G[k & 1][dd][u0]);
        dst[0] = o01;
        dst[1] = o23;
      }
    }
    __syncthreads();
    ok = (*(volatile int*)&abortFlag) == 0;
  }
  if (warp > 0) {
    if (ok) post(nBlocks - 1);
    sAcc[hg][0][hu] = accB;
    sAcc[hg][1][hu] = accL;
  }
  __syncthreads();
  if (warp > 0 && hg == 0 && hu < U) {
    float sb = 0.0f, sl = 0.0f;
#pragma unroll
    for (int j = 0; j < kHelperGroups; ++j) {
      sb += sAcc[j][0][hu];
      sl += sAcc[j][1][hu];
    }
    const float bad = __int_as_float(0x7fc00000);  // a copy never landed: visible in the result
    pBlank[(i64)b * maxU + hu] = ok ? sb : bad;
    pLabel[(i64)b * maxU + hu] = ok ? ((hu < U - 1) ? sl : 0.0f) : bad;
  }
  if (!ok && tid == 32) {  // give the copies still in flight a bounded time to land
    for (int j = max(0, min(issuedN, nBlocks) - kRing); j < min(issuedN, nBlocks); ++j) {
      const unsigned long long t1 = global_timer_ns();
      while (!mbar_try_wait(&bar[j % kRing], (j / kRing) & 1) &&
             global_timer_ns() - t1 < 50000000ull) {
      }
    }
  }
}

template <typename K>
void allow_dyn_smem(K kernel, int bytes) {
  TB200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

}  // namespace

bool lattice_warp_supported(Dims d) { return d.maxU >= 1 && d.maxU <= 128; }

void launch_alpha_warp(const float2* arcs, float* costs, float* alphasS, SkewGeom g,
                       const int* inLens, const int* labLens, Dims d, float* lossSum,
                       unsigned* ticket, int* status, cudaStream_t stream) {
  if (d.B <= 0) return;
  const int smem = kRing * kDiag * g.ld * 8;
  ScopedKernel sk("alpha_warp", stream);
  allow_dyn_smem(alpha_warp_kernel, smem);
  alpha_warp_kernel<<<d.B, 32, smem, stream>>>(arcs, costs, alphasS, g.ld, g.stride, g.nDiag,
                                               inLens, labLens, d.B, d.maxT, d.maxU, lossSum,
                                               ticket, status);
  TB200_CHECK_LAUNCH();
}

void launch_gamma_warp(const float2* arcs, const float* alphasS, SkewGeom g, const int* inLens,
                       const int* labLens, float* stayS, float* stepS, float* pBlank,
                       float* pLabel, Dims d, int* status, cudaStream_t stream) {
  if (d.B <= 0) return;
  const int slotBytes = kDiag * g.ld * 8 + (kDiag + 2) * g.ld * 4;
  const int smem = kRing * slotBytes + 4 * kDiag * 128 * (int)sizeof(float2);
  ScopedKernel sk("gamma_warp", stream);
  allow_dyn_smem(gamma_warp_kernel, smem);
  gamma_warp_kernel<<<d.B, kGammaThreads, smem, stream>>>(arcs, alphasS, g.ld, g.stride, inLens,
                                                          labLens, stayS, stepS, pBlank, pLabel,
                                                          d.maxT, d.maxU, status);
  TB200_CHECK_LAUNCH();
}

}  // namespace tb200
