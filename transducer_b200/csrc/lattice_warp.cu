// Lattice sweeps for label axes of at most 128 positions: the recursion runs in ONE warp.
//
// The wavefront kernels of lattice.cu spend a block barrier and a shared-memory exchange on
// every anti-diagonal.  Here lane l of a single warp owns the label positions u = l + 32 r;
// all nodes of a diagonal are independent, the value that crosses from u-1 (or u+1) arrives
// by one warp shuffle per r, and nothing else sits on the dependent chain:
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
template <int NR>
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
  float stayIn[NR], stepOut[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) stayIn[r] = stepOut[r] = kNone;
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
      float2 f[NR];
      float rot[NR], left[NR], m[NR], e[NR], a[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) f[r] = blk[dd * ld + lane + 32 * r];
#pragma unroll
      for (int r = 0; r < NR; ++r) rot[r] = __shfl_sync(0xffffffffu, stepOut[r], (lane + 31) & 31);
#pragma unroll
      for (int r = 0; r < NR; ++r) left[r] = lane ? rot[r] : (r ? rot[r ? r - 1 : 0] : kNone);
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        m[r] = fmaxf(left[r], stayIn[r]);
        e[r] = ex2_approx(-fabsf(left[r] - stayIn[r]));
      }
#pragma unroll
      for (int r = 0; r < NR; ++r) a[r] = m[r] + lg2_approx(1.0f + e[r]);
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        stayIn[r] = a[r] + f[r].x;
        stepOut[r] = a[r] + f[r].y;
        al[d * ld + lane + 32 * r] = a[r];
      }
      if (d == S - 1) {
#pragma unroll
        for (int r = 0; r < NR; ++r)
          if (lane + 32 * r == U - 1) {
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
// back the same way.  Warps 1..4 (thread <-> label position u): one thread issues the bulk
// copies of the arc terms and the alphas, kRing-1 blocks ahead; all of them turn the block
// after the current one into (FB, FL), write the (stay, step) of the block before it to the
// skewed lattices stayS / stepS, and accumulate per label position sum_t stay -> pBlank[u],
// sum_t step -> pLabel[u] in a fixed order.
// Block k holds the diagonals dTop(k) = S-1-16k down to dLo(k) = max(dTop-15, 0).
constexpr int kGammaThreads = 160;

template <int NR>
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
  const int hu = tid - 32;  // helper threads: label position
  float accB = 0.0f, accL = 0.0f;
  auto stage = [&](int k) -> bool {  // helpers: (FB, FL) of block k -> F[k & 1]
    bool ok = mbar_wait(&bar[k % kRing], (k / kRing) & 1, &abortFlag, status, kStatusTimeoutTma);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok || hu >= ld) return ok;
    const int dTop = S - 1 - k * kDiag, dLo = max(dTop - (kDiag - 1), 0), nd = dTop - dLo + 1;
    const uint8_t* src = smemG + (size_t)(k % kRing) * slotBytes;
    const float2* tb = reinterpret_cast<const float2*>(src);
    const float* aa = reinterpret_cast<const float*>(src + arcBytes);
#pragma unroll 4
    for (int dd = 0; dd < nd; ++dd) {
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
    for (int dd = 0; dd < nd; ++dd) {
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

  float g[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) g[r] = (lane + 32 * r == U - 1) ? 1.0f : 0.0f;

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
        float2 f[NR], o[NR];
        float rot[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) f[r] = F[k & 1][dd][lane + 32 * r];
#pragma unroll
        for (int r = 0; r < NR; ++r) rot[r] = __shfl_sync(0xffffffffu, g[r], (lane + 1) & 31);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          const float right = (lane < 31) ? rot[r] : (r < NR - 1 ? rot[r < NR - 1 ? r + 1 : r] : 0.0f);
          o[r].x = g[r] * f[r].x;
          o[r].y = right * f[r].y;
          g[r] = o[r].x + o[r].y;
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) G[k & 1][dd][lane + 32 * r] = o[r];
      }
    }
    __syncthreads();
    ok = (*(volatile int*)&abortFlag) == 0;
  }
  if (warp > 0) {
    if (ok) post(nBlocks - 1);
    if (hu < U) {
      const float bad = __int_as_float(0x7fc00000);  // a copy never landed: visible in the result
      pBlank[(i64)b * maxU + hu] = ok ? accB : bad;
      pLabel[(i64)b * maxU + hu] = ok ? ((hu < U - 1) ? accL : 0.0f) : bad;
    }
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
#define CALL(NR)                                                                                \
  do {                                                                                          \
    allow_dyn_smem(alpha_warp_kernel<NR>, smem);                                                \
    alpha_warp_kernel<NR><<<d.B, 32, smem, stream>>>(arcs, costs, alphasS, g.ld, g.stride,      \
                                                     g.nDiag, inLens, labLens, d.B, d.maxT,     \
                                                     d.maxU, lossSum, ticket, status);          \
  } while (0)
  switch (g.ld / 32) {
    case 1: CALL(1); break;
    case 2: CALL(2); break;
    case 3: CALL(3); break;
    default: CALL(4); break;
  }
#undef CALL
  TB200_CHECK_LAUNCH();
}

void launch_gamma_warp(const float2* arcs, const float* alphasS, SkewGeom g, const int* inLens,
                       const int* labLens, float* stayS, float* stepS, float* pBlank,
                       float* pLabel, Dims d, int* status, cudaStream_t stream) {
  if (d.B <= 0) return;
  const int slotBytes = kDiag * g.ld * 8 + (kDiag + 2) * g.ld * 4;
  const int smem = kRing * slotBytes + 4 * kDiag * 128 * (int)sizeof(float2);
  ScopedKernel sk("gamma_warp", stream);
#define CALL(NR)                                                                               \
  do {                                                                                         \
    allow_dyn_smem(gamma_warp_kernel<NR>, smem);                                               \
    gamma_warp_kernel<NR><<<d.B, kGammaThreads, smem, stream>>>(                               \
        arcs, alphasS, g.ld, g.stride, inLens, labLens, stayS, stepS, pBlank, pLabel, d.maxT,  \
        d.maxU, status);                                                                       \
  } while (0)
  switch (g.ld / 32) {
    case 1: CALL(1); break;
    case 2: CALL(2); break;
    case 3: CALL(3); break;
    default: CALL(4); break;
  }
#undef CALL
  TB200_CHECK_LAUNCH();
}

}  // namespace tb200
