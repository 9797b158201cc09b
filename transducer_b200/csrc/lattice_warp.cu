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
#include <algorithm>

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
// rounding as here, or the occupancies stop being a conserved flow.
//
// REBASED alphas.  After 2000 frames an alpha is of magnitude 1e4 and an fp32 ulp there is
// 1e-3: the reference carries its alphas at that magnitude (transducer_cpu.cpp:30-79) and its
// gradients are 2e-3..6e-3 of their maximum away from a float64 evaluation for it (measured).
// Here every block of 16 diagonals stores its alphas relative to an offset of its own: at the
// start of block k the whole carried state is lowered by delta_k = the floor of its largest
// entry (an integer, so that the running offset -- needed only for the final cost -- adds up
// exactly), which keeps every stored number below ~500 in magnitude (ulp 3e-5).  delta_k is
// written to `deltas` for the reverse sweep, which subtracts it at the same point of the same
// sum.  The loss and the gradients then sit ~1e-4 from the float64 result.
// Lane l owns the label positions u = 4l + r, r = 0..3: the value crossing from u-1 is the
// lane's own for r > 0 and comes from lane l-1 by ONE shuffle per diagonal for r = 0; the four
// arc pairs and the four alphas of a lane are contiguous (two 16-byte loads, one store).  The
// pace is set by the dependent chain of a diagonal -- the four ex2 and then the four lg2 queue
// in the quarter-rate special-function unit -- so the loop holds nothing else: no validity
// tests, no address arithmetic beyond an increment, the final cost read after the loop.
// (Cutting the label axis over two or four warps that run a block apart, with one or two
// positions per lane, was measured and is slower: every node then waits for a shuffle.)
__global__ void __launch_bounds__(32) alpha_warp_kernel(
    const float2* __restrict__ arcs, float* __restrict__ costs, float* __restrict__ alphas,
    float* __restrict__ deltas, int ld, i64 latStride, int nDiag,
    const int* __restrict__ inLens, const int* __restrict__ labLens, int B, int maxT, int maxU,
    float* lossSum, unsigned* ticket, int* status) {
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
  // large negative and finite: the identity of the recursion without -inf arithmetic
  const float kNone = __uint_as_float(kNoArcBits);

  if (lane == 0) {
    for (int s = 0; s < kRing; ++s) mbar_init(&bar[s], 1);
    abortFlag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  int issuedN = 0;  // lane 0: blocks whose copies were issued
  auto issue = [&](int k) {  // lane 0: rows [16k, 16k+16) of arcs -> ring slot k % kRing
    if (k < nBlocks) {
      const int rows = min(kDiag, nDiag - k * kDiag);
      const uint32_t bytes = (uint32_t)(rows * ld) * 8u;
      mbar_arrive_expect_tx(&bar[k % kRing], bytes);
      bulk_load_1d(ring + (size_t)(k % kRing) * slot, ar + (size_t)k * slot, bytes, &bar[k % kRing]);
      issuedN = k + 1;
    }
  };
  if (lane == 0)
    for (int k = 0; k < kRing - 1; ++k) issue(k);

  // lanes past the row (ld is a multiple of 4, at most 128) compute on a clamped column: finite
  // values that are never stored and never reach a lane below them
  const int u0 = 4 * lane, uc = min(u0, ld - 4);
  const bool act = u0 < ld;
  float stayIn[4], stepOut[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) stayIn[r] = stepOut[r] = kNone;
  if (lane == 0) stayIn[0] = 0.0f;  // alpha(0,0) = 0
  bool ok = true;
  float up = kNone;  // stepOut[3] of the lane below, one diagonal back
  float offset = 0.0f;  // sum of the deltas so far: an integer, exact in fp32
  float* dl = deltas + (i64)b * ((nDiag + kDiag - 1) / kDiag);
  float nextDelta = 0.0f;  // by how much the state is lowered at the start of the next block
  for (int k = 0; k < nBlocks; ++k) {
    if (k > 0) {
      // rebase (entries of nodes outside the lattice are ~ -6e29 and stay there)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        stayIn[r] -= nextDelta;
        stepOut[r] -= nextDelta;
      }
      up -= nextDelta;
      offset += nextDelta;
      if (lane == 0) dl[k] = nextDelta;
    }
    // The slot refilled next was read by ALL lanes one block ago: the warp barrier orders those
    // reads before lane 0's proxy fence and copy issue.
    __syncwarp();
    if (lane == 0) {
      fence_proxy_async_smem();
      issue(k + kRing - 1);
    }
    ok = mbar_wait(&bar[k % kRing], (k / kRing) & 1, &abortFlag, status, kStatusTimeoutTma);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const float4* blk = reinterpret_cast<const float4*>(ring + (size_t)(k % kRing) * slot + uc);
    const int d0 = k * kDiag, nd = min(kDiag, S - d0), ld4 = ld / 2;  // float4 per diagonal
    float* out = al + (size_t)d0 * ld + u0;
    // The delta applied at the start of the NEXT block is the floor of the largest entry of
    // the state now, at the start of this one: the warp-wide maximum then has a whole block to
    // arrive, off the dependent chain.  (By then the state has sunk by another ~16 arcs; all
    // that matters is that the stored numbers stay small: below ~1000, ulp 6e-5.)
    {
      float m = fmaxf(fmaxf(stayIn[0], stayIn[1]), fmaxf(stayIn[2], stayIn[3]));
      m = fmaxf(m, fmaxf(fmaxf(stepOut[0], stepOut[1]), fmaxf(stepOut[2], stepOut[3])));
      nextDelta = (float)__reduce_max_sync(0xffffffffu, __float2int_rd(fmaxf(m, -1.0e9f)));
    }
#pragma unroll 4
    for (int dd = 0; dd < nd; ++dd) {
      const float4 f01 = blk[dd * ld4], f23 = blk[dd * ld4 + 1];
      const float fx[4] = {f01.x, f01.z, f23.x, f23.z}, fy[4] = {f01.y, f01.w, f23.y, f23.w};
      // Position 3 first: its result feeds the shuffle of the next diagonal; position 0 last: it
      // waits for the shuffle of this one.  (A warp issues in order.)
      float left[4], m[4], e[4], a[4];
      left[0] = lane ? up : kNone;
#pragma unroll
      for (int r = 1; r < 4; ++r) left[r] = stepOut[r - 1];
#pragma unroll
      for (int r = 3; r >= 0; --r) {
        m[r] = fmaxf(left[r], stayIn[r]);
        e[r] = ex2_approx(-fabsf(left[r] - stayIn[r]));
      }
#pragma unroll
      for (int r = 3; r >= 0; --r) {
        a[r] = m[r] + lg2_approx(1.0f + e[r]);
        stayIn[r] = a[r] + fx[r];
        stepOut[r] = a[r] + fy[r];
        if (r == 3) up = __shfl_up_sync(0xffffffffu, stepOut[3], 1);
      }
      if (act) *reinterpret_cast<float4*>(out + dd * ld) = make_float4(a[0], a[1], a[2], a[3]);
    }
  }
  if (!ok) {  // a copy never landed: make the failure visible in the result
    if (lane == 0) {  // give the copies still in flight a bounded time to land
      for (int j = max(0, issuedN - kRing); j < issuedN; ++j) {
        const unsigned long long t1 = global_timer_ns();
        while (!mbar_try_wait(&bar[j % kRing], (j / kRing) & 1) &&
               global_timer_ns() - t1 < 50000000ull) {
        }
      }
      finish_cost_w(costs, b, __int_as_float(0x7fc00000), B, lossSum, ticket);
    }
    return;
  }
  // the last diagonal holds only the terminal node (T-1, U-1); its blank arc ends the path
#pragma unroll
  for (int r = 0; r < 4; ++r)
    if (u0 + r == U - 1) finish_cost_w(costs, b, -(stayIn[r] + offset) * kLn2F, B, lossSum, ticket);
}

// ---------------------------------------------------------------------------
// reverse occupancy sweep
// ---------------------------------------------------------------------------
// With g(t,u) the occupancy of node (t,u) (the reference's dalphas, sign dropped):
//   stay(t,u) = g(t+1,u) * FB(t,u),  FB = 2^((alpha(t,u) + blank arc) - alpha(t+1,u))
//   step(t,u) = g(t,u+1) * FL(t,u),  FL = 2^((alpha(t,u) + label arc) - alpha(t,u+1))
//   (alphas and arcs in log2 units; the parenthesised sums are rounded exactly as in the alpha
//   kernel, so FB and FL of the arcs entering a node add up to 1 to within the error of ex2/lg2.
//   The stored alphas are relative to a per-block offset, see alpha_warp_kernel: where the
//   successors' diagonal opens a new block of the alpha kernel, that block's delta is
//   subtracted from the sum first, exactly as the alpha kernel lowered its carried state.)
//   g(t,u) = stay + step,            g(T-1,U-1) = 1 (the terminating blank, booked as stay)
// Warp 0 runs the recursion on (FB, FL) pairs staged in shared memory and hands (stay, step)
// back the same way.  The helper warps (kHelperGroups groups of four, thread <-> label position
// u, the diagonals of a block dealt round-robin to the groups) turn the block
// after the current one into (FB, FL), write the (stay, step) of the block before it to the
// skewed lattices stayS / stepS, and accumulate per label position sum_t stay -> pBlank[u],
// sum_t step -> pLabel[u] in a fixed order (per group, the groups' partial sums added in
// group order at the end).  One thread of a last warp issues the bulk copies of the arc terms
// and the alphas, kRing-1 blocks ahead (the proxy fence and the copy issue cost ~500 cycles,
// which no helper warp should carry).
// Block k holds the diagonals dTop(k) = S-1-16k down to dLo(k) = max(dTop-15, 0).
constexpr int kHelperGroups = 4;  // helper group j takes the diagonals dd = j (mod 4) of a block
constexpr int kPerHelper = kDiag / kHelperGroups;  // diagonals of a block per helper thread
constexpr int kCopyTid = 32 + 128 * kHelperGroups;  // first thread of the copy warp
constexpr int kGammaThreads = kCopyTid + 32;

__global__ void __launch_bounds__(kGammaThreads) gamma_warp_kernel(
    const float2* __restrict__ arcs, const float* __restrict__ alphas,
    const float* __restrict__ deltas, int nDiag, int ld, i64 latStride,
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
  // the alpha kernel's per-block deltas of this utterance, staged once (after the F/G buffers)
  float* dl = reinterpret_cast<float*>(G + 2);
  {
    const float* src = deltas + (i64)b * ((nDiag + kDiag - 1) / kDiag);
    for (int k = 1 + tid; k < nBlocks; k += kGammaThreads) dl[k] = src[k];
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
    // all operands of the thread's diagonals first (clamped, unconditional), then the arithmetic:
    // the shared-memory latency is paid once per block, not once per diagonal
    float2 arc[kPerHelper];
    float a[kPerHelper], adn[kPerHelper], art[kPerHelper];
    // Exactly one diagonal of the block, ddB, has its successors on a diagonal that opens a block
    // of the alpha kernel (dNext = dTop - ddB + 1 a multiple of 16): there the carried sums were
    // lowered by that block's delta before they entered it.
    const int ddB = (dTop + 1) & (kDiag - 1);
    const int dNextB = dTop - ddB + 1;
    const float deltaB = (dNextB >= kDiag && dNextB < S) ? dl[dNextB / kDiag] : 0.0f;
#pragma unroll
    for (int j = 0; j < kPerHelper; ++j) {
      const int row = dTop - min(hg + j * kHelperGroups, nd - 1) - dLo;
      arc[j] = tb[row * ld + hu];
      a[j] = aa[row * ld + hu];
      adn[j] = aa[(row + 1) * ld + hu];
      art[j] = aa[(row + 1) * ld + hu + 1];
    }
#pragma unroll
    for (int j = 0; j < kPerHelper; ++j) {
      const int dd = hg + j * kHelperGroups, t = dTop - dd - hu;
      const bool valid = hu < U && t >= 0 && t < T;
      const float dlt = (dd == ddB) ? deltaB : 0.0f;
      float2 f;
      f.x = (valid && t < T - 1) ? ex2_approx(((a[j] + arc[j].x) - dlt) - adn[j]) : 0.0f;
      if (t == T - 1 && hu == U - 1) f.x = 1.0f;  // terminating blank, fed by g(T,U-1) := 1
      f.y = (valid && hu < U - 1) ? ex2_approx(((a[j] + arc[j].y) - dlt) - art[j]) : 0.0f;
      if (dd < nd) F[k & 1][dd][hu] = f;
    }
    return ok;
  };
  auto post = [&](int k) {  // helpers: (stay, step) of block k -> global, running sums
    if (hu >= U) return;
    const int dTop = S - 1 - k * kDiag, nd = min(kDiag, dTop + 1);
    float2 g[kPerHelper];
#pragma unroll
    for (int j = 0; j < kPerHelper; ++j) g[j] = G[k & 1][min(hg + j * kHelperGroups, nd - 1)][hu];
#pragma unroll
    for (int j = 0; j < kPerHelper; ++j) {
      const int dd = hg + j * kHelperGroups, d = dTop - dd, t = d - hu;
      if (dd < nd && t >= 0 && t < T) {
        sS[d * ld + hu] = g[j].x;
        pS[d * ld + hu] = g[j].y;
        accB += g[j].x;
        accL += g[j].y;
      }
    }
  };

  const bool helper = tid >= 32 && tid < kCopyTid;
  int issuedN = 0;  // copy thread: blocks whose copies were issued
  if (tid == kCopyTid)
    for (; issuedN < kRing - 1; ++issuedN) issue(issuedN);
  if (helper) stage(0);
  __syncthreads();

  // recursion warp: lane l owns u = 4l + r; the value crossing from u+1 is the lane's own
  // for r < 3 and comes from lane l+1 by one shuffle per diagonal for r = 3
  const int u0 = 4 * lane;
  float g[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) g[r] = (u0 + r == U - 1) ? 1.0f : 0.0f;

  bool ok = true;
  for (int k = 0; k < nBlocks && ok; ++k) {
    if (helper) {
      if (k > 0) post(k - 1);
      if (k + 1 < nBlocks) stage(k + 1);
    } else if (tid == kCopyTid) {
      fence_proxy_async_smem();  // the slot refilled next was read two blocks ago
      issue(issuedN++);
    } else if (warp == 0) {
      const int nd = min(kDiag, S - k * kDiag);
#pragma unroll 4
      for (int dd = 0; dd < nd; ++dd) {
        const float4* src = reinterpret_cast<const float4*>(&F[k & 1][dd][u0]);
        const float4 f01 = src[0], f23 = src[1];
        // (lane 31 gets its own g[0] back: harmless, the label arc of position 127 never
        // exists, its factor f23.w is 0)
        const float right3 = __shfl_down_sync(0xffffffffu, g[0], 1);
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
  if (helper) {
    if (ok) post(nBlocks - 1);
    sAcc[hg][0][hu] = accB;
    sAcc[hg][1][hu] = accL;
  }
  __syncthreads();
  if (helper && hg == 0 && hu < U) {
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
  if (!ok && tid == kCopyTid) {  // give the copies still in flight a bounded time to land
    for (int j = max(0, min(issuedN, nBlocks) - kRing); j < min(issuedN, nBlocks); ++j) {
      const unsigned long long t1 = global_timer_ns();
      while (!mbar_try_wait(&bar[j % kRing], (j / kRing) & 1) &&
             global_timer_ns() - t1 < 50000000ull) {
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Viterbi: max-plus sweep in one warp, bit-packed decisions, backtrack, label argmax
// ---------------------------------------------------------------------------
// Per node the sweep needs E[t,blank], LN[t,u] and best[t,u] (the max-plus label score of
// maxplus.cu); viterbi_prep_kernel lays them out skewed as one float4 per node, so that a block
// of diagonals is one bulk copy.  The scores are formed in the reference's operation order,
// ((score + E[t,blank]) + P[u,blank]) - LN and (score + best) - LN, so every comparison, and
// with it the path, is bit-identical to transducer_cpu.cpp:145-222.
// Nodes outside the lattice hold the record (-1e30, 0, -1e30): whatever enters them leaves as
// about -1e30, which loses every comparison against a real score.  With that the sweep needs
// no case distinctions at all: the blank arc into frame 0 and the label arc into position 0
// come from such nodes (or from the -inf fed to lane 0) and lose by themselves.
constexpr float kNoNode = -1.0e30f;

__global__ void __launch_bounds__(256) viterbi_fill_kernel(float4* __restrict__ nodes, i64 n) {
  const float4 none = make_float4(kNoNode, 0.0f, kNoNode, 0.0f);
  for (i64 k = (i64)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += (i64)gridDim.x * blockDim.x)
    nodes[k] = none;
}

__global__ void __launch_bounds__(256) viterbi_prep_kernel(
    const float* __restrict__ E, const float* __restrict__ LN, const float* __restrict__ best,
    float4* __restrict__ nodes, const int* __restrict__ inLens, const int* __restrict__ labLens,
    int maxT, int maxU, int V, int blank, int ld, i64 latStride) {
  __shared__ float tLn[32][33], tBs[32][33], tEb[32];
  const int b = blockIdx.z, t0 = blockIdx.y * 32, u0 = blockIdx.x * 32;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  if (t0 >= T || u0 >= U) return;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const float* ln = LN + (i64)b * maxT * maxU;
  const float* bs = best + (i64)b * maxT * maxU;
  const int u = u0 + lane, uc = min(u, U - 1), ub = min(u, max(U - 2, 0));
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int tt = w * 4 + k, tc = min(t0 + tt, T - 1);
    tLn[tt][lane] = ln[(i64)tc * maxU + uc];
    // the label arc of the last position does not exist
    tBs[tt][lane] = (u < U - 1) ? bs[(i64)tc * maxU + ub] : kNoNode;
  }
  if (threadIdx.x < 32)
    tEb[lane] = E[((i64)b * maxT + min(t0 + lane, T - 1)) * V + blank];
  __syncthreads();
  for (int ds = w; ds < 63; ds += 8) {
    const int tt = ds - lane;
    if (tt >= 0 && tt < 32 && t0 + tt < T && u < U)
      nodes[(i64)b * latStride + (i64)(t0 + u0 + ds) * ld + u] =
          make_float4(tEb[tt], tLn[tt][lane], tBs[tt][lane], 0.0f);
  }
}

// Decision bits of the single-warp sweep are packed along the DIAGONAL d = t + u: word
// [(b*maxU + u)*wordsD + d/32] bit (d%32) is 1 when node (t,u) was entered by the label arc
// from (t,u-1).  All positions then flush their words at the same steps.
__host__ __device__ inline int viterbi_words_d(int maxT, int maxU) { return (maxT + maxU + 31) / 32; }

// NPL label positions per lane: u = NPL*lane + r.  One warp per utterance sweeps, then its
// first thread backtracks and writes, for every label position, the frame at which the label was
// emitted (frames [B,maxU], -1 where there is none); viterbi_labels_kernel resolves the labels.
// The decision bits live in shared memory behind the ring where they fit (decInSmem), in the
// decBits scratch otherwise: the backtrack is a chain of dependent reads of them.
template <int NPL>
__global__ void __launch_bounds__(32) viterbi_warp_kernel(
    const float* __restrict__ P, const float4* __restrict__ nodes,
    int ld, i64 latStride, int nDiag, int ringDepth, uint32_t* __restrict__ decBits, int decInSmem,
    int* __restrict__ frames, int* __restrict__ labelsOut, const int* __restrict__ inLens,
    const int* __restrict__ labLens, int maxT, int maxU, int V, int blank, int* status) {
  extern __shared__ __align__(128) uint8_t smemV[];
  __shared__ uint64_t bar[kRing];
  __shared__ int abortFlag;
  __shared__ int sFrame[256];  // frame at which label u-1 was emitted (U <= 256 here)
  const int b = blockIdx.x, i = threadIdx.x, lane = i & 31, warp = i >> 5;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  int* fr = frames + (i64)b * maxU;
  if (T <= 0 || U <= 0) {
    for (int u = i; u < maxU; u += 32) fr[u] = -1;
    return;
  }
  const float* p = P + (i64)b * maxU * V;
  const float4* nd = nodes + (i64)b * latStride;
  const int wordsD = viterbi_words_d(maxT, maxU);
  uint32_t* dec = decInSmem
                      ? reinterpret_cast<uint32_t*>(smemV + (size_t)ringDepth * kDiag * ld * 16)
                      : decBits + (i64)b * maxU * wordsD;
  for (int u = i; u < 256; u += 32) sFrame[u] = -1;
  if (i == 0) {
    for (int s = 0; s < kRing; ++s) mbar_init(&bar[s], 1);
    abortFlag = 0;
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == 0) {
    float4* ring = reinterpret_cast<float4*>(smemV);  // [ringDepth][kDiag * ld]
    const int S = T + U - 1;
    const int nBlocks = (S + kDiag - 1) / kDiag;
    const int slot = kDiag * ld;
    auto issue = [&](int k) {  // lane 0
      if (k < nBlocks) {
        const int rows = min(kDiag, nDiag - k * kDiag);
        const uint32_t bytes = (uint32_t)(rows * ld) * 16u;
        mbar_arrive_expect_tx(&bar[k % ringDepth], bytes);
        bulk_load_1d(ring + (size_t)(k % ringDepth) * slot, nd + (size_t)k * slot, bytes,
                     &bar[k % ringDepth]);
      }
    };
    if (lane == 0)
      for (int k = 0; k < ringDepth - 1; ++k) issue(k);
    const int u0 = NPL * lane;
    float pbl[NPL], stay[NPL], stepOut[NPL];
    uint32_t bits[NPL];
    uint32_t* decU[NPL];
#pragma unroll
    for (int r = 0; r < NPL; ++r) {
      pbl[r] = (u0 + r < U) ? p[(i64)(u0 + r) * V + blank] : 0.0f;
      stay[r] = stepOut[r] = kNoNode;
      bits[r] = 0u;
      decU[r] = dec + (i64)min(u0 + r, maxU - 1) * wordsD;
    }
    if (lane == 0) stay[0] = 0.0f;  // score 0 enters the origin (as if by its blank arc)
    bool ok = true;
    int kFail = 0;
    for (int k = 0; k < nBlocks; ++k) {
      __syncwarp();  // all lanes have read the slot that is refilled next
      if (lane == 0) {
        fence_proxy_async_smem();
        issue(k + ringDepth - 1);
      }
      ok = mbar_wait(&bar[k % ringDepth], (k / ringDepth) & 1, &abortFlag, status, kStatusTimeoutTma);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        kFail = k;
        break;
      }
      const float4* blk = ring + (size_t)(k % ringDepth) * slot;
      const int ndg = min(kDiag, S - k * kDiag);
#pragma unroll 2
      for (int dd = 0; dd < ndg; ++dd) {
        const int d = k * kDiag + dd;
        float4 nv[NPL];
#pragma unroll
        for (int r = 0; r < NPL; ++r) nv[r] = blk[dd * ld + min(u0 + r, ld - 1)];
        const float up = __shfl_up_sync(0xffffffffu, stepOut[NPL - 1], 1);
        const uint32_t bit = 1u << (d & 31);
        float left[NPL];
        left[0] = lane ? up : neg_inf();
#pragma unroll
        for (int r = 1; r < NPL; ++r) left[r] = stepOut[r - 1];
#pragma unroll
        for (int r = 0; r < NPL; ++r) {
          // the larger of the two arcs, the blank arc on ties (strict '>', as the reference)
          const bool takeStep = left[r] > stay[r];
          const float sc = takeStep ? left[r] : stay[r];
          bits[r] |= takeStep ? bit : 0u;
          stay[r] = ((sc + nv[r].x) + pbl[r]) - nv[r].y;   // E[t,blank], LN[t,u]
          stepOut[r] = (sc + nv[r].z) - nv[r].y;           // best[t,u]
        }
        if ((d & 31) == 31 || d == S - 1) {
#pragma unroll
          for (int r = 0; r < NPL; ++r) {
            if (u0 + r < U) decU[r][d >> 5] = bits[r];
            bits[r] = 0u;
          }
        }
      }
    }
    if (!ok && lane == 0) {  // give the copies still in flight a bounded time to land
      for (int j = kFail; j < min(kFail + ringDepth, nBlocks); ++j) {
        const unsigned long long t1 = global_timer_ns();
        while (!mbar_try_wait(&bar[j % ringDepth], (j / ringDepth) & 1) &&
               global_timer_ns() - t1 < 50000000ull) {
        }
      }
    }
    __threadfence_block();
  }
  __syncthreads();
  if (abortFlag) {  // a copy never landed (recorded in the status word): no path, labels = -1
    for (int u = i; u < U - 1; u += 32) labelsOut[(i64)b * (maxU - 1) + u] = -1;
    for (int u = i; u < maxU; u += 32) fr[u] = -1;
    return;
  }

  // Backtrack from (T-1,U-1) along row u in diagonal coordinates d = t + u.  Each iteration
  // consumes either one label or one 32-diagonal word of blanks, so it ends within
  // U + (T+U)/32 + 1 iterations; the explicit cap only guards against corrupted scratch.
  // (Node (0,u), u > 0, is always entered by its label arc, so the scan of a row never runs
  // into the bits of nodes before frame 0.)
  if (i == 0) {
    int t = T - 1, u = U - 1;
    int guard = U + wordsD + 2;
    while (u > 0 && t >= 0 && guard-- > 0) {
      const int d = t + u;
      const uint32_t keep = 0xffffffffu >> (31 - (d & 31));
      const uint32_t w = ((volatile uint32_t*)dec)[(i64)u * wordsD + (d >> 5)] & keep;
      if (w == 0u) { t = (d & ~31) - 1 - u; continue; }
      t = (d & ~31) + (31 - __clz(w)) - u;
      sFrame[u] = t;
      --u;
    }
  }
  __syncthreads();
  for (int u = i; u < maxU; u += 32) fr[u] = (u < U) ? sFrame[u] : -1;
}

// Label on each emitting arc of the path: lowest-index argmax over v != blank of
// E[t,v] + P[u-1,v] (strict '>' in index order, as the reference's getMax,
// transducer_cpu.cpp:156-169), one warp per label position, t = frames[b,u].
__global__ void __launch_bounds__(256) viterbi_labels_kernel(
    const float* __restrict__ E, const float* __restrict__ P, const int* __restrict__ frames,
    int* __restrict__ labelsOut, const int* __restrict__ labLens, int B, int maxT, int maxU,
    int V, int blank) {
  const int lane = threadIdx.x & 31;
  const int u = 1 + blockIdx.x * 8 + (threadIdx.x >> 5);
  for (int b = blockIdx.y; b < B; b += gridDim.y) {
  if (u >= min(labLens[b] + 1, maxU)) continue;
  const int t = frames[(i64)b * maxU + u];
  if (t < 0) continue;
  const float* er = E + ((i64)b * maxT + t) * V;
  const float* pr = P + ((i64)b * maxU + u - 1) * V;
  const bool vec4 = (V & 3) == 0 && ((reinterpret_cast<uintptr_t>(er) | reinterpret_cast<uintptr_t>(pr)) & 15) == 0;
  float m = neg_inf();
  int arg = 0x7fffffff;
  if (vec4) {  // 16 loads in flight per lane; each lane still visits its entries in index order
    const float4* e4 = reinterpret_cast<const float4*>(er);
    const float4* p4 = reinterpret_cast<const float4*>(pr);
    const int n4 = V >> 2;
    for (int q0 = lane; q0 < n4; q0 += 128) {
      float4 a[4], c[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int q = min(q0 + 32 * j, n4 - 1);
        a[j] = e4[q];
        c[j] = p4[q];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int q = q0 + 32 * j;
        if (q < n4) {
          const float x[4] = {a[j].x + c[j].x, a[j].y + c[j].y, a[j].z + c[j].z, a[j].w + c[j].w};
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const int v = 4 * q + h;
            if (v != blank && x[h] > m) { m = x[h]; arg = v; }
          }
        }
      }
    }
  } else {
    for (int v = lane; v < V; v += 32) {
      if (v == blank) continue;
      const float x = er[v] + pr[v];
      if (x > m) { m = x; arg = v; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const int a2 = __shfl_xor_sync(0xffffffffu, arg, o);
    if (m2 > m || (m2 == m && a2 < arg)) { m = m2; arg = a2; }
  }
  if (lane == 0) labelsOut[(i64)b * (maxU - 1) + u - 1] = (arg == 0x7fffffff) ? 0 : arg;
  }
}

template <typename K>
void allow_dyn_smem(K kernel, int bytes) {
  TB200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

}  // namespace

bool lattice_warp_supported(Dims d) { return d.maxU >= 1 && d.maxU <= 128; }

size_t lattice_warp_delta_floats(Dims d) {
  const SkewGeom g = skew_geom(d);
  return (size_t)d.B * (size_t)((g.nDiag + kDiag - 1) / kDiag);
}

void launch_alpha_warp(const float2* arcs, float* costs, float* alphasS, float* deltas, SkewGeom g,
                       const int* inLens, const int* labLens, Dims d, float* lossSum,
                       unsigned* ticket, int* status, cudaStream_t stream) {
  if (d.B <= 0) return;
  const int smem = kRing * kDiag * g.ld * 8;
  ScopedKernel sk("alpha_warp", stream);
  allow_dyn_smem(alpha_warp_kernel, smem);
  alpha_warp_kernel<<<d.B, 32, smem, stream>>>(arcs, costs, alphasS, deltas, g.ld, g.stride, g.nDiag,
                                               inLens, labLens, d.B, d.maxT, d.maxU, lossSum,
                                               ticket, status);
  TB200_CHECK_LAUNCH();
}

void launch_gamma_warp(const float2* arcs, const float* alphasS, const float* deltas, SkewGeom g,
                       const int* inLens, const int* labLens, float* stayS, float* stepS, float* pBlank,
                       float* pLabel, Dims d, int* status, cudaStream_t stream) {
  if (d.B <= 0) return;
  const int slotBytes = kDiag * g.ld * 8 + (kDiag + 2) * g.ld * 4;
  const int smem = kRing * slotBytes + 4 * kDiag * 128 * (int)sizeof(float2) +
                   (int)sizeof(float) * ((g.nDiag + kDiag - 1) / kDiag + 1);
  if (smem > 225 * 1024) throw std::invalid_argument("input too long for the single-warp reverse sweep");
  ScopedKernel sk("gamma_warp", stream);
  allow_dyn_smem(gamma_warp_kernel, smem);
  gamma_warp_kernel<<<d.B, kGammaThreads, smem, stream>>>(arcs, alphasS, deltas, g.nDiag, g.ld, g.stride, inLens,
                                                          labLens, stayS, stepS, pBlank, pLabel,
                                                          d.maxT, d.maxU, status);
  TB200_CHECK_LAUNCH();
}

bool viterbi_warp_supported(Dims d) { return d.maxU >= 1 && d.maxU <= 256; }

size_t viterbi_warp_decbits_words(Dims d) {
  // decision bits, then the frames at which the labels are emitted [B,maxU]
  return viterbi_warp_supported(d)
             ? (size_t)d.B * (size_t)d.maxU * (size_t)(viterbi_words_d(d.maxT, d.maxU) + 1)
             : 0;
}

size_t viterbi_warp_nodes(Dims d) {
  const SkewGeom g = skew_geom(d);
  return viterbi_warp_supported(d) ? (size_t)d.B * (size_t)g.stride : 0;
}

void launch_viterbi_warp(const float* E, const float* P, const float* LN, const float* best,
                         float4* nodes, uint32_t* decBits, int* labels, const int* inLens,
                         const int* labLens, Dims d, int* status, cudaStream_t stream) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 0) return;
  const SkewGeom g = skew_geom(d);
  {
    dim3 grid(div_up(d.maxU, 32), div_up(d.maxT, 32), d.B);
    ScopedKernel sk("viterbi_prep", stream);
    viterbi_fill_kernel<<<148 * 8, 256, 0, stream>>>(nodes, (i64)d.B * g.stride);
    viterbi_prep_kernel<<<grid, 256, 0, stream>>>(E, LN, best, nodes, inLens, labLens, d.maxT,
                                                  d.maxU, d.V, d.blank, g.ld, g.stride);
    TB200_CHECK_LAUNCH();
  }
  // shared memory: the decision bits (if they leave room for a ring of at least three blocks
  // of node records), then the ring
  const int slotBytes = kDiag * g.ld * 16;
  const int decBytes = d.maxU * viterbi_words_d(d.maxT, d.maxU) * 4;
  const int room = 216 * 1024;
  const int decInSmem = decBytes + 3 * slotBytes <= room ? 1 : 0;
  const int ringDepth = std::max(2, std::min(kRing, (room - (decInSmem ? decBytes : 0)) / slotBytes));
  const int smem = ringDepth * slotBytes + (decInSmem ? decBytes : 0);
  int* frames = reinterpret_cast<int*>(decBits) +
                (size_t)d.B * d.maxU * viterbi_words_d(d.maxT, d.maxU);
  {
  ScopedKernel sk("viterbi_warp", stream);
#define CALL(NPL)                                                                              \
  do {                                                                                         \
    allow_dyn_smem(viterbi_warp_kernel<NPL>, smem);                                            \
    viterbi_warp_kernel<NPL><<<d.B, 32, smem, stream>>>(                                       \
        P, nodes, g.ld, g.stride, g.nDiag, ringDepth, decBits, decInSmem, frames, labels,      \
        inLens, labLens, d.maxT, d.maxU, d.V, d.blank, status);                                \
  } while (0)
  switch (g.ld / 32) {
    case 1: CALL(1); break;
    case 2: CALL(2); break;
    case 3: CALL(3); break;
    case 4: CALL(4); break;
    case 5: CALL(5); break;
    case 6: CALL(6); break;
    case 7: CALL(7); break;
    default: CALL(8); break;
  }
#undef CALL
  }
  TB200_CHECK_LAUNCH();
  if (d.maxU > 1) {
    ScopedKernel sk("viterbi_labels", stream);
    viterbi_labels_kernel<<<dim3(div_up(d.maxU - 1, 8), std::min(d.B, 65535)), 256, 0, stream>>>(
        E, P, frames, labels, labLens, d.B, d.maxT, d.maxU, d.V, d.blank);
    TB200_CHECK_LAUNCH();
  }
}

}  // namespace tb200
