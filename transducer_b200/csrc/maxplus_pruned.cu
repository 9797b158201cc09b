// best[b,t,u] = max over v != blank of (E[b,t,v] + P[b,u,v]) WITHOUT visiting every v: an exact
// branch-and-bound form of the loop the reference runs inside its Viterbi sweep
// (transducer/transducer_cpu.cpp:156-169, transducer_cuda.cu:233-242).
//
// For every frame t the (up to) kETop largest entries of E[t,:] are listed, with thE[t] = the
// largest entry NOT listed; for every label position u the (up to) kPTop largest entries of
// P[u,:] are listed in descending order, with thP[u] = the largest entry not listed.  For a
// node (t,u):
//   1. L = max over the frame's list of E[t,v] + P[u,v]           (P read from a transposed copy)
//   2. walk the position's list while  P[u,v_j] + thE[t] > L:  L = max(L, E[t,v_j] + P[u,v_j])
//   3. the node is settled if  thP[u] + thE[t] <= L.
// Every v outside the frame's list has E[t,v] <= thE[t].  The position's list is descending, so
// when the walk stops at entry j no later entry can reach L (fp32 addition is monotone in each
// argument: fl(E+P) <= fl(thE + P_j) <= L), and thP[u] <= P_j, so test 3 then holds by itself;
// when the walk runs off the end of the list, test 3 decides.  The maximum of fp32 sums does
// not depend on the order in which they are taken, so a settled L is bit-identical to the full
// loop.  Nodes that are not settled are appended to a list and evaluated in full by a second
// kernel; if they are more than the list holds (flat scores: pruning does not pay), the full
// kernel redoes every node.  Correctness never depends on how good the lists are, only the
// speed does -- a list that could not be built (its copy did not land) is replaced by an empty
// one with an infinite bound.
//
// Which v attains the maximum is resolved after the backtrack, on the path only (as with the
// full kernel).
#include "kernels.h"
#include "profile.h"
#include "sm100.cuh"

namespace tb200 {
namespace {
using namespace sm100;

constexpr int kETop = 128;    // entries listed per frame
constexpr int kPTop = 128;    // entries listed per label position
constexpr int kBatchP = 8;    // list entries fetched at a time beyond the head
constexpr int kPre = 32;      // entries of every position's list kept in shared memory
constexpr int kPRows = kPTop + kBatchP;   // rows of a position list in memory
// A frame's list in memory: offsets v*us (int) [kETop], values [kETop], bound, count, padding.
// Entries from `count` up to the next multiple of 32 repeat entry 0.
constexpr int kEWords = 2 * kETop + 4;
constexpr size_t kSelSmemBytes = 96 * 1024;   // rows staged per CTA of the selection kernels

__device__ __forceinline__ int warp_sum_int(int v) { return __reduce_add_sync(0xffffffffu, v); }

// Copies a row into shared memory (vp = V rounded up to 4; the padding becomes -inf): one bulk
// copy where the row is 16-byte aligned, plain loads otherwise.  Warp-wide; `bar` is this
// warp's barrier (initialised, first use).  Returns false if the copy did not land in time
// (recorded in the status word).
__device__ __forceinline__ bool stage_row(const float* __restrict__ src, float* dst, int V, int vp,
                                          int lane, uint64_t* bar, int* abortFlag, int* status) {
  bool ok = true;
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar, (uint32_t)V * 4u);
      bulk_load_1d(dst, src, (uint32_t)V * 4u, bar);
    }
    ok = mbar_wait(bar, 0, abortFlag, status, kStatusTimeoutTma);
    if (!ok) {   // give the copy a bounded time to finish before shared memory is released
      const unsigned long long t1 = global_timer_ns();
      while (!mbar_try_wait(bar, 0) && global_timer_ns() - t1 < 50000000ull) {
      }
    }
    ok = __all_sync(0xffffffffu, ok);
  } else {
#pragma unroll 8
    for (int v = lane; v < vp; v += 32) dst[v] = (v < V) ? __ldg(src + v) : neg_inf();
  }
  __syncwarp();
  return ok;
}

// Number of entries of the staged row above `th` (NaN and -inf never count).
__device__ __forceinline__ int count_above(const float* row, int vp, float th, int lane) {
  int c = 0;
  const float4* r4 = reinterpret_cast<const float4*>(row);
  for (int i = lane; i < (vp >> 2); i += 32) {
    const float4 x = r4[i];
    c += (x.x > th) + (x.y > th) + (x.z > th) + (x.w > th);
  }
  return warp_sum_int(c);
}

// Upper quantile of the standard normal (Abramowitz & Stegun 26.2.22), p in (0, 0.5].
__device__ __forceinline__ float normal_quantile(float p) {
  const float t = sqrtf(-2.0f * logf(p));
  return t - (2.30753f + 0.27061f * t) / (1.0f + t * (0.99229f + 0.04481f * t));
}

// Overwrites the blank entry of the staged row with -inf (from here on it is never counted or
// listed) and returns a threshold with at most K entries of the row above it (and, where the
// data allow, at least K/2).  Warp-wide.  -inf selects every entry that is not -inf.
__device__ float pick_threshold(float* row, int V, int vp, int blank, int K, int lane) {
  // maximum, minimum, mean and spread (only the starting point of the search, so the blank
  // entry may take part): first without looking at the values ...
  const float4* r4 = reinterpret_cast<const float4*>(row);
  float mx = neg_inf(), mn = pos_inf(), s = 0.0f, s2 = 0.0f;
  int n = vp;
  for (int i = lane; i < (vp >> 2); i += 32) {
    const float4 x = r4[i];
    mx = fmaxf(fmaxf(mx, fmaxf(x.x, x.y)), fmaxf(x.z, x.w));
    mn = fminf(fminf(mn, fminf(x.x, x.y)), fminf(x.z, x.w));
    s += (x.x + x.y) + (x.z + x.w);
    s2 += (x.x * x.x + x.y * x.y) + (x.z * x.z + x.w * x.w);
  }
  mx = warp_max(mx); mn = -warp_max(-mn); s = warp_sum(s); s2 = warp_sum(s2);
  __syncwarp();
  if (lane == 0 && blank >= 0 && blank < V) row[blank] = neg_inf();
  __syncwarp();
  bool plain = true;   // every entry finite: nothing is above the maximum, all but blank above -inf
  if (!(s2 < 3.0e38f) || !(mn > -3.0e38f)) {
    plain = false;
    // ... and over the finite entries only if some are not
    mx = neg_inf(); mn = pos_inf(); s = 0.0f; s2 = 0.0f; n = 0;
    for (int v = lane; v < vp; v += 32) {
      const float x = row[v];
      if (x > -3.0e38f && x < 3.0e38f) {
        mx = fmaxf(mx, x); mn = fminf(mn, x); s += x; s2 += x * x; ++n;
      }
    }
    mx = warp_max(mx); mn = -warp_max(-mn); s = warp_sum(s); s2 = warp_sum(s2); n = warp_sum_int(n);
  }
  if (plain ? vp - 1 <= K : count_above(row, vp, neg_inf(), lane) <= K) return neg_inf();
  if (n == 0) return pos_inf();                       // only +inf entries, more than K of them
  float hi = mx;                                      // invariant: count(> hi) <= K
  if (!plain && count_above(row, vp, hi, lane) > K) return pos_inf();
  float lo = mn;
  const float mean = s / n, sd = sqrtf(fmaxf(s2 / n - mean * mean, 0.0f));
  float probe = mean + sd * normal_quantile(fminf(0.5f, 0.75f * K / (float)n));
  if (!(probe > lo && probe < hi)) probe = 0.5f * lo + 0.5f * hi;
  for (int it = 0; it < 24; ++it) {
    if (!(probe > lo && probe < hi)) break;
    const int c = count_above(row, vp, probe, lane);
    if (c > K) lo = probe;
    else {
      hi = probe;
      if (2 * c >= K) break;
    }
    probe = 0.5f * lo + 0.5f * hi;
  }
  return hi;
}

// Copies the entries above `th` to out (index, value bits; any order; at most K of them by the
// choice of th), sets *cnt (shared memory) to their number and returns the largest entry not
// copied.  Warp-wide.  Rows of up to 4096 words: one branch-free pass marks the entries in a
// bit mask per lane, then every lane copies its own few (a branch per entry would be taken by
// the whole warp ~100 times per row); longer rows: appended one by one through the counter.
__device__ __forceinline__ float collect_above(const float* row, int vp, float th, int lane,
                                               int2* out, int* cnt) {
  float rest = neg_inf();
  const float4* r4 = reinterpret_cast<const float4*>(row);
  const int n4 = vp >> 2;
  if (n4 <= 1024) {
    unsigned mask[4] = {0u, 0u, 0u, 0u};   // bit 4q + k of word q / 8: entry k of float4 lane + 32q
#pragma unroll
    for (int q = 0; q < 32; ++q) {
      const int i = lane + 32 * q;
      if (i < n4) {
        const float4 x4 = r4[i];
        const float x[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const bool sel = x[k] > th;
          mask[q >> 3] |= sel ? 1u << ((4 * q + k) & 31) : 0u;
          rest = sel ? rest : fmaxf(rest, x[k]);   // (NaN entries are ignored, as by the reference's '>')
        }
      }
    }
    const int mine = __popc(mask[0]) + __popc(mask[1]) + __popc(mask[2]) + __popc(mask[3]);
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    int at = incl - mine;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      unsigned m = mask[w];
      while (m) {
        const int e = 32 * w + __ffs(m) - 1;   // entry (e & 3) of float4 lane + 32 * (e >> 2)
        m &= m - 1;
        const int v = 4 * (lane + 32 * (e >> 2)) + (e & 3);
        out[at++] = make_int2(v, __float_as_int(row[v]));
      }
    }
    if (lane == 31) *cnt = incl;
  } else {
    for (int i = lane; i < n4; i += 32) {
      const float4 x4 = r4[i];
      const float x[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (x[k] > th) out[atomicAdd(cnt, 1)] = make_int2(4 * i + k, __float_as_int(x[k]));
        else rest = fmaxf(rest, x[k]);
      }
    }
  }
  __syncwarp();
  return warp_max(rest);
}

// ---- P transposed: PT[b][v][u] (u < maxU-1, row stride us) ---------------------------
__global__ void __launch_bounds__(256) transpose_p_kernel(const float* __restrict__ P,
                                                          float* __restrict__ PT,
                                                          const int* __restrict__ labLens, int maxU,
                                                          int V, int us) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z, v0 = blockIdx.x * 32, u0 = blockIdx.y * 32;
  const int nLab = min(labLens[b] + 1, maxU) - 1;
  if (u0 >= nLab) return;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int k = ty; k < 32; k += 8) {
    const int u = u0 + k, v = v0 + tx;
    tile[k][tx] = (u < nLab && v < V) ? P[((i64)b * maxU + u) * V + v] : neg_inf();
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const int v = v0 + k, u = u0 + tx;
    if (v < V && u < us) PT[((i64)b * V + v) * us + u] = tile[tx][k];
  }
}

// ---- per frame: the kETop largest entries (unordered) and the largest entry not listed ----
// One warp per row, `warps` rows per CTA, every row staged in shared memory.
__global__ void select_e_kernel(const float* __restrict__ E, int* __restrict__ eList,
                                const int* __restrict__ inLens, int maxT, int V, int vp,
                                int blank, int us, int warps, int* status) {
  extern __shared__ __align__(16) float staged[];
  __shared__ uint64_t bars[8];
  __shared__ int aborts[8], counts[8];
  __shared__ int2 picked[8][kETop];
  const int b = blockIdx.y, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * warps + w;
  if (lane == 0) {
    mbar_init(&bars[w], 1);
    aborts[w] = 0;
    counts[w] = 0;
    fence_mbar_init();
  }
  __syncwarp();
  if (t >= min(inLens[b], maxT)) return;
  int* out = eList + ((i64)b * maxT + t) * kEWords;
  float* row = staged + (size_t)w * vp;
  if (!stage_row(E + ((i64)b * maxT + t) * V, row, V, vp, lane, &bars[w], &aborts[w], status)) {
    // nothing listed and an infinite bound: every node of the frame is evaluated in full
    if (lane == 0) {
      out[2 * kETop] = __float_as_int(pos_inf());
      out[2 * kETop + 1] = 0;
    }
    return;
  }
  const float th = pick_threshold(row, V, vp, blank, kETop, lane);
  const float rest = collect_above(row, vp, th, lane, picked[w], &counts[w]);
  const int n = counts[w], nPad = (n + 31) & ~31;
  for (int k = lane; k < nPad; k += 32) {
    const int2 c = picked[w][k < n ? k : 0];
    out[k] = c.x * us;
    out[kETop + k] = c.y;
  }
  if (lane == 0) {
    out[2 * kETop] = __float_as_int(rest);
    out[2 * kETop + 1] = n;
  }
}

// ---- per label position: the kPTop largest entries in descending order ----
// pList[b][j][u] (row stride us): entry j of position u as (v, value bits); the entry after the
// last one is (0, -inf).  pMeta[b][u] = (largest value not listed, entries).
__global__ void select_p_kernel(const float* __restrict__ P, int2* __restrict__ pList,
                                int2* __restrict__ pMeta, const int* __restrict__ labLens,
                                int maxU, int V, int vp, int blank, int us, int warps,
                                int* status) {
  extern __shared__ __align__(16) float staged[];
  __shared__ uint64_t bars[8];
  __shared__ int aborts[8], counts[8];
  const int b = blockIdx.y, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int u = blockIdx.x * warps + w;
  if (lane == 0) {
    mbar_init(&bars[w], 1);
    aborts[w] = 0;
    counts[w] = 0;
    fence_mbar_init();
  }
  __syncwarp();
  if (u >= min(labLens[b] + 1, maxU) - 1) return;
  float* row = staged + (size_t)w * vp;
  int2* sel = reinterpret_cast<int2*>(staged + (size_t)warps * vp) + (size_t)w * kPTop;
  int2* out = pList + (i64)b * kPRows * us + u;
  if (!stage_row(P + ((i64)b * maxU + u) * V, row, V, vp, lane, &bars[w], &aborts[w], status)) {
    // an empty list that bounds nothing: the position's nodes are evaluated in full
    if (lane == 0) {
      out[0] = make_int2(0, __float_as_int(neg_inf()));
      pMeta[(i64)b * us + u] = make_int2(__float_as_int(pos_inf()), 0);
    }
    return;
  }
  const float th = pick_threshold(row, V, vp, blank, kPTop, lane);
  const float rest = collect_above(row, vp, th, lane, sel, &counts[w]);
  const int n = counts[w];
  // rank sort (value descending, then index ascending) on one 64-bit key per entry, four
  // entries per lane at a time
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(sel);
  for (int i = lane; i < n; i += 32) {
    const int2 c = sel[i];
    const unsigned bits = (unsigned)c.y;   // order-preserving map of the value (no NaN here)
    const unsigned ord = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    keys[i] = ((unsigned long long)ord << 32) | (unsigned)(0x7fffffff - c.x);
  }
  __syncwarp();
  for (int i0 = 0; i0 < n; i0 += 128) {
    unsigned long long me[4];
    int rank[4] = {0, 0, 0, 0};
#pragma unroll
    for (int m = 0; m < 4; ++m) me[m] = keys[min(i0 + lane + 32 * m, n - 1)];
    for (int k = 0; k < n; ++k) {
      const unsigned long long o = keys[k];
#pragma unroll
      for (int m = 0; m < 4; ++m) rank[m] += (o > me[m]) ? 1 : 0;
    }
#pragma unroll
    for (int m = 0; m < 4; ++m)
      if (i0 + lane + 32 * m < n) {
        const unsigned ord = (unsigned)(me[m] >> 32);
        const unsigned bits = (ord & 0x80000000u) ? (ord & 0x7fffffffu) : ~ord;
        out[(i64)rank[m] * us] = make_int2(0x7fffffff - (int)(unsigned)me[m], (int)bits);
      }
  }
  if (lane == 0) {
    out[(i64)n * us] = make_int2(0, __float_as_int(neg_inf()));
    pMeta[(i64)b * us + u] = make_int2(__float_as_int(rest), n);
  }
}

// ---- the pruned evaluation ---------------------------------------------------------
struct PrunedParams {
  const float* E;
  const float* PT;
  const int* eList;
  const int2* pList;
  const int2* pMeta;
  float* best;
  const int* inLens;
  const int* labLens;
  unsigned long long* fbList;
  int* fbCount;
  int* status;
  int maxT, maxU, V, us, groups, warpsPerGroup, framesPerCta, fbCap;
};

// CTA = `groups` groups of `warpsPerGroup` warps over a chunk of frames of one utterance.  A
// group takes every groups-th frame: its row of E and its list arrive by bulk copy, one frame
// ahead, in the group's own pair of buffers; inside a group, warp w evaluates the label
// positions 32w .. 32w+31 (+ 32*warpsPerGroup ...) of the frame.  The heads of the positions'
// lists (kPre entries, 16-bit indices) sit in shared memory for the whole CTA.
__global__ void __launch_bounds__(512) maxplus_pruned_kernel(const PrunedParams p) {
  extern __shared__ __align__(16) uint8_t stagedBytes[];
  __shared__ uint64_t bar[4][2];
  __shared__ int abortFlag;
  const int b = blockIdx.y;
  const int T = min(p.inLens[b], p.maxT), nLab = min(p.labLens[b] + 1, p.maxU) - 1;
  const int tBeg = blockIdx.x * p.framesPerCta;
  if (nLab <= 0 || tBeg >= T) return;
  const int tEnd = min(T, tBeg + p.framesPerCta);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = warp / p.warpsPerGroup, wInG = warp - grp * p.warpsPerGroup;
  const bool leader = wInG == 0 && lane == 0;
  const int nUB = (nLab + 31) >> 5;
  const float* e = p.E + (i64)b * p.maxT * p.V;
  const bool bulk = (p.V & 3) == 0 && (reinterpret_cast<uintptr_t>(e) & 15) == 0;
  // (rows are kept a multiple of 16 bytes apart, so that the lists behind them stay aligned)
  const int rowStride = (p.V + 3) & ~3;
  const size_t rowBytes = (size_t)rowStride * 4, listBytes = (size_t)kEWords * 4;
  const size_t bufBytes = rowBytes + listBytes;
  uint8_t* myBufs = stagedBytes + (size_t)grp * 2 * bufBytes;
  float* sPreVal = reinterpret_cast<float*>(stagedBytes + (size_t)p.groups * 2 * bufBytes);  // [kPre][us]
  float* sThP = sPreVal + (size_t)kPre * p.us;                                                // [us]
  unsigned short* sPreIdx = reinterpret_cast<unsigned short*>(sThP + p.us);                   // [kPre][us]
  if (threadIdx.x == 0) {
    for (int g = 0; g < 4; ++g) {
      mbar_init(&bar[g][0], 1);
      mbar_init(&bar[g][1], 1);
    }
    abortFlag = 0;
    fence_mbar_init();
  }
  {  // the heads of the lists and the positions' bounds
    const int2* pl0 = p.pList + (i64)b * kPRows * p.us;
    for (int i = threadIdx.x; i < kPre * p.us; i += blockDim.x) {
      const int2 c = __ldg(pl0 + i);
      sPreVal[i] = __int_as_float(c.y);
      sPreIdx[i] = (unsigned short)c.x;
    }
    for (int i = threadIdx.x; i < p.us; i += blockDim.x)
      sThP[i] = i < nLab ? __int_as_float(__ldg(p.pMeta + (i64)b * p.us + i).x) : neg_inf();
  }
  __syncthreads();
  const int first = tBeg + grp;                       // my group's frames: first, first + groups, ...
  const int nMine = first < tEnd ? (tEnd - first + p.groups - 1) / p.groups : 0;
  const int groupThreads = p.warpsPerGroup * 32;
  auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(groupThreads) : "memory"); };
  auto fetch = [&](int i) {   // my group's i-th frame -> buffer i & 1
    const int t = first + i * p.groups, buf = i & 1;
    float* rows = reinterpret_cast<float*>(myBufs + buf * bufBytes);
    int* ls = reinterpret_cast<int*>(myBufs + buf * bufBytes + rowBytes);
    const int* el = p.eList + ((i64)b * p.maxT + t) * kEWords;
    if (bulk) {
      if (leader) {
        mbar_arrive_expect_tx(&bar[grp][buf], (uint32_t)(rowBytes + listBytes));
        bulk_load_1d(rows, e + (i64)t * p.V, (uint32_t)rowBytes, &bar[grp][buf]);
        bulk_load_1d(ls, el, (uint32_t)listBytes, &bar[grp][buf]);
      }
    } else {
      const int tid = wInG * 32 + lane;
      for (int v = tid; v < p.V; v += groupThreads) rows[v] = __ldg(e + (i64)t * p.V + v);
      for (int k = tid; k < kEWords; k += groupThreads) ls[k] = __ldg(el + k);
    }
  };
  if (nMine > 0) fetch(0);
  bool ok = true;
  for (int i = 0; i < nMine; ++i) {
    const int t = first + i * p.groups, buf = i & 1;
    group_sync();   // every warp of the group has left frame i-1, whose buffer the next copy takes
    if (i + 1 < nMine) fetch(i + 1);
    if (bulk) {
      ok = mbar_wait(&bar[grp][buf], (i >> 1) & 1, &abortFlag, p.status, kStatusTimeoutTma);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
    } else {
      group_sync();
    }
    const float* row = reinterpret_cast<const float*>(myBufs + buf * bufBytes);
    const int* el = reinterpret_cast<const int*>(myBufs + buf * bufBytes + rowBytes);
    const int4* off4 = reinterpret_cast<const int4*>(el);
    const float4* val4 = reinterpret_cast<const float4*>(el + kETop);
    const float thE = __int_as_float(el[2 * kETop]);
    const int nE = el[2 * kETop + 1];
    for (int ub = wInG; ub < nUB; ub += p.warpsPerGroup) {
      const int u = ub * 32 + lane;
      const bool mine = u < nLab;
      float L = neg_inf();
      // 1. the frame's own candidates against this position, 16 loads in flight
      const float* pt = p.PT + (i64)b * p.V * p.us + u;   // (u < us: the stride is a multiple of 32)
      for (int j4 = 0; 4 * j4 < nE; j4 += 4) {
        float x[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int4 o = off4[j4 + q];
          x[4 * q] = __ldg(pt + o.x); x[4 * q + 1] = __ldg(pt + o.y);
          x[4 * q + 2] = __ldg(pt + o.z); x[4 * q + 3] = __ldg(pt + o.w);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 ev = val4[j4 + q];
          L = fmaxf(fmaxf(L, ev.x + x[4 * q]), ev.y + x[4 * q + 1]);
          L = fmaxf(fmaxf(L, ev.z + x[4 * q + 2]), ev.w + x[4 * q + 3]);
        }
      }
      // 2. the position's candidates, best first, while one of them could still win: the
      //    head of the list from shared memory, the rest kBatchP entries at a time (a lane
      //    that has stopped ignores what was fetched for it; the entry behind a list is -inf)
      bool live = mine;
      for (int k0 = 0; k0 < kPre && __any_sync(0xffffffffu, live); k0 += 4) {
#pragma unroll
        for (int k = k0; k < k0 + 4; ++k) {
          const float pv = sPreVal[k * p.us + u];
          const int v = sPreIdx[k * p.us + u];
          live = live && (pv + thE > L);
          if (live) L = fmaxf(L, row[v] + pv);
        }
      }
      const int2* pl = p.pList + (i64)b * kPRows * p.us + u;
      for (int j0 = kPre; __any_sync(0xffffffffu, live); j0 += kBatchP) {
        int2 c[kBatchP];
#pragma unroll
        for (int k = 0; k < kBatchP; ++k) c[k] = __ldg(pl + (i64)(j0 + k) * p.us);
#pragma unroll
        for (int k = 0; k < kBatchP; ++k) {
          const float pv = __int_as_float(c[k].y);
          live = live && (pv + thE > L);
          if (live) L = fmaxf(L, row[c[k].x] + pv);
        }
      }
      // 3. settled?
      if (mine) {
        const i64 node = ((i64)b * p.maxT + t) * p.maxU + u;
        if (sThP[u] + thE > L) {
          const int at = atomicAdd(p.fbCount, 1);
          if (at < p.fbCap) p.fbList[at] = (unsigned long long)node;
        } else {
          p.best[node] = L;
        }
      }
    }
  }
  if (!ok) {
    // A copy did not land (recorded in the status word): declare the list overflowed, so that
    // the full evaluation redoes every node, and give the group's copies a bounded time.
    if (leader) {
      atomicAdd(p.fbCount, p.fbCap + 1);
      for (int k = 0; k < 2; ++k) {
        const unsigned long long t1 = global_timer_ns();
        while (!mbar_try_wait(&bar[grp][k], 0) && !mbar_try_wait(&bar[grp][k], 1) &&
               global_timer_ns() - t1 < 50000000ull) {
        }
      }
    }
    group_sync();
  }
}

// Nodes that were not settled: the full loop, one warp per node.  Does nothing when the list
// overflowed (the full kernel then redoes every node).
__global__ void __launch_bounds__(256) maxplus_listed_kernel(
    const float* __restrict__ E, const float* __restrict__ P, float* __restrict__ best,
    const unsigned long long* __restrict__ fbList, const int* __restrict__ fbCount, int fbCap,
    int maxT, int maxU, int V, int blank) {
  const int n = *fbCount;
  if (n > fbCap) return;
  const int lane = threadIdx.x & 31;
  for (int i = blockIdx.x * 8 + (threadIdx.x >> 5); i < n; i += gridDim.x * 8) {
    const i64 node = (i64)fbList[i];
    const int u = (int)(node % maxU);
    const i64 bt = node / maxU;
    const i64 b = bt / maxT;
    const float* e = E + bt * V;
    const float* pr = P + (b * maxU + u) * V;
    float m = neg_inf();
    for (int v = lane; v < V; v += 32)
      if (v != blank) m = fmaxf(m, e[v] + pr[v]);
    m = warp_max(m);
    if (lane == 0) best[node] = m;
  }
}

int label_stride(Dims d) { return (int)round_up64(d.maxU > 1 ? d.maxU - 1 : 1, 32); }
int fallback_capacity(Dims d) {
  const i64 nodes = (i64)d.B * d.maxT * (d.maxU - 1);
  return (int)std::min<i64>(1 << 22, std::max<i64>(4096, nodes / 64));
}
// one row fits a selection warp's staging area, two rows a group of the evaluation kernel,
// and an index fits the 16 bits of a list head
constexpr int kMaxWords = 16384;

struct Scratch {
  float* PT;
  int2* pList;
  int2* pMeta;
  int* eList;
  unsigned long long* fbList;
  int* fbCount;
  size_t bytes;
  Scratch(void* base, Dims d) {
    const size_t us = (size_t)label_stride(d);
    size_t off = 0;
    auto take = [&](size_t n) {
      const size_t at = off;
      off += (n + 255) & ~size_t(255);
      return base ? static_cast<char*>(base) + at : nullptr;
    };
    PT = reinterpret_cast<float*>(take(sizeof(float) * d.B * (size_t)d.V * us));
    pList = reinterpret_cast<int2*>(take(sizeof(int2) * d.B * (size_t)kPRows * us));
    pMeta = reinterpret_cast<int2*>(take(sizeof(int2) * d.B * us));
    eList = reinterpret_cast<int*>(take(sizeof(int) * d.B * (size_t)d.maxT * kEWords));
    fbList = reinterpret_cast<unsigned long long*>(take(sizeof(unsigned long long) * fallback_capacity(d)));
    fbCount = reinterpret_cast<int*>(take(256));
    bytes = off;
  }
};

}  // namespace

bool maxplus_pruned_supported(Dims d) {
  // below ~1000 words the lists are most of the row
  return d.B > 0 && d.B <= 65535 && d.maxT > 0 && d.maxU > 1 && d.V >= 1024 && d.V <= kMaxWords &&
         (i64)d.V * label_stride(d) < (i64(1) << 31);
}

size_t maxplus_pruned_scratch_bytes(Dims d) {
  if (!maxplus_pruned_supported(d)) return 0;
  return Scratch(nullptr, d).bytes;
}

void launch_maxplus_pruned(const float* E, const float* P, float* best, const int* inLens,
                           const int* labLens, Dims d, void* scratch, int* status,
                           cudaStream_t stream) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 1) return;
  Scratch s(scratch, d);
  const int us = label_stride(d);
  {
    ScopedKernel sk("maxplus_transpose", stream);
    TB200_CUDA_CHECK(cudaMemsetAsync(s.fbCount, 0, sizeof(int), stream));
    transpose_p_kernel<<<dim3(div_up(d.V, 32), div_up(d.maxU - 1, 32), d.B), 256, 0, stream>>>(
        P, s.PT, labLens, d.maxU, d.V, us);
  }
  TB200_CHECK_LAUNCH();
  const int vp = (int)round_up64(d.V, 4);
  const size_t rowB = (size_t)vp * sizeof(float);
  {
    ScopedKernel sk("maxplus_select_p", stream);
    const int wp = (int)std::max<size_t>(1, std::min<size_t>(8, kSelSmemBytes / (rowB + kPTop * sizeof(int2))));
    const size_t smemP = wp * (rowB + kPTop * sizeof(int2));
    TB200_CUDA_CHECK(cudaFuncSetAttribute(select_p_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smemP));
    select_p_kernel<<<dim3(div_up(d.maxU - 1, wp), d.B), wp * 32, smemP, stream>>>(
        P, s.pList, s.pMeta, labLens, d.maxU, d.V, vp, d.blank, us, wp, status);
  }
  TB200_CHECK_LAUNCH();
  {
    ScopedKernel sk("maxplus_select_e", stream);
    const int we = (int)std::max<size_t>(1, std::min<size_t>(8, kSelSmemBytes / rowB));
    const size_t smemE = we * rowB;
    TB200_CUDA_CHECK(cudaFuncSetAttribute(select_e_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smemE));
    select_e_kernel<<<dim3(div_up(d.maxT, we), d.B), we * 32, smemE, stream>>>(
        E, s.eList, inLens, d.maxT, d.V, vp, d.blank, us, we, status);
  }
  TB200_CHECK_LAUNCH();
  PrunedParams p;
  p.E = E; p.PT = s.PT; p.eList = s.eList; p.pList = s.pList; p.pMeta = s.pMeta; p.best = best;
  p.inLens = inLens; p.labLens = labLens; p.fbList = s.fbList; p.fbCount = s.fbCount;
  p.maxT = d.maxT; p.maxU = d.maxU; p.V = d.V; p.us = us;
  p.status = status;
  // warps of a group: one per 32 label positions (at most 8); groups: as many as keep the CTA
  // near ten warps and its buffers within ~100 KB
  p.warpsPerGroup = std::min(8, div_up(d.maxU - 1, 32));
  const size_t perGroup = 2 * (rowB + kEWords * sizeof(int));
  p.groups = (int)std::max<size_t>(1, std::min<size_t>(std::min(4, 10 / p.warpsPerGroup),
                                                       (100 * 1024) / perGroup));
  p.framesPerCta = 16 * p.groups;
  p.fbCap = fallback_capacity(d);
  const size_t smem = p.groups * perGroup +
                      (size_t)us * (kPre * (sizeof(float) + sizeof(unsigned short)) + sizeof(float));
  const int threads = 32 * p.warpsPerGroup * p.groups;
  {
    ScopedKernel sk("maxplus_pruned", stream);
    TB200_CUDA_CHECK(cudaFuncSetAttribute(maxplus_pruned_kernel,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    maxplus_pruned_kernel<<<dim3(div_up(d.maxT, p.framesPerCta), d.B), threads, smem, stream>>>(p);
  }
  TB200_CHECK_LAUNCH();
  {
    ScopedKernel sk("maxplus_listed", stream);
    maxplus_listed_kernel<<<592, 256, 0, stream>>>(E, P, best, s.fbList, s.fbCount, p.fbCap,
                                                   d.maxT, d.maxU, d.V, d.blank);
  }
  TB200_CHECK_LAUNCH();
  // the full kernel, which returns at once unless the list overflowed
  launch_maxplus(E, P, best, inLens, labLens, d, stream, s.fbCount, p.fbCap);
}

}  // namespace tb200
