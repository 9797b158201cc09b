// Emission and prediction gradients in ONE pass over E on the tensor cores.
//
// The reference computes (transducer/torch_binding.py:85-89, after the sparse terms of
// transducer_cpu.cpp:81-143):
//   egrads[t,v] = delta * ( expE[t,v] * sum_u W[t,u] expP[u,v]  - sparse_E[t,v] )
//   pgrads[u,v] = delta * ( expP[u,v] * sum_t W[t,u] expE[t,v]  - sparse_P[u,v] )
// with two batched SGEMMs and ~8 elementwise passes over E-sized tensors, keeping
// expE = exp(E - maxE) from the forward pass.  Here E is read once, expE is recomputed,
// every gradient element is written once, and nothing E-sized is stored.
//
// Work decomposition: one CTA per (utterance b, block of 128 vocabulary columns); it walks
// the frames of the utterance in tiles of TB.  Everything is laid out with the VOCABULARY
// column on the 128 TMEM lanes (UMMA M = 128):
//   GEMM1  D1[v, t] = sum_u expP^T[v,u] * W[t,u]    A = expP^T in TMEM (resident for the whole
//                                                    CTA), B = W tile in smem, K-major
//   GEMM2  D2[v, u] += sum_t expE^T[v,t] * W[t,u]   A = expE^T in TMEM (per tile), B = the W
//                                                    tile again, MN-major.  An MN-major TF32
//                                                    operand must use the 128-byte swizzle with
//                                                    32-byte atoms, so the tile is fetched a
//                                                    second time by a tensor map with that swizzle.
//
// All global<->shared traffic is TMA.  Two rings of shared-memory stages:
//   E ring  raw E tile + the tile's row shifts.  The owner of column v in the exp group turns
//           its column of the tile into exp(E - ref), split hi + lo for TF32, in TMEM; the owner
//           in the gradient group reads it back from TMEM together with D1 and writes the
//           finished gradient over the dead raw tile; a storer thread then writes the tile to
//           egrads with TMA stores (same tensor-map geometry as E) and releases the stage.
//           (Shared-memory bandwidth is the scarce resource of this kernel: per tile the TMA
//           writes, the MMA operand reads and one read + one write by the owners already use
//           most of it, so the exponentials are not written back to shared memory.)
//           The stage also carries the tile's sparse-term rows (blank-arc sums, label-arc
//           occupancies of the labels that fall into this column block).
//   W ring  the two copies of the W tile; released by the two GEMMs alone.
// Roles (20 warps): 8 column-owner warps of the exp group (TMEM lane quarter x frame half;
// raw E -> exp(E - ref) in TMEM), 8 column-owner warps of the gradient group (D1 x exponentials
// from TMEM - sparse terms -> the gradient, into the E stage), a mover warp (fills E stages,
// stores finished tiles and refills the stage at once), a W loader warp, and one MMA-issuing
// warp per GEMM (different accumulators, so their barrier waits and commits overlap each
// other's MMAs).  expE^T and D1 each have two copies in TMEM when the 512 columns allow, which
// takes GEMM2 -> next exponentials and gradient reads -> next GEMM1 off the critical path.
// D2 stays in TMEM across all tiles and becomes pgrads[:, v-block] at the end.
//
// Operand precision (`passes`): the lattice weights W are always rounded once to TF32
// (round-to-nearest, 2^-12 relative, unbiased).  passes = 1: exp(E) and exp(P) likewise.
// passes = 2 (default): exp(E) is split hi + lo with hi exactly representable in TF32, two
// MMAs per k-step of GEMM2, so pgrads carry only W's rounding.  passes = 3: exp(P) split
// as well (GEMM1), at the price of a smaller frame tile because both halves of exp(P)^T
// must stay resident in tensor memory.
#include <cuda.h>

#include <algorithm>
#include <type_traits>

#include "kernels.h"
#include "profile.h"
#include "sm100.cuh"

namespace tb200 {
namespace {

using namespace sm100;

constexpr int kVBlock = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kMaxStagedLabels = 16;  // label columns per block whose occupancies are staged
constexpr int kGroupWarps = 8;  // column-owner warps per group (exp group, gradient group)
constexpr int kWarpMove = 16, kWarpWLoad = 17, kWarpMma1 = 18, kWarpMma2 = 19;
constexpr int kGradThreads = 20 * 32;
constexpr int kStageRows = 2 + kMaxStagedLabels;  // row shifts, blank-arc sums, staged label rows
constexpr int kMaxRing = 4;

struct GradParams {
  const void* P;         // [B,maxU,V] fp32 or bf16, as are egrads and pgrads
  const float* maxP;     // [B,maxU]
  const float* pBlank;   // [B,maxU]
  const float* pLabel;   // [B,maxU]
  const float* emT;      // [B,maxU,ldT] label-arc occupancies, frames contiguous
  const int* labels;
  const int* inLens;
  const int* labLens;
  const float* deltas;
  void* egrads;
  void* pgrads;
  int* status;
  int maxT, maxU, V, blank;
  // Label axes of 129..256 positions run as two launches over the position ranges
  // [uOff, uOff + 128): each computes its rows of pgrads and its share of egrads (the sum over
  // its positions and their label-arc terms); the first launch writes egrads (and carries the
  // blank-arc terms and the zero padding), the second ADDS its tiles to it (accumulate: the
  // stores become TMA reduce-adds).
  int uOff, accumulate;
  int ldT;      // maxT rounded up to 4: row length of nref / eBlank / emT
  int ldW;      // columns of W (multiple of 32, <= 128)
  int N2;       // GEMM2 N: maxU rounded up to 16 (<= ldW)
  int Ku;       // maxU rounded up to 8 = GEMM1 K
  int stagesE, stagesW;
  int eBufs;    // copies of the expE^T operand in tensor memory (2 if the columns allow)
  int dBufs;    // copies of the D1 accumulator (likewise)
  int tmemCols;
};

struct GradMaps {
  CUtensorMap E, G, Wk, Wmn, nref, ebl, emT;
};

__host__ __device__ constexpr int row_stride_bytes(int tb) { return (tb * 4 + 127) & ~127; }
// an E tile is 128 columns x tb frames in boxes of 128-byte rows: 4 boxes of 32 fp32 columns or
// 2 boxes of 64 bf16 columns
__host__ __device__ constexpr int e_boxes(bool bf) { return bf ? 2 : 4; }
__host__ __device__ constexpr int e_stage_bytes(int tb, bool bf = false) {
  return (e_boxes(bf) * tb * 128 + kStageRows * row_stride_bytes(tb) + 1023) & ~1023;
}

__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}

// ESPLIT / PSPLIT: split exp(E) / exp(P) into TF32 hi + lo (two MMAs per k-step) instead
// of rounding once.  BF: E, P and both gradients are bf16 in memory (converted exactly to fp32
// on the way in, rounded to nearest on the way out; everything in between is the fp32 path).
template <int TB, bool ESPLIT, bool PSPLIT, bool BF = false>
__global__ void __launch_bounds__(kGradThreads, 1) grads_umma_kernel(
    const __grid_constant__ GradMaps tm, const GradParams p) {
  using TIO = typename std::conditional<BF, bf16, float>::type;
  constexpr int TBH = TB / 2;  // frames per owner half
  static_assert(TBH % 8 == 0, "tile halves move through TMEM in 8-column pieces");
  const int b = blockIdx.y, v0 = blockIdx.x * kVBlock;
  const int T = min(p.inLens[b], p.maxT), Utot = min(p.labLens[b] + 1, p.maxU);
  // my range of label positions: local u <-> position uOff + u; U of them belong to the utterance
  const int U = max(0, min(Utot - p.uOff, 128));
  const int rowsMine = min(128, p.maxU - p.uOff);   // rows of pgrads this launch owns
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float delta = p.deltas ? p.deltas[b] : 1.0f;
  TIO* eg = static_cast<TIO*>(p.egrads) + (i64)b * p.maxT * p.V;
  TIO* pg = static_cast<TIO*>(p.pgrads) + ((i64)b * p.maxU + p.uOff) * p.V;

  if (T <= 0 || U <= 0) {
    // nothing flows through (this range of) the utterance: its rows of pgrads are zero, and so
    // is egrads if this is the launch that writes it (an accumulating launch adds nothing)
    const int v = v0 + threadIdx.x;
    if (threadIdx.x < kVBlock && v < p.V) {
      if (!p.accumulate)
        for (int t = 0; t < p.maxT; ++t) from_f32(eg[(i64)t * p.V + v], 0.0f);
      for (int u = 0; u < rowsMine; ++u) from_f32(pg[(i64)u * p.V + v], 0.0f);
    }
    return;
  }

  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) &
                                             ~uintptr_t(1023));
  const int SE = p.stagesE, SW = p.stagesW;
  const int nUB = p.ldW / 32;
  constexpr int kBoxBytes = TB * 128;          // one box of a tile: TB rows of 128 bytes
  constexpr int kBoxes = e_boxes(BF);          // boxes of an E / gradient tile
  constexpr int kBoxCols = 128 / kBoxes;       // vocabulary columns per box
  constexpr int kEBytes = kBoxes * kBoxBytes;  // E tile
  constexpr int kRowBytes = TB * 4;            // one row of per-frame scalars
  constexpr int kRowStride = row_stride_bytes(TB);  // TMA destinations are 128-byte aligned
  constexpr int kEStage = e_stage_bytes(TB, BF);   // E tile + kStageRows rows of scalars
  const int wBytes = nUB * kBoxBytes;
  const int wStage = 2 * wBytes;               // K-major copy, MN-major copy
  uint8_t* smemW = smem + (size_t)SE * kEStage;

  __shared__ uint64_t barEFull[kMaxRing], barStore[kMaxRing];
  __shared__ uint64_t barWFull[kMaxRing], barWFree[kMaxRing];
  __shared__ uint64_t barEReady[2], barE2Free[2], barD1Full[2], barD1Free[2];
  __shared__ uint64_t barPReady, barD2Done;
  __shared__ uint32_t tmemBase;
  __shared__ int abortFlag;
  __shared__ int sWarpCnt[4];
  __shared__ short sListU[128], sListV[128];
  __shared__ int sLab[128];
  __shared__ float sPb[128], sPl[128];

  const int nTiles = (T + TB - 1) / TB;
  // (the blank-arc terms go with the launch that writes egrads)
  const bool blankHere = !p.accumulate && p.blank >= v0 && p.blank < v0 + kVBlock;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SE; ++s) {
      mbar_init(&barEFull[s], 1);
      mbar_init(&barStore[s], kGroupWarps);   // gradient tile complete in shared memory
    }
    for (int s = 0; s < SW; ++s) {
      mbar_init(&barWFull[s], 1);
      mbar_init(&barWFree[s], 2);             // both MMA issuers done with it
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&barEReady[s], kGroupWarps);
      mbar_init(&barE2Free[s], 1 + kGroupWarps);  // GEMM2 done with it + gradient warps have read it
      mbar_init(&barD1Full[s], 1);
      mbar_init(&barD1Free[s], kGroupWarps);
    }
    mbar_init(&barPReady, 2 * kGroupWarps);
    mbar_init(&barD2Done, 1);
    abortFlag = 0;
    fence_mbar_init();
  }
  // Per-position data of this utterance and the labels that fall into this column block
  // (kept in label-position order so repeated labels are combined deterministically).
  bool inBlock = false;
  int myLab = -1;
  if (threadIdx.x < 128) {
    const int u = threadIdx.x;
    if (u < U) {
      sPb[u] = p.pBlank[(i64)b * p.maxU + p.uOff + u];
      sPl[u] = p.pLabel[(i64)b * p.maxU + p.uOff + u];
      if (p.uOff + u < Utot - 1) myLab = p.labels[(i64)b * (p.maxU - 1) + p.uOff + u];
    }
    sLab[u] = myLab;
    inBlock = myLab >= v0 && myLab < v0 + kVBlock;
    const unsigned m = __ballot_sync(0xffffffffu, inBlock);
    if (lane == 0) sWarpCnt[warp] = __popc(m);
  }
  if (warp == kWarpMma1) {
    tmem_alloc(&tmemBase, (uint32_t)p.tmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x < 128) {
    const unsigned m = __ballot_sync(0xffffffffu, inBlock);
    int pos = __popc(m & ((1u << lane) - 1));
    for (int w = 0; w < warp; ++w) pos += sWarpCnt[w];
    if (inBlock) {
      sListU[pos] = (short)threadIdx.x;
      sListV[pos] = (short)(myLab - v0);
    }
  }
  __syncthreads();
  const int nList = sWarpCnt[0] + sWarpCnt[1] + sWarpCnt[2] + sWarpCnt[3];
  const int nStaged = min(nList, kMaxStagedLabels);

  const uint32_t tBase = tmemBase;
  const uint32_t cPhi = 0, cPlo = p.Ku;
  constexpr uint32_t kECols = (ESPLIT ? 2 : 1) * TB;  // one copy of expE^T (hi, then lo)
  const int EB = p.eBufs, DB = p.dBufs;
  const uint32_t cE = (PSPLIT ? 2 : 1) * p.Ku;
  const uint32_t cD1 = cE + EB * kECols;
  const uint32_t cD2 = cD1 + DB * TB;
  volatile int* abortp = &abortFlag;

  if (warp == kWarpMove) {
    // ---------------- mover: E stage i % SE <- tile i (raw E + scalar rows); finished tile -> egrads ----------------
    // One TMA load per lane (a single thread would issue them one after the other): lanes 0..3
    // the boxes of E, lane 4 the row shifts, lane 5 the blank-arc sums, lanes 6.. one staged
    // label row each.  The same warp stores finished tiles, so a stage is refilled as soon as
    // its stores have read it.
    if (lane == 0) {
      tma_prefetch_desc(&tm.E);
      tma_prefetch_desc(&tm.G);
      tma_prefetch_desc(&tm.nref);
      tma_prefetch_desc(&tm.emT);
    }
    const uint32_t bytes =
        (uint32_t)(kEBytes + kRowBytes + (blankHere ? kRowBytes : 0) + nStaged * kRowBytes);
    // What this lane copies for every tile -- all through ONE call site, so that the warp issues
    // its copies together instead of one divergent branch after the other (a branch with a TMA
    // issue costs a lone lane ~200 cycles): which tensor map, where in the stage, and the two
    // tile-independent coordinates.
    const CUtensorMap* myMap = nullptr;
    int myDst = 0, myX = 0, myZ = 0;
    bool yIsT0 = true;   // E: (x = column, y = t0, z = b); scalar rows: (x = t0, y, z)
    if (lane < kBoxes) {  // (a box beyond the vocabulary reads as zeros and still counts its bytes)
      myMap = &tm.E; myDst = lane * kBoxBytes; myX = v0 + kBoxCols * lane; myZ = b;
    } else if (lane == 4) {
      myMap = &tm.nref; myDst = kEBytes; myX = b; myZ = 0; yIsT0 = false;
    } else if (lane == 5) {
      if (blankHere) { myMap = &tm.ebl; myDst = kEBytes + kRowStride; myX = b; myZ = 0; yIsT0 = false; }
    } else if (lane >= 6 && lane - 6 < nStaged) {
      myMap = &tm.emT; myDst = kEBytes + (lane - 4) * kRowStride; myX = p.uOff + sListU[lane - 6]; myZ = b; yIsT0 = false;
    }
    int fs = 0;  // stage of the next fill
    auto fill = [&](int i) {
      const int t0 = i * TB;
      uint8_t* st = smem + (size_t)fs * kEStage;
      if (lane == 0) mbar_arrive_expect_tx(&barEFull[fs], bytes);
      __syncwarp();
      if (myMap != nullptr)
        tma_load_3d(st + myDst, myMap, &barEFull[fs], yIsT0 ? myX : t0, yIsT0 ? t0 : myX, myZ);
      if (++fs == SE) fs = 0;
    };
    int issued = 0;
    for (; issued < nTiles && issued < SE; ++issued) fill(issued);
    int ss = 0;        // stage of the tile stored next
    uint32_t sph = 0;  // its phase
    for (int i = 0; i < nTiles; ++i) {
      const bool ok = mbar_wait(&barStore[ss], sph, abortp, p.status, kStatusTimeoutOperand);
      if (!__all_sync(0xffffffffu, ok)) break;
      // lanes 0..3 store one 32-column box each (every lane has a bulk group of its own), and
      // wait until the store engine has read their box before the stage is refilled
      if (lane < kBoxes && v0 + kBoxCols * lane < p.V) {
        if (p.accumulate)
          tma_reduce_add_3d(&tm.G, smem + (size_t)ss * kEStage + lane * kBoxBytes, v0 + kBoxCols * lane, i * TB, b);
        else
          tma_store_3d(&tm.G, smem + (size_t)ss * kEStage + lane * kBoxBytes, v0 + kBoxCols * lane, i * TB, b);
        tma_store_commit();
        if (issued < nTiles) tma_store_wait_read();
      }
      __syncwarp();
      if (issued < nTiles) fill(issued++);
      if (++ss == SE) { ss = 0; sph ^= 1u; }
    }
    if (lane < kBoxes) {
      // all stores complete (not only read) before the CTA ends
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    if (lane == 0 && *abortp) {  // give copies still in flight a bounded time to land
      for (int i = max(0, issued - SE); i < issued; ++i) {
        const unsigned long long t1 = global_timer_ns();
        while (!mbar_try_wait(&barEFull[i % SE], (i / SE) & 1) &&
               global_timer_ns() - t1 < 50000000ull) {
        }
      }
    }
  } else if (warp == kWarpWLoad) {
    // ---------------- W loader: both copies of W tile i into W stage i % SW ----------------
    // Lanes 0..7: one 32-column box each (even lanes the K-major copy, odd the MN-major one).
    if (lane == 0) {
      tma_prefetch_desc(&tm.Wk);
      tma_prefetch_desc(&tm.Wmn);
    }
    int issued = 0;
    int s = 0;
    uint32_t wph = 1;  // phase of the PREVIOUS release of the stage (no division by a run-time ring
                       // depth in the per-tile loops: it costs a warp ~100 cycles each time)
    for (int i = 0; i < nTiles; ++i) {
      bool ok = true;
      if (i >= SW) ok = mbar_wait(&barWFree[s], wph, abortp, p.status, kStatusTimeoutStageFree);
      if (!__all_sync(0xffffffffu, ok)) break;
      uint8_t* st = smemW + (size_t)s * wStage;
      const int t0 = i * TB;
      if (lane == 0) mbar_arrive_expect_tx(&barWFull[s], (uint32_t)(2 * wBytes));
      __syncwarp();
      const int j = lane >> 1;
      if (lane < 8 && j < nUB) {
        if (lane & 1) tma_load_3d(st + wBytes + j * kBoxBytes, &tm.Wmn, &barWFull[s], p.uOff + 32 * j, t0, b);
        else tma_load_3d(st + j * kBoxBytes, &tm.Wk, &barWFull[s], p.uOff + 32 * j, t0, b);
      }
      issued = i + 1;
      if (++s == SW) { s = 0; wph ^= 1u; }
    }
    if (lane == 0 && *abortp) {
      for (int i = max(0, issued - SW); i < issued; ++i) {
        const unsigned long long t1 = global_timer_ns();
        while (!mbar_try_wait(&barWFull[i % SW], (i / SW) & 1) &&
               global_timer_ns() - t1 < 50000000ull) {
        }
      }
    }
  } else if (warp == kWarpMma1) {
    // ---------------- MMA issuer 1: GEMM1, D1[v, t] = expP^T . W^T per tile ----------------
    if (lane == 0) {
      const uint32_t idesc1 = idesc_tf32(128, TB, 0, 0);  // B = W tile, K-major (K = u)
      const int kSteps1 = p.Ku / 8;
      // operand descriptor of W stage 0, k-step 0; the address field counts 16-byte units
      const uint64_t descW = smem_desc_sw128(smem_u32(smemW), 16, 1024);
      int s = 0, db = 0;
      uint32_t wph = 0, dph = 1;  // phase of the W stage; phase of the PREVIOUS use of the D1 copy
      // expP^T resident in TMEM.  (Its own barrier: a warp whose columns lie beyond the
      // vocabulary finishes the prologue early and must not be able to complete a per-tile
      // phase with that arrival.)
      bool ok = mbar_wait(&barPReady, 0, abortp, p.status, kStatusTimeoutOperand);
      for (int i = 0; i < nTiles && ok; ++i) {
        ok = mbar_wait(&barWFull[s], wph, abortp, p.status, kStatusTimeoutTma);
        if (ok && i >= DB)  // the gradient warps have read this copy of D1
          ok = mbar_wait(&barD1Free[db], dph, abortp, p.status, kStatusTimeoutOperand);
        if (!ok) break;
        tc_fence_after();
        const uint64_t bW0 = descW + (uint64_t)((uint32_t)(s * wStage) >> 4);
        const uint32_t d1 = tBase + cD1 + db * TB;
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {  // Ku <= 128: at most 16 k-steps, constants when unrolled
          if (ks < kSteps1) {
            const uint64_t bW = bW0 + (uint64_t)(((ks >> 2) * kBoxBytes + (ks & 3) * 32) >> 4);
            mma_tf32_ts(d1, tBase + cPhi + ks * 8, bW, idesc1, ks ? 1u : 0u);
            if (PSPLIT) mma_tf32_ts(d1, tBase + cPlo + ks * 8, bW, idesc1, 1u);
          }
        }
        mma_commit(&barD1Full[db]);
        mma_commit(&barWFree[s]);
        if (++s == SW) { s = 0; wph ^= 1u; }
        if (++db == DB) { db = 0; dph ^= 1u; }
      }
    }
  } else if (warp == kWarpMma2) {
    // ---------------- MMA issuer 2: GEMM2, D2[v, u] += expE^T . W over all tiles ----------------
    if (lane == 0) {
      const uint32_t idesc2 = idesc_tf32(128, p.N2, 0, 1);  // B = W tile, MN-major (K = t)
      // descriptor of the MN-major copy in W stage 0, frames 0..7: 8 frames = two 4-row atoms 512
      // bytes apart; 32-column atoms one box apart
      const uint64_t descW = smem_desc_sw128_base32(smem_u32(smemW) + (uint32_t)wBytes, (uint32_t)kBoxBytes, 512);
      bool ok = true;
      int s = 0, eb = 0;
      uint32_t wph = 0, eph = 0;
      for (int i = 0; i < nTiles && ok; ++i) {
        const uint32_t cEhi = cE + eb * kECols, cElo = cEhi + TB;
        ok = mbar_wait(&barWFull[s], wph, abortp, p.status, kStatusTimeoutTma) &&
             mbar_wait(&barEReady[eb], eph, abortp, p.status, kStatusTimeoutOperand);
        if (!ok) break;
        tc_fence_after();
        const uint64_t bW0 = descW + (uint64_t)((uint32_t)(s * wStage) >> 4);
#pragma unroll
        for (int ks = 0; ks < TB / 8; ++ks) {
          const uint64_t bW = bW0 + (uint64_t)((ks * 1024) >> 4);
          mma_tf32_ts(tBase + cD2, tBase + cEhi + ks * 8, bW, idesc2, (i | ks) ? 1u : 0u);
          if (ESPLIT) mma_tf32_ts(tBase + cD2, tBase + cElo + ks * 8, bW, idesc2, 1u);
        }
        mma_commit(&barE2Free[eb]);
        mma_commit(&barWFree[s]);
        if (++s == SW) { s = 0; wph ^= 1u; }
        if (++eb == EB) { eb = 0; eph ^= 1u; }
      }
      if (ok) mma_commit(&barD2Done);
    }
  } else {
    // ---------------- column owners ----------------
    // Thread (q, lane) owns vocabulary column v0 + q*32 + lane = TMEM lane q*32 + lane.  Two
    // groups of 8 warps: group 0 turns raw E into exp(E - ref) (shared memory in place + TMEM),
    // group 1 turns that into the gradient, so tile i+1's exponentials overlap tile i's
    // gradient arithmetic.  Within a group the halves h = 0,1 split the frames of a tile; all
    // 16 warps split the label positions of the prologue and the epilogue.
    const int grp = warp >> 3, q = warp & 3, h = (warp >> 2) & 1;
    const int part = grp * 2 + h;  // 0..3: share of the prologue / epilogue
    const int vl = q * 32 + lane;
    const int v = v0 + vl;
    const bool vOk = v < p.V;
    const uint32_t laneAddr = (uint32_t)(q * 32) << 16;
    bool ok = true;

    // expP^T[v, u] = exp(P[u,v] - maxP[u]) for u < U, zero beyond: resident A operand of GEMM1
    {
      const TIO* pp = static_cast<const TIO*>(p.P) + ((i64)b * p.maxU + p.uOff) * p.V;
      const float* mp = p.maxP + (i64)b * p.maxU + p.uOff;
      const int vc = min(v, p.V - 1);
      for (int u0 = 8 * part; u0 < p.Ku; u0 += 32) {
        // unconditional loads from clamped addresses: all eight are in flight together
        float raw[8], sh[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int uc = min(u0 + j, U - 1);
          raw[j] = to_f32(pp[(i64)uc * p.V + vc]);
          sh[j] = mp[uc];
        }
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float x = ex2_approx((raw[j] - sh[j]) * kLog2e);
          if (u0 + j >= U || !vOk) x = 0.0f;
          if (PSPLIT) split_tf32(x, hi[j], lo[j]);
          else hi[j] = __float_as_uint(tf32_round(x));
        }
        tmem_st8(tBase + laneAddr + cPhi + u0, hi);
        if (PSPLIT) tmem_st8(tBase + laneAddr + cPlo + u0, lo);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&barPReady);
    }

    // my column inside an E stage: fp32: box q, 4-byte element `lane` of each (swizzled) 128-byte
    // row; bf16: box q/2, 2-byte element (q&1)*32 + lane
    const int colOff = BF ? (q >> 1) * kBoxBytes + (lane & 7) * 2 : q * kBoxBytes + (lane & 3) * 4;
    const int chunk = BF ? (q & 1) * 4 + (lane >> 3) : lane >> 2;
    auto elemAt = [&](uint8_t* col, int t) {
      return reinterpret_cast<TIO*>(col + t * 128 + ((chunk ^ (t & 7)) << 4));
    };

    if (grp == 0) {
      // ---- exp group: raw E -> exp(E - ref), in place, and into TMEM as GEMM2's A operand ----
      int se = 0, eb = 0;          // E stage and expE^T copy of tile i
      uint32_t sph = 0, eph = 0;   // and their phases
      for (int i = 0; i < nTiles && ok; ++i) {
        const int t0 = i * TB;
        // live frames in my half (may be <= 0); none for a column beyond the vocabulary
        const int tValid = vOk ? min(TB, T - t0) - h * TBH : 0;
        ok = mbar_wait(&barEFull[se], sph, abortp, p.status, kStatusTimeoutTma);
        if (ok && i >= EB)  // this copy of expE^T must have been consumed by GEMM2
          ok = mbar_wait(&barE2Free[eb], eph ^ 1u, abortp, p.status, kStatusTimeoutMma);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint8_t* stE = smem + (size_t)se * kEStage;
        uint8_t* col = stE + colOff;
        const float* nr = reinterpret_cast<const float*>(stE + kEBytes) + h * TBH;
        const uint32_t cEhi = cE + eb * kECols + h * TBH, cElo = cEhi + TB;
        float xs[TBH];
#pragma unroll
        for (int j = 0; j < TBH; j += 4) {
          const float4 sh = *reinterpret_cast<const float4*>(nr + j);
          const float shj[4] = {sh.x, sh.y, sh.z, sh.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int t = h * TBH + j + k;
            xs[j + k] = fmaf(to_f32(*elemAt(col, t)), kLog2e, shj[k]);
          }
        }
        if (tValid < TBH) {  // last tile of the utterance (or a column beyond the vocabulary):
#pragma unroll             // frames at or beyond T_b contribute nothing, exp2(-inf) = 0
          for (int j = 0; j < TBH; ++j)
            if (j >= tValid) xs[j] = -INFINITY;
        }
#pragma unroll
        for (int c = 0; c < TBH; c += 8) {
          uint32_t hi[8], lo[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float x = ex2_approx(xs[c + j]);
            if (ESPLIT) split_tf32(x, hi[j], lo[j]);
            else hi[j] = __float_as_uint(tf32_round(x));
          }
          tmem_st8(tBase + laneAddr + cEhi + c, hi);
          if (ESPLIT) tmem_st8(tBase + laneAddr + cElo + c, lo);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        // exp(E - ref) of the tile is in TMEM and the raw tile in shared memory is dead
        if (lane == 0) mbar_arrive(&barEReady[eb]);
        if (++se == SE) { se = 0; sph ^= 1u; }
        if (++eb == EB) { eb = 0; eph ^= 1u; }
      }
    } else {
      // ---- gradient group: egrads tile = expE * D1 - sparse (delta_b is inside W and the rows) ----
      // which of the block's label positions carry MY column (almost always none)
      // (labels of this block beyond the kMaxStagedLabels staged ones are subtracted afterwards by
      // label_overflow_kernel; that only happens for tiny vocabularies)
      unsigned stagedMine = 0;
      for (int k = 0; k < nStaged; ++k)
        if (sListV[k] == vl) stagedMine |= 1u << k;
      int se = 0, eb = 0, db = 0;            // E stage, expE^T copy and D1 copy of tile i
      uint32_t sph = 0, eph = 0, dph = 0;    // and their phases
      for (int i = 0; i < nTiles && ok; ++i) {
        const int t0 = i * TB;
        const int tValid = vOk ? min(TB, T - t0) - h * TBH : 0;
        ok = mbar_wait(&barEFull[se], sph, abortp, p.status, kStatusTimeoutTma) &&
             mbar_wait(&barD1Full[db], dph, abortp, p.status, kStatusTimeoutMma) &&
             mbar_wait(&barEReady[eb], eph, abortp, p.status, kStatusTimeoutOperand);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // expE * D1, both from tensor memory (expE = hi + lo exactly)
        const uint32_t cEhi = cE + eb * kECols + h * TBH, cElo = cEhi + TB;
        float d1[TBH];
#pragma unroll
        for (int c = 0; c < TBH; c += 8) {
          uint32_t r[8], xh[8], xl[8];
          tmem_ld8(tBase + laneAddr + cD1 + db * TB + h * TBH + c, r);
          tmem_ld8(tBase + laneAddr + cEhi + c, xh);
          if (ESPLIT) tmem_ld8(tBase + laneAddr + cElo + c, xl);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float x = __uint_as_float(xh[j]);
            if (ESPLIT) x += __uint_as_float(xl[j]);
            d1[c + j] = x * __uint_as_float(r[j]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&barD1Free[db]);
          mbar_arrive(&barE2Free[eb]);
        }
        uint8_t* stE = smem + (size_t)se * kEStage;
        uint8_t* col = stE + colOff;
        const float* rows = reinterpret_cast<const float*>(stE + kEBytes + kRowStride) + h * TBH;
        if (v == p.blank && !p.accumulate) {
#pragma unroll
          for (int j = 0; j < TBH; ++j) d1[j] -= rows[j];
        }
        for (unsigned m0 = stagedMine; m0; m0 &= m0 - 1) {
          const float* m = rows + (1 + (__ffs(m0) - 1)) * (kRowStride / 4);
#pragma unroll
          for (int j = 0; j < TBH; ++j) d1[j] -= m[j];
        }
#pragma unroll
        for (int j = 0; j < TBH; ++j) {
          const int t = h * TBH + j;
          // (frames at or beyond T_b: expE and the rows of W are zero there, so is d1)
          from_f32(*elemAt(col, t), d1[j]);
        }
        fence_proxy_async_smem();  // the tile is read next by TMA stores
        __syncwarp();
        if (lane == 0) mbar_arrive(&barStore[se]);  // my part of the gradient tile is in place
        if (++se == SE) { se = 0; sph ^= 1u; }
        if (++eb == EB) { eb = 0; eph ^= 1u; }
        if (++db == DB) { db = 0; dph ^= 1u; }
      }
    }

    // padded frames beyond the last tile: exact zeros
    if (vOk && !p.accumulate)
      for (int t = nTiles * TB + part; t < p.maxT; t += 4) from_f32(eg[(i64)t * p.V + v], 0.0f);

    // pgrads[u, v] = delta * (expP[u,v] * D2[v,u] - sparse)
    if (ok) ok = mbar_wait(&barD2Done, 0, abortp, p.status, kStatusTimeoutMma);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      for (int u0 = 8 * part; u0 < p.Ku; u0 += 32) {
        uint32_t d2[8], xh[8], xl[8];
        tmem_ld8(tBase + laneAddr + cD2 + u0, d2);
        tmem_ld8(tBase + laneAddr + cPhi + u0, xh);
        if (PSPLIT) tmem_ld8(tBase + laneAddr + cPlo + u0, xl);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int u = u0 + j;
          if (u < rowsMine && vOk) {
            float val = 0.0f;
            if (u < U) {
              float xp = __uint_as_float(xh[j]);
              if (PSPLIT) xp += __uint_as_float(xl[j]);
              val = xp * __uint_as_float(d2[j]);
              if (v == p.blank) val -= delta * sPb[u];
              if (sLab[u] == v) val -= delta * sPl[u];
            }
            from_f32(pg[(i64)u * p.V + v], val);
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kWarpMma1) tmem_dealloc(tBase, (uint32_t)p.tmemCols);
  if (*abortp && threadIdx.x < kVBlock && v0 + (int)threadIdx.x < p.V) {
    // a wait ran out (recorded in the status word): whatever this CTA wrote is incomplete, so
    // its whole slice of both gradients becomes NaN rather than a plausible-looking number
    const float bad = __int_as_float(0x7fc00000);
    const int v = v0 + threadIdx.x;
    for (int t = 0; t < p.maxT; ++t) from_f32(eg[(i64)t * p.V + v], bad);
    for (int u = 0; u < rowsMine; ++u) from_f32(pg[(i64)u * p.V + v], bad);
  }
}

int pow2_cols(int x) {
  int c = 32;
  while (c < x) c <<= 1;
  return c;
}

// Re-layout after the reverse sweep (gamma_warp_kernel), one CTA per 32 frames of one utterance,
// the (up to four) 32x32 lattice tiles of the label axis side by side.  With delta_b the upstream gradient:
//   stayS + stepS (skewed) -> W [B,maxT,ldW] = delta_b * g * exp(ref(t) + maxP(u) - LN(t,u)),
//                   g = stay + step, rounded to TF32 (round-to-nearest; the tensor core would
//                   otherwise truncate), zero outside the valid lattice.  (The exponent is
//                   clamped at 80: it only gets there where the factored log-normaliser had
//                   underflowed.)
//   stepS (skewed) -> emT [B,maxU,ldT] = delta_b * label-arc occupancies with the frames
//                   contiguous, so a tile's slice for one label is one TMA row; zero outside;
//   stayS          -> ebl [B,ldT] = delta_b * sum_u stay(t,u), added in a fixed order;
//   rowRef         -> nref [B,ldT] = -rowRef * log2(e)   (row lengths: multiples of 4 floats
//                   as TMA requires).
// With delta_b folded in here the gradient kernel never multiplies by it per element, and
// frames at or beyond T_b come out as exact zeros without a select.
// TC = false serves the SIMT gradient kernels instead: W unrounded and unscaled, the label-arc
// occupancies row-major [B,maxT,maxU] (through emT), the row sums with row length maxT
// (through ebl), no nref.
template <bool TC>
__global__ void __launch_bounds__(1024, 2) unskew_round_kernel(
    const float* __restrict__ stayS, const float* __restrict__ stepS,
    const float* __restrict__ LNs, const float* __restrict__ rowRef,
    const float* __restrict__ maxP, const float* __restrict__ deltas, float* __restrict__ W,
    float* __restrict__ emT, float* __restrict__ nref, float* __restrict__ ebl,
    const int* __restrict__ inLens, const int* __restrict__ labLens, int maxT, int maxU, int ld,
    i64 latStride, int ldW, int ldT) {
  // 32 warps: 8 per 32-wide block of label positions (ldW <= 128), all four blocks at once
  extern __shared__ float smemU[];
  float (*tW)[32][33] = reinterpret_cast<float (*)[32][33]>(smemU);                // [4]
  float (*tE)[32][33] = tW + 4;
  float (*tS)[32][33] = tE + 4;
  __shared__ float sRow[4][32];
  const int b = blockIdx.y, t0 = blockIdx.x * 32;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  const int lane = threadIdx.x & 31, w = (threadIdx.x >> 5) & 7, ub = threadIdx.x >> 8;
  const float delta = (TC && deltas) ? deltas[b] : 1.0f;
  const int u0 = ub * 32, u = u0 + lane;
  const bool inRange = u0 < ldW;
  const bool live = inRange && t0 < T && u0 < U;
  if (live) {
    const int uc = min(u, U - 1);
    const float mp = maxP[(i64)b * maxU + uc];
    // Lane `lane` of local warp w holds the tile's diagonals ds = w + 8i with 0 <= ds - lane < 32:
    // exactly four of them.  All their loads are issued before the first use (unconditional,
    // clamped into the lattice).
    const int i0 = (lane > w) ? (lane - w + 7) >> 3 : 0;
    float vSt[4], vSp[4], vLn[4], vRef[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int tt = w + 8 * (i0 + j) - lane;
      const int tc = min(t0 + tt, T - 1);
      const i64 o = (i64)b * latStride + (i64)(tc + uc) * ld + uc;
      vSt[j] = stayS[o];
      vSp[j] = stepS[o];
      vLn[j] = LNs[o];
      vRef[j] = rowRef[(i64)b * maxT + tc];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int tt = w + 8 * (i0 + j) - lane;
      float a = 0.0f, c = 0.0f, st = 0.0f;
      if (t0 + tt < T && u < U) {
        st = vSt[j];
        const float sh = fminf((vRef[j] + mp) - vLn[j], 80.0f);
        a = (st + vSp[j]) * expf(sh) * delta;
        c = vSp[j] * delta;
      }
      tW[ub][tt][lane] = a;
      tE[ub][tt][lane] = c;
      tS[ub][tt][lane] = st;
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int tt = w * 4 + k, t = t0 + tt;
    if (inRange) {
      if (t < maxT && u < ldW)
        W[((i64)b * maxT + t) * ldW + u] = live ? (TC ? tf32_round(tW[ub][tt][lane]) : tW[ub][tt][lane]) : 0.0f;
      if (TC) {  // transposed: lane <-> frame, row <-> label position
        const int uu = u0 + tt, t2 = t0 + lane;
        if (uu < maxU && t2 < ldT) emT[((i64)b * maxU + uu) * ldT + t2] = live ? tE[ub][lane][tt] : 0.0f;
      } else if (t < maxT && u < maxU) {
        emT[((i64)b * maxT + t) * maxU + u] = live ? tE[ub][tt][lane] : 0.0f;
      }
    }
    float v = live ? tS[ub][tt][lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) sRow[ub][tt] = v;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int t = t0 + lane;
    const bool ok = t < T;
    const float rs = ((sRow[0][lane] + sRow[1][lane]) + sRow[2][lane]) + sRow[3][lane];
    if (TC) {
      if (t < ldT) {
        nref[(i64)b * ldT + t] = ok ? -rowRef[(i64)b * maxT + t] * kLog2e : 0.0f;
        ebl[(i64)b * ldT + t] = ok ? rs * delta : 0.0f;
      }
    } else if (t < maxT) {
      ebl[(i64)b * maxT + t] = ok ? rs : 0.0f;
    }
  }
}

// Label-arc terms that grads_umma_kernel does not stage: within one block of 128 vocabulary
// columns it subtracts the occupancies of the first kMaxStagedLabels label positions (in
// position order) whose label falls into the block; with a vocabulary of ten thousand entries a
// block sees one or two labels, but a vocabulary of 100 puts all of an utterance's labels into
// one block.  The remaining positions are applied here, one CTA per (block, utterance,
// framesPerCta frames), in position order (so that repeated labels are combined in a fixed order):
//   egrads[b, t, label_u] -= emT[b, u, t]        (emT already carries delta_b)
// The CTA rebuilds the block's list exactly as the gradient kernel does and returns at once if
// it is short enough, which is the normal case.
template <typename TIO>
__global__ void __launch_bounds__(256) label_overflow_kernel(
    const int* __restrict__ labels, const float* __restrict__ emT, TIO* __restrict__ egrads,
    const int* __restrict__ inLens, const int* __restrict__ labLens, int maxT, int maxU, int V,
    int ldT, int uOff, int framesPerCta) {
  __shared__ short sU[128];
  __shared__ short sV[128];
  __shared__ int sCount;
  const int b = blockIdx.y, v0 = blockIdx.x * kVBlock;
  const int T = min(inLens[b], maxT), Utot = min(labLens[b] + 1, maxU);
  // the labelled positions of this launch's range: uOff + u, u < U - 1 in the code below
  const int U = min(Utot - uOff, 129);
  if (T <= 0 || U <= 1) return;
  __shared__ int sLab[128];
  int mine = -1;
  if ((int)threadIdx.x < U - 1 && threadIdx.x < 128) mine = labels[(i64)b * (maxU - 1) + uOff + threadIdx.x];
  if (threadIdx.x < 128) sLab[threadIdx.x] = mine;
  // the normal case, decided by all threads at once: the block holds no more labels than are staged
  if (__syncthreads_count(mine >= v0 && mine < v0 + kVBlock) <= kMaxStagedLabels) return;
  if (threadIdx.x == 0) {
    int n = 0;
    for (int u = 0; u < U - 1 && u < 128; ++u) {
      const int lab = sLab[u];
      if (lab >= v0 && lab < v0 + kVBlock) {
        if (n >= kMaxStagedLabels) {
          sU[n - kMaxStagedLabels] = (short)u;
          sV[n - kMaxStagedLabels] = (short)(lab - v0);
        }
        ++n;
      }
    }
    sCount = max(0, n - kMaxStagedLabels);
  }
  __syncthreads();
  // a thread owns frames t = blockIdx.z * framesPerCta + thread + 256 j and applies the positions one
  // after the other, so repeated labels are combined in position order
  const int n = sCount;
  for (int t = blockIdx.z * framesPerCta + threadIdx.x; t < min(T, (int)(blockIdx.z + 1) * framesPerCta); t += 256) {
    TIO* row = egrads + ((i64)b * maxT + t) * V + v0;
    for (int k = 0; k < n; ++k)
      from_f32(row[sV[k]], to_f32(row[sV[k]]) - emT[((i64)b * maxU + uOff + sU[k]) * ldT + t]);
  }
}

// Operands of the gradient kernel from the outputs of the block-wide reverse sweep (label axes
// of more than 128 positions): W [B,maxT,ldW] = occupancy * exp(ref + maxP - LN), unrounded,
// becomes delta_b * W rounded to TF32, in place; the label-arc occupancies em [B,maxT,maxU]
// become emT [B,maxU,ldT] = delta_b * em, frames contiguous; the blank-arc sums eBlank [B,maxT]
// become ebl [B,ldT] = delta_b * eBlank; rowRef becomes nref = -rowRef * log2(e); all three zero
// for frames at or beyond T_b.  One CTA per 32 frames x 32 positions.
__global__ void __launch_bounds__(256) tc_operands_kernel(
    float* __restrict__ W, const float* __restrict__ em, const float* __restrict__ eBlank,
    const float* __restrict__ rowRef, const float* __restrict__ deltas, float* __restrict__ emT,
    float* __restrict__ nref, float* __restrict__ ebl, const int* __restrict__ inLens, int maxT,
    int maxU, int ldW, int ldT) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z, t0 = blockIdx.x * 32, u0 = blockIdx.y * 32;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int T = min(inLens[b], maxT);
  const float delta = deltas ? deltas[b] : 1.0f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int tt = w * 4 + k, t = t0 + tt, u = u0 + lane;
    float e = 0.0f;
    if (t < maxT) {
      if (u < ldW) {
        float* x = W + ((i64)b * maxT + t) * ldW + u;
        *x = t < T ? tf32_round(*x * delta) : 0.0f;
      }
      if (t < T && u < maxU) e = em[((i64)b * maxT + t) * maxU + u] * delta;
    }
    tile[tt][lane] = e;
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int uu = u0 + w * 4 + k, t = t0 + lane;
    if (uu < maxU && t < ldT) emT[((i64)b * maxU + uu) * ldT + t] = tile[lane][w * 4 + k];
  }
  if (blockIdx.y == 0 && threadIdx.x < 32) {
    const int t = t0 + lane;
    if (t < ldT) {
      const bool ok = t < T;
      nref[(i64)b * ldT + t] = ok ? -rowRef[(i64)b * maxT + t] * kLog2e : 0.0f;
      ebl[(i64)b * ldT + t] = ok ? eBlank[(i64)b * maxT + t] * delta : 0.0f;
    }
  }
}

struct TileCfg {
  int TB, SE, SW, EB, DB;
};

// Tile height, ring depths and TMEM copies.  TMEM: (1|2)*Ku (expP^T) + EB*(1|2)*TB (expE^T) +
// DB*TB (D1) + N2 (D2) <= 512 columns.  Shared memory: SE E stages + SW W stages within the
// 227 KB of a CTA.  Preference: at least three E stages (copies issued two tiles ahead), then
// the double-buffered TMEM operands, then the taller tile.
TileCfg pick_tile(int Ku, int ldW, int N2, int passes, int staticSmem, bool bf = false) {
  const int fp = passes == 3 ? 2 : 1, fe = passes >= 2 ? 2 : 1;
  const int room = 227 * 1024 - staticSmem - 2048;
  TileCfg best{0, 0, 0, 0, 0};
  long bestScore = -1;
  for (int TB : {64, 48, 32}) {
    const int wStage = 2 * (ldW / 32) * TB * 128;
    const int SW = 2;
    const int SE = std::min(kMaxRing, (room - SW * wStage) / e_stage_bytes(TB, bf));
    if (SE < 2) continue;
    for (int bufs = 3; bufs >= 0; --bufs) {  // (EB,DB) = (2,2), (2,1), (1,2), (1,1)
      const int EB = 1 + (bufs >> 1), DB = 1 + (bufs & 1);
      if (fp * Ku + EB * fe * TB + DB * TB + N2 > 512) continue;
      const long score = (long)std::min(SE, 3) * 10000 + (EB + DB) * 1000 + TB;
      if (score > bestScore) {
        bestScore = score;
        best = TileCfg{TB, SE, SW, EB, DB};
      }
      break;
    }
  }
  return best;
}

template <int TB, bool ESPLIT, bool PSPLIT, bool BF = false>
void launch_variant(const GradMaps& tm, GradParams p, TileCfg cfg, Dims d, cudaStream_t stream) {
  const int eStage = e_stage_bytes(TB, BF);
  const int wStage = 2 * (p.ldW / 32) * TB * 128;
  p.stagesE = cfg.SE;
  p.stagesW = cfg.SW;
  p.eBufs = cfg.EB;
  p.dBufs = cfg.DB;
  const int cols = (PSPLIT ? 2 : 1) * p.Ku + cfg.EB * (ESPLIT ? 2 : 1) * TB + cfg.DB * TB + p.N2;
  p.tmemCols = pow2_cols(cols);
  size_t smem = (size_t)cfg.SE * eStage + (size_t)cfg.SW * wStage + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: it may hold all 512 TMEM columns
  TB200_CUDA_CHECK(cudaFuncSetAttribute(grads_umma_kernel<TB, ESPLIT, PSPLIT, BF>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(div_up(d.V, kVBlock), d.B);
  ScopedKernel sk("grads_umma", stream);
  grads_umma_kernel<TB, ESPLIT, PSPLIT, BF><<<grid, kGradThreads, smem, stream>>>(tm, p);
}

constexpr int kStaticSmemBound = 3 * 1024;  // barriers + per-position tables of the kernel

}  // namespace

int grads_umma_ld_w(Dims d) { return (int)round_up64(d.maxU > 0 ? d.maxU : 1, 32); }
int grads_umma_ld_t(Dims d) { return (int)round_up64(d.maxT > 0 ? d.maxT : 1, 4); }

bool grads_umma_supported(const void* E, const void* P, const void* egrads,
                          const void* pgrads, Dims d, int passes) {
  const bool bf = d.dtype == kDtypeBf16;
  // (label axes of 129..256 positions: two launches, the second adding to egrads -- fp32 only,
  // a bf16 sum would be rounded twice)
  if (d.V % (bf ? 8 : 4) != 0 || d.V < 32 || d.maxU < 1 || d.maxU > (bf ? 128 : 256) || d.B > 65535)
    return false;
  if (bf && passes != 2) return false;   // one operand precision is built for bf16 storage
  // E and egrads are TMA operands (16-byte base); the column owners read P and write pgrads
  // with plain 4-byte accesses, but a caller whose P / pgrads are offset by a few bytes gets
  // the same routing as for E: the SIMT kernels
  for (const void* ptr : {E, P, egrads, pgrads})
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return false;
  const int n = std::min(d.maxU, 128);   // positions of the (first) launch
  return pick_tile((int)round_up64(n, 8), (int)round_up64(n, 32), (int)round_up64(n, 16), passes,
                   kStaticSmemBound, bf).TB > 0;
}

void launch_unskew_round(const float* stayS, const float* stepS, const float* LNs,
                         const float* rowRef, const float* maxP, const float* deltas, float* W,
                         float* emT, float* nref, float* ebl, const int* inLens,
                         const int* labLens, SkewGeom g, Dims d, bool tensorCore,
                         cudaStream_t stream) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 0) return;
  const int ldW = grads_umma_ld_w(d), ldT = grads_umma_ld_t(d);
  dim3 grid(div_up(ldT, 32), d.B);
  ScopedKernel sk("lattice_unskew_round", stream);
  const int smem = 12 * 32 * 33 * (int)sizeof(float);
  // (a function attribute belongs to the device that is current when it is set: set it on every
  // launch, it is a host-side table update)
  TB200_CUDA_CHECK(cudaFuncSetAttribute(tensorCore ? unskew_round_kernel<true> : unskew_round_kernel<false>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  if (tensorCore)
    unskew_round_kernel<true><<<grid, 1024, smem, stream>>>(stayS, stepS, LNs, rowRef, maxP, deltas, W,
                                                        emT, nref, ebl, inLens, labLens, d.maxT,
                                                        d.maxU, g.ld, g.stride, ldW, ldT);
  else
    unskew_round_kernel<false><<<grid, 1024, smem, stream>>>(stayS, stepS, LNs, rowRef, maxP, nullptr,
                                                         W, emT, nullptr, ebl, inLens, labLens,
                                                         d.maxT, d.maxU, g.ld, g.stride, ldW, ldT);
  TB200_CHECK_LAUNCH();
}

void launch_tc_operands(float* W, const float* em, const float* eBlank, const float* rowRef,
                        const float* deltas, float* emT, float* nref, float* ebl,
                        const int* inLens, Dims d, cudaStream_t stream) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 0) return;
  const int ldW = grads_umma_ld_w(d), ldT = grads_umma_ld_t(d);
  ScopedKernel sk("lattice_tc_operands", stream);
  tc_operands_kernel<<<dim3(div_up(ldT, 32), div_up(ldW, 32), d.B), 256, 0, stream>>>(
      W, em, eBlank, rowRef, deltas, emT, nref, ebl, inLens, d.maxT, d.maxU, ldW, ldT);
  TB200_CHECK_LAUNCH();
}

void launch_grads_umma(const void* E, const void* P, const float* maxP, const float* W,
                       const float* emT, const float* nref, const float* ebl, const float* pBlank,
                       const float* pLabel, const int* labels, const float* deltas, void* egrads,
                       void* pgrads, const int* inLens, const int* labLens, Dims d, int passes,
                       int* status, cudaStream_t stream) {
  if (d.B <= 0 || d.V <= 0) return;
  const bool bf = d.dtype == kDtypeBf16;
  if (bf && passes != 2) throw std::invalid_argument("bf16 gradients are built for grad_passes = 2 only");
  GradParams p;
  p.P = P; p.maxP = maxP; p.pBlank = pBlank; p.pLabel = pLabel; p.emT = emT; p.labels = labels;
  p.inLens = inLens; p.labLens = labLens; p.deltas = deltas; p.egrads = egrads; p.pgrads = pgrads;
  p.status = status;
  p.maxT = d.maxT; p.maxU = d.maxU; p.V = d.V; p.blank = d.blank;
  p.ldT = grads_umma_ld_t(d);
  const uint64_t V = d.V, T = d.maxT, B = d.B, ldWall = grads_umma_ld_w(d), ldT = p.ldT, U = d.maxU;
  // one launch per range of 128 label positions (see GradParams::uOff)
  for (int uOff = 0; uOff < d.maxU; uOff += 128) {
    const int n = std::min(128, d.maxU - uOff);
    p.uOff = uOff;
    p.accumulate = uOff > 0 ? 1 : 0;
    p.ldW = (int)round_up64(n, 32);
    p.Ku = (int)round_up64(n, 8);
    p.N2 = (int)round_up64(n, 16);
    p.stagesE = p.stagesW = p.eBufs = p.dBufs = p.tmemCols = 0;
    const TileCfg cfg = pick_tile(p.Ku, p.ldW, p.N2, passes, kStaticSmemBound, bf);
    if (cfg.TB == 0) throw std::invalid_argument("label axis too long for the tensor-core gradient kernel");
    const int TB = cfg.TB;
    GradMaps tm;
    if (bf) {
      tm.E = make_tmap_bf16_3d(E, V, T, B, V * 2, T * V * 2, 64, TB);
      tm.G = make_tmap_bf16_3d(egrads, V, T, B, V * 2, T * V * 2, 64, TB);
    } else {
      tm.E = make_tmap_f32_3d(E, V, T, B, V * 4, T * V * 4, TB);
      tm.G = make_tmap_f32_3d(egrads, V, T, B, V * 4, T * V * 4, TB);
    }
    tm.Wk = make_tmap_f32_3d(W, ldWall, T, B, ldWall * 4, T * ldWall * 4, TB);
    tm.Wmn = make_tmap_f32_3d(W, ldWall, T, B, ldWall * 4, T * ldWall * 4, TB, /*atom32=*/true);
    tm.nref = make_tmap_f32_rows(nref, ldT, B, 1, ldT * 4, B * ldT * 4, TB);
    tm.ebl = make_tmap_f32_rows(ebl, ldT, B, 1, ldT * 4, B * ldT * 4, TB);
    tm.emT = make_tmap_f32_rows(emT, ldT, U, B, ldT * 4, U * ldT * 4, TB);
#define GO(TBV, EV, PV) launch_variant<TBV, EV, PV>(tm, p, cfg, d, stream)
#define GO_TB(EV, PV) \
  do { if (TB == 64) GO(64, EV, PV); else if (TB == 48) GO(48, EV, PV); else GO(32, EV, PV); } while (0)
    if (bf) {
      if (TB == 64) launch_variant<64, true, false, true>(tm, p, cfg, d, stream);
      else if (TB == 48) launch_variant<48, true, false, true>(tm, p, cfg, d, stream);
      else launch_variant<32, true, false, true>(tm, p, cfg, d, stream);
    } else if (passes == 3) GO_TB(true, true);
    else if (passes == 2) GO_TB(true, false);
    else GO_TB(false, false);
#undef GO_TB
#undef GO
    TB200_CHECK_LAUNCH();
    // only a vocabulary block that can hold more labels than are staged needs the second kernel
    if (n - (uOff + n == d.maxU ? 1 : 0) > kMaxStagedLabels) {
      ScopedKernel sk("label_overflow", stream);
      // (few vocabulary blocks: the kernel will have work -- spread the frames over more CTAs;
      // many blocks: almost every CTA returns at once -- keep them few)
      const int framesPerCta = d.V <= 1024 ? 256 : 1024;
      const dim3 grid(div_up(d.V, kVBlock), d.B, div_up(d.maxT, framesPerCta));
      if (bf)
        label_overflow_kernel<bf16><<<grid, 256, 0, stream>>>(
            labels, emT, static_cast<bf16*>(egrads), inLens, labLens, d.maxT, d.maxU, d.V, p.ldT, uOff, framesPerCta);
      else
        label_overflow_kernel<float><<<grid, 256, 0, stream>>>(
            labels, emT, static_cast<float*>(egrads), inLens, labLens, d.maxT, d.maxU, d.V, p.ldT, uOff, framesPerCta);
      TB200_CHECK_LAUNCH();
    }
  }
}

}  // namespace tb200
