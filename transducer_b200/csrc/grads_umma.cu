// Emission and prediction gradients in ONE pass over E on the tensor cores.
//
// The reference computes (transducer/torch_binding.py:85-89, after the sparse terms of
// transducer_cpu.cpp:81-143):
//   egrads[t,v] = delta * ( expE[t,v] * sum_u W[t,u] expP[u,v]  - sparse_E[t,v] )
//   pgrads[u,v] = delta * ( expP[u,v] * sum_t W[t,u] expE[t,v]  - sparse_P[u,v] )
// with two batched SGEMMs and ~8 elementwise passes over E-sized tensors, keeping
// expE = exp(E - maxE) from the forward pass.  Here E is read once, expE is recomputed
// in registers, every gradient element is written once, and nothing E-sized is stored.
//
// Work decomposition: one CTA per (utterance b, block of 128 vocabulary columns); it walks
// the frames of the utterance in tiles of Tb.  Everything is laid out with the VOCABULARY
// column on the 128 TMEM lanes (UMMA M = 128):
//   GEMM1  D1[v, t] = sum_u expP^T[v,u] * W[t,u]        A = expP^T in TMEM (resident for the
//                                                        whole CTA), B = W tile in smem, K-major
//   GEMM2  D2[v, u] += sum_t expE^T[v,t] * W[t,u]       A = expE^T in TMEM (per tile),
//                                                        B = the W tile again, MN-major.  An
//                                                        MN-major TF32 operand must use the
//                                                        128-byte swizzle with 32-byte atoms, so
//                                                        the tile is fetched a second time by a
//                                                        tensor map with that swizzle.
// Thread v of warps 0-3 owns column v: it exponentiates its column of the raw E tile
// (TMA -> smem), writes the TF32 hi/lo split straight to TMEM, keeps the fp32 values in
// registers, and after GEMM1 multiplies them with D1[v, :] to emit egrads[:, v] -- a warp
// writes 32 consecutive columns of one frame, i.e. coalesced 128-byte stores.  D2 stays in
// TMEM across all tiles and becomes pgrads[:, v-block] at the end.
//
// Operand precision (`passes`): the lattice weights W are always rounded once to TF32
// (round-to-nearest, 2^-12 relative, unbiased).  passes = 1: exp(E) and exp(P) likewise.
// passes = 2 (default): exp(E) is split hi + lo with hi exactly representable in TF32, two
// MMAs per k-step of GEMM2, so pgrads carry only W's rounding.  passes = 3: exp(P) split
// as well (GEMM1), at the price of a smaller frame tile because both halves of exp(P)^T
// must stay resident in tensor memory.
#include <cuda.h>

#include <algorithm>

#include "kernels.h"
#include "profile.h"
#include "sm100.cuh"

namespace tb200 {
namespace {

using namespace sm100;

constexpr int kVBlock = 128;
constexpr float kLog2e = 1.4426950408889634f;

struct GradParams {
  const float* E;
  const float* P;
  const float* rowRef;   // [B,maxT]
  const float* maxP;     // [B,maxU]
  const float* eBlank;   // [B,maxT]
  const float* pBlank;   // [B,maxU]
  const float* pLabel;   // [B,maxU]
  const float* em;       // [B,maxT,maxU] label-arc occupancies
  const int* labels;
  const int* inLens;
  const int* labLens;
  const float* deltas;
  float* egrads;
  float* pgrads;
  int* status;
  int maxT, maxU, V, blank;
  int ldW;      // columns of W (multiple of 32, <= 128) = GEMM2 N
  int Ku;       // maxU rounded up to 8 = GEMM1 K
  int stages;
  int tmemCols;
};

__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}

constexpr int kMaxStagedLabels = 16;  // label columns per block whose occupancies are staged
constexpr int kOwnerWarps = 8;
constexpr int kGradThreads = (kOwnerWarps + 3) * 32;  // + producer + two MMA issuers

// ESPLIT / PSPLIT: split exp(E) / exp(P) into TF32 hi + lo (two MMAs per k-step) instead
// of rounding once.
template <int TB, bool ESPLIT, bool PSPLIT>
__global__ void __launch_bounds__(kGradThreads, 1) grads_umma_kernel(
    const __grid_constant__ CUtensorMap tmE, const __grid_constant__ CUtensorMap tmWk,
    const __grid_constant__ CUtensorMap tmWmn, const GradParams p) {
  constexpr int TBH = TB / 2;  // frames per owner half
  static_assert(TBH % 8 == 0, "tile halves move through TMEM in 8-column pieces");
  const int b = blockIdx.y, v0 = blockIdx.x * kVBlock;
  const int T = min(p.inLens[b], p.maxT), U = min(p.labLens[b] + 1, p.maxU);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float delta = p.deltas ? p.deltas[b] : 1.0f;
  float* eg = p.egrads + (i64)b * p.maxT * p.V;
  float* pg = p.pgrads + (i64)b * p.maxU * p.V;

  if (T <= 0 || U <= 0) {  // nothing flows through this utterance: gradients are zero
    const int v = v0 + threadIdx.x;
    if (threadIdx.x < kVBlock && v < p.V) {
      for (int t = 0; t < p.maxT; ++t) eg[(i64)t * p.V + v] = 0.0f;
      for (int u = 0; u < p.maxU; ++u) pg[(i64)u * p.V + v] = 0.0f;
    }
    return;
  }

  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) &
                                             ~uintptr_t(1023));
  const int S = p.stages;
  const int nUB = p.ldW / 32;
  constexpr int kEBoxBytes = TB * 128;  // one 32-column box of the E tile
  constexpr int kEBytes = 4 * kEBoxBytes;
  const int wBoxBytes = TB * 128;
  const int wBytes = nUB * wBoxBytes;
  const int stageBytes = kEBytes + 2 * wBytes;  // E tile, W tile (K-major), W tile (MN-major)

  __shared__ uint64_t barFull[3], barFree[3], barPReady, barEReady, barE2Free, barD1Full, barD1Free,
      barD2Done;
  __shared__ uint32_t tmemBase;
  __shared__ int abortFlag;
  __shared__ int sWarpCnt[4];
  __shared__ short sListU[128], sListV[128];
  __shared__ int sLab[128];
  __shared__ float sPb[128], sPl[128];
  __shared__ float sNref[3][TB];  // per stage: -rowRef[t] * log2(e) for the tile's frames
  __shared__ float sEbl[3][TB];   // per stage: blank-arc sums of the tile's frames
  __shared__ float sEm[3][kMaxStagedLabels][TB];  // per stage: label-arc occupancies

  const int nTiles = (T + TB - 1) / TB;
  const bool blankHere = p.blank >= v0 && p.blank < v0 + kVBlock;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&barFull[s], 2);  // the copies (transaction bytes) + the staged scalars
      mbar_init(&barFree[s], kOwnerWarps + 2);  // owner warps + both MMA issuers done with it
    }
    mbar_init(&barPReady, kOwnerWarps);
    mbar_init(&barEReady, kOwnerWarps);
    mbar_init(&barE2Free, 1);
    mbar_init(&barD1Full, 1);
    mbar_init(&barD1Free, kOwnerWarps);
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
      sPb[u] = p.pBlank[(i64)b * p.maxU + u];
      sPl[u] = p.pLabel[(i64)b * p.maxU + u];
      if (u < U - 1) myLab = p.labels[(i64)b * (p.maxU - 1) + u];
    }
    sLab[u] = myLab;
    inBlock = myLab >= v0 && myLab < v0 + kVBlock;
    const unsigned m = __ballot_sync(0xffffffffu, inBlock);
    if (lane == 0) sWarpCnt[warp] = __popc(m);
  }
  if (warp == kOwnerWarps + 1) {
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
  const uint32_t cEhi = (PSPLIT ? 2 : 1) * p.Ku, cElo = cEhi + TB;
  const uint32_t cD1 = cEhi + (ESPLIT ? 2 : 1) * TB;
  const uint32_t cD2 = cD1 + TB;
  volatile int* abortp = &abortFlag;

  if (warp == kOwnerWarps) {
    // ---------------- producer ----------------
    // All lanes stage the tile's per-frame scalars (row shifts, blank-arc sums, label-arc
    // occupancies of this block's labels) in shared memory; lane 0 then arms the barrier
    // and issues the tile copies.  This runs up to S tiles ahead of the owners, so the
    // scattered global reads are off their critical path.
    if (lane == 0) {
      tma_prefetch_desc(&tmE);
      tma_prefetch_desc(&tmWk);
      tma_prefetch_desc(&tmWmn);
    }
    const float* refg = p.rowRef + (i64)b * p.maxT;
    const float* eblg = p.eBlank + (i64)b * p.maxT;
    const float* emg = p.em + (i64)b * p.maxT * p.maxU;
    int issued = 0;
    bool ok = true;
    for (int i = 0; i < nTiles && ok; ++i) {
      const int s = i % S;
      if (i >= S) {
        ok = mbar_wait(&barFree[s], ((i / S) - 1) & 1, abortp, p.status, kStatusTimeoutStageFree);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      const int t0 = i * TB;
      if (lane == 0) {  // copies first: their latency overlaps the scalar staging below
        uint8_t* st = smem + (size_t)s * stageBytes;
        mbar_arrive_expect_tx(&barFull[s], (uint32_t)stageBytes);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          tma_load_3d(st + j * kEBoxBytes, &tmE, &barFull[s], v0 + 32 * j, t0, b);
        for (int j = 0; j < nUB; ++j) {
          tma_load_3d(st + kEBytes + j * wBoxBytes, &tmWk, &barFull[s], 32 * j, t0, b);
          tma_load_3d(st + kEBytes + wBytes + j * wBoxBytes, &tmWmn, &barFull[s], 32 * j, t0, b);
        }
      }
      for (int t = lane; t < TB; t += 32) {
        const bool live = t0 + t < T;
        sNref[s][t] = live ? -refg[t0 + t] * kLog2e : 0.0f;
        if (blankHere) sEbl[s][t] = live ? eblg[t0 + t] : 0.0f;
        for (int k = 0; k < nStaged; ++k)
          sEm[s][k][t] = live ? emg[(i64)(t0 + t) * p.maxU + sListU[k]] : 0.0f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&barFull[s]);
      issued = i + 1;
    }
    if (lane == 0 && *abortp) {
      // after an abort: give the copies still in flight a bounded time to land
      for (int i = max(0, issued - S); i < issued; ++i) {
        const unsigned long long t1 = global_timer_ns();
        while (!mbar_try_wait(&barFull[i % S], (i / S) & 1) &&
               global_timer_ns() - t1 < 50000000ull) {
        }
      }
    }
  } else if (warp == kOwnerWarps + 1) {
    // ---------------- MMA issuer 1: GEMM1, D1[v, t] = expP^T . W^T per tile ----------------
    // (GEMM1 and GEMM2 write different accumulators and read different A operands, so each
    // has its own issuing thread: the barrier waits and commits of one overlap the MMAs of
    // the other.)
    if (lane == 0) {
      const uint32_t idesc1 = idesc_tf32(128, TB, 0, 0);  // B = W tile, K-major (K = u)
      const int kSteps1 = p.Ku / 8;
      // expP^T resident in TMEM.  (Its own barrier: a warp whose columns lie beyond the
      // vocabulary finishes the prologue early and must not be able to complete a per-tile
      // phase with that arrival.)
      bool ok = mbar_wait(&barPReady, 0, abortp, p.status, kStatusTimeoutOperand);
      for (int i = 0; i < nTiles && ok; ++i) {
        const int s = i % S;
        ok = mbar_wait(&barFull[s], (i / S) & 1, abortp, p.status, kStatusTimeoutTma);
        if (ok && i > 0)
          ok = mbar_wait(&barD1Free, (i - 1) & 1, abortp, p.status, kStatusTimeoutOperand);
        if (!ok) break;
        tc_fence_after();
        const uint32_t wK = smem_u32(smem + (size_t)s * stageBytes + kEBytes);
        for (int ks = 0; ks < kSteps1; ++ks) {
          const uint32_t off = (uint32_t)((ks >> 2) * wBoxBytes + (ks & 3) * 32);
          const uint64_t bW = smem_desc_sw128(wK + off, 16, 1024);
          mma_tf32_ts(tBase + cD1, tBase + cPhi + ks * 8, bW, idesc1, ks ? 1u : 0u);
          if (PSPLIT) mma_tf32_ts(tBase + cD1, tBase + cPlo + ks * 8, bW, idesc1, 1u);
        }
        mma_commit(&barD1Full);
        mma_commit(&barFree[s]);
      }
    }
  } else if (warp == kOwnerWarps + 2) {
    // ---------------- MMA issuer 2: GEMM2, D2[v, u] += expE^T . W over all tiles ----------------
    if (lane == 0) {
      const uint32_t idesc2 = idesc_tf32(128, p.ldW, 0, 1);  // B = W tile, MN-major (K = t)
      bool ok = true;
      for (int i = 0; i < nTiles && ok; ++i) {
        const int s = i % S;
        ok = mbar_wait(&barFull[s], (i / S) & 1, abortp, p.status, kStatusTimeoutTma) &&
             mbar_wait(&barEReady, i & 1, abortp, p.status, kStatusTimeoutOperand);
        if (!ok) break;
        tc_fence_after();
        const uint32_t wMn = smem_u32(smem + (size_t)s * stageBytes + kEBytes) + (uint32_t)wBytes;
        for (int ks = 0; ks < TB / 8; ++ks) {
          // 8 frames = two 4-row atoms 512 bytes apart; 32-column atoms one box apart
          const uint64_t bW = smem_desc_sw128_base32(wMn + ks * 1024, (uint32_t)wBoxBytes, 512);
          mma_tf32_ts(tBase + cD2, tBase + cEhi + ks * 8, bW, idesc2, (i | ks) ? 1u : 0u);
          if (ESPLIT) mma_tf32_ts(tBase + cD2, tBase + cElo + ks * 8, bW, idesc2, 1u);
        }
        mma_commit(&barE2Free);
        mma_commit(&barFree[s]);
      }
      if (ok) mma_commit(&barD2Done);
    }
  } else {
    // ---------------- column owners ----------------
    // Thread (q, lane) owns vocabulary column v0 + q*32 + lane = TMEM lane q*32 + lane; the
    // two halves h = 0,1 of the owner warps split the frames of each tile (and the label
    // positions of the prologue/epilogue) between them.
    const int q = warp & 3, h = warp >> 2;
    const int vl = q * 32 + lane;
    const int v = v0 + vl;
    const bool vOk = v < p.V;
    const uint32_t laneAddr = (uint32_t)(q * 32) << 16;
    bool ok = true;

    // expP^T[v, u] = exp(P[u,v] - maxP[u]) for u < U, zero beyond: resident A operand of GEMM1
    {
      const float* pp = p.P + (i64)b * p.maxU * p.V;
      const float* mp = p.maxP + (i64)b * p.maxU;
      for (int u0 = 8 * h; u0 < p.Ku; u0 += 16) {
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int u = u0 + j;
          float x = 0.0f;
          if (u < U && vOk) x = ex2_approx((pp[(i64)u * p.V + v] - mp[u]) * kLog2e);
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

    const float* emb = p.em + (i64)b * p.maxT * p.maxU;

    for (int i = 0; i < nTiles && ok; ++i) {
      const int s = i % S, t0 = i * TB;
      ok = mbar_wait(&barFull[s], (i / S) & 1, abortp, p.status, kStatusTimeoutTma);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // my column of the raw tile: box q, 4-byte element `lane` of each 128-byte row
      const uint8_t* col = smem + (size_t)s * stageBytes + q * kEBoxBytes + (lane & 3) * 4;
      const float* nr = sNref[s] + h * TBH;
      const int tValid = min(TB, T - t0) - h * TBH;  // live frames in my half (may be <= 0)
      float x[TBH];
      if (tValid >= TBH) {
#pragma unroll
        for (int j = 0; j < TBH; ++j) {
          const int t = h * TBH + j;
          const float raw =
              *reinterpret_cast<const float*>(col + t * 128 + (((lane >> 2) ^ (t & 7)) << 4));
          x[j] = ex2_approx(fmaf(raw, kLog2e, nr[j]));
        }
      } else {  // frames at or beyond T_b contribute nothing
#pragma unroll
        for (int j = 0; j < TBH; ++j) {
          const int t = h * TBH + j;
          const float raw =
              *reinterpret_cast<const float*>(col + t * 128 + (((lane >> 2) ^ (t & 7)) << 4));
          x[j] = (j < tValid) ? ex2_approx(fmaf(raw, kLog2e, nr[j])) : 0.0f;
        }
      }
      // expE^T of the previous tile must have been consumed by GEMM2 before it is replaced
      if (i > 0) {
        ok = mbar_wait(&barE2Free, (i - 1) & 1, abortp, p.status, kStatusTimeoutMma);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
#pragma unroll
      for (int c = 0; c < TBH; c += 8) {
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (ESPLIT) split_tf32(x[c + j], hi[j], lo[j]);
          else hi[j] = __float_as_uint(tf32_round(x[c + j]));
        }
        tmem_st8(tBase + laneAddr + cEhi + h * TBH + c, hi);
        if (ESPLIT) tmem_st8(tBase + laneAddr + cElo + h * TBH + c, lo);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&barEReady);  // phase i

      // egrads[t0.., v] = delta * (expE * D1 - sparse)
      ok = mbar_wait(&barD1Full, i & 1, abortp, p.status, kStatusTimeoutMma);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float d1[TBH];
#pragma unroll
      for (int c = 0; c < TBH; c += 8) {
        uint32_t r[8];
        tmem_ld8(tBase + laneAddr + cD1 + h * TBH + c, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) d1[c + j] = __uint_as_float(r[j]);
      }
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&barD1Free);
#pragma unroll
      for (int j = 0; j < TBH; ++j) d1[j] *= x[j];
      if (v == p.blank) {
        const float* eb = sEbl[s] + h * TBH;
#pragma unroll
        for (int j = 0; j < TBH; ++j) d1[j] -= eb[j];
      }
      for (int k = 0; k < nStaged; ++k) {
        if (sListV[k] == vl) {
          const float* m = sEm[s][k] + h * TBH;
#pragma unroll
          for (int j = 0; j < TBH; ++j) d1[j] -= m[j];
        }
      }
      for (int k = nStaged; k < nList; ++k) {  // more labels in this block than are staged
        if (sListV[k] == vl) {
          const int u = sListU[k];
#pragma unroll
          for (int j = 0; j < TBH; ++j)
            if (j < tValid) d1[j] -= emb[(i64)(t0 + h * TBH + j) * p.maxU + u];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&barFree[s]);  // stage s (tile + staged scalars) released
      if (vOk) {
        float* dst = eg + (i64)(t0 + h * TBH) * p.V + v;
        if (tValid >= TBH) {
#pragma unroll
          for (int j = 0; j < TBH; ++j) dst[(i64)j * p.V] = delta * d1[j];
        } else {
#pragma unroll
          for (int j = 0; j < TBH; ++j)
            if (t0 + h * TBH + j < p.maxT) dst[(i64)j * p.V] = (j < tValid) ? delta * d1[j] : 0.0f;
        }
      }
    }

    // padded frames beyond the last tile: exact zeros
    if (vOk)
      for (int t = nTiles * TB + h; t < p.maxT; t += 2) eg[(i64)t * p.V + v] = 0.0f;

    // pgrads[u, v] = delta * (expP[u,v] * D2[v,u] - sparse)
    if (ok) ok = mbar_wait(&barD2Done, 0, abortp, p.status, kStatusTimeoutMma);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      for (int u0 = 8 * h; u0 < p.Ku; u0 += 16) {
        uint32_t d2[8], xh[8], xl[8];
        tmem_ld8(tBase + laneAddr + cD2 + u0, d2);
        tmem_ld8(tBase + laneAddr + cPhi + u0, xh);
        if (PSPLIT) tmem_ld8(tBase + laneAddr + cPlo + u0, xl);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int u = u0 + j;
          if (u < p.maxU && vOk) {
            float val = 0.0f;
            if (u < U) {
              float xp = __uint_as_float(xh[j]);
              if (PSPLIT) xp += __uint_as_float(xl[j]);
              val = xp * __uint_as_float(d2[j]);
              if (v == p.blank) val -= sPb[u];
              if (sLab[u] == v) val -= sPl[u];
              val *= delta;
            }
            pg[(i64)u * p.V + v] = val;
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kOwnerWarps + 1) tmem_dealloc(tBase, (uint32_t)p.tmemCols);
}

int pow2_cols(int x) {
  int c = 32;
  while (c < x) c <<= 1;
  return c;
}

// W (skewed) -> W row-major [B,maxT,ldW] rounded to TF32 (round-to-nearest; the tensor
// core would otherwise truncate), zero outside the valid lattice; em row-major.
__global__ void __launch_bounds__(256) unskew_round_kernel(
    const float* __restrict__ Ws, const float* __restrict__ EMs, float* __restrict__ W,
    float* __restrict__ em, const int* __restrict__ inLens, const int* __restrict__ labLens,
    int maxT, int maxU, int ld, i64 latStride, int ldW) {
  __shared__ float tW[32][33], tE[32][33];
  const int b = blockIdx.z, t0 = blockIdx.y * 32, u0 = blockIdx.x * 32;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int u = u0 + lane;
  const bool live = t0 < T && u0 < U;
  if (live) {
    for (int ds = w; ds < 63; ds += 8) {
      const int tt = ds - lane;
      if (tt >= 0 && tt < 32) {
        float a = 0.0f, c = 0.0f;
        if (t0 + tt < T && u < U) {
          const i64 o = (i64)b * latStride + (i64)(t0 + u0 + ds) * ld + u;
          a = Ws[o];
          c = EMs[o];
        }
        tW[tt][lane] = a;
        tE[tt][lane] = c;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int tt = w * 4 + k, t = t0 + tt;
    if (t >= maxT) continue;
    if (u < ldW) W[((i64)b * maxT + t) * ldW + u] = live ? tf32_round(tW[tt][lane]) : 0.0f;
    if (u < maxU) em[((i64)b * maxT + t) * maxU + u] = live ? tE[tt][lane] : 0.0f;
  }
}

template <int TB, bool ESPLIT, bool PSPLIT>
void launch_variant(const CUtensorMap& tmE, const CUtensorMap& tmWk, const CUtensorMap& tmWmn,
                    GradParams p, Dims d, cudaStream_t stream) {
  const int nUB = p.ldW / 32;
  const int stageBytes = 4 * TB * 128 + 2 * nUB * TB * 128;
  cudaFuncAttributes fa;
  TB200_CUDA_CHECK(cudaFuncGetAttributes(&fa, grads_umma_kernel<TB, ESPLIT, PSPLIT>));
  const int room = 227 * 1024 - (int)fa.sharedSizeBytes - 2048;
  int stages = std::min(3, room / stageBytes);
  if (stages < 1) throw std::invalid_argument("gradient tile does not fit shared memory");
  p.stages = stages;
  const int cols = (PSPLIT ? 2 : 1) * p.Ku + (ESPLIT ? 2 : 1) * TB + TB + p.ldW;
  if (cols > 512) throw std::invalid_argument("gradient tile does not fit tensor memory");
  p.tmemCols = pow2_cols(cols);
  size_t smem = (size_t)stages * stageBytes + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: it may hold all 512 TMEM columns
  TB200_CUDA_CHECK(cudaFuncSetAttribute(grads_umma_kernel<TB, ESPLIT, PSPLIT>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(div_up(d.V, kVBlock), d.B);
  ScopedKernel sk("grads_umma", stream);
  grads_umma_kernel<TB, ESPLIT, PSPLIT><<<grid, kGradThreads, smem, stream>>>(tmE, tmWk, tmWmn, p);
}

// Largest frame tile whose operands and accumulators fit the 512 TMEM columns:
// (1|2)*Ku (expP^T) + (1|2)*TB (expE^T) + TB (D1) + ldW (D2).
int pick_tile(int Ku, int ldW, int passes) {
  const int fp = passes == 3 ? 2 : 1, fe = passes >= 2 ? 2 : 1;
  const int room = (512 - fp * Ku - ldW) / (fe + 1);
  if (room >= 64) return 64;
  if (room >= 48) return 48;
  if (room >= 32) return 32;
  return 0;
}

}  // namespace

int grads_umma_ld_w(Dims d) { return (int)round_up64(d.maxU > 0 ? d.maxU : 1, 32); }

bool grads_umma_supported(const float* E, Dims d, int passes) {
  if (d.V % 4 != 0 || d.V < 32 || d.maxU < 1 || d.maxU > 128 || d.B > 65535) return false;
  if ((reinterpret_cast<uintptr_t>(E) & 15) != 0) return false;
  const int Ku = (int)round_up64(d.maxU, 8);
  return pick_tile(Ku, grads_umma_ld_w(d), passes) > 0;
}

void launch_unskew_round(const float* Ws, const float* EMs, float* W, float* em,
                         const int* inLens, const int* labLens, SkewGeom g, Dims d,
                         cudaStream_t stream) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 0) return;
  const int ldW = grads_umma_ld_w(d);
  dim3 grid(div_up(ldW, 32), div_up(d.maxT, 32), d.B);
  ScopedKernel sk("lattice_unskew_round", stream);
  unskew_round_kernel<<<grid, 256, 0, stream>>>(Ws, EMs, W, em, inLens, labLens, d.maxT, d.maxU,
                                                g.ld, g.stride, ldW);
  TB200_CHECK_LAUNCH();
}

void launch_grads_umma(const float* E, const float* P, const float* rowRef, const float* maxP,
                       const float* W, const float* em, const float* eBlank,
                       const float* pBlank, const float* pLabel, const int* labels,
                       const float* deltas, float* egrads, float* pgrads, const int* inLens,
                       const int* labLens, Dims d, int passes, int* status,
                       cudaStream_t stream) {
  if (d.B <= 0 || d.V <= 0) return;
  GradParams p;
  p.E = E; p.P = P; p.rowRef = rowRef; p.maxP = maxP; p.eBlank = eBlank; p.pBlank = pBlank;
  p.pLabel = pLabel; p.em = em; p.labels = labels; p.inLens = inLens; p.labLens = labLens;
  p.deltas = deltas; p.egrads = egrads; p.pgrads = pgrads; p.status = status;
  p.maxT = d.maxT; p.maxU = d.maxU; p.V = d.V; p.blank = d.blank;
  p.ldW = grads_umma_ld_w(d);
  p.Ku = (int)round_up64(d.maxU, 8);
  p.stages = 0; p.tmemCols = 0;
  const int TB = pick_tile(p.Ku, p.ldW, passes);
  if (TB == 0) throw std::invalid_argument("label axis too long for the tensor-core gradient kernel");
  const CUtensorMap tmE = make_tmap_f32_3d(E, (uint64_t)d.V, (uint64_t)d.maxT, (uint64_t)d.B,
                                           (uint64_t)d.V * 4, (uint64_t)d.maxT * d.V * 4, TB);
  const CUtensorMap tmWk =
      make_tmap_f32_3d(W, (uint64_t)p.ldW, (uint64_t)d.maxT, (uint64_t)d.B, (uint64_t)p.ldW * 4,
                       (uint64_t)d.maxT * p.ldW * 4, TB);
  const CUtensorMap tmWmn =
      make_tmap_f32_3d(W, (uint64_t)p.ldW, (uint64_t)d.maxT, (uint64_t)d.B, (uint64_t)p.ldW * 4,
                       (uint64_t)d.maxT * p.ldW * 4, TB, /*atom32=*/true);
#define GO(TBV, EV, PV) launch_variant<TBV, EV, PV>(tmE, tmWk, tmWmn, p, d, stream)
#define GO_TB(EV, PV) \
  do { if (TB == 64) GO(64, EV, PV); else if (TB == 48) GO(48, EV, PV); else GO(32, EV, PV); } while (0)
  if (passes == 3) GO_TB(true, true);
  else if (passes == 2) GO_TB(true, false);
  else GO_TB(false, false);
#undef GO_TB
#undef GO
  TB200_CHECK_LAUNCH();
}

}  // namespace tb200
