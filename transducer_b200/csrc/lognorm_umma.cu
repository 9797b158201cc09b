// Log-normalisers as an exp-factored tensor-core contraction (tcgen05 / TMEM / TMA).
//
//   LN[b,t,u] = log( sum_v exp(E[b,t,v]-ref[b,t]) * exp(P[b,u,v]-maxP[b,u]) ) + ref[b,t] + maxP[b,u]
//
// which is what the reference computes with torch ops (transducer/torch_binding.py:35-40:
// row maxima, exp, bmm, log) -- here in ONE pass over E and without storing exp(E).
//
// Work item: 128 frames of one utterance (UMMA M=128) x up to 128 label positions (N = the
// positions rounded up to 16; a label axis of 129..256 positions is cut into two column ranges,
// each a work item of its own that reads the tile's chunks of E again) x the whole vocabulary
// in K-chunks of 32 words.  Emissions fp32 or bf16 (converted in the transform).
//
// Roles inside a CTA (one CTA per SM, 19 warps):
//   warps 0-7   operand transform, two groups of four that take alternate chunks.  Thread r of
//               a group owns frame r of the tile (= TMEM lane r): reads its row of the raw E
//               chunk from shared memory, computes x = exp(E - ref), splits x = hi + lo with hi
//               exactly representable in TF32, and stores hi/lo straight into TENSOR MEMORY
//               (the A operand of the MMA is read from TMEM, so the transformed tile never goes
//               back through shared memory).  On the way it hands out E[t,label_u] and
//               E[t,blank] for the lattice sweeps.
//   warps 8-15  accumulator drain + epilogue, one warpgroup per 64 accumulator columns: after
//               every kGroup chunks they add the TMEM accumulator into fp32 registers
//               (round-to-nearest) and hand the accumulator back, so the tensor core's
//               truncating accumulation never runs over more than 24 steps.
//   warp 16     TMA producer: raw E chunk + pre-split exp(P) hi/lo chunks per stage (4 stages).
//   warps 17-18 MMA issuers (one accumulator each): per 8-wide k-step three kind::tf32 MMAs
//               hi*Bhi + lo*Bhi + hi*Blo into the current accumulator (the 3xTF32 split
//               reproduces fp32 products to ~2^-21 relative).
//
// ref[b,t] is NOT the row maximum (that would cost a second pass over E): it is the
// maximum of the first 32 entries of the row.  Any reference gives the same LN as long
// as the factored sum neither overflows nor underflows in fp32; nodes where it does
// (sum not in [1e-30, 1e30], or non-finite) are marked and recomputed by the exact fp32
// SIMT logsumexp in lognorm_fixup_kernel.
#include <cuda.h>

#include <algorithm>
#include <atomic>

#include "kernels.h"
#include "profile.h"
#include "sm100.cuh"

namespace tb200 {

namespace sm100 {

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                             const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, resolved through the runtime once per process (a pure host function
// of the driver; the same pointer serves every device).
static EncodeFn tensor_map_encoder() {
  static std::atomic<EncodeFn> cached{nullptr};
  EncodeFn encode = cached.load(std::memory_order_acquire);
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    TB200_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || !fn)
      throw CudaError("cuTensorMapEncodeTiled is not available from this driver");
    encode = reinterpret_cast<EncodeFn>(fn);
    cached.store(encode, std::memory_order_release);
  }
  return encode;
}

CUtensorMap make_tmap_f32_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                             uint64_t stride1Bytes, uint64_t stride2Bytes, uint32_t box1,
                             bool atom32) {
  const EncodeFn encode = tensor_map_encoder();
  CUtensorMap m;
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {stride1Bytes, stride2Bytes};
  const cuuint32_t box[3] = {32, box1, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult rc = encode(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims,
                             strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    throw CudaError("cuTensorMapEncodeTiled failed with code " + std::to_string((int)rc));
  return m;
}

CUtensorMap make_tmap_bf16_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint64_t stride1Bytes, uint64_t stride2Bytes, uint32_t box0,
                              uint32_t box1) {
  const EncodeFn encode = tensor_map_encoder();
  CUtensorMap m;
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {stride1Bytes, stride2Bytes};
  const cuuint32_t box[3] = {box0, box1, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  // rows of the box are 64 or 128 bytes: the swizzle of that width
  const CUresult rc = encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims,
                             strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             box0 * 2 == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    throw CudaError("cuTensorMapEncodeTiled (bf16) failed with code " + std::to_string((int)rc));
  return m;
}

CUtensorMap make_tmap_f32_rows(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                               uint64_t stride1Bytes, uint64_t stride2Bytes, uint32_t box0) {
  const EncodeFn encode = tensor_map_encoder();
  CUtensorMap m;
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {stride1Bytes, stride2Bytes};
  const cuuint32_t box[3] = {box0, 1, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult rc = encode(
      &m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    throw CudaError("cuTensorMapEncodeTiled (rows) failed with code " + std::to_string((int)rc));
  return m;
}

}  // namespace sm100

namespace {

using namespace sm100;

constexpr int kTileM = 128;
constexpr int kMaxSMs = 256;                      // slots for the partial sums of split tiles
constexpr int kChunkK = 32;                       // floats per K-chunk = one 128-byte swizzle row
// raw E chunk of a stage: 128 frames x 32 words, rows of 128 bytes (fp32) or 64 bytes (bf16)
__host__ __device__ constexpr int raw_bytes(bool bf) { return kTileM * kChunkK * (bf ? 2 : 4); }
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kSumLo = 1e-30f, kSumHi = 1e30f;

// ---------------------------------------------------------------------------------
// exp(P - maxP) split into TF32 hi/lo as [B][nPad][kPad]: rows u < U_b, columns zero-padded to kPad
// ---------------------------------------------------------------------------------
template <typename TIn>
__global__ void __launch_bounds__(256) expp_split_kernel(
    const TIn* __restrict__ P, float* __restrict__ bHi, float* __restrict__ bLo,
    float* __restrict__ maxP, const int* __restrict__ labLens, int maxU, int V, int nPad,
    int kPad) {
  __shared__ float red[8];
  const int b = blockIdx.y, u = blockIdx.x;
  const int U = min(labLens[b] + 1, maxU);
  float* hi = bHi + ((i64)b * nPad + u) * kPad;
  float* lo = bLo + ((i64)b * nPad + u) * kPad;
  // rows are read and written as float4 (the caller guarantees V % 4 == 0 and 16-byte aligned
  // P; kPad is a multiple of 32)
  float4* hi4 = reinterpret_cast<float4*>(hi);
  float4* lo4 = reinterpret_cast<float4*>(lo);
  if (u >= U) {
    // Rows beyond the utterance's label axis are left as they are: row u of the operand only
    // feeds column u of the accumulator, which nobody reads for u >= U_b -- whatever the row
    // holds (stale numbers, NaN patterns) stays in that column.
    if (u < maxU && threadIdx.x == 0 && maxP) maxP[(i64)b * maxU + u] = 0.0f;
    return;
  }
  const TIn* p = P + ((i64)b * maxU + u) * V;
  float m = neg_inf();
  for (int v = threadIdx.x; v < V / 4; v += blockDim.x) {
    const float4 x = ld4(p + 4 * v);
    m = fmaxf(fmaxf(m, fmaxf(x.x, x.y)), fmaxf(x.z, x.w));
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) m = fmaxf(m, red[k]);
  for (int v = threadIdx.x; v < kPad / 4; v += blockDim.x) {
    float xs[4] = {0.0f, 0.0f, 0.0f, 0.0f}, h[4], l[4];
    if (4 * v < V) {
      const float4 x = ld4(p + 4 * v);
      xs[0] = expf(x.x - m); xs[1] = expf(x.y - m); xs[2] = expf(x.z - m); xs[3] = expf(x.w - m);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      h[k] = __uint_as_float(__float_as_uint(xs[k]) & 0xffffe000u);
      l[k] = tf32_round(xs[k] - h[k]);
    }
    hi4[v] = make_float4(h[0], h[1], h[2], h[3]);
    lo4[v] = make_float4(l[0], l[1], l[2], l[3]);
  }
  if (threadIdx.x == 0 && maxP) maxP[(i64)b * maxU + u] = m;
}

// ---------------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------------
struct LnParams {
  float* LN;
  float* rowRef;
  const float* maxP;
  const int* inLens;
  const int* labLens;
  int* status;       // [0] first error code, [1] number of nodes handed to the fix-up
  int maxT, maxU, V, stages, nAcc, tmemCols;
  // A label axis of more than 128 positions is cut into `halves` = 2 column ranges of nPad
  // positions; a work item is then (tile, range) and reads the tile's chunks of E again.
  int nPad, halves;
  // last-wave splitting (see lognorm_umma_kernel)
  int B, tilesX, nSM;
  float* partial;    // [nSM][kTileM][nPad] partial sums of split tiles
  unsigned* tickets; // [nSM] parts finished per split tile (zero on entry, zero again on exit)
  // label / blank emissions gathered on the fly (null: not wanted)
  const int* labels; // [B, maxU-1]
  float* EL;         // [B, maxU, maxT], frames contiguous: EL[b,u,t] = E[b,t,labels[b,u]], u < U_b - 1
  float* ebl;        // [B, maxT]: E[b,t,blank]
  int blank;
};

// Chunks per accumulation group.  The tensor core adds into its fp32 accumulator with
// truncation: measured on B200, every tcgen05.mma step loses ~2^-24 of the running sum
// (always downward), i.e. -2e-4 on LN after the 3750 steps of a 10000-word vocabulary.
// So an accumulator only ever sees kGroup chunks (12*kGroup steps); the drain warps then
// add it, round-to-nearest, into fp32 registers and the MMA starts a fresh accumulator.
constexpr int kGroup = 2;
// NTW   transform warpgroups (1 or 2): with 2, the groups take alternate chunks, so that one
//       group's wait for its tile and for its TMEM stores overlaps the other's exponentials.
// NDRAIN drain warpgroups, each owning DCOLS accumulator columns (fp32 sums in registers).
//
// Work items.  A tile (128 frames of one utterance x the whole vocabulary) takes the same time
// whatever it holds, and one CTA fits an SM, so n live tiles on nSM SMs cost ceil(n / nSM)
// rounds: 454 tiles on 148 SMs pay for 592.  The tiles of the last, partly filled round are
// therefore split along the vocabulary into k = min(8, nSM / rem) parts (rem = n mod nSM):
// part 0 runs in the tile's own CTA, parts 1..k-1 in `worker` CTAs appended to the grid (the
// hardware dispatches CTAs in index order, so they start exactly when the last round does).
// Every part keeps the frame's shift of the whole tile (a part that does not begin at chunk 0
// first fetches chunk 0 for it and feeds zeros to the tensor core for that chunk), writes its
// partial sums to `partial`, and the part that finishes last adds the parts in index order.
// The grid is (tilesX * B + nSM) x 1; lengths are on the device, so every CTA derives the
// schedule from them itself (B <= 1024; larger batches are not split).
constexpr int kMaxParts = 8;
constexpr int kMaxLabels = 256;
// BF: the emissions are bf16 (the raw chunk of a stage then has 64-byte rows, 64-byte swizzle).
template <int NTW, int NDRAIN, int DCOLS, bool BF = false>
__global__ void __launch_bounds__((4 * NTW + 4 * NDRAIN + 3) * 32, 1) lognorm_umma_kernel(
    const __grid_constant__ CUtensorMap tmE, const __grid_constant__ CUtensorMap tmHi,
    const __grid_constant__ CUtensorMap tmLo, const LnParams p) {
  constexpr int kDrainWarp0 = 4 * NTW;
  constexpr int kProducerWarp = kDrainWarp0 + 4 * NDRAIN, kMmaWarp = kProducerWarp + 1;
  constexpr int kThreads = (kMmaWarp + 2) * 32;  // two MMA-issuing warps
  constexpr int kDrainCols = DCOLS;
  constexpr int kRawBytes = raw_bytes(BF);
  constexpr int kRowBytes = BF ? 64 : 128;
  // 16 consecutive words of frame r's row of the raw chunk, starting at word 16 * half, as fp32
  auto load16 = [](const uint8_t* row, int r, int half, float (&x)[16]) {
    if constexpr (BF) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int jj = half * 2 + j;  // 16-byte piece (8 words) of the 64-byte row
        const uint4 q = *reinterpret_cast<const uint4*>(row + ((jj ^ ((r >> 1) & 3)) << 4));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          x[8 * j + 2 * k] = __uint_as_float(w[k] << 16);
          x[8 * j + 2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int jj = half * 4 + j;  // 16-byte piece of the 128-byte row
        const float4 v4 = *reinterpret_cast<const float4*>(row + ((jj ^ (r & 7)) << 4));
        x[4 * j] = v4.x; x[4 * j + 1] = v4.y; x[4 * j + 2] = v4.z; x[4 * j + 3] = v4.w;
      }
    }
  };
  // word `off` (0..31) of frame r's row
  auto load1 = [](const uint8_t* row, int r, int off) {
    if constexpr (BF) {
      const unsigned short h = *reinterpret_cast<const unsigned short*>(
          row + (((off >> 3) ^ ((r >> 1) & 3)) << 4) + (off & 7) * 2);
      return __uint_as_float((uint32_t)h << 16);
    } else {
      return *reinterpret_cast<const float*>(row + (((off >> 2) ^ (r & 7)) << 4) + (off & 3) * 4);
    }
  };
  // ---- which work item is this CTA? (warp 0 scans the lengths; before any allocation) ----
  __shared__ int sItem[6];  // b, tile, part, parts, split-tile index, valid
  if (threadIdx.x < 32) {
    const int lane0 = threadIdx.x;
    const int perUtt = p.tilesX * p.halves;   // grid slots per utterance
    const int nNatural = perUtt * p.B;
    const bool worker = (int)blockIdx.x >= nNatural;
    const int myB = worker ? -1 : (int)blockIdx.x / perUtt, myX = worker ? 0 : (int)blockIdx.x % perUtt;
    // live work items of an utterance: tiles x column ranges that hold positions (item ix is
    // range ix % ranges of tile ix / ranges, so the ranges of a tile run side by side and
    // share its chunks of E in L2)
    auto ranges = [&](int bb) {
      const int Ub = min(p.labLens[bb] + 1, p.maxU);
      return min(p.halves, (Ub + p.nPad - 1) / p.nPad);
    };
    auto liveTiles = [&](int bb) {
      if (bb >= p.B) return 0;
      const int Tb = min(p.inLens[bb], p.maxT), Ub = min(p.labLens[bb] + 1, p.maxU);
      return (Tb > 0 && Ub > 0) ? ((Tb + kTileM - 1) / kTileM) * ranges(bb) : 0;
    };
    int n = 0, before = 0;  // live tiles in all, and in the utterances before mine
    for (int b0 = 0; b0 < p.B; b0 += 32) {
      const int v = liveTiles(b0 + lane0);
      const int tot = __reduce_add_sync(0xffffffffu, v);
      const int pre = __reduce_add_sync(0xffffffffu, (b0 + lane0 < myB) ? v : 0);
      n += tot;
      before += pre;
    }
    const int full = (n / p.nSM) * p.nSM, rem = n - full;
    int k = (rem > 0 && p.B <= 1024) ? min(kMaxParts, p.nSM / rem) : 1;
    k = min(k, ((p.V + kChunkK - 1) / kChunkK) / 16);  // a part is worth >= 16 chunks
    if (k < 2) k = 1;
    int ib = -1, ix = 0, part = 0, parts = 1, split = 0, valid = 0;
    if (!worker) {
      if (myX < liveTiles(myB)) {
        valid = 1; ib = myB; ix = myX;
        const int r = before + myX;
        if (k > 1 && r >= full) { parts = k; split = r - full; }
      }
    } else if (k > 1) {
      const int w = (int)blockIdx.x - nNatural;
      if (w < rem * (k - 1)) {
        split = w / (k - 1);
        part = 1 + w % (k - 1);
        parts = k;
        // locate the tile of live rank full + split
        const int target = full + split;
        int run = 0;
        for (int b0 = 0; b0 < p.B && !valid; b0 += 32) {
          const int v = liveTiles(b0 + lane0);
          int incl = v;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane0 >= o) incl += up;
          }
          const int lo = run + incl - v, hi = run + incl;  // my utterance holds ranks [lo, hi)
          const unsigned hit = __ballot_sync(0xffffffffu, target >= lo && target < hi);
          if (hit) {
            const int src = __ffs(hit) - 1;
            ib = b0 + src;
            ix = target - __shfl_sync(0xffffffffu, lo, src);
            valid = 1;
          }
          run += __shfl_sync(0xffffffffu, incl, 31);
        }
      }
    }
    if (lane0 == 0) {
      sItem[0] = ib; sItem[1] = ix; sItem[2] = part; sItem[3] = parts; sItem[4] = split; sItem[5] = valid;
    }
  }
  __syncthreads();
  if (!sItem[5]) return;
  const int b = sItem[0];
  const int part = sItem[2], parts = sItem[3], splitIdx = sItem[4];
  const int T = min(p.inLens[b], p.maxT), U = min(p.labLens[b] + 1, p.maxU);
  const int nRanges = min(p.halves, (U + p.nPad - 1) / p.nPad);
  const int t0 = (sItem[1] / nRanges) * kTileM;
  const int uOff = (sItem[1] % nRanges) * p.nPad;   // first label position of my column range

  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) &
                                             ~uintptr_t(1023));
  const int S = p.stages, nAcc = p.nAcc;
  const int bBytes = p.nPad * kChunkK * 4;
  const int stageBytes = kRawBytes + 2 * bBytes;
  __shared__ uint64_t barFull[4], barReady[4], barDone[4], barAccFull[2], barAccEmpty[2], barRef;
  __shared__ uint32_t tmemBase;
  __shared__ int abortFlag;
  __shared__ float sMaxP[256];
  __shared__ float sRef[kTileM];
  __shared__ int sLast;
  // While a transform thread holds its frame's row of a chunk it also hands out the entries
  // the lattice sweeps need: E[t, label_u] for the labels whose column lies in the chunk (the
  // utterance's labels are sorted by column once per CTA) and E[t, blank].  That replaces a
  // gather pass that fetched one DRAM sector per lattice node (transducer_cuda.cu:84 does that
  // gather inside its wavefront).
  __shared__ int sKey[kMaxLabels];      // (column << 8 | label position u), ascending

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // this part's chunks [cBegin, cEnd); iteration i of the pipeline handles chunk chunkOf(i)
  const int nChunksAll = (p.V + kChunkK - 1) / kChunkK;
  const int cBegin = (int)((i64)part * nChunksAll / parts), cEnd = (int)((i64)(part + 1) * nChunksAll / parts);
  const bool refFirst = part > 0;  // iteration 0 fetches chunk 0 for the frames' shifts only
  const int nChunks = cEnd - cBegin + (refFirst ? 1 : 0);  // pipeline iterations
  auto chunkOf = [&](int i) { return refFirst ? (i == 0 ? 0 : cBegin + i - 1) : cBegin + i; };
  const int nGroups = (nChunks + kGroup - 1) / kGroup;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&barFull[s], 1);
      mbar_init(&barReady[s], 4);   // the one transform group that owns the chunk
      mbar_init(&barDone[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&barAccFull[a], 1);
      mbar_init(&barAccEmpty[a], 4 * NDRAIN);
    }
    mbar_init(&barRef, 4);
    abortFlag = 0;
    fence_mbar_init();
  }
  for (int u = threadIdx.x; u < p.nPad; u += kThreads)
    sMaxP[u] = (uOff + u < U) ? p.maxP[(i64)b * p.maxU + uOff + u] : 0.0f;
  const bool gather = p.EL != nullptr && uOff == 0;   // (one range hands out the emissions)
  const int nLab = gather ? min(U - 1, kMaxLabels) : 0;
  if (gather) {  // rank sort by column (from a shared-memory copy); ties keep position order
    __shared__ int sLab[kMaxLabels];
    const int* lab = p.labels + (i64)b * (p.maxU - 1);
    for (int i = threadIdx.x; i < nLab; i += kThreads) sLab[i] = lab[i];
    __syncthreads();
    for (int i = threadIdx.x; i < nLab; i += kThreads) {
      const int mine = sLab[i];
      int rank = 0;
      for (int j = 0; j < nLab; ++j) {
        const int o = sLab[j];
        rank += (o < mine || (o == mine && j < i)) ? 1 : 0;
      }
      sKey[rank] = (mine << 8) | i;
    }
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&tmemBase, (uint32_t)p.tmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tBase = tmemBase;                          // accumulators: nAcc x nPad columns
  const uint32_t tA = tBase + (uint32_t)(nAcc * p.nPad);    // operand stages: [hi 32 | lo 32] each
  volatile int* abortp = &abortFlag;

  if (warp == kProducerWarp) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmE);
      tma_prefetch_desc(&tmHi);
      tma_prefetch_desc(&tmLo);
      int issued = 0, s = 0;
      uint32_t ph = 1;  // phase of the PREVIOUS release of the stage (stage and phase are carried
                        // along: a division by the run-time ring depth costs a lone thread ~100 cycles)
      for (int c = 0; c < nChunks; ++c) {
        if (c >= S && !mbar_wait(&barDone[s], ph, abortp, p.status, kStatusTimeoutStageFree)) break;
        uint8_t* st = smem + (size_t)s * stageBytes;
        mbar_arrive_expect_tx(&barFull[s], (uint32_t)stageBytes);
        const int col = chunkOf(c) * kChunkK;
        tma_load_3d(st, &tmE, &barFull[s], col, t0, b);
        tma_load_3d(st + kRawBytes, &tmHi, &barFull[s], col, uOff, b);
        tma_load_3d(st + kRawBytes + bBytes, &tmLo, &barFull[s], col, uOff, b);
        issued = c + 1;
        if (++s == S) { s = 0; ph ^= 1u; }
      }
      if (*abortp) {
        // after an abort: give the copies still in flight a bounded time to land
        // before the CTA's shared memory is released
        for (int c = max(0, issued - S); c < issued; ++c) {
          const unsigned long long t1 = global_timer_ns();
          while (!mbar_try_wait(&barFull[c % S], (c / S) & 1) &&
                 global_timer_ns() - t1 < 50000000ull) {
          }
        }
      }
    }
  } else if (warp >= kMmaWarp) {
    // ---------------- MMA issuers ----------------
    // One elected thread in each of two warps.  Issuer m owns accumulator m and therefore
    // the chunk groups g with g % 2 == m: while one issuer is blocked on its barrier waits
    // and commits (~800 cycles per chunk, measured), the other keeps the tensor pipe fed.
    // The two never touch the same accumulator or operand stage, so no order between their
    // MMAs is needed.
    const int m = warp - kMmaWarp;
    if (lane == 0 && m < nAcc) {
      const uint32_t idesc = idesc_tf32(kTileM, p.nPad, 0, 0);
      bool ok = true;
      int s = -1;
      uint32_t ph = 1;
      for (int c = 0; c < nChunks && ok; ++c) {
        if (++s == S) s = 0;
        if (s == 0) ph ^= 1u;   // stage c % S, phase (c / S) & 1, without the division
        const int g = c / kGroup, a = (nAcc == 2) ? (g & 1) : 0;
        if (a != m) continue;
        const int gUse = (nAcc == 2) ? (g >> 1) : g;   // how often accumulator a was used before
        if (c % kGroup == 0 && g >= nAcc)
          ok = mbar_wait(&barAccEmpty[a], (gUse - 1) & 1, abortp, p.status,
                         kStatusTimeoutStageFree);
        // the transform warps arrive on barReady only after they saw barFull complete, so
        // the copies of this stage (the exp(P) tiles among them) have landed as well
        ok = ok && mbar_wait(&barReady[s], ph, abortp, p.status, kStatusTimeoutOperand);
        if (!ok) break;
        tc_fence_after();
        const uint32_t bHi = smem_u32(smem + (size_t)s * stageBytes + kRawBytes);
        const uint32_t bLo = bHi + (uint32_t)bBytes;
        const uint32_t aHi = tA + (uint32_t)(s * 64), aLo = aHi + 32;
        const uint32_t dAcc = tBase + (uint32_t)(a * p.nPad);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t dHi = smem_desc_sw128(bHi + k * 32, 16, 1024);
          const uint64_t dLo = smem_desc_sw128(bLo + k * 32, 16, 1024);
          mma_tf32_ts(dAcc, aHi + k * 8, dHi, idesc, ((c % kGroup) | k) ? 1u : 0u);
          mma_tf32_ts(dAcc, aLo + k * 8, dHi, idesc, 1u);
          mma_tf32_ts(dAcc, aHi + k * 8, dLo, idesc, 1u);
        }
        mma_commit(&barDone[s]);
        if (c % kGroup == kGroup - 1 || c == nChunks - 1) mma_commit(&barAccFull[a]);
      }
    }
  } else if (warp < kDrainWarp0) {
    // ---------------- operand transform (thread = frame = TMEM lane) ----------------
    const int q = warp & 3, grp = warp >> 2;    // lane quarter, transform group
    const int r = q * 32 + lane;                // frame within the tile, 0..127
    const uint32_t laneAddr = (uint32_t)(q * 32) << 16;
    float ref = 0.0f;
    bool ok = true;
    if (grp > 0) {  // the frame's shift is found by group 0 in chunk 0
      ok = mbar_wait(&barRef, 0, abortp, p.status, kStatusTimeoutOperand);
      ok = __all_sync(0xffffffffu, ok);
      ref = sRef[r];
    }
    int cur = 0;  // cursor into the sorted label list (the same in every thread)
    // column of the next entry that this group has not passed yet, kept in a register so that a
    // chunk without any costs one comparison and no shared-memory access
    int nextCol = (gather && nLab > 0) ? (sKey[0] >> 8) : 0x7fffffff;
    float* elCol = gather ? p.EL + (i64)b * p.maxU * p.maxT + t0 + r : nullptr;  // my frame
    int s = grp % S;
    uint32_t ph = (grp / S) & 1;
    for (int c = grp; c < nChunks && ok; c += NTW) {
      ok = mbar_wait(&barFull[s], ph, abortp, p.status, kStatusTimeoutTma);
      ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the aligned TMEM ops
      if (!ok) break;
      const uint8_t* row = smem + (size_t)s * stageBytes + r * kRowBytes;
      const int kLeft = p.V - chunkOf(c) * kChunkK;  // valid columns in this chunk
      const bool refOnly = refFirst && c == 0;           // its terms belong to part 0
      if (c == 0) {
        // the frame's shift: maximum of the first 32 entries of the row
        float m = neg_inf();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float x[16];
          load16(row, r, half, x);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (half * 16 + j < kLeft) m = fmaxf(m, x[j]);
        }
        // a -inf/NaN prefix would poison every term; fall back to 0 and let the
        // range check route the row to the exact path if needed
        ref = (m > -3.0e38f && m < 3.0e38f) ? m : 0.0f;
        sRef[r] = ref;
        if (t0 + r < T && part == 0 && uOff == 0) p.rowRef[(i64)b * p.maxT + t0 + r] = ref;
      }
      const int col0 = chunkOf(c) * kChunkK;
      if (gather && !refOnly && nextCol < col0 + kChunkK) {
        // (uniform control flow: the list and the cursor are the same in all threads)
        int key = sKey[cur];
        while ((key >> 8) < col0 && ++cur < nLab) key = sKey[cur];   // the other group's chunks
        while (cur < nLab && (key >> 8) < col0 + kChunkK) {
          const int off = (key >> 8) - col0;
          const float v = load1(row, r, off);
          // (the 128 threads of the group write 128 consecutive floats of row u)
          if (t0 + r < T) elCol[(i64)(key & 0xff) * p.maxT] = v;
          if (++cur < nLab) key = sKey[cur];
        }
        nextCol = cur < nLab ? (key >> 8) : 0x7fffffff;
      }
      if (gather && !refOnly) {
        if (p.blank >= col0 && p.blank < col0 + kChunkK) {
          const int off = p.blank - col0;
          const float v = load1(row, r, off);
          if (t0 + r < T) p.ebl[(i64)b * p.maxT + t0 + r] = v;
        }
      }
      const float nref = -ref * kLog2e;
      const uint32_t dst = tA + laneAddr + (uint32_t)(s * 64);
#pragma unroll
      for (int half = 0; half < 2; ++half) {  // 16 columns at a time (registers)
        float x[16];
        load16(row, r, half, x);
        const int kLeftMine = refOnly ? 0 : kLeft - half * 16;
        uint32_t hi[16], lo[16];
        if (kLeftMine >= 16) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float e = ex2_approx(fmaf(x[j], kLog2e, nref));
            const uint32_t hbits = __float_as_uint(e) & 0xffffe000u;
            hi[j] = hbits;
            lo[j] = __float_as_uint(e - __uint_as_float(hbits));
          }
        } else {  // last chunk of a vocabulary that is not a multiple of 32
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float e = (j < kLeftMine) ? ex2_approx(fmaf(x[j], kLog2e, nref)) : 0.0f;
            const uint32_t hbits = __float_as_uint(e) & 0xffffe000u;
            hi[j] = hbits;
            lo[j] = __float_as_uint(e - __uint_as_float(hbits));
          }
        }
        tmem_st16(dst + half * 16, hi);
        tmem_st16(dst + 32 + half * 16, lo);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&barReady[s]);
        if (c == 0) mbar_arrive(&barRef);
      }
      s += NTW;   // (NTW <= 2 steps at a time; the ring holds at least one stage)
      while (s >= S) { s -= S; ph ^= 1u; }
    }
  } else {
    // ---------------- accumulator drain + epilogue ----------------
    const int h = (warp - kDrainWarp0) >> 2;     // which column slice
    const int q = warp & 3;                      // TMEM lane quarter this warp may touch
    const int r = q * 32 + lane;
    const uint32_t laneAddr = (uint32_t)(q * 32) << 16;
    const int c0 = h * kDrainCols, c1 = min(p.nPad, c0 + kDrainCols);
    float sum[kDrainCols];
#pragma unroll
    for (int j = 0; j < kDrainCols; ++j) sum[j] = 0.0f;
    bool ok = true;
    for (int g = 0; g < nGroups && ok; ++g) {
      const int a = (nAcc == 2) ? (g & 1) : 0;
      ok = mbar_wait(&barAccFull[a], ((nAcc == 2) ? (g >> 1) : g) & 1, abortp, p.status, kStatusTimeoutMma);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t src = tBase + laneAddr + (uint32_t)(a * p.nPad + c0);
      constexpr int kBatch = (DCOLS >= 128) ? 2 : 1;  // TMEM loads in flight per wait
#pragma unroll
      for (int i0 = 0; i0 < kDrainCols / 16; i0 += kBatch) {
        uint32_t v[kBatch][16];
#pragma unroll
        for (int i = 0; i < kBatch; ++i)
          if (c0 + (i0 + i) * 16 < c1) tmem_ld16(src + (i0 + i) * 16, v[i]);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < kBatch; ++i)
          if (c0 + (i0 + i) * 16 < c1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) sum[(i0 + i) * 16 + j] += __uint_as_float(v[i][j]);
          }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&barAccEmpty[a]);
    }
    if (ok) ok = mbar_wait(&barRef, 0, abortp, p.status, kStatusTimeoutOperand);
    ok = __all_sync(0xffffffffu, ok);
    // A warp that gave up (ok == false; the cause is in the status word) turns its sums into
    // NaN: the nodes then carry the "recompute exactly" marker instead of stale memory.
    const float bad = __int_as_float(0x7fc00000);
    if (!ok) {
#pragma unroll
      for (int j = 0; j < kDrainCols; ++j) sum[j] = bad;
    }
    bool writer = true;  // does this CTA write the tile's log-normalisers?
    if (parts > 1) {
      // split tile: park the partial sums; the part that finishes last adds all of them in
      // part order (so the result does not depend on which part that is) and goes on
      float* mine = p.partial + ((size_t)(splitIdx * parts + part) * kTileM + r) * p.nPad + c0;
#pragma unroll
      for (int j = 0; j < kDrainCols; ++j)
        if (c0 + j < c1) mine[j] = sum[j];
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"r"(4 * NDRAIN * 32) : "memory");
      if (warp == kDrainWarp0 && lane == 0) {
        const unsigned done = atomicAdd(&p.tickets[splitIdx], 1u);
        sLast = (done == (unsigned)(parts - 1)) ? 1 : 0;
        if (sLast) p.tickets[splitIdx] = 0u;  // ready for the next launch
      }
      asm volatile("bar.sync 1, %0;" ::"r"(4 * NDRAIN * 32) : "memory");
      writer = sLast != 0;
      if (writer) {
        __threadfence();
#pragma unroll
        for (int j = 0; j < kDrainCols; ++j) sum[j] = 0.0f;
        for (int z = 0; z < parts; ++z) {
          const float* src = p.partial + ((size_t)(splitIdx * parts + z) * kTileM + r) * p.nPad + c0;
#pragma unroll
          for (int j = 0; j < kDrainCols; ++j)
            if (c0 + j < c1) sum[j] += __ldcg(src + j);
        }
      }
    }
    if (writer) {
      const int t = t0 + r;
      const float ref = ok ? sRef[r] : 0.0f;
      int flagged = 0;
      if (t < T) {
        float* out = p.LN + ((i64)b * p.maxT + t) * p.maxU;
#pragma unroll
        for (int j = 0; j < kDrainCols; ++j) {
          const int u = uOff + c0 + j;
          if (c0 + j < c1 && u < U) {
            const float acc = sum[j];
            float ln = (logf(acc) + ref) + sMaxP[c0 + j];
            if (!(acc >= kSumLo && acc <= kSumHi)) {
              ln = bad;  // marker: recompute exactly
              ++flagged;
            }
            out[u] = ln;
          }
        }
      }
      if (flagged) atomicAdd(&p.status[1], flagged);
    }
  }

  // ---------------- teardown (all roles, also after an abort) ----------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kMmaWarp) tmem_dealloc(tBase, (uint32_t)p.tmemCols);
}

// Recomputes marked nodes (NaN in LN) with the exact fp32 logsumexp.  One warp per frame
// (b, t): it scans the frame's nodes 32 at a time; marked ones are evaluated by the whole warp.
template <typename TIn>
__global__ void __launch_bounds__(256) lognorm_fixup_kernel(
    const TIn* __restrict__ E, const TIn* __restrict__ P, float* __restrict__ LN,
    const int* __restrict__ inLens, const int* __restrict__ labLens, int B, int maxT, int maxU,
    int V) {
  const int lane = threadIdx.x & 31;
  const i64 row = (i64)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= (i64)B * maxT) return;
  const int b = (int)(row / maxT), t = (int)(row % maxT);
  if (t >= min(inLens[b], maxT)) return;
  const int U = min(labLens[b] + 1, maxU);
  const TIn* er = E + row * V;
  float* ln = LN + row * maxU;
  for (int u0 = 0; u0 < U; u0 += 32) {
    const int u = u0 + lane;
    const float v0 = (u < U) ? ln[u] : 0.0f;
    unsigned todo = __ballot_sync(0xffffffffu, v0 != v0);
    while (todo) {
      const int src = __ffs(todo) - 1;
      todo &= todo - 1;
      const TIn* pr = P + ((i64)b * maxU + u0 + src) * V;
      float m = neg_inf();
      for (int v = lane; v < V; v += 32) m = fmaxf(m, to_f32(er[v]) + to_f32(pr[v]));
      m = warp_max(m);
      float s = 0.0f;
      if (m != neg_inf() && m != pos_inf())
        for (int v = lane; v < V; v += 32) s += expf((to_f32(er[v]) + to_f32(pr[v])) - m);
      s = warp_sum(s);
      if (lane == 0) ln[u0 + src] = logf(s) + m;
    }
  }
}

int pow2_at_least(int x) {
  int p = 32;
  while (p < x) p <<= 1;
  return p;
}

}  // namespace

bool lognorm_umma_supported(const void* E, const void* P, Dims d) {
  return d.V % (d.dtype == kDtypeBf16 ? 8 : 4) == 0 && d.V >= 32 && d.maxU >= 1 && d.maxU <= 256 &&
         (reinterpret_cast<uintptr_t>(E) & 15) == 0 && (reinterpret_cast<uintptr_t>(P) & 15) == 0 &&
         d.B <= 65535;
}

// Label axis as the kernel sees it: up to 128 positions in one column range, more in two equal
// ranges (each a multiple of 16); the operand arrays hold ranges * part rows.
struct LabelAxis {
  int ranges, part;
  int rows() const { return ranges * part; }
};
LabelAxis label_axis(int maxU) {
  const int n = (int)round_up64(maxU > 0 ? maxU : 1, 16);
  if (n <= 128) return LabelAxis{1, n};
  return LabelAxis{2, (int)round_up64((n + 1) / 2, 16)};
}

size_t lognorm_umma_workspace_floats(Dims d) {
  const size_t nPad = (size_t)label_axis(d.maxU).rows();
  const size_t kPad = (size_t)round_up64(d.V, kChunkK);
  // exp(P) hi and lo; partial sums of split tiles (one slot per SM at most); their tickets
  return 2 * (size_t)d.B * nPad * kPad + (size_t)kMaxSMs * kTileM * nPad + kMaxSMs;
}

bool lognorm_umma_gathers(Dims d) { return d.maxU >= 1 && d.maxU <= kMaxLabels; }

void launch_lognorm_umma(const void* E, const void* P, float* LN, float* rowRef, float* maxP,
                         const int* inLens, const int* labLens, Dims d, float* splitWs,
                         int* status, bool fixup, cudaStream_t stream, const int* labels,
                         float* EL, float* ebl) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 0) return;
  const LabelAxis axis = label_axis(d.maxU);
  const int nPad = axis.rows();          // rows of the exp(P) operand arrays
  const int nPart = axis.part;           // label positions per work item
  const int kPad = (int)round_up64(d.V, kChunkK);
  const bool bf = d.dtype == kDtypeBf16;
  float* bHi = splitWs;
  float* bLo = splitWs + (size_t)d.B * nPad * kPad;
  {
    ScopedKernel sk("expp_split", stream);
    if (bf)
      expp_split_kernel<bf16><<<dim3(nPad, d.B), 256, 0, stream>>>(
          static_cast<const bf16*>(P), bHi, bLo, maxP, labLens, d.maxU, d.V, nPad, kPad);
    else
      expp_split_kernel<float><<<dim3(nPad, d.B), 256, 0, stream>>>(
          static_cast<const float*>(P), bHi, bLo, maxP, labLens, d.maxU, d.V, nPad, kPad);
  }
  TB200_CHECK_LAUNCH();

  const CUtensorMap tmE =
      bf ? make_tmap_bf16_3d(E, (uint64_t)d.V, (uint64_t)d.maxT, (uint64_t)d.B, (uint64_t)d.V * 2,
                             (uint64_t)d.maxT * d.V * 2, kChunkK, kTileM)
         : make_tmap_f32_3d(E, (uint64_t)d.V, (uint64_t)d.maxT, (uint64_t)d.B, (uint64_t)d.V * 4,
                            (uint64_t)d.maxT * d.V * 4, kTileM);
  const CUtensorMap tmHi = make_tmap_f32_3d(bHi, (uint64_t)kPad, (uint64_t)nPad, (uint64_t)d.B,
                                            (uint64_t)kPad * 4, (uint64_t)nPad * kPad * 4, nPart);
  const CUtensorMap tmLo = make_tmap_f32_3d(bLo, (uint64_t)kPad, (uint64_t)nPad, (uint64_t)d.B,
                                            (uint64_t)kPad * 4, (uint64_t)nPad * kPad * 4, nPart);

  LnParams p;
  p.LN = LN; p.rowRef = rowRef; p.maxP = maxP; p.inLens = inLens; p.labLens = labLens;
  p.status = status;
  p.maxT = d.maxT; p.maxU = d.maxU; p.V = d.V; p.nPad = nPart; p.halves = axis.ranges;
  p.labels = nullptr; p.EL = nullptr; p.ebl = nullptr; p.blank = d.blank;
  int dev = 0, nSM = 0;
  TB200_CUDA_CHECK(cudaGetDevice(&dev));
  TB200_CUDA_CHECK(cudaDeviceGetAttribute(&nSM, cudaDevAttrMultiProcessorCount, dev));
  p.B = d.B;
  p.tilesX = div_up(d.maxT, kTileM);
  p.nSM = std::min(nSM, kMaxSMs);
  p.partial = bLo + (size_t)d.B * nPad * kPad;
  p.tickets = reinterpret_cast<unsigned*>(p.partial + (size_t)kMaxSMs * kTileM * nPad);
  TB200_CUDA_CHECK(cudaMemsetAsync(p.tickets, 0, sizeof(unsigned) * kMaxSMs, stream));
  const int stageBytes = raw_bytes(bf) + 2 * nPart * kChunkK * 4;
  // Tensor memory (512 columns): two accumulators of nPart <= 128 columns (the MMA of one group
  // of chunks runs while the previous group is drained), then four operand stages of 64 columns.
  // Four stages exactly: the two MMA-issuing threads take the chunks in groups of two, and only
  // then does every stage have a single consumer of each kind, in program order (with fewer, a
  // fast issuer could mistake an older phase of a stage's barrier for its own).  One CTA per SM.
  const int stages = 4, nAcc = 2;
  if (stages * stageBytes + 2048 > 220 * 1024 || nAcc * nPart + stages * 64 > 512)
    throw std::invalid_argument("label axis too long for the tensor-core log-normaliser");
  p.stages = stages;
  p.nAcc = nAcc;
  p.tmemCols = pow2_at_least(nAcc * nPart + stages * 64);
  size_t smem = (size_t)stages * stageBytes + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;
  // one CTA per (tile, column range) + workers for the split items of the last round
  dim3 grid((unsigned)(p.tilesX * p.halves * d.B + p.nSM));
  {
    ScopedKernel sk("lognorm_umma", stream);
    if (labels != nullptr && EL != nullptr && ebl != nullptr && lognorm_umma_gathers(d)) {
      p.labels = labels; p.EL = EL; p.ebl = ebl;
    }
    // 8 transform + 8 drain (64 columns each) warps, producer, two MMA issuers
    if (bf) {
      auto k = lognorm_umma_kernel<2, 2, 64, true>;
      TB200_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      k<<<grid, 19 * 32, smem, stream>>>(tmE, tmHi, tmLo, p);
    } else {
      auto k = lognorm_umma_kernel<2, 2, 64>;
      TB200_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      k<<<grid, 19 * 32, smem, stream>>>(tmE, tmHi, tmLo, p);
    }
  }
  TB200_CHECK_LAUNCH();
  if (fixup) {
    ScopedKernel sk("lognorm_fixup", stream);
    const unsigned rows = (unsigned)d.B * (unsigned)d.maxT;
    if (bf)
      lognorm_fixup_kernel<bf16><<<(rows + 7) / 8, 256, 0, stream>>>(
          static_cast<const bf16*>(E), static_cast<const bf16*>(P), LN, inLens, labLens, d.B,
          d.maxT, d.maxU, d.V);
    else
      lognorm_fixup_kernel<float><<<(rows + 7) / 8, 256, 0, stream>>>(
          static_cast<const float*>(E), static_cast<const float*>(P), LN, inLens, labLens, d.B,
          d.maxT, d.maxU, d.V);
  }
  TB200_CHECK_LAUNCH();
}

}  // namespace tb200
