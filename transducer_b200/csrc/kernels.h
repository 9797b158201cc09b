// Host-side launchers of the sm_100a kernels.  Every launcher enqueues work on
// `stream` and returns without synchronising; errors are thrown as tb200::CudaError.
#pragma once

#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

#include "common.cuh"

namespace tb200 {

// Problem geometry shared by all launchers (names follow transducer/transducer.h):
// emissions [B,maxT,V], predictions [B,maxU,V] (maxU = longest label + 1),
// lattices [B,maxT,maxU], labels [B,maxU-1].
// dtype: storage type of emissions, predictions and their gradients (kDtypeF32 / kDtypeBf16);
// launchers that take them as `const void*` read it, all others are fp32 only.
struct Dims {
  int B, maxT, maxU, V, blank;
  int dtype = kDtypeF32;
};

constexpr int kMaxLatticeU = 8192;  // widest label axis the wavefront kernels take

// ---- lattice.cu ------------------------------------------------------------
// transducer.h `forward`: row-major lattices, emission terms gathered from E.
void launch_alpha(const float* E, const float* P, float* costs, float* alphas,
                  const float* LN, const int* labels, const int* inLens,
                  const int* labLens, Dims d, float* lossSum, unsigned* ticket,
                  cudaStream_t stream);

// transducer.h `backward`: the three outputs must already be zero-filled; lngrads
// receives the node occupancies and the sparse blank/label terms are subtracted in
// place from egrads/pgrads.
void launch_gamma_abi(const float* E, const float* P, float* egrads, float* pgrads,
                      float* lngrads, const float* alphas, const float* LN,
                      const int* labels, const int* inLens, const int* labLens,
                      Dims d, cudaStream_t stream);

// Skewed lattice storage used by the fused path: node (t,u) of utterance b lives at
// b*stride + (t+u)*ld + u, so one wavefront step reads and writes one contiguous row.
struct SkewGeom {
  int ld;       // floats per anti-diagonal row (maxU rounded up to 32)
  int nDiag;    // rows per utterance
  i64 stride;   // floats per utterance
};
SkewGeom skew_geom(Dims d);

// "No such arc" in the skewed arc-term array of the single-warp sweeps: a large negative
// finite float (-5.97e29) whose four bytes are equal, so that memset can write it.
constexpr unsigned kNoArcBits = 0xF0F0F0F0u;
constexpr int kNoArcByte = 0xF0;

// LN (row-major) -> LNs (skewed); ELs[t,u] = E[t,label_u] (skewed, skipped if null);
// ebl[b,t] = E[t,blank].  NaN entries of LN (nodes the tensor-core log-normaliser marked)
// are recomputed here with the exact fp32 logsumexp.
// If arcs is not null: arcs[t,u] (skewed, [B,nDiag,ld] float2) = log2-unit log-probabilities of
// the blank arc and the label arc leaving node (t,u), kNoArcBits where there is none.
// If ELrow is not null it holds E[t,label_u] as [B,maxU,maxT] (frames contiguous) and ebl is an
// INPUT (both written by launch_lognorm_umma): nothing is gathered from E here.
// E and P are of d.dtype.
void launch_lattice_prep(const void* E, const void* P, const float* LN, float* LNs,
                         float* ELs, float* ebl, float2* arcs, const int* labels,
                         const int* inLens, const int* labLens, SkewGeom g, Dims d,
                         cudaStream_t stream, const float* ELrow = nullptr);

void launch_alpha_skew(const float* P, float* costs, float* alphasS, const float* LNs,
                       const float* ELs, const float* ebl, SkewGeom g, const int* labels,
                       const int* inLens, const int* labLens, Dims d, float* lossSum,
                       unsigned* ticket, cudaStream_t stream);

// Fused-path reverse sweep on skewed lattices.  Writes (skewed) Ws[t,u] = occupancy *
// exp(rowRef[t] + maxP[u] - LN[t,u]) and the label-arc occupancies EMs, plus the summed
// sparse terms eBlank [B,maxT], pBlank [B,maxU], pLabel [B,maxU].
void launch_gamma_skew(const float* P, const float* alphasS, const float* LNs,
                       const float* ELs, const float* ebl, SkewGeom g, const float* rowRef,
                       const float* maxP, const int* labels, const int* inLens,
                       const int* labLens, float* Ws, float* EMs, float* eBlank,
                       float* pBlank, float* pLabel, Dims d, cudaStream_t stream);

// Ws/EMs (skewed) -> W [B,maxT,ldW] (zero outside the valid lattice) and em [B,maxT,maxU].
void launch_lattice_unskew(const float* Ws, const float* EMs, float* W, int ldW, float* em,
                           const int* inLens, const int* labLens, SkewGeom g, Dims d,
                           cudaStream_t stream);

// Max-plus wavefront + bounded on-device backtrack + label argmax on the path.
// best [B,maxT,maxU] holds max_{v != blank}(E[t,v]+P[u,v]); decBits is scratch of
// viterbi_decbits_words(d) 32-bit words.
size_t viterbi_decbits_words(Dims d);
void launch_viterbi_lattice(const float* E, const float* P, const float* LN,
                            const float* best, uint32_t* decBits, int* labels,
                            const int* inLens, const int* labLens, Dims d,
                            cudaStream_t stream);

// ---- lognorm_simt.cu ---------------------------------------------------------
// Exact fp32 logsumexp_v(E[t,v]+P[u,v]) for every valid (t,u); one warp per node.
void launch_lognorm_exact(const float* E, const float* P, float* LN, const int* inLens,
                          const int* labLens, Dims d, cudaStream_t stream);
// The same for a device-resident list of nodes (packed b,t,u triples), count read
// from *count on the device (at most maxCount entries are processed).
void launch_lognorm_exact_list(const float* E, const float* P, float* LN,
                               const int* cells, const int* count, int maxCount,
                               Dims d, cudaStream_t stream);
// rowRef[b,t] = max_v E[b,t,v] for t < T_b (0 elsewhere).
void launch_row_max(const float* X, float* rowMax, const int* lens, int lenOffset,
                    int B, int maxRows, int V, cudaStream_t stream);
// expP[b,u,v] = exp(P[b,u,v]-maxP[b,u]) for u <= labLens[b], 0 for padded rows;
// also writes maxP[b,u] (0 for padded rows).
void launch_exp_rows(const float* P, float* expP, float* maxP, const int* labLens,
                     int B, int maxU, int V, cudaStream_t stream);

// ---- lognorm_umma.cu ----------------------------------------------------------
// Tensor-core log-normalisers (one pass over E; E and P of d.dtype, bf16 only for label axes of
// at most 128 positions).  Usable when lognorm_umma_supported();
// splitWs holds lognorm_umma_workspace_floats(d) floats; status is the device status word
// (api_internal.h): [0] first device-side error code (0 = none), [1] nodes recomputed exactly.
bool lognorm_umma_supported(const void* E, const void* P, Dims d);
size_t lognorm_umma_workspace_floats(Dims d);
// Nodes whose factored sum left the fp32 range come out of the kernel as NaN; with `fixup` a
// second kernel recomputes them exactly, without it the caller must (lattice_prep does).
// With labels, EL [B,maxU,maxT] (frames contiguous) and ebl [B,maxT] (all three non-null) and
// lognorm_umma_gathers(d), the kernel also writes EL[b,u,t] = E[b,t,labels[b,u]] (u < U_b - 1)
// and ebl[b,t] = E[b,t,blank] for the valid frames, from the chunks it streams anyway.
bool lognorm_umma_gathers(Dims d);
void launch_lognorm_umma(const void* E, const void* P, float* LN, float* rowRef, float* maxP,
                         const int* inLens, const int* labLens, Dims d, float* splitWs,
                         int* status, bool fixup, cudaStream_t stream,
                         const int* labels = nullptr, float* EL = nullptr, float* ebl = nullptr);

// ---- grads_umma.cu --------------------------------------------------------------
// Tensor-core gradients: one pass over E produces egrads and pgrads.  Usable when
// grads_umma_supported(); passes = 1..3 selects the operand precision (see grads_umma.cu).
int grads_umma_ld_w(Dims d);  // row length of W: maxU rounded up to 32
int grads_umma_ld_t(Dims d);  // row length of nref / ebl / emT: maxT rounded up to 4
bool grads_umma_supported(const void* E, const void* P, const void* egrads,
                          const void* pgrads, Dims d, int passes);
// After the reverse sweep of lattice_warp.cu: stayS/stepS/LNs (skewed) ->
//   tensorCore: W [B,maxT,ldW] rounded to TF32, emT [B,maxU,ldT], ebl [B,ldT] (row sums of
//               stay); rowRef -> nref = -rowRef*log2(e) [B,ldT].  W, emT and ebl are scaled by
//               deltas[b] (1 if deltas is null).  Operands of launch_grads_umma.
//   otherwise:  W [B,maxT,ldW] unrounded and unscaled, em [B,maxT,maxU] (passed as emT),
//               eBlank [B,maxT] (passed as ebl); nref and deltas unused.  Operands of the SIMT
//               gradient kernels.
void launch_unskew_round(const float* stayS, const float* stepS, const float* LNs,
                         const float* rowRef, const float* maxP, const float* deltas, float* W,
                         float* emT, float* nref, float* ebl, const int* inLens,
                         const int* labLens, SkewGeom g, Dims d, bool tensorCore,
                         cudaStream_t stream);
// Operands of launch_grads_umma from the outputs of the block-wide reverse sweep
// (launch_gamma_skew + launch_lattice_unskew; label axes of more than 128 positions): W is
// scaled by deltas[b] and rounded to TF32 in place, em [B,maxT,maxU] becomes emT, eBlank becomes
// ebl, rowRef becomes nref (layouts as written by launch_unskew_round with tensorCore = true).
void launch_tc_operands(float* W, const float* em, const float* eBlank, const float* rowRef,
                        const float* deltas, float* emT, float* nref, float* ebl,
                        const int* inLens, Dims d, cudaStream_t stream);
// E, P, egrads and pgrads are of d.dtype (bf16: passes = 2 only, label axes up to 128; fp32:
// label axes up to 256 positions, those above 128 as two launches over halves of the axis).
void launch_grads_umma(const void* E, const void* P, const float* maxP, const float* W,
                       const float* emT, const float* nref, const float* ebl, const float* pBlank,
                       const float* pLabel, const int* labels, const float* deltas, void* egrads,
                       void* pgrads, const int* inLens, const int* labLens, Dims d, int passes,
                       int* status, cudaStream_t stream);

// ---- lattice_warp.cu -------------------------------------------------------------
// Single-warp lattice sweeps on skewed lattices for label axes of at most 128 positions.
bool lattice_warp_supported(Dims d);
// alpha recursion from the arc terms; writes costs (and the loss sum, see launch_alpha_skew)
// and alphasS -- in LOG2 units, for launch_gamma_warp only (the nodes of the stored diagonals
// that lie outside the lattice receive large negative numbers).  status: device error word (a copy that never lands
// is recorded there and the cost becomes NaN).
// The stored alphas are REBASED: block k of 16 diagonals is relative to an offset of its own;
// deltas [B, ceil(nDiag/16)] (lattice_warp_delta_floats(d) floats) receives, at index k >= 1, by
// how much the carried state was lowered at the start of block k.
size_t lattice_warp_delta_floats(Dims d);
void launch_alpha_warp(const float2* arcs, float* costs, float* alphasS, float* deltas, SkewGeom g,
                       const int* inLens, const int* labLens, Dims d, float* lossSum,
                       unsigned* ticket, int* status, cudaStream_t stream);
// Reverse sweep: blank-arc and label-arc occupancies of every valid node to the skewed
// lattices stayS / stepS (the terminating blank counts as the blank arc of node (T-1,U-1)),
// their sums over frames to pBlank / pLabel [B,maxU].
void launch_gamma_warp(const float2* arcs, const float* alphasS, const float* deltas, SkewGeom g,
                       const int* inLens, const int* labLens, float* stayS, float* stepS,
                       float* pBlank, float* pLabel, Dims d, int* status, cudaStream_t stream);

// Viterbi sweep in one warp per utterance (label axis <= 256): same results as
// launch_viterbi_lattice.  `nodes` is scratch of viterbi_warp_nodes(d) float4, decBits of
// viterbi_warp_decbits_words(d) words.
bool viterbi_warp_supported(Dims d);
size_t viterbi_warp_nodes(Dims d);
size_t viterbi_warp_decbits_words(Dims d);  // its decision bits are packed along t+u
void launch_viterbi_warp(const float* E, const float* P, const float* LN, const float* best,
                         float4* nodes, uint32_t* decBits, int* labels, const int* inLens,
                         const int* labLens, Dims d, int* status, cudaStream_t stream);

// ---- maxplus.cu --------------------------------------------------------------
// best[b,t,u] = max over v != blank of E[b,t,v] + P[b,u,v] for t < T_b, u < U_b - 1.  With
// `guard`, the kernel does nothing unless *guard > guardCap (read on the device).
void launch_maxplus(const float* E, const float* P, float* best, const int* inLens,
                    const int* labLens, Dims d, cudaStream_t stream, const int* guard = nullptr,
                    int guardCap = 0);

// ---- maxplus_pruned.cu -------------------------------------------------------
// The same result, bit for bit, from candidate lists with an exact bound; nodes the bound does
// not settle are evaluated densely.  `scratch` holds maxplus_pruned_scratch_bytes(d) bytes.
bool maxplus_pruned_supported(Dims d);
size_t maxplus_pruned_scratch_bytes(Dims d);
void launch_maxplus_pruned(const float* E, const float* P, float* best, const int* inLens,
                           const int* labLens, Dims d, void* scratch, int* status,
                           cudaStream_t stream);

// ---- grads_simt.cu -----------------------------------------------------------
// egrads[b,t,v] = delta_b*(exp(E-rowRef)*sum_u W[t,u]*expP[u,v] - [v==blank]*eBlank[t]),
// zero for t >= T_b; then the label-arc terms are scattered in.
void launch_egrad_simt(const float* E, const float* rowRef, const float* W, int ldW,
                       const float* expP, const float* eBlank, const float* em,
                       const int* labels, const float* deltas, float* egrads,
                       const int* inLens, const int* labLens, Dims d,
                       cudaStream_t stream);
// pgrads[b,u,v] = delta_b*(expP*sum_t W[t,u]*exp(E[t,v]-rowRef[t]) - [v==blank]*pBlank[u]
//                          - [v==label_u]*pLabel[u]), zero for u >= U_b.
void launch_pgrad_simt(const float* E, const float* rowRef, const float* W, int ldW,
                       const float* expP, const float* pBlank, const float* pLabel,
                       const int* labels, const float* deltas, float* pgrads,
                       const int* inLens, const int* labLens, Dims d,
                       cudaStream_t stream);

}  // namespace tb200
