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
struct Dims {
  int B, maxT, maxU, V, blank;
};

constexpr int kMaxLatticeU = 8192;  // widest label axis the wavefront kernels take

// ---- lattice.cu ------------------------------------------------------------
void launch_alpha(const float* E, const float* P, float* costs, float* alphas,
                  const float* LN, const int* labels, const int* inLens,
                  const int* labLens, Dims d, float* lossSum, unsigned* ticket,
                  cudaStream_t stream);

// Reverse sweep.  abi=true reproduces transducer.h's backward contract: the three
// outputs must already be zero-filled; lngrads receives the node occupancies and
// the sparse blank/label terms are subtracted in place from egrads/pgrads.
void launch_gamma_abi(const float* E, const float* P, float* egrads, float* pgrads,
                      float* lngrads, const float* alphas, const float* LN,
                      const int* labels, const int* inLens, const int* labLens,
                      Dims d, cudaStream_t stream);

// Fused-path reverse sweep: writes W[t,u] = occupancy * exp(rowRef[t] + maxP[u] - LN[t,u])
// (row stride ldW >= maxU, rows/cols outside the valid lattice are NOT touched: the
// caller zero-fills W), the label-arc occupancies `em` [B,maxT,maxU], and the summed
// sparse terms eBlank [B,maxT], pBlank [B,maxU], pLabel [B,maxU].
void launch_gamma_fused(const float* E, const float* P, const float* alphas,
                        const float* LN, const float* rowRef, const float* maxP,
                        const int* labels, const int* inLens, const int* labLens,
                        float* W, int ldW, float* em, float* eBlank, float* pBlank,
                        float* pLabel, Dims d, cudaStream_t stream);

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
// Tensor-core log-normalisers (one pass over E).  Usable when lognorm_umma_supported();
// splitWs holds lognorm_umma_workspace_floats(d) floats, status two ints (zeroed by the
// caller): [0] first device-side error code (0 = none), [1] nodes recomputed exactly.
bool lognorm_umma_supported(const float* E, const float* P, Dims d);
size_t lognorm_umma_workspace_floats(Dims d);
void launch_lognorm_umma(const float* E, const float* P, float* LN, float* rowRef, float* maxP,
                         const int* inLens, const int* labLens, Dims d, float* splitWs,
                         int* status, cudaStream_t stream);

// ---- maxplus.cu --------------------------------------------------------------
void launch_maxplus(const float* E, const float* P, float* best, const int* inLens,
                    const int* labLens, Dims d, cudaStream_t stream);

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
