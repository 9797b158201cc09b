// Anti-diagonal wavefront kernels over the (t,u) lattice: alpha recursion, reverse
// occupancy sweep, and the Viterbi max-plus sweep with on-device backtrack.
//
// One CTA per utterance.  Thread i owns a strip of R consecutive label positions
// u in [i*R, i*R+R) and walks time: at step s it processes row t = s - i (forward
// kernels) of its strip.  The value that crosses a strip boundary travels through
// a double-buffered shared-memory slot, so one block barrier per step suffices.
// Each lattice term is kept in registers; the only global accesses per node are
// operand prefetches issued PF steps ahead (they do not depend on the recursion)
// and fire-and-forget stores.
//
// Arithmetic follows the reference's fp32 operand order so that rounding matches:
//   alpha   transducer/transducer_cpu.cpp:30-79   (transducer_cuda.cu:32-97)
//   reverse transducer/transducer_cpu.cpp:81-143  (transducer_cuda.cu:99-176)
//   viterbi transducer/transducer_cpu.cpp:145-222 (transducer_cuda.cu:178-267)
#include "kernels.h"
#include "profile.h"

namespace tb200 {
namespace {

// ---------------------------------------------------------------------------
// alpha
// ---------------------------------------------------------------------------

// The last CTA to finish adds the per-utterance costs in index order into
// *lossSum (deterministic), so a data-parallel caller can hand that scalar
// straight to its all-reduce without another kernel.
__device__ __forceinline__ void finish_cost(float* costs, int b, float cost, int B, float* lossSum,
                            unsigned* ticket) {
  costs[b] = cost;
  if (lossSum == nullptr) return;
  __threadfence();
  unsigned done = atomicAdd(ticket, 1u);
  if (done == (unsigned)(B - 1)) {
    __threadfence();
    float s = 0.0f;
    for (int k = 0; k < B; ++k) s += ((volatile float*)costs)[k];
    *lossSum = s;
    *ticket = 0u;
  }
}

// Lattice addressing.  Row-major: node (t,u) at t*ld + u (the reference's layout).
// Skewed: node (t,u) at (t+u)*ld + u, i.e. one anti-diagonal per row, so that the
// threads of a wavefront step touch consecutive addresses.
// Offsets within one utterance fit 32 bits (checked by the launchers).
template <bool SKEW>
__device__ __forceinline__ int node(int t, int u, int ld) {
  return SKEW ? (t + u) * ld + u : t * ld + u;
}

// log(exp(a)+exp(b)) for the alpha recursion.  Same -inf handling and operation order
// as the reference's logSumExp; the correction term log1p(exp(-|a-b|)) <= ln 2 is
// evaluated with the hardware ex2/lg2 units (absolute error ~2e-7, far below one ulp of
// the alphas it is added to once they exceed a few units in magnitude).
__device__ __forceinline__ float lse2_fast(float a, float b) {
  if (a == neg_inf()) return b;
  if (b == neg_inf()) return a;
  return fmaxf(a, b) + __logf(1.0f + __expf(-fabsf(a - b)));
}

// SKEW=false: LN/alphas row-major [B,maxT,maxU], emission terms gathered from E.
// SKEW=true : LN/alphas/ELs skewed [B,nDiag,ld]; ELs[t,u] = E[t,label_u] and
//             ebl[b,t] = E[t,blank] were gathered by lattice_prep_kernel, so the
//             sweep itself issues only coalesced loads and stores.
template <int R, int PF, int MAXNT, bool SKEW>
__global__ void __launch_bounds__(MAXNT) alpha_kernel(
    const float* __restrict__ E, const float* __restrict__ P, float* __restrict__ costs,
    float* __restrict__ alphas, const float* __restrict__ LN,
    const float* __restrict__ ELs, const float* __restrict__ ebl, int ld, i64 latStride,
    const int* __restrict__ labels, const int* __restrict__ inLens,
    const int* __restrict__ labLens, int B, int maxT, int maxU, int V, int blank,
    float* lossSum, unsigned* ticket) {
  __shared__ float xch[2][MAXNT + 1];
  const int b = blockIdx.x, i = threadIdx.x;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  if (T <= 0 || U <= 0) {
    if (i == 0) finish_cost(costs, b, pos_inf(), B, lossSum, ticket);
    return;
  }
  const float* e = E + (i64)b * maxT * V;
  const float* p = P + (i64)b * maxU * V;
  const float* ln = LN + (i64)b * latStride;
  const float* el = SKEW ? ELs + (i64)b * latStride : nullptr;
  const float* eb = SKEW ? ebl + (i64)b * maxT : nullptr;
  float* al = alphas + (i64)b * latStride;
  const int* lab_g = labels + (i64)b * (maxU - 1);

  const int nStrips = (U + R - 1) / R;
  const int S = T + nStrips - 1;
  const bool mine = i < nStrips;

  int lab[R];
  float pbl[R], plab[R], stay[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int u = i * R + r;
    lab[r] = blank;
    pbl[r] = 0.0f;
    plab[r] = 0.0f;
    stay[r] = neg_inf();
    if (u < U) {
      pbl[r] = p[(i64)u * V + blank];
      if (u < U - 1) {
        lab[r] = lab_g[u];
        plab[r] = p[(i64)u * V + lab[r]];
      }
    }
  }

  float cost = 0.0f;
  bool owner = false;
  float q_ln[PF][R], q_el[PF][R], q_eb[PF];
  // Operand prefetch for step s into ring slot k.  The loads are UNCONDITIONAL, with
  // the node clamped into the lattice: predicated loads were scheduled next to their
  // use by the compiler, which put the whole memory latency on the recursion.
  auto issue = [&](int s, int k) {
    const int t = min(max(s - i, 0), T - 1);
    q_eb[k] = SKEW ? eb[t] : e[(i64)t * V + blank];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int u = min(i * R + r, U - 1);
      q_ln[k][r] = ln[node<SKEW>(t, u, ld)];
      q_el[k][r] = SKEW ? el[node<SKEW>(t, u, ld)] : e[(i64)t * V + lab[r]];
    }
  };
#pragma unroll
  for (int k = 0; k < PF; ++k) issue(k, k);

  for (int s0 = 0; s0 < S; s0 += PF) {
#pragma unroll
    for (int k = 0; k < PF; ++k) {
      // no early exit: a `break` here keeps the compiler from unrolling, which sends the
      // prefetch ring to local memory; steps past the end are simply empty
      const int s = s0 + k;
      const int t = s - i;
      if (mine && t >= 0 && t < T) {
        float step_in = (i == 0) ? neg_inf() : xch[(s + 1) & 1][i];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int u = i * R + r;
          if (u < U) {
            const float a = (s == 0 && u == 0) ? 0.0f : (SKEW ? lse2_fast(step_in, stay[r]) : lse2(step_in, stay[r]));
            al[node<SKEW>(t, u, ld)] = a;
            const float lnv = q_ln[k][r];
            stay[r] = ((a + q_eb[k]) + pbl[r]) - lnv;
            step_in = ((a + q_el[k][r]) + plab[r]) - lnv;
            if (t == T - 1 && u == U - 1) {
              cost = -stay[r];
              owner = true;
            }
          }
        }
        xch[s & 1][i + 1] = step_in;
      }
      issue(s + PF, k);
      __syncthreads();
    }
  }
  if (owner) finish_cost(costs, b, cost, B, lossSum, ticket);
}

// ---------------------------------------------------------------------------
// reverse occupancy sweep
// ---------------------------------------------------------------------------

// ABI=true : the transducer.h contract (row-major lattices, read-modify-write of the
//            zero-filled egrads/pgrads, occupancies to lngrads).
// ABI=false: fused path.  With SKEW the lattices (alphas, LN, ELs in; W, em out) are
//            skewed with row length ld; without it they are row-major (W with ldW).
template <int R, int PF, int MAXNT, bool ABI, bool SKEW>
__global__ void __launch_bounds__(MAXNT) gamma_kernel(
    const float* __restrict__ E, const float* __restrict__ P,
    const float* __restrict__ alphas, const float* __restrict__ LN,
    const float* __restrict__ ELs, const float* __restrict__ ebl, int ld, i64 latStride,
    const float* __restrict__ rowRef, const float* __restrict__ maxP,
    const int* __restrict__ labels, const int* __restrict__ inLens,
    const int* __restrict__ labLens,
    float* egrads, float* pgrads, float* lngrads,           // ABI outputs
    float* __restrict__ W, int ldW, float* __restrict__ em, // fused outputs
    float* __restrict__ eBlank, float* __restrict__ pBlank, float* __restrict__ pLabel,
    int maxT, int maxU, int V, int blank) {
  extern __shared__ float sEB[];  // [T] running sum of blank-arc occupancies per frame
  __shared__ float xg[2][MAXNT + 1];
  __shared__ float xa[2][MAXNT + 1];
  const int b = blockIdx.x, i = threadIdx.x, NT = blockDim.x;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  const bool empty = (T <= 0 || U <= 0);
  if (!ABI) {
    // padded tails of the per-frame / per-position outputs are defined (zero)
    for (int t = (empty ? 0 : T) + i; t < maxT; t += NT) eBlank[(i64)b * maxT + t] = 0.0f;
    for (int u = (empty ? 0 : U) + i; u < maxU; u += NT) {
      pBlank[(i64)b * maxU + u] = 0.0f;
      pLabel[(i64)b * maxU + u] = 0.0f;
    }
  }
  if (empty) return;

  const float* e = E + (i64)b * maxT * V;
  const float* p = P + (i64)b * maxU * V;
  const float* al = alphas + (i64)b * latStride;
  const float* ln = LN + (i64)b * latStride;
  const float* el = SKEW ? ELs + (i64)b * latStride : nullptr;
  const float* eb = SKEW ? ebl + (i64)b * maxT : nullptr;
  const int* lab_g = labels + (i64)b * (maxU - 1);

  for (int t = i; t < T; t += NT) sEB[t] = (t == T - 1) ? 1.0f : 0.0f;

  const int nStrips = (U + R - 1) / R;
  const int S = T + nStrips - 1;
  const bool mine = i < nStrips;
  const int ir = nStrips - 1 - i;  // strips start from the high-u end

  int lab[R];
  float pbl[R], plab[R], mp[R], g_dn[R], a_dn[R], accB[R], accL[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int u = i * R + r;
    lab[r] = blank;
    pbl[r] = plab[r] = mp[r] = 0.0f;
    g_dn[r] = a_dn[r] = 0.0f;
    accB[r] = (u == U - 1) ? 1.0f : 0.0f;
    accL[r] = 0.0f;
    if (u < U) {
      pbl[r] = p[(i64)u * V + blank];
      if (!ABI) mp[r] = maxP[(i64)b * maxU + u];
      if (u < U - 1) {
        lab[r] = lab_g[u];
        plab[r] = p[(i64)u * V + lab[r]];
      }
    }
  }

  float q_a[PF][R], q_ln[PF][R], q_el[PF][R], q_eb[PF], q_ref[PF];
  auto issue = [&](int s, int k) {  // unconditional, clamped: see alpha_kernel
    const int t = min(max(T - 1 - (s - ir), 0), T - 1);
    q_eb[k] = SKEW ? eb[t] : e[(i64)t * V + blank];
    if (!ABI) q_ref[k] = rowRef[(i64)b * maxT + t];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int u = min(i * R + r, U - 1);
      q_a[k][r] = al[node<SKEW>(t, u, ld)];
      q_ln[k][r] = ln[node<SKEW>(t, u, ld)];
      q_el[k][r] = SKEW ? el[node<SKEW>(t, u, ld)] : e[(i64)t * V + lab[r]];
    }
  };
#pragma unroll
  for (int k = 0; k < PF; ++k) issue(k, k);
  __syncthreads();  // sEB initialised

  for (int s0 = 0; s0 < S; s0 += PF) {
#pragma unroll
    for (int k = 0; k < PF; ++k) {
      const int s = s0 + k;
      const int t = T - 1 - (s - ir);
      if (mine && t >= 0 && t < T) {
        float g_rt = 0.0f, a_rt = 0.0f;
        if (i < nStrips - 1) {
          g_rt = xg[(s + 1) & 1][i + 1];
          a_rt = xa[(s + 1) & 1][i + 1];
        }
        float eb_run = sEB[t];
#pragma unroll
        for (int r = R - 1; r >= 0; --r) {
          const int u = i * R + r;
          if (u < U) {
            const float a = q_a[k][r], lnv = q_ln[k][r];
            float stay = 0.0f, step = 0.0f;
            if (t < T - 1) {
              stay = g_dn[r] * expf((((a + q_eb[k]) + pbl[r]) - lnv) - a_dn[r]);
              eb_run += stay;
              accB[r] += stay;
            }
            if (u < U - 1) {
              step = g_rt * expf((((a + q_el[k][r]) + plab[r]) - lnv) - a_rt);
              accL[r] += step;
            }
            float g;
            if (t == T - 1) g = (u == U - 1) ? 1.0f : step;
            else g = (u == U - 1) ? stay : stay + step;
            if (ABI) {
              lngrads[(i64)b * maxT * maxU + (i64)t * maxU + u] = g;
              if (u < U - 1) {
                float* dst = egrads + (i64)b * maxT * V + (i64)t * V + lab[r];
                *dst -= step;
              }
            } else {
              // exponent clamp keeps W finite where the factored sum had underflowed
              const float sh = fminf((q_ref[k] + mp[r]) - lnv, 80.0f);
              if (SKEW) {
                W[(i64)b * latStride + node<true>(t, u, ld)] = g * expf(sh);
                em[(i64)b * latStride + node<true>(t, u, ld)] = step;
              } else {
                W[(i64)b * maxT * ldW + (i64)t * ldW + u] = g * expf(sh);
                em[(i64)b * maxT * maxU + (i64)t * maxU + u] = step;
              }
            }
            g_dn[r] = g;
            a_dn[r] = a;
            g_rt = g;
            a_rt = a;
          }
        }
        sEB[t] = eb_run;
        xg[s & 1][i] = g_rt;
        xa[s & 1][i] = a_rt;
      }
      issue(s + PF, k);
      __syncthreads();
    }
  }

  if (ABI) {
    float* eg = egrads + (i64)b * maxT * V;
    float* pg = pgrads + (i64)b * maxU * V;
    for (int t = i; t < T; t += NT) eg[(i64)t * V + blank] -= sEB[t];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int u = i * R + r;
      if (mine && u < U) {
        pg[(i64)u * V + blank] -= accB[r];
        if (u < U - 1) pg[(i64)u * V + lab[r]] -= accL[r];
      }
    }
  } else {
    for (int t = i; t < T; t += NT) eBlank[(i64)b * maxT + t] = sEB[t];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int u = i * R + r;
      if (mine && u < U) {
        pBlank[(i64)b * maxU + u] = accB[r];
        pLabel[(i64)b * maxU + u] = (u < U - 1) ? accL[r] : 0.0f;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Viterbi: max-plus wavefront, bit-packed decisions, bounded backtrack, argmax
// ---------------------------------------------------------------------------

// Decision bits: word[(b*maxU + u)*wordsT + t/32] bit (t%32) is 1 when node (t,u)
// was entered by the label arc from (t,u-1), 0 when by the blank arc from (t-1,u).
template <int R, int PF, int MAXNT>
__global__ void __launch_bounds__(MAXNT) viterbi_kernel(
    const float* __restrict__ E, const float* __restrict__ P,
    const float* __restrict__ LN, const float* __restrict__ best,
    uint32_t* __restrict__ decBits, int* __restrict__ labelsOut,
    const int* __restrict__ inLens, const int* __restrict__ labLens,
    int maxT, int maxU, int V, int blank) {
  extern __shared__ int sFrame[];  // [U] frame at which label u-1 was emitted
  __shared__ float xch[2][MAXNT + 1];
  const int b = blockIdx.x, i = threadIdx.x, NT = blockDim.x;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  if (T <= 0 || U <= 0) return;
  const float* e = E + (i64)b * maxT * V;
  const float* p = P + (i64)b * maxU * V;
  const float* ln = LN + (i64)b * maxT * maxU;
  const float* bs = best + (i64)b * maxT * maxU;
  const int wordsT = (maxT + 31) / 32;
  uint32_t* dec = decBits + (i64)b * maxU * wordsT;

  const int nStrips = (U + R - 1) / R;
  const int S = T + nStrips - 1;
  const bool mine = i < nStrips;

  float pbl[R], stay[R];
  uint32_t bits[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int u = i * R + r;
    pbl[r] = (u < U) ? p[(i64)u * V + blank] : 0.0f;
    stay[r] = neg_inf();
    bits[r] = 0u;
  }
  for (int u = i; u < U; u += NT) sFrame[u] = -1;

  float q_ln[PF][R], q_bs[PF][R], q_eb[PF];
  auto issue = [&](int s, int k) {  // unconditional, clamped: see alpha_kernel
    const int t = min(max(s - i, 0), T - 1);
    q_eb[k] = e[(i64)t * V + blank];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int u = min(i * R + r, U - 1);
      q_ln[k][r] = ln[(i64)t * maxU + u];
      q_bs[k][r] = bs[(i64)t * maxU + min(u, max(U - 2, 0))];
    }
  };
#pragma unroll
  for (int k = 0; k < PF; ++k) issue(k, k);

  for (int s0 = 0; s0 < S; s0 += PF) {
#pragma unroll
    for (int k = 0; k < PF; ++k) {
      const int s = s0 + k;
      const int t = s - i;
      if (mine && t >= 0 && t < T) {
        float step_in = (i == 0) ? neg_inf() : xch[(s + 1) & 1][i];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int u = i * R + r;
          if (u < U) {
            float sc;
            uint32_t d;
            if (u == 0) { sc = (t == 0) ? 0.0f : stay[r]; d = 0u; }
            else if (t == 0) { sc = step_in; d = 1u; }
            else { d = (step_in > stay[r]) ? 1u : 0u; sc = d ? step_in : stay[r]; }
            bits[r] |= d << (t & 31);
            if ((t & 31) == 31 || t == T - 1) {
              dec[(i64)u * wordsT + (t >> 5)] = bits[r];
              bits[r] = 0u;
            }
            const float lnv = q_ln[k][r];
            stay[r] = ((sc + q_eb[k]) + pbl[r]) - lnv;
            step_in = (sc + q_bs[k][r]) - lnv;
          }
        }
        xch[s & 1][i + 1] = step_in;
      }
      issue(s + PF, k);
      __syncthreads();
    }
  }
  __syncthreads();

  // Backtrack from (T-1,U-1).  Each iteration consumes either one label or one
  // 32-frame word of blanks, so it ends within U + T/32 + 1 iterations; the
  // explicit cap only guards against corrupted scratch.
  if (i == 0) {
    int t = T - 1, u = U - 1;
    int guard = U + wordsT + 2;
    while (u > 0 && t >= 0 && guard-- > 0) {
      const uint32_t keep = 0xffffffffu >> (31 - (t & 31));
      const uint32_t w = ((volatile uint32_t*)dec)[(i64)u * wordsT + (t >> 5)] & keep;
      if (w == 0u) { t = (t & ~31) - 1; continue; }
      t = (t & ~31) + (31 - __clz(w));
      sFrame[u] = t;
      --u;
    }
  }
  __syncthreads();

  // Label on each emitting arc of the path: lowest-index argmax over v != blank
  // of E[t,v] + P[u-1,v] (strict '>' in index order, as the reference's getMax).
  int* out = labelsOut + (i64)b * (maxU - 1);
  const int lane = i & 31, warp = i >> 5, nWarps = NT >> 5;
  for (int u = 1 + warp; u < U; u += nWarps) {
    const int t = sFrame[u];
    if (t < 0) continue;
    const float* er = e + (i64)t * V;
    const float* pr = p + (i64)(u - 1) * V;
    float m = neg_inf();
    int arg = 0x7fffffff;
    for (int v = lane; v < V; v += 32) {
      if (v == blank) continue;
      const float x = er[v] + pr[v];
      if (x > m) { m = x; arg = v; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const int a2 = __shfl_xor_sync(0xffffffffu, arg, o);
      if (m2 > m || (m2 == m && a2 < arg)) { m = m2; arg = a2; }
    }
    if (lane == 0) out[u - 1] = (arg == 0x7fffffff) ? 0 : arg;
  }
}

struct StripCfg {
  int R, threads;
};

StripCfg pick_strips(int maxU) {
  if (maxU > kMaxLatticeU)
    throw std::invalid_argument("label axis longer than 8192 is not supported");
  int R = 1;
  while (div_up(maxU, R) > 1024) R *= 2;
  int threads = div_up(div_up(maxU, R), 32) * 32;
  if (threads < 32) threads = 32;
  return {R, threads};
}

void check_lattice_fits_int(Dims d) {
  if ((i64)(d.maxT + d.maxU) * round_up64(d.maxU > 0 ? d.maxU : 1, 32) >= 2147483647LL)
    throw std::invalid_argument("lattice of one utterance exceeds 2^31 nodes");
}

}  // namespace

#define TB200_DISPATCH_STRIPS(cfg, CALL)                  \
  do {                                                    \
    if ((cfg).R == 1 && (cfg).threads <= 256) { CALL(1, 8, 256); } \
    else if ((cfg).R == 1) { CALL(1, 4, 1024); }          \
    else if ((cfg).R == 2) { CALL(2, 2, 1024); }          \
    else if ((cfg).R == 4) { CALL(4, 1, 1024); }          \
    else { CALL(8, 1, 1024); }                            \
  } while (0)

void launch_alpha(const float* E, const float* P, float* costs, float* alphas,
                  const float* LN, const int* labels, const int* inLens,
                  const int* labLens, Dims d, float* lossSum, unsigned* ticket,
                  cudaStream_t stream) {
  if (d.B <= 0) return;
  check_lattice_fits_int(d);
  const StripCfg cfg = pick_strips(d.maxU);
  ScopedKernel sk("alpha_wavefront_abi", stream);
#define CALL(R, PF, NT)                                                              \
  alpha_kernel<R, PF, NT, false><<<d.B, cfg.threads, 0, stream>>>(                   \
      E, P, costs, alphas, LN, nullptr, nullptr, d.maxU, (i64)d.maxT * d.maxU, labels, \
      inLens, labLens, d.B, d.maxT, d.maxU, d.V, d.blank, lossSum, ticket)
  TB200_DISPATCH_STRIPS(cfg, CALL);
#undef CALL
  TB200_CHECK_LAUNCH();
}

SkewGeom skew_geom(Dims d) {
  SkewGeom g;
  g.ld = (int)round_up64(d.maxU > 0 ? d.maxU : 1, 32);
  g.nDiag = d.maxT + d.maxU;  // one spare row
  g.stride = (i64)g.ld * g.nDiag;
  return g;
}

void launch_alpha_skew(const float* P, float* costs, float* alphasS, const float* LNs,
                       const float* ELs, const float* ebl, SkewGeom g, const int* labels,
                       const int* inLens, const int* labLens, Dims d, float* lossSum,
                       unsigned* ticket, cudaStream_t stream) {
  if (d.B <= 0) return;
  check_lattice_fits_int(d);
  const StripCfg cfg = pick_strips(d.maxU);
  ScopedKernel sk("alpha_wavefront", stream);
#define CALL(R, PF, NT)                                                              \
  alpha_kernel<R, PF, NT, true><<<d.B, cfg.threads, 0, stream>>>(                    \
      nullptr, P, costs, alphasS, LNs, ELs, ebl, g.ld, g.stride, labels, inLens,    \
      labLens, d.B, d.maxT, d.maxU, d.V, d.blank, lossSum, ticket)
  TB200_DISPATCH_STRIPS(cfg, CALL);
#undef CALL
  TB200_CHECK_LAUNCH();
}

namespace {
constexpr size_t kMaxDynSmem = 200 * 1024;

template <typename K>
void allow_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024)
    TB200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)bytes));
}
}  // namespace

void launch_gamma_abi(const float* E, const float* P, float* egrads, float* pgrads,
                      float* lngrads, const float* alphas, const float* LN,
                      const int* labels, const int* inLens, const int* labLens,
                      Dims d, cudaStream_t stream) {
  if (d.B <= 0) return;
  check_lattice_fits_int(d);
  const StripCfg cfg = pick_strips(d.maxU);
  const size_t smem = sizeof(float) * (size_t)(d.maxT > 0 ? d.maxT : 1);
  if (smem > kMaxDynSmem) throw std::invalid_argument("input length above 51200 frames is not supported");
  ScopedKernel sk("gamma_wavefront_abi", stream);
#define CALL(R, PF, NT)                                                               \
  allow_smem(gamma_kernel<R, PF, NT, true, false>, smem);                             \
  gamma_kernel<R, PF, NT, true, false><<<d.B, cfg.threads, smem, stream>>>(           \
      E, P, alphas, LN, nullptr, nullptr, d.maxU, (i64)d.maxT * d.maxU, nullptr,      \
      nullptr, labels, inLens, labLens, egrads, pgrads, lngrads, nullptr, 0, nullptr, \
      nullptr, nullptr, nullptr, d.maxT, d.maxU, d.V, d.blank)
  TB200_DISPATCH_STRIPS(cfg, CALL);
#undef CALL
  TB200_CHECK_LAUNCH();
}

void launch_gamma_skew(const float* P, const float* alphasS, const float* LNs,
                       const float* ELs, const float* ebl, SkewGeom g, const float* rowRef,
                       const float* maxP, const int* labels, const int* inLens,
                       const int* labLens, float* Ws, float* EMs, float* eBlank,
                       float* pBlank, float* pLabel, Dims d, cudaStream_t stream) {
  if (d.B <= 0) return;
  check_lattice_fits_int(d);
  const StripCfg cfg = pick_strips(d.maxU);
  const size_t smem = sizeof(float) * (size_t)(d.maxT > 0 ? d.maxT : 1);
  if (smem > kMaxDynSmem) throw std::invalid_argument("input length above 51200 frames is not supported");
  ScopedKernel sk("gamma_wavefront", stream);
#define CALL(R, PF, NT)                                                               \
  allow_smem(gamma_kernel<R, PF, NT, false, true>, smem);                             \
  gamma_kernel<R, PF, NT, false, true><<<d.B, cfg.threads, smem, stream>>>(           \
      nullptr, P, alphasS, LNs, ELs, ebl, g.ld, g.stride, rowRef, maxP, labels,       \
      inLens, labLens, nullptr, nullptr, nullptr, Ws, g.ld, EMs, eBlank, pBlank,      \
      pLabel, d.maxT, d.maxU, d.V, d.blank)
  TB200_DISPATCH_STRIPS(cfg, CALL);
#undef CALL
  TB200_CHECK_LAUNCH();
}

// ---------------------------------------------------------------------------
// layout changes between row-major and skewed lattices
// ---------------------------------------------------------------------------
namespace {

// One CTA per 32x32 (t,u) tile.  Reads LN row-major and gathers E[t,label_u]; writes
// both skewed.  Column tile 0 also writes ebl[t] = E[t,blank].  With `arcs` it also writes,
// skewed and in log2 units, the log-probabilities of the two arcs leaving every valid node:
//   arcs[t,u].x = (E[t,blank]   + P[u,blank]   - LN[t,u]) * log2(e)
//   arcs[t,u].y = (E[t,label_u] + P[u,label_u] - LN[t,u]) * log2(e),  u < U-1
// (the caller pre-fills the array with a large negative number: nodes outside the lattice and
// the label arc of the last position keep it).
// With ELrow ([B,maxU,maxT], frames contiguous, written by the tensor-core log-normaliser
// together with ebl) the label and blank emissions are read from there, coalesced, instead of
// being gathered from E one DRAM sector per node.
template <typename TIn>
__global__ void __launch_bounds__(256) lattice_prep_kernel(
    const TIn* __restrict__ E, const TIn* __restrict__ P, const float* __restrict__ LN,
    float* __restrict__ LNs, float* __restrict__ ELs, float* __restrict__ ebl,
    float2* __restrict__ arcs, const float* __restrict__ ELrow, const int* __restrict__ labels,
    const int* __restrict__ inLens, const int* __restrict__ labLens, int maxT, int maxU, int V,
    int blank, int ld, i64 latStride) {
  __shared__ float tLn[32][33], tEl[32][33], tEb[32];
  const int b = blockIdx.z, t0 = blockIdx.y * 32, u0 = blockIdx.x * 32;
  const int T = min(inLens[b], maxT), U = min(labLens[b] + 1, maxU);
  if (t0 >= T || u0 >= U) return;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const TIn* e = E + (i64)b * maxT * V;
  const float* ln = LN + (i64)b * maxT * maxU;
  const float* elr = ELrow ? ELrow + (i64)b * maxU * maxT : nullptr;
  const int* lab = labels + (i64)b * (maxU - 1);
  const int u = u0 + lane;
  const int myLab = (u < U - 1) ? lab[u] : blank;
  float pbl = 0.0f, plab = 0.0f;
  if (arcs != nullptr && u < U) {
    const TIn* p = P + (i64)b * maxU * V;
    pbl = to_f32(p[(i64)u * V + blank]);
    plab = to_f32(p[(i64)u * V + myLab]);
  }
  // all loads first (unconditional, clamped into the lattice): the gathers of the four rows
  // are in flight together
  float va[4], vc[4];
  {
    const int uc = min(u, U - 1);
    const int labc = (uc < U - 1) ? lab[uc] : blank;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int tc = min(t0 + w * 4 + k, T - 1);
      va[k] = ln[(i64)tc * maxU + uc];
      vc[k] = elr ? 0.0f : to_f32(e[(i64)tc * V + labc]);
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int tt = w * 4 + k, t = t0 + tt;
    float a = 0.0f, c = 0.0f;
    if (t < T && u < U) {
      a = va[k];
      c = vc[k];
    }
    // marked by the tensor-core log-normaliser (its factored sum left the fp32 range):
    // exact logsumexp by the whole warp
    unsigned todo = __ballot_sync(0xffffffffu, a != a);
    while (todo) {
      const int src = __ffs(todo) - 1;
      todo &= todo - 1;
      const TIn* er = e + (i64)t * V;
      const TIn* pr = P + ((i64)b * maxU + u0 + src) * V;
      float m = neg_inf();
      for (int v = lane; v < V; v += 32) m = fmaxf(m, to_f32(er[v]) + to_f32(pr[v]));
      m = warp_max(m);
      float s = 0.0f;
      if (m != neg_inf() && m != pos_inf())
        for (int v = lane; v < V; v += 32) s += expf((to_f32(er[v]) + to_f32(pr[v])) - m);
      s = warp_sum(s);
      if (lane == src) a = logf(s) + m;
    }
    tLn[tt][lane] = a;
    if (!elr) tEl[tt][lane] = c;
  }
  if (elr) {  // transposed tile load: lane <-> frame, row <-> label position
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int uu = u0 + w * 4 + k, tl = t0 + lane;
      const float v = elr[(i64)min(uu, max(U - 2, 0)) * maxT + min(tl, T - 1)];
      tEl[lane][w * 4 + k] = (uu < U - 1 && tl < T) ? v : 0.0f;
    }
  }
  if (threadIdx.x < 32) {
    float v = 0.0f;
    if (t0 + lane < T) v = elr ? ebl[(i64)b * maxT + t0 + lane] : to_f32(e[(i64)(t0 + lane) * V + blank]);
    tEb[lane] = v;
    if (!elr && u0 == 0 && t0 + lane < T) ebl[(i64)b * maxT + t0 + lane] = v;
  }
  __syncthreads();
  // diagonal s = t + u of this tile: s - (t0+u0) in [0, 62]; lane <-> u
  for (int ds = w; ds < 63; ds += 8) {
    const int tt = ds - lane;
    if (tt >= 0 && tt < 32 && t0 + tt < T && u < U) {
      const i64 o = (i64)b * latStride + (i64)(t0 + u0 + ds) * ld + u;
      const float lnv = tLn[tt][lane], elv = tEl[tt][lane];
      LNs[o] = lnv;
      if (ELs != nullptr) ELs[o] = elv;
      if (arcs != nullptr) {
        float2 f;
        f.x = ((tEb[tt] + pbl) - lnv) * 1.4426950408889634f;
        f.y = (u < U - 1) ? ((elv + plab) - lnv) * 1.4426950408889634f : __uint_as_float(kNoArcBits);
        arcs[o] = f;
      }
    }
  }
}

// Skewed -> row-major for two arrays at once (W with row length ldW, em with maxU);
// everything outside the valid lattice of W is written as zero so the matrix can be
// used as a GEMM operand without a separate fill.
__global__ void __launch_bounds__(256) lattice_unskew_kernel(
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
    if (u < ldW) W[((i64)b * maxT + t) * ldW + u] = live ? tW[tt][lane] : 0.0f;
    if (u < maxU) em[((i64)b * maxT + t) * maxU + u] = live ? tE[tt][lane] : 0.0f;
  }
}

}  // namespace

void launch_lattice_prep(const void* E, const void* P, const float* LN, float* LNs,
                         float* ELs, float* ebl, float2* arcs, const int* labels,
                         const int* inLens, const int* labLens, SkewGeom g, Dims d,
                         cudaStream_t stream, const float* ELrow) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 0) return;
  if (arcs != nullptr)
    TB200_CUDA_CHECK(cudaMemsetAsync(arcs, kNoArcByte, sizeof(float2) * (size_t)d.B * g.stride, stream));
  dim3 grid(div_up(d.maxU, 32), div_up(d.maxT, 32), d.B);
  ScopedKernel sk("lattice_prep", stream);
  if (d.dtype == kDtypeBf16)
    lattice_prep_kernel<bf16><<<grid, 256, 0, stream>>>(
        static_cast<const bf16*>(E), static_cast<const bf16*>(P), LN, LNs, ELs, ebl, arcs, ELrow,
        labels, inLens, labLens, d.maxT, d.maxU, d.V, d.blank, g.ld, g.stride);
  else
    lattice_prep_kernel<float><<<grid, 256, 0, stream>>>(
        static_cast<const float*>(E), static_cast<const float*>(P), LN, LNs, ELs, ebl, arcs, ELrow,
        labels, inLens, labLens, d.maxT, d.maxU, d.V, d.blank, g.ld, g.stride);
  TB200_CHECK_LAUNCH();
}

void launch_lattice_unskew(const float* Ws, const float* EMs, float* W, int ldW, float* em,
                           const int* inLens, const int* labLens, SkewGeom g, Dims d,
                           cudaStream_t stream) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 0) return;
  dim3 grid(div_up(ldW, 32), div_up(d.maxT, 32), d.B);
  ScopedKernel sk("lattice_unskew", stream);
  lattice_unskew_kernel<<<grid, 256, 0, stream>>>(Ws, EMs, W, em, inLens, labLens, d.maxT,
                                                  d.maxU, g.ld, g.stride, ldW);
  TB200_CHECK_LAUNCH();
}

size_t viterbi_decbits_words(Dims d) {
  return (size_t)d.B * (size_t)d.maxU * (size_t)((d.maxT + 31) / 32);
}

void launch_viterbi_lattice(const float* E, const float* P, const float* LN,
                            const float* best, uint32_t* decBits, int* labels,
                            const int* inLens, const int* labLens, Dims d,
                            cudaStream_t stream) {
  if (d.B <= 0 || d.maxT <= 0) return;
  const StripCfg cfg = pick_strips(d.maxU);
  const size_t smem = sizeof(int) * (size_t)d.maxU;
  ScopedKernel sk("viterbi_wavefront", stream);
#define CALL(R, PF, NT)                                                               \
  viterbi_kernel<R, PF, NT><<<d.B, cfg.threads, smem, stream>>>(                      \
      E, P, LN, best, decBits, labels, inLens, labLens, d.maxT, d.maxU, d.V, d.blank)
  TB200_DISPATCH_STRIPS(cfg, CALL);
#undef CALL
  TB200_CHECK_LAUNCH();
}

}  // namespace tb200
