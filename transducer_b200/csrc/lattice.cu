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
__device__ void finish_cost(float* costs, int b, float cost, int B, float* lossSum,
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

template <int R, int PF, int MAXNT>
__global__ void __launch_bounds__(MAXNT) alpha_kernel(
    const float* __restrict__ E, const float* __restrict__ P, float* __restrict__ costs,
    float* __restrict__ alphas, const float* __restrict__ LN,
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
  const float* ln = LN + (i64)b * maxT * maxU;
  float* al = alphas + (i64)b * maxT * maxU;
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

  float q_ln[PF][R], q_el[PF][R], q_eb[PF];
  auto issue = [&](int s, int k) {
    const int t = s - i;
    if (mine && t >= 0 && t < T) {
      q_eb[k] = e[(i64)t * V + blank];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int u = i * R + r;
        if (u < U) {
          q_ln[k][r] = ln[(i64)t * maxU + u];
          q_el[k][r] = e[(i64)t * V + lab[r]];
        }
      }
    }
  };
#pragma unroll
  for (int k = 0; k < PF; ++k) issue(k, k);

  for (int s0 = 0; s0 < S; s0 += PF) {
#pragma unroll
    for (int k = 0; k < PF; ++k) {
      const int s = s0 + k;
      if (s >= S) break;  // uniform across the block
      const int t = s - i;
      if (mine && t >= 0 && t < T) {
        float step_in = (i == 0) ? neg_inf() : xch[(s + 1) & 1][i];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int u = i * R + r;
          if (u < U) {
            const float a = (s == 0 && u == 0) ? 0.0f : lse2(step_in, stay[r]);
            al[(i64)t * maxU + u] = a;
            const float lnv = q_ln[k][r];
            stay[r] = ((a + q_eb[k]) + pbl[r]) - lnv;
            step_in = ((a + q_el[k][r]) + plab[r]) - lnv;
            if (t == T - 1 && u == U - 1)
              finish_cost(costs, b, -stay[r], B, lossSum, ticket);
          }
        }
        xch[s & 1][i + 1] = step_in;
      }
      issue(s + PF, k);
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------
// reverse occupancy sweep
// ---------------------------------------------------------------------------

template <int R, int PF, int MAXNT, bool ABI>
__global__ void __launch_bounds__(MAXNT) gamma_kernel(
    const float* __restrict__ E, const float* __restrict__ P,
    const float* __restrict__ alphas, const float* __restrict__ LN,
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
  const float* al = alphas + (i64)b * maxT * maxU;
  const float* ln = LN + (i64)b * maxT * maxU;
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
  auto issue = [&](int s, int k) {
    const int t = T - 1 - (s - ir);
    if (mine && t >= 0 && t < T) {
      q_eb[k] = e[(i64)t * V + blank];
      if (!ABI) q_ref[k] = rowRef[(i64)b * maxT + t];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int u = i * R + r;
        if (u < U) {
          q_a[k][r] = al[(i64)t * maxU + u];
          q_ln[k][r] = ln[(i64)t * maxU + u];
          q_el[k][r] = e[(i64)t * V + lab[r]];
        }
      }
    }
  };
#pragma unroll
  for (int k = 0; k < PF; ++k) issue(k, k);
  __syncthreads();  // sEB initialised

  for (int s0 = 0; s0 < S; s0 += PF) {
#pragma unroll
    for (int k = 0; k < PF; ++k) {
      const int s = s0 + k;
      if (s >= S) break;
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
              W[(i64)b * maxT * ldW + (i64)t * ldW + u] = g * expf(sh);
              em[(i64)b * maxT * maxU + (i64)t * maxU + u] = step;
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
  auto issue = [&](int s, int k) {
    const int t = s - i;
    if (mine && t >= 0 && t < T) {
      q_eb[k] = e[(i64)t * V + blank];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int u = i * R + r;
        if (u < U) {
          q_ln[k][r] = ln[(i64)t * maxU + u];
          q_bs[k][r] = (u < U - 1) ? bs[(i64)t * maxU + u] : 0.0f;
        }
      }
    }
  };
#pragma unroll
  for (int k = 0; k < PF; ++k) issue(k, k);

  for (int s0 = 0; s0 < S; s0 += PF) {
#pragma unroll
    for (int k = 0; k < PF; ++k) {
      const int s = s0 + k;
      if (s >= S) break;
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
  const StripCfg cfg = pick_strips(d.maxU);
  ScopedKernel sk("alpha_wavefront", stream);
#define CALL(R, PF, NT)                                                              \
  alpha_kernel<R, PF, NT><<<d.B, cfg.threads, 0, stream>>>(                          \
      E, P, costs, alphas, LN, labels, inLens, labLens, d.B, d.maxT, d.maxU, d.V,   \
      d.blank, lossSum, ticket)
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
  const StripCfg cfg = pick_strips(d.maxU);
  const size_t smem = sizeof(float) * (size_t)(d.maxT > 0 ? d.maxT : 1);
  if (smem > kMaxDynSmem) throw std::invalid_argument("input length above 51200 frames is not supported");
  ScopedKernel sk("gamma_wavefront_abi", stream);
#define CALL(R, PF, NT)                                                               \
  allow_smem(gamma_kernel<R, PF, NT, true>, smem);                                    \
  gamma_kernel<R, PF, NT, true><<<d.B, cfg.threads, smem, stream>>>(                  \
      E, P, alphas, LN, nullptr, nullptr, labels, inLens, labLens, egrads, pgrads,    \
      lngrads, nullptr, 0, nullptr, nullptr, nullptr, nullptr, d.maxT, d.maxU, d.V,   \
      d.blank)
  TB200_DISPATCH_STRIPS(cfg, CALL);
#undef CALL
  TB200_CHECK_LAUNCH();
}

void launch_gamma_fused(const float* E, const float* P, const float* alphas,
                        const float* LN, const float* rowRef, const float* maxP,
                        const int* labels, const int* inLens, const int* labLens,
                        float* W, int ldW, float* em, float* eBlank, float* pBlank,
                        float* pLabel, Dims d, cudaStream_t stream) {
  if (d.B <= 0) return;
  const StripCfg cfg = pick_strips(d.maxU);
  const size_t smem = sizeof(float) * (size_t)(d.maxT > 0 ? d.maxT : 1);
  if (smem > kMaxDynSmem) throw std::invalid_argument("input length above 51200 frames is not supported");
  ScopedKernel sk("gamma_wavefront", stream);
#define CALL(R, PF, NT)                                                               \
  allow_smem(gamma_kernel<R, PF, NT, false>, smem);                                   \
  gamma_kernel<R, PF, NT, false><<<d.B, cfg.threads, smem, stream>>>(                 \
      E, P, alphas, LN, rowRef, maxP, labels, inLens, labLens, nullptr, nullptr,      \
      nullptr, W, ldW, em, eBlank, pBlank, pLabel, d.maxT, d.maxU, d.V, d.blank)
  TB200_DISPATCH_STRIPS(cfg, CALL);
#undef CALL
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
