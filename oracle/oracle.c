/*
 * CPU oracle for the additive-joiner RNN-T loss / Viterbi path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the algorithm of
 * awni/transducer's CPU backend and of the torch-op arithmetic that surrounds
 * it.  It is the checker used by tests/, by the smoke check and by the
 * cpu_baseline leg of bench.py.  Nothing in the product package links, imports
 * or executes it.
 *
 * Parity of this restatement is pinned two ways (tests/test_oracle.py):
 *   - the literal known-answer vectors of the reference's own tests
 *     (transducer/test.cpp:92-309, torch_test.py:41-158), kept as JSON under
 *     tests/golden/;
 *   - bit-for-bit agreement with the reference's CPU backend compiled
 *     unchanged from its sources (oracle/Makefile -> oracle/_ref/), on seeded
 *     inputs; outputs of that build are stored as fixtures under tests/golden/.
 *
 * Indexing conventions (transducer/transducer_cpu.cpp:242-256): per utterance
 * b, T = inputLengths[b], U = labelLengths[b] + 1; emissions are [B,maxT,V],
 * predictions [B,maxU,V], logNorms/alphas/lngrads [B,maxT,maxU] (row stride
 * maxU), labels [B,maxU-1].  64-bit offsets are used throughout (the
 * reference's 32-bit offsets overflow for B*maxT*V >= 2^31).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

typedef int64_t i64;

/* transducer/transducer_cpu.cpp:16-24 -- two-term log-sum-exp with the
 * -inf short-circuits; fp32 libm calls, same as std::log1p/std::exp on float. */
static inline float lse2(float a, float b) {
  if (a == -INFINITY) return b;
  if (b == -INFINITY) return a;
  float hi = (a < b) ? b : a;
  return hi + log1pf(expf(-fabsf(a - b)));
}

/* ------------------------------------------------------------------------ */
/* log-normalisers                                                           */
/* ------------------------------------------------------------------------ */

/* transducer/test.h:51-80 -- exact, max-subtracted logsumexp over v of
 * E[t,v]+P[u,v] for the valid (t<T_b, u<U_b) region; padding left untouched. */
ORACLE_API void oracle_log_norms_exact(
    const float* E, const float* P, float* LN,
    const int* inLens, const int* labLens,
    int B, int maxT, int maxU, int V) {
#pragma omp parallel for schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    const int T = inLens[b], U = labLens[b] + 1;
    const float* e = E + (i64)b * maxT * V;
    const float* p = P + (i64)b * maxU * V;
    float* ln = LN + (i64)b * maxT * maxU;
    for (int t = 0; t < T; ++t) {
      for (int u = 0; u < U; ++u) {
        const float* er = e + (i64)t * V;
        const float* pr = p + (i64)u * V;
        float m = -INFINITY;
        for (int v = 0; v < V; ++v) {
          float s = er[v] + pr[v];
          if (s > m) m = s;
        }
        float acc = 0.0f;
        for (int v = 0; v < V; ++v) acc += expf(er[v] + pr[v] - m);
        ln[(i64)t * maxU + u] = logf(acc) + m;
      }
    }
  }
}

/* transducer/torch_binding.py:35-40 -- the exp-factored form over the FULL
 * padded [maxT,maxU] rectangle: rowwise maxima, exp of the shifted rows, their
 * inner products, log, then the maxima added back (maxE first, then maxP).
 * The inner product is accumulated in fp32 in index order (torch's blocked
 * SGEMM sums in another order; both are fp32 sums of the same terms). */
ORACLE_API void oracle_log_norms_factored(
    const float* E, const float* P, float* LN,
    int B, int maxT, int maxU, int V) {
#pragma omp parallel for schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    const float* e = E + (i64)b * maxT * V;
    const float* p = P + (i64)b * maxU * V;
    float* ln = LN + (i64)b * maxT * maxU;
    float* xp = (float*)malloc(sizeof(float) * (size_t)maxU * V);
    float* mp = (float*)malloc(sizeof(float) * (size_t)maxU);
    float* xe = (float*)malloc(sizeof(float) * (size_t)V);
    for (int u = 0; u < maxU; ++u) {
      float m = -INFINITY;
      for (int v = 0; v < V; ++v) if (p[(i64)u * V + v] > m) m = p[(i64)u * V + v];
      mp[u] = m;
      for (int v = 0; v < V; ++v) xp[(i64)u * V + v] = expf(p[(i64)u * V + v] - m);
    }
    for (int t = 0; t < maxT; ++t) {
      float me = -INFINITY;
      for (int v = 0; v < V; ++v) if (e[(i64)t * V + v] > me) me = e[(i64)t * V + v];
      for (int v = 0; v < V; ++v) xe[v] = expf(e[(i64)t * V + v] - me);
      for (int u = 0; u < maxU; ++u) {
        float acc = 0.0f;
        for (int v = 0; v < V; ++v) acc += xe[v] * xp[(i64)u * V + v];
        ln[(i64)t * maxU + u] = (logf(acc) + me) + mp[u];
      }
    }
    free(xp); free(mp); free(xe);
  }
}

/* ------------------------------------------------------------------------ */
/* alpha recursion                                                           */
/* ------------------------------------------------------------------------ */

/* transducer/transducer_cpu.cpp:30-79.  The reference fills row 0 and column 0
 * by direct sums and the interior by lse2(emit, noEmit); lse2's -inf
 * short-circuit makes the single loop below produce the same bits. */
static float alpha_one(const float* e, const float* p, float* al, const float* ln,
                       const int* lab, int blank, int T, int U, int maxU, int V) {
  if (T == 0 || U == 0) return INFINITY;
  for (int t = 0; t < T; ++t) {
    for (int u = 0; u < U; ++u) {
      if (t == 0 && u == 0) { al[0] = 0.0f; continue; }
      float stay = -INFINITY, step = -INFINITY;
      if (t > 0) {
        i64 k = (i64)(t - 1) * maxU + u;
        stay = al[k] + e[(i64)(t - 1) * V + blank] + p[(i64)u * V + blank] - ln[k];
      }
      if (u > 0) {
        i64 k = (i64)t * maxU + (u - 1);
        int l = lab[u - 1];
        step = al[k] + e[(i64)t * V + l] + p[(i64)(u - 1) * V + l] - ln[k];
      }
      al[(i64)t * maxU + u] = lse2(step, stay);
    }
  }
  i64 k = (i64)(T - 1) * maxU + (U - 1);
  float end = al[k] + e[(i64)(T - 1) * V + blank] + p[(i64)(U - 1) * V + blank] - ln[k];
  return -end;
}

/* transducer/transducer_cpu.cpp:228-257 */
ORACLE_API void oracle_forward(
    const float* E, const float* P, float* costs, float* alphas, const float* LN,
    const int* labels, const int* inLens, const int* labLens,
    int B, int maxT, int maxU, int V, int blank) {
#pragma omp parallel for schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    i64 lo = (i64)b * maxT * maxU;
    costs[b] = alpha_one(E + (i64)b * maxT * V, P + (i64)b * maxU * V, alphas + lo,
                         LN + lo, labels + (i64)b * (maxU - 1), blank,
                         inLens[b], labLens[b] + 1, maxU, V);
  }
}

/* ------------------------------------------------------------------------ */
/* reverse sweep: node occupancies and the sparse part of the gradients       */
/* ------------------------------------------------------------------------ */

/* transducer/transducer_cpu.cpp:81-143.  g[t,u] (the reference's dalphas,
 * returned as lngrads) is the occupancy of lattice node (t,u).  Every
 * read-modify-write below hits a given address in the same order as the
 * reference's three loops do (t descending, then u descending; within a node:
 * blank column of egrads, blank column of pgrads, label column of egrads,
 * label column of pgrads), so the fp32 sums agree bit for bit. */
static void gamma_one(const float* e, const float* p, float* ge, float* gp, float* g,
                      const float* al, const float* ln, const int* lab,
                      int blank, int T, int U, int maxU, int V) {
  if (T == 0 || U == 0) return;
  g[(i64)(T - 1) * maxU + (U - 1)] = 1.0f;
  ge[(i64)(T - 1) * V + blank] = -1.0f;
  gp[(i64)(U - 1) * V + blank] = -1.0f;
  for (int t = T - 1; t >= 0; --t) {
    for (int u = U - 1; u >= 0; --u) {
      if (t == T - 1 && u == U - 1) continue;
      i64 k = (i64)t * maxU + u;
      float stay = 0.0f, step = 0.0f;
      if (t < T - 1) {
        i64 kn = (i64)(t + 1) * maxU + u;
        stay = g[kn] * expf(al[k] + e[(i64)t * V + blank] + p[(i64)u * V + blank]
                            - ln[k] - al[kn]);
      }
      if (u < U - 1) {
        i64 kn = k + 1;
        int l = lab[u];
        step = g[kn] * expf(al[k] + e[(i64)t * V + l] + p[(i64)u * V + l]
                            - ln[k] - al[kn]);
      }
      /* the reference's boundary loops store the single term; 0+x and x+0 are x */
      if (t == T - 1) g[k] = step;
      else if (u == U - 1) g[k] = stay;
      else g[k] = stay + step;
      if (t < T - 1) {
        ge[(i64)t * V + blank] -= stay;
        gp[(i64)u * V + blank] -= stay;
      }
      if (u < U - 1) {
        int l = lab[u];
        ge[(i64)t * V + l] -= step;
        gp[(i64)u * V + l] -= step;
      }
    }
  }
}

/* transducer/transducer_cpu.cpp:259-306: all three outputs are zero-filled over
 * their full padded extent before the sweep. */
ORACLE_API void oracle_backward(
    const float* E, const float* P, float* egrads, float* pgrads, float* lngrads,
    const float* alphas, const float* LN,
    const int* labels, const int* inLens, const int* labLens,
    int B, int maxT, int maxU, int V, int blank) {
#pragma omp parallel for schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    i64 eo = (i64)b * maxT * V, po = (i64)b * maxU * V, lo = (i64)b * maxT * maxU;
    memset(egrads + eo, 0, sizeof(float) * (size_t)maxT * V);
    memset(pgrads + po, 0, sizeof(float) * (size_t)maxU * V);
    memset(lngrads + lo, 0, sizeof(float) * (size_t)maxT * maxU);
    gamma_one(E + eo, P + po, egrads + eo, pgrads + po, lngrads + lo, alphas + lo,
              LN + lo, labels + (i64)b * (maxU - 1), blank,
              inLens[b], labLens[b] + 1, maxU, V);
  }
}

/* transducer/test.h:82-113 -- brute-force dense part of the gradient:
 * egrads[t,v] += g[t,u]*softmax(t,u)[v], pgrads[u,v] += the same, over the
 * valid region.  O(T*U*V) exps: small cases only. */
ORACLE_API void oracle_accumulate_grads_exact(
    const float* E, const float* P, float* egrads, float* pgrads,
    const float* lngrads, const float* LN,
    const int* inLens, const int* labLens,
    int B, int maxT, int maxU, int V) {
  for (int b = 0; b < B; ++b) {
    const int T = inLens[b], U = labLens[b] + 1;
    i64 eo = (i64)b * maxT * V, po = (i64)b * maxU * V, lo = (i64)b * maxT * maxU;
    for (int t = 0; t < T; ++t)
      for (int u = 0; u < U; ++u) {
        float w = lngrads[lo + (i64)t * maxU + u];
        float z = LN[lo + (i64)t * maxU + u];
        for (int v = 0; v < V; ++v) {
          float s = expf(E[eo + (i64)t * V + v] + P[po + (i64)u * V + v] - z);
          egrads[eo + (i64)t * V + v] += w * s;
          pgrads[po + (i64)u * V + v] += w * s;
        }
      }
  }
}

/* ------------------------------------------------------------------------ */
/* Viterbi                                                                   */
/* ------------------------------------------------------------------------ */

/* transducer/transducer_cpu.cpp:156-169: best non-blank label of E[t,:]+P[u,:];
 * strict '>' keeps the lowest index among ties; starts from (-inf, 0). */
static inline float best_label(const float* er, const float* pr, int V, int blank, int* arg) {
  float m = -INFINITY;
  int a = 0;
  for (int v = 0; v < V; ++v) {
    if (v == blank) continue;
    float s = er[v] + pr[v];
    if (s > m) { m = s; a = v; }
  }
  *arg = a;
  return m;
}

/* transducer/transducer_cpu.cpp:145-222.  Scores/paths have row stride U (not
 * maxU).  Row 0 always takes the label, column 0 always the blank; elsewhere
 * the label wins only on strict emit > noEmit.  The backtrack is bounded here
 * (the reference's loop is not): it stops if t would leave the lattice. */
static void viterbi_one(const float* e, const float* p, const float* ln, int* out,
                        int blank, int T, int U, int maxU, int V) {
  if (T == 0 || U == 0) return;
  float* sc = (float*)malloc(sizeof(float) * (size_t)T * U);
  int* bp = (int*)malloc(sizeof(int) * (size_t)T * U);
  sc[0] = 0.0f;
  bp[0] = blank;
  for (int t = 0; t < T; ++t) {
    for (int u = 0; u < U; ++u) {
      if (t == 0 && u == 0) continue;
      i64 k = (i64)t * U + u;
      if (u == 0) {
        sc[k] = sc[k - U] + e[(i64)(t - 1) * V + blank] + p[blank] - ln[(i64)(t - 1) * maxU];
        bp[k] = blank;
        continue;
      }
      int arg;
      float best = best_label(e + (i64)t * V, p + (i64)(u - 1) * V, V, blank, &arg);
      if (t == 0) {
        sc[k] = best + sc[k - 1] - ln[u - 1];
        bp[k] = arg;
        continue;
      }
      float stay = sc[k - U] + e[(i64)(t - 1) * V + blank] + p[(i64)u * V + blank]
                   - ln[(i64)(t - 1) * maxU + u];
      float step = sc[k - 1] + best - ln[(i64)t * maxU + (u - 1)];
      if (step > stay) { sc[k] = step; bp[k] = arg; }
      else { sc[k] = stay; bp[k] = blank; }
    }
  }
  int t = T - 1, u = U - 1;
  while (u > 0 && t >= 0) {
    int l = bp[(i64)t * U + u];
    if (l == blank) --t;
    else { out[u - 1] = l; --u; }
  }
  free(sc); free(bp);
}

/* transducer/transducer_cpu.cpp:308-331 */
ORACLE_API void oracle_viterbi(
    const float* E, const float* P, const float* LN, int* labels,
    const int* inLens, const int* labLens,
    int B, int maxT, int maxU, int V, int blank) {
#pragma omp parallel for schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    viterbi_one(E + (i64)b * maxT * V, P + (i64)b * maxU * V,
                LN + (i64)b * maxT * maxU, labels + (i64)b * (maxU - 1), blank,
                inLens[b], labLens[b] + 1, maxU, V);
  }
}
