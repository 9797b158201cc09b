// C ABI (include/transducer_b200.h) and the reference-compatible C++-linkage entry
// points (include/transducer.h) on top of the kernel launchers.
#include <atomic>
#include <cstring>
#include <sstream>
#include <string>

#include "../../include/transducer.h"
#include "../../include/transducer_b200.h"
#include "../../include/transducer_cuda.h"
#include "api_internal.h"
#include "kernels.h"
#include "profile.h"

namespace tb200 {
namespace {

thread_local cudaStream_t g_stream = nullptr;
thread_local std::string g_error;

// Process-wide switches (tb200_set_option); atomics, because the stream and the error
// message are per thread but these are shared.
struct Options {
  std::atomic<int> lognorm_path{0};
  std::atomic<int> grads_path{0};
  std::atomic<int> grad_passes{2};
  std::atomic<int> fused_gather{1};
  std::atomic<int> maxplus_path{0};   // 0 auto, 1 dense, 2 pruned (error if unsupported)
};
Options g_opt;

int fail(int code, const std::string& msg) {
  g_error = msg;
  return code;
}

// Runs `body`, mapping exceptions to status codes.
template <typename F>
int guarded(F&& body) {
  try {
    body();
    return kOk;
  } catch (const CudaError& e) {
    return fail(kErrCuda, e.what());
  } catch (const std::invalid_argument& e) {
    return fail(kErrInvalidArgument, e.what());
  } catch (const std::exception& e) {
    return fail(kErrCuda, e.what());
  }
}

void check_dims(const Dims& d) {
  if (d.B < 0 || d.maxT < 0 || d.maxU < 0 || d.V <= 0)
    throw std::invalid_argument("negative batch/length or non-positive alphabet size");
  if (d.blank < 0 || d.blank >= d.V) throw std::invalid_argument("blank outside [0, alphabetSize)");
}

// Bump allocator over the caller's workspace; every block is 256-byte aligned.
struct Carver {
  char* base;
  size_t used = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  template <typename T>
  T* take(size_t n) {
    used = (used + 255) & ~size_t(255);
    T* p = base ? reinterpret_cast<T*>(base + used) : nullptr;
    used += n * sizeof(T);
    return p;
  }
  size_t total() const { return (used + 255) & ~size_t(255); }
};

int ld_w(const Dims& d) { return (int)round_up64(d.maxU > 0 ? d.maxU : 1, 32); }

struct LogNormWs {
  unsigned* ticket;  // alpha kernel's completion counter
  float* split;      // exp(P) hi/lo operand of the tensor-core path
  float* maxPScratch;
  LogNormWs(Carver& c, const Dims& d) {
    ticket = c.take<unsigned>(16);
    maxPScratch = c.take<float>((size_t)d.B * d.maxU);
    split = c.take<float>(lognorm_umma_workspace_floats(d));
  }
};

// What the forward call leaves for the backward call (opaque to the caller).
struct SavedState {
  float *alphasS, *LNs, *ELs, *ebl, *rowRef, *maxP;
  float2* arcs;   // arc terms of the single-warp sweeps (label axis <= 128), else null
  float* deltas;  // per-block offsets of their rebased alphas
  SavedState(Carver& c, const Dims& d) {
    const SkewGeom g = skew_geom(d);
    const size_t B = d.B;
    alphasS = c.take<float>(B * g.stride);
    LNs = c.take<float>(B * g.stride);
    ELs = c.take<float>(B * g.stride);
    ebl = c.take<float>(B * d.maxT);
    rowRef = c.take<float>(B * d.maxT);
    maxP = c.take<float>(B * d.maxU);
    arcs = c.take<float2>(lattice_warp_supported(d) ? B * g.stride : 0);
    deltas = c.take<float>(lattice_warp_supported(d) ? lattice_warp_delta_floats(d) : 0);
    if (!lattice_warp_supported(d)) arcs = nullptr;
  }
};

struct ForwardWs {
  float* LN;  // row-major log-normalisers before the re-layout
  float* EL;  // row-major label emissions E[t,label_u] gathered by the log-normaliser pass
  ForwardWs(Carver& c, const Dims& d) {
    LN = c.take<float>((size_t)d.B * d.maxT * d.maxU);
    EL = c.take<float>(lognorm_umma_gathers(d) ? (size_t)d.B * d.maxT * d.maxU : 0);
  }
};

struct BackwardWs {
  float *expP, *Ws, *EMs, *W, *em, *emT, *nref, *ebl, *eBlank, *pBlank, *pLabel, *maxPScratch;
  BackwardWs(Carver& c, const Dims& d) {
    const SkewGeom g = skew_geom(d);
    const size_t B = d.B, T = d.maxT, U = d.maxU, V = d.V;
    expP = c.take<float>(B * U * V);  // SIMT path only
    Ws = c.take<float>(B * g.stride);
    EMs = c.take<float>(B * g.stride);
    W = c.take<float>(B * T * ld_w(d));
    em = c.take<float>(B * T * U);            // SIMT path
    emT = c.take<float>(B * U * grads_umma_ld_t(d));  // tensor-core path
    nref = c.take<float>(B * grads_umma_ld_t(d));
    ebl = c.take<float>(B * grads_umma_ld_t(d));
    eBlank = c.take<float>(B * T);
    pBlank = c.take<float>(B * U);
    pLabel = c.take<float>(B * U);
    maxPScratch = c.take<float>(B * U);
  }
};

struct ViterbiWs {
  float *LN, *rowRef, *maxP, *best;
  uint32_t* decBits;
  float4* nodes;  // skewed per-node operands of the single-warp sweep (label axis <= 256)
  char* prune;    // candidate lists of the pruned max-plus (null where it does not apply)
  ViterbiWs(Carver& c, const Dims& d) {
    const size_t B = d.B, T = d.maxT, U = d.maxU;
    LN = c.take<float>(B * T * U);
    rowRef = c.take<float>(B * T);
    maxP = c.take<float>(B * U);
    best = c.take<float>(B * T * U);
    decBits = c.take<uint32_t>(std::max(viterbi_decbits_words(d), viterbi_warp_decbits_words(d)));
    nodes = c.take<float4>(viterbi_warp_nodes(d));
    prune = c.take<char>(maxplus_pruned_scratch_bytes(d));
  }
};

// Label-arc scores of every node, by the pruned evaluation where it applies.
void best_label_scores(const float* E, const float* P, float* best, const int* inLens,
                       const int* labLens, const Dims& d, void* pruneScratch) {
  const bool can = maxplus_pruned_supported(d) && pruneScratch != nullptr;
  if (g_opt.maxplus_path == 2 && !can)
    throw std::invalid_argument("pruned max-plus does not apply to these sizes");
  if (can && g_opt.maxplus_path != 1)
    launch_maxplus_pruned(E, P, best, inLens, labLens, d, pruneScratch, device_status_word(),
                          g_stream);
  else
    launch_maxplus(E, P, best, inLens, labLens, d, g_stream);
}

void need(size_t have, size_t want, const void* ws) {
  if (want > 0 && (ws == nullptr || have < want))
    throw std::invalid_argument("workspace too small: need " + std::to_string(want) +
                                " bytes, got " + std::to_string(have));
}

// Log-normalisers plus the row shifts.  With the exact path rowRef is the true row
// maximum of E.
// Returns true if the pass also produced the label / blank emissions (EL, ebl) it was offered.
bool log_norms_impl(const void* E, const void* P, float* LN, float* rowRef, float* maxP,
                    const int* inLens, const int* labLens, const Dims& d, LogNormWs& ws,
                    bool fixup = true, const int* labels = nullptr, float* EL = nullptr,
                    float* ebl = nullptr) {
  if (d.B <= 0 || d.maxT <= 0 || d.maxU <= 0) return false;
  const bool can = lognorm_umma_supported(E, P, d);
  if (g_opt.lognorm_path == 2 && !can)
    throw std::invalid_argument(
        "tensor-core log-normaliser needs alphabetSize % 4 == 0, alphabetSize >= 32, "
        "maxLabelLength <= 256 and 16-byte aligned emissions");
  if (d.dtype != kDtypeF32 && !(can && g_opt.lognorm_path != 1))
    throw std::invalid_argument(
        "bf16 emissions need the tensor-core log-normaliser: alphabetSize % 8 == 0, "
        "alphabetSize >= 32, 16-byte aligned emissions and predictions");
  if (can && g_opt.lognorm_path != 1) {
    // the kernel needs somewhere to put the row shifts even if the caller does not want them
    float* mp = maxP ? maxP : ws.maxPScratch;
    if (!rowRef) throw std::invalid_argument("rowRef must not be null");
    const bool gathers = labels && EL && ebl && lognorm_umma_gathers(d) && g_opt.fused_gather != 0;
    launch_lognorm_umma(E, P, LN, rowRef, mp, inLens, labLens, d, ws.split,
                        device_status_word(), fixup, g_stream, gathers ? labels : nullptr,
                        gathers ? EL : nullptr, gathers ? ebl : nullptr);
    return gathers;
  }
  const float* Ef = static_cast<const float*>(E);
  const float* Pf = static_cast<const float*>(P);
  launch_lognorm_exact(Ef, Pf, LN, inLens, labLens, d, g_stream);
  if (rowRef) launch_row_max(Ef, rowRef, inLens, 0, d.B, d.maxT, d.V, g_stream);
  if (maxP) launch_row_max(Pf, maxP, labLens, 1, d.B, d.maxU, d.V, g_stream);
  return false;
}

}  // namespace

int api_fail(int code, const std::string& msg) { return fail(code, msg); }
cudaStream_t api_stream() { return g_stream; }

}  // namespace tb200

using namespace tb200;

extern "C" {

int tb200_version(void) { return 100; }

const char* tb200_last_error(void) { return g_error.c_str(); }

int tb200_set_stream(void* stream) {
  g_stream = static_cast<cudaStream_t>(stream);
  return kOk;
}
void* tb200_get_stream(void) { return g_stream; }

int tb200_set_option(const char* key, int value) {
  if (!key) return fail(kErrInvalidArgument, "null option key");
  if (!strcmp(key, "lognorm_path") && value >= 0 && value <= 2) g_opt.lognorm_path = value;
  else if (!strcmp(key, "grads_path") && value >= 0 && value <= 2) g_opt.grads_path = value;
  else if (!strcmp(key, "grad_passes") && value >= 1 && value <= 3) g_opt.grad_passes = value;
  else if (!strcmp(key, "fused_gather") && value >= 0 && value <= 1) g_opt.fused_gather = value;
  else if (!strcmp(key, "maxplus_path") && value >= 0 && value <= 2) g_opt.maxplus_path = value;
  else return fail(kErrInvalidArgument, std::string("unknown option or bad value: ") + key);
  return kOk;
}

int tb200_get_option(const char* key, int* value) {
  if (!key || !value) return fail(kErrInvalidArgument, "null argument");
  if (!strcmp(key, "lognorm_path")) *value = g_opt.lognorm_path;
  else if (!strcmp(key, "grads_path")) *value = g_opt.grads_path;
  else if (!strcmp(key, "grad_passes")) *value = g_opt.grad_passes;
  else if (!strcmp(key, "fused_gather")) *value = g_opt.fused_gather;
  else if (!strcmp(key, "maxplus_path")) *value = g_opt.maxplus_path;
  else return fail(kErrInvalidArgument, std::string("unknown option: ") + key);
  return kOk;
}

long long tb200_launch_count(void) { return launch_count(); }
int tb200_profile_enable(int on) {
  profile_enable(on != 0);
  return kOk;
}
int tb200_profile_reset(void) {
  profile_reset();
  return kOk;
}
size_t tb200_profile_report(char* buf, size_t bufBytes) {
  const std::string s = profile_report();
  if (buf && bufBytes > 0) {
    const size_t n = s.size() < bufBytes - 1 ? s.size() : bufBytes - 1;
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return s.size();
}

int tb200_forward(const float* E, const float* P, float* costs, float* alphas,
                  const float* LN, const int* labels, const int* inLens,
                  const int* labLens, int B, int maxT, int maxU, int V, int blank) {
  return guarded([&] {
    Dims d{B, maxT, maxU, V, blank};
    check_dims(d);
    launch_alpha(E, P, costs, alphas, LN, labels, inLens, labLens, d, nullptr, nullptr,
                 g_stream);
  });
}

int tb200_backward(const float* E, const float* P, float* egrads, float* pgrads,
                   float* lngrads, const float* alphas, const float* LN,
                   const int* labels, const int* inLens, const int* labLens, int B,
                   int maxT, int maxU, int V, int blank) {
  return guarded([&] {
    Dims d{B, maxT, maxU, V, blank};
    check_dims(d);
    const size_t b = B, t = maxT, u = maxU, v = V;
    if (b * t * v) TB200_CUDA_CHECK(cudaMemsetAsync(egrads, 0, sizeof(float) * b * t * v, g_stream));
    if (b * u * v) TB200_CUDA_CHECK(cudaMemsetAsync(pgrads, 0, sizeof(float) * b * u * v, g_stream));
    if (b * t * u) TB200_CUDA_CHECK(cudaMemsetAsync(lngrads, 0, sizeof(float) * b * t * u, g_stream));
    launch_gamma_abi(E, P, egrads, pgrads, lngrads, alphas, LN, labels, inLens, labLens, d,
                     g_stream);
  });
}

int tb200_viterbi(const float* E, const float* P, const float* LN, int* labels,
                  const int* inLens, const int* labLens, int B, int maxT, int maxU, int V,
                  int blank) {
  return guarded([&] {
    Dims d{B, maxT, maxU, V, blank};
    check_dims(d);
    if (B == 0 || maxT == 0 || maxU == 0) return;
    const size_t cells = (size_t)B * maxT * maxU;
    const bool warp = viterbi_warp_supported(d);  // label axis <= 256: single-warp sweep
    const size_t decWords = warp ? viterbi_warp_decbits_words(d) : viterbi_decbits_words(d);
    // Temporaries from the stream-ordered allocator, as the reference takes them
    // (transducer_cuda.cu:364-369); released in stream order on every way out.
    struct Temporaries {
      float* best = nullptr;
      uint32_t* dec = nullptr;
      float4* nodes = nullptr;
      void* prune = nullptr;
      cudaStream_t stream;
      ~Temporaries() {
        if (best) cudaFreeAsync(best, stream);
        if (dec) cudaFreeAsync(dec, stream);
        if (nodes) cudaFreeAsync(nodes, stream);
        if (prune) cudaFreeAsync(prune, stream);
      }
    } tmp;
    tmp.stream = g_stream;
    TB200_CUDA_CHECK(cudaMallocAsync((void**)&tmp.best, sizeof(float) * cells, g_stream));
    TB200_CUDA_CHECK(cudaMallocAsync((void**)&tmp.dec, sizeof(uint32_t) * decWords, g_stream));
    if (warp)
      TB200_CUDA_CHECK(cudaMallocAsync((void**)&tmp.nodes, sizeof(float4) * viterbi_warp_nodes(d),
                                       g_stream));
    if (maxplus_pruned_supported(d) && g_opt.maxplus_path != 1)
      TB200_CUDA_CHECK(cudaMallocAsync(&tmp.prune, maxplus_pruned_scratch_bytes(d), g_stream));
    best_label_scores(E, P, tmp.best, inLens, labLens, d, tmp.prune);
    if (warp)
      launch_viterbi_warp(E, P, LN, tmp.best, tmp.nodes, tmp.dec, labels, inLens, labLens, d,
                          device_status_word(), g_stream);
    else
      launch_viterbi_lattice(E, P, LN, tmp.best, tmp.dec, labels, inLens, labLens, d, g_stream);
  });
}

size_t tb200_log_norms_workspace_bytes(int B, int maxT, int maxU, int V) {
  Dims d{B, maxT, maxU, V, 0};
  Carver c(nullptr);
  LogNormWs ws(c, d);
  return c.total();
}

int tb200_log_norms(const float* E, const float* P, float* LN, float* rowRef, float* maxP,
                    const int* inLens, const int* labLens, int B, int maxT, int maxU, int V,
                    void* workspace, size_t workspaceBytes) {
  return guarded([&] {
    Dims d{B, maxT, maxU, V, 0};
    check_dims(d);
    need(workspaceBytes, tb200_log_norms_workspace_bytes(B, maxT, maxU, V), workspace);
    Carver c(workspace);
    LogNormWs ws(c, d);
    log_norms_impl(E, P, LN, rowRef, maxP, inLens, labLens, d, ws);
  });
}

size_t tb200_loss_saved_bytes(int B, int maxT, int maxU, int V) {
  Dims d{B, maxT, maxU, V, 0};
  Carver c(nullptr);
  SavedState s(c, d);
  return c.total();
}

size_t tb200_loss_forward_workspace_bytes(int B, int maxT, int maxU, int V) {
  Dims d{B, maxT, maxU, V, 0};
  Carver c(nullptr);
  ForwardWs f(c, d);
  LogNormWs l(c, d);
  return c.total();
}

namespace {

int loss_forward_any(const void* E, const void* P, const int* labels, const int* inLens,
                     const int* labLens, float* costs, float* lossSum, void* saved,
                     size_t savedBytes, int B, int maxT, int maxU, int V, int blank,
                     void* workspace, size_t workspaceBytes, int dtype) {
  return guarded([&] {
    Dims d{B, maxT, maxU, V, blank, dtype};
    check_dims(d);
    if (dtype != kDtypeF32 && !lattice_warp_supported(d))
      throw std::invalid_argument("bf16 emissions: the label axis must not exceed 128 positions");
    need(workspaceBytes, tb200_loss_forward_workspace_bytes(B, maxT, maxU, V), workspace);
    need(savedBytes, tb200_loss_saved_bytes(B, maxT, maxU, V), saved);
    Carver cs(saved);
    SavedState st(cs, d);
    Carver c(workspace);
    ForwardWs fw(c, d);
    LogNormWs ws(c, d);
    const SkewGeom g = skew_geom(d);
    // (nodes the tensor-core log-normaliser could not represent are recomputed by the re-layout)
    const bool gathered = log_norms_impl(E, P, fw.LN, st.rowRef, st.maxP, inLens, labLens, d, ws,
                                         /*fixup=*/false, labels, fw.EL, st.ebl);
    launch_lattice_prep(E, P, fw.LN, st.LNs, st.arcs ? nullptr : st.ELs, st.ebl, st.arcs, labels,
                        inLens, labLens, g, d, g_stream, gathered ? fw.EL : nullptr);
    if (lossSum) {
      TB200_CUDA_CHECK(cudaMemsetAsync(ws.ticket, 0, sizeof(unsigned), g_stream));
      if (B == 0) TB200_CUDA_CHECK(cudaMemsetAsync(lossSum, 0, sizeof(float), g_stream));
    }
    // The shape alone decides which pair of sweeps runs (the backward call must pick the
    // reverse sweep that matches the format of the saved alphas).
    if (lattice_warp_supported(d))
      launch_alpha_warp(st.arcs, costs, st.alphasS, st.deltas, g, inLens, labLens, d, lossSum,
                        lossSum ? ws.ticket : nullptr, device_status_word(), g_stream);
    else
      launch_alpha_skew(static_cast<const float*>(P), costs, st.alphasS, st.LNs, st.ELs, st.ebl, g,
                        labels, inLens, labLens, d, lossSum, lossSum ? ws.ticket : nullptr, g_stream);
  });
}

}  // namespace

int tb200_loss_forward(const float* E, const float* P, const int* labels, const int* inLens,
                       const int* labLens, float* costs, float* lossSum, void* saved,
                       size_t savedBytes, int B, int maxT, int maxU, int V, int blank,
                       void* workspace, size_t workspaceBytes) {
  return loss_forward_any(E, P, labels, inLens, labLens, costs, lossSum, saved, savedBytes, B, maxT,
                          maxU, V, blank, workspace, workspaceBytes, kDtypeF32);
}

int tb200_loss_forward_bf16(const void* E, const void* P, const int* labels, const int* inLens,
                            const int* labLens, float* costs, float* lossSum, void* saved,
                            size_t savedBytes, int B, int maxT, int maxU, int V, int blank,
                            void* workspace, size_t workspaceBytes) {
  return loss_forward_any(E, P, labels, inLens, labLens, costs, lossSum, saved, savedBytes, B, maxT,
                          maxU, V, blank, workspace, workspaceBytes, kDtypeBf16);
}

size_t tb200_loss_backward_workspace_bytes(int B, int maxT, int maxU, int V) {
  Dims d{B, maxT, maxU, V, 0};
  Carver c(nullptr);
  BackwardWs ws(c, d);
  return c.total();
}

namespace {

int loss_backward_any(const void* E, const void* P, const int* labels, const int* inLens,
                      const int* labLens, const void* saved, size_t savedBytes,
                      const float* deltas, void* egrads, void* pgrads, int B, int maxT,
                      int maxU, int V, int blank, void* workspace, size_t workspaceBytes,
                      int dtype) {
  return guarded([&] {
    Dims d{B, maxT, maxU, V, blank, dtype};
    check_dims(d);
    need(workspaceBytes, tb200_loss_backward_workspace_bytes(B, maxT, maxU, V), workspace);
    need(savedBytes, tb200_loss_saved_bytes(B, maxT, maxU, V), saved);
    if (B == 0) return;
    Carver cs(const_cast<void*>(saved));
    SavedState st(cs, d);
    Carver c(workspace);
    BackwardWs ws(c, d);
    const SkewGeom g = skew_geom(d);
    const int ldW = ld_w(d);
    const int passes = g_opt.grad_passes;
    const bool can = grads_umma_supported(E, P, egrads, pgrads, d, passes);
    if (g_opt.grads_path == 2 && !can)
      throw std::invalid_argument(
          "tensor-core gradients need alphabetSize % 4 == 0, alphabetSize >= 32, "
          "maxLabelLength <= 256 and 16-byte aligned emissions and egrads");
    const bool tensorCore = can && g_opt.grads_path != 1;
    if (dtype != kDtypeF32 && !(tensorCore && lattice_warp_supported(d)))
      throw std::invalid_argument(
          "bf16 gradients need the tensor-core gradient kernel: alphabetSize % 8 == 0, "
          "maxLabelLength <= 128, grad_passes = 2, 16-byte aligned buffers");
    if ((egrads == E || pgrads == P) && !(tensorCore && lattice_warp_supported(d)))   // (one launch only)
      throw std::invalid_argument(
          "gradients in place (egrads == emissions / pgrads == predictions) need the "
          "tensor-core gradient kernel: alphabetSize % 4 == 0, maxLabelLength <= 128");
    const float* Ef = static_cast<const float*>(E);   // (fp32 from here on where used as such)
    const float* Pf = static_cast<const float*>(P);
    float* egf = static_cast<float*>(egrads);
    float* pgf = static_cast<float*>(pgrads);
    if (lattice_warp_supported(d)) {
      // single-warp reverse sweep: blank/label arc occupancies to the skewed lattices
      // ws.Ws / ws.EMs, then re-laid out for whichever gradient kernels follow
      int* status = device_status_word();
      launch_gamma_warp(st.arcs, st.alphasS, st.deltas, g, inLens, labLens, ws.Ws, ws.EMs, ws.pBlank,
                        ws.pLabel, d, status, g_stream);
      if (tensorCore) {
        launch_unskew_round(ws.Ws, ws.EMs, st.LNs, st.rowRef, st.maxP, deltas, ws.W, ws.emT,
                            ws.nref, ws.ebl, inLens, labLens, g, d, true, g_stream);
        launch_grads_umma(E, P, st.maxP, ws.W, ws.emT, ws.nref, ws.ebl, ws.pBlank, ws.pLabel,
                          labels, deltas, egrads, pgrads, inLens, labLens, d, passes, status,
                          g_stream);
        return;
      }
      launch_unskew_round(ws.Ws, ws.EMs, st.LNs, st.rowRef, st.maxP, nullptr, ws.W, ws.em,
                          nullptr, ws.eBlank, inLens, labLens, g, d, false, g_stream);
    } else {
      launch_gamma_skew(Pf, st.alphasS, st.LNs, st.ELs, st.ebl, g, st.rowRef, st.maxP, labels,
                        inLens, labLens, ws.Ws, ws.EMs, ws.eBlank, ws.pBlank, ws.pLabel, d,
                        g_stream);
      launch_lattice_unskew(ws.Ws, ws.EMs, ws.W, ldW, ws.em, inLens, labLens, g, d, g_stream);
      if (tensorCore) {
        // label axes of 129..256 positions: the block-wide sweep's outputs re-laid out as the
        // tensor-core kernel's operands; the kernel runs once per half of the label axis
        launch_tc_operands(ws.W, ws.em, ws.eBlank, st.rowRef, deltas, ws.emT, ws.nref, ws.ebl,
                           inLens, d, g_stream);
        launch_grads_umma(E, P, st.maxP, ws.W, ws.emT, ws.nref, ws.ebl, ws.pBlank, ws.pLabel,
                          labels, deltas, egrads, pgrads, inLens, labLens, d, passes,
                          device_status_word(), g_stream);
        return;
      }
    }
    launch_exp_rows(Pf, ws.expP, ws.maxPScratch, labLens, B, maxU, V, g_stream);
    launch_egrad_simt(Ef, st.rowRef, ws.W, ldW, ws.expP, ws.eBlank, ws.em, labels, deltas,
                      egf, inLens, labLens, d, g_stream);
    launch_pgrad_simt(Ef, st.rowRef, ws.W, ldW, ws.expP, ws.pBlank, ws.pLabel, labels, deltas,
                      pgf, inLens, labLens, d, g_stream);
  });
}

}  // namespace

int tb200_loss_backward(const float* E, const float* P, const int* labels, const int* inLens,
                        const int* labLens, const void* saved, size_t savedBytes,
                        const float* deltas, float* egrads, float* pgrads, int B, int maxT,
                        int maxU, int V, int blank, void* workspace, size_t workspaceBytes) {
  return loss_backward_any(E, P, labels, inLens, labLens, saved, savedBytes, deltas, egrads, pgrads,
                           B, maxT, maxU, V, blank, workspace, workspaceBytes, kDtypeF32);
}

int tb200_loss_backward_bf16(const void* E, const void* P, const int* labels, const int* inLens,
                             const int* labLens, const void* saved, size_t savedBytes,
                             const float* deltas, void* egrads, void* pgrads, int B, int maxT,
                             int maxU, int V, int blank, void* workspace, size_t workspaceBytes) {
  return loss_backward_any(E, P, labels, inLens, labLens, saved, savedBytes, deltas, egrads, pgrads,
                           B, maxT, maxU, V, blank, workspace, workspaceBytes, kDtypeBf16);
}

size_t tb200_label_arc_scores_workspace_bytes(int B, int maxT, int maxU, int V) {
  Dims d{B, maxT, maxU, V, 0};
  return (maxplus_pruned_scratch_bytes(d) + 255) & ~size_t(255);
}

int tb200_label_arc_scores(const float* E, const float* P, const int* inLens, const int* labLens,
                           float* best, int B, int maxT, int maxU, int V, int blank,
                           void* workspace, size_t workspaceBytes) {
  return guarded([&] {
    Dims d{B, maxT, maxU, V, blank};
    check_dims(d);
    need(workspaceBytes, tb200_label_arc_scores_workspace_bytes(B, maxT, maxU, V), workspace);
    if (B == 0 || maxT == 0 || maxU == 0) return;
    best_label_scores(E, P, best, inLens, labLens, d,
                      maxplus_pruned_supported(d) ? workspace : nullptr);
  });
}

size_t tb200_viterbi_decode_workspace_bytes(int B, int maxT, int maxU, int V) {
  Dims d{B, maxT, maxU, V, 0};
  Carver c(nullptr);
  ViterbiWs ws(c, d);
  LogNormWs lw(c, d);
  return c.total();
}

int tb200_viterbi_decode(const float* E, const float* P, const int* inLens,
                         const int* labLens, int* labels, int B, int maxT, int maxU, int V,
                         int blank, void* workspace, size_t workspaceBytes) {
  return guarded([&] {
    Dims d{B, maxT, maxU, V, blank};
    check_dims(d);
    need(workspaceBytes, tb200_viterbi_decode_workspace_bytes(B, maxT, maxU, V), workspace);
    if (B == 0 || maxT == 0 || maxU == 0) return;
    Carver c(workspace);
    ViterbiWs ws(c, d);
    LogNormWs lw(c, d);
    log_norms_impl(E, P, ws.LN, ws.rowRef, ws.maxP, inLens, labLens, d, lw);
    best_label_scores(E, P, ws.best, inLens, labLens, d, ws.prune);
    if (viterbi_warp_supported(d))
      launch_viterbi_warp(E, P, ws.LN, ws.best, ws.nodes, ws.decBits, labels, inLens, labLens, d,
                          device_status_word(), g_stream);
    else
      launch_viterbi_lattice(E, P, ws.LN, ws.best, ws.decBits, labels, inLens, labLens, d,
                             g_stream);
  });
}

}  // extern "C"

// ---- transducer.h-compatible C++ entry points --------------------------------

namespace {
void rethrow(int rc) {
  if (rc == kOk) return;
  if (rc == kErrInvalidArgument) throw std::invalid_argument(tb200_last_error());
  throw std::runtime_error(tb200_last_error());
}
void require_cuda(bool useCuda) {
  if (!useCuda) throw std::invalid_argument("Transducer not built with a CPU backend.");
}
}  // namespace

void forward(const float* emissions, const float* predictions, float* costs, float* alphas,
             const float* logNorms, const int* labels, const int* inputLengths,
             const int* labelLengths, int batchSize, int maxInputLength, int maxLabelLength,
             int alphabetSize, int blank, bool useCuda) {
  require_cuda(useCuda);
  rethrow(tb200_forward(emissions, predictions, costs, alphas, logNorms, labels, inputLengths,
                        labelLengths, batchSize, maxInputLength, maxLabelLength, alphabetSize,
                        blank));
}

void backward(const float* emissions, const float* predictions, float* egrads, float* pgrads,
              float* lngrads, const float* alphas, const float* logNorms, const int* labels,
              const int* inputLengths, const int* labelLengths, int batchSize,
              int maxInputLength, int maxLabelLength, int alphabetSize, int blank,
              bool useCuda) {
  require_cuda(useCuda);
  rethrow(tb200_backward(emissions, predictions, egrads, pgrads, lngrads, alphas, logNorms,
                         labels, inputLengths, labelLengths, batchSize, maxInputLength,
                         maxLabelLength, alphabetSize, blank));
}

void viterbi(const float* emissions, const float* predictions, const float* logNorms,
             int* labels, const int* inputLengths, const int* labelLengths, int batchSize,
             int maxInputLength, int maxLabelLength, int alphabetSize, int blank,
             bool useCuda) {
  require_cuda(useCuda);
  rethrow(tb200_viterbi(emissions, predictions, logNorms, labels, inputLengths, labelLengths,
                        batchSize, maxInputLength, maxLabelLength, alphabetSize, blank));
}

// ---- transducer_cuda.h-compatible namespace (transducer/transducer_cuda.h:7-59) ----------

namespace cuda {

void cudaCheck(cudaError_t err, const char* file, int line) {
  if (err != cudaSuccess) {
    std::ostringstream ess;
    ess << '[' << file << ':' << line << "] CUDA error: " << cudaGetErrorString(err);
    throw std::runtime_error(ess.str());
  }
}

void forward(const float* emissions, const float* predictions, float* costs, float* alphas,
             const float* logNorms, const int* labels, const int* inputLengths,
             const int* labelLengths, int batchSize, int maxInputLength, int maxLabelLength,
             int alphabetSize, int blank) {
  rethrow(tb200_forward(emissions, predictions, costs, alphas, logNorms, labels, inputLengths,
                        labelLengths, batchSize, maxInputLength, maxLabelLength, alphabetSize,
                        blank));
}

void backward(const float* emissions, const float* predictions, float* egrads, float* pgrads,
              float* lngrads, const float* alphas, const float* logNorms, const int* labels,
              const int* inputLengths, const int* labelLengths, int batchSize,
              int maxInputLength, int maxLabelLength, int alphabetSize, int blank) {
  rethrow(tb200_backward(emissions, predictions, egrads, pgrads, lngrads, alphas, logNorms,
                         labels, inputLengths, labelLengths, batchSize, maxInputLength,
                         maxLabelLength, alphabetSize, blank));
}

void viterbi(const float* emissions, const float* predictions, const float* logNorms, int* labels,
             const int* inputLengths, const int* labelLengths, int batchSize, int maxInputLength,
             int maxLabelLength, int alphabetSize, int blank) {
  rethrow(tb200_viterbi(emissions, predictions, logNorms, labels, inputLengths, labelLengths,
                        batchSize, maxInputLength, maxLabelLength, alphabetSize, blank));
}

}  // namespace cuda
