// tb200_viterbi_static: the Viterbi entry point for callers that cannot allocate.
//
// tb200_viterbi borrows its two temporaries (the per-node best label score and the packed
// back-pointers) from the CUDA stream-ordered allocator on every call.  Some hosts of this
// library cannot do that:
//   * processes in which another component owns all device memory up front -- a training
//     framework's caching allocator configured to take the whole card, or an inference
//     server with a fixed arena -- so a request to the driver's pool fails with
//     out-of-memory although the application itself has room to spare;
//   * devices or virtualised GPUs whose driver does not offer memory pools at all
//     (cudaDevAttrMemoryPoolsSupported == 0), where cudaMallocAsync is simply unavailable;
//   * latency-sensitive decoding loops that must not meet the occasional pool growth,
//     trim or implicit synchronisation an allocation can bring.
// For them the temporaries live here, in a fixed array that is part of the library image.
// The price: every GPU that loads the library carries the array until the process exits,
// and the lattice that fits is bounded (kStaticBestFloats / kStaticDecWords below).
#include <mutex>
#include <string>

#include "../../include/transducer_b200.h"
#include "api_internal.h"
#include "kernels.h"

namespace tb200 {
namespace {

// 4 Mi lattice nodes of best-label scores (16 MiB) + 160 Ki words of back-pointer bits.
constexpr size_t kStaticBestFloats = size_t(4) << 20;
constexpr size_t kStaticDecWords = size_t(160) << 10;
constexpr size_t kStaticBytes = kStaticBestFloats * sizeof(float) + kStaticDecWords * sizeof(uint32_t);

// File-scope device array.  In host code this NAME is only a handle for the runtime, not a
// device address: a kernel handed `g_viterbi_scratch` directly would fault (or, where the GPU
// can reach host memory, quietly scribble over the wrong bytes).  Host code must ask the
// runtime for the address, per device -- see scratch_for_current_device().
static __device__ __align__(256) unsigned char g_viterbi_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_addr[kMaxDevices] = {};

// Device address of the array on the current device; looked up once per device, with that
// device current, and cached.  Returns nullptr and sets *err on failure.
unsigned char* scratch_for_current_device(std::string* err) {
  int dev = -1;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *err = rc != cudaSuccess ? cudaGetErrorString(rc) : "device ordinal out of range";
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_addr[dev] == nullptr) {
    void* p = nullptr;
    rc = cudaGetSymbolAddress(&p, g_viterbi_scratch);
    if (rc != cudaSuccess || p == nullptr) {
      cudaGetLastError();  // consume it: the next launch check must not report this failure
      *err = std::string("cudaGetSymbolAddress(static Viterbi scratch): ") + cudaGetErrorString(rc);
      return nullptr;
    }
    g_addr[dev] = static_cast<unsigned char*>(p);
  }
  return g_addr[dev];
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" {

size_t tb200_viterbi_static_max_nodes(void) { return kStaticBestFloats; }

int tb200_viterbi_static(const float* emissions, const float* predictions, const float* logNorms,
                         int* labels, const int* inputLengths, const int* labelLengths,
                         int batchSize, int maxInputLength, int maxLabelLength, int alphabetSize,
                         int blank) {
  Dims d{batchSize, maxInputLength, maxLabelLength, alphabetSize, blank};
  if (d.B < 0 || d.maxT < 0 || d.maxU < 0 || d.V <= 0 || blank < 0 || blank >= d.V)
    return api_fail(kErrInvalidArgument, "bad batch/length/alphabet/blank argument");
  if (d.B == 0 || d.maxT == 0 || d.maxU == 0) {
    // nothing to decode, but do the per-device set-up: an empty call at start-up is how a host
    // brings the array onto the device before its own allocator takes the rest of the card
    std::string e0;
    return scratch_for_current_device(&e0) ? kOk : api_fail(kErrCuda, e0);
  }
  const size_t nodes = (size_t)d.B * d.maxT * d.maxU;
  const size_t words = viterbi_decbits_words(d);
  if (nodes > kStaticBestFloats || words > kStaticDecWords)
    return api_fail(kErrWorkspace,
                    "tb200_viterbi_static: lattice of " + std::to_string(nodes) +
                        " nodes (batch*maxInputLength*maxLabelLength) exceeds the built-in scratch of " +
                        std::to_string(kStaticBestFloats) + " nodes / " +
                        std::to_string(kStaticDecWords) +
                        " back-pointer words; use tb200_viterbi or tb200_viterbi_decode");
  std::string err;
  unsigned char* base = scratch_for_current_device(&err);
  if (!base) return api_fail(kErrCuda, err);
  float* best = reinterpret_cast<float*>(base);
  uint32_t* dec = reinterpret_cast<uint32_t*>(base + kStaticBestFloats * sizeof(float));
  try {
    // Nothing in the scratch has to start at zero: within one call every score and every
    // back-pointer word that is read has been written first by that same call.
    launch_maxplus(emissions, predictions, best, inputLengths, labelLengths, d, api_stream());
    launch_viterbi_lattice(emissions, predictions, logNorms, best, dec, labels, inputLengths,
                           labelLengths, d, api_stream());
  } catch (const std::invalid_argument& e) {
    return api_fail(kErrInvalidArgument, e.what());
  } catch (const std::exception& e) {
    return api_fail(kErrCuda, e.what());
  }
  return kOk;
}

}  // extern "C"
