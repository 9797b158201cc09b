// Device status word: how a bounded wait that ran out inside a kernel reaches the host.
//
// Every wait of the tensor-core and single-warp sweep kernels (on an mbarrier that a TMA copy,
// an MMA commit or another role completes) gives up after sm100::kWaitLimitNs.  The kernel then
// records WHICH wait in this word (first failure wins, the word is sticky), drains its roles,
// frees its tensor memory, poisons its outputs (NaN costs / log-normalisers / gradients, -1
// labels) and returns normally -- the context stays usable.  The reference has no device-side
// waits; its host-side error path is cudaCheck -> std::runtime_error
// (transducer/transducer_cuda.cu:271-278), launches unchecked.
//
// The word lives in the library image (one per device that loads the library), so no call has
// to allocate or carry it; host code obtains its device address once per device with
// cudaGetSymbolAddress.  tb200_check_status() synchronises the calling thread's stream, reads
// the word, clears it and reports.
#include <mutex>
#include <string>

#include "../../include/transducer_b200.h"
#include "api_internal.h"
#include "kernels.h"
#include "profile.h"
#include "sm100.cuh"

namespace tb200 {
namespace {

// [0] first error code since the last check (sm100::kStatus*), [1] lattice nodes whose
// factored log-normaliser left the fp32 range and were recomputed exactly (diagnostic).
static __device__ int g_device_status[4];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
int* g_addr[kMaxDevices] = {};

__global__ void __launch_bounds__(32) selftest_wait_kernel(int* status, unsigned long long limitNs,
                                                           int* observed) {
  __shared__ uint64_t bar;
  __shared__ int abortFlag;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 1);
    abortFlag = 0;
    sm100::fence_mbar_init();
  }
  __syncwarp();
  // nobody ever arrives on `bar`: the wait must end by its time limit
  const bool ok = sm100::mbar_wait_limit(&bar, 0, &abortFlag, status,
                                         sm100::kStatusTimeoutSelfTest, limitNs);
  const bool all = __all_sync(0xffffffffu, ok);
  if (threadIdx.x == 0) *observed = all ? 1 : 0;  // 0: the wait gave up, as it should
}

}  // namespace

const char* status_name(int code) {
  switch (code) {
    case sm100::kStatusOk: return "ok";
    case sm100::kStatusTimeoutTma: return "a TMA / bulk copy never landed";
    case sm100::kStatusTimeoutOperand: return "an operand stage was never produced";
    case sm100::kStatusTimeoutMma: return "an MMA completion was never signalled";
    case sm100::kStatusTimeoutStageFree: return "a pipeline stage was never released";
    case sm100::kStatusTimeoutPeer: return "a peer's loss sum never arrived";
    case sm100::kStatusTimeoutSelfTest: return "self-test wait (nothing arrives on its barrier)";
    default: return "unknown device status code";
  }
}

int* device_status_word() {
  int dev = -1;
  TB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) throw CudaError("device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_addr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t rc = cudaGetSymbolAddress(&p, g_device_status);
    if (rc != cudaSuccess || p == nullptr) {
      cudaGetLastError();  // consumed here, so that the next launch check does not report it
      throw CudaError(std::string("cudaGetSymbolAddress(device status word): ") +
                      cudaGetErrorString(rc));
    }
    g_addr[dev] = static_cast<int*>(p);
  }
  return g_addr[dev];
}

}  // namespace tb200

using namespace tb200;

extern "C" {

int tb200_check_status(void) {
  try {
    int* word = device_status_word();
    int host[2] = {0, 0};
    cudaStream_t s = api_stream();
    TB200_CUDA_CHECK(cudaMemcpyAsync(host, word, sizeof(host), cudaMemcpyDeviceToHost, s));
    TB200_CUDA_CHECK(cudaStreamSynchronize(s));
    if (host[0] != 0 || host[1] != 0) {
      TB200_CUDA_CHECK(cudaMemsetAsync(word, 0, sizeof(host), s));
      TB200_CUDA_CHECK(cudaStreamSynchronize(s));
    }
    if (host[0] != 0)
      return api_fail(kErrDeviceStatus,
                      "device status " + std::to_string(host[0]) + ": " + status_name(host[0]) +
                          " within the time limit; the kernel returned early and its outputs "
                          "are poisoned (NaN / -1)");
    return kOk;
  } catch (const std::exception& e) {
    return api_fail(kErrCuda, e.what());
  }
}

const char* tb200_status_name(int code) { return status_name(code); }

int tb200_selftest_wait_timeout(unsigned limitMicroseconds) {
  try {
    int* word = device_status_word();
    cudaStream_t s = api_stream();
    {
      ScopedKernel sk("selftest_wait", s);
      selftest_wait_kernel<<<1, 32, 0, s>>>(word, (unsigned long long)limitMicroseconds * 1000ull,
                                            word + 2);
    }
    TB200_CHECK_LAUNCH();
    return kOk;
  } catch (const std::exception& e) {
    return api_fail(kErrCuda, e.what());
  }
}

}  // extern "C"
