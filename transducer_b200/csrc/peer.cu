// One-shot exchange of the per-rank loss sums over peer memory (NVLink / NVSwitch P2P stores):
// an alternative to an NCCL all-reduce for the path's only collective, whose payload is 4 bytes.
// The reference is single-GPU and has no counterpart.
//
// Every rank owns a buffer of slots, one per peer and two per step parity:
//   slot[parity][r] = (sequence number, value bits) written by rank r with ONE 8-byte store.
// A step is one launch of ONE warp on every rank: lane r stores this rank's (seq, value) into
// rank r's buffer -- its own included -- and then waits, with a time limit, until slot r of its
// own buffer carries this step's sequence number; the values are added in rank order, so every
// rank obtains the same bits.  Two parities suffice: a rank cannot start step s+2 before every
// peer has finished step s, because its step s+1 waits for their step s+1 stores.
// A peer that never writes makes the wait run out: the total becomes NaN, the device status
// word records it, the context stays usable.
//
// Buffers are plain cudaMalloc memory shared between processes with CUDA IPC handles (the
// ranks are separate processes, one per GPU); how the 64-byte handles travel is the caller's
// business (transducer_b200.distributed.PeerLossSum sends them through torch.distributed).
// No multicast object, no multimem instruction, no TMA: plain peer stores and local loads.
#include <cstring>

#include "../../include/transducer_b200.h"
#include "api_internal.h"
#include "kernels.h"
#include "profile.h"
#include "sm100.cuh"

namespace tb200 {
namespace {

constexpr int kMaxPeers = 32;

struct PeerPtrs {
  unsigned long long* p[kMaxPeers];
};

__global__ void __launch_bounds__(32) loss_sum_exchange_kernel(
    const float* __restrict__ lossSum, PeerPtrs peers, unsigned long long* mine, int rank, int world,
    unsigned seq, float* __restrict__ total, unsigned long long limitNs, int* status) {
  const int lane = threadIdx.x;
  const int parity = seq & 1u;
  float v = 0.0f;
  bool ok = true;
  if (lane < world) {
    const unsigned long long word =
        ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(*lossSum);
    // (a single aligned 8-byte store: sequence number and value arrive together)
    unsigned long long* dst = peers.p[lane] + (size_t)parity * kMaxPeers + rank;
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(word) : "memory");
    const unsigned long long* src = mine + (size_t)parity * kMaxPeers + lane;
    const unsigned long long t0 = sm100::global_timer_ns();
    unsigned long long got;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(src) : "memory");
      if ((unsigned)(got >> 32) == seq) break;
      if (sm100::global_timer_ns() - t0 > limitNs) { ok = false; break; }
    }
    v = __uint_as_float((unsigned)got);
  }
  ok = __all_sync(0xffffffffu, ok);
  float sum = 0.0f;
  for (int r = 0; r < world; ++r) sum += __shfl_sync(0xffffffffu, v, r);   // rank order
  if (lane == 0) {
    if (!ok) {
      atomicCAS(status, sm100::kStatusOk, sm100::kStatusTimeoutPeer);
      sum = __int_as_float(0x7fc00000);
    }
    *total = sum;
  }
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" {

size_t tb200_peer_slots_bytes(void) { return sizeof(unsigned long long) * 2 * kMaxPeers; }

int tb200_peer_alloc(void** ptr) {
  try {
    if (ptr == nullptr) return api_fail(kErrInvalidArgument, "ptr is null");
    TB200_CUDA_CHECK(cudaMalloc(ptr, tb200_peer_slots_bytes()));
    TB200_CUDA_CHECK(cudaMemset(*ptr, 0, tb200_peer_slots_bytes()));
    return kOk;
  } catch (const std::exception& e) {
    return api_fail(kErrCuda, e.what());
  }
}

int tb200_peer_free(void* ptr) {
  return ptr && cudaFree(ptr) != cudaSuccess ? api_fail(kErrCuda, "cudaFree failed") : kOk;
}

int tb200_peer_export(const void* ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is 64 bytes");
  cudaIpcMemHandle_t h;
  const cudaError_t rc = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
  if (rc != cudaSuccess) return api_fail(kErrCuda, std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(rc));
  std::memcpy(handle64, &h, 64);
  return kOk;
}

int tb200_peer_import(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  const cudaError_t rc = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (rc != cudaSuccess) return api_fail(kErrCuda, std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(rc));
  return kOk;
}

int tb200_peer_close(void* ptr) {
  return ptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess ? api_fail(kErrCuda, "cudaIpcCloseMemHandle failed") : kOk;
}

int tb200_loss_sum_exchange(const float* lossSum, void* const* peerSlots, int rank, int world,
                            unsigned seq, float* total, unsigned timeoutUs) {
  try {
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || seq == 0 ||
        lossSum == nullptr || peerSlots == nullptr || total == nullptr)
      return api_fail(kErrInvalidArgument,
                      "loss_sum_exchange: 1 <= world <= 32, 0 <= rank < world, seq >= 1, no null pointers");
    PeerPtrs pp;
    for (int r = 0; r < kMaxPeers; ++r)
      pp.p[r] = static_cast<unsigned long long*>(r < world ? peerSlots[r] : nullptr);
    for (int r = 0; r < world; ++r)
      if (pp.p[r] == nullptr) return api_fail(kErrInvalidArgument, "loss_sum_exchange: null peer buffer");
    const unsigned long long limitNs = timeoutUs ? (unsigned long long)timeoutUs * 1000ull : sm100::kWaitLimitNs;
    cudaStream_t stream = api_stream();
    ScopedKernel sk("loss_sum_exchange", stream);
    loss_sum_exchange_kernel<<<1, 32, 0, stream>>>(lossSum, pp, pp.p[rank], rank, world, seq, total,
                                                   limitNs, device_status_word());
    TB200_CHECK_LAUNCH();
    return kOk;
  } catch (const std::exception& e) {
    return api_fail(kErrCuda, e.what());
  }
}

}  // extern "C"
