// Shared device/host helpers for the sm_100a RNN-T loss / Viterbi kernels.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

namespace tb200 {

using i64 = long long;

constexpr int kOk = 0;
constexpr int kErrInvalidArgument = 1;
constexpr int kErrCuda = 2;
constexpr int kErrWorkspace = 3;
constexpr int kErrUnsupported = 4;
constexpr int kErrDeviceStatus = 5;

// Thrown by the launchers; the C-ABI layer turns it into a status code + message,
// the C++-linkage entry points let it propagate (as the reference's CUDA_CHECK does,
// transducer/transducer_cuda.cu:271-278).
struct CudaError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

inline void cuda_check(cudaError_t err, const char* file, int line) {
  if (err != cudaSuccess) {
    throw CudaError(std::string("[") + file + ":" + std::to_string(line) +
                    "] CUDA error: " + cudaGetErrorString(err));
  }
}
#define TB200_CUDA_CHECK(expr) ::tb200::cuda_check((expr), __FILE__, __LINE__)
#define TB200_CHECK_LAUNCH() ::tb200::cuda_check(cudaGetLastError(), __FILE__, __LINE__)

struct bf16 {
  unsigned short bits;
};
constexpr int kDtypeF32 = 0, kDtypeBf16 = 1;

__host__ __device__ inline int div_up(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline i64 div_up64(i64 a, i64 b) { return (a + b - 1) / b; }
__host__ __device__ inline i64 round_up64(i64 a, i64 b) { return div_up64(a, b) * b; }

#ifdef __CUDACC__
__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }
__device__ __forceinline__ float pos_inf() { return __int_as_float(0x7f800000); }

// Two-term log-sum-exp with the reference's -inf short-circuits and operation
// order (transducer/transducer_cpu.cpp:16-24, transducer_cuda.cu:21-30).
__device__ __forceinline__ float lse2(float a, float b) {
  if (a == neg_inf()) return b;
  if (b == neg_inf()) return a;
  return fmaxf(a, b) + log1pf(expf(-fabsf(a - b)));
}

// Storage types of emissions / predictions / gradients: fp32, or bf16 held as raw bits.  All
// arithmetic is fp32 on the exactly converted values.
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __uint_as_float((unsigned)x.bits << 16); }
__device__ __forceinline__ void from_f32(float& d, float x) { d = x; }
__device__ __forceinline__ void from_f32(bf16& d, float x) {   // round to nearest even
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(d.bits) : "f"(x));
}
// four consecutive elements (16-byte resp. 8-byte aligned)
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                     __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
#endif

}  // namespace tb200
