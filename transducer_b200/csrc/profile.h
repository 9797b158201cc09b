// Launch accounting: every kernel launch of the library passes through a
// ScopedKernel, which counts it and, when profiling is switched on, brackets it with
// CUDA events on the launching stream so per-kernel device time can be read back
// without an external profiler.
#pragma once

#include <cuda_runtime.h>

#include <string>

namespace tb200 {

struct ScopedKernel {
  ScopedKernel(const char* name, cudaStream_t stream);
  ~ScopedKernel();
  ScopedKernel(const ScopedKernel&) = delete;
  ScopedKernel& operator=(const ScopedKernel&) = delete;

 private:
  int slot_;
  cudaStream_t stream_;
};

long long launch_count();
void profile_enable(bool on);
void profile_reset();
// Synchronises the recorded events and returns "name launches total_ms" lines.
std::string profile_report();

}  // namespace tb200
