// Pieces of the C-ABI layer shared between translation units.
#pragma once

#include <cuda_runtime.h>

#include <string>

namespace tb200 {

// Records `msg` as the calling thread's last error and returns `code`.
int api_fail(int code, const std::string& msg);
// Stream selected with tb200_set_stream on the calling thread.
cudaStream_t api_stream();

// Device address, on the current device, of the library's status word (status.cu): int[4],
// [0] first code recorded by a bounded wait that ran out since the last tb200_check_status,
// [1] lattice nodes recomputed exactly since then.  Throws CudaError.
int* device_status_word();
const char* status_name(int code);

}  // namespace tb200
