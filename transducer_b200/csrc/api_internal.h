// Pieces of the C-ABI layer shared between translation units.
#pragma once

#include <cuda_runtime.h>

#include <string>

namespace tb200 {

// Records `msg` as the calling thread's last error and returns `code`.
int api_fail(int code, const std::string& msg);
// Stream selected with tb200_set_stream on the calling thread.
cudaStream_t api_stream();

}  // namespace tb200
