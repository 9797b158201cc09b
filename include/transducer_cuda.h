/*
 * Declarations of the reference's CUDA backend namespace (transducer/transducer_cuda.h:7-59),
 * implemented by libtransducer_b200.so, so that programs written against that header --
 * the reference's own transducer/test_cuda.cu and benchmark_cuda.cu use CUDA_CHECK from it --
 * compile and link against this library unchanged.
 *
 *   CUDA_CHECK(err)        transducer_cuda.h:7-8   -> cuda::cudaCheck(err, __FILE__, __LINE__)
 *   cuda::cudaCheck        transducer_cuda.h:12, transducer_cuda.cu:271-278: throws
 *                          std::runtime_error("[file:line] CUDA error: ...") on failure
 *   cuda::forward/backward/viterbi   transducer_cuda.h:14-57: the device-pointer entry points
 *                          behind transducer.h's useCuda=true; here they run the sm_100a kernels
 *                          (same contract as tb200_forward / tb200_backward / tb200_viterbi).
 */
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#define CUDA_CHECK(err) cuda::cudaCheck(err, __FILE__, __LINE__)

namespace cuda {

void cudaCheck(cudaError_t err, const char* file, int line);

void forward(const float* emissions, const float* predictions, float* costs, float* alphas,
             const float* logNorms, const int* labels, const int* inputLengths,
             const int* labelLengths, int batchSize, int maxInputLength, int maxLabelLength,
             int alphabetSize, int blank);

void backward(const float* emissions, const float* predictions, float* egrads, float* pgrads,
              float* lngrads, const float* alphas, const float* logNorms, const int* labels,
              const int* inputLengths, const int* labelLengths, int batchSize,
              int maxInputLength, int maxLabelLength, int alphabetSize, int blank);

void viterbi(const float* emissions, const float* predictions, const float* logNorms, int* labels,
             const int* inputLengths, const int* labelLengths, int batchSize, int maxInputLength,
             int maxLabelLength, int alphabetSize, int blank);

}  // namespace cuda
