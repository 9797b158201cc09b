// C++-linkage entry points with the signatures of awni/transducer's
// transducer/transducer.h:3-49, so code written against that header (its pybind
// shim, its C++ tests and benchmarks) links against libtransducer_b200.so
// unchanged.  This library has no CPU backend: useCuda=false throws
// std::invalid_argument (the reference throws the same type when a backend was not
// built, transducer/transducer.cpp:41).  CUDA failures throw std::runtime_error with
// the reference's "[file:line] CUDA error: ..." text (transducer_cuda.cu:271-278).
#pragma once

void forward(
    const float* emissions, const float* predictions, float* costs, float* alphas,
    const float* logNorms, const int* labels, const int* inputLengths,
    const int* labelLengths, int batchSize, int maxInputLength, int maxLabelLength,
    int alphabetSize, int blank, bool useCuda);

void backward(
    const float* emissions, const float* predictions, float* egrads, float* pgrads,
    float* lngrads, const float* alphas, const float* logNorms, const int* labels,
    const int* inputLengths, const int* labelLengths, int batchSize, int maxInputLength,
    int maxLabelLength, int alphabetSize, int blank, bool useCuda);

void viterbi(
    const float* emissions, const float* predictions, const float* logNorms, int* labels,
    const int* inputLengths, const int* labelLengths, int batchSize, int maxInputLength,
    int maxLabelLength, int alphabetSize, int blank, bool useCuda);
