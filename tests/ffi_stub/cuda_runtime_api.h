// TEST STAND-IN for the two CUDA runtime names xla_ffi.cc uses (no CUDA toolkit needed to type-check it)
#pragma once
#include <cstddef>
typedef struct CUstream_st* cudaStream_t;
enum cudaError_t { cudaSuccess = 0 };
inline cudaError_t cudaMemsetAsync(void*, int, size_t, cudaStream_t) { return cudaSuccess; }
