// Stand-in for <cuda_runtime.h> used only by the FFI adapter's CPU test (driver.cc): the two things
// the adapter takes from the runtime, with cudaMemsetAsync acting on host memory.
#ifndef TESTS_XLA_FFI_STUB_CUDA_RUNTIME_H_
#define TESTS_XLA_FFI_STUB_CUDA_RUNTIME_H_
#include <cstddef>
#include <cstring>
typedef struct CUstream_st* cudaStream_t;
enum cudaError_t { cudaSuccess = 0 };
extern int g_stub_memsets;
inline cudaError_t cudaMemsetAsync(void* p, int v, size_t n, cudaStream_t) {
  std::memset(p, v, n);
  ++g_stub_memsets;
  return cudaSuccess;
}
#endif
