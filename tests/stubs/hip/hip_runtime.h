// Stand-in for <hip/hip_runtime.h>, for SYNTAX checks only (tests/test_shim_compiles.py): just the names strixite's headers
// mention, declared the way CUDA declares their twins, so that the reference's declarations can be parsed on a machine that has
// no ROCm. Nothing here is ever linked or run.
#pragma once
#include <cstddef>

typedef struct ihipStream_t *hipStream_t;
typedef enum hipError_t { hipSuccess = 0, hipErrorOutOfMemory = 2 } hipError_t;
typedef enum hipMemcpyKind { hipMemcpyHostToDevice = 1, hipMemcpyDeviceToHost = 2 } hipMemcpyKind;
constexpr unsigned int hipHostMallocDefault = 0;
const char *hipGetErrorName(hipError_t);
const char *hipGetErrorString(hipError_t);
hipError_t hipGetLastError();
hipError_t hipMalloc(void **, size_t);
template <typename T>
hipError_t hipMalloc(T **p, size_t n) { return hipMalloc(reinterpret_cast<void **>(p), n); }
hipError_t hipFree(void *);
hipError_t hipHostMalloc(void **, size_t, unsigned int);
template <typename T>
hipError_t hipHostMalloc(T **p, size_t n, unsigned int f) { return hipHostMalloc(reinterpret_cast<void **>(p), n, f); }
hipError_t hipHostFree(void *);
hipError_t hipMemcpy(void *, const void *, size_t, hipMemcpyKind);
