/*
 * Test-only stand-in for the part of the CUDA runtime API the host side of the library uses
 * (csrc/runner.cpp).  Never on a production include path: the Makefile target `fakecuda` puts this
 * directory first, so that the production runner compiles unchanged against a deterministic model
 * of the runtime (fake_runtime.cpp) whose calls can be made to fail one at a time.  No GPU is
 * involved.  Same idea as the reference's fake driver (projects/secant/tests/support/fake_cuda/cuda.h).
 */
#ifndef SECANT_B200_FAKE_CUDA_RUNTIME_H
#define SECANT_B200_FAKE_CUDA_RUNTIME_H
#include <stddef.h>
#include <stdint.h>

typedef enum cudaError {
    cudaSuccess = 0,
    cudaErrorInvalidValue = 1,
    cudaErrorMemoryAllocation = 2,
    cudaErrorCudartUnloading = 4,
    cudaErrorInvalidConfiguration = 9,
    cudaErrorUnknown = 999
} cudaError_t;
typedef struct FakeStream* cudaStream_t;
typedef struct FakeEvent* cudaEvent_t;
enum { cudaStreamNonBlocking = 1 };
enum { cudaEventDefault = 0, cudaEventDisableTiming = 2 };
enum { cudaHostAllocDefault = 0 };
enum cudaMemcpyKind { cudaMemcpyHostToDevice = 1 };
enum cudaDeviceAttr { cudaDevAttrMultiProcessorCount = 16, cudaDevAttrMaxSharedMemoryPerBlockOptin = 97 };
enum { cudaEnableDefault = 0 };
typedef enum cudaDriverEntryPointQueryResult { cudaDriverEntryPointSuccess = 0, cudaDriverEntryPointSymbolNotFound = 1 } cudaDriverEntryPointQueryResult;

#ifdef __cplusplus
extern "C" {
#endif
cudaError_t cudaGetDevice(int* device);
cudaError_t cudaDeviceGetAttribute(int* value, enum cudaDeviceAttr attr, int device);
cudaError_t cudaGetDriverEntryPoint(const char* symbol, void** entry, unsigned long long flags, cudaDriverEntryPointQueryResult* status);
cudaError_t cudaGetLastError(void);
const char* cudaGetErrorString(cudaError_t error);
cudaError_t cudaMalloc(void** ptr, size_t bytes);
cudaError_t cudaFree(void* ptr);
cudaError_t cudaHostAlloc(void** ptr, size_t bytes, unsigned flags);
cudaError_t cudaFreeHost(void* ptr);
cudaError_t cudaMemcpyAsync(void* dst, const void* src, size_t bytes, enum cudaMemcpyKind kind, cudaStream_t stream);
cudaError_t cudaMemset2DAsync(void* ptr, size_t pitch, int value, size_t width, size_t height, cudaStream_t stream);
cudaError_t cudaStreamCreateWithFlags(cudaStream_t* stream, unsigned flags);
cudaError_t cudaStreamDestroy(cudaStream_t stream);
cudaError_t cudaStreamSynchronize(cudaStream_t stream);
cudaError_t cudaStreamWaitEvent(cudaStream_t stream, cudaEvent_t event, unsigned flags);
cudaError_t cudaEventCreate(cudaEvent_t* event);
cudaError_t cudaEventCreateWithFlags(cudaEvent_t* event, unsigned flags);
cudaError_t cudaEventDestroy(cudaEvent_t event);
cudaError_t cudaEventRecord(cudaEvent_t event, cudaStream_t stream);
cudaError_t cudaEventSynchronize(cudaEvent_t event);
cudaError_t cudaEventElapsedTime(float* ms, cudaEvent_t start, cudaEvent_t stop);
#ifdef __cplusplus
}
#endif
#endif
