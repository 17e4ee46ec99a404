// A stand-in for the CUDA runtime, for compiling the library's host-side files (runtime.cu, memory.cu,
// caching.cu) with a plain C++ compiler and driving their failure paths without a GPU: calls that fail while
// cleaning up, allocations the device refuses, the error a failing call leaves as the thread's last error, and
// a host heap that stays exhausted. "Device memory" is host memory; a "kernel launch" runs the kernel function
// on the calling thread. The knobs are the variables of namespace fake. TEST INFRASTRUCTURE.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <cstring>

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline

enum cudaError_t {
    cudaSuccess = 0,
    cudaErrorInvalidValue = 1,
    cudaErrorMemoryAllocation = 2,
    cudaErrorInvalidDevice = 101,
    cudaErrorInvalidResourceHandle = 400,
};
enum cudaMemcpyKind { cudaMemcpyHostToDevice = 1, cudaMemcpyDeviceToHost = 2, cudaMemcpyDeviceToDevice = 3 };
struct fake_stream_record { int device; };
struct fake_event_record { int device; };
typedef fake_stream_record *cudaStream_t;
typedef fake_event_record *cudaEvent_t;
constexpr unsigned cudaStreamNonBlocking = 1;
constexpr unsigned cudaHostAllocPortable = 1;
struct cudaDeviceProp {
    char name[256];
    int major, minor, multiProcessorCount, warpSize;
    size_t totalGlobalMem;
};

namespace fake {
inline int device_count = 2;
inline int current_device = 1;          // the harness starts on device 1 and creates contexts on device 0
inline cudaError_t last_error = cudaSuccess;  // what cudaGetLastError returns (and clears)
inline int live_streams = 0;
inline int destroyed_on = -1;           // the device that was current when a stream was last destroyed
inline cudaError_t launch_error = cudaSuccess;   // the next launches fail with this
inline cudaError_t destroy_error = cudaSuccess;  // cudaStreamDestroy fails with this (and keeps the stream)
inline cudaError_t memset_error = cudaSuccess;
inline cudaError_t synchronize_error = cudaSuccess;
inline int malloc_failures = 0;         // the next n cudaMalloc calls report out of memory
inline bool malloc_always_fails = false;
inline int mallocs = 0, frees = 0, synchronizes = 0;
inline size_t free_bytes = size_t{1} << 34, total_bytes = size_t{1} << 35;
// the host heap: when set, every operator new throws (the harness replaces operator new)
inline bool deny_new = false;
inline bool deny_new_after_destroy = false;  // the heap runs out once a stream destruction has been attempted
inline bool deny_new_after_launch = false;   // ... once a launch has been attempted

inline cudaError_t record(cudaError_t e) {
    if (e != cudaSuccess) last_error = e;
    return e;
}
template <class Kernel>
inline void launch(Kernel &&kernel) {
    if (deny_new_after_launch) deny_new = true;
    if (launch_error != cudaSuccess) {
        last_error = launch_error;
        return;
    }
    kernel();
}
}  // namespace fake

inline const char *cudaGetErrorString(cudaError_t e) {
    switch (e) {
        case cudaSuccess: return "no error";
        case cudaErrorInvalidValue: return "invalid argument";
        case cudaErrorMemoryAllocation: return "out of memory";
        case cudaErrorInvalidDevice: return "invalid device ordinal";
        case cudaErrorInvalidResourceHandle: return "invalid resource handle";
    }
    return "unknown error";
}
inline cudaError_t cudaGetLastError() {
    const cudaError_t e = fake::last_error;
    fake::last_error = cudaSuccess;
    return e;
}
inline cudaError_t cudaGetDeviceCount(int *n) {
    *n = fake::device_count;
    return cudaSuccess;
}
inline cudaError_t cudaGetDevice(int *d) {
    *d = fake::current_device;
    return cudaSuccess;
}
inline cudaError_t cudaSetDevice(int d) {
    if (d < 0 || d >= fake::device_count) return fake::record(cudaErrorInvalidDevice);
    fake::current_device = d;
    return cudaSuccess;
}
inline cudaError_t cudaGetDeviceProperties(cudaDeviceProp *p, int d) {
    if (d < 0 || d >= fake::device_count) return fake::record(cudaErrorInvalidDevice);
    std::memset(p, 0, sizeof *p);
    std::strcpy(p->name, "stand-in B200");
    p->major = 10;
    p->minor = 0;
    p->multiProcessorCount = 148;
    p->warpSize = 32;
    p->totalGlobalMem = fake::total_bytes;
    return cudaSuccess;
}
inline cudaError_t cudaMemGetInfo(size_t *f, size_t *t) {
    *f = fake::free_bytes;
    *t = fake::total_bytes;
    return cudaSuccess;
}
inline cudaError_t cudaStreamCreateWithFlags(cudaStream_t *s, unsigned) {
    *s = static_cast<cudaStream_t>(std::malloc(sizeof(fake_stream_record)));
    (*s)->device = fake::current_device;
    fake::live_streams += 1;
    return cudaSuccess;
}
inline cudaError_t cudaStreamDestroy(cudaStream_t s) {
    fake::destroyed_on = fake::current_device;
    if (fake::deny_new_after_destroy) fake::deny_new = true;
    if (fake::destroy_error != cudaSuccess) return fake::record(fake::destroy_error);
    std::free(s);
    fake::live_streams -= 1;
    return cudaSuccess;
}
inline cudaError_t cudaStreamSynchronize(cudaStream_t) {
    fake::synchronizes += 1;
    return fake::record(fake::synchronize_error);
}
inline cudaError_t cudaMalloc(void **p, size_t n) {
    fake::mallocs += 1;
    if (fake::malloc_always_fails || fake::malloc_failures > 0) {
        if (fake::malloc_failures > 0) fake::malloc_failures -= 1;
        *p = nullptr;
        return fake::record(cudaErrorMemoryAllocation);
    }
    *p = std::malloc(n ? n : 1);
    return *p != nullptr ? cudaSuccess : fake::record(cudaErrorMemoryAllocation);
}
template <class T>
inline cudaError_t cudaMalloc(T **p, size_t n) {
    return cudaMalloc(reinterpret_cast<void **>(p), n);
}
inline cudaError_t cudaFree(void *p) {
    fake::frees += 1;
    std::free(p);
    return cudaSuccess;
}
inline cudaError_t cudaHostAlloc(void **p, size_t n, unsigned) {
    *p = std::malloc(n ? n : 1);
    return *p != nullptr ? cudaSuccess : fake::record(cudaErrorMemoryAllocation);
}
inline cudaError_t cudaFreeHost(void *p) {
    std::free(p);
    return cudaSuccess;
}
inline cudaError_t cudaMemsetAsync(void *p, int value, size_t n, cudaStream_t) {
    if (fake::memset_error != cudaSuccess) return fake::record(fake::memset_error);
    std::memset(p, value, n);
    return cudaSuccess;
}
inline cudaError_t cudaMemcpyAsync(void *dst, const void *src, size_t n, cudaMemcpyKind, cudaStream_t) {
    std::memmove(dst, src, n);
    return cudaSuccess;
}
inline cudaError_t cudaEventCreate(cudaEvent_t *e) {
    *e = static_cast<cudaEvent_t>(std::malloc(sizeof(fake_event_record)));
    return cudaSuccess;
}
inline cudaError_t cudaEventDestroy(cudaEvent_t e) {
    std::free(e);
    return cudaSuccess;
}
inline cudaError_t cudaEventRecord(cudaEvent_t, cudaStream_t) { return cudaSuccess; }
inline cudaError_t cudaEventSynchronize(cudaEvent_t) { return cudaSuccess; }
inline cudaError_t cudaEventElapsedTime(float *ms, cudaEvent_t, cudaEvent_t) {
    *ms = 0.0f;
    return cudaSuccess;
}
