// Host-visible twin of the time-out flags. Every kernel file keeps its own flag in device
// memory (read by nvfp4r_check_device_status, which synchronises the device); report_timeout
// additionally writes a code into one word of pinned, mapped host memory when the host has asked
// for it (nvfp4r_status_mirror), so that a serving loop can notice a bounded wait that gave up by
// reading an ordinary host variable between steps, without synchronising anything.
// Each translation unit that includes this header gets its own copy of the device pointer; the
// launcher of nvfp4r_status_mirror sets all of them.
#pragma once

#include <cuda_runtime.h>

namespace nvfp4r {

static __device__ int* g_status_mirror = nullptr;

// code: which family gave up (1 GEMV ring, 2 tensor-core GEMM, 3 packed linear, 4 peer
// all-reduce, 5 ReSET step).
__device__ __forceinline__ void report_timeout(int* flag, int code) {
    atomicExch(flag, 1);
    int* m = g_status_mirror;
    if (m != nullptr) *reinterpret_cast<volatile int*>(m) = code;
}

// Called once per translation unit by the host (with the target device current).
static inline cudaError_t set_status_mirror_here(int* device_ptr) {
    return cudaMemcpyToSymbol(g_status_mirror, &device_ptr, sizeof(int*));
}

}  // namespace nvfp4r
