// ReSET step for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need the
// logits processor: a sampler plug-in that runs inside an engine whose memory pool has
// already claimed the whole GPU (vLLM sizes its KV cache from what is free after model
// load, so a later cudaMalloc can fail or fragment), code running while a stream is being
// captured, or a C host that was handed fixed buffers for inputs and outputs only. The
// regular entry point nvfp4r_reset_step needs a caller-provided workspace; this variant
// keeps that scratch inside the library image instead, in a file-scope __device__ array
// that every GPU that loads the library holds until the process exits
// (NVFP4R_RESET_STATIC_MAX_ROWS rows x sizeof(RowScratch) = 64 x 656 B = 41 984 B).
#include "../../include/nvfp4r_b200.h"
#include "kernels.h"
#include "reset_kernels.h"

namespace nvfp4r {
namespace {

// The scratch itself. In host code this name is only a handle for the runtime's symbol
// table, never a device address; the address is looked up once per device below.
static __device__ __align__(256) unsigned char g_reset_static_scratch[
    NVFP4R_RESET_STATIC_MAX_ROWS * sizeof(RowScratch)];

constexpr int kMaxDevices = 64;
RowScratch* g_scratch_ptr[kMaxDevices] = {};

// First call on a device (with that device current): resolve the array's device address.
cudaError_t static_scratch(RowScratch** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_reset_static_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_ptr[dev] = static_cast<RowScratch*>(p);
    }
    *out = g_scratch_ptr[dev];
    return cudaSuccess;
}

}  // namespace

cudaError_t launch_reset_static(ResetLaunch p, cudaStream_t stream) {
    RowScratch* scratch = nullptr;
    cudaError_t e = static_scratch(&scratch);
    if (e != cudaSuccess) return e;
    p.scratch = scratch;
    // Nothing in the scratch has to start at zero: the first kernel of a step rewrites
    // every field the later ones read (slice partials, and the arrival ticket is reset to
    // 0 by slice 0 of each row), so the previous call's contents are harmless.
    return launch_reset(p, true, stream);
}

}  // namespace nvfp4r
