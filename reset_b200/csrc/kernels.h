// Internal launch interface between the C ABI (api.cu) and the kernel files.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace nvfp4r {

// ---- quant.cu -------------------------------------------------------------
cudaError_t launch_quant(const void* x, int64_t x_row_stride, int M, int K, const float* gs,
                         void* codes, void* scales, bool swizzled, int rcp_mode,
                         cudaStream_t stream);
cudaError_t launch_sf_layout(const void* src, void* dst, int rows, int K, bool to_flat,
                             cudaStream_t stream);

// ---- gemv.cu --------------------------------------------------------------
// One weight [N,K/2] + [N,K/16] against M tokens. Either pre-quantized tokens
// (x/xsf with byte strides between tokens) or bf16 tokens quantized on the fly
// (xb/gs). Row strides of the weight are in bytes.
struct GemvArgs {
    const uint8_t* w;
    const uint8_t* wsf;
    int64_t w_stride_n;
    int64_t wsf_stride_n;
    const uint8_t* x;        // pre-quantized path (xb == nullptr)
    const uint8_t* xsf;
    int64_t x_stride;
    int64_t xsf_stride;
    const void* xb;          // fused path: bf16 tokens
    int64_t xb_stride;       // elements
    const float* gs;         // device scalar input_global_scale_inv
    int rcp_mode;
    void* out;
    int64_t out_stride;      // elements between tokens
    int out_dtype;
    int N, K, M;
    float alpha;
};

// True when the streaming (bulk-copy ring) kernel can take these arguments.
bool gemv_stream_supported(const GemvArgs& a);
cudaError_t launch_gemv_stream(const GemvArgs& a, cudaStream_t stream);
cudaError_t launch_gemv_generic(const GemvArgs& a, cudaStream_t stream);

// Tuning knobs of the streaming kernel (process-wide; 0 = built-in default).
struct GemvTuning {
    int ctas_per_sm;   // grid = SMs * ctas_per_sm
    int use_pdl;       // launch with programmatic stream serialization
    int force_generic; // route everything to the generic kernel (tests)
};
GemvTuning& gemv_tuning();

// ---- gemm_tcgen05.cu ------------------------------------------------------
struct GemmArgs {
    const void* A;      // [M, K/2] activation codes
    const void* B;      // [N, K/2] weight codes
    const void* SFA;    // swizzled activation scales
    const void* SFB;    // swizzled weight scales
    void* C;
    int M, N, K;
    float alpha;
    int out_dtype;
    bool c_n_major;
    void* workspace;
};
size_t gemm_workspace_bytes(int M, int N);
// `*why` is set (and cudaSuccess returned) when the shape is outside what the
// kernel handles.
cudaError_t launch_gemm(const GemmArgs& g, cudaStream_t stream, const char** why);

// Synchronises the device, returns the time-out flag set by bounded waits
// inside the kernels and clears it.
cudaError_t read_and_clear_device_status(int* flag);

int device_sm_count();

}  // namespace nvfp4r
