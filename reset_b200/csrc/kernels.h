// Internal launch interface between the C ABI (api.cu) and the kernel files.
#pragma once

#include "../../include/nvfp4r_b200.h"

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
    // Fused producer of the activation (register-resident kernel, one token): 0 none,
    // 1 add + RMSNorm (xb unused), 2 SiLU * up (xb = [M, 2K] gate|up). Same arithmetic and
    // roundings as the packed linear's prologues.
    int pro_kind;
    const void* delta;
    const void* residual_in;
    void* residual_out;
    const void* norm_w;
    float eps;
    // Row-parallel shard of a tensor-parallel layer (ring kernel, one token, bf16 out): the lane that
    // finishes a pair of rows stores it into every rank's receive memory (layout and protocol of
    // peer_allreduce.cu), then sums the ranks' contributions to that pair out of its own receive
    // memory into `out`: the all-reduce inside the GEMV's launch. push_world <= 1: plain store.
    int push_world, push_rank;
    unsigned long long push_max_pairs;
    unsigned char* push_base[NVFP4R_PEER_MAX_WORLD];
    uint32_t push_poll_limit;
};

// True when the streaming (bulk-copy ring) kernel can take these arguments.
bool gemv_stream_supported(const GemvArgs& a);
cudaError_t launch_gemv_stream(const GemvArgs& a, cudaStream_t stream);
cudaError_t launch_gemv_generic(const GemvArgs& a, cudaStream_t stream);

// The register-resident kernel for one or two tokens (gemv_rows.cu).
bool gemv_rows_supported(const GemvArgs& a);
cudaError_t launch_gemv_rows(const GemvArgs& a, cudaStream_t stream);
// mode: 0 automatic, 1 whenever supported, -1 never; rows per step 0 (automatic), 2 or 4;
// warps per SM 0 (automatic) .. 32.
void set_gemv_rows_tuning(int mode, int rows, int target_warps);
// Picks the kernel for one launch of at most 8 tokens and launches it.
cudaError_t launch_gemv_auto(const GemvArgs& a, cudaStream_t stream);

// Tuning knobs of the streaming kernel (process-wide; 0 = built-in default).
struct GemvTuning {
    int ctas_per_sm;   // grid = SMs * ctas_per_sm
    int use_pdl;       // launch with programmatic stream serialization
    int force_generic; // route everything to the generic kernel (tests)
};
GemvTuning& gemv_tuning();

// ---- gemm_tcgen05.cu ------------------------------------------------------
// One NVFP4 weight [N,K/2] (+ swizzled scales) against M activation rows, either
// bf16 rows quantized on the fly (xb) or pre-quantized codes + swizzled scales.
struct TcLinearArgs {
    const void* w;               // [N, K/2] weight codes
    const void* wsf_swizzled;    // 128x4-tiled weight scales
    const void* xb;              // bf16 [M, K] (fused quantizer) or nullptr
    int64_t xb_stride;           // elements
    const float* gs;
    int rcp_mode;
    const void* a_codes;         // [M, K/2] when xb == nullptr
    const void* a_sf_swizzled;
    void* out;
    int out_dtype;
    bool c_n_major;              // element (m,n) at out[n*M + m] instead of out[m*N + n]
    int M, N, K;
    float alpha;
    void* workspace;
};
size_t gemm_workspace_bytes(int M, int N, int K);
// `*why` is set (and cudaSuccess returned) when the shape is outside what the
// kernel handles.
cudaError_t launch_linear_tc(const TcLinearArgs& g, cudaStream_t stream, const char** why);
cudaError_t read_and_clear_tc_status(int* flag);
// 0 = automatic
void set_tc_tuning(int splits, int stages);

// ---- linear_packed.cu -----------------------------------------------------
struct PackedLinearArgs {
    const void* packed;          // weight in the packed block format
    const void* xb;              // bf16 [M, K]
    int64_t xb_stride;
    const float* gs;
    int rcp_mode;
    void* out;                   // [M, N]
    int out_dtype;
    int M, N, K;
    float alpha;
    void* workspace;
    // fused prologue: 0 none, 1 add + RMSNorm, 2 SiLU * up
    int pro_kind;
    const void* delta;
    const void* residual_in;
    void* residual_out;
    const void* norm_w;
    float eps;
    // epilogue: push the bf16 result into the peers' receive memory instead of writing `out`
    const nvfp4r_peer_comm* push;
    bool push_gather;            // finish the all-reduce inside the launch (see nvfp4r_prologue)
};
size_t packed_weight_bytes(int N, int K);
size_t packed_workspace_bytes(int M, int N, int K);
cudaError_t launch_pack_weight(const void* w, const void* sf_flat, void* packed, int N, int K,
                               cudaStream_t stream);
cudaError_t launch_linear_packed(const PackedLinearArgs& g, cudaStream_t stream, const char** why);
cudaError_t read_and_clear_packed_status(int* flag);
void set_packed_tuning(int splits);
#ifdef NVFP4R_TRACE
cudaError_t read_packed_trace(unsigned long long* out16);
#endif

// Synchronises the device, returns the time-out flag set by bounded waits
// inside the kernels and clears it.
cudaError_t read_and_clear_device_status(int* flag);

cudaError_t read_and_clear_peer_status(int* flag);
uint32_t peer_poll_limit();      // polls a wait for a peer GPU may take (nvfp4r_set_peer_poll_limit)
cudaError_t read_and_clear_reset_status(int* flag);
cudaError_t read_and_clear_head_status(int* flag);

// Pinned-host twin of the time-out flags: one setter per kernel file (status_mirror.cuh).
cudaError_t set_status_mirror_gemv(int* device_ptr);
cudaError_t set_status_mirror_tc(int* device_ptr);
cudaError_t set_status_mirror_packed(int* device_ptr);
cudaError_t set_status_mirror_peer(int* device_ptr);
cudaError_t set_status_mirror_reset(int* device_ptr);
cudaError_t set_status_mirror_head(int* device_ptr);

int device_sm_count();

}  // namespace nvfp4r
