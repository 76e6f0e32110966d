// Stand-alone activation quantizer and block-scale layout conversion kernels.
#include "kernels.h"
#include "quant_core.cuh"

namespace nvfp4r {
namespace {

template <int kMode, bool kSwizzled>
__global__ void __launch_bounds__(128)
quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_row_stride, int M, int K,
             const float* __restrict__ gs_ptr, uint8_t* __restrict__ codes,
             uint8_t* __restrict__ scales, int rows_out, int cols_out) {
    pdl_wait_prior();
    const int cols = K / kBlockElems;
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<int64_t>(rows_out) * cols_out) return;
    const int row = static_cast<int>(idx / cols_out);
    const int col = static_cast<int>(idx % cols_out);
    if (row >= M || col >= cols) {            // padding of the swizzled layout
        if (kSwizzled) scales[swizzled_sf_offset(row, col, cols_out)] = 0;
        return;
    }
    const QuantScales q = make_quant_scales<kMode>(__ldg(gs_ptr));
    const uint4* src = reinterpret_cast<const uint4*>(x + row * x_row_stride + col * kBlockElems);
    const uint4 lo = __ldg(src), hi = __ldg(src + 1);
    uint32_t c[2];
    const uint32_t sf = quantize_block16<kMode>(lo, hi, q, c);
    *reinterpret_cast<uint2*>(codes + (static_cast<int64_t>(row) * K) / 2 + col * 8) =
        make_uint2(c[0], c[1]);
    const int64_t so = kSwizzled ? swizzled_sf_offset(row, col, cols_out)
                                 : static_cast<int64_t>(row) * cols + col;
    scales[so] = static_cast<uint8_t>(sf);
    pdl_launch_dependents();
}

template <bool kToFlat>
__global__ void __launch_bounds__(256)
sf_layout_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                 int rows, int cols, int rows_padded, int cols_padded) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (kToFlat) {
        if (idx >= static_cast<int64_t>(rows) * cols) return;
        const int r = static_cast<int>(idx / cols), c = static_cast<int>(idx % cols);
        dst[idx] = src[swizzled_sf_offset(r, c, cols_padded)];
    } else {
        if (idx >= static_cast<int64_t>(rows_padded) * cols_padded) return;
        const int r = static_cast<int>(idx / cols_padded), c = static_cast<int>(idx % cols_padded);
        const uint8_t v = (r < rows && c < cols) ? src[static_cast<int64_t>(r) * cols + c] : 0;
        dst[swizzled_sf_offset(r, c, cols_padded)] = v;
    }
}

}  // namespace

cudaError_t launch_quant(const void* x, int64_t x_row_stride, int M, int K, const float* gs,
                         void* codes, void* scales, bool swizzled, int rcp_mode,
                         cudaStream_t stream) {
    const int cols = K / kBlockElems;
    const int rows_out = swizzled ? (M + 127) / 128 * 128 : M;
    const int cols_out = swizzled ? (cols + 3) / 4 * 4 : cols;
    const int64_t total = static_cast<int64_t>(rows_out) * cols_out;
    const int threads = 128;
    const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
    auto xb = static_cast<const __nv_bfloat16*>(x);
    auto c = static_cast<uint8_t*>(codes);
    auto s = static_cast<uint8_t*>(scales);
#define NVFP4R_LAUNCH_Q(MODE, SW) \
    quant_kernel<MODE, SW><<<blocks, threads, 0, stream>>>(xb, x_row_stride, M, K, gs, c, s, rows_out, cols_out)
    if (rcp_mode == kRcpExact) { if (swizzled) NVFP4R_LAUNCH_Q(kRcpExact, true); else NVFP4R_LAUNCH_Q(kRcpExact, false); }
    else                       { if (swizzled) NVFP4R_LAUNCH_Q(kRcpApprox, true); else NVFP4R_LAUNCH_Q(kRcpApprox, false); }
#undef NVFP4R_LAUNCH_Q
    return cudaGetLastError();
}

cudaError_t launch_sf_layout(const void* src, void* dst, int rows, int K, bool to_flat,
                             cudaStream_t stream) {
    const int cols = K / kBlockElems;
    const int rp = (rows + 127) / 128 * 128, cp = (cols + 3) / 4 * 4;
    const int64_t total = to_flat ? static_cast<int64_t>(rows) * cols : static_cast<int64_t>(rp) * cp;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    if (to_flat)
        sf_layout_kernel<true><<<blocks, 256, 0, stream>>>(
            static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, cols, rp, cp);
    else
        sf_layout_kernel<false><<<blocks, 256, 0, stream>>>(
            static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, cols, rp, cp);
    return cudaGetLastError();
}

}  // namespace nvfp4r
