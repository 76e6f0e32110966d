// Per-block (16 element) NVFP4 quantisation arithmetic shared by the stand-alone
// quantizer and the fused decode linear. One thread quantizes one block.
#pragma once

#include "nvfp4_ptx.cuh"

namespace nvfp4r {

enum RcpMode : int { kRcpExact = 0, kRcpApprox = 1 };

__device__ __forceinline__ float rcp_approx_ftz(float v) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}

// Per-launch constants derived from the layer's global scale.
struct QuantScales {
    float gs;       // input_global_scale_inv
    float gs_rcp;   // 1 / gs in the selected arithmetic
    float inv6;     // 1 / 6 in the selected arithmetic
};

template <int kMode>
__device__ __forceinline__ QuantScales make_quant_scales(float gs) {
    QuantScales q;
    q.gs = gs;
    if (kMode == kRcpExact) {
        q.gs_rcp = __fdiv_rn(1.0f, gs);
        q.inv6 = 0.16666667163372039794921875f;   // float32 nearest to 1/6
    } else {
        q.gs_rcp = rcp_approx_ftz(gs);
        q.inv6 = rcp_approx_ftz(6.0f);
    }
    return q;
}

// v: 16 bf16 values as two 16-byte vectors (elements 0-7, 8-15).
// Returns the e4m3 scale byte; codes[0] = elements 0-7, codes[1] = 8-15.
//   amax = max|x| ; s = gs*(amax*inv6) clamped to 448 ; sf = e4m3_rne(s)
//   r = sf == 0 ? 0 : 1/(float(sf)*gs_rcp) ; code_i = e2m1_rne(sat6(x_i*r))
// `exact` selects the reciprocal: IEEE division (kRcpExact) or rcp.approx.ftz (kRcpApprox);
// `q` must have been made for the same mode.
__device__ __forceinline__ uint32_t quantize_block16_rt(const uint4& lo, const uint4& hi,
                                                        const QuantScales& q, bool exact, uint32_t codes[2]) {
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    float f[16];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        // bf16 -> f32 is a 16-bit shift
        f[2 * i]     = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        amax = fmaxf(amax, fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1])));
    }
    float s = __fmul_rn(q.gs, __fmul_rn(amax, q.inv6));
    s = fminf(s, 448.0f);
    const uint32_t sf_byte = f32_to_e4m3(s);
    const float sf = e4m3_to_f32(sf_byte);
    const float denom = __fmul_rn(sf, q.gs_rcp);
    float r;
    if (exact) r = (denom == 0.0f) ? 0.0f : __fdiv_rn(1.0f, denom);
    else r = (sf != 0.0f) ? rcp_approx_ftz(denom) : 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = __fmul_rn(f[i], r);
    codes[0] = f32x8_to_e2m1x8(&f[0]);
    codes[1] = f32x8_to_e2m1x8(&f[8]);
    return sf_byte;
}

template <int kMode>
__device__ __forceinline__ uint32_t quantize_block16(const uint4& lo, const uint4& hi,
                                                     const QuantScales& q, uint32_t codes[2]) {
    return quantize_block16_rt(lo, hi, q, kMode == kRcpExact, codes);
}

// Byte offset of scale (row, col) in the 128x4-tiled layout with `cols_padded`
// scale columns per row (a multiple of 4).
__device__ __host__ __forceinline__ int64_t swizzled_sf_offset(int row, int col, int cols_padded) {
    const int64_t tile = static_cast<int64_t>(row / 128) * (cols_padded / 4) + col / 4;
    const int r = row % 128;
    return tile * 512 + (r % 32) * 16 + (r / 32) * 4 + (col % 4);
}

}  // namespace nvfp4r
