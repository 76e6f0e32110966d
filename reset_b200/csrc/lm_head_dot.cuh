// Dot product of one bf16 weight row with the fp32 activation row in shared memory, one warp
// per row: the inner loop of the vocabulary projection, shared by lm_head_kernel and
// lm_head_reset_kernel so that both produce the same bits. Four 16-byte streaming loads per lane
// are issued before any arithmetic (64 KB in flight per SM at 1024 threads).
#pragma once

#include "nvfp4_ptx.cuh"

namespace nvfp4r {

__device__ __forceinline__ float lm_head_fma8(const uint4& w, const float* xs8, float acc) {
    const float4 a = *reinterpret_cast<const float4*>(xs8);
    const float4 b = *reinterpret_cast<const float4*>(xs8 + 4);
    acc += __uint_as_float(w.x << 16) * a.x + __uint_as_float(w.x & 0xFFFF0000u) * a.y;
    acc += __uint_as_float(w.y << 16) * a.z + __uint_as_float(w.y & 0xFFFF0000u) * a.w;
    acc += __uint_as_float(w.z << 16) * b.x + __uint_as_float(w.z & 0xFFFF0000u) * b.y;
    acc += __uint_as_float(w.w << 16) * b.z + __uint_as_float(w.w & 0xFFFF0000u) * b.w;
    return acc;
}

// `units` = H / 8 (16-byte units per row). Returns this lane's partial sum.
__device__ __forceinline__ float lm_head_row_dot(const uint4* __restrict__ row, const float* xs, int units, int lane) {
    float acc = 0.0f;
    int u = lane;
#pragma unroll 1
    for (; u + 96 < units; u += 128) {
        uint4 w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = ldg_stream_16(row + u + 32 * j);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc = lm_head_fma8(w[j], xs + (u + 32 * j) * 8, acc);
    }
#pragma unroll 1
    for (; u < units; u += 32) acc = lm_head_fma8(ldg_stream_16(row + u), xs + u * 8, acc);
    return acc;
}

}  // namespace nvfp4r
