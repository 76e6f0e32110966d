// Batch-1 decode-step scaffolding around the NVFP4 linears: the operators a Qwen3 decoder
// layer needs between two linears (residual add + RMSNorm, per-head q/k RMSNorm + rotary
// embedding + KV-cache write, GQA decode attention, SiLU*up, bf16 lm_head, arg-max).
// vLLM supplies these in the reference's deployment; they exist here so that the full
// decode step of the benchmark runs from one CUDA graph with nothing but this library's
// kernels and NCCL. bf16 activations, fp32 arithmetic.
#include <cuda_bf16.h>

#include "../../include/nvfp4r_b200.h"
#include "kernels.h"
#include "lm_head_dot.cuh"
#include "nvfp4_ptx.cuh"

namespace nvfp4r {
namespace {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
    return v;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float block_sum_f(float v, float* red) {      // blockDim multiple of 32
    v = warp_sum_f(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nw; ++w) t += red[w];
    return t;
}

// residual (+= x) ; out = residual * rsqrt(mean(residual^2) + eps) * weight. One CTA per row.
__global__ void __launch_bounds__(512)
add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out,
                   int H, float eps) {
    __shared__ float red[16];
    pdl_wait_prior();
    const int64_t row = blockIdx.x;
    constexpr int kMaxPerThread = 32;                          // H <= 512 * 32
    float keep[kMaxPerThread];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxPerThread; ++j) {
        const int i = threadIdx.x + j * 512;
        if (i < H) {
            float v = __bfloat162float(residual[row * H + i]);
            if (x != nullptr) {
                v = __bfloat162float(__float2bfloat16_rn(v + __bfloat162float(x[row * H + i])));
                residual[row * H + i] = __float2bfloat16_rn(v);   // the residual stream is bf16
            }
            keep[j] = v;
            ss += v * v;
        }
    }
    const float inv = rsqrtf(block_sum_f(ss, red) / static_cast<float>(H) + eps);
#pragma unroll
    for (int j = 0; j < kMaxPerThread; ++j) {
        const int i = threadIdx.x + j * 512;
        if (i < H) out[row * H + i] = __float2bfloat16_rn(keep[j] * inv * __bfloat162float(weight[i]));
    }
    pdl_launch_dependents();
}

// RMSNorm(head) * w followed by the rotary embedding (rotate-half pairs d, d + D/2) of one
// 128-wide head by one warp: lane holds dims lane, lane+32 (first half), lane+64, lane+96.
// `table` (optional): cos/sin of pos * theta^(-2d/D) as float2 [Tmax][D/2], prepared once by the
// host; without it the angles are computed here (powf + sincosf: a few hundred instructions
// that run once per launch).
__device__ __forceinline__ void head_norm_rope(const __nv_bfloat16* __restrict__ src,
                                               const __nv_bfloat16* __restrict__ w, int pos, float theta,
                                               float eps, int lane, float o[4],
                                               const float2* __restrict__ table = nullptr) {
    constexpr int D = 128;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(src[lane + 32 * j]);
    const float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    const float inv = rsqrtf(warp_sum_f(ss) / static_cast<float>(D) + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j)
        v[j] = __bfloat162float(__float2bfloat16_rn(v[j] * inv * __bfloat162float(w[lane + 32 * j])));
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int d = lane + 32 * j;                           // 0..63
        float sn, cs;
        if (table != nullptr) {
            const float2 t = __ldg(table + static_cast<int64_t>(pos) * (D / 2) + d);
            cs = t.x;
            sn = t.y;
        } else {
            const float freq = powf(theta, -static_cast<float>(2 * d) / static_cast<float>(D));
            sincosf(static_cast<float>(pos) * freq, &sn, &cs);
        }
        o[j] = v[j] * cs - v[j + 2] * sn;
        o[j + 2] = v[j + 2] * cs + v[j] * sn;
    }
}

// The same with the layer constants already in registers: wv = the four norm weights of this
// lane, cs/sn = cos and sin of its two rotary pairs. Only `src` is read here, so a caller that
// fetched the constants before its dependency wait pays one trip to L2 after it, not three.
__device__ __forceinline__ void head_norm_rope_pre(const __nv_bfloat16* __restrict__ src, const float wv[4],
                                                   const float cs[2], const float sn[2], float eps, int lane,
                                                   float o[4]) {
    constexpr int D = 128;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(src[lane + 32 * j]);
    const float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    const float inv = rsqrtf(warp_sum_f(ss) / static_cast<float>(D) + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j] * inv * wv[j]));
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        o[j] = v[j] * cs[j] - v[j + 2] * sn[j];
        o[j + 2] = v[j + 2] * cs[j] + v[j] * sn[j];
    }
}

// One warp per head of the fused qkv row: q and k heads get RMSNorm(head) * w and the
// rotary embedding (rotate-half pairs d, d + D/2); k and v are written to the cache at
// `*position`; q goes to q_out. D == 128.
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ q_w,
                       const __nv_bfloat16* __restrict__ k_w, const int* __restrict__ position,
                       __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                       __nv_bfloat16* __restrict__ q_out, int Hq, int Hkv, int Tmax, float theta,
                       float eps, const float2* __restrict__ table) {
    constexpr int D = 128;
    pdl_wait_prior();
    const int head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (head >= Hq + 2 * Hkv) return;
    const int pos = *position;
    const __nv_bfloat16* src = qkv + static_cast<int64_t>(head) * D;
    // lane holds dims lane, lane+32 (first half) and lane+64, lane+96 (second half)
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(src[lane + 32 * j]);
    if (head >= Hq + Hkv) {                                    // value head: plain copy
        __nv_bfloat16* dst = vcache + (static_cast<int64_t>(head - Hq - Hkv) * Tmax + pos) * D;
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = __float2bfloat16_rn(v[j]);
        return;
    }
    const bool is_q = head < Hq;
    float o[4];
    head_norm_rope(src, is_q ? q_w : k_w, pos, theta, eps, lane, o, table);
    __nv_bfloat16* dst = is_q ? q_out + static_cast<int64_t>(head) * D
                              : kcache + (static_cast<int64_t>(head - Hq) * Tmax + pos) * D;
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = __float2bfloat16_rn(o[j]);
    pdl_launch_dependents();
}

// GQA decode attention in ONE launch, split over the context. CTA (kv head, split) stages its
// chunk of K and V in shared memory once for the `group` (<= 8) query heads of that kv head and
// runs both products on the tensor cores (mma.sync m16n8k16, bf16 in, fp32 accumulate; the
// heads are the M rows of the tile, padded to 16):
//   warp w: S[heads, 16 positions] = Q K^T over its 16 positions of the chunk -> chunk-wide
//   max through shared memory -> P = exp(S - max) as bf16 in shared memory -> warp w:
//   O[heads, 16 dims] = P V over ALL positions of the chunk for its 16 output dims.
// The partial (max, sum, O[128]) per (q head, split) goes to scratch, and the last CTA of a kv
// head to arrive (atomic ticket, nothing waits) merges the partials of its heads.
// The cache rows of earlier tokens do not depend on the kernel that precedes this one, so they
// are fetched BEFORE griddepcontrol.wait; only the newest row (*seq_len - 1, written by
// qk_norm_rope_kv) and q are read after it. *seq_len itself must therefore be stable since
// before the preceding launch (it is step input, not a product of the layer).
constexpr int kAttnChunk = 128;                                // positions per CTA
constexpr int kAttnD = 128;
constexpr int kAttnPitch = kAttnD * 2 + 16;                    // bytes per staged row (bank skew, 16-byte aligned)
constexpr int kAttnRec = kAttnD + 4;                           // floats per partial record
constexpr int kAttnLoads = kAttnChunk * (kAttnD / 8) / 256;    // 16-byte units per thread per tensor
constexpr size_t kAttnSmem = (2 * kAttnChunk + 32) * kAttnPitch;   // K, V, Q (16 rows), P (16 rows)

__device__ __forceinline__ void ldsm_x4(uint32_t r[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t r[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// kFusedRope: `q` is the raw fused qkv row [(Hq + 2 Hkv) * 128]; the CTA applies the q/k head
// norms and the rotary embedding itself (what qk_norm_rope_kv does as a separate launch) and the
// CTA whose chunk holds the newest position appends the new K/V row to the caches.
struct AttnRope {
    const __nv_bfloat16* q_w;
    const __nv_bfloat16* k_w;
    float theta, eps;
    const float2* table;
};

template <bool kFusedRope>
__global__ void __launch_bounds__(256)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ kcache,
                   __nv_bfloat16* __restrict__ vcache, const int* __restrict__ seq_len,
                   float* __restrict__ scratch, unsigned* __restrict__ tickets,
                   __nv_bfloat16* __restrict__ out, int Hq, int Hkv, int Tmax, float scale, AttnRope rope) {
    extern __shared__ __align__(16) uint8_t sm[];
    uint8_t* ks = sm;
    uint8_t* vs = ks + kAttnChunk * kAttnPitch;
    uint8_t* qs = vs + kAttnChunk * kAttnPitch;                // bf16 [16][pitch], rows >= group unused
    uint8_t* pb = qs + 16 * kAttnPitch;                        // bf16 [16][pitch]: P over the chunk
    __shared__ float smax[8][8], ssum[8][8];                   // [warp][head]
    __shared__ int s_last;
    pdl_launch_dependents();
    const int kvh = blockIdx.x, split = blockIdx.y, n_splits = gridDim.y;
    const int group = Hq / Hkv;
    const int len = *seq_len;
    const int p0 = split * kAttnChunk;
    const int np = min(kAttnChunk, len - p0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qh = kvh * group + warp;                         // the head this warp merges at the end

    // stage the chunk: all loads of a thread are issued before the first store
    {
        uint4 kk[kAttnLoads], vv[kAttnLoads];
#pragma unroll
        for (int j = 0; j < kAttnLoads; ++j) {
            const int i = threadIdx.x + j * 256;
            const int r = i / (kAttnD / 8), u = i % (kAttnD / 8);
            if (r < np && p0 + r != len - 1) {
                const int64_t g = (static_cast<int64_t>(kvh) * Tmax + p0 + r) * kAttnD + u * 8;
                kk[j] = ldg_stream_16(kcache + g);
                vv[j] = ldg_stream_16(vcache + g);
            } else {
                kk[j] = make_uint4(0, 0, 0, 0);                // rows past the end: finite values (P is 0 there)
                vv[j] = kk[j];
            }
        }
#pragma unroll
        for (int j = 0; j < kAttnLoads; ++j) {
            const int i = threadIdx.x + j * 256;
            const int r = i / (kAttnD / 8), u = i % (kAttnD / 8);
            if (p0 + r != len - 1) {
                *reinterpret_cast<uint4*>(ks + r * kAttnPitch + u * 16) = kk[j];
                *reinterpret_cast<uint4*>(vs + r * kAttnPitch + u * 16) = vv[j];
            }
        }
    }
    // Fused rope: the head-norm weights and the rotary angles of position len - 1 are layer / step
    // constants, fetched (or computed) before the wait like the cache rows above.
    float wq[4] = {0.f, 0.f, 0.f, 0.f}, wk[4] = {0.f, 0.f, 0.f, 0.f}, rcs[2] = {1.f, 1.f}, rsn[2] = {0.f, 0.f};
    if (kFusedRope && np > 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            wq[j] = __bfloat162float(rope.q_w[lane + 32 * j]);
            wk[j] = __bfloat162float(rope.k_w[lane + 32 * j]);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int d = lane + 32 * j;
            if (rope.table != nullptr) {
                const float2 t = __ldg(rope.table + static_cast<int64_t>(len - 1) * (kAttnD / 2) + d);
                rcs[j] = t.x;
                rsn[j] = t.y;
            } else {
                const float freq = powf(rope.theta, -static_cast<float>(2 * d) / static_cast<float>(kAttnD));
                sincosf(static_cast<float>(len - 1) * freq, &rsn[j], &rcs[j]);
            }
        }
    }
    pdl_wait_prior();
    if (np > 0) {
        const int r = len - 1 - p0;                            // the newest row, if it is in this chunk
        if (!kFusedRope) {
            if (r >= 0 && r < np && threadIdx.x < 2 * (kAttnD / 8)) {
                const int u = threadIdx.x & (kAttnD / 8 - 1);
                const int64_t g = (static_cast<int64_t>(kvh) * Tmax + len - 1) * kAttnD + u * 8;
                if (threadIdx.x < kAttnD / 8)
                    *reinterpret_cast<uint4*>(ks + r * kAttnPitch + u * 16) = *reinterpret_cast<const uint4*>(kcache + g);
                else
                    *reinterpret_cast<uint4*>(vs + r * kAttnPitch + u * 16) = *reinterpret_cast<const uint4*>(vcache + g);
            }
            // q heads of this kv head: 16 rows x 16 units of 16 bytes, rows >= group zero
            const int r16 = threadIdx.x >> 4, u = threadIdx.x & 15;
            uint4 v4 = make_uint4(0, 0, 0, 0);
            if (r16 < group)
                v4 = *reinterpret_cast<const uint4*>(q + (static_cast<int64_t>(kvh) * group + r16) * kAttnD + u * 8);
            *reinterpret_cast<uint4*>(qs + r16 * kAttnPitch + u * 16) = v4;
        } else {
            // the row position is len - 1 (the token being decoded)
            if (warp < group) {
                float o[4];
                head_norm_rope_pre(q + static_cast<int64_t>(qh) * kAttnD, wq, rcs, rsn, rope.eps, lane, o);
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(qs + warp * kAttnPitch);
#pragma unroll
                for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = __float2bfloat16_rn(o[j]);
            }
            if (r >= 0 && r < np) {
                // new K row (warp 0) and V row (warp 1): into shared memory and into the caches
                const int64_t g = (static_cast<int64_t>(kvh) * Tmax + len - 1) * kAttnD;
                if (warp == 0) {
                    float o[4];
                    head_norm_rope_pre(q + static_cast<int64_t>(Hq + kvh) * kAttnD, wk, rcs, rsn, rope.eps, lane, o);
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(ks + r * kAttnPitch);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const __nv_bfloat16 b = __float2bfloat16_rn(o[j]);
                        dst[lane + 32 * j] = b;
                        kcache[g + lane + 32 * j] = b;
                    }
                } else if (warp == 1) {
                    const __nv_bfloat16* src = q + static_cast<int64_t>(Hq + Hkv + kvh) * kAttnD;
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(vs + r * kAttnPitch);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const __nv_bfloat16 b = src[lane + 32 * j];
                        dst[lane + 32 * j] = b;
                        vcache[g + lane + 32 * j] = b;
                    }
                }
            }
        }
    }
    __syncthreads();
    if (np > 0) {
        const uint32_t ks_a = smem_u32(ks), vs_a = smem_u32(vs), qs_a = smem_u32(qs), pb_a = smem_u32(pb);
        const int h = lane >> 2;                               // head row of this thread's c0/c1
        // ---- S = Q K^T for this warp's 16 positions -------------------------------------------
        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int kt = 0; kt < kAttnD / 16; kt += 2) {
            uint32_t a0[4], a1[4];
            ldsm_x4(a0, qs_a + (lane & 15) * kAttnPitch + kt * 32 + (lane >> 4) * 16);
            ldsm_x4(a1, qs_a + (lane & 15) * kAttnPitch + (kt + 1) * 32 + (lane >> 4) * 16);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                uint32_t b[4];                                 // {k 0-7, k 8-15} of kt, then of kt + 1
                ldsm_x4(b, ks_a + (16 * warp + 8 * nt + (lane & 7)) * kAttnPitch + kt * 32 + (lane >> 3) * 16);
                mma_bf16_16816(sc[nt], a0, b[0], b[1]);
                mma_bf16_16816(sc[nt], a1, b[2], b[3]);
            }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int pos = 16 * warp + 8 * nt + (lane & 3) * 2 + e;
                sc[nt][e] = (pos < np) ? sc[nt][e] * scale : -INFINITY;
                mx = fmaxf(mx, sc[nt][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        if ((lane & 3) == 0) smax[warp][h] = mx;
        __syncthreads();
        float m = smax[0][h];
#pragma unroll
        for (int w = 1; w < 8; ++w) m = fmaxf(m, smax[w][h]);
        // ---- P = exp(S - max) as bf16, and this warp's share of the sums ------------------------
        float sum = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const float e0 = __expf(sc[nt][0] - m), e1 = __expf(sc[nt][1] - m);     // exp(-inf) = 0
            const uint32_t pk = pack_bf16x2(e0, e1);
            // the sums use the rounded values, like the product below
            sum += __uint_as_float(pk << 16) + __uint_as_float(pk & 0xFFFF0000u);
            *reinterpret_cast<uint32_t*>(pb + h * kAttnPitch + (16 * warp + 8 * nt + (lane & 3) * 2) * 2) = pk;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((lane & 3) == 0) ssum[warp][h] = sum;
        __syncthreads();
        // ---- O[heads, 16 dims of this warp] = P V over the whole chunk -----------------------------
        float o[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int kt = 0; kt < kAttnChunk / 16; ++kt) {
            uint32_t a[4], b[4];
            ldsm_x4(a, pb_a + (lane & 15) * kAttnPitch + kt * 32 + (lane >> 4) * 16);
            // V rows are positions (k), columns are dims (n): transposed 8x8 loads give the col-major fragment
            ldsm_x4_trans(b, vs_a + (16 * kt + (lane & 7) + ((lane >> 3) & 1) * 8) * kAttnPitch +
                                 (16 * warp + (lane >> 4) * 8) * 2);
            mma_bf16_16816(o[0], a, b[0], b[1]);
            mma_bf16_16816(o[1], a, b[2], b[3]);
        }
        if (h < group) {
            float* rec = scratch + (static_cast<int64_t>(kvh * group + h) * n_splits + split) * kAttnRec;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
                __stcg(reinterpret_cast<float2*>(rec + 4 + 16 * warp + 8 * nt + (lane & 3) * 2),
                       make_float2(o[nt][0], o[nt][1]));
            if (warp == 0 && (lane & 3) == 0) {
                float tot = 0.0f;
#pragma unroll
                for (int w = 0; w < 8; ++w) tot += ssum[w][h];
                __stcg(reinterpret_cast<float2*>(rec), make_float2(m, tot));
            }
        }
    } else if (warp < group && lane == 0) {
        float* rec = scratch + (static_cast<int64_t>(qh) * n_splits + split) * kAttnRec;
        __stcg(reinterpret_cast<float2*>(rec), make_float2(-INFINITY, 0.0f));
    }
    // ticket: the barrier orders every warp's partial stores before thread 0's fence + atomic
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned t = atomicAdd(tickets + kvh, 1u);
        s_last = (t == static_cast<unsigned>(n_splits) - 1u) ? 1 : 0;
        if (s_last) tickets[kvh] = 0u;
        __threadfence();
    }
    __syncthreads();
    if (!s_last || warp >= group) return;
    // merge the splits of this warp's head: lane s owns the (max, sum) of split s0 + s, the
    // accumulator loads of a group of splits are independent of one another
    const float* base = scratch + static_cast<int64_t>(qh) * n_splits * kAttnRec;
    float mx = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) {
        const float2 ms = __ldcg(reinterpret_cast<const float2*>(base + s * kAttnRec));
        if (ms.y > 0.0f) mx = fmaxf(mx, ms.x);
    }
    mx = warp_max_f(mx);
    float denom = 0.0f, o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int s0 = 0; s0 < n_splits; s0 += 32) {
        float wgt = 0.0f;
        if (s0 + lane < n_splits) {
            const float2 ms = __ldcg(reinterpret_cast<const float2*>(base + (s0 + lane) * kAttnRec));
            if (ms.y > 0.0f) {
                wgt = __expf(ms.x - mx);
                denom += wgt * ms.y;
            }
        }
        const int cnt = min(32, n_splits - s0);
#pragma unroll 8
        for (int j = 0; j < cnt; ++j) {
            const float w = __shfl_sync(0xffffffffu, wgt, j);
            const float4 a = __ldcg(reinterpret_cast<const float4*>(base + (s0 + j) * kAttnRec + 4 + lane * 4));
            // a split without positions left its record unwritten: select, do not multiply
            o[0] += (w > 0.0f) ? w * a.x : 0.0f;
            o[1] += (w > 0.0f) ? w * a.y : 0.0f;
            o[2] += (w > 0.0f) ? w * a.z : 0.0f;
            o[3] += (w > 0.0f) ? w * a.w : 0.0f;
        }
    }
    denom = warp_sum_f(denom);
    const float inv = 1.0f / denom;
    const uint32_t lo = pack_bf16x2(o[0] * inv, o[1] * inv), hi = pack_bf16x2(o[2] * inv, o[3] * inv);
    *reinterpret_cast<uint2*>(out + static_cast<int64_t>(qh) * kAttnD + lane * 4) = make_uint2(lo, hi);
}

// out[m, i] = silu(gate_up[m, i]) * gate_up[m, I + i]
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int M, int I) {
    pdl_wait_prior();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<int64_t>(M) * I) return;
    const int64_t m = idx / I, i = idx % I;
    const float g = __bfloat162float(gate_up[m * 2 * I + i]);
    const float u = __bfloat162float(gate_up[m * 2 * I + I + i]);
    out[idx] = __float2bfloat16_rn(g / (1.0f + __expf(-g)) * u);
    pdl_launch_dependents();
}

// logits[v] = sum_h W[v, h] * x[h]; bf16 weight streamed once, one warp per row, x in
// shared memory as fp32. H % 256 == 0.
__global__ void __launch_bounds__(1024)
lm_head_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W,
               float* __restrict__ logits, int V, int H) {
    extern __shared__ __align__(16) float xs[];
    pdl_wait_prior();
    for (int i = threadIdx.x; i < H; i += blockDim.x) xs[i] = __bfloat162float(x[i]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = gridDim.x * (blockDim.x >> 5);
    for (int v = blockIdx.x * (blockDim.x >> 5) + warp; v < V; v += warps) {
        const uint4* row = reinterpret_cast<const uint4*>(W + static_cast<int64_t>(v) * H);
        float acc = lm_head_row_dot(row, xs, H / 8, lane);
        acc = warp_sum_f(acc);
        if (lane == 0) logits[v] = acc;
    }
    pdl_launch_dependents();
}

// Row arg-max (lowest index among equal values) in two stages: kArgmaxParts CTAs per row
// each reduce a slice into a (value, index) pair kept in a small static device array, then
// one CTA per row reduces the pairs.
constexpr int kArgmaxParts = 64;
constexpr int kArgmaxMaxRows = 256;
__device__ float g_argmax_val[kArgmaxMaxRows * kArgmaxParts];
__device__ int g_argmax_idx[kArgmaxMaxRows * kArgmaxParts];

__device__ __forceinline__ void argmax_block_reduce(float& best, int& arg, float* smax, int* sarg) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, s);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, s);
        if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { smax[warp] = best; sarg[warp] = arg; }
    __syncthreads();
    if (threadIdx.x == 0)
        for (int w = 1; w < (blockDim.x >> 5); ++w)
            if (smax[w] > best || (smax[w] == best && sarg[w] < arg)) { best = smax[w]; arg = sarg[w]; }
}

// Standard Gumbel noise -log(-log(u)) for element i of a row, from a counter-based generator:
// the 64-bit finalizer of splitmix64 over (key + i * odd constant), top 23 bits -> u in (0, 1).
// `key` already mixes the seed, the row and the row's draw counter, so every draw of every row
// uses its own stream and a replayed CUDA graph keeps drawing fresh numbers.
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float gumbel_noise(unsigned long long key, int i) {
    const unsigned long long r = mix64(key + static_cast<unsigned long long>(i) * 0x9E3779B97F4A7C15ull);
    // 23 bits: (x + 0.5) / 2^23 is exact in fp32 and stays strictly inside (0, 1)
    const float u = (static_cast<float>(static_cast<unsigned>(r >> 41)) + 0.5f) * (1.0f / 8388608.0f);
    return -logf(-logf(u));
}

// kGumbel: the slice's maximum of logits[i] + Gumbel noise (sampling from softmax(logits) by
// the Gumbel-max rule) instead of the plain maximum.
// Order-preserving map of a float onto an unsigned key (larger value, larger key): the top-k /
// top-p truncation selects on these keys with a radix descent.
__device__ __forceinline__ uint32_t sortable_key(float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Per-row state of the truncated sampler, in caller scratch (all zero before its first use;
// every call leaves the histograms zeroed again).
constexpr int kSampleBins = 2048;
struct SampleRow {
    unsigned long long mass[kSampleBins];   // fixed-point sum of exp(x - max) per bin
    unsigned int count[kSampleBins];
    unsigned long long above_mass;          // mass of the keys above the current prefix
    unsigned long long target_mass;         // top_p * (mass of the candidate set)
    unsigned long long set_mass;            // mass of the keys kept by top-k (candidate set of top-p)
    unsigned int above_count;
    unsigned int prefix;                    // the high bits selected so far
    unsigned int min_key;                   // candidates have key >= min_key (result of top-k)
    unsigned int thr_key;                   // final threshold: sample among key >= thr_key
    unsigned int all;                       // 1: truncation keeps everything left (no bin reached the target)
    unsigned int pad;
};

template <bool kGumbel>
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, int64_t row_stride, int V, unsigned long long seed,
                      const unsigned long long* __restrict__ draws, const SampleRow* __restrict__ trunc) {
    __shared__ float smax[8];
    __shared__ int sarg[8];
    pdl_wait_prior();
    const float* row = logits + blockIdx.y * row_stride;
    const int per = (V + kArgmaxParts - 1) / kArgmaxParts;
    const int lo = blockIdx.x * per, hi = min(V, lo + per);
    float best = -INFINITY;
    int arg = 0x7fffffff;
    unsigned long long key = 0;
    if (kGumbel)
        key = mix64(seed ^ mix64((static_cast<unsigned long long>(blockIdx.y) << 40) + draws[blockIdx.y]));
    const uint32_t thr = (kGumbel && trunc != nullptr) ? trunc[blockIdx.y].thr_key : 0u;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float v = row[i];
        if (kGumbel) {
            if (sortable_key(v) < thr) continue;           // outside the top-k / top-p set
            v += gumbel_noise(key, i);
        }
        if (v > best) { best = v; arg = i; }
    }
    argmax_block_reduce(best, arg, smax, sarg);
    if (threadIdx.x == 0) {
        g_argmax_val[blockIdx.y * kArgmaxParts + blockIdx.x] = best;
        g_argmax_idx[blockIdx.y * kArgmaxParts + blockIdx.x] = arg;
    }
    pdl_launch_dependents();
}

// draws / last_ids (sampling only, may be null): the row's draw counter advances by one and
// the row's pair of most recent ids is shifted with the new id appended.
__global__ void __launch_bounds__(64)
argmax_final_kernel(int* __restrict__ out, unsigned long long* __restrict__ draws, int* __restrict__ last_ids) {
    __shared__ float smax[2];
    __shared__ int sarg[2];
    pdl_wait_prior();
    float best = g_argmax_val[blockIdx.x * kArgmaxParts + threadIdx.x];
    int arg = g_argmax_idx[blockIdx.x * kArgmaxParts + threadIdx.x];
    argmax_block_reduce(best, arg, smax, sarg);
    if (threadIdx.x == 0) {
        // a row without any finite candidate (all -inf or NaN) yields id 0, never the sentinel
        if (arg == 0x7fffffff) arg = 0;
        out[blockIdx.x] = arg;
        if (draws != nullptr) draws[blockIdx.x] += 1ull;
        if (last_ids != nullptr) {
            last_ids[2 * blockIdx.x] = last_ids[2 * blockIdx.x + 1];
            last_ids[2 * blockIdx.x + 1] = arg;
        }
    }
}

// ---- top-k / top-p truncation: radix descent over the sortable keys ---------------------------
// Three levels (11 + 11 + 10 key bits). A level is two launches: sample_hist_kernel adds count and
// fixed-point probability mass of the keys that share the prefix found so far into 2048 bins,
// sample_select_kernel walks the bins from the top and picks the one in which the running count
// reaches k (top-k) or the running mass reaches top_p * (mass of the candidate set) (top-p),
// extends the prefix and zeroes the bins. After the last level the prefix IS the key of the last
// token kept; keys equal to it are all kept (ties are not split). Mass is exp(x - row max) scaled by
// 2^32 and truncated to an integer, summed with integer atomics: the result does not depend on the
// order of the additions, so the draw is reproducible.
__host__ __device__ constexpr int level_shift(int level) { return level == 0 ? 21 : (level == 1 ? 10 : 0); }
__host__ __device__ constexpr int level_bins(int level) { return level == 2 ? 1024 : 2048; }

__global__ void __launch_bounds__(256)
sample_hist_kernel(const float* __restrict__ logits, int64_t row_stride, int V, SampleRow* __restrict__ rows,
                   int level) {
    __shared__ unsigned long long s_mass[kSampleBins];
    __shared__ unsigned int s_cnt[kSampleBins];
    __shared__ float s_max;
    pdl_launch_dependents();
    pdl_wait_prior();
    SampleRow* r = rows + blockIdx.y;
    if (r->all) return;
    for (int i = threadIdx.x; i < kSampleBins; i += blockDim.x) { s_mass[i] = 0ull; s_cnt[i] = 0u; }
    if (threadIdx.x < 32) {
        float m = fmaxf(g_argmax_val[blockIdx.y * kArgmaxParts + threadIdx.x],
                        g_argmax_val[blockIdx.y * kArgmaxParts + 32 + threadIdx.x]);
        m = warp_max_f(m);
        if (threadIdx.x == 0) s_max = m;
    }
    __syncthreads();
    const float m = s_max;
    const float* row = logits + blockIdx.y * row_stride;
    const int per = (V + kArgmaxParts - 1) / kArgmaxParts;
    const int lo = blockIdx.x * per, hi = min(V, lo + per);
    const uint32_t prefix = r->prefix, min_key = r->min_key;
    const int shift = level_shift(level);
    const int prev_shift = level == 0 ? 31 : level_shift(level - 1);
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float x = row[i];
        if (!(x > -INFINITY)) continue;                               // -inf and NaN never enter the set
        const uint32_t key = sortable_key(x);
        if (key < min_key) continue;
        if (level > 0 && (key >> prev_shift) != prefix) continue;
        const int bin = static_cast<int>((key >> shift) & static_cast<uint32_t>(level_bins(level) - 1));
        const unsigned long long w = __float2ull_rd(__expf(x - m) * 4294967296.0f);
        atomicAdd(&s_mass[bin], w);
        atomicAdd(&s_cnt[bin], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kSampleBins; i += blockDim.x)
        if (s_cnt[i] != 0u) {
            atomicAdd(&r->mass[i], s_mass[i]);
            atomicAdd(&r->count[i], s_cnt[i]);
        }
}

// mode 0: top-k (by count, k > 0); mode 1: top-p (by mass). One CTA of 1024 threads per row, thread t
// owns bins 2047 - 2t and 2046 - 2t (descending order).
__global__ void __launch_bounds__(1024)
sample_select_kernel(SampleRow* __restrict__ rows, int level, int mode, int k, float top_p) {
    __shared__ unsigned long long s_wm[32], s_wc[32];
    __shared__ int s_pick;
    pdl_launch_dependents();
    pdl_wait_prior();
    SampleRow* r = rows + blockIdx.x;
    if (r->all) return;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int b0 = kSampleBins - 1 - 2 * t, b1 = b0 - 1;
    const unsigned long long m0 = r->mass[b0], m1 = r->mass[b1];
    const unsigned long long c0 = r->count[b0], c1 = r->count[b1];
    if (t == 0) s_pick = 0x7fffffff;
    // inclusive scan (descending bins) of mass and count over the block
    unsigned long long sm = m0 + m1, sc = c0 + c1;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long om = __shfl_up_sync(0xffffffffu, sm, d), oc = __shfl_up_sync(0xffffffffu, sc, d);
        if (lane >= d) { sm += om; sc += oc; }
    }
    if (lane == 31) { s_wm[warp] = sm; s_wc[warp] = sc; }
    __syncthreads();
    if (warp == 0) {
        unsigned long long wm = s_wm[lane], wc = s_wc[lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned long long om = __shfl_up_sync(0xffffffffu, wm, d), oc = __shfl_up_sync(0xffffffffu, wc, d);
            if (lane >= d) { wm += om; wc += oc; }
        }
        s_wm[lane] = wm;
        s_wc[lane] = wc;
    }
    __syncthreads();
    const unsigned long long base_m = warp > 0 ? s_wm[warp - 1] : 0ull, base_c = warp > 0 ? s_wc[warp - 1] : 0ull;
    const unsigned long long incl1_m = base_m + sm, incl1_c = base_c + sc;           // through bin b1
    const unsigned long long incl0_m = incl1_m - m1, incl0_c = incl1_c - c1;         // through bin b0
    const unsigned long long total_m = s_wm[31];
    unsigned long long target = r->target_mass;
    if (mode == 1 && level == 0) {
        // candidate set = everything counted at level 0 (the top-k set when top-k ran before)
        target = static_cast<unsigned long long>(ceil(static_cast<double>(top_p) * static_cast<double>(total_m)));
        if (target < 1ull) target = 1ull;
    }
    const unsigned long long am = r->above_mass;
    const unsigned int ac = r->above_count;
    auto reached = [&](unsigned long long im, unsigned long long ic) {
        return mode == 0 ? (ac + ic >= static_cast<unsigned long long>(k)) : (am + im >= target);
    };
    int mine = 0x7fffffff;                    // position in descending order of the first bin that reaches the goal
    if (c0 != 0ull && reached(incl0_m, incl0_c)) mine = 2 * t;
    else if (c1 != 0ull && reached(incl1_m, incl1_c)) mine = 2 * t + 1;
    if (mine != 0x7fffffff) atomicMin(&s_pick, mine);
    __syncthreads();
    const int pick = s_pick;
    // zero this level's bins for the next level / the next call
    r->mass[b0] = 0ull; r->mass[b1] = 0ull; r->count[b0] = 0u; r->count[b1] = 0u;
    if (pick == 0x7fffffff) {
        // the goal is never reached (fewer finite candidates than k): keep everything that is left
        if (t == 0) { r->all = 1u; r->thr_key = r->min_key; }
        return;
    }
    if (pick == 2 * t || pick == 2 * t + 1) {
        const bool first = pick == 2 * t;
        const int bin = first ? b0 : b1;
        const unsigned long long strictly_m = (first ? incl0_m - m0 : incl1_m - m1);
        const unsigned long long strictly_c = (first ? incl0_c - c0 : incl1_c - c1);
        const unsigned long long bin_m = first ? m0 : m1;
        const int bits = level == 2 ? 10 : 11;
        const unsigned int prefix = (level == 0 ? 0u : (r->prefix << bits)) | static_cast<unsigned int>(bin);
        r->prefix = prefix;
        r->above_mass = am + strictly_m;
        r->above_count = ac + static_cast<unsigned int>(strictly_c);
        if (mode == 1 && level == 0) r->target_mass = target;
        if (level == 2) {
            r->thr_key = prefix;
            if (mode == 0) {              // top-k done: its set is the candidate set of a following top-p
                r->min_key = prefix;
                r->set_mass = am + strictly_m + bin_m;
            }
            r->prefix = 0u; r->above_mass = 0ull; r->above_count = 0u; r->target_mass = 0ull;
        }
    }
}

// Start of a call (keep_set = 0: no truncation decided yet; the histograms are zero already) or
// of the top-p descent after top-k (keep_set = 1: the top-k set stays, the descent state restarts).
__global__ void sample_reset_kernel(SampleRow* __restrict__ rows, int keep_set) {
    pdl_launch_dependents();
    pdl_wait_prior();
    SampleRow* r = rows + blockIdx.x;
    if (threadIdx.x == 0) {
        r->above_mass = 0ull; r->target_mass = 0ull;
        r->above_count = 0u; r->prefix = 0u; r->all = 0u;
        if (!keep_set) { r->set_mass = 0ull; r->min_key = 0u; r->thr_key = 0u; }
    }
}

template <typename Kern, typename... Args>
cudaError_t launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gemv_tuning().use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

inline cudaStream_t st(void* s) { return static_cast<cudaStream_t>(s); }
inline int done(cudaError_t e) { return e == cudaSuccess ? NVFP4R_OK : NVFP4R_ERR_CUDA; }

}  // namespace
}  // namespace nvfp4r

using namespace nvfp4r;

// Optional rotary table of the current process (one device per process): set by
// nvfp4r_set_rope_table, read by the two rotary entry points.
static const float2* g_rope_table = nullptr;
static int g_rope_table_rows = 0;

extern "C" {

int nvfp4r_add_rmsnorm(const void* x, void* residual, const void* weight, void* out, int M, int H,
                       float eps, void* stream) {
    if (!residual || !weight || !out || M <= 0 || H <= 0) return NVFP4R_ERR_INVALID_ARGUMENT;
    if (H > 512 * 32) return NVFP4R_ERR_UNSUPPORTED_SHAPE;
    return done(launch_pdl(add_rmsnorm_kernel, dim3(M), dim3(512), 0, st(stream),
                           static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(residual),
                           static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out), H, eps));
}

int nvfp4r_qk_norm_rope_kv(const void* qkv, const void* q_weight, const void* k_weight,
                           const int32_t* position, void* kcache, void* vcache, void* q_out, int Hq,
                           int Hkv, int D, int Tmax, float theta, float eps, void* stream) {
    if (!qkv || !q_weight || !k_weight || !position || !kcache || !vcache || !q_out)
        return NVFP4R_ERR_INVALID_ARGUMENT;
    if (D != 128) return NVFP4R_ERR_UNSUPPORTED_SHAPE;
    const int heads = Hq + 2 * Hkv;
    return done(launch_pdl(qk_norm_rope_kv_kernel, dim3((heads + 3) / 4), dim3(128), 0, st(stream),
                           static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(q_weight),
                           static_cast<const __nv_bfloat16*>(k_weight), position,
                           static_cast<__nv_bfloat16*>(kcache), static_cast<__nv_bfloat16*>(vcache),
                           static_cast<__nv_bfloat16*>(q_out), Hq, Hkv, Tmax, theta, eps,
                           (g_rope_table != nullptr && g_rope_table_rows >= Tmax) ? g_rope_table : nullptr));
}

int nvfp4r_set_rope_table(const float* cos_sin, int rows) {
    if (cos_sin != nullptr && rows <= 0) return NVFP4R_ERR_INVALID_ARGUMENT;
    g_rope_table = reinterpret_cast<const float2*>(cos_sin);
    g_rope_table_rows = cos_sin ? rows : 0;
    return NVFP4R_OK;
}

size_t nvfp4r_attn_decode_workspace_bytes(int Hq, int Tmax) {
    const size_t splits = (static_cast<size_t>(Tmax) + kAttnChunk - 1) / kAttnChunk;
    // partial records, then one ticket per kv head (at most Hq of them)
    return static_cast<size_t>(Hq) * splits * kAttnRec * sizeof(float) + static_cast<size_t>(Hq) * sizeof(unsigned);
}

static int attn_launch(bool fused, const void* q, void* kcache, void* vcache, const int32_t* seq_len, void* out,
                       int Hq, int Hkv, int D, int Tmax, void* workspace, size_t workspace_bytes, AttnRope rope,
                       void* stream) {
    if (!q || !kcache || !vcache || !seq_len || !out || !workspace) return NVFP4R_ERR_INVALID_ARGUMENT;
    if (D != 128 || Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > 8) return NVFP4R_ERR_UNSUPPORTED_SHAPE;
    if (workspace_bytes < nvfp4r_attn_decode_workspace_bytes(Hq, Tmax)) return NVFP4R_ERR_INVALID_ARGUMENT;
    const int splits = (Tmax + kAttnChunk - 1) / kAttnChunk;
    if (splits > 65535) return NVFP4R_ERR_UNSUPPORTED_SHAPE;
    float* records = static_cast<float*>(workspace);
    unsigned* tickets = reinterpret_cast<unsigned*>(records + static_cast<size_t>(Hq) * splits * kAttnRec);
    auto kern = fused ? attn_decode_kernel<true> : attn_decode_kernel<false>;
    static bool attr_done[2][64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return NVFP4R_ERR_CUDA;
    if (dev >= 0 && dev < 64 && !attr_done[fused ? 1 : 0][dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kAttnSmem)) != cudaSuccess) return NVFP4R_ERR_CUDA;
        attr_done[fused ? 1 : 0][dev] = true;
    }
    return done(launch_pdl(kern, dim3(Hkv, splits), dim3(256), kAttnSmem, st(stream),
                           static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(kcache),
                           static_cast<__nv_bfloat16*>(vcache), seq_len, records, tickets,
                           static_cast<__nv_bfloat16*>(out), Hq, Hkv, Tmax, rsqrtf(static_cast<float>(D)), rope));
}

int nvfp4r_attn_decode(const void* q, const void* kcache, const void* vcache, const int32_t* seq_len,
                       void* out, int Hq, int Hkv, int D, int Tmax, void* workspace,
                       size_t workspace_bytes, void* stream) {
    return attn_launch(false, q, const_cast<void*>(kcache), const_cast<void*>(vcache), seq_len, out, Hq, Hkv, D,
                       Tmax, workspace, workspace_bytes, AttnRope{nullptr, nullptr, 0.0f, 0.0f, nullptr}, stream);
}

int nvfp4r_attn_decode_rope(const void* qkv, const void* q_weight, const void* k_weight, void* kcache,
                            void* vcache, const int32_t* seq_len, void* out, int Hq, int Hkv, int D, int Tmax,
                            float theta, float eps, void* workspace, size_t workspace_bytes, void* stream) {
    if (!q_weight || !k_weight) return NVFP4R_ERR_INVALID_ARGUMENT;
    return attn_launch(true, qkv, kcache, vcache, seq_len, out, Hq, Hkv, D, Tmax, workspace, workspace_bytes,
                       AttnRope{static_cast<const __nv_bfloat16*>(q_weight),
                                static_cast<const __nv_bfloat16*>(k_weight), theta, eps,
                                (g_rope_table != nullptr && g_rope_table_rows >= Tmax) ? g_rope_table : nullptr},
                       stream);
}

int nvfp4r_silu_mul(const void* gate_up, void* out, int M, int I, void* stream) {
    if (!gate_up || !out || M <= 0 || I <= 0) return NVFP4R_ERR_INVALID_ARGUMENT;
    const int64_t total = static_cast<int64_t>(M) * I;
    return done(launch_pdl(silu_mul_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0,
                           st(stream), static_cast<const __nv_bfloat16*>(gate_up),
                           static_cast<__nv_bfloat16*>(out), M, I));
}

int nvfp4r_lm_head(const void* x, const void* weight, float* logits, int V, int H, void* stream) {
    if (!x || !weight || !logits || V <= 0 || H <= 0) return NVFP4R_ERR_INVALID_ARGUMENT;
    if (H % 256 != 0 || H > 12288) return NVFP4R_ERR_UNSUPPORTED_SHAPE;
    const int grid = device_sm_count();
    // One CTA of 32 warps per SM, enforced through the shared-memory request: at 32 registers per
    // thread two such CTAs fit on an SM, and in a chain of launches some SMs then get two and
    // others none (measured on the 1.56 GB weight of Qwen3-32B: 383 us; four CTAs of 8 warps per
    // SM: 277 us; this form: 246 us).
    constexpr size_t kExclusiveSmem = 120 * 1024;
    static bool attr_done[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return NVFP4R_ERR_CUDA;
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        if (cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kExclusiveSmem)) != cudaSuccess)
            return NVFP4R_ERR_CUDA;
        attr_done[dev] = true;
    }
    return done(launch_pdl(lm_head_kernel, dim3(grid), dim3(1024), kExclusiveSmem, st(stream),
                           static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight),
                           logits, V, H));
}

int nvfp4r_argmax(const float* logits, int64_t row_stride, int B, int V, int32_t* out, void* stream) {
    if (!logits || !out || B <= 0 || V <= 0) return NVFP4R_ERR_INVALID_ARGUMENT;
    if (B > kArgmaxMaxRows) return NVFP4R_ERR_UNSUPPORTED_SHAPE;
    cudaError_t e = launch_pdl(argmax_partial_kernel<false>, dim3(kArgmaxParts, B), dim3(256), 0, st(stream), logits,
                               row_stride, V, 0ull, static_cast<const unsigned long long*>(nullptr),
                               static_cast<const SampleRow*>(nullptr));
    if (e != cudaSuccess) return NVFP4R_ERR_CUDA;
    return done(launch_pdl(argmax_final_kernel, dim3(B), dim3(kArgmaxParts), 0, st(stream), out,
                           static_cast<unsigned long long*>(nullptr), static_cast<int*>(nullptr)));
}

int nvfp4r_sample(const float* logits, int64_t row_stride, int B, int V, uint64_t seed, uint64_t* draws,
                  int32_t* last_ids, int32_t* out, void* stream) {
    if (!logits || !out || !draws || B <= 0 || V <= 0) return NVFP4R_ERR_INVALID_ARGUMENT;
    if (B > kArgmaxMaxRows) return NVFP4R_ERR_UNSUPPORTED_SHAPE;
    cudaError_t e = launch_pdl(argmax_partial_kernel<true>, dim3(kArgmaxParts, B), dim3(256), 0, st(stream), logits,
                               row_stride, V, static_cast<unsigned long long>(seed),
                               reinterpret_cast<const unsigned long long*>(draws),
                               static_cast<const SampleRow*>(nullptr));
    if (e != cudaSuccess) return NVFP4R_ERR_CUDA;
    return done(launch_pdl(argmax_final_kernel, dim3(B), dim3(kArgmaxParts), 0, st(stream), out,
                           reinterpret_cast<unsigned long long*>(draws), last_ids));
}

size_t nvfp4r_sample_workspace_bytes(int B) {
    return B > 0 ? static_cast<size_t>(B) * sizeof(SampleRow) : 0;
}

int nvfp4r_sample_top_k_top_p(const float* logits, int64_t row_stride, int B, int V, int top_k, float top_p,
                              uint64_t seed, uint64_t* draws, int32_t* last_ids, int32_t* out,
                              void* workspace, size_t workspace_bytes, void* stream) {
    if (!logits || !out || !draws || B <= 0 || V <= 0) return NVFP4R_ERR_INVALID_ARGUMENT;
    if (B > kArgmaxMaxRows) return NVFP4R_ERR_UNSUPPORTED_SHAPE;
    if (!(top_p > 0.0f)) return NVFP4R_ERR_INVALID_ARGUMENT;
    const bool use_k = top_k > 0 && top_k < V, use_p = top_p < 1.0f;
    if (!use_k && !use_p) return nvfp4r_sample(logits, row_stride, B, V, seed, draws, last_ids, out, stream);
    if (!workspace || workspace_bytes < nvfp4r_sample_workspace_bytes(B) ||
        (reinterpret_cast<uintptr_t>(workspace) & 7))
        return NVFP4R_ERR_INVALID_ARGUMENT;
    SampleRow* rows = static_cast<SampleRow*>(workspace);
    // row maxima (the partial maxima stay in the arg-max scratch, which the histogram kernels read)
    cudaError_t e = launch_pdl(argmax_partial_kernel<false>, dim3(kArgmaxParts, B), dim3(256), 0, st(stream), logits,
                               row_stride, V, 0ull, static_cast<const unsigned long long*>(nullptr),
                               static_cast<const SampleRow*>(nullptr));
    if (e == cudaSuccess) e = launch_pdl(sample_reset_kernel, dim3(B), dim3(32), 0, st(stream), rows, 0);
    for (int mode = 0; mode < 2 && e == cudaSuccess; ++mode) {
        if ((mode == 0 && !use_k) || (mode == 1 && !use_p)) continue;
        if (mode == 1 && use_k) e = launch_pdl(sample_reset_kernel, dim3(B), dim3(32), 0, st(stream), rows, 1);
        for (int level = 0; level < 3 && e == cudaSuccess; ++level) {
            e = launch_pdl(sample_hist_kernel, dim3(kArgmaxParts, B), dim3(256), 0, st(stream), logits, row_stride, V,
                           rows, level);
            if (e == cudaSuccess)
                e = launch_pdl(sample_select_kernel, dim3(B), dim3(1024), 0, st(stream), rows, level, mode, top_k, top_p);
        }
    }
    if (e == cudaSuccess)
        e = launch_pdl(argmax_partial_kernel<true>, dim3(kArgmaxParts, B), dim3(256), 0, st(stream), logits, row_stride,
                       V, static_cast<unsigned long long>(seed), reinterpret_cast<const unsigned long long*>(draws),
                       static_cast<const SampleRow*>(rows));
    if (e != cudaSuccess) return NVFP4R_ERR_CUDA;
    return done(launch_pdl(argmax_final_kernel, dim3(B), dim3(kArgmaxParts), 0, st(stream), out,
                           reinterpret_cast<unsigned long long*>(draws), last_ids));
}

}  // extern "C"
