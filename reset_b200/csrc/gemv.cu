// NVFP4 W4A4 small-M GEMV for sm_100a.
//
// Two kernels:
//   * gemv_stream_kernel - the product path. Every warp runs a private ring of
//     shared-memory slots that it fills itself with 1-D bulk copies (TMA,
//     mbarrier complete_tx) and drains with CUDA-core math. A slot holds a
//     4-row x 2048-element tile of the weight (codes + block scales). The
//     activations (1..8 tokens) are quantized or copied into shared memory once
//     per CTA. No cross-warp synchronisation after the prologue. A second instance
//     (one token) ends in the tensor-parallel sum: every finished pair of rows is stored
//     into the receive memory of all ranks, and after its last group a warp adds the
//     ranks' contributions to its pairs out of its own receive memory.
//   * gemv_generic_kernel - any stride / any K % 32 == 0; one warp per output
//     row with direct global loads. Correctness fallback for odd shapes.
//
// Arithmetic (both kernels): e2m1 -> f16 exactly; the 16 products of a block
// are summed in f16 (exact: multiples of 1/4 with |sum| <= 576); the block sum
// is multiplied by the activation scale in f32 (exact) and accumulated with
// one f32 FMA by the weight scale; alpha is applied in f32 at the store.
#include "kernels.h"
#include "quant_core.cuh"
#include "status_mirror.cuh"

namespace nvfp4r {
namespace {

constexpr int kRowsPerGroup = 4;
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * kWarp;
constexpr int kUnitBytes = 16;                       // 32 elements = 2 scale blocks
constexpr int kChunkBytes = 1024;                    // code bytes per row per tile
constexpr int kUnitsPerLane = kChunkBytes / kUnitBytes / kWarp;   // 2
constexpr int kSlotRowBytes = kChunkBytes + kChunkBytes / 8;      // codes + scales
constexpr int kSlotBytes = kRowsPerGroup * kSlotRowBytes;         // 4608
constexpr int kMaxTokens = 8;
// Ring depth per warp: 3 slots (110592 B per CTA) or 2 slots (73728 B, three
// CTAs per SM).
__host__ __device__ constexpr int ring_bytes(int slots) { return kWarps * slots * kSlotBytes; }

struct StreamParams {
    GemvArgs a;
    int n_groups;        // ceil(N / 4)
    int n_chunks;        // ceil(K/2 / kChunkBytes)
    int x_token_bytes;   // K/2 + K/16
};

// Set to 1 by a kernel whose bounded wait ran out; read by the host on demand.
__device__ int g_device_status = 0;

// ---- decode helpers (operate on register values) ---------------------------

struct Unit16 {              // 32 elements as 16 f16x2
    uint32_t h[16];
};

__device__ __forceinline__ void decode_codes(const uint4& c, Unit16& u) {
    e2m1x8_to_f16x8(c.x, &u.h[0]);
    e2m1x8_to_f16x8(c.y, &u.h[4]);
    e2m1x8_to_f16x8(c.z, &u.h[8]);
    e2m1x8_to_f16x8(c.w, &u.h[12]);
}

__device__ __forceinline__ float2 decode_scale_pair(uint32_t two_bytes) {
    return __half22float2(as_half2(e4m3x2_to_f16x2(two_bytes)));
}

// Exact f16 dot product of one 16-element block (8 f16x2 pairs).
__device__ __forceinline__ float block_dot(const uint32_t* w, const uint32_t* x) {
    __half2 acc = __hmul2(as_half2(w[0]), as_half2(x[0]));
#pragma unroll
    for (int i = 1; i < 8; ++i) acc = __hfma2(as_half2(w[i]), as_half2(x[i]), acc);
    return __half2float(__hadd(__low2half(acc), __high2half(acc)));
}

__device__ __forceinline__ void store_out(void* out, int dtype, int64_t idx, float v) {
    if (dtype == 0)      static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
    else if (dtype == 1) static_cast<__half*>(out)[idx] = __float2half_rn(v);
    else                 static_cast<float*>(out)[idx] = v;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

// ---- streaming kernel -------------------------------------------------------

// Issue the copies of tile `t` of this warp into slot t % kSlots. Called by
// all lanes; lane 0 arms the barrier, lanes 0..7 issue one copy each.
__device__ __forceinline__ void issue_tile(const StreamParams& p, int lane, int group, int chunk,
                                           uint32_t slot_addr, uint32_t bar, uint64_t policy) {
    const int K2 = p.a.K / 2;
    const int off = chunk * kChunkBytes;
    const int bytes = min(kChunkBytes, K2 - off);
    const int row0 = group * kRowsPerGroup;
    const int rows = min(kRowsPerGroup, p.a.N - row0);
    if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(rows * (bytes + bytes / 8)));
    __syncwarp();
    if (lane < 2 * kRowsPerGroup) {
        const int r = lane >> 1;
        if (r < rows) {
            const int64_t row = row0 + r;
            if ((lane & 1) == 0)
                bulk_g2s(slot_addr + r * kSlotRowBytes, p.a.w + row * p.a.w_stride_n + off,
                         bytes, bar, policy);
            else
                bulk_g2s(slot_addr + r * kSlotRowBytes + kChunkBytes,
                         p.a.wsf + row * p.a.wsf_stride_n + off / 8, bytes / 8, bar, policy);
        }
    }
}

// kPush: the tensor-parallel epilogue (GemvArgs::push_*) is compiled in; one token only.
template <int MT, int kSlots, bool kPush = false>
__global__ void __launch_bounds__(kThreads, kSlots == 2 ? 3 : 1)
gemv_stream_kernel(const __grid_constant__ StreamParams p) {
    constexpr int kRingBytes = ring_bytes(kSlots);
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[kWarps * kSlots];

    const int tid = threadIdx.x;
    const int warp = tid / kWarp;
    const int lane = tid % kWarp;
    const int K = p.a.K, N = p.a.N, M = p.a.M;
    const int K2 = K / 2;

    uint8_t* ring = smem;
    uint8_t* xs = smem + kRingBytes;                       // [M][K/2 codes | K/16 scales]
    const uint32_t my_ring = smem_u32(ring) + warp * (kSlots * kSlotBytes);
    const uint32_t my_bars = smem_u32(&bars[warp * kSlots]);

    // This warp's groups: g = blockIdx.x + gridDim.x * (warp + kWarps * i)
    const int g_first = blockIdx.x + gridDim.x * warp;
    const int g_step = gridDim.x * kWarps;
    const int my_groups = (g_first < p.n_groups) ? (p.n_groups - g_first + g_step - 1) / g_step : 0;
    const int my_tiles = my_groups * p.n_chunks;

    const uint64_t policy = l2_policy_evict_first();
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kSlots; ++s) mbar_init(my_bars + 8 * s, 1);
        mbar_fence_init();
    }
    __syncwarp();

    // Weights do not depend on the preceding kernel: start streaming at once.
    // (group, chunk) of the next tile to issue, advanced one tile at a time: no division per tile
    int nxt_g = 0, nxt_c = 0;
#pragma unroll
    for (int t = 0; t < kSlots; ++t) {
        if (t < my_tiles) {
            issue_tile(p, lane, g_first + nxt_g * g_step, nxt_c, my_ring + t * kSlotBytes,
                       my_bars + 8 * t, policy);
            if (++nxt_c == p.n_chunks) { nxt_c = 0; ++nxt_g; }
        }
    }
    // The global scale is a constant of the layer (not written by the preceding kernel): its
    // trip to L2 happens here, not after the wait.
    const float gs = (p.a.xb != nullptr) ? __ldg(p.a.gs) : 1.0f;
    pdl_launch_dependents();

    // Activations come from the preceding kernel.
    pdl_wait_prior();
    // which half of the receive memory this call uses: the call counter in this rank's own header,
    // final before this kernel started (its writer is an earlier kernel)
    unsigned push_parity = 0;
    if (kPush) push_parity = *reinterpret_cast<volatile unsigned*>(p.a.push_base[p.a.push_rank]) & 1u;
    if (p.a.xb != nullptr) {
        const int blocks_per_tok = K / kBlockElems;
        const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(p.a.xb);
        const QuantScales qe = make_quant_scales<kRcpExact>(gs);
        const QuantScales qa = make_quant_scales<kRcpApprox>(gs);
        for (int i = tid; i < M * blocks_per_tok; i += kThreads) {
            // one token (the usual case): no division on the path between the wait and the loads
            const int m = (MT == 1) ? 0 : i / blocks_per_tok, b = i - m * blocks_per_tok;
            const uint4* src = reinterpret_cast<const uint4*>(xb + m * p.a.xb_stride + b * kBlockElems);
            const uint4 lo = __ldg(src), hi = __ldg(src + 1);
            uint32_t c[2];
            const uint32_t sf = (p.a.rcp_mode == kRcpExact)
                                    ? quantize_block16<kRcpExact>(lo, hi, qe, c)
                                    : quantize_block16<kRcpApprox>(lo, hi, qa, c);
            uint8_t* tok = xs + m * p.x_token_bytes;
            *reinterpret_cast<uint2*>(tok + b * 8) = make_uint2(c[0], c[1]);
            tok[K2 + b] = static_cast<uint8_t>(sf);
        }
    } else {
        const int code_vecs = K2 / 16, sf_vecs = K / 256;
        const int per_tok = code_vecs + sf_vecs;
        for (int i = tid; i < M * per_tok; i += kThreads) {
            const int m = i / per_tok, v = i - m * per_tok;
            const uint4 val = (v < code_vecs)
                ? ldg_keep_16(p.a.x + m * p.a.x_stride + v * 16)
                : ldg_keep_16(p.a.xsf + m * p.a.xsf_stride + (v - code_vecs) * 16);
            *reinterpret_cast<uint4*>(xs + m * p.x_token_bytes + v * 16) = val;
        }
    }
    __syncthreads();

    const uint32_t xs_addr = smem_u32(xs);
    float acc[kRowsPerGroup][MT];
#pragma unroll
    for (int r = 0; r < kRowsPerGroup; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

    bool timed_out = false;
    int gi = 0, c = 0, slot = 0;
    uint32_t phase = 0;                                  // parity of this slot's current fill
    for (int t = 0; t < my_tiles; ++t) {
        const uint32_t slot_addr = my_ring + slot * kSlotBytes;
        const uint32_t bar = my_bars + 8 * slot;
        const int group = g_first + gi * g_step;
        const int chunk_off = c * kChunkBytes;
        const int chunk_bytes = min(kChunkBytes, K2 - chunk_off);

        if (!mbar_wait_bounded(bar, phase)) { timed_out = true; break; }

#pragma unroll
        for (int j = 0; j < kUnitsPerLane; ++j) {
            const int u = lane + j * kWarp;
            if (u * kUnitBytes < chunk_bytes) {
                Unit16 wu[kRowsPerGroup];
                float2 ws[kRowsPerGroup];
#pragma unroll
                for (int r = 0; r < kRowsPerGroup; ++r) {
                    const uint32_t base = slot_addr + r * kSlotRowBytes;
                    decode_codes(lds128(base + u * kUnitBytes), wu[r]);
                    ws[r] = decode_scale_pair(lds16(base + kChunkBytes + u * 2));
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    if (m < M) {
                        const uint32_t tok = xs_addr + m * p.x_token_bytes;
                        Unit16 xu;
                        decode_codes(lds128(tok + chunk_off + u * kUnitBytes), xu);
                        const float2 sx = decode_scale_pair(lds16(tok + K2 + chunk_off / 8 + u * 2));
                        // eight independent f16 chains (4 rows x 2 blocks), interleaved
                        __half2 d[kRowsPerGroup][2];
#pragma unroll
                        for (int r = 0; r < kRowsPerGroup; ++r) {
                            d[r][0] = __hmul2(as_half2(wu[r].h[0]), as_half2(xu.h[0]));
                            d[r][1] = __hmul2(as_half2(wu[r].h[8]), as_half2(xu.h[8]));
                        }
#pragma unroll
                        for (int i = 1; i < 8; ++i)
#pragma unroll
                            for (int r = 0; r < kRowsPerGroup; ++r) {
                                d[r][0] = __hfma2(as_half2(wu[r].h[i]), as_half2(xu.h[i]), d[r][0]);
                                d[r][1] = __hfma2(as_half2(wu[r].h[8 + i]), as_half2(xu.h[8 + i]), d[r][1]);
                            }
#pragma unroll
                        for (int r = 0; r < kRowsPerGroup; ++r) {
                            const float d0 = __half2float(__hadd(__low2half(d[r][0]), __high2half(d[r][0]))) * sx.x;
                            const float d1 = __half2float(__hadd(__low2half(d[r][1]), __high2half(d[r][1]))) * sx.y;
                            acc[r][m] = fmaf(d0, ws[r].x, acc[r][m]);
                            acc[r][m] = fmaf(d1, ws[r].y, acc[r][m]);
                        }
                    }
                }
            }
        }
        __syncwarp();

        // Refill this slot with the tile kSlots ahead.
        if (t + kSlots < my_tiles) {
            issue_tile(p, lane, g_first + nxt_g * g_step, nxt_c, slot_addr, bar, policy);
            if (++nxt_c == p.n_chunks) { nxt_c = 0; ++nxt_g; }
        }

        if (c == p.n_chunks - 1) {                 // group finished: reduce and store
#pragma unroll
            for (int r = 0; r < kRowsPerGroup; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float v = acc[r][m];
#pragma unroll
                    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
                    acc[r][m] = v;
                }
            float mine = 0.0f;
#pragma unroll
            for (int r = 0; r < kRowsPerGroup; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (lane == m * kRowsPerGroup + r) mine = acc[r][m];
            const int r = lane % kRowsPerGroup, m = lane / kRowsPerGroup;
            const int row = group * kRowsPerGroup + r;
            if (kPush) {
                // lanes 0 and 2 hold rows 0 and 2 of the group: each sends the pair (row, row + 1)
                const float o = mine * p.a.alpha;
                const float o2 = __shfl_down_sync(0xffffffffu, o, 1);
                if (lane < kRowsPerGroup && (lane & 1) == 0 && row < N) {
                    const __nv_bfloat162 pk = __floats2bfloat162_rn(o, row + 1 < N ? o2 : 0.0f);
                    const unsigned long long w = (1ull << 32) | *reinterpret_cast<const uint32_t*>(&pk);
                    const unsigned long long i = static_cast<unsigned long long>(row) >> 1;
                    const int W = p.a.push_world;
#pragma unroll 1
                    for (int d = 0; d < W; ++d) {
                        const int dst = (p.a.push_rank + d) % W;
                        unsigned long long* slot = reinterpret_cast<unsigned long long*>(p.a.push_base[dst] + 256) +
                            (static_cast<unsigned long long>(push_parity) * W + p.a.push_rank) * p.a.push_max_pairs + i;
                        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(slot), "l"(w) : "memory");
                    }
                }
            } else if (m < M && m < MT && row < N)
                store_out(p.a.out, p.a.out_dtype, m * p.a.out_stride + row, mine * p.a.alpha);
#pragma unroll
            for (int rr = 0; rr < kRowsPerGroup; ++rr)
#pragma unroll
                for (int mm = 0; mm < MT; ++mm) acc[rr][mm] = 0.0f;
        }
        if (++c == p.n_chunks) { c = 0; ++gi; }
        if (++slot == kSlots) { slot = 0; phase ^= 1u; }
    }

    if (kPush && !timed_out) {
        // Second half, after all of this warp's pushes are on their way (waiting inside the loop
        // would hold back the pushes of its later groups, which the peers wait for): sum the
        // ranks' contributions to every pair this warp pushed, out of this rank's own receive memory.
        const int W = p.a.push_world;
#pragma unroll 1
        for (int g2 = 0; g2 < my_groups; ++g2) {
            const int row = (g_first + g2 * g_step) * kRowsPerGroup + lane;
            if (lane < kRowsPerGroup && (lane & 1) == 0 && row < N) {
                const unsigned long long i = static_cast<unsigned long long>(row) >> 1;
                unsigned long long* own = reinterpret_cast<unsigned long long*>(p.a.push_base[p.a.push_rank] + 256) +
                                          static_cast<unsigned long long>(push_parity) * W * p.a.push_max_pairs + i;
                float lo = 0.0f, hi = 0.0f;
#pragma unroll 1
                for (int s = 0; s < W; ++s) {            // rank order: every rank adds the same sequence
                    unsigned long long v = 0;
                    uint32_t it = 0;
                    do {
                        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(own + s * p.a.push_max_pairs) : "memory");
                    } while ((v >> 32) != 1ull && ++it <= p.a.push_poll_limit);
                    if ((v >> 32) != 1ull) timed_out = true;
                    const uint32_t bits = static_cast<uint32_t>(v);
                    lo += __uint_as_float(bits << 16);
                    hi += __uint_as_float(bits & 0xFFFF0000u);
                    own[s * p.a.push_max_pairs] = 0ull;
                }
                const __nv_bfloat162 sum = __floats2bfloat162_rn(lo, hi);
                static_cast<uint32_t*>(p.a.out)[i] = *reinterpret_cast<const uint32_t*>(&sum);
            }
        }
    }
    if (kPush) {
        // the last CTA of the grid to finish advances the call counter: nobody of this launch reads
        // it any more (same rule as the stand-alone all-reduce kernel)
        __syncthreads();
        if (tid == 0) {
            unsigned* header = reinterpret_cast<unsigned*>(p.a.push_base[p.a.push_rank]);
            __threadfence();
            const unsigned t = atomicAdd(header + 1, 1u);
            if (t == gridDim.x - 1) {
                header[1] = 0u;
                header[0] = header[0] + 1u;
            }
        }
    }
    if (__any_sync(0xffffffffu, timed_out)) {
        if (lane == 0) report_timeout(&g_device_status, 1);
        // Give copies that are still in flight a bounded time to land before
        // this CTA's shared memory is released.
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
}

// ---- generic kernel ---------------------------------------------------------

// Quantize the 32 bf16 values of unit `u` of one token and decode them again.
__device__ __forceinline__ float2 quantize_unit(const GemvArgs& a, int m, int u, Unit16& xu) {
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(a.xb) + m * a.xb_stride + u * 32;
    const uint4* src = reinterpret_cast<const uint4*>(xb);
    const float gs = __ldg(a.gs);
    uint32_t c0[2], c1[2], sf0, sf1;
    if (a.rcp_mode == kRcpExact) {
        const QuantScales q = make_quant_scales<kRcpExact>(gs);
        sf0 = quantize_block16<kRcpExact>(__ldg(src), __ldg(src + 1), q, c0);
        sf1 = quantize_block16<kRcpExact>(__ldg(src + 2), __ldg(src + 3), q, c1);
    } else {
        const QuantScales q = make_quant_scales<kRcpApprox>(gs);
        sf0 = quantize_block16<kRcpApprox>(__ldg(src), __ldg(src + 1), q, c0);
        sf1 = quantize_block16<kRcpApprox>(__ldg(src + 2), __ldg(src + 3), q, c1);
    }
    decode_codes(make_uint4(c0[0], c0[1], c1[0], c1[1]), xu);
    return decode_scale_pair(sf0 | (sf1 << 8));
}

template <int MT>
__global__ void __launch_bounds__(kThreads)
gemv_generic_kernel(const GemvArgs a, int m0) {
    pdl_wait_prior();
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
    if (row >= a.N) return;
    const int units = a.K / 32;
    const uint8_t* wrow = a.w + row * a.w_stride_n;
    const uint8_t* srow = a.wsf + row * a.wsf_stride_n;
    const int mcount = min(MT, a.M - m0);
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
    for (int u = lane; u < units; u += kWarp) {
        Unit16 wu;
        decode_codes(ldg_stream_16(wrow + u * kUnitBytes), wu);
        const float2 ws = decode_scale_pair(ldg_stream_2(srow + u * 2));
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < mcount) {
                Unit16 xu;
                float2 sx;
                if (a.xb != nullptr) {
                    sx = quantize_unit(a, m0 + m, u, xu);
                } else {
                    decode_codes(ldg_keep_16(a.x + (m0 + m) * a.x_stride + u * kUnitBytes), xu);
                    sx = decode_scale_pair(__ldg(reinterpret_cast<const unsigned short*>(
                        a.xsf + (m0 + m) * a.xsf_stride + u * 2)));
                }
                const float d0 = block_dot(&wu.h[0], &xu.h[0]) * sx.x;
                const float d1 = block_dot(&wu.h[8], &xu.h[8]) * sx.y;
                acc[m] = fmaf(d0, ws.x, acc[m]);
                acc[m] = fmaf(d1, ws.y, acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        float v = acc[m];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
        if (lane == 0 && m < mcount)
            store_out(a.out, a.out_dtype, (m0 + m) * a.out_stride + row, v * a.alpha);
    }
}

}  // namespace

cudaError_t read_and_clear_device_status(int* flag) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    e = cudaMemcpyFromSymbol(flag, g_device_status, sizeof(int));
    if (e != cudaSuccess) return e;
    const int zero = 0;
    return cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
}

cudaError_t set_status_mirror_gemv(int* p) { return set_status_mirror_here(p); }

GemvTuning& gemv_tuning() {
    static GemvTuning t = {0, 1, 0};
    return t;
}

int device_sm_count() {
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (sms[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
            v = 148;
        sms[dev] = v;
    }
    return sms[dev];
}

bool gemv_stream_supported(const GemvArgs& a) {
    if (gemv_tuning().force_generic) return false;
    if (a.M < 1 || a.M > kMaxTokens) return false;
    if (a.K % 256 != 0) return false;
    if (a.w_stride_n % 16 != 0 || a.wsf_stride_n % 16 != 0) return false;
    if ((reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.wsf)) & 15) return false;
    if (a.xb != nullptr) {
        if ((reinterpret_cast<uintptr_t>(a.xb) & 15) || (a.xb_stride % 8) != 0) return false;
    } else {
        if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.xsf)) & 15) return false;
        if (a.x_stride % 16 != 0 || a.xsf_stride % 16 != 0) return false;
    }
    const int64_t xbytes = static_cast<int64_t>(a.M) * (a.K / 2 + a.K / 16);
    return ring_bytes(3) + xbytes <= 227 * 1024 - 1024;
}

cudaError_t launch_gemv_stream(const GemvArgs& a, cudaStream_t stream) {
    StreamParams p;
    p.a = a;
    p.n_groups = (a.N + kRowsPerGroup - 1) / kRowsPerGroup;
    p.n_chunks = (a.K / 2 + kChunkBytes - 1) / kChunkBytes;
    p.x_token_bytes = a.K / 2 + a.K / 16;
    const GemvTuning& tune = gemv_tuning();
    // Automatic choice (measured, M = 1: 24576x4096 17.4 -> 12.8 us, 6144x4096 5.8 -> 5.1 us with
    // three CTAs per SM; 4096x4096 3.6 -> 4.7 us and 5120x25600 34 -> 41 us, hence the bounds:
    // every CTA quantizes the whole activation row, which is what long rows pay for).
    // K <= 4096: three CTAs of 73 728 B ring + activations + 1 KB reserved fit an SM (231 KB for
    // 227 KB would not at K = 5120); longer rows stay on one CTA per SM.
    const bool wide = a.M == 1 && p.n_groups >= 1536 && a.K <= 4096;
    int ctas_per_sm = tune.ctas_per_sm > 0 ? tune.ctas_per_sm : (wide ? 3 : 1);
    if (a.M > 1 && ctas_per_sm > 2) ctas_per_sm = 2;     // register budget of the M > 1 variants
    const bool two_slots = ctas_per_sm >= 3;
    const size_t smem = ring_bytes(two_slots ? 2 : 3) + static_cast<size_t>(a.M) * p.x_token_bytes;

    using Kern = void (*)(StreamParams);
    static const Kern table[4][2] = {
        {gemv_stream_kernel<1, 3>, gemv_stream_kernel<1, 2>},
        {gemv_stream_kernel<2, 3>, gemv_stream_kernel<2, 3>},
        {gemv_stream_kernel<4, 3>, gemv_stream_kernel<4, 3>},
        {gemv_stream_kernel<8, 3>, gemv_stream_kernel<8, 3>}};
    const int ki = a.M == 1 ? 0 : a.M == 2 ? 1 : a.M <= 4 ? 2 : 3;
    Kern kern = table[ki][two_slots ? 1 : 0];
    const bool push = a.push_world > 1;
    if (push) {
        // the all-reduce inside the launch: one token, bf16 pairs of rows
        if (a.M != 1 || a.out_dtype != 0 || (a.N & 1) || a.out_stride != a.N) return cudaErrorInvalidValue;
        kern = two_slots ? gemv_stream_kernel<1, 2, true> : gemv_stream_kernel<1, 3, true>;
    }

    static bool attr_done[5][2][64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const int ai = push ? 4 : ki;
    if (dev >= 0 && dev < 64 && !attr_done[ai][two_slots][dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
        if (e != cudaSuccess) return e;
        attr_done[ai][two_slots][dev] = true;
    }

    int grid = device_sm_count() * ctas_per_sm;
    if (grid > p.n_groups) grid = p.n_groups;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tune.use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

cudaError_t launch_gemv_generic(const GemvArgs& a, cudaStream_t stream) {
    const unsigned blocks = static_cast<unsigned>((a.N + kWarps - 1) / kWarps);
    for (int m0 = 0; m0 < a.M; m0 += 4) {
        const int left = a.M - m0;
        if (left == 1) gemv_generic_kernel<1><<<blocks, kThreads, 0, stream>>>(a, m0);
        else if (left == 2) gemv_generic_kernel<2><<<blocks, kThreads, 0, stream>>>(a, m0);
        else gemv_generic_kernel<4><<<blocks, kThreads, 0, stream>>>(a, m0);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace nvfp4r
