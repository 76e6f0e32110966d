// Decode linear on the tensor cores over a PRE-PACKED weight: the product path of the
// vLLM adapter for every M <= 32.
//
// Packed weight format (built once per layer by pack_weight_kernel): the weight is cut
// into blocks of 128 rows x 256 K-elements; block (tile, kb) occupies 18 432 contiguous
// bytes at ((tile * K/256) + kb) * 18432:
//   [0, 16384)      the block's codes exactly as the tensor core wants them in shared
//                   memory: K-major rows of 128 B, 128-byte swizzle (16-byte unit index
//                   XOR row%8), 8-row groups 1024 B apart
//   [16384, 18432)  the block's 128 x 16 scales as four 512-byte chunks (one per 64
//                   K-elements) in the 32x4x4 order that tcgen05.cp 32x128b.warpx4 copies
// Consecutive K blocks of a tile are contiguous, so a pipeline stage of 1 or 2 blocks is
// ONE 1-D bulk copy of 18 or 36 KB: perfectly sequential DRAM reads, one TMA instruction
// and one mbarrier transaction per 36 KB, no tensor map.
//
// Why this shape (measured on B200, see the profile notes of this kernel):
//   * a thread that issues bulk copies is held ~190 cycles per copy and the MMA thread
//     spends ~550 cycles per stage on barrier wait + commit regardless of the work in it,
//     so stages must be few and large;
//   * shared memory per CTA stays under half an SM (two 36 KB stages + the activations of
//     a K part of at most 2048 elements) so that the CTA of the NEXT linear, launched with
//     programmatic stream serialization, becomes resident while this one still runs and
//     starts pulling its own weights at once;
//   * the activation block scales are copied into tensor memory once per kernel and stay
//     there (128 columns), the weight scales ride with each stage.
//
// Persistent CTAs (one per SM), roles and split-K protocol as in gemm_tcgen05.cu.
#include "kernels.h"
#include "quant_core.cuh"
#include "tcgen05_ptx.cuh"

namespace nvfp4r {
namespace {

using namespace tc;

constexpr int kTileRows = 128;
constexpr int kBlockK = 256;
constexpr int kCodesBytes = kTileRows * (kBlockK / 2);      // 16384
constexpr int kSfBytes = kTileRows * (kBlockK / 16);        // 2048
constexpr int kBlockBytes = kCodesBytes + kSfBytes;         // 18432
constexpr int kBlocksPerStage = 2;
constexpr int kStageBytes = kBlocksPerStage * kBlockBytes;  // 36864
constexpr int kStages = 2;
constexpr int kMaxPartBlocks = 8;                           // K part <= 2048 elements
constexpr int kThreadsP = 192;
constexpr int kEpilogueThreads = 128;

struct PackedParams {
    const uint8_t* packed;
    const void* xb;            // bf16 [M, K]
    int64_t xb_stride;
    const float* gs;
    int rcp_mode;
    void* out;
    int out_dtype;
    int64_t ldc;               // elements between tokens in out
    int M, m0, N, K;
    float alpha;
    int tiles, splits, kblocks;
    float* partials;
    unsigned* tickets;
    // fused prologue (what produces the bf16 activations that get quantized)
    int pro_kind;                  // 0: xb as is; 1: RMSNorm(residual_in + delta) * norm_w; 2: silu(g) * u
    const void* delta;             // kind 1: bf16 [M, K] or nullptr
    const void* residual_in;       // kind 1: bf16 [M, K]
    void* residual_out;            // kind 1: bf16 [M, K], receives residual_in + delta
    const void* norm_w;            // kind 1: bf16 [K]
    float eps;
};

__device__ int g_packed_status = 0;
// Optional time line of CTA 0 (nanoseconds of %globaltimer), filled when g_packed_trace != 0.
__device__ int g_packed_trace = 0;
__device__ unsigned long long g_packed_times[4 * 16];
__device__ unsigned g_packed_launch = 0;
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TRACE(slot) do { if (trace) g_packed_times[(launch_id & 3) * 16 + (slot)] = gtime(); } while (0)

// ---- one-time re-layout ----------------------------------------------------------

// One thread moves one 16-byte unit of codes; the first K/256*... threads of each block
// also move the scales. grid = (K/256, N/128), block = 1024 threads (128 rows x 8 units).
__global__ void __launch_bounds__(1024)
pack_weight_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ sf_flat,
                   uint8_t* __restrict__ packed, int N, int K) {
    const int kb = blockIdx.x, tile = blockIdx.y;
    const int row = threadIdx.x >> 3, unit = threadIdx.x & 7;
    uint8_t* dst = packed + (static_cast<int64_t>(tile) * (K / kBlockK) + kb) * kBlockBytes;
    const int64_t n = static_cast<int64_t>(tile) * kTileRows + row;
    const uint4 v = *reinterpret_cast<const uint4*>(w + n * (K / 2) + kb * 128 + unit * 16);
    *reinterpret_cast<uint4*>(dst + swz128(row, unit * 16)) = v;
    // scales: 16 per row in this block = 4 chunks x 4; threads with unit < 4 move 4 bytes
    if (unit < 4) {
        const uint32_t s4 = *reinterpret_cast<const uint32_t*>(sf_flat + n * (K / 16) + kb * 16 + unit * 4);
        *reinterpret_cast<uint32_t*>(dst + kCodesBytes + unit * 512 + (row % 32) * 16 + (row / 32) * 4) = s4;
    }
}

// ---- bf16 vector helpers for the fused prologues ----------------------------------------
__device__ __forceinline__ void unpack8(const uint4& v, float f[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ uint32_t pack2_bf16(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8(const float f[8]) {
    return make_uint4(pack2_bf16(f[0], f[1]), pack2_bf16(f[2], f[3]), pack2_bf16(f[4], f[5]),
                      pack2_bf16(f[6], f[7]));
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// ---- thread-block cluster helpers (split-K reduction through distributed shared memory)
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" :: "r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < 20000000u; ++i)
        if (mbar_try_wait_cluster(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ unsigned ticket_acq_rel(unsigned* addr) {
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(addr) : "memory");
    return old;
}

// ---- the linear ---------------------------------------------------------------------

// kCluster: the S CTAs that share a tile form a thread-block cluster (cluster rank = K
// part) and reduce their partial tiles through distributed shared memory: every CTA owns
// 128/S rows of the tile, receives the other parts' values for those rows with
// st.shared::cluster + a remote mbarrier arrive, adds them in part order and stores.
// Without it (S == 1, or S not a cluster size) partials go through global scratch and a
// ticket.
template <int BN, bool kCluster>
__global__ void __launch_bounds__(kThreadsP, 2)
linear_packed_kernel(const __grid_constant__ PackedParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));

    __shared__ __align__(8) uint64_t bars[2 * kStages + 6];
    __shared__ uint32_t s_tmem;
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid / kWarp, lane = tid % kWarp;
    const bool trace = (g_packed_trace != 0) && blockIdx.x == 0 && lane == 0;
    __shared__ unsigned s_launch_id;
    if (g_packed_trace != 0 && blockIdx.x == 0) {
        if (tid == 0) s_launch_id = atomicAdd(&g_packed_launch, 1u);
        __syncthreads();
    }
    const unsigned launch_id = (g_packed_trace != 0 && blockIdx.x == 0) ? s_launch_id : 0u;
    if (warp == 0) TRACE(0);
    const int S = p.splits;
    const int ctas_per_part = gridDim.x / S;           // CTAs beyond S * ctas_per_part idle
    const int c = blockIdx.x;
    const bool active = c < S * ctas_per_part;
    const int part = c % S, rank_in_part = c / S;
    const int kb0 = static_cast<int>((static_cast<int64_t>(p.kblocks) * part) / S);
    const int kb1 = static_cast<int>((static_cast<int64_t>(p.kblocks) * (part + 1)) / S);
    const int nkb = kb1 - kb0;                                        // <= kMaxPartBlocks
    const int stages_per_tile = (nkb + kBlocksPerStage - 1) / kBlocksPerStage;
    const int my_tiles = (active && rank_in_part < p.tiles)
                             ? (p.tiles - rank_in_part + ctas_per_part - 1) / ctas_per_part : 0;
    const int total = my_tiles * stages_per_tile;

    const uint32_t ring = smem_base;
    const uint32_t b_tile = ring + kStages * kStageBytes;            // nkb blocks of BN x 128 B
    // activation scale chunks: tcgen05.cp reads 32 rows x 16 B per chunk, but only rows
    // < BN matter, so with BN == 16 consecutive chunks overlap by half (stride 256 B)
    constexpr int kSfbStride = (BN == 16) ? 256 : 512;
    constexpr int kSfbBytes = kMaxPartBlocks * 4 * kSfbStride + 256;
    const uint32_t b_sf = b_tile + kMaxPartBlocks * (BN * 128);
    uint8_t* b_tile_g = smem + kStages * kStageBytes;
    uint8_t* b_sf_g = b_tile_g + kMaxPartBlocks * (BN * 128);
    // cluster reduction: values received for the rows this CTA owns, [part][token][row]
    const uint32_t recv = b_sf + kSfbBytes;
    float* recv_g = reinterpret_cast<float*>(b_sf_g + kSfbBytes);

    const uint32_t bar_full = smem_u32(&bars[0]);
    const uint32_t bar_empty = smem_u32(&bars[kStages]);
    const uint32_t bar_accfull = smem_u32(&bars[2 * kStages]);
    const uint32_t bar_accempty = smem_u32(&bars[2 * kStages + 2]);
    const uint32_t bar_redfull = smem_u32(&bars[2 * kStages + 4]);
    const uint32_t bar_redfree = smem_u32(&bars[2 * kStages + 5]);

    constexpr uint32_t kTmemCols = 256;
    constexpr uint32_t kColSFA = 2 * BN;                              // 16 columns per block in a stage
    constexpr uint32_t kColSFB = kColSFA + 16 * kBlocksPerStage;      // likewise for the activations
    constexpr uint32_t kColSFBres = kColSFB + 16 * kBlocksPerStage;   // 16 per block of the K part

    if (warp == 0 && lane == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_accfull + 8 * b, 1);
            mbar_init(bar_accempty + 8 * b, kEpilogueThreads / kWarp);
        }
        if (kCluster) {
            mbar_init(bar_redfull, (S - 1) * (kTileRows / S));   // one arrival per sending thread
            mbar_init(bar_redfree, S - 1);                       // one arrival per peer CTA
        }
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    const uint64_t policy = l2_policy_evict_first();
    auto stage_blocks = [&](int j) { return min(kBlocksPerStage, nkb - j * kBlocksPerStage); };
    auto issue = [&](int i) {                          // stage i of this CTA's sequence
        const int ti = i / stages_per_tile, j = i - ti * stages_per_tile;
        const int tile = rank_in_part + ti * ctas_per_part;
        const int s = i % kStages;
        const uint32_t bytes = static_cast<uint32_t>(stage_blocks(j)) * kBlockBytes;
        mbar_expect_tx(bar_full + 8 * s, bytes);
        bulk_g2s(ring + s * kStageBytes,
                 p.packed + (static_cast<int64_t>(tile) * p.kblocks + kb0 + j * kBlocksPerStage) * kBlockBytes,
                 bytes, bar_full + 8 * s, policy);
    };

    int issued = 0;
    if (warp == 0 && lane == 0) {
        const int first = min(kStages, total);
        for (; issued < first; ++issued) issue(issued);
    }
    if (warp == 0) TRACE(1);
    pdl_launch_dependents();
    if (kCluster) cluster_sync_all();      // every CTA's reduction barriers are initialised
    pdl_wait_prior();
    if (warp == 0) TRACE(2);

    // ---- prologue: quantize this part's activations into operand layout --------------
    if (active) {
        const int blk0 = kb0 * (kBlockK / 16);
        const int blocks = nkb * (kBlockK / 16);
        const float gs = __ldg(p.gs);
        const QuantScales qe = make_quant_scales<kRcpExact>(gs);
        const QuantScales qa = make_quant_scales<kRcpApprox>(gs);
        const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(p.xb);
        const int n_items = p.M * blocks;
        auto quantize_store = [&](int m, int blk, const uint4& lo, const uint4& hi) {
            uint32_t cw[2];
            const uint32_t sf = (p.rcp_mode == kRcpExact) ? quantize_block16<kRcpExact>(lo, hi, qe, cw)
                                                          : quantize_block16<kRcpApprox>(lo, hi, qa, cw);
            *reinterpret_cast<uint2*>(b_tile_g + (blk >> 4) * (BN * 128) + swz128(m, (blk & 15) * 8)) =
                make_uint2(cw[0], cw[1]);
            b_sf_g[(blk >> 2) * kSfbStride + m * 16 + (blk & 3)] = static_cast<uint8_t>(sf);
        };
        if (p.pro_kind == 0) {
            // four blocks per thread per round: all eight 16-byte loads are issued before any
            // of the arithmetic, so a round costs one memory round trip
            for (int i0 = tid; i0 < n_items; i0 += 4 * kThreadsP) {
                uint4 lo[4], hi[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * kThreadsP;
                    if (i < n_items) {
                        const int m = i / blocks, blk = i - m * blocks;
                        const uint4* src = reinterpret_cast<const uint4*>(
                            xb + (p.m0 + m) * p.xb_stride + static_cast<int64_t>(blk0 + blk) * 16);
                        lo[u] = __ldg(src);
                        hi[u] = __ldg(src + 1);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * kThreadsP;
                    if (i < n_items) quantize_store(i / blocks, i % blocks, lo[u], hi[u]);
                }
            }
        } else if (p.pro_kind == 2) {
            // activation = bf16(silu(gate) * up), gate_up row = [gate (K) | up (K)]
            for (int i = tid; i < n_items; i += kThreadsP) {
                const int m = i / blocks, blk = i - m * blocks;
                const __nv_bfloat16* row = xb + (p.m0 + m) * p.xb_stride + static_cast<int64_t>(blk0 + blk) * 16;
                const uint4 g0 = __ldg(reinterpret_cast<const uint4*>(row));
                const uint4 g1 = __ldg(reinterpret_cast<const uint4*>(row) + 1);
                const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(row + p.K));
                const uint4 u1 = __ldg(reinterpret_cast<const uint4*>(row + p.K) + 1);
                float g[16], u[16];
                unpack8(g0, g); unpack8(g1, g + 8); unpack8(u0, u); unpack8(u1, u + 8);
#pragma unroll
                for (int j = 0; j < 16; ++j) g[j] = g[j] / (1.0f + __expf(-g[j])) * u[j];
                quantize_store(m, blk, pack8(g), pack8(g + 8));
            }
        } else {
            // activation = bf16( bf16(residual + delta) * rsqrt(mean_sq + eps) * norm_w ).
            // Every CTA needs the row's mean square over the whole K: it is recomputed
            // here from L2 (2 x 2K bytes per row) instead of being passed between kernels.
            float* red = reinterpret_cast<float*>(recv_g);            // reduction buffer is free now
            const __nv_bfloat16* rin = static_cast<const __nv_bfloat16*>(p.residual_in);
            const __nv_bfloat16* dl = static_cast<const __nv_bfloat16*>(p.delta);
            const __nv_bfloat16* nw = static_cast<const __nv_bfloat16*>(p.norm_w);
            __nv_bfloat16* rout = static_cast<__nv_bfloat16*>(p.residual_out);
            for (int m = 0; m < p.M; ++m) {
                const int64_t base = static_cast<int64_t>(p.m0 + m) * p.K;
                float ss = 0.0f;
                for (int c8 = tid; c8 < p.K / 8; c8 += kThreadsP) {
                    float r[8], d[8];
                    unpack8(__ldg(reinterpret_cast<const uint4*>(rin + base) + c8), r);
                    if (dl != nullptr) {
                        unpack8(__ldg(reinterpret_cast<const uint4*>(dl + base) + c8), d);
#pragma unroll
                        for (int j = 0; j < 8; ++j) r[j] = round_bf16(r[j] + d[j]);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss += r[j] * r[j];
                }
#pragma unroll
                for (int sft = 16; sft > 0; sft >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sft);
                if (lane == 0) red[m * 8 + warp] = ss;
            }
            __syncthreads();
            const bool writer = (rank_in_part == 0);                  // one CTA per K part writes the residual
            for (int i = tid; i < n_items; i += kThreadsP) {
                const int m = i / blocks, blk = i - m * blocks;
                float tot = 0.0f;
#pragma unroll
                for (int w = 0; w < kThreadsP / kWarp; ++w) tot += red[m * 8 + w];
                const float inv = rsqrtf(tot / static_cast<float>(p.K) + p.eps);
                const int64_t off = static_cast<int64_t>(p.m0 + m) * p.K + static_cast<int64_t>(blk0 + blk) * 16;
                float r[16], d[16], w16[16];
                unpack8(__ldg(reinterpret_cast<const uint4*>(rin + off)), r);
                unpack8(__ldg(reinterpret_cast<const uint4*>(rin + off) + 1), r + 8);
                if (dl != nullptr) {
                    unpack8(__ldg(reinterpret_cast<const uint4*>(dl + off)), d);
                    unpack8(__ldg(reinterpret_cast<const uint4*>(dl + off) + 1), d + 8);
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = round_bf16(r[j] + d[j]);
                }
                if (writer) {
                    *reinterpret_cast<uint4*>(rout + off) = pack8(r);
                    *(reinterpret_cast<uint4*>(rout + off) + 1) = pack8(r + 8);
                }
                const int64_t koff = static_cast<int64_t>(blk0 + blk) * 16;
                unpack8(__ldg(reinterpret_cast<const uint4*>(nw + koff)), w16);
                unpack8(__ldg(reinterpret_cast<const uint4*>(nw + koff) + 1), w16 + 8);
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = r[j] * inv * w16[j];
                quantize_store(m, blk, pack8(r), pack8(r + 8));
            }
            __syncthreads();                                          // red is handed back to the reduction
        }
        // Rows M..BN-1 of the operand are never written: whatever they hold only reaches
        // accumulator columns that are not stored.
        fence_proxy_async_smem();
    }
    __syncthreads();
    if (warp == 0) TRACE(3);

    WaitFail wf;
    if (warp == 0) {
        // ---------------- producer -------------------------------------------------------
        if (lane == 0) {
            for (int i = issued; i < total; ++i) {
                const int s = i % kStages;
                if (!wf.wait(bar_empty + 8 * s, ((i / kStages) - 1) & 1)) break;
                issue(i);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer -----------------------------------------------------
        if (lane == 0 && my_tiles > 0) {
            constexpr uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                       (static_cast<uint32_t>(kTileRows >> 7) << 27);
            // A CTA that walks several tiles copies the activation scales into tensor
            // memory once; a single-tile CTA copies them with the stage that uses them.
            const bool sfb_resident = my_tiles >= 2;
            if (sfb_resident)
                for (int ch = 0; ch < nkb * 4; ++ch)
                    tc_cp_scales(tmem + kColSFBres + 4 * ch, desc_scales(b_sf + ch * kSfbStride));
            int i = 0;
            for (int ti = 0; ti < my_tiles && !wf.failed; ++ti) {
                const int buf = ti & 1;
                if (ti >= 2 && !wf.wait(bar_accempty + 8 * buf, ((ti >> 1) - 1) & 1)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem + buf * BN;
                for (int j = 0; j < stages_per_tile; ++j, ++i) {
                    const int s = i % kStages;
                    if (!wf.wait(bar_full + 8 * s, (i / kStages) & 1)) break;
                    if (i == 0) TRACE(4);
                    tc_fence_after();
                    const int nb = stage_blocks(j);
                    for (int b = 0; b < nb; ++b) {
                        const uint32_t a_smem = ring + s * kStageBytes + b * kBlockBytes;
                        const int blk = j * kBlocksPerStage + b;              // block within the part
                        const uint32_t b_smem = b_tile + blk * (BN * 128);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            tc_cp_scales(tmem + kColSFA + 16 * b + 4 * k,
                                         desc_scales(a_smem + kCodesBytes + k * 512));
                            if (!sfb_resident)
                                tc_cp_scales(tmem + kColSFB + 16 * b + 4 * k,
                                             desc_scales(b_sf + (blk * 4 + k) * kSfbStride));
                        }
                        const uint32_t sfb_col = sfb_resident ? kColSFBres + 16 * blk : kColSFB + 16 * b;
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            tc_mma_nvf4(d_tmem, desc_operand(a_smem + k * 32), desc_operand(b_smem + k * 32),
                                        idesc, tmem + kColSFA + 16 * b + 4 * k,
                                        tmem + sfb_col + 4 * k, (blk > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_empty + 8 * s);
                }
                tc_commit(bar_accfull + 8 * buf);
                if (ti == 0) TRACE(5);
            }
            TRACE(6);
        }
    } else {
        // ---------------- epilogue (warps 2..5) ------------------------------------------
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        const int et = tid - 2 * kWarp;
        for (int ti = 0; ti < my_tiles; ++ti) {
            const int buf = ti & 1;
            const int tile = rank_in_part + ti * ctas_per_part;
            if (!wf.wait(bar_accfull + 8 * buf, (ti >> 1) & 1)) break;
            if (warp == 2 && ti == 0) TRACE(7);
            if (warp == 2 && ti == my_tiles - 1) TRACE(8);
            tc_fence_after();
            float acc[BN];
#pragma unroll
            for (int h = 0; h < BN / 16; ++h)
                tmem_ld16(tmem + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + h * 16, &acc[h * 16]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_accempty + 8 * buf);

            const int64_t n = static_cast<int64_t>(tile) * kTileRows + row_in_tile;
            auto store = [&](int m, float v) {
                const int64_t idx = (p.m0 + m) * p.ldc + n;
                v *= p.alpha;
                if (p.out_dtype == 0) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(v);
                else if (p.out_dtype == 1) static_cast<__half*>(p.out)[idx] = __float2half_rn(v);
                else static_cast<float*>(p.out)[idx] = v;
            };
            if (S == 1) {
#pragma unroll
                for (int m = 0; m < BN; ++m)
                    if (m < p.M) store(m, acc[m]);
            } else if (kCluster) {
                // reduce-scatter over the cluster: rows [o*R, (o+1)*R) of the tile belong to
                // the CTA of rank o; recv[part][token][row - o*R] in the owner's shared memory
                const int R = kTileRows / S;
                const int owner = row_in_tile / R, r_local = row_in_tile - owner * R;
                if (ti >= 1) {                              // peers have read tile ti-1's values
                    if (!mbar_wait_cluster_bounded(bar_redfree, (ti - 1) & 1)) wf.failed = true;
                }
                if (owner != part) {
                    const uint32_t dst = map_to_rank(recv, owner) +
                                         static_cast<uint32_t>((part * BN * R + r_local) * 4);
#pragma unroll
                    for (int m = 0; m < BN; ++m)
                        if (m < p.M) st_cluster_f32(dst + m * R * 4, acc[m]);
                    mbar_arrive_remote(map_to_rank(bar_redfull, owner));
                } else {
                    if (!mbar_wait_cluster_bounded(bar_redfull, ti & 1)) wf.failed = true;
#pragma unroll
                    for (int m = 0; m < BN; ++m) {
                        if (m < p.M) {
                            float v = 0.0f;
                            for (int s = 0; s < S; ++s)     // part order: deterministic
                                v += (s == part) ? acc[m] : recv_g[(s * BN + m) * R + r_local];
                            store(m, v);
                        }
                    }
                }
                named_barrier(1, kEpilogueThreads);         // this CTA's owners are done reading
                if (et == 0)
                    for (int r = 0; r < S; ++r)
                        if (r != part) mbar_arrive_remote(map_to_rank(bar_redfree, r));
            } else {
                float* slot = p.partials + (static_cast<int64_t>(tile) * S + part) * (BN * kTileRows);
#pragma unroll
                for (int m = 0; m < BN; ++m)
                    if (m < p.M) __stcg(slot + m * kTileRows + row_in_tile, acc[m]);
                // The CTA barrier orders every thread's partial stores before thread 0's
                // release; the acquire side is the same atomic followed by the second barrier.
                named_barrier(1, kEpilogueThreads);
                if (et == 0) {
                    const unsigned t = ticket_acq_rel(p.tickets + tile);
                    s_last = (t == static_cast<unsigned>(S) - 1u) ? 1 : 0;
                    if (s_last) p.tickets[tile] = 0u;
                }
                named_barrier(1, kEpilogueThreads);
                if (s_last) {
                    // all loads first (independent, many in flight), parts added in part order
                    const float* base = p.partials + static_cast<int64_t>(tile) * S * (BN * kTileRows);
#pragma unroll
                    for (int m = 0; m < BN; ++m) acc[m] = 0.0f;
                    for (int s = 0; s < S; ++s) {
#pragma unroll
                        for (int m = 0; m < BN; ++m)
                            if (m < p.M)
                                acc[m] += __ldcg(base + s * (BN * kTileRows) + m * kTileRows + row_in_tile);
                    }
#pragma unroll
                    for (int m = 0; m < BN; ++m)
                        if (m < p.M) store(m, acc[m]);
                }
                named_barrier(1, kEpilogueThreads);
            }
        }
    }

    if (warp == 2) TRACE(9);
    if (wf.failed && lane == 0) atomicExch(&g_packed_status, 1);
    tc_fence_before();
    __syncthreads();
    // no CTA leaves while a peer may still write to its shared memory or its barriers
    if (kCluster) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

struct PackedPlan { int splits, grid, bn; size_t smem; bool cluster; };
// Off by default: measured slower than the ticket path on B200 (cluster scheduling
// granularity and lock-step between the CTAs of a cluster); kept selectable for study.
int g_packed_use_cluster = 0;
int g_force_packed_splits = 0;
int g_packed_ctas_per_sm = 2;

// Parts of at most kMaxPartBlocks K blocks; among the admissible split counts take the
// one that keeps the most SMs busy (fewer parts on a tie).
bool plan_packed(int M, int N, int K, PackedPlan* plan) {
    const int bn = M <= 16 ? 16 : 32;
    const int per_sm = (bn == 16 && g_packed_ctas_per_sm == 2) ? 2 : 1;
    const int G = device_sm_count() * per_sm;
    const int tiles = N / kTileRows, kblocks = K / kBlockK;
    const int min_s = (kblocks + kMaxPartBlocks - 1) / kMaxPartBlocks;
    if (min_s > G) return false;
    // Estimated time of a split count, fitted to sweeps on B200: the CTAs make
    // ceil(units / G) rounds; a round streams one unit (largest K part) at the per-CTA share
    // of HBM bandwidth and pays about a microsecond for the partial-sum hand-over.
    int best = -1;
    double best_score = 1e30;
    const double kb_per_us = 6400.0 * 1000.0 / 1024.0 / G;      // KB per microsecond per CTA
    for (int s = min_s; s <= kblocks && s <= G && s <= 64; ++s) {
        const bool clusterable = (s == 2 || s == 4 || s == 8);
        if (g_packed_use_cluster && min_s <= 8 && s > 1 && !clusterable) continue;
        const int rounds = (tiles * s + G - 1) / G;
        const int unit_blocks = (kblocks + s - 1) / s;
        const double score = rounds * (unit_blocks * 18.0 / kb_per_us + (s > 1 ? 1.0 : 0.3)) + 0.01 * s;
        if (score < best_score) { best_score = score; best = s; }
    }
    if (g_force_packed_splits >= min_s && g_force_packed_splits <= kblocks && g_force_packed_splits <= G)
        best = g_force_packed_splits;
    if (best < 0) return false;
    plan->splits = best;
    plan->bn = bn;
    plan->cluster = g_packed_use_cluster && (best == 2 || best == 4 || best == 8);
    // whole clusters only; never more CTAs than there is work
    int clusters = G / best;
    if (clusters > tiles) clusters = tiles;
    plan->grid = plan->cluster ? clusters * best : G;
    const int sfb_stride = bn == 16 ? 256 : 512;
    plan->smem = static_cast<size_t>(kStages) * kStageBytes + kMaxPartBlocks * (bn * 128) +
                 (kMaxPartBlocks * 4 * sfb_stride + 256) + static_cast<size_t>(bn) * kTileRows * 4 + 1024;
    return true;
}

}  // namespace

size_t packed_weight_bytes(int N, int K) {
    return static_cast<size_t>(N / kTileRows) * (K / kBlockK) * kBlockBytes;
}

size_t packed_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || N % kTileRows || K % kBlockK) return 16;
    PackedPlan plan;
    if (!plan_packed(M < 32 ? M : 32, N, K, &plan)) return 16;
    const size_t tiles = N / kTileRows;
    const size_t tickets = (tiles * sizeof(unsigned) + 255) / 256 * 256;
    const size_t partials = plan.splits > 1 ? tiles * plan.splits * plan.bn * kTileRows * sizeof(float) : 0;
    return tickets + partials + 256;
}

cudaError_t launch_pack_weight(const void* w, const void* sf_flat, void* packed, int N, int K,
                               cudaStream_t stream) {
    const dim3 grid(static_cast<unsigned>(K / kBlockK), static_cast<unsigned>(N / kTileRows));
    pack_weight_kernel<<<grid, 1024, 0, stream>>>(static_cast<const uint8_t*>(w),
                                                  static_cast<const uint8_t*>(sf_flat),
                                                  static_cast<uint8_t*>(packed), N, K);
    return cudaGetLastError();
}

cudaError_t launch_linear_packed(const PackedLinearArgs& g, cudaStream_t stream, const char** why) {
    *why = nullptr;
    if (g.N % kTileRows != 0) { *why = "packed linear: N must be a multiple of 128"; return cudaSuccess; }
    if (g.K % kBlockK != 0) { *why = "packed linear: K must be a multiple of 256"; return cudaSuccess; }
    for (int m0 = 0; m0 < g.M; m0 += 32) {
        const int m = g.M - m0 < 32 ? g.M - m0 : 32;
        PackedPlan plan;
        if (!plan_packed(m, g.N, g.K, &plan)) { *why = "packed linear: K too large for this device"; return cudaSuccess; }
        PackedParams p = {};
        p.packed = static_cast<const uint8_t*>(g.packed);
        p.xb = g.xb;
        p.xb_stride = g.xb_stride;
        p.gs = g.gs;
        p.rcp_mode = g.rcp_mode;
        p.out = g.out;
        p.out_dtype = g.out_dtype;
        p.ldc = g.N;
        p.M = m;
        p.m0 = m0;
        p.N = g.N;
        p.K = g.K;
        p.alpha = g.alpha;
        p.tiles = g.N / kTileRows;
        p.splits = plan.splits;
        p.kblocks = g.K / kBlockK;
        p.pro_kind = g.pro_kind;
        p.delta = g.delta;
        p.residual_in = g.residual_in;
        p.residual_out = g.residual_out;
        p.norm_w = g.norm_w;
        p.eps = g.eps;
        const size_t tickets = (static_cast<size_t>(p.tiles) * sizeof(unsigned) + 255) / 256 * 256;
        p.tickets = static_cast<unsigned*>(g.workspace);
        p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(g.workspace) + tickets);

        void (*kern)(PackedParams) =
            plan.bn == 16 ? (plan.cluster ? linear_packed_kernel<16, true> : linear_packed_kernel<16, false>)
                          : (plan.cluster ? linear_packed_kernel<32, true> : linear_packed_kernel<32, false>);
        static bool attr_done[4][64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const int ki = (plan.bn == 16 ? 0 : 1) + (plan.cluster ? 2 : 0);
        if (dev >= 0 && dev < 64 && !attr_done[ki][dev]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            if (e != cudaSuccess) return e;
            attr_done[ki][dev] = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
        cfg.blockDim = dim3(kThreadsP);
        cfg.dynamicSmemBytes = plan.smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        int na = 0;
        if (gemv_tuning().use_pdl) {
            attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[na].val.programmaticStreamSerializationAllowed = 1;
            ++na;
        }
        if (plan.cluster) {
            attr[na].id = cudaLaunchAttributeClusterDimension;
            attr[na].val.clusterDim.x = static_cast<unsigned>(plan.splits);
            attr[na].val.clusterDim.y = 1;
            attr[na].val.clusterDim.z = 1;
            ++na;
        }
        cfg.attrs = attr;
        cfg.numAttrs = na;
        e = cudaLaunchKernelEx(&cfg, kern, p);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

void set_packed_tuning(int splits) {
    g_force_packed_splits = splits & 0xff;
    g_packed_ctas_per_sm = ((splits >> 9) & 1) ? 1 : 2;
    g_packed_use_cluster = ((splits >> 10) & 1) ? 1 : 0;
    const int trace = (splits >> 8) & 1;
    cudaMemcpyToSymbol(g_packed_trace, &trace, sizeof(int));
}

cudaError_t read_packed_trace(unsigned long long* out16) {
    return cudaMemcpyFromSymbol(out16, g_packed_times, 64 * sizeof(unsigned long long));
}

cudaError_t read_and_clear_packed_status(int* flag) {
    cudaError_t e = cudaMemcpyFromSymbol(flag, g_packed_status, sizeof(int));
    if (e != cudaSuccess) return e;
    const int zero = 0;
    return cudaMemcpyToSymbol(g_packed_status, &zero, sizeof(int));
}

}  // namespace nvfp4r
