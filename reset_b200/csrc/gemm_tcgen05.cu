// Small-M NVFP4 W4A4 linear on the 5th-generation tensor cores (sm_100a).
//
//   out[m, n] = alpha * sum_k dq(W[n, k]) * dq(X[m, k])        M <= 32 per pass
//
// The weight is the 128-row "A" operand of tcgen05.mma kind::mxf4nvf4 (block scale,
// one ue4m3 scale per 16 elements, scale_vec::4X); the M decode tokens are the
// N = 16 or 32 columns of the "B" operand. Nothing is decoded on the CUDA cores: weight
// codes travel TMA -> 128B-swizzled shared memory -> tensor core, weight scales travel
// bulk copy -> shared memory -> tcgen05.cp -> tensor memory, and the fp32 accumulator
// lives in tensor memory. The kernel is a weight stream bounded by HBM bandwidth.
//
// Persistent CTAs, one per SM, three roles:
//   warp 0      producer: TMA of weight tiles (128 rows x 256 K-elements, 16 KB) and
//               their 2 KB of block scales into a ring of shared-memory stages
//   warp 1      MMA issuer: per stage 8 x tcgen05.cp (scales) + 4 x tcgen05.mma, commit
//               to the stage's "empty" barrier; double-buffered accumulator
//   warps 2-5   epilogue: tcgen05.ld, alpha, store (or split-K partial + ticket)
// Prologue (all threads): the activations of this CTA's K range are quantized from bf16
// (or copied, if already quantized) straight into the swizzled B-operand layout and the
// 128x4 scale-chunk layout in shared memory, where they stay for the whole kernel.
//
// Work split: tile t = 128 weight rows; each tile's K range is cut into `splits` parts;
// CTA c always works on part c % splits (so its activations are loaded once) and walks
// the tiles round-robin within its part group. With splits > 1 every part writes its
// fp32 partial tile to scratch and takes a ticket; the last arriver adds the parts in
// part order (deterministic) and writes the result.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "kernels.h"
#include "status_mirror.cuh"
#include "quant_core.cuh"
#include "tcgen05_ptx.cuh"

namespace nvfp4r {
namespace {

constexpr int kTileRows = 128;
constexpr int kBK = 256;                         // K elements per pipeline stage
constexpr int kStageA = kTileRows * (kBK / 2);   // 16384 B of codes
constexpr int kStageSF = kTileRows * (kBK / 16); // 2048 B of scales (4 chunks of 512 B)
constexpr int kStageBytes = kStageA + kStageSF;  // 18432 = 18 * 1024
constexpr int kMaxStages = 10;
constexpr int kThreadsTc = 192;
constexpr int kEpilogueThreads = 128;
constexpr int kMaxSplits = 16;
constexpr int kSmemLimit = 227 * 1024 - 2048;     // dynamic part; the rest is static

struct alignas(64) TcParams {
    CUtensorMap tmap_w;        // weight codes as {256 elems, N rows, K/256 chunks}
    const uint8_t* wsf;        // swizzled weight scales
    const void* xb;            // bf16 activations (fused quantizer) or nullptr
    int64_t xb_stride;
    const float* gs;
    int rcp_mode;
    const uint8_t* a_codes;    // pre-quantized activations [M, K/2] (xb == nullptr)
    const uint8_t* a_sf;       // their swizzled scales
    void* out;
    int out_dtype;
    int c_n_major;             // element (m, n) at out[n*ldc + m] instead of out[m*ldc + n]
    int64_t ldc;
    int M;                     // rows of this pass (<= BN)
    int m0;                    // first activation row of this pass
    int N, K;
    float alpha;
    int tiles, splits, iters;  // N/128, K-parts per tile, K/256
    int stages;
    float* partials;           // [tiles][splits][BN][128] fp32
    unsigned* tickets;         // [tiles]
};

__device__ int g_tc_status = 0;

using namespace tc;

// -------------------------------------------------------------------------------

template <int BN>
__global__ void __launch_bounds__(kThreadsTc, 1)
linear_tc_kernel(const __grid_constant__ TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // carve: [ring][B tile][B scales]; the dynamic base is 1024-aligned by declaration,
    // re-aligned here in case the static part shifts it
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));

    __shared__ __align__(8) uint64_t bars[2 * kMaxStages + 4];
    __shared__ uint32_t s_tmem;
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid / kWarp, lane = tid % kWarp;
    const int G = gridDim.x, c = blockIdx.x;
    const int S = p.splits;
    const int part = c % S, rank_in_part = c / S;
    const int ctas_in_part = (G - part + S - 1) / S;
    const int it0 = static_cast<int>((static_cast<int64_t>(p.iters) * part) / S);
    const int it1 = static_cast<int>((static_cast<int64_t>(p.iters) * (part + 1)) / S);
    const int n_it = it1 - it0;                        // stages per tile for this CTA
    const int my_tiles = (rank_in_part < p.tiles)
                             ? (p.tiles - rank_in_part + ctas_in_part - 1) / ctas_in_part : 0;

    const uint32_t ring = smem_base;
    const uint32_t b_tile = ring + p.stages * kStageBytes;         // n_it chunks of BN x 128 B
    const uint32_t b_sf = b_tile + n_it * (BN * 128);              // n_it*4 chunks of 512 B
    uint8_t* b_tile_g = smem + p.stages * kStageBytes;
    uint8_t* b_sf_g = b_tile_g + n_it * (BN * 128);

    const uint32_t bar_full = smem_u32(&bars[0]);
    const uint32_t bar_empty = smem_u32(&bars[kMaxStages]);
    const uint32_t bar_accfull = smem_u32(&bars[2 * kMaxStages]);
    const uint32_t bar_accempty = smem_u32(&bars[2 * kMaxStages + 2]);

    constexpr uint32_t kTmemCols = (BN == 16) ? 64 : 128;
    constexpr uint32_t kColSFA = 2 * BN;
    constexpr uint32_t kColSFB = 2 * BN + 16;

    if (warp == 0 && lane == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_accfull + 8 * b, 1);
            mbar_init(bar_accempty + 8 * b, kEpilogueThreads / kWarp);
        }
        mbar_fence_init();
        asm volatile("prefetch.tensormap [%0];" :: "l"(&p.tmap_w) : "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    const uint64_t policy = l2_policy_evict_first();
    const int total = my_tiles * n_it;                 // stages this CTA consumes

    auto issue = [&](int i) {                          // producer: stage i of the CTA's sequence
        const int ti = i / n_it, it = it0 + (i - ti * n_it);
        const int tile = rank_in_part + ti * ctas_in_part;
        const int s = i % p.stages;
        const uint32_t dst = ring + s * kStageBytes;
        mbar_expect_tx(bar_full + 8 * s, kStageBytes);
        tma_load_3d(dst, &p.tmap_w, 0, tile * kTileRows, it, bar_full + 8 * s, policy);
        bulk_g2s(dst + kStageA,
                 p.wsf + (static_cast<int64_t>(tile) * (p.K / 64) + it * 4) * 512, kStageSF,
                 bar_full + 8 * s, policy);
    };

    // The weight stream does not depend on the preceding kernel: fill the ring now.
    int issued = 0;
    if (warp == 0 && lane == 0) {
        const int first = min(p.stages, total);
        for (; issued < first; ++issued) issue(issued);
    }
    pdl_launch_dependents();
    pdl_wait_prior();

    // ---- prologue: activations of K range [it0*256, it1*256) into operand layout -------
    {
        // zero the scale chunks first (rows >= M and unused row groups must not be NaN)
        for (int i = tid; i < n_it * 4 * 512 / 16; i += kThreadsTc)
            reinterpret_cast<uint4*>(b_sf_g)[i] = make_uint4(0, 0, 0, 0);
        for (int i = tid; i < n_it * BN * 128 / 16; i += kThreadsTc)
            reinterpret_cast<uint4*>(b_tile_g)[i] = make_uint4(0, 0, 0, 0);
        __syncthreads();
        const int kb0 = it0 * (kBK / 16);              // first 16-element block of the range
        const int blocks = n_it * (kBK / 16);
        if (p.xb != nullptr) {
            const float gs = __ldg(p.gs);
            const QuantScales qe = make_quant_scales<kRcpExact>(gs);
            const QuantScales qa = make_quant_scales<kRcpApprox>(gs);
            const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(p.xb);
            for (int i = tid; i < p.M * blocks; i += kThreadsTc) {
                const int m = i / blocks, blk = i - m * blocks;
                const uint4* src = reinterpret_cast<const uint4*>(
                    xb + (p.m0 + m) * p.xb_stride + static_cast<int64_t>(kb0 + blk) * 16);
                const uint4 lo = __ldg(src), hi = __ldg(src + 1);
                uint32_t cw[2];
                const uint32_t sf = (p.rcp_mode == kRcpExact)
                                        ? quantize_block16<kRcpExact>(lo, hi, qe, cw)
                                        : quantize_block16<kRcpApprox>(lo, hi, qa, cw);
                const int chunk = blk >> 4, b = (blk & 15) * 8;         // byte within 128-B row
                *reinterpret_cast<uint2*>(b_tile_g + chunk * (BN * 128) + swz128(m, b)) =
                    make_uint2(cw[0], cw[1]);
                b_sf_g[(blk >> 2) * 512 + m * 16 + (blk & 3)] = static_cast<uint8_t>(sf);
            }
        } else {
            // codes: 16-byte units of each row's K range
            const int units = n_it * 8;                                // 16-B units per row
            for (int i = tid; i < p.M * units; i += kThreadsTc) {
                const int m = i / units, u = i - m * units;
                const uint4 v = ldg_keep_16(p.a_codes + static_cast<int64_t>(p.m0 + m) * (p.K / 2) +
                                            static_cast<int64_t>(it0) * 128 + u * 16);
                *reinterpret_cast<uint4*>(b_tile_g + (u >> 3) * (BN * 128) + swz128(m, (u & 7) * 16)) = v;
            }
            // scales: row (m0+m) of the swizzled source -> row m (lane m, column 0) here
            for (int i = tid; i < p.M * n_it * 4; i += kThreadsTc) {
                const int m = i / (n_it * 4), ch = i - m * (n_it * 4);
                const int r = p.m0 + m;
                const uint8_t* src = p.a_sf + (static_cast<int64_t>(r / 128) * (p.K / 64) + it0 * 4 + ch) * 512 +
                                     (r % 32) * 16 + ((r % 128) / 32) * 4;
                *reinterpret_cast<uint32_t*>(b_sf_g + ch * 512 + m * 16) =
                    __ldg(reinterpret_cast<const uint32_t*>(src));
            }
        }
        fence_proxy_async_smem();
        __syncthreads();
    }

    WaitFail wf;
    if (warp == 0) {
        // ---------------- producer -------------------------------------------------------
        if (lane == 0) {
            for (int i = issued; i < total; ++i) {
                const int s = i % p.stages;
                if (!wf.wait(bar_empty + 8 * s, ((i / p.stages) - 1) & 1)) break;
                issue(i);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer -----------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                       (static_cast<uint32_t>(kTileRows >> 7) << 27);
            int i = 0;
            for (int ti = 0; ti < my_tiles && !wf.failed; ++ti) {
                const int buf = ti & 1;
                if (ti >= 2 && !wf.wait(bar_accempty + 8 * buf, ((ti >> 1) - 1) & 1)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem + buf * BN;
                for (int j = 0; j < n_it; ++j, ++i) {
                    const int s = i % p.stages;
                    if (!wf.wait(bar_full + 8 * s, (i / p.stages) & 1)) break;
                    tc_fence_after();
                    const uint32_t a_smem = ring + s * kStageBytes;
                    const uint32_t sfa_smem = a_smem + kStageA;
                    const uint32_t b_smem = b_tile + j * (BN * 128);
                    const uint32_t sfb_smem = b_sf + j * 4 * 512;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        tc_cp_scales(tmem + kColSFA + 4 * k, desc_scales(sfa_smem + k * 512));
                        tc_cp_scales(tmem + kColSFB + 4 * k, desc_scales(sfb_smem + k * 512));
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        tc_mma_nvf4(d_tmem, desc_operand(a_smem + k * 32), desc_operand(b_smem + k * 32),
                                    idesc, tmem + kColSFA + 4 * k, tmem + kColSFB + 4 * k,
                                    (j > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_empty + 8 * s);
                }
                tc_commit(bar_accfull + 8 * buf);
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ------------------------------------------
        const int q = warp & 3;                        // TMEM lane quadrant this warp may read
        const int row_in_tile = q * 32 + lane;
        const int et = tid - 2 * kWarp;                // 0..127
        for (int ti = 0; ti < my_tiles; ++ti) {
            const int buf = ti & 1;
            const int tile = rank_in_part + ti * ctas_in_part;
            if (!wf.wait(bar_accfull + 8 * buf, (ti >> 1) & 1)) break;
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
                const int64_t idx = p.c_n_major ? n * p.ldc + (p.m0 + m) : (p.m0 + m) * p.ldc + n;
                v *= p.alpha;
                if (p.out_dtype == 0) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(v);
                else if (p.out_dtype == 1) static_cast<__half*>(p.out)[idx] = __float2half_rn(v);
                else static_cast<float*>(p.out)[idx] = v;
            };
            if (S == 1) {
#pragma unroll
                for (int m = 0; m < BN; ++m)
                    if (m < p.M) store(m, acc[m]);
            } else {
                float* slot = p.partials + (static_cast<int64_t>(tile) * S + part) * (BN * kTileRows);
#pragma unroll
                for (int m = 0; m < BN; ++m)
                    if (m < p.M) __stcg(slot + m * kTileRows + row_in_tile, acc[m]);
                __threadfence();
                named_barrier(1, kEpilogueThreads);
                if (et == 0) {
                    const unsigned t = atomicAdd(p.tickets + tile, 1u);
                    s_last = (t == static_cast<unsigned>(S) - 1u) ? 1 : 0;
                    if (s_last) p.tickets[tile] = 0u;   // leave the scratch ready for the next call
                    __threadfence();
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
                named_barrier(1, kEpilogueThreads);    // s_last is reused by the next tile
            }
        }
    }

    if (wf.failed && lane == 0) report_timeout(&g_tc_status, 2);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// ---- host side ------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(sym);
    });
    return fn;
}

struct MapKey {
    const void* ptr; int N, K, dev;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && N == o.N && K == o.K && dev == o.dev; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (static_cast<size_t>(k.N) * 1000003u) ^
               (static_cast<size_t>(k.K) * 7919u) ^ static_cast<size_t>(k.dev);
    }
};

// The descriptor depends on (pointer, N, K) only; encoding is host arithmetic, the cache
// just keeps it off the per-call path.
bool weight_map(const void* w, int N, int K, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    const MapKey key{w, N, K, dev};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeFn fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[3] = {256, static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(K / 256)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(K / 2), 128};
    const cuuint32_t box[3] = {256, static_cast<cuuint32_t>(kTileRows), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B, 3, const_cast<void*>(w), dims, strides,
                          box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

struct Plan { int splits, stages, grid, bn; size_t smem; };
int g_force_splits = 0, g_force_stages = 0;

// Choose the K split: smallest number of parts whose unit count fills the SMs well and
// whose per-CTA activation footprint leaves room for a deep ring.
bool make_plan(int M, int N, int K, Plan* plan) {
    const int G = device_sm_count();
    const int tiles = N / kTileRows, iters = K / kBK;
    const int bn = M <= 16 ? 16 : 32;
    int best = -1;
    double best_eff = -1.0;
    for (int s = 1; s <= kMaxSplits && s <= iters; ++s) {
        const int n_it = (iters + s - 1) / s;
        const size_t act = static_cast<size_t>(n_it) * (bn * 128 + 4 * 512);
        if (act + 4 * kStageBytes + 2048 > static_cast<size_t>(kSmemLimit)) continue;
        // CTAs of part p walk `tiles` tiles with about G/s CTAs: rounds = ceil(tiles / (G/s))
        const int per_part = G / s > 0 ? G / s : 1;
        const int rounds = (tiles + per_part - 1) / per_part;
        const double eff = static_cast<double>(tiles) * s / (static_cast<double>(rounds) * G) ;
        const double score = eff - 0.01 * (s - 1);     // prefer fewer parts at equal fill
        if (score > best_eff) { best_eff = score; best = s; }
    }
    if (g_force_splits > 0 && g_force_splits <= iters) best = g_force_splits;
    if (best < 0) return false;
    const int n_it = (iters + best - 1) / best;
    const size_t act = static_cast<size_t>(n_it) * (bn * 128 + 4 * 512);
    int stages = static_cast<int>((kSmemLimit - 2048 - act) / kStageBytes);
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > 2 * n_it + 2 && stages > 4) stages = 2 * n_it + 2 > 4 ? 2 * n_it + 2 : 4;
    if (g_force_stages > 0 && g_force_stages < stages) stages = g_force_stages;
    plan->splits = best;
    plan->stages = stages;
    plan->bn = bn;
    plan->grid = G < tiles * best ? G : tiles * best;
    plan->smem = static_cast<size_t>(stages) * kStageBytes + act + 1024;
    return true;
}

}  // namespace

size_t gemm_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || N % kTileRows || K % kBK) return 16;
    Plan plan;
    if (!make_plan(M < 32 ? M : 32, N, K, &plan)) return 16;
    const size_t tiles = N / kTileRows;
    const size_t tickets = (tiles * sizeof(unsigned) + 255) / 256 * 256;
    const size_t partials = plan.splits > 1 ? tiles * plan.splits * plan.bn * kTileRows * sizeof(float) : 0;
    return tickets + partials + 256;
}

cudaError_t launch_linear_tc(const TcLinearArgs& g, cudaStream_t stream, const char** why) {
    *why = nullptr;
    if (g.N % kTileRows != 0) { *why = "tensor-core path: N must be a multiple of 128"; return cudaSuccess; }
    if (g.K % kBK != 0) { *why = "tensor-core path: K must be a multiple of 256"; return cudaSuccess; }
    CUtensorMap map;
    if (!weight_map(g.w, g.N, g.K, &map)) { *why = "tensor-core path: cuTensorMapEncodeTiled failed"; return cudaSuccess; }

    for (int m0 = 0; m0 < g.M; m0 += 32) {
        const int m = g.M - m0 < 32 ? g.M - m0 : 32;
        Plan plan;
        if (!make_plan(m, g.N, g.K, &plan)) { *why = "tensor-core path: no plan fits shared memory"; return cudaSuccess; }
        TcParams p = {};
        p.tmap_w = map;
        p.wsf = static_cast<const uint8_t*>(g.wsf_swizzled);
        p.xb = g.xb;
        p.xb_stride = g.xb_stride;
        p.gs = g.gs;
        p.rcp_mode = g.rcp_mode;
        p.a_codes = static_cast<const uint8_t*>(g.a_codes);
        p.a_sf = static_cast<const uint8_t*>(g.a_sf_swizzled);
        p.out = g.out;
        p.out_dtype = g.out_dtype;
        p.c_n_major = g.c_n_major ? 1 : 0;
        p.ldc = g.c_n_major ? g.M : g.N;
        p.M = m;
        p.m0 = m0;
        p.N = g.N;
        p.K = g.K;
        p.alpha = g.alpha;
        p.tiles = g.N / kTileRows;
        p.splits = plan.splits;
        p.iters = g.K / kBK;
        p.stages = plan.stages;
        const size_t tickets = (static_cast<size_t>(p.tiles) * sizeof(unsigned) + 255) / 256 * 256;
        p.tickets = static_cast<unsigned*>(g.workspace);
        p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(g.workspace) + tickets);

        void (*kern)(TcParams) = plan.bn == 16 ? linear_tc_kernel<16> : linear_tc_kernel<32>;
        static bool attr_done[2][64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const int ki = plan.bn == 16 ? 0 : 1;
        if (dev >= 0 && dev < 64 && !attr_done[ki][dev]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
            if (e != cudaSuccess) return e;
            attr_done[ki][dev] = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
        cfg.blockDim = dim3(kThreadsTc);
        cfg.dynamicSmemBytes = plan.smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = gemv_tuning().use_pdl ? 1 : 0;
        e = cudaLaunchKernelEx(&cfg, kern, p);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

void set_tc_tuning(int splits, int stages) {
    g_force_splits = splits;
    g_force_stages = stages;
}

cudaError_t set_status_mirror_tc(int* p) { return set_status_mirror_here(p); }

cudaError_t read_and_clear_tc_status(int* flag) {
    cudaError_t e = cudaMemcpyFromSymbol(flag, g_tc_status, sizeof(int));
    if (e != cudaSuccess) return e;
    const int zero = 0;
    return cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
}

}  // namespace nvfp4r
