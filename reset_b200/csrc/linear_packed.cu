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
// K may end in the middle of a block (K % 128 == 0, e.g. the 3200-wide row-parallel shard of
// Qwen3-32B at TP = 8): the last block is then half zeros (codes and scales), and the linear
// quantizes zeros for the activation blocks past K, so the padding adds nothing to the sums.
// Consecutive K blocks of a tile are contiguous, so a pipeline stage of 1 or 2 blocks is
// ONE 1-D bulk copy of 18 or 36 KB: perfectly sequential DRAM reads, one TMA instruction
// and one mbarrier transaction per 36 KB, no tensor map.
//
// Why this shape (measured on B200):
//   * a thread that issues bulk copies is held ~190 cycles per copy and the MMA thread
//     spends some hundred cycles per stage on barrier wait + commit regardless of the work
//     in it, so stages must be few and large;
//   * shared memory per CTA stays under half an SM (two 36 KB stages + the activations of
//     a K part of at most 2048 elements) so that the CTA of the NEXT linear, launched with
//     programmatic stream serialization, becomes resident while this one still runs and
//     starts pulling its own weights at once;
//   * every phase of a decode-sized launch runs ONCE per CTA, so its instructions are
//     fetched cold: straight-line code that runs once costs about 8 cycles per instruction
//     (measured: 15 KB of unrolled epilogue took 4 us). The kernel is therefore written for
//     small code: loops are not unrolled unless that removes a memory round trip, there is
//     one quantizer instance, and accumulators are read from tensor memory four tokens at
//     a time instead of into a register image of the whole tile;
//   * the activation block scales are copied into tensor memory once per kernel and stay
//     there (128 columns), the weight scales ride with each stage.
//
// Grid: persistent CTAs, two per SM. CTA c works on K part c % S of tiles
// c / S, c / S + G/S, ... Roles: warp 0 = bulk-copy producer, warp 1 = MMA issuer,
// warps 2-5 = epilogue (one TMEM lane quadrant each).
#include "../../include/nvfp4r_b200.h"
#include "kernels.h"
#include "status_mirror.cuh"
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
constexpr int kWarpsP = kThreadsP / 32;

struct PackedParams {
    const uint8_t* packed;
    const void* xb;            // bf16 [M, K] (prologue 0) or [M, 2K] (prologue 2)
    int64_t xb_stride;
    const float* gs;
    int rcp_mode;
    void* out;
    int out_dtype;
    int64_t ldc;               // elements between tokens in out
    int M, m0, N, K;
    float alpha;
    // work split, computed on the host: S parts of kb_q or kb_q + 1 K blocks (the first
    // kb_r parts have one more), ctas_per_part CTAs per part
    int tiles, splits, kblocks, ctas_per_part, kb_q, kb_r;
    // the same split without divisions in the kernel: ceil(2^32 / splits) (exact quotients for
    // CTA indices below 2^16), and tiles = tiles_q * ctas_per_part + tiles_r
    uint32_t inv_splits;
    int tiles_q, tiles_r;
    // ceil(2^20 / (16 * K blocks of a part)) for parts of kb_q + 1 and of kb_q blocks
    uint32_t inv_blocks_hi, inv_blocks_lo;
    unsigned long long* slots; // split-K hand-over slots {flag:32 | fp32 bits:32}, all zero between launches
    // fused prologue (what produces the bf16 activations that get quantized)
    int pro_kind;                  // 0: xb as is; 1: RMSNorm(residual_in + delta) * norm_w; 2: silu(g) * u
    const void* delta;             // kind 1: bf16 [M, K] or nullptr
    const void* residual_in;       // kind 1: bf16 [M, K]
    void* residual_out;            // kind 1: bf16 [M, K], receives residual_in + delta
    const void* norm_w;            // kind 1: bf16 [K]
    float eps;
    // fused first half of the tensor-parallel sum exchange (row-parallel linears): instead of
    // writing `out`, the CTA that finishes a tile stores its bf16 results, two per 64-bit slot
    // {1 : bf16x2}, into the receive memory of every rank (layout and protocol of
    // peer_allreduce.cu); the gather half of nvfp4r_peer_allreduce_bf16 completes the sum.
    int push_world, push_rank;
    unsigned long long push_max_pairs;
    unsigned char* push_base[NVFP4R_PEER_MAX_WORLD];
    // push_gather != 0: the thread that pushed a pair also completes it: it polls the W
    // contributions to that pair in this rank's own receive memory, adds them in rank order in
    // fp32, rounds once, writes `out` and zeroes the slots, and the last CTA of the grid advances
    // the call counter - the whole all-reduce inside this launch, no gather kernel after it.
    int push_gather;
    uint32_t push_poll_limit;
    // stages beyond the ring that the producer asks L2 to fetch before the activations are ready
    int l2_stages;
};

__device__ int g_packed_status = 0;
// Optional time line (nanoseconds of %globaltimer) of eight consecutive CTAs, compiled in only
// with -DNVFP4R_TRACE (the default build carries none of it): filled when g_packed_trace != 0,
// CTAs base .. base+7 with base = g_packed_trace - 1 (a multiple of 8), the last four launches
// each.
#ifdef NVFP4R_TRACE
__device__ int g_packed_trace = 0;
__device__ unsigned long long g_packed_times[8 * 4 * 16];
__device__ unsigned g_packed_launch[8] = {};
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TRACE(slot) do { if (trace) g_packed_times[((blockIdx.x & 7) * 4 + (launch_id & 3)) * 16 + (slot)] = gtime(); } while (0)
#else
#define TRACE(slot) do { } while (0)
#endif

// ---- one-time re-layout ----------------------------------------------------------

// One thread moves one 16-byte unit of codes; the threads with unit < 4 also move four
// scale bytes. grid = (K/256, N/128), block = 1024 threads (128 rows x 8 units).
__global__ void __launch_bounds__(1024)
pack_weight_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ sf_flat,
                   uint8_t* __restrict__ packed, int N, int K) {
    const int kb = blockIdx.x, tile = blockIdx.y;
    const int row = threadIdx.x >> 3, unit = threadIdx.x & 7;
    const int kblocks = (K + kBlockK - 1) / kBlockK;           // the last block may be half padding
    uint8_t* dst = packed + (static_cast<int64_t>(tile) * kblocks + kb) * kBlockBytes;
    const int64_t n = static_cast<int64_t>(tile) * kTileRows + row;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (kb * 128 + unit * 16 < K / 2) v = *reinterpret_cast<const uint4*>(w + n * (K / 2) + kb * 128 + unit * 16);
    *reinterpret_cast<uint4*>(dst + swz128(row, unit * 16)) = v;
    // scales: 16 per row in this block = 4 chunks x 4; threads with unit < 4 move 4 bytes
    if (unit < 4) {
        uint32_t s4 = 0;
        if (kb * 16 + unit * 4 < K / 16)
            s4 = *reinterpret_cast<const uint32_t*>(sf_flat + n * (K / 16) + kb * 16 + unit * 4);
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
// bf16(a + b) for eight packed values: one rounding of the exact sum per element, the same bits as
// adding in fp32 and rounding to bf16 (the sum of two bf16 values is exact in fp32 unless one is
// below a quarter ulp of the other, where both give the larger operand).
__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint4 add_bf16x8(const uint4& a, const uint4& b) {
    return make_uint4(add_bf16x2(a.x, b.x), add_bf16x2(a.y, b.y), add_bf16x2(a.z, b.z), add_bf16x2(a.w, b.w));
}

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float v[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(taddr) : "memory");
}

// ---- split-K hand-over through self-validating 8-byte slots ------------------------------
// Token m of a tile is finished by the CTA of K part m % S. The other parts publish their
// partial value for it as ONE 64-bit store {flag = 1 : fp32 bits}; the finishing CTA polls
// those slots, adds all S values in part order and writes zeros back, so the scratch is
// all-zero again when the kernel ends. A 64-bit
// scalar access is single-copy atomic, so a slot is either still zero or complete: no
// fence, no ticket, one store latency plus one load latency on the critical path. All CTAs
// of the grid are resident at once (the grid never exceeds two CTAs per SM), so the part
// the poll waits for is running; the poll is bounded all the same.
__device__ __forceinline__ void slot_store(unsigned long long* p, float v) {
    const unsigned long long w = (1ull << 32) | static_cast<unsigned long long>(__float_as_uint(v));
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(w) : "memory");
}
// Poll of a slot that a peer GPU writes (system scope).
__device__ __forceinline__ unsigned long long peer_poll(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ unsigned long long slot_load(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
constexpr uint32_t kSlotPollLimit = 4000000u;      // polls per group before giving up (~ a second)

// Sum of one token's partial values over the parts 0..S-1 in ascending part order for this
// thread's weight row: `own` stands at position `part`, the others come from the slots
// (`tok` points at the slot of (token, part 0, this row); parts are kTileRows slots apart).
// Eight parts are polled together (all loads in flight at once: one round trip per group).
// Gathering two tokens per call was measured slower (more registers and code for the same
// number of round trips on the shapes of the bench).
__device__ __forceinline__ bool token_gather(unsigned long long* tok, int S, int part, float own, float* result) {
    float acc = 0.0f;
#pragma unroll 1
    for (int s0 = 0; s0 < S; s0 += 8) {
        unsigned long long w[8];
#pragma unroll
        for (int g = 0; g < 8; ++g)
            if (s0 + g < S && s0 + g != part) w[g] = slot_load(tok + (s0 + g) * kTileRows);
        for (uint32_t it = 0;; ++it) {
            bool all = true;
#pragma unroll
            for (int g = 0; g < 8; ++g)
                if (s0 + g < S && s0 + g != part && (w[g] >> 32) != 1ull) {
                    w[g] = slot_load(tok + (s0 + g) * kTileRows);
                    all = false;
                }
            if (all) break;
            if (it > kSlotPollLimit) return false;
        }
#pragma unroll
        for (int g = 0; g < 8; ++g)
            if (s0 + g < S) {
                if (s0 + g == part) {
                    acc += own;
                } else {
                    acc += __uint_as_float(static_cast<uint32_t>(w[g]));
                    tok[(s0 + g) * kTileRows] = 0ull;
                }
            }
    }
    *result = acc;
    return true;
}

// ---- the linear ---------------------------------------------------------------------

// kKind = p.pro_kind as a compile-time value: one kernel per prologue, so that each carries only
// its own prologue's code and registers (with the three in one kernel, a change to the plain
// path moved the RMSNorm path by up to 1.1 us per launch).
// kPush: how much of the tensor-parallel epilogue is compiled in: 0 none (single-GPU launches),
// 1 the push to the peers' receive memory, 2 the push and the sum in the same launch.
template <int BN, int kKind, int kPush>
__global__ void __launch_bounds__(kThreadsP, 2)
linear_packed_kernel(const __grid_constant__ PackedParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));

    __shared__ __align__(8) uint64_t bars[2 * kStages + 4 + kMaxPartBlocks / kBlocksPerStage];
    __shared__ uint32_t s_tmem;
    __shared__ float s_red[32 * 8];                    // RMSNorm: per token, per warp sum of squares

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef NVFP4R_TRACE
    __shared__ unsigned s_launch_id;
    const bool traced_cta = (g_packed_trace != 0) && (static_cast<int>(blockIdx.x) >> 3) == ((g_packed_trace - 1) >> 3);
    const bool trace = traced_cta && lane == 0;
    if (traced_cta) {
        if (tid == 0) s_launch_id = atomicAdd(&g_packed_launch[blockIdx.x & 7], 1u);
        __syncthreads();
    }
    const unsigned launch_id = traced_cta ? s_launch_id : 0u;
#endif
    if (warp == 0) TRACE(0);

    const int S = p.splits;
    const int rank = S == 1 ? static_cast<int>(blockIdx.x) : static_cast<int>(__umulhi(blockIdx.x, p.inv_splits));
    const int part = static_cast<int>(blockIdx.x) - rank * S;
    const int kb0 = part * p.kb_q + min(part, p.kb_r);
    const int nkb = p.kb_q + (part < p.kb_r ? 1 : 0);                   // 1 .. kMaxPartBlocks
    const int stages_per_tile = (nkb + kBlocksPerStage - 1) / kBlocksPerStage;
    const int cpp = p.ctas_per_part;
    const int my_tiles = rank < cpp ? p.tiles_q + (rank < p.tiles_r ? 1 : 0) : 0;
    const int total = my_tiles * stages_per_tile;

    const uint32_t ring = smem_base;
    const uint32_t b_tile = ring + kStages * kStageBytes;            // nkb blocks of BN x 128 B
    // activation scale chunks: tcgen05.cp reads 32 rows x 16 B per chunk, but only rows
    // < BN matter, so with BN == 16 consecutive chunks overlap by half (stride 256 B)
    constexpr int kSfbStride = (BN == 16) ? 256 : 512;
    const uint32_t b_sf = b_tile + kMaxPartBlocks * (BN * 128);
    uint8_t* b_tile_g = smem + kStages * kStageBytes;
    uint8_t* b_sf_g = b_tile_g + kMaxPartBlocks * (BN * 128);

    const uint32_t bar_full = smem_u32(&bars[0]);
    const uint32_t bar_empty = smem_u32(&bars[kStages]);
    const uint32_t bar_accfull = smem_u32(&bars[2 * kStages]);
    const uint32_t bar_accempty = smem_u32(&bars[2 * kStages + 2]);
    const uint32_t bar_sfb = smem_u32(&bars[2 * kStages + 4]);       // one per stage of the K part, used once

    constexpr uint32_t kTmemCols = 256;
    constexpr uint32_t kColSFA = 2 * BN;                              // 16 columns per block of a stage
    constexpr uint32_t kColSFB = kColSFA + 16 * kBlocksPerStage;      // 16 per block of the K part

    // producer state (kept by every lane of warp 0, one elected lane issues): next stage = K-block
    // pair p_j of this CTA's p_ti-th tile. Addresses and sizes are computed by the whole warp so
    // that they are warp-uniform values when the bulk copy takes them.
    int issued = 0, p_ti = 0, p_j = 0;
    if (warp == 0) TRACE(13);
    const uint64_t policy = l2_policy_evict_first();
    const bool lead0 = (warp == 0) && elect_one();
    auto issue_next = [&]() {
        const int tile = rank + p_ti * cpp;
        const int s = issued & (kStages - 1);
        const int nb = min(kBlocksPerStage, nkb - p_j * kBlocksPerStage);
        const uint32_t bytes = static_cast<uint32_t>(nb) * kBlockBytes;
        const uint8_t* src =
            p.packed + (static_cast<int64_t>(tile) * p.kblocks + kb0 + p_j * kBlocksPerStage) * kBlockBytes;
        if (lead0) {
            mbar_expect_tx(bar_full + 8 * s, bytes);
            bulk_g2s(ring + s * kStageBytes, src, bytes, bar_full + 8 * s, policy);
        }
        ++issued;
        if (++p_j == stages_per_tile) { p_j = 0; ++p_ti; }
    };

    // The weights do not depend on the previous kernel: warp 0 arms the barriers and starts
    // the first stages before anything else happens in this CTA.
    if (warp == 0) {
        // one barrier per lane (a rolled loop of eleven initialisations on one lane, fetched
        // cold, held the first copy back by 0.45 us); accempty counts one arrival per epilogue warp
        constexpr int kBars = 2 * kStages + 4 + kMaxPartBlocks / kBlocksPerStage;
        static_assert(kBars <= 32, "one barrier per lane");
        if (lane < kBars) {
            mbar_init(bar_full + 8 * lane, (lane >= 2 * kStages + 2 && lane < 2 * kStages + 4) ? 4u : 1u);
            mbar_fence_init();
        }
        __syncwarp();
        TRACE(14);
#pragma unroll 1
        while (issued < total && issued < kStages) issue_next();
    }
    // The layer's global scale is a constant of the layer, not a product of the previous kernel:
    // it is fetched here, under the ring set-up, instead of costing a trip to L2 after the wait.
    const float gs = __ldg(p.gs);
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem), kTmemCols);
    if (warp == 0) TRACE(1);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const bool exact = (p.rcp_mode == kRcpExact);
    const QuantScales q = exact ? make_quant_scales<kRcpExact>(gs) : make_quant_scales<kRcpApprox>(gs);
    // RMSNorm prologue: the norm weight is a constant of the layer too; the 16 weights of this
    // thread's first block are fetched before the wait (the other operands of that block come
    // out of L1 after the mean-square pass, so the norm weight was the prologue's second trip
    // to L2).
    uint4 nw_first0 = make_uint4(0, 0, 0, 0), nw_first1 = nw_first0;
    if (kKind == 1 && my_tiles > 0 && tid < p.M * nkb * (kBlockK / 16)) {
        const int blocks = nkb * (kBlockK / 16);
        const int blk = tid % blocks;
        if (kb0 * (kBlockK / 16) + blk < p.K / 16) {
            const uint4* src = reinterpret_cast<const uint4*>(
                static_cast<const __nv_bfloat16*>(p.norm_w) + static_cast<int64_t>(kb0 * (kBlockK / 16) + blk) * 16);
            nw_first0 = __ldg(src);
            nw_first1 = __ldg(src + 1);
        }
    }
    // Plain-input prologue: where this thread's first two activation blocks live is known before
    // the wait (only their contents are not), so the loads can go out the moment it returns.
    const uint4* pre_a = nullptr;
    const uint4* pre_b = nullptr;
    if (kKind == 0 && my_tiles > 0) {
        const int blk0 = kb0 * (kBlockK / 16), blocks = nkb * (kBlockK / 16);
        const int n_items = p.M * blocks, real = min(blocks, p.K / 16 - blk0);
        const uint32_t inv_blocks = part < p.kb_r ? p.inv_blocks_hi : p.inv_blocks_lo;
        auto where = [&](int i) -> const uint4* {
            if (i >= n_items) return nullptr;
            const int m = static_cast<int>((static_cast<uint32_t>(i) * inv_blocks) >> 20), blk = i - m * blocks;
            if (blk >= real) return nullptr;
            return reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.xb) + (p.m0 + m) * p.xb_stride +
                                                  static_cast<int64_t>(blk0 + blk) * 16);
        };
        pre_a = where(tid);
        pre_b = where(tid + kThreadsP);
    }
    // RMSNorm prologue: the residual and delta values of this thread's first block are requested
    // right after the wait, together with the loads of the mean-square pass, and kept for the
    // second pass (addresses worked out here).
    int64_t own_off = -1;
    if (kKind == 1 && my_tiles > 0) {
        const int blocks = nkb * (kBlockK / 16), blk0 = kb0 * (kBlockK / 16);
        if (tid < p.M * blocks) {
            const int m = tid / blocks, blk = tid - m * blocks;
            if (blk0 + blk < p.K / 16)
                own_off = static_cast<int64_t>(p.m0 + m) * p.K + static_cast<int64_t>(blk0 + blk) * 16;
        }
    }
    // SiLU prologue: likewise the gate and up values of this thread's first block (offset of the
    // gate block in the [M, 2K] input, -1 = none).
    int64_t silu_off = -1;
    if (kKind == 2 && my_tiles > 0) {
        const int blocks = nkb * (kBlockK / 16), blk0 = kb0 * (kBlockK / 16);
        if (tid < p.M * blocks) {
            const int m = tid / blocks, blk = tid - m * blocks;
            if (blk0 + blk < p.K / 16)
                silu_off = (p.m0 + m) * p.xb_stride + static_cast<int64_t>(blk0 + blk) * 16;
        }
    }
    // sources of the L2 run-ahead (the two stages after the ring in this CTA's sequence)
    const uint8_t* pf_src0 = nullptr;
    const uint8_t* pf_src1 = nullptr;
    uint32_t pf_bytes0 = 0, pf_bytes1 = 0;
    if (warp == 0) {
        int ti = p_ti, j = p_j;
        if (issued < total && p.l2_stages >= 1) {
            pf_src0 = p.packed + (static_cast<int64_t>(rank + ti * cpp) * p.kblocks + kb0 + j * kBlocksPerStage) * kBlockBytes;
            pf_bytes0 = static_cast<uint32_t>(min(kBlocksPerStage, nkb - j * kBlocksPerStage)) * kBlockBytes;
            if (++j == stages_per_tile) { j = 0; ++ti; }
            if (issued + 1 < total && p.l2_stages >= 2) {
                pf_src1 = p.packed + (static_cast<int64_t>(rank + ti * cpp) * p.kblocks + kb0 + j * kBlocksPerStage) * kBlockBytes;
                pf_bytes1 = static_cast<uint32_t>(min(kBlocksPerStage, nkb - j * kBlocksPerStage)) * kBlockBytes;
            }
        }
    }
    pdl_launch_dependents();
    pdl_wait_prior();
    uint4 a_lo = make_uint4(0, 0, 0, 0), a_hi = a_lo, b_lo = a_lo, b_hi = a_lo;
    if (pre_a != nullptr) { a_lo = __ldg(pre_a); a_hi = __ldg(pre_a + 1); }
    if (pre_b != nullptr) { b_lo = __ldg(pre_b); b_hi = __ldg(pre_b + 1); }
    uint4 own_r0 = make_uint4(0, 0, 0, 0), own_r1 = own_r0, own_d0 = own_r0, own_d1 = own_r0;
    if (kKind == 1 && own_off >= 0) {
        const __nv_bfloat16* rin_e = static_cast<const __nv_bfloat16*>(p.residual_in);
        own_r0 = __ldg(reinterpret_cast<const uint4*>(rin_e + own_off));
        own_r1 = __ldg(reinterpret_cast<const uint4*>(rin_e + own_off) + 1);
        if (p.delta != nullptr) {
            const __nv_bfloat16* dl_e = static_cast<const __nv_bfloat16*>(p.delta);
            own_d0 = __ldg(reinterpret_cast<const uint4*>(dl_e + own_off));
            own_d1 = __ldg(reinterpret_cast<const uint4*>(dl_e + own_off) + 1);
        }
    }
    if (kKind == 2 && silu_off >= 0) {
        // gate into own_r*, up into own_d* (the registers the RMSNorm instance uses for its own block)
        const __nv_bfloat16* gate = static_cast<const __nv_bfloat16*>(p.xb) + silu_off;
        own_r0 = __ldg(reinterpret_cast<const uint4*>(gate));
        own_r1 = __ldg(reinterpret_cast<const uint4*>(gate) + 1);
        own_d0 = __ldg(reinterpret_cast<const uint4*>(gate + p.K));
        own_d1 = __ldg(reinterpret_cast<const uint4*>(gate + p.K) + 1);
    }
    if (warp == 0) TRACE(2);
    // The ring is full until the first MMA frees a stage, which is the prologue away (load and
    // quantize the activations). The two stages that follow are asked into L2 now - not before
    // the wait, where they would compete with the last stages of the kernel before - so that
    // HBM keeps streaming through the prologue and the ring later refills from L2. (Their
    // addresses were worked out before the wait: warp 0 is part of the prologue.)
    if (lead0) {
        if (pf_bytes0 != 0) bulk_prefetch_l2(pf_src0, pf_bytes0);
        if (pf_bytes1 != 0) bulk_prefetch_l2(pf_src1, pf_bytes1);
    }

    // ---- prologue: quantize this part's activations into operand layout --------------
    if (my_tiles > 0) {
        const int blk0 = kb0 * (kBlockK / 16);
        const int blocks = nkb * (kBlockK / 16);
        const int n_items = p.M * blocks;
        // blocks of this part that lie inside K; the ones past it (K % 256 == 128, last part only)
        // are quantized from zeros, which gives zero codes and a zero scale
        const int real = min(blocks, p.K / 16 - blk0);
        // i / blocks as a multiply and a shift: exact for blocks = 16 .. 128 in steps of 16 and
        // i < 4608 (M <= 32 tokens of at most 128 blocks); a real division costs ~20 instructions
        // and the loop below needs two per block
        const uint32_t inv_blocks = part < p.kb_r ? p.inv_blocks_hi : p.inv_blocks_lo;   // from the host: no division here
        const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(p.xb);
        const __nv_bfloat16* rin = static_cast<const __nv_bfloat16*>(p.residual_in);
        const __nv_bfloat16* dl = static_cast<const __nv_bfloat16*>(p.delta);
        constexpr int kind = kKind;

        if (kind == 1) {
            // Every CTA needs each row's mean square over the whole K: recomputed here from
            // L2 (2 x 2K bytes per row) instead of being passed between kernels. Four 16-byte
            // chunks per thread are loaded before any arithmetic: one round trip for K <= 6144.
#pragma unroll 1
            for (int m = 0; m < p.M; ++m) {
                const int64_t base = static_cast<int64_t>(p.m0 + m) * p.K;
                float ss = 0.0f;
#pragma unroll 1
                for (int c0 = tid; c0 < p.K / 8; c0 += 4 * kThreadsP) {
                    uint4 r4[4], d4[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int c8 = c0 + u * kThreadsP;
                        if (c8 < p.K / 8) {
                            r4[u] = __ldg(reinterpret_cast<const uint4*>(rin + base) + c8);
                            if (dl != nullptr) d4[u] = __ldg(reinterpret_cast<const uint4*>(dl + base) + c8);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (c0 + u * kThreadsP < p.K / 8) {
                            float r[8];
                            unpack8(dl != nullptr ? add_bf16x8(r4[u], d4[u]) : r4[u], r);
#pragma unroll
                            for (int j = 0; j < 8; ++j) ss += r[j] * r[j];
                        }
                    }
                }
#pragma unroll
                for (int sft = 16; sft > 0; sft >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sft);
                if (lane == 0) s_red[m * 8 + warp] = ss;
            }
            __syncthreads();
        }

        auto src0 = [&](int i) {
            const int m = static_cast<int>((static_cast<uint32_t>(i) * inv_blocks) >> 20), blk = i - m * blocks;
            return reinterpret_cast<const uint4*>(xb + (p.m0 + m) * p.xb_stride + static_cast<int64_t>(blk0 + blk) * 16);
        };
        auto inside = [&](int i) {
            const int m = static_cast<int>((static_cast<uint32_t>(i) * inv_blocks) >> 20);
            return i - m * blocks < real;
        };
        // quantize block i (16 bf16 values in lo, hi) into the operand layout
        auto emit = [&](int i, const uint4& lo, const uint4& hi) {
            const int m = static_cast<int>((static_cast<uint32_t>(i) * inv_blocks) >> 20), blk = i - m * blocks;
            uint32_t cw[2];
            const uint32_t sf = quantize_block16_rt(lo, hi, q, exact, cw);
            *reinterpret_cast<uint2*>(b_tile_g + (blk >> 4) * (BN * 128) + swz128(m, (blk & 15) * 8)) =
                make_uint2(cw[0], cw[1]);
            b_sf_g[(blk >> 2) * kSfbStride + m * 16 + (blk & 3)] = static_cast<uint8_t>(sf);
        };
        if (kind == 0) {
            // Two 16-element blocks per thread per round (two independent quantizer chains), the
            // next round's two blocks fetched while the current ones are quantized.
            auto fetch = [&](int i, uint4& lo, uint4& hi) {
                lo = make_uint4(0, 0, 0, 0);
                hi = lo;
                if (i < n_items && inside(i)) {
                    const uint4* s0 = src0(i);
                    lo = __ldg(s0);
                    hi = __ldg(s0 + 1);
                }
            };
#pragma unroll 1
            for (int i = tid; i < n_items; i += 2 * kThreadsP) {
                uint4 na_lo, na_hi, nb_lo, nb_hi;
                fetch(i + 2 * kThreadsP, na_lo, na_hi);
                fetch(i + 3 * kThreadsP, nb_lo, nb_hi);
                emit(i, a_lo, a_hi);
                if (i + kThreadsP < n_items) emit(i + kThreadsP, b_lo, b_hi);
                a_lo = na_lo; a_hi = na_hi; b_lo = nb_lo; b_hi = nb_hi;
            }
        }
        // prologues 1 and 2: one block per thread per round
#pragma unroll 1
        for (int i = tid; kind != 0 && i < n_items; i += kThreadsP) {
            const int m = static_cast<int>((static_cast<uint32_t>(i) * inv_blocks) >> 20), blk = i - m * blocks;
            uint4 lo, hi;
            if (kind == 2) {
                // activation = bf16(silu(gate) * up), gate_up row = [gate (K) | up (K)]
                const __nv_bfloat16* row = xb + (p.m0 + m) * p.xb_stride + static_cast<int64_t>(blk0 + blk) * 16;
                uint4 g0 = own_r0, g1 = own_r1, u0 = own_d0, u1 = own_d1;     // the first block: fetched right after the wait
                if (i != tid) {
                    g0 = make_uint4(0, 0, 0, 0);
                    g1 = g0; u0 = g0; u1 = g0;
                }
                if (i != tid && blk < real) {
                    g0 = __ldg(reinterpret_cast<const uint4*>(row));
                    g1 = __ldg(reinterpret_cast<const uint4*>(row) + 1);
                    u0 = __ldg(reinterpret_cast<const uint4*>(row + p.K));
                    u1 = __ldg(reinterpret_cast<const uint4*>(row + p.K) + 1);
                }
                float g[16], u[16];
                unpack8(g0, g); unpack8(g1, g + 8); unpack8(u0, u); unpack8(u1, u + 8);
#pragma unroll
                for (int j = 0; j < 16; ++j) g[j] = g[j] / (1.0f + __expf(-g[j])) * u[j];
                lo = pack8(g);
                hi = pack8(g + 8);
            } else {
                // activation = bf16( bf16(residual + delta) * rsqrt(mean_sq + eps) * norm_w );
                // the CTAs of rank 0 (one per K part) also write the new residual
                const __nv_bfloat16* nw = static_cast<const __nv_bfloat16*>(p.norm_w);
                __nv_bfloat16* rout = static_cast<__nv_bfloat16*>(p.residual_out);
                const int64_t koff = static_cast<int64_t>(blk0 + blk) * 16;
                const int64_t off = static_cast<int64_t>(p.m0 + m) * p.K + koff;
                uint4 r0 = own_r0, r1 = own_r1, w0 = nw_first0, w1 = nw_first1;
                if (i != tid) {
                    r0 = __ldg(reinterpret_cast<const uint4*>(rin + off));
                    r1 = __ldg(reinterpret_cast<const uint4*>(rin + off) + 1);
                    w0 = __ldg(reinterpret_cast<const uint4*>(nw + koff));
                    w1 = __ldg(reinterpret_cast<const uint4*>(nw + koff) + 1);
                }
                if (dl != nullptr) {
                    uint4 d0 = own_d0, d1 = own_d1;
                    if (i != tid) {
                        d0 = __ldg(reinterpret_cast<const uint4*>(dl + off));
                        d1 = __ldg(reinterpret_cast<const uint4*>(dl + off) + 1);
                    }
                    r0 = add_bf16x8(r0, d0);
                    r1 = add_bf16x8(r1, d1);
                }
                if (rank == 0) {
                    *reinterpret_cast<uint4*>(rout + off) = r0;
                    *(reinterpret_cast<uint4*>(rout + off) + 1) = r1;
                }
                float r[16], t[16];
                unpack8(r0, r); unpack8(r1, r + 8);
                float tot = 0.0f;
#pragma unroll
                for (int w = 0; w < kWarpsP; ++w) tot += s_red[m * 8 + w];
                const float inv = rsqrtf(tot / static_cast<float>(p.K) + p.eps);
                unpack8(w0, t); unpack8(w1, t + 8);
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = r[j] * inv * t[j];
                lo = pack8(r);
                hi = pack8(r + 8);
            }
            emit(i, lo, hi);
        }
        // Rows M..BN-1 of the operand are never written: whatever they hold only reaches
        // accumulator columns that are not stored.
        fence_proxy_async_smem();
    }
    __syncthreads();
    if (warp == 0) TRACE(3);

    WaitFail wf;
    if (warp == 0) {
        // ---------------- producer (whole warp waits, the elected lane issues) --------------
#pragma unroll 1
        while (issued < total) {
            const int s = issued & (kStages - 1);
            if (!wf.wait(bar_empty + 8 * s, ((issued / kStages) - 1) & 1)) break;
            issue_next();
            __syncwarp();
        }
    } else if (warp == 1 && my_tiles > 0) {
        // ---------------- MMA issuer -----------------------------------------------------
        // The whole warp walks the loops (waits included) and one elected lane issues: descriptors
        // and addresses are then warp-uniform values, which is what the tensor-core instructions
        // take their operands from (a single active lane of a diverged warp paid about 70 cycles
        // per instruction to get them there).
        const bool leader = elect_one();
        constexpr uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                   (static_cast<uint32_t>(kTileRows >> 7) << 27);
        int i = 0;
#pragma unroll 1
        for (int ti = 0; ti < my_tiles && !wf.failed; ++ti) {
            const int buf = ti & 1;
            if (ti >= 2 && !wf.wait(bar_accempty + 8 * buf, ((ti >> 1) - 1) & 1)) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem + buf * BN;
#pragma unroll 1
            for (int j = 0; j < stages_per_tile; ++j, ++i) {
                const int s = i & (kStages - 1);
                if (!wf.wait(bar_full + 8 * s, (i / kStages) & 1)) break;
                if (i == 0) TRACE(4);
                // the activation scales of this stage's blocks are in tensor memory (first tile only)
                if (ti == 0 && !wf.wait(bar_sfb + 8 * j, 0)) break;
                if (i == 0) TRACE(10);
                tc_fence_after();
                const int nb = min(kBlocksPerStage, nkb - j * kBlocksPerStage);
#pragma unroll 1
                for (int b = 0; b < nb; ++b) {
                    const uint32_t a_smem = ring + s * kStageBytes + b * kBlockBytes;
                    const int blk = j * kBlocksPerStage + b;              // block within the part
                    const uint64_t a_desc = desc_operand(a_smem);
                    const uint64_t b_desc = desc_operand(b_tile + blk * (BN * 128));
                    const uint64_t sfa_desc = desc_scales(a_smem + kCodesBytes);
                    const uint32_t sfa_col = tmem + kColSFA + 16 * b;
                    const uint32_t sfb_col = tmem + kColSFB + 16 * blk;
                    if (leader) {
                        // descriptors advance by (bytes >> 4): 512 B per scale chunk, 32 B per K64 of
                        // codes; the four weight-scale copies go first so that no MMA waits behind
                        // its own copy
#pragma unroll
                        for (int k = 0; k < 4; ++k) tc_cp_scales(sfa_col + 4 * k, sfa_desc + 32 * k);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            tc_mma_nvf4(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, sfa_col + 4 * k,
                                        sfb_col + 4 * k, (blk | k) != 0 ? 1u : 0u);
                    }
                }
                if (i == 0) TRACE(11);
                if (leader) tc_commit(bar_empty + 8 * s);
                if (i == 0) TRACE(12);
                __syncwarp();
            }
            if (leader) tc_commit(bar_accfull + 8 * buf);
            if (ti == 0) TRACE(5);
        }
        TRACE(6);
    } else if (warp >= 2) {
        // ---------------- epilogue (warps 2..5) ------------------------------------------
        const int q = warp & 3;                                   // TMEM lane quadrant of this warp
        const int row_in_tile = q * 32 + lane;
        if (warp == 2 && my_tiles > 0) {
            // activation scales of the whole K part go into tensor memory once, issued from
            // this warp's elected lane so that they overlap the MMA warp's weight-scale copies;
            // one commit per stage of the K part
            const bool lead2 = elect_one();
            const uint64_t d0 = desc_scales(b_sf);
#pragma unroll 1
            for (int j = 0; j < stages_per_tile; ++j) {
                const int c0 = j * kBlocksPerStage * 4, c1 = min(nkb * 4, c0 + kBlocksPerStage * 4);
                if (lead2) {
#pragma unroll 1
                    for (int ch = c0; ch < c1; ++ch)
                        tc_cp_scales(tmem + kColSFB + 4 * ch, d0 + ch * (kSfbStride >> 4));
                    tc_commit(bar_sfb + 8 * j);
                }
            }
        }
        __syncwarp();
        // Which half of the peers' receive memory this call uses: the call counter in this rank's
        // own header, final before this kernel started (its writer is an earlier kernel).
        const unsigned push_parity =
            (kPush != 0 && p.push_world > 1) ? (*reinterpret_cast<volatile unsigned*>(p.push_base[p.push_rank]) & 1u) : 0u;
#pragma unroll 1
        for (int ti = 0; ti < my_tiles; ++ti) {
            const int buf = ti & 1;
            const int tile = rank + ti * cpp;
            if (!wf.wait(bar_accfull + 8 * buf, (ti >> 1) & 1)) break;
            if (warp == 2 && ti == 0) TRACE(7);
            if (warp == 2 && ti == my_tiles - 1) TRACE(8);
            tc_fence_after();
            const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
            const int64_t n = static_cast<int64_t>(tile) * kTileRows + row_in_tile;
            // Token m is finished by the CTA of part m % S: the hand-over work of a tile is spread
            // over its S CTAs instead of falling on one of them.
            unsigned long long* tile_slots =
                p.slots + static_cast<int64_t>(tile) * p.M * S * kTileRows + row_in_tile;
            // pass 1: publish this part's values for the tokens that other parts finish (nothing
            // waits here, so no part holds up another); with a single token part 0 has none
            if (S > 1 && (p.M > 1 || part != 0)) {
                int owner = 0;                                     // part that finishes token mf + j
#pragma unroll 1
                for (int mf = 0; mf < p.M; mf += 4) {
                    const int cnt = min(4, p.M - mf);
                    float v[4];
                    tmem_ld4(taddr + mf, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (j < cnt && owner != part)
                            slot_store(tile_slots + (static_cast<int64_t>(mf + j) * S + part) * kTileRows, v[j]);
                        owner = (owner + 1 == S) ? 0 : owner + 1;
                    }
                }
            }
            // pass 2: finish this part's own tokens part, part + S, ...
#pragma unroll 1
            for (int m = part; m < p.M; m += S) {
                float val;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=f"(val) : "r"(taddr + m) : "memory");
                tmem_ld_wait();
                if (S > 1 && !token_gather(tile_slots + static_cast<int64_t>(m) * S * kTileRows, S, part, val, &val))
                    wf.failed = true;
                const float o = val * p.alpha;
                if (kPush != 0 && p.push_world > 1) {
                    // adjacent weight rows sit in adjacent lanes: the even lane sends the pair
                    const float o2 = __shfl_down_sync(0xffffffffu, o, 1);
                    if ((lane & 1) == 0) {
                        const unsigned long long w = (1ull << 32) | pack2_bf16(o, o2);
                        const unsigned long long i =
                            (static_cast<unsigned long long>(p.m0 + m) * p.N + static_cast<unsigned long long>(n)) >> 1;
#pragma unroll 1
                        for (int d = 0; d < p.push_world; ++d) {
                            const int dst = (p.push_rank + d) % p.push_world;
                            unsigned long long* slot =
                                reinterpret_cast<unsigned long long*>(p.push_base[dst] + 256) +
                                (static_cast<unsigned long long>(push_parity) * p.push_world + p.push_rank) * p.push_max_pairs + i;
                            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(slot), "l"(w) : "memory");
                        }
                        if (kPush == 2 && p.push_gather) {
                            unsigned long long* mine =
                                reinterpret_cast<unsigned long long*>(p.push_base[p.push_rank] + 256) +
                                static_cast<unsigned long long>(push_parity) * p.push_world * p.push_max_pairs + i;
                            unsigned long long v[NVFP4R_PEER_MAX_WORLD];
#pragma unroll
                            for (int r = 0; r < NVFP4R_PEER_MAX_WORLD; ++r)
                                if (r < p.push_world) v[r] = peer_poll(mine + r * p.push_max_pairs);
                            for (uint32_t it = 0;; ++it) {
                                bool all = true;
#pragma unroll
                                for (int r = 0; r < NVFP4R_PEER_MAX_WORLD; ++r)
                                    if (r < p.push_world && (v[r] >> 32) != 1ull) {
                                        v[r] = peer_poll(mine + r * p.push_max_pairs);
                                        all = false;
                                    }
                                if (all) break;
                                if (it > p.push_poll_limit) { wf.failed = true; break; }
                            }
                            float lo = 0.0f, hi = 0.0f;
#pragma unroll
                            for (int r = 0; r < NVFP4R_PEER_MAX_WORLD; ++r)
                                if (r < p.push_world) {
                                    const uint32_t bits = static_cast<uint32_t>(v[r]);
                                    lo += __uint_as_float(bits << 16);
                                    hi += __uint_as_float(bits & 0xFFFF0000u);
                                    mine[r * p.push_max_pairs] = 0ull;
                                }
                            static_cast<uint32_t*>(p.out)[i] = pack2_bf16(lo, hi);
                        }
                    }
                } else {
                    const int64_t idx = (p.m0 + m) * p.ldc + n;
                    if (p.out_dtype == 0) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(o);
                    else if (p.out_dtype == 1) static_cast<__half*>(p.out)[idx] = __float2half_rn(o);
                    else static_cast<float*>(p.out)[idx] = o;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_accempty + 8 * buf);
        }
        if (warp == 2) TRACE(9);
    }

    if (wf.failed && lane == 0) report_timeout(&g_packed_status, 3);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
    if (kPush == 2 && p.push_world > 1 && p.push_gather && tid == 0) {
        // the last CTA of the grid to finish advances the call counter: nobody of this launch
        // reads it any more (same rule as the stand-alone gather kernel)
        unsigned* header = reinterpret_cast<unsigned*>(p.push_base[p.push_rank]);
        __threadfence();
        const unsigned t = atomicAdd(header + 1, 1u);
        if (t == gridDim.x - 1) {
            header[1] = 0u;
            header[0] = header[0] + 1u;
        }
    }
}

struct PackedPlan { int splits, grid, bn; size_t smem; };
int g_force_packed_splits = 0;
int g_packed_ctas_per_sm = 2;
int g_packed_l2_stages = 2;          // measured best on B200 (0: 3248, 2: 3254 -> with the warp-uniform issuer 3459 GB/s; 3+: worse)

// Parts of at most kMaxPartBlocks K blocks; among the admissible split counts take the
// one with the smallest estimated time.
bool plan_packed(int M, int N, int K, PackedPlan* plan) {
    const int bn = M <= 16 ? 16 : 32;
    const int per_sm = (bn == 16 && g_packed_ctas_per_sm == 2) ? 2 : 1;
    const int G = device_sm_count() * per_sm;
    const int tiles = N / kTileRows, kblocks = (K + kBlockK - 1) / kBlockK;
    const int min_s = (kblocks + kMaxPartBlocks - 1) / kMaxPartBlocks;
    if (min_s > G) return false;
    // Estimated time of a split count, fitted to sweeps on B200: the CTAs make
    // ceil(units / G) rounds; a round streams one unit (largest K part) at the per-CTA share
    // of HBM bandwidth and pays about a microsecond per tile for the pipeline restart and the
    // partial-sum hand-over.
    int best = -1;
    double best_score = 1e30;
    const double kb_per_us = 6400.0 * 1000.0 / 1024.0 / G;      // KB per microsecond per CTA
    for (int s = min_s; s <= kblocks && s <= G && s <= 64; ++s) {
        const int rounds = (tiles + G / s - 1) / (G / s);
        const int unit_blocks = (kblocks + s - 1) / s;
        const double score = rounds * (unit_blocks * 18.0 / kb_per_us + (s > 1 ? 1.2 : 0.3)) + 0.01 * s;
        if (score < best_score) { best_score = score; best = s; }
    }
    if (g_force_packed_splits >= min_s && g_force_packed_splits <= kblocks && g_force_packed_splits <= G)
        best = g_force_packed_splits;
    if (best < 0) return false;
    plan->splits = best;
    plan->bn = bn;
    plan->grid = G;
    const int sfb_stride = bn == 16 ? 256 : 512;
    plan->smem = static_cast<size_t>(kStages) * kStageBytes + kMaxPartBlocks * (bn * 128) +
                 (kMaxPartBlocks * 4 * sfb_stride + 256) + 1024;
    return true;
}

}  // namespace

size_t packed_weight_bytes(int N, int K) {
    return static_cast<size_t>(N / kTileRows) * ((K + kBlockK - 1) / kBlockK) * kBlockBytes;
}

size_t packed_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || N % kTileRows || K % (kBlockK / 2)) return 16;
    PackedPlan plan;
    if (!plan_packed(M < 32 ? M : 32, N, K, &plan)) return 16;
    const size_t tiles = N / kTileRows;
    const size_t m = M < 32 ? M : 32;
    const size_t slots = plan.splits > 1 ? tiles * plan.splits * m * kTileRows * sizeof(unsigned long long) : 0;
    return slots + 256;
}

cudaError_t launch_pack_weight(const void* w, const void* sf_flat, void* packed, int N, int K,
                               cudaStream_t stream) {
    const dim3 grid(static_cast<unsigned>((K + kBlockK - 1) / kBlockK), static_cast<unsigned>(N / kTileRows));
    pack_weight_kernel<<<grid, 1024, 0, stream>>>(static_cast<const uint8_t*>(w),
                                                  static_cast<const uint8_t*>(sf_flat),
                                                  static_cast<uint8_t*>(packed), N, K);
    return cudaGetLastError();
}

cudaError_t launch_linear_packed(const PackedLinearArgs& g, cudaStream_t stream, const char** why) {
    *why = nullptr;
    if (g.N % kTileRows != 0) { *why = "packed linear: N must be a multiple of 128"; return cudaSuccess; }
    if (g.K % (kBlockK / 2) != 0) { *why = "packed linear: K must be a multiple of 128"; return cudaSuccess; }
    if (g.pro_kind == 1 && g.K % kBlockK != 0) { *why = "packed linear: the RMSNorm prologue needs K % 256 == 0"; return cudaSuccess; }
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
        p.kblocks = (g.K + kBlockK - 1) / kBlockK;
        p.ctas_per_part = plan.grid / plan.splits;
        p.kb_q = p.kblocks / plan.splits;
        p.kb_r = p.kblocks % plan.splits;
        p.inv_splits = static_cast<uint32_t>((0x100000000ull + static_cast<unsigned>(plan.splits) - 1) / static_cast<unsigned>(plan.splits));
        {
            const uint32_t b_hi = static_cast<uint32_t>(p.kb_q + 1) * (kBlockK / 16), b_lo = static_cast<uint32_t>(p.kb_q) * (kBlockK / 16);
            p.inv_blocks_hi = ((1u << 20) + b_hi - 1u) / b_hi;
            p.inv_blocks_lo = b_lo ? ((1u << 20) + b_lo - 1u) / b_lo : 0u;
        }
        p.tiles_q = p.tiles / p.ctas_per_part;
        p.tiles_r = p.tiles % p.ctas_per_part;
        p.pro_kind = g.pro_kind;
        p.delta = g.delta;
        p.residual_in = g.residual_in;
        p.residual_out = g.residual_out;
        p.norm_w = g.norm_w;
        p.eps = g.eps;
        p.slots = static_cast<unsigned long long*>(g.workspace);
        p.push_world = 0;
        if (g.push != nullptr && g.push->world > 1) {
            p.push_world = g.push->world;
            p.push_rank = g.push->rank;
            p.push_max_pairs = (g.push->max_elems + 1) / 2;
            for (int r = 0; r < g.push->world; ++r) p.push_base[r] = static_cast<unsigned char*>(g.push->base[r]);
            p.push_gather = g.push_gather ? 1 : 0;
            p.push_poll_limit = peer_poll_limit();
        }
        p.l2_stages = g_packed_l2_stages;

        using Kern = void (*)(PackedParams);
#define NVFP4R_PACKED_ROW(BN, PUSH) \
    {linear_packed_kernel<BN, 0, PUSH>, linear_packed_kernel<BN, 1, PUSH>, linear_packed_kernel<BN, 2, PUSH>}
        static const Kern table[3][2][3] = {{NVFP4R_PACKED_ROW(16, 0), NVFP4R_PACKED_ROW(32, 0)},
                                            {NVFP4R_PACKED_ROW(16, 1), NVFP4R_PACKED_ROW(32, 1)},
                                            {NVFP4R_PACKED_ROW(16, 2), NVFP4R_PACKED_ROW(32, 2)}};
#undef NVFP4R_PACKED_ROW
        if (g.pro_kind < 0 || g.pro_kind > 2) { *why = "packed linear: unknown prologue kind"; return cudaSuccess; }
        const int pi = p.push_world > 1 ? (p.push_gather ? 2 : 1) : 0;
        const Kern kern = table[pi][plan.bn == 16 ? 0 : 1][g.pro_kind];
        static bool attr_done[3][2][3][64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const int ki = plan.bn == 16 ? 0 : 1;
        if (dev >= 0 && dev < 64 && !attr_done[pi][ki][g.pro_kind][dev]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            if (e != cudaSuccess) return e;
            attr_done[pi][ki][g.pro_kind][dev] = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
        cfg.blockDim = dim3(kThreadsP);
        cfg.dynamicSmemBytes = plan.smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        int na = 0;
        if (gemv_tuning().use_pdl) {
            attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[na].val.programmaticStreamSerializationAllowed = 1;
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
    if ((splits >> 24) & 0xf) g_packed_l2_stages = ((splits >> 24) & 0xf) - 1;   // bits 24..27: L2 run-ahead depth + 1 (0..2 stages)
#ifdef NVFP4R_TRACE
    // bit 8: record the time line of eight CTAs; bits 12..23: the first of them
    const int trace = ((splits >> 8) & 1) ? 1 + ((splits >> 12) & 0xfff) : 0;
    cudaMemcpyToSymbol(g_packed_trace, &trace, sizeof(int));
#endif
}

#ifdef NVFP4R_TRACE
cudaError_t read_packed_trace(unsigned long long* out512) {
    return cudaMemcpyFromSymbol(out512, g_packed_times, 8 * 64 * sizeof(unsigned long long));
}
#endif

cudaError_t set_status_mirror_packed(int* p) { return set_status_mirror_here(p); }

cudaError_t read_and_clear_packed_status(int* flag) {
    cudaError_t e = cudaMemcpyFromSymbol(flag, g_packed_status, sizeof(int));
    if (e != cudaSuccess) return e;
    const int zero = 0;
    return cudaMemcpyToSymbol(g_packed_status, &zero, sizeof(int));
}

}  // namespace nvfp4r
