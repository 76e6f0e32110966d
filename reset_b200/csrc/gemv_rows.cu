// NVFP4 W4A4 GEMV for one token: activations stay in registers, weights
// stream straight from global memory into registers.
//
// Decomposition. A lane owns one 32-element unit of K (16 code bytes, 2 block
// scales) for the whole launch: it quantizes (or loads) that slice of the
// activations once, decodes it to f16 and keeps it in 16 registers per token.
// A warp therefore covers 1024 consecutive K elements, `cw` warps side by side
// cover a weight row, and such a group of warps (a row stream) walks down its
// own contiguous range of rows, R rows per step, with the next step's loads in
// flight while the current one is multiplied. Every weight byte is requested
// exactly once by a 16-byte load that is part of a 512-byte warp request; no
// shared-memory staging, no barrier on the load path. The first steps are
// requested before the wait for the preceding kernel (weights are constants).
//
// Per row and lane: 16 conversions e2m1x2 -> f16x2, two exact 8-deep f16 FMA
// chains (products are multiples of 1/4, |sum| <= 576), one f32 multiply-add
// with the product of the two block scales. The R (x tokens) values of a step
// are summed over the warp with a halving butterfly (9 shuffles for 8 values
// instead of 40), over the warps of the stream through shared memory in fixed
// order: results are bit-identical run to run.
#include "kernels.h"
#include "quant_core.cuh"

namespace nvfp4r {
namespace {

constexpr int kUnitBytes = 16;     // 32 elements
constexpr int kMaxWarps = 32;

struct RowsParams {
    GemvArgs a;
    int units;            // K / 32
    int cw;               // warps side by side along K
    int streams;          // row streams per CTA
    int total_streams;    // streams * gridDim.x
    int pairs;            // ceil(N / (2 R)): units of work dealt to the streams
    int stream_rows;      // most rows a stream can get (a multiple of 2 R)
    int stream_floats;    // stream_rows * MT * cw: floats of shared memory per stream
};

struct Unit16 {
    uint32_t h[16];
};

__device__ __forceinline__ void decode_codes(const uint4& c, Unit16& u) {
    e2m1x8_to_f16x8(c.x, &u.h[0]);
    e2m1x8_to_f16x8(c.y, &u.h[4]);
    e2m1x8_to_f16x8(c.z, &u.h[8]);
    e2m1x8_to_f16x8(c.w, &u.h[12]);
}

// acc += a * b with a, b f16 and the product and sum in f32 (the product of two f16 values is
// exact in f32).
__device__ __forceinline__ float fma_f16_f32(__half a, __half b, float acc) {
    asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(__half_as_ushort(a)), "h"(__half_as_ushort(b)));
    return acc;
}

// 2^-6 in both halves: the activation scales are kept multiplied by it so that the product of
// a weight scale and an activation scale (up to 448 * 448) stays inside f16. Every product of
// two e4m3 values is a multiple of 2^-18 with at most 8 significant bits, so
// weight scale * (activation scale * 2^-6) is EXACT in f16, subnormals included.
constexpr uint32_t kTwoPowMinus6x2 = 0x24002400u;
constexpr float kScaleFix = 64.0f;

__device__ __forceinline__ void store_out(void* out, int dtype, int64_t idx, float v) {
    if (dtype == 0)      static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
    else if (dtype == 1) static_cast<__half*>(out)[idx] = __float2half_rn(v);
    else                 static_cast<float*>(out)[idx] = v;
}

// Sum NV values per lane over the 32 lanes. Each step halves the number of
// values a lane still carries; afterwards v[0] of lane l is the total of value
// l >> (5 - log2(NV)).
template <int NV>
__device__ __forceinline__ void butterfly(float (&v)[NV], int lane) {
    int n = NV;
#pragma unroll
    for (int step = 16; step >= 1; step >>= 1) {
        if (n > 1) {
            const int half = n / 2;
            const bool upper = (lane & step) != 0;
#pragma unroll
            for (int i = 0; i < NV / 2; ++i) {
                if (i < half) {
                    const float keep = upper ? v[i + half] : v[i];
                    const float send = upper ? v[i] : v[i + half];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, step);
                }
            }
            n = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], step);
        }
    }
}

// ---- bf16 vector helpers of the fused prologues (same roundings as the packed linear's) ------
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

template <int R>
struct Stage {
    uint4 c[R];
    uint32_t s[R];
};

// Loads of one step: R rows below `wq` / `sq` (this lane's unit in the step's first row), no
// bounds tests: the caller guarantees that all R rows exist.
template <int R>
__device__ __forceinline__ void load_stage(Stage<R>& st, const uint8_t* wbase, const uint8_t* sbase,
                                           uint32_t w0, uint32_t s0, uint32_t w_stride, uint32_t sf_stride) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
        st.c[r] = ldg_stream_16(wbase + (w0 + r * w_stride));
        st.s[r] = ldg_stream_2(sbase + (s0 + r * sf_stride));
    }
}

// Last step of the matrix when N is not a multiple of R: rows past the end read row N - 1
// again (their results are never stored).
template <int R>
__device__ __forceinline__ void load_stage_clamped(Stage<R>& st, const uint8_t* wbase, const uint8_t* sbase,
                                                   uint32_t w0, uint32_t s0, uint32_t w_stride,
                                                   uint32_t sf_stride, int rows_left) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int rr = r < rows_left ? r : rows_left - 1;
        st.c[r] = ldg_stream_16(wbase + (w0 + rr * w_stride));
        st.s[r] = ldg_stream_2(sbase + (s0 + rr * sf_stride));
    }
}

// Work is dealt in steps of R consecutive rows and in pairs of steps (one butterfly sums the
// 2 R MT values of a pair). A row stream owns the pairs [pair_begin, pair_end); its per-warp
// sums go to shared memory and are added over the stream's warps once, at the end.
// kPlain: the instance without the fused prologues' code (activations arrive quantized, or as
// bf16 to quantize), for launches whose prologue kind is 0.
template <int MT, int R, int MAXT, int MINB, bool kPlain>
__global__ void __launch_bounds__(MAXT, MINB)
gemv_rows_kernel(const __grid_constant__ RowsParams p) {
    constexpr int NV = 2 * R * MT;
    constexpr int kShift = NV == 2 ? 4 : NV == 4 ? 3 : NV == 8 ? 2 : NV == 16 ? 1 : 0;
    extern __shared__ float part[];      // [stream][local row * MT + m][kc]
    __shared__ float s_ss[kMaxWarps];    // RMSNorm prologue: per-warp sum of squares

    const int tid = threadIdx.x, lane = tid & 31, wi = tid >> 5;
    const int cw = p.cw;
    const int s = wi / cw, kc = wi - s * cw;
    const int u_raw = kc * 32 + lane;
    const bool active = u_raw < p.units;
    const int u = active ? u_raw : p.units - 1;          // idle lanes re-read the last unit against zeros
    const int N = p.a.N, M = p.a.M;
    const int sid = blockIdx.x * p.streams + s;
    const int pair_begin = static_cast<int>(static_cast<int64_t>(sid) * p.pairs / p.total_streams);
    const int pair_end = static_cast<int>(static_cast<int64_t>(sid + 1) * p.pairs / p.total_streams);
    const int row_begin = pair_begin * 2 * R;
    const int row_end = min(pair_end * 2 * R, N);
    const int steps = (row_end - row_begin + R - 1) / R;     // the last one may be partial (end of the matrix)

    // Byte offsets from the weight's base fit 32 bits (checked by the launcher): one integer add
    // per address.
    const uint32_t w_stride = static_cast<uint32_t>(p.a.w_stride_n), sf_stride = static_cast<uint32_t>(p.a.wsf_stride_n);
    const uint32_t wq = static_cast<uint32_t>(row_begin) * w_stride + u * kUnitBytes;
    const uint32_t sq = static_cast<uint32_t>(row_begin) * sf_stride + u * 2;
    const uint8_t* __restrict__ wbase = p.a.w;
    const uint8_t* __restrict__ sbase = p.a.wsf;

    auto load = [&](Stage<R>& st, int step) {
        if (step >= steps) return;
        const int left = row_end - (row_begin + step * R);
        const uint32_t w0 = wq + static_cast<uint32_t>(step) * (R * w_stride);
        const uint32_t s0 = sq + static_cast<uint32_t>(step) * (R * sf_stride);
        if (left >= R) load_stage<R>(st, wbase, sbase, w0, s0, w_stride, sf_stride);
        else load_stage_clamped<R>(st, wbase, sbase, w0, s0, w_stride, sf_stride, left);
    };

    // Weights do not depend on the preceding kernel.
    Stage<R> sa, sb;
    load(sa, 0);
    load(sb, 1);
    const float gs = (p.a.xb != nullptr || (!kPlain && p.a.pro_kind != 0)) ? __ldg(p.a.gs) : 1.0f;
    pdl_launch_dependents();
    pdl_wait_prior();

    // This lane's slice of the activations, decoded once.
    uint32_t xh[MT][16];
    __half2 xs[MT];                 // the two block scales of the slice, times 2^-6
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        uint4 codes = make_uint4(0u, 0u, 0u, 0u);
        uint32_t sf2 = 0u;
        if (!kPlain && p.a.pro_kind == 1) {
            // activation = bf16( bf16(residual + delta) * rsqrt(mean_sq + eps) * norm_w ); every
            // stream computes the whole row (its cw warps cover it once); the first stream of the
            // first CTA writes the new residual. All warps of the CTA pass the barrier.
            const __nv_bfloat16* rin = static_cast<const __nv_bfloat16*>(p.a.residual_in) + static_cast<int64_t>(m) * p.a.K;
            const __nv_bfloat16* dl = p.a.delta ? static_cast<const __nv_bfloat16*>(p.a.delta) + static_cast<int64_t>(m) * p.a.K : nullptr;
            // The 32 values of the slice stay packed as bf16 pairs (they are bf16 after the add)
            // across the barrier: 16 registers instead of 32.
            uint4 rr[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
            float ss = 0.0f;
            if (active && m < M) {
                const uint4* rp = reinterpret_cast<const uint4*>(rin + u * 32);
                const uint4* dp = reinterpret_cast<const uint4*>(dl + u * 32);
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) rr[qd] = __ldg(rp + qd);
                if (dl != nullptr) {
                    uint4 dd[4];
#pragma unroll
                    for (int qd = 0; qd < 4; ++qd) dd[qd] = __ldg(dp + qd);
#pragma unroll
                    for (int qd = 0; qd < 4; ++qd) {
                        float r[8], d[8];
                        unpack8(rr[qd], r);
                        unpack8(dd[qd], d);
#pragma unroll
                        for (int j = 0; j < 8; ++j) r[j] = r[j] + d[j];
                        rr[qd] = pack8(r);                      // the bf16 rounding of the separate add
                    }
                }
                if (blockIdx.x == 0 && s == 0) {
                    uint4* op = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.a.residual_out) +
                                                         static_cast<int64_t>(m) * p.a.K + u * 32);
#pragma unroll
                    for (int qd = 0; qd < 4; ++qd) op[qd] = rr[qd];
                }
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) {
                    float r[8];
                    unpack8(rr[qd], r);
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss += r[j] * r[j];
                }
            }
#pragma unroll
            for (int sft = 16; sft > 0; sft >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sft);
            __syncthreads();                         // s_ss free (a previous token's readers are done)
            if (lane == 0) s_ss[wi] = ss;
            __syncthreads();
            float tot = 0.0f;
            for (int j = 0; j < cw; ++j) tot += s_ss[s * cw + j];
            const float inv = rsqrtf(tot / static_cast<float>(p.a.K) + p.a.eps);
            if (active && m < M) {
                const uint4* wp4 = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.a.norm_w) + u * 32);
                uint4 vq[4];
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) {
                    float r[8], t[8];
                    unpack8(rr[qd], r);
                    unpack8(__ldg(wp4 + qd), t);
#pragma unroll
                    for (int j = 0; j < 8; ++j) r[j] = r[j] * inv * t[j];
                    vq[qd] = pack8(r);
                }
                uint32_t c0[2], c1[2];
                const bool exact = p.a.rcp_mode == kRcpExact;
                const QuantScales q = exact ? make_quant_scales<kRcpExact>(gs) : make_quant_scales<kRcpApprox>(gs);
                const uint32_t sf0 = quantize_block16_rt(vq[0], vq[1], q, exact, c0);
                const uint32_t sf1 = quantize_block16_rt(vq[2], vq[3], q, exact, c1);
                codes = make_uint4(c0[0], c0[1], c1[0], c1[1]);
                sf2 = sf0 | (sf1 << 8);
            }
        } else if (!kPlain && p.a.pro_kind == 2) {
            // activation = bf16(silu(gate) * up), row = [gate (K) | up (K)]
            if (active && m < M) {
                const __nv_bfloat16* row = static_cast<const __nv_bfloat16*>(p.a.xb) + m * p.a.xb_stride + u * 32;
                const uint4* gp = reinterpret_cast<const uint4*>(row);
                const uint4* up = reinterpret_cast<const uint4*>(row + p.a.K);
                uint4 vq[4];
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) {
                    float g[8], uu[8];
                    unpack8(__ldg(gp + qd), g);
                    unpack8(__ldg(up + qd), uu);
#pragma unroll
                    for (int j = 0; j < 8; ++j) g[j] = g[j] / (1.0f + __expf(-g[j])) * uu[j];
                    vq[qd] = pack8(g);
                }
                uint32_t c0[2], c1[2];
                const bool exact = p.a.rcp_mode == kRcpExact;
                const QuantScales q = exact ? make_quant_scales<kRcpExact>(gs) : make_quant_scales<kRcpApprox>(gs);
                const uint32_t sf0 = quantize_block16_rt(vq[0], vq[1], q, exact, c0);
                const uint32_t sf1 = quantize_block16_rt(vq[2], vq[3], q, exact, c1);
                codes = make_uint4(c0[0], c0[1], c1[0], c1[1]);
                sf2 = sf0 | (sf1 << 8);
            }
        } else if (active && m < M) {
            if (p.a.xb != nullptr) {
                const uint4* src = reinterpret_cast<const uint4*>(
                    static_cast<const __nv_bfloat16*>(p.a.xb) + m * p.a.xb_stride + u * 32);
                const uint4 v0 = __ldg(src), v1 = __ldg(src + 1), v2 = __ldg(src + 2), v3 = __ldg(src + 3);
                uint32_t c0[2], c1[2], sf0, sf1;
                if (p.a.rcp_mode == kRcpExact) {
                    const QuantScales q = make_quant_scales<kRcpExact>(gs);
                    sf0 = quantize_block16<kRcpExact>(v0, v1, q, c0);
                    sf1 = quantize_block16<kRcpExact>(v2, v3, q, c1);
                } else {
                    const QuantScales q = make_quant_scales<kRcpApprox>(gs);
                    sf0 = quantize_block16<kRcpApprox>(v0, v1, q, c0);
                    sf1 = quantize_block16<kRcpApprox>(v2, v3, q, c1);
                }
                codes = make_uint4(c0[0], c0[1], c1[0], c1[1]);
                sf2 = sf0 | (sf1 << 8);
            } else {
                codes = ldg_keep_16(p.a.x + m * p.a.x_stride + u * kUnitBytes);
                sf2 = __ldg(reinterpret_cast<const unsigned short*>(p.a.xsf + m * p.a.xsf_stride + u * 2));
            }
        }
        Unit16 xu;
        decode_codes(codes, xu);
#pragma unroll
        for (int i = 0; i < 16; ++i) xh[m][i] = xu.h[i];
        xs[m] = __hmul2(as_half2(e4m3x2_to_f16x2(sf2)), as_half2(kTwoPowMinus6x2));
    }

    auto compute = [&](const Stage<R>& st, float* v) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            Unit16 wu;
            decode_codes(st.c[r], wu);
            const __half2 ws = as_half2(e4m3x2_to_f16x2(st.s[r]));
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                __half2 d0 = __hmul2(as_half2(wu.h[0]), as_half2(xh[m][0]));
                __half2 d1 = __hmul2(as_half2(wu.h[8]), as_half2(xh[m][8]));
#pragma unroll
                for (int i = 1; i < 8; ++i) {
                    d0 = __hfma2(as_half2(wu.h[i]), as_half2(xh[m][i]), d0);
                    d1 = __hfma2(as_half2(wu.h[8 + i]), as_half2(xh[m][8 + i]), d1);
                }
                const __half2 sc = __hmul2(ws, xs[m]);                       // exact (see kTwoPowMinus6x2)
                const __half b0 = __hadd(__low2half(d0), __high2half(d0));   // the two block sums
                const __half b1 = __hadd(__low2half(d1), __high2half(d1));
                v[r * MT + m] = fma_f16_f32(b1, __high2half(sc), fma_f16_f32(b0, __low2half(sc), 0.0f));
            }
        }
    };

    // part index of (local row lr, token m, warp kc) of this stream
    float* my_part = part + static_cast<size_t>(s) * p.stream_floats;
    const int writer = (lane & ((1 << kShift) - 1)) == 0;
    const int idx = lane >> kShift;                       // which of the pair's NV values this lane ends up with

    for (int st2 = 0; st2 < steps; st2 += 2) {
        float v[NV];
        compute(sa, v);
        load(sa, st2 + 2);
        if (st2 + 1 < steps) {
            compute(sb, v + R * MT);
            load(sb, st2 + 3);
        } else {
#pragma unroll
            for (int i = 0; i < R * MT; ++i) v[R * MT + i] = 0.0f;
        }
        butterfly<NV>(v, lane);
        if (writer) my_part[(st2 * R * MT + idx) * cw + kc] = v[0];
    }

    // Sum over the warps of each stream, in warp order, and store.
    __syncthreads();
    for (int t = tid; t < p.streams * p.stream_rows * MT; t += blockDim.x) {
        const int ss = t / (p.stream_rows * MT), e = t - ss * (p.stream_rows * MT);
        const int lr = e / MT, m = e - lr * MT;
        const int sid2 = blockIdx.x * p.streams + ss;
        const int rb = static_cast<int>(static_cast<int64_t>(sid2) * p.pairs / p.total_streams) * 2 * R;
        const int re = min(static_cast<int>(static_cast<int64_t>(sid2 + 1) * p.pairs / p.total_streams) * 2 * R, N);
        const int row = rb + lr;
        if (row < re && m < M) {
            const float* src = part + static_cast<size_t>(ss) * p.stream_floats + static_cast<size_t>(e) * cw;
            float sum = src[0];
            for (int j = 1; j < cw; ++j) sum += src[j];
            store_out(p.a.out, p.a.out_dtype, m * p.a.out_stride + row, sum * (p.a.alpha * kScaleFix));
        }
    }
}

struct RowsTuning {
    int mode;          // 0 automatic, 1 always when supported, -1 never
    int rows;          // R: 0 automatic, else 2 or 4
    int target_warps;  // warps per SM: 0 automatic
};
RowsTuning g_rows_tuning = {0, 0, 0};

}  // namespace

void set_gemv_rows_tuning(int mode, int rows, int target_warps) {
    g_rows_tuning.mode = mode;
    g_rows_tuning.rows = rows;
    g_rows_tuning.target_warps = target_warps;
}

// Kernel choice for one launch of at most 8 tokens. One token: the register-resident kernel
// for weights of 16 MB and more, for rows longer than 8192 elements and for every shape the
// ring kernel cannot take (K % 256 != 0), the ring kernel below that (measured on B200,
// L2-cold: 6144x4096 5.1 vs 5.3 us, 6400x5120 6.7 vs 6.3 us, 4096x12288 10.9 vs 7.8 us,
// 5120x3200 11.1 (plain loads) vs 4.9 us), and for N where the ring kernel's groups of 4 rows
// leave a second round to under a quarter of its warps (N = 5120: 5120x5120 7.3 us on the ring
// kernel). More tokens: the ring kernel.
cudaError_t launch_gemv_auto(const GemvArgs& a, cudaStream_t stream) {
    if (a.push_world > 1)        // the all-reduce inside the launch exists in the ring kernel only
        return (a.pro_kind == 0 && gemv_stream_supported(a)) ? launch_gemv_stream(a, stream) : cudaErrorNotSupported;
    if (a.pro_kind != 0)         // fused prologues exist in the register-resident kernel only
        return gemv_rows_supported(a) ? launch_gemv_rows(a, stream) : cudaErrorNotSupported;
    const bool ring = gemv_stream_supported(a);
    if (!gemv_tuning().force_generic && gemv_rows_supported(a)) {
        const int64_t wbytes = static_cast<int64_t>(a.N) * a.K * 9 / 16;
        const int ring_warps = device_sm_count() * 8, groups = (a.N + 3) / 4;
        // (only for rows long enough for the second round to matter: 5120x1024 runs in 2.7 us on
        // the ring kernel against 4.0 us here)
        const bool poor_ring_fit = groups > ring_warps && groups <= ring_warps + ring_warps / 4 && a.K >= 4096;
        if (g_rows_tuning.mode > 0 || !ring || wbytes >= 16000000 || a.K > 8192 || poor_ring_fit)
            return launch_gemv_rows(a, stream);
    }
    return ring ? launch_gemv_stream(a, stream) : launch_gemv_generic(a, stream);
}

namespace {

constexpr size_t kRowsMaxSmem = 96 * 1024;

// CTA shapes. A row narrower than 12 warps (K <= 12288) runs in CTAs of at most 12 warps, two
// of which fit an SM (80 registers per thread): either both belong to this launch (24 warps
// per SM hide the latency of the decode chains), or only one does and the other half of the SM
// is free for the NEXT launch, whose CTAs then request their first weights while this launch
// is still running (small weights, where the fixed part of a launch dominates). Rows of 13..24
// warps take one CTA per SM, wider ones one CTA of up to 32 warps at 64 registers.
enum RowsShape { kShapeHalf = 0, kShapeFull = 1, kShapeWide = 2 };

// Grid, block and shared-memory plan of one launch; false when the shape does not fit.
bool plan_rows(const GemvArgs& a, RowsParams* out, size_t* smem_bytes, int* rows_per_step, int* shape) {
    RowsParams p;
    p.a = a;
    p.units = a.K / 32;
    p.cw = (p.units + 31) / 32;
    if (p.cw < 1 || p.cw > kMaxWarps) return false;
    const RowsTuning& t = g_rows_tuning;
    const int sms = device_sm_count();
    const int MT = a.M == 1 ? 1 : 2;
    const int sh = p.cw <= 12 ? kShapeHalf : (p.cw <= 24 ? kShapeFull : kShapeWide);
    const int R = sh == kShapeWide ? (MT == 1 ? 2 : 1) : (MT == 1 ? (t.rows == 2 ? 2 : 4) : 2);
    int streams = sh == kShapeHalf ? 12 / p.cw : 1;
    // CTAs per SM of this launch (half shape only): both halves of the SM for weights of more
    // than about 12 MB, one half (leaving room for the next launch) below.
    int per_sm = 1;
    if (sh == kShapeHalf) {
        const int64_t wbytes = static_cast<int64_t>(a.N) * a.K * 9 / 16;
        per_sm = wbytes > 12000000 ? 2 : 1;
        if (t.target_warps > 0) per_sm = t.target_warps > 12 ? 2 : 1;
    }
    p.pairs = (a.N + 2 * R - 1) / (2 * R);
    int grid = sms * per_sm;
    while (streams > 1 && static_cast<int64_t>(streams) * grid > p.pairs) --streams;   // no idle streams
    if (static_cast<int64_t>(grid) * streams > p.pairs) grid = (p.pairs + streams - 1) / streams;
    p.streams = streams;
    p.total_streams = streams * grid;
    p.stream_rows = ((p.pairs + p.total_streams - 1) / p.total_streams) * 2 * R;
    p.stream_floats = p.stream_rows * MT * p.cw;
    const size_t smem = static_cast<size_t>(p.streams) * p.stream_floats * sizeof(float);
    if (smem > kRowsMaxSmem) return false;
    *out = p;
    *smem_bytes = smem;
    *rows_per_step = R;
    *shape = sh;
    return true;
}

}  // namespace

bool gemv_rows_supported(const GemvArgs& a) {
    if (g_rows_tuning.mode < 0) return false;
    if (a.M != 1 || a.N < 1) return false;      // two tokens spill at these register budgets: measured slower than the ring kernel
    if (static_cast<int64_t>(a.N) * a.w_stride_n >= (1ll << 32) || static_cast<int64_t>(a.N) * a.wsf_stride_n >= (1ll << 32))
        return false;                            // 32-bit byte offsets inside the weight
    if (a.K % 32 != 0 || a.K > 32 * 32 * kMaxWarps) return false;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) || (a.w_stride_n % 16) != 0) return false;
    if ((reinterpret_cast<uintptr_t>(a.wsf) & 1) || (a.wsf_stride_n % 2) != 0) return false;
    if (a.w_stride_n > (1 << 28) || a.wsf_stride_n > (1 << 28)) return false;     // 32-bit row offsets inside a step
    if (a.pro_kind == 1) {
        if (!a.residual_in || !a.residual_out || !a.norm_w || !a.gs) return false;
        if ((reinterpret_cast<uintptr_t>(a.residual_in) | reinterpret_cast<uintptr_t>(a.residual_out) |
             reinterpret_cast<uintptr_t>(a.norm_w) | reinterpret_cast<uintptr_t>(a.delta)) & 15)
            return false;
        if (a.K % 8 != 0) return false;
    } else if (a.xb != nullptr) {
        if ((reinterpret_cast<uintptr_t>(a.xb) & 15) || (a.xb_stride % 8) != 0) return false;
        if (a.pro_kind == 2 && (a.K % 8 != 0 || a.xb_stride < 2 * static_cast<int64_t>(a.K))) return false;
    } else {
        if (a.pro_kind != 0) return false;
        if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (a.x_stride % 16) != 0) return false;
        if ((reinterpret_cast<uintptr_t>(a.xsf) & 1) || (a.xsf_stride % 2) != 0) return false;
    }
    RowsParams p;
    size_t smem;
    int R, shape;
    return plan_rows(a, &p, &smem, &R, &shape);
}

cudaError_t launch_gemv_rows(const GemvArgs& a, cudaStream_t stream) {
    RowsParams p;
    size_t smem = 0;
    int R = 4, shape = kShapeHalf;
    if (!plan_rows(a, &p, &smem, &R, &shape)) return cudaErrorInvalidConfiguration;
    const int grid = p.total_streams / p.streams;
    const int streams = p.streams;

    using Kern = void (*)(RowsParams);
#define NVFP4R_ROWS_SHAPES(PLAIN)                                                           \
    {{gemv_rows_kernel<1, 4, 384, 2, PLAIN>, gemv_rows_kernel<1, 2, 384, 2, PLAIN>},        \
     {gemv_rows_kernel<1, 4, 768, 1, PLAIN>, gemv_rows_kernel<1, 2, 768, 1, PLAIN>},        \
     {gemv_rows_kernel<1, 2, 1024, 1, false>, gemv_rows_kernel<1, 2, 1024, 1, false>}}
    // [with prologues / plain][half (R 4 / R 2), full (R 4 / R 2), wide (R 2)]; at the wide shape's
    // 64 registers the plain instance spills more than the full one, so both entries are the latter
    static const Kern table[2][3][2] = {NVFP4R_ROWS_SHAPES(false), NVFP4R_ROWS_SHAPES(true)};
#undef NVFP4R_ROWS_SHAPES
    const int plain = a.pro_kind == 0 ? 1 : 0;
    const int rsel = R == 2 ? 1 : 0;
    const Kern kern = table[plain][shape][rsel];
    const int ki = (plain * 3 + shape) * 2 + rsel;
    static bool attr_done[12][64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && !attr_done[ki][dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kRowsMaxSmem));
        if (e != cudaSuccess) return e;
        attr_done[ki][dev] = true;
    }

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(static_cast<unsigned>(streams * p.cw * 32));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gemv_tuning().use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace nvfp4r
