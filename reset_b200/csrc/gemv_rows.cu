// NVFP4 W4A4 GEMV for one or two tokens: activations stay in registers, weights
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

__device__ __forceinline__ float2 decode_scale_pair(uint32_t two_bytes) {
    return __half22float2(as_half2(e4m3x2_to_f16x2(two_bytes)));
}

__device__ __forceinline__ void store_out(void* out, int dtype, int64_t idx, float v) {
    if (dtype == 0)      static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
    else if (dtype == 1) static_cast<__half*>(out)[idx] = __float2half_rn(v);
    else                 static_cast<float*>(out)[idx] = v;
}

__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(threads) : "memory");
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

template <int R>
struct Stage {
    uint4 c[R];
    uint32_t s[R];
};

template <int R>
__device__ __forceinline__ void load_stage(Stage<R>& st, const uint8_t* wp, const uint8_t* sp,
                                           int64_t w_stride, int64_t sf_stride, int row0, int row_end,
                                           bool active) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = row0 + r;
        if (active && row < row_end) {
            st.c[r] = ldg_stream_16(wp + row * w_stride);
            st.s[r] = ldg_stream_2(sp + row * sf_stride);
        } else {
            st.c[r] = make_uint4(0u, 0u, 0u, 0u);
            st.s[r] = 0u;
        }
    }
}

template <int MT, int R, int MAXT>
__global__ void __launch_bounds__(MAXT, 1)
gemv_rows_kernel(const __grid_constant__ RowsParams p) {
    constexpr int NV = R * MT;
    constexpr int kShift = NV == 1 ? 5 : NV == 2 ? 4 : NV == 4 ? 3 : NV == 8 ? 2 : 1;
    __shared__ float part[2 * NV * kMaxWarps];

    const int tid = threadIdx.x, lane = tid & 31, wi = tid >> 5;
    const int cw = p.cw;
    const int s = wi / cw, kc = wi - s * cw;
    const int nwarps = blockDim.x >> 5;
    const int u = kc * 32 + lane;
    const bool active = u < p.units;
    const int N = p.a.N, M = p.a.M;
    const int sid = blockIdx.x * p.streams + s;
    const int row_begin = static_cast<int>(static_cast<int64_t>(sid) * N / p.total_streams);
    const int row_end = static_cast<int>(static_cast<int64_t>(sid + 1) * N / p.total_streams);

    const uint8_t* wp = p.a.w + u * kUnitBytes;
    const uint8_t* sp = p.a.wsf + u * 2;
    const int64_t w_stride = p.a.w_stride_n, sf_stride = p.a.wsf_stride_n;

    // Weights do not depend on the preceding kernel.
    Stage<R> sa, sb;
    load_stage<R>(sa, wp, sp, w_stride, sf_stride, row_begin, row_end, active);
    load_stage<R>(sb, wp, sp, w_stride, sf_stride, row_begin + R, row_end, active);
    const float gs = (p.a.xb != nullptr) ? __ldg(p.a.gs) : 1.0f;
    pdl_launch_dependents();
    pdl_wait_prior();

    // This lane's slice of the activations, decoded once.
    uint32_t xh[MT][16];
    float2 xs[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        uint4 codes = make_uint4(0u, 0u, 0u, 0u);
        uint32_t sf2 = 0u;
        if (active && m < M) {
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
        xs[m] = decode_scale_pair(sf2);
    }

    int parity = 0;
    auto compute = [&](const Stage<R>& st, int row0) {
        float v[NV];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            Unit16 wu;
            decode_codes(st.c[r], wu);
            const float2 ws = decode_scale_pair(st.s[r]);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                __half2 d0 = __hmul2(as_half2(wu.h[0]), as_half2(xh[m][0]));
                __half2 d1 = __hmul2(as_half2(wu.h[8]), as_half2(xh[m][8]));
#pragma unroll
                for (int i = 1; i < 8; ++i) {
                    d0 = __hfma2(as_half2(wu.h[i]), as_half2(xh[m][i]), d0);
                    d1 = __hfma2(as_half2(wu.h[8 + i]), as_half2(xh[m][8 + i]), d1);
                }
                const float f0 = __half2float(__hadd(__low2half(d0), __high2half(d0)));
                const float f1 = __half2float(__hadd(__low2half(d1), __high2half(d1)));
                v[r * MT + m] = fmaf(f1, ws.y * xs[m].y, f0 * (ws.x * xs[m].x));
            }
        }
        butterfly<NV>(v, lane);
        const int idx = lane >> kShift;
        if (cw == 1) {
            if ((lane & ((1 << kShift) - 1)) == 0) {
                const int r = idx / MT, m = idx - r * MT;
                const int row = row0 + r;
                if (row < row_end && m < M)
                    store_out(p.a.out, p.a.out_dtype, m * p.a.out_stride + row, v[0] * p.a.alpha);
            }
        } else {
            if ((lane & ((1 << kShift) - 1)) == 0) part[(parity * NV + idx) * nwarps + wi] = v[0];
            named_barrier(1 + s, cw * 32);
            if (kc == 0 && lane < NV) {
                const float* src = &part[(parity * NV + lane) * nwarps + s * cw];
                float sum = src[0];
                for (int j = 1; j < cw; ++j) sum += src[j];
                const int r = lane / MT, m = lane - r * MT;
                const int row = row0 + r;
                if (row < row_end && m < M)
                    store_out(p.a.out, p.a.out_dtype, m * p.a.out_stride + row, sum * p.a.alpha);
            }
            parity ^= 1;
        }
    };

    for (int row0 = row_begin; row0 < row_end; row0 += 2 * R) {
        compute(sa, row0);
        load_stage<R>(sa, wp, sp, w_stride, sf_stride, row0 + 2 * R, row_end, active);
        if (row0 + R < row_end) {
            compute(sb, row0 + R);
            load_stage<R>(sb, wp, sp, w_stride, sf_stride, row0 + 3 * R, row_end, active);
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

cudaError_t launch_gemv_auto(const GemvArgs& a, cudaStream_t stream) {
    if (!gemv_tuning().force_generic && gemv_rows_supported(a)) return launch_gemv_rows(a, stream);
    return gemv_stream_supported(a) ? launch_gemv_stream(a, stream) : launch_gemv_generic(a, stream);
}

bool gemv_rows_supported(const GemvArgs& a) {
    if (g_rows_tuning.mode < 0) return false;
    if (a.M < 1 || a.M > 2) return false;
    if (a.K % 32 != 0 || a.K > 32 * 32 * kMaxWarps) return false;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) || (a.w_stride_n % 16) != 0) return false;
    if ((reinterpret_cast<uintptr_t>(a.wsf) & 1) || (a.wsf_stride_n % 2) != 0) return false;
    if (a.xb != nullptr) {
        if ((reinterpret_cast<uintptr_t>(a.xb) & 15) || (a.xb_stride % 8) != 0) return false;
    } else {
        if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (a.x_stride % 16) != 0) return false;
        if ((reinterpret_cast<uintptr_t>(a.xsf) & 1) || (a.xsf_stride % 2) != 0) return false;
    }
    return true;
}

cudaError_t launch_gemv_rows(const GemvArgs& a, cudaStream_t stream) {
    RowsParams p;
    p.a = a;
    p.units = a.K / 32;
    p.cw = (p.units + 31) / 32;
    const RowsTuning& t = g_rows_tuning;
    const int sms = device_sm_count();

    // Warps per SM: bounded by the register file (MAXT = 768 threads of <= 78 registers, or
    // 1024 of 64 for rows wider than 24 warps).
    const bool wide = p.cw > 24;
    const int max_warps = wide ? 32 : 24;
    int target = t.target_warps > 0 ? t.target_warps : 24;
    if (target > max_warps) target = max_warps;
    int streams = target / p.cw;
    if (streams < 1) streams = 1;
    if (p.cw > 1 && streams > 15) streams = 15;       // one named barrier per stream
    if (streams * p.cw > max_warps) streams = max_warps / p.cw;
    // No more streams than rows / 2 over the whole grid.
    while (streams > 1 && static_cast<int64_t>(streams) * sms * 2 > a.N) --streams;
    int grid = sms;
    if (static_cast<int64_t>(grid) * streams > a.N) grid = (a.N + streams - 1) / streams;
    p.streams = streams;
    p.total_streams = streams * grid;

    const int R = t.rows > 0 ? t.rows : 4;
    using Kern = void (*)(RowsParams);
    Kern kern;
    if (a.M == 1) {
        if (wide) kern = gemv_rows_kernel<1, 2, 1024>;
        else kern = (R == 2) ? gemv_rows_kernel<1, 2, 768> : gemv_rows_kernel<1, 4, 768>;
    } else {
        if (wide) kern = gemv_rows_kernel<2, 1, 1024>;
        else kern = (R == 2) ? gemv_rows_kernel<2, 2, 768> : gemv_rows_kernel<2, 2, 768>;
    }

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(static_cast<unsigned>(streams * p.cw * 32));
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gemv_tuning().use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace nvfp4r
