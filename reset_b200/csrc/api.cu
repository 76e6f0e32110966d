// extern "C" entry points: argument checks, then the kernel launchers.
#include <cstdio>
#include <cstring>
#include <mutex>

#include <nvtx3/nvToolsExt.h>

#include "../../include/nvfp4r_b200.h"
#include "kernels.h"
#include "reset_kernels.h"

namespace {

// One NVTX range per launching entry point (domain "nvfp4r"): a timeline tool shows which
// call of the C ABI issued which kernels. Costs a few nanoseconds when no tool is attached
// (the header-only NVTX v3 resolves to no-ops then).
struct NvtxRange {
    static nvtxDomainHandle_t domain() {
        static nvtxDomainHandle_t d = nvtxDomainCreateA("nvfp4r");
        return d;
    }
    explicit NvtxRange(const char* name) { nvtxDomainRangePushEx(domain(), &attr(name)); }
    ~NvtxRange() { nvtxDomainRangePop(domain()); }
    static const nvtxEventAttributes_t& attr(const char* name) {
        thread_local nvtxEventAttributes_t a = {};
        a.version = NVTX_VERSION;
        a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
        a.messageType = NVTX_MESSAGE_TYPE_ASCII;
        a.message.ascii = name;
        return a;
    }
};
#define NVFP4R_RANGE(name) NvtxRange nvtx_range_(name)

thread_local char g_last_error[256] = "";

int cuda_fail(cudaError_t e, const char* where) {
    std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s", where, cudaGetErrorString(e));
    return NVFP4R_ERR_CUDA;
}
int fail(int code, const char* why) {
    std::snprintf(g_last_error, sizeof(g_last_error), "%s", why);
    return code;
}
inline bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

}  // namespace

extern "C" {

const char* nvfp4r_status_string(int status) {
    switch (status) {
        case NVFP4R_OK: return "ok";
        case NVFP4R_ERR_INVALID_ARGUMENT: return "invalid argument";
        case NVFP4R_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
        case NVFP4R_ERR_ALIGNMENT: return "pointer or stride alignment";
        case NVFP4R_ERR_CUDA: return "CUDA runtime error";
        case NVFP4R_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
        default: return "unknown status";
    }
}

const char* nvfp4r_last_error(void) { return g_last_error; }

int nvfp4r_version(void) { return 1000 * 0 + 1; }

int nvfp4r_quant(const void* x, int64_t x_row_stride, int M, int K, const float* gs,
                 void* codes, void* scales, int sf_layout, int rcp_mode, void* stream) {
    NVFP4R_RANGE("nvfp4r_quant");
    if (!x || !gs || !codes || !scales) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "quant: null pointer");
    if (M < 0 || K <= 0) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "quant: M/K must be positive");
    if (sf_layout != NVFP4R_SF_FLAT && sf_layout != NVFP4R_SF_SWIZZLED)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "quant: bad sf_layout");
    if (rcp_mode != NVFP4R_RCP_EXACT && rcp_mode != NVFP4R_RCP_APPROX)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "quant: bad rcp_mode");
    if (K % 16 != 0) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "quant: K must be a multiple of 16");
    if (!aligned(x, 16) || (x_row_stride % 8) != 0 || !aligned(codes, 8))
        return fail(NVFP4R_ERR_ALIGNMENT, "quant: x rows must be 16-byte aligned, codes 8-byte");
    if (x_row_stride < K) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "quant: row stride < K");
    if (M == 0) return NVFP4R_OK;
    cudaError_t e = nvfp4r::launch_quant(x, x_row_stride, M, K, gs, codes, scales,
                                         sf_layout == NVFP4R_SF_SWIZZLED, rcp_mode, as_stream(stream));
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "quant launch");
}

int nvfp4r_gemv(const void* weight, const void* weight_scale, const void* x, const void* x_scale,
                void* out, int L, int N, int K, int64_t w_stride_l, int64_t w_stride_n,
                int64_t wsf_stride_l, int64_t wsf_stride_n, int64_t x_stride_l,
                int64_t xsf_stride_l, float alpha, int out_dtype, void* stream) {
    NVFP4R_RANGE("nvfp4r_gemv");
    if (!weight || !weight_scale || !x || !x_scale || !out)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "gemv: null pointer");
    if (L < 0 || N < 0 || K <= 0) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "gemv: bad sizes");
    if (out_dtype < NVFP4R_BF16 || out_dtype > NVFP4R_F32)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "gemv: bad out_dtype");
    if (K % 32 != 0) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "gemv: K must be a multiple of 32");
    if (w_stride_n < K / 2 || wsf_stride_n < K / 16)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "gemv: weight row stride smaller than a row");
    if (!aligned(weight, 16) || !aligned(x, 16) || (w_stride_n % 16) || (x_stride_l % 16) ||
        (w_stride_l % 16) || !aligned(weight_scale, 2) || !aligned(x_scale, 2) ||
        (wsf_stride_n % 2) || (xsf_stride_l % 2) || (wsf_stride_l % 2))
        return fail(NVFP4R_ERR_ALIGNMENT, "gemv: codes need 16-byte, scales 2-byte alignment");
    if (L == 0 || N == 0) return NVFP4R_OK;

    const size_t out_elt = out_dtype == NVFP4R_F32 ? 4 : 2;
    nvfp4r::GemvArgs a = {};
    a.w_stride_n = w_stride_n;
    a.wsf_stride_n = wsf_stride_n;
    a.x_stride = x_stride_l;
    a.xsf_stride = xsf_stride_l;
    a.out_stride = N;
    a.out_dtype = out_dtype;
    a.N = N;
    a.K = K;
    a.alpha = alpha;
    const bool broadcast = (w_stride_l == 0 && wsf_stride_l == 0);
    const int group = broadcast ? 8 : 1;
    for (int l0 = 0; l0 < L; l0 += group) {
        const int m = broadcast ? (L - l0 < group ? L - l0 : group) : 1;
        a.w = static_cast<const uint8_t*>(weight) + (broadcast ? 0 : l0 * w_stride_l);
        a.wsf = static_cast<const uint8_t*>(weight_scale) + (broadcast ? 0 : l0 * wsf_stride_l);
        a.x = static_cast<const uint8_t*>(x) + l0 * x_stride_l;
        a.xsf = static_cast<const uint8_t*>(x_scale) + l0 * xsf_stride_l;
        a.out = static_cast<uint8_t*>(out) + static_cast<size_t>(l0) * N * out_elt;
        a.M = m;
        cudaError_t e = nvfp4r::launch_gemv_auto(a, as_stream(stream));
        if (e != cudaSuccess) return cuda_fail(e, "gemv launch");
    }
    return NVFP4R_OK;
}

int nvfp4r_linear(const void* x, int64_t x_row_stride, int M, int K, const float* gs,
                  const void* weight, const void* weight_scale, int N, float alpha, void* out,
                  int out_dtype, int rcp_mode, void* stream) {
    NVFP4R_RANGE("nvfp4r_linear");
    if (!x || !gs || !weight || !weight_scale || !out)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear: null pointer");
    if (M < 0 || N < 0 || K <= 0) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear: bad sizes");
    if (M > NVFP4R_LINEAR_MAX_M) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear: M above NVFP4R_LINEAR_MAX_M");
    if (out_dtype < NVFP4R_BF16 || out_dtype > NVFP4R_F32)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear: bad out_dtype");
    if (rcp_mode != NVFP4R_RCP_EXACT && rcp_mode != NVFP4R_RCP_APPROX)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear: bad rcp_mode");
    if (K % 32 != 0) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear: K must be a multiple of 32");
    if (!aligned(x, 16) || (x_row_stride % 8) || !aligned(weight, 16) || !aligned(weight_scale, 2))
        return fail(NVFP4R_ERR_ALIGNMENT, "linear: x/weight need 16-byte alignment");
    if (x_row_stride < K) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear: row stride < K");
    if (M == 0 || N == 0) return NVFP4R_OK;

    const size_t out_elt = out_dtype == NVFP4R_F32 ? 4 : 2;
    nvfp4r::GemvArgs a = {};
    a.w = static_cast<const uint8_t*>(weight);
    a.wsf = static_cast<const uint8_t*>(weight_scale);
    a.w_stride_n = K / 2;
    a.wsf_stride_n = K / 16;
    a.xb_stride = x_row_stride;
    a.gs = gs;
    a.rcp_mode = rcp_mode;
    a.out_stride = N;
    a.out_dtype = out_dtype;
    a.N = N;
    a.K = K;
    a.alpha = alpha;
    for (int m0 = 0; m0 < M; m0 += 8) {
        a.M = M - m0 < 8 ? M - m0 : 8;
        a.xb = static_cast<const uint8_t*>(x) + static_cast<size_t>(m0) * x_row_stride * 2;
        a.out = static_cast<uint8_t*>(out) + static_cast<size_t>(m0) * N * out_elt;
        cudaError_t e = nvfp4r::launch_gemv_auto(a, as_stream(stream));
        if (e != cudaSuccess) return cuda_fail(e, "linear launch");
    }
    return NVFP4R_OK;
}

int nvfp4r_linear_ex(const nvfp4r_prologue* pro, const void* x, int64_t x_row_stride, int M, int K,
                     const float* gs, const void* weight, const void* weight_scale, int N, float alpha,
                     void* out, int out_dtype, int rcp_mode, void* stream) {
    NVFP4R_RANGE("nvfp4r_linear_ex");
    if (!pro) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: null prologue");
    if (pro->push_to != nullptr) {
        // Row-parallel shard small enough for the GEMV: push and sum inside the GEMV's launch.
        const nvfp4r_peer_comm* c = pro->push_to;
        if (pro->kind != NVFP4R_PROLOGUE_NONE || !pro->push_gather)
            return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE,
                        "linear_ex: with push_to the GEMV takes no fused prologue and always sums in its own launch "
                        "(push_gather = 1); other forms need the packed linear (nvfp4r_linear_packed_ex)");
        if (!x || !gs || !weight || !weight_scale || !out) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: null pointer");
        if (M != 1 || out_dtype != NVFP4R_BF16 || N <= 0 || (N & 1) || K <= 0)
            return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear_ex: push_to takes one token, bf16 output, even N");
        if (c->world < 2 || c->world > NVFP4R_PEER_MAX_WORLD || c->rank < 0 || c->rank >= c->world ||
            static_cast<size_t>(N) > c->max_elems)
            return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: bad communicator or output larger than its slots");
        if (rcp_mode != NVFP4R_RCP_EXACT && rcp_mode != NVFP4R_RCP_APPROX)
            return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: bad rcp_mode");
        nvfp4r::GemvArgs a = {};
        a.w = static_cast<const uint8_t*>(weight);
        a.wsf = static_cast<const uint8_t*>(weight_scale);
        a.w_stride_n = K / 2;
        a.wsf_stride_n = K / 16;
        a.xb = x;
        a.xb_stride = x_row_stride;
        a.gs = gs;
        a.rcp_mode = rcp_mode;
        a.out = out;
        a.out_stride = N;
        a.out_dtype = out_dtype;
        a.N = N;
        a.K = K;
        a.M = 1;
        a.alpha = alpha;
        a.push_world = c->world;
        a.push_rank = c->rank;
        a.push_max_pairs = (c->max_elems + 1) / 2;
        for (int r = 0; r < c->world; ++r) a.push_base[r] = static_cast<unsigned char*>(c->base[r]);
        a.push_poll_limit = nvfp4r::peer_poll_limit();
        if (!nvfp4r::gemv_stream_supported(a))
            return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear_ex: shape or alignment outside the streaming GEMV (K % 256, 16-byte rows)");
        cudaError_t e = nvfp4r::launch_gemv_auto(a, as_stream(stream));
        return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "linear_ex launch");
    }
    if (pro->kind == NVFP4R_PROLOGUE_NONE)
        return nvfp4r_linear(x, x_row_stride, M, K, gs, weight, weight_scale, N, alpha, out, out_dtype, rcp_mode, stream);
    if (pro->kind != NVFP4R_PROLOGUE_ADD_RMSNORM && pro->kind != NVFP4R_PROLOGUE_SILU_MUL)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: bad prologue kind");
    if (!gs || !weight || !weight_scale || !out) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: null pointer");
    if (M != 1) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear_ex: the GEMV's fused prologues take one token (M = 1)");
    if (N <= 0 || K <= 0 || K % 32 != 0) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear_ex: K must be a multiple of 32");
    if (out_dtype < NVFP4R_BF16 || out_dtype > NVFP4R_F32) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: bad out_dtype");
    if (rcp_mode != NVFP4R_RCP_EXACT && rcp_mode != NVFP4R_RCP_APPROX)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: bad rcp_mode");
    if (!aligned(weight, 16) || !aligned(weight_scale, 2)) return fail(NVFP4R_ERR_ALIGNMENT, "linear_ex: weight alignment");
    nvfp4r::GemvArgs a = {};
    a.w = static_cast<const uint8_t*>(weight);
    a.wsf = static_cast<const uint8_t*>(weight_scale);
    a.w_stride_n = K / 2;
    a.wsf_stride_n = K / 16;
    a.gs = gs;
    a.rcp_mode = rcp_mode;
    a.out = out;
    a.out_stride = N;
    a.out_dtype = out_dtype;
    a.N = N;
    a.K = K;
    a.M = 1;
    a.alpha = alpha;
    a.pro_kind = pro->kind;
    if (pro->kind == NVFP4R_PROLOGUE_ADD_RMSNORM) {
        if (!pro->residual_in || !pro->residual_out || !pro->norm_weight)
            return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: RMSNorm prologue needs residual_in/out and norm_weight");
        if (pro->residual_in == pro->residual_out)
            return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: residual_out must not alias residual_in");
        a.delta = pro->delta; a.residual_in = pro->residual_in; a.residual_out = pro->residual_out;
        a.norm_w = pro->norm_weight; a.eps = pro->eps;
    } else {
        if (!x || !aligned(x, 16) || (x_row_stride % 8) || x_row_stride < 2 * static_cast<int64_t>(K))
            return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_ex: SiLU prologue needs x = [M, 2K] gate|up, 16-byte aligned");
        a.xb = x; a.xb_stride = x_row_stride;
    }
    if (!nvfp4r::gemv_rows_supported(a))
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear_ex: shape or alignment outside the register-resident GEMV");
    cudaError_t e = nvfp4r::launch_gemv_auto(a, as_stream(stream));
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "linear_ex launch");
}

size_t nvfp4r_gemm_workspace_bytes(int M, int N, int K) {
    return nvfp4r::gemm_workspace_bytes(M, N, K);
}

static int tc_common_checks(const char* who, int M, int N, int K, int out_dtype, const void* workspace,
                            size_t workspace_bytes) {
    if (M < 0 || N < 0 || K <= 0) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "tensor-core path: bad sizes");
    if (out_dtype < NVFP4R_BF16 || out_dtype > NVFP4R_F32)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "tensor-core path: bad out_dtype");
    if (N % 128 != 0) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "tensor-core path: N must be a multiple of 128");
    if (K % 256 != 0) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "tensor-core path: K must be a multiple of 256");
    if (M == 0 || N == 0) return NVFP4R_OK;
    if (!workspace || workspace_bytes < nvfp4r_gemm_workspace_bytes(M, N, K) || !aligned(workspace, 16))
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "tensor-core path: workspace missing, too small or misaligned");
    (void)who;
    return NVFP4R_OK;
}

int nvfp4r_gemm(const void* A, const void* B, const void* SFA, const void* SFB, void* C, int M, int N,
                int K, float alpha, int out_dtype, int c_layout, void* workspace,
                size_t workspace_bytes, void* stream) {
    NVFP4R_RANGE("nvfp4r_gemm");
    if (!A || !B || !SFA || !SFB || !C) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "gemm: null pointer");
    if (c_layout != NVFP4R_C_M_MAJOR && c_layout != NVFP4R_C_N_MAJOR)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "gemm: bad c_layout");
    int st = tc_common_checks("gemm", M, N, K, out_dtype, workspace, workspace_bytes);
    if (st != NVFP4R_OK || M == 0 || N == 0) return st;
    if (!aligned(A, 16) || !aligned(B, 16) || !aligned(SFA, 16) || !aligned(SFB, 16))
        return fail(NVFP4R_ERR_ALIGNMENT, "gemm: operands need 16-byte alignment");
    nvfp4r::TcLinearArgs g = {};
    g.w = B; g.wsf_swizzled = SFB;
    g.a_codes = A; g.a_sf_swizzled = SFA;
    g.out = C; g.out_dtype = out_dtype; g.c_n_major = (c_layout == NVFP4R_C_N_MAJOR);
    g.M = M; g.N = N; g.K = K; g.alpha = alpha; g.workspace = workspace;
    const char* why = nullptr;
    cudaError_t e = nvfp4r::launch_linear_tc(g, as_stream(stream), &why);
    if (why != nullptr) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, why);
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "gemm launch");
}

int nvfp4r_linear_tc(const void* x, int64_t x_row_stride, int M, int K, const float* gs,
                     const void* weight, const void* weight_scale_swizzled, int N, float alpha,
                     void* out, int out_dtype, int rcp_mode, void* workspace, size_t workspace_bytes,
                     void* stream) {
    NVFP4R_RANGE("nvfp4r_linear_tc");
    if (!x || !gs || !weight || !weight_scale_swizzled || !out)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_tc: null pointer");
    if (rcp_mode != NVFP4R_RCP_EXACT && rcp_mode != NVFP4R_RCP_APPROX)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_tc: bad rcp_mode");
    int st = tc_common_checks("linear_tc", M, N, K, out_dtype, workspace, workspace_bytes);
    if (st != NVFP4R_OK || M == 0 || N == 0) return st;
    if (!aligned(x, 16) || (x_row_stride % 8) || !aligned(weight, 16) || !aligned(weight_scale_swizzled, 16))
        return fail(NVFP4R_ERR_ALIGNMENT, "linear_tc: x/weight need 16-byte alignment");
    if (x_row_stride < K) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_tc: row stride < K");
    nvfp4r::TcLinearArgs g = {};
    g.w = weight; g.wsf_swizzled = weight_scale_swizzled;
    g.xb = x; g.xb_stride = x_row_stride; g.gs = gs; g.rcp_mode = rcp_mode;
    g.out = out; g.out_dtype = out_dtype; g.c_n_major = false;
    g.M = M; g.N = N; g.K = K; g.alpha = alpha; g.workspace = workspace;
    const char* why = nullptr;
    cudaError_t e = nvfp4r::launch_linear_tc(g, as_stream(stream), &why);
    if (why != nullptr) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, why);
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "linear_tc launch");
}

#ifdef NVFP4R_TRACE
// Diagnostics of a -DNVFP4R_TRACE build only (not in the header, not in the default library):
// the %globaltimer time line of eight CTAs of the last four packed-linear launches (enabled by
// bit 8 of nvfp4r_set_packed_tuning).
NVFP4R_API int nvfp4r_debug_read_trace(unsigned long long* out16) {
    cudaDeviceSynchronize();
    return nvfp4r::read_packed_trace(out16) == cudaSuccess ? 0 : -4;
}
#endif
size_t nvfp4r_packed_weight_bytes(int N, int K) {
    if (N <= 0 || K <= 0 || N % 128 || K % 128) return 0;
    return nvfp4r::packed_weight_bytes(N, K);
}

size_t nvfp4r_linear_packed_workspace_bytes(int M, int N, int K) {
    return nvfp4r::packed_workspace_bytes(M, N, K);
}

int nvfp4r_pack_weight(const void* weight, const void* weight_scale_flat, void* packed, int N, int K,
                       void* stream) {
    NVFP4R_RANGE("nvfp4r_pack_weight");
    if (!weight || !weight_scale_flat || !packed) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "pack_weight: null pointer");
    if (N <= 0 || K <= 0) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "pack_weight: bad sizes");
    if (N % 128 != 0 || K % 128 != 0)
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "pack_weight: N % 128 == 0 and K % 128 == 0 required");
    if (!aligned(weight, 16) || !aligned(weight_scale_flat, 4) || !aligned(packed, 16))
        return fail(NVFP4R_ERR_ALIGNMENT, "pack_weight: weight 16-byte, scales 4-byte, packed 16-byte aligned");
    cudaError_t e = nvfp4r::launch_pack_weight(weight, weight_scale_flat, packed, N, K, as_stream(stream));
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "pack_weight launch");
}

int nvfp4r_linear_packed(const void* x, int64_t x_row_stride, int M, int K, const float* gs,
                         const void* packed, int N, float alpha, void* out, int out_dtype, int rcp_mode,
                         void* workspace, size_t workspace_bytes, void* stream) {
    NVFP4R_RANGE("nvfp4r_linear_packed");
    if (!x || !gs || !packed || !out) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed: null pointer");
    if (rcp_mode != NVFP4R_RCP_EXACT && rcp_mode != NVFP4R_RCP_APPROX)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed: bad rcp_mode");
    if (M < 0 || N < 0 || K <= 0) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed: bad sizes");
    if (out_dtype < NVFP4R_BF16 || out_dtype > NVFP4R_F32)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed: bad out_dtype");
    if (N % 128 != 0 || K % 128 != 0)
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear_packed: N % 128 == 0 and K % 128 == 0 required");
    if (M == 0 || N == 0) return NVFP4R_OK;
    if (!workspace || workspace_bytes < nvfp4r_linear_packed_workspace_bytes(M, N, K) || !aligned(workspace, 16))
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed: workspace missing, too small or misaligned");
    if (!aligned(x, 16) || (x_row_stride % 8) || !aligned(packed, 16))
        return fail(NVFP4R_ERR_ALIGNMENT, "linear_packed: x and packed weight need 16-byte alignment");
    if (x_row_stride < K) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed: row stride < K");
    nvfp4r::PackedLinearArgs g = {};
    g.packed = packed; g.xb = x; g.xb_stride = x_row_stride; g.gs = gs; g.rcp_mode = rcp_mode;
    g.out = out; g.out_dtype = out_dtype; g.M = M; g.N = N; g.K = K; g.alpha = alpha; g.workspace = workspace;
    const char* why = nullptr;
    cudaError_t e = nvfp4r::launch_linear_packed(g, as_stream(stream), &why);
    if (why != nullptr) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, why);
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "linear_packed launch");
}

int nvfp4r_linear_packed_ex(const nvfp4r_prologue* pro, const void* x, int64_t x_row_stride, int M, int K,
                            const float* gs, const void* packed, int N, float alpha, void* out,
                            int out_dtype, int rcp_mode, void* workspace, size_t workspace_bytes,
                            void* stream) {
    NVFP4R_RANGE("nvfp4r_linear_packed_ex");
    if (!pro) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: null prologue");
    if (pro->kind == NVFP4R_PROLOGUE_NONE && pro->push_to == nullptr)
        return nvfp4r_linear_packed(x, x_row_stride, M, K, gs, packed, N, alpha, out, out_dtype, rcp_mode,
                                    workspace, workspace_bytes, stream);
    if (pro->kind != NVFP4R_PROLOGUE_NONE && pro->kind != NVFP4R_PROLOGUE_ADD_RMSNORM &&
        pro->kind != NVFP4R_PROLOGUE_SILU_MUL)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: bad prologue kind");
    if (pro->push_to != nullptr) {
        const nvfp4r_peer_comm* c = pro->push_to;
        if (c->world < 1 || c->world > NVFP4R_PEER_MAX_WORLD || c->rank < 0 || c->rank >= c->world)
            return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: bad peer communicator");
        if (out_dtype != NVFP4R_BF16 || (N & 1) ||
            static_cast<size_t>(M) * static_cast<size_t>(N) > c->max_elems)
            return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear_packed_ex: push needs bf16 output of at most max_elems elements");
        for (int r = 0; r < c->world; ++r)
            if (!c->base[r]) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: peer base missing");
    }
    if (!gs || !packed || !out) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: null pointer");
    if (rcp_mode != NVFP4R_RCP_EXACT && rcp_mode != NVFP4R_RCP_APPROX)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: bad rcp_mode");
    if (M < 0 || N < 0 || K <= 0) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: bad sizes");
    if (out_dtype < NVFP4R_BF16 || out_dtype > NVFP4R_F32)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: bad out_dtype");
    if (N % 128 != 0 || K % 128 != 0)
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear_packed_ex: N % 128 == 0 and K % 128 == 0 required");
    if (pro->kind == NVFP4R_PROLOGUE_ADD_RMSNORM && K % 256 != 0)
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear_packed_ex: the RMSNorm prologue needs K % 256 == 0");
    if (M == 0 || N == 0) return NVFP4R_OK;
    if (!workspace || workspace_bytes < nvfp4r_linear_packed_workspace_bytes(M, N, K) || !aligned(workspace, 16))
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: workspace missing, too small or misaligned");
    nvfp4r::PackedLinearArgs g = {};
    g.packed = packed; g.gs = gs; g.rcp_mode = rcp_mode;
    g.out = out; g.out_dtype = out_dtype; g.M = M; g.N = N; g.K = K; g.alpha = alpha; g.workspace = workspace;
    g.pro_kind = pro->kind;
    if (pro->kind == NVFP4R_PROLOGUE_ADD_RMSNORM) {
        if (!pro->residual_in || !pro->residual_out || !pro->norm_weight)
            return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: RMSNorm prologue needs residual_in/out and norm_weight");
        if (pro->residual_in == pro->residual_out)
            return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: residual_out must not alias residual_in");
        if (!aligned(pro->residual_in, 16) || !aligned(pro->residual_out, 16) || !aligned(pro->norm_weight, 16) ||
            (pro->delta && !aligned(pro->delta, 16)))
            return fail(NVFP4R_ERR_ALIGNMENT, "linear_packed_ex: prologue tensors need 16-byte alignment");
        g.delta = pro->delta; g.residual_in = pro->residual_in; g.residual_out = pro->residual_out;
        g.norm_w = pro->norm_weight; g.eps = pro->eps;
        g.xb = pro->residual_in; g.xb_stride = K;
    } else if (pro->kind == NVFP4R_PROLOGUE_NONE) {
        if (!x || !aligned(x, 16) || (x_row_stride % 8) || x_row_stride < static_cast<int64_t>(K))
            return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: x must be bf16 [M, K], 16-byte aligned rows");
        g.xb = x; g.xb_stride = x_row_stride;
    } else {
        if (!x || !aligned(x, 16) || (x_row_stride % 8) || x_row_stride < 2 * static_cast<int64_t>(K))
            return fail(NVFP4R_ERR_INVALID_ARGUMENT, "linear_packed_ex: SiLU prologue needs x = [M, 2K] gate|up, 16-byte aligned");
        g.xb = x; g.xb_stride = x_row_stride;
    }
    g.push = (pro->push_to != nullptr && pro->push_to->world > 1) ? pro->push_to : nullptr;
    g.push_gather = g.push != nullptr && pro->push_gather != 0;
    if (g.push_gather && M > 32)
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "linear_packed_ex: push_gather takes at most 32 rows (one launch)");
    const char* why = nullptr;
    cudaError_t e = nvfp4r::launch_linear_packed(g, as_stream(stream), &why);
    if (why != nullptr) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, why);
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "linear_packed_ex launch");
}

int nvfp4r_set_packed_tuning(int splits) {
    if (splits < 0 || (splits & 0xff) > 64 || splits >= (1 << 28)) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "packed tuning: splits 0..64");
    nvfp4r::set_packed_tuning(splits);
    return NVFP4R_OK;
}

int nvfp4r_set_gemm_tuning(int splits, int stages) {
    if (splits < 0 || splits > 16 || stages < 0 || stages > 10)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "gemm tuning: splits 0..16, stages 0..10");
    nvfp4r::set_tc_tuning(splits, stages);
    return NVFP4R_OK;
}

int nvfp4r_unswizzle_blockscale(const void* swizzled, void* flat, int rows, int K, void* stream) {
    NVFP4R_RANGE("nvfp4r_unswizzle_blockscale");
    if (!swizzled || !flat) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "unswizzle: null pointer");
    if (rows < 0 || K <= 0 || K % 16) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "unswizzle: K % 16");
    if (rows == 0) return NVFP4R_OK;
    cudaError_t e = nvfp4r::launch_sf_layout(swizzled, flat, rows, K, true, as_stream(stream));
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "unswizzle launch");
}

int nvfp4r_swizzle_blockscale(const void* flat, void* swizzled, int rows, int K, void* stream) {
    NVFP4R_RANGE("nvfp4r_swizzle_blockscale");
    if (!swizzled || !flat) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "swizzle: null pointer");
    if (rows < 0 || K <= 0 || K % 16) return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "swizzle: K % 16");
    if (rows == 0) return NVFP4R_OK;
    cudaError_t e = nvfp4r::launch_sf_layout(flat, swizzled, rows, K, false, as_stream(stream));
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "swizzle launch");
}

size_t nvfp4r_reset_workspace_bytes(int B) {
    return B > 0 ? static_cast<size_t>(B) * (sizeof(nvfp4r::RowScratch) + sizeof(nvfp4r::RowSlots)) : 0;
}

int nvfp4r_reset_step(float* logits, int64_t row_stride, int B, int V, nvfp4r_reset_state* states,
                      const int32_t* state_slots, const int32_t* last_ids,
                      const uint32_t* nl_bitmap, const uint32_t* dnl_bitmap,
                      const nvfp4r_reset_params* params, nvfp4r_reset_decision* decisions,
                      void* workspace, size_t workspace_bytes, void* stream) {
    NVFP4R_RANGE("nvfp4r_reset_step");
    if (!logits || !states || !params || !workspace)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "reset_step: null pointer");
    if (B < 0 || V <= 0 || row_stride < V) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "reset_step: bad sizes");
    if (params->window < 1 || params->window > NVFP4R_RESET_MAX_WINDOW)
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "reset_step: window outside 1..NVFP4R_RESET_MAX_WINDOW");
    if (workspace_bytes < nvfp4r_reset_workspace_bytes(B))
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "reset_step: workspace too small");
    if (!aligned(workspace, 8) || !aligned(logits, 4) || !aligned(states, 8))
        return fail(NVFP4R_ERR_ALIGNMENT, "reset_step: workspace/states need 8-byte alignment");
    if (B == 0) return NVFP4R_OK;
    nvfp4r::ResetLaunch p = {};
    p.logits = logits;
    p.row_stride = row_stride;
    p.B = B;
    p.V = V;
    p.scratch = static_cast<nvfp4r::RowScratch*>(workspace);
    p.slots = reinterpret_cast<nvfp4r::RowSlots*>(static_cast<nvfp4r::RowScratch*>(workspace) + B);
    p.states = states;
    p.state_slots = state_slots;
    p.last_ids = last_ids;
    p.nl_bitmap = nl_bitmap;
    p.dnl_bitmap = dnl_bitmap;
    p.params = *params;
    p.params.id_set = 0;
    p.decisions = decisions;
    p.entropy_out = nullptr;
    p.needs_state = 1;
    cudaError_t e = nvfp4r::launch_reset(p, true, as_stream(stream));
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "reset_step launch");
}

int nvfp4r_reset_step_per_request(float* logits, int64_t row_stride, int B, int V,
                                  nvfp4r_reset_state* states, const int32_t* state_slots,
                                  const int32_t* last_ids, const uint32_t* nl_bitmaps,
                                  const uint32_t* dnl_bitmaps, int n_id_sets,
                                  const nvfp4r_reset_params* slot_params,
                                  nvfp4r_reset_decision* decisions, void* workspace,
                                  size_t workspace_bytes, void* stream) {
    NVFP4R_RANGE("nvfp4r_reset_step_per_request");
    if (!logits || !states || !slot_params || !workspace)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "reset_step_per_request: null pointer");
    if (B < 0 || V <= 0 || row_stride < V || n_id_sets < 0)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "reset_step_per_request: bad sizes");
    if (workspace_bytes < nvfp4r_reset_workspace_bytes(B))
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "reset_step_per_request: workspace too small");
    if (!aligned(workspace, 8) || !aligned(logits, 4) || !aligned(states, 8) || !aligned(slot_params, 8))
        return fail(NVFP4R_ERR_ALIGNMENT, "reset_step_per_request: workspace/states/params need 8-byte alignment");
    if (B == 0) return NVFP4R_OK;
    nvfp4r::ResetLaunch p = {};
    p.logits = logits;
    p.row_stride = row_stride;
    p.B = B;
    p.V = V;
    p.scratch = static_cast<nvfp4r::RowScratch*>(workspace);
    p.slots = reinterpret_cast<nvfp4r::RowSlots*>(static_cast<nvfp4r::RowScratch*>(workspace) + B);
    p.states = states;
    p.state_slots = state_slots;
    p.last_ids = last_ids;
    p.nl_bitmap = n_id_sets > 0 ? nl_bitmaps : nullptr;
    p.dnl_bitmap = n_id_sets > 0 ? dnl_bitmaps : nullptr;
    p.slot_params = slot_params;
    p.bitmap_words = (V + 31) / 32;
    p.decisions = decisions;
    p.entropy_out = nullptr;
    p.needs_state = 1;
    cudaError_t e = nvfp4r::launch_reset(p, true, as_stream(stream));
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "reset_step_per_request launch");
}

size_t nvfp4r_lm_head_reset_workspace_bytes(void) { return nvfp4r::lm_head_reset_workspace_bytes(); }

int nvfp4r_lm_head_reset_step(const void* x, const void* weight, float* logits, int V, int H,
                              nvfp4r_reset_state* states, const int32_t* state_slots,
                              const int32_t* last_ids, const uint32_t* nl_bitmaps,
                              const uint32_t* dnl_bitmaps, int n_id_sets,
                              const nvfp4r_reset_params* slot_params,
                              nvfp4r_reset_decision* decisions, void* workspace,
                              size_t workspace_bytes, void* stream) {
    NVFP4R_RANGE("nvfp4r_lm_head_reset_step");
    if (!x || !weight || !logits || !states || !slot_params || !workspace)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "lm_head_reset_step: null pointer");
    if (V <= 0 || H <= 0 || n_id_sets < 0)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "lm_head_reset_step: bad sizes");
    if (H % 256 != 0 || H > 12288)
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "lm_head_reset_step: H must be a multiple of 256, at most 12288");
    if (workspace_bytes < nvfp4r::lm_head_reset_workspace_bytes())
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "lm_head_reset_step: workspace too small");
    if (!aligned(workspace, 8) || !aligned(logits, 4) || !aligned(states, 8) || !aligned(slot_params, 8) ||
        !aligned(x, 2) || !aligned(weight, 16))
        return fail(NVFP4R_ERR_ALIGNMENT, "lm_head_reset_step: weight needs 16-byte, workspace/states/params 8-byte alignment");
    nvfp4r::ResetLaunch p = {};
    p.logits = logits;
    p.row_stride = V;
    p.B = 1;
    p.V = V;
    p.states = states;
    p.state_slots = state_slots;
    p.last_ids = last_ids;
    p.nl_bitmap = n_id_sets > 0 ? nl_bitmaps : nullptr;
    p.dnl_bitmap = n_id_sets > 0 ? dnl_bitmaps : nullptr;
    p.slot_params = slot_params;
    p.bitmap_words = (V + 31) / 32;
    p.decisions = decisions;
    p.needs_state = 1;
    cudaError_t e = nvfp4r::launch_lm_head_reset(x, weight, H, p, workspace, as_stream(stream));
    if (e == cudaErrorInvalidConfiguration)
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE,
                    "lm_head_reset_step: vocabulary too large for one resident grid; use nvfp4r_lm_head "
                    "followed by nvfp4r_reset_step_per_request");
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "lm_head_reset_step launch");
}

int nvfp4r_reset_step_static(float* logits, int64_t row_stride, int B, int V,
                             nvfp4r_reset_state* states, const int32_t* state_slots,
                             const int32_t* last_ids, const uint32_t* nl_bitmap,
                             const uint32_t* dnl_bitmap, const nvfp4r_reset_params* params,
                             nvfp4r_reset_decision* decisions, void* stream) {
    NVFP4R_RANGE("nvfp4r_reset_step_static");
    if (!logits || !states || !params)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "reset_step_static: null pointer");
    if (B < 0 || V <= 0 || row_stride < V)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "reset_step_static: bad sizes");
    if (B > NVFP4R_RESET_STATIC_MAX_ROWS)
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE,
                    "reset_step_static: more rows than NVFP4R_RESET_STATIC_MAX_ROWS; use "
                    "nvfp4r_reset_step with a workspace");
    if (params->window < 1 || params->window > NVFP4R_RESET_MAX_WINDOW)
        return fail(NVFP4R_ERR_UNSUPPORTED_SHAPE, "reset_step_static: window outside 1..NVFP4R_RESET_MAX_WINDOW");
    if (!aligned(logits, 4) || !aligned(states, 8))
        return fail(NVFP4R_ERR_ALIGNMENT, "reset_step_static: states need 8-byte alignment");
    if (B == 0) return NVFP4R_OK;
    nvfp4r::ResetLaunch p = {};
    p.logits = logits;
    p.row_stride = row_stride;
    p.B = B;
    p.V = V;
    p.states = states;
    p.state_slots = state_slots;
    p.last_ids = last_ids;
    p.nl_bitmap = nl_bitmap;
    p.dnl_bitmap = dnl_bitmap;
    p.params = *params;
    p.params.id_set = 0;
    p.decisions = decisions;
    p.entropy_out = nullptr;
    p.needs_state = 1;
    cudaError_t e = nvfp4r::launch_reset_static(p, as_stream(stream));
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "reset_step_static launch");
}

int nvfp4r_entropy(const float* logits, int64_t row_stride, int B, int V, float* entropy,
                   void* workspace, size_t workspace_bytes, void* stream) {
    NVFP4R_RANGE("nvfp4r_entropy");
    if (!logits || !entropy || !workspace) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "entropy: null pointer");
    if (B < 0 || V <= 0 || row_stride < V) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "entropy: bad sizes");
    if (workspace_bytes < nvfp4r_reset_workspace_bytes(B))
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "entropy: workspace too small");
    if (!aligned(workspace, 8) || !aligned(logits, 4))
        return fail(NVFP4R_ERR_ALIGNMENT, "entropy: workspace needs 8-byte alignment");
    if (B == 0) return NVFP4R_OK;
    nvfp4r::ResetLaunch p = {};
    p.logits = logits;
    p.row_stride = row_stride;
    p.B = B;
    p.V = V;
    p.scratch = static_cast<nvfp4r::RowScratch*>(workspace);
    p.slots = reinterpret_cast<nvfp4r::RowSlots*>(static_cast<nvfp4r::RowScratch*>(workspace) + B);
    p.entropy_out = entropy;
    p.needs_state = 0;
    cudaError_t e = nvfp4r::launch_reset(p, false, as_stream(stream));
    return e == cudaSuccess ? NVFP4R_OK : cuda_fail(e, "entropy launch");
}

int nvfp4r_set_gemv_tuning(int ctas_per_sm, int use_pdl, int force_generic) {
    nvfp4r::GemvTuning& t = nvfp4r::gemv_tuning();
    if (ctas_per_sm > 8) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "tuning: ctas_per_sm > 8");
    if (ctas_per_sm >= 0) t.ctas_per_sm = ctas_per_sm;      // 0 = automatic
    if (use_pdl >= 0) t.use_pdl = use_pdl ? 1 : 0;
    if (force_generic >= 0) t.force_generic = force_generic ? 1 : 0;
    return NVFP4R_OK;
}

int nvfp4r_set_gemv_rows_tuning(int mode, int rows_per_step, int warps_per_sm) {
    if (mode < -1 || mode > 1) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "rows tuning: mode is -1, 0 or 1");
    if (rows_per_step != 0 && rows_per_step != 2 && rows_per_step != 4)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "rows tuning: rows_per_step is 0, 2 or 4");
    if (warps_per_sm < 0 || warps_per_sm > 32)
        return fail(NVFP4R_ERR_INVALID_ARGUMENT, "rows tuning: warps_per_sm 0..32");
    nvfp4r::set_gemv_rows_tuning(mode, rows_per_step, warps_per_sm);
    return NVFP4R_OK;
}

int nvfp4r_status_mirror(volatile int** host_word) {
    if (!host_word) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "status_mirror: null pointer");
    static int* host_ptr[64] = {};
    static std::mutex mu;                       // two threads may make the first call at once
    std::lock_guard<std::mutex> lock(mu);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "status_mirror");
    if (dev < 0 || dev >= 64) return fail(NVFP4R_ERR_INVALID_ARGUMENT, "status_mirror: device index");
    if (host_ptr[dev] == nullptr) {
        int* h = nullptr;
        int* d = nullptr;
        e = cudaHostAlloc(reinterpret_cast<void**>(&h), sizeof(int), cudaHostAllocMapped);
        if (e != cudaSuccess) return cuda_fail(e, "status_mirror: cudaHostAlloc");
        *h = 0;
        e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), h, 0);
        if (e == cudaSuccess) e = nvfp4r::set_status_mirror_gemv(d);
        if (e == cudaSuccess) e = nvfp4r::set_status_mirror_tc(d);
        if (e == cudaSuccess) e = nvfp4r::set_status_mirror_packed(d);
        if (e == cudaSuccess) e = nvfp4r::set_status_mirror_peer(d);
        if (e == cudaSuccess) e = nvfp4r::set_status_mirror_reset(d);
        if (e == cudaSuccess) e = nvfp4r::set_status_mirror_head(d);
        if (e != cudaSuccess) { cudaFreeHost(h); return cuda_fail(e, "status_mirror: set-up"); }
        host_ptr[dev] = h;
    }
    *host_word = host_ptr[dev];
    return NVFP4R_OK;
}

int nvfp4r_check_device_status(void) {
    int flag = 0, flag2 = 0;
    cudaError_t e = nvfp4r::read_and_clear_device_status(&flag);
    int flag3 = 0;
    if (e == cudaSuccess) e = nvfp4r::read_and_clear_tc_status(&flag2);
    if (e == cudaSuccess) e = nvfp4r::read_and_clear_packed_status(&flag3);
    int flag4 = 0, flag5 = 0;
    if (e == cudaSuccess) e = nvfp4r::read_and_clear_peer_status(&flag4);
    if (e == cudaSuccess) e = nvfp4r::read_and_clear_reset_status(&flag5);
    int flag6 = 0;
    if (e == cudaSuccess) e = nvfp4r::read_and_clear_head_status(&flag6);
    flag4 |= flag5 | flag6;
    if (e != cudaSuccess) return cuda_fail(e, "device status");
    flag |= flag2 | flag3 | flag4;
    return flag ? fail(NVFP4R_ERR_DEVICE_TIMEOUT, "a bounded device-side wait gave up") : NVFP4R_OK;
}

}  // extern "C"
