// PyTorch operator registration for the nvfp4r surface. Host C++ only: every op
// validates its tensors, then calls the C ABI of include/nvfp4r_b200.h with raw
// device pointers and the current CUDA stream.
//
// Schemas of `gemv` and `gemm` are those of the reference
// (kernels/csrc/bindings.cpp:108-121): out-variants that mutate their last tensor
// and return nothing. `quant`, `linear`, `reset_step` and `entropy` are additions
// that replace multi-op sequences of the reference with one dispatch each.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <c10/cuda/CUDAGraphsC10Utils.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "nvfp4r_b200.h"

namespace {

inline bool is_code_dtype(at::ScalarType t) {
    return t == at::kByte || t == at::kFloat4_e2m1fn_x2;
}
inline bool is_scale_dtype(at::ScalarType t) { return t == at::kByte || t == at::kFloat8_e4m3fn; }

inline int dtype_code(at::ScalarType t, const char* who) {
    if (t == at::kBFloat16) return NVFP4R_BF16;
    if (t == at::kHalf) return NVFP4R_F16;
    if (t == at::kFloat) return NVFP4R_F32;
    TORCH_CHECK(false, who, ": out must be float16, bfloat16 or float32");
    return -1;
}

inline void check_status(int st, const char* who) {
    TORCH_CHECK(st == NVFP4R_OK, who, ": ", nvfp4r_status_string(st), " (", st, "): ", nvfp4r_last_error());
}

inline void* current_stream() { return static_cast<void*>(at::cuda::getCurrentCUDAStream().stream()); }

// torch.ops.nvfp4r.gemv - same checks and messages as kernels/csrc/bindings.cpp:27-84.
void gemv_op(const at::Tensor& weight, const at::Tensor& weight_scale, const at::Tensor& x,
             const at::Tensor& x_scale, at::Tensor out, double alpha) {
    TORCH_CHECK(weight.is_cuda() && weight_scale.is_cuda() && x.is_cuda() && x_scale.is_cuda(),
                "gemv: all inputs must be CUDA");
    TORCH_CHECK(is_code_dtype(weight.scalar_type()), "gemv: weight must be uint8 / fp4_e2m1fn_x2");
    TORCH_CHECK(is_scale_dtype(weight_scale.scalar_type()),
                "gemv: weight_scale must be uint8 / float8_e4m3fn");
    TORCH_CHECK(is_code_dtype(x.scalar_type()), "gemv: x must be uint8 / fp4_e2m1fn_x2");
    TORCH_CHECK(is_scale_dtype(x_scale.scalar_type()), "gemv: x_scale must be uint8 / float8_e4m3fn");
    TORCH_CHECK(weight.dim() == 3 && weight_scale.dim() == 3 && x.dim() == 3 && x_scale.dim() == 3,
                "gemv: inputs must be 3D [L, M_or_N, K/2_or_K/16]");
    TORCH_CHECK(x.is_contiguous() && x_scale.is_contiguous(), "gemv: x / x_scale must be contiguous");
    const int64_t L = weight.size(0), N = weight.size(1), K2 = weight.size(2), K = 2 * K2;
    TORCH_CHECK(weight_scale.size(0) == L && weight_scale.size(1) == N && weight_scale.size(2) * 16 == K,
                "weight_scale shape mismatch with weight");
    TORCH_CHECK(x.size(0) == L && x.size(2) == K2, "x.K mismatch with weight.K");
    TORCH_CHECK(x_scale.size(0) == L && x_scale.size(1) == x.size(1) && x_scale.size(2) * 16 == K,
                "x_scale shape mismatch with x");
    TORCH_CHECK(out.is_cuda() && out.is_contiguous(), "out must be CUDA contiguous");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == L && out.size(1) == N, "out must be [L, M]");
    TORCH_CHECK(weight.stride(2) == 1 && weight_scale.stride(2) == 1,
                "gemv: weight / weight_scale must have unit inner stride");
    const int dt = dtype_code(out.scalar_type(), "gemv");
    const c10::cuda::OptionalCUDAGuard guard(weight.device());
    const int st = nvfp4r_gemv(weight.data_ptr(), weight_scale.data_ptr(), x.data_ptr(),
                               x_scale.data_ptr(), out.data_ptr(), static_cast<int>(L),
                               static_cast<int>(N), static_cast<int>(K), weight.stride(0),
                               weight.stride(1), weight_scale.stride(0), weight_scale.stride(1),
                               x.stride(0), x_scale.stride(0), static_cast<float>(alpha), dt,
                               current_stream());
    check_status(st, "gemv");
}

// Hidden scratch of the operators whose schema (the reference's) has no workspace argument:
// ONE zero-initialised buffer per device and per kernel family, allocated at the first call on
// that device with a fixed size and never replaced, so that a pointer recorded in a CUDA graph
// stays valid for the life of the process. A call that needs more than the fixed size raises
// (set NVFP4R_WORKSPACE_MB before the first call to change it); a first call inside a stream
// capture raises too, because memory allocated there belongs to the capturing graph.
// kind 0: tickets + fp32 split-K partials of `gemm` / `linear_tc` (the kernel leaves the
// tickets zeroed); kind 1: the split-K slots of `linear_packed` (all zero between launches).
// The two never share memory.
size_t workspace_capacity() {
    static const size_t cap = [] {
        const char* env = std::getenv("NVFP4R_WORKSPACE_MB");
        long mb = env ? std::atol(env) : 128;
        if (mb < 1) mb = 1;
        return static_cast<size_t>(mb) << 20;
    }();
    return cap;
}

at::Tensor& fixed_workspace(int kind, const at::Device& dev, size_t bytes, const char* who) {
    static std::mutex mu;
    static std::unordered_map<int, at::Tensor> cache[2];
    std::lock_guard<std::mutex> lock(mu);
    at::Tensor& t = cache[kind][dev.index()];
    if (!t.defined()) {
        TORCH_CHECK(c10::cuda::currentStreamCaptureStatusMayInitCtx() == c10::cuda::CaptureStatus::None, who,
                    ": the first call on a device allocates the operator's scratch; make it before "
                    "capturing a CUDA graph");
        t = at::zeros({static_cast<int64_t>(workspace_capacity())},
                      at::TensorOptions().device(dev).dtype(at::kByte));
    }
    TORCH_CHECK(bytes <= static_cast<size_t>(t.nbytes()), who, ": this shape needs ", bytes,
                " bytes of split-K scratch, the fixed buffer holds ", t.nbytes(),
                "; set NVFP4R_WORKSPACE_MB before the first call");
    return t;
}

// torch.ops.nvfp4r.gemm - kernels/csrc/bindings.cpp:86-103. A [M,K/2] activations,
// B [N,K/2] weights, SFA/SFB swizzled scales, C [M,N] buffer that receives the
// result N-major (viewed as [N,M]), as the reference kernel writes it.
void gemm_op(const at::Tensor& A, const at::Tensor& B, const at::Tensor& SFA, const at::Tensor& SFB,
             at::Tensor C, double alpha) {
    TORCH_CHECK(A.is_cuda() && B.is_cuda() && SFA.is_cuda() && SFB.is_cuda() && C.is_cuda(),
                "gemm: all tensors must be CUDA");
    TORCH_CHECK(is_code_dtype(A.scalar_type()) && is_code_dtype(B.scalar_type()),
                "gemm: A/B must be uint8 (FP4 packed) or fp4_e2m1fn_x2");
    TORCH_CHECK(is_scale_dtype(SFA.scalar_type()) && is_scale_dtype(SFB.scalar_type()),
                "gemm: SFA/SFB must be uint8 or float8_e4m3fn");
    TORCH_CHECK(C.scalar_type() == at::kHalf || C.scalar_type() == at::kBFloat16,
                "gemm: C must be float16 or bfloat16");
    TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && C.dim() == 2 && A.is_contiguous() &&
                    B.is_contiguous() && C.is_contiguous() && SFA.is_contiguous() && SFB.is_contiguous(),
                "gemm: A [M,K/2], B [N,K/2], C [M,N] must be contiguous 2-D tensors");
    const int64_t M = A.size(0), K2 = A.size(1), N = B.size(0);
    TORCH_CHECK(B.size(1) == K2 && C.size(0) == M && C.size(1) == N, "gemm: shape mismatch");
    const c10::cuda::OptionalCUDAGuard guard(A.device());
    at::Tensor& ws = fixed_workspace(0, A.device(),
                                     nvfp4r_gemm_workspace_bytes(static_cast<int>(M), static_cast<int>(N),
                                                                 static_cast<int>(2 * K2)), "gemm");
    const int st = nvfp4r_gemm(A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), C.data_ptr(),
                               static_cast<int>(M), static_cast<int>(N), static_cast<int>(2 * K2),
                               static_cast<float>(alpha), dtype_code(C.scalar_type(), "gemm"),
                               /*c_layout=*/NVFP4R_C_N_MAJOR, ws.data_ptr(),
                               static_cast<size_t>(ws.nbytes()), current_stream());
    check_status(st, "gemm");
}

std::tuple<at::Tensor, at::Tensor> quant_op(const at::Tensor& x, const at::Tensor& global_scale_inv,
                                            bool swizzled, int64_t rcp_mode) {
    TORCH_CHECK(x.is_cuda() && global_scale_inv.is_cuda(), "quant: tensors must be CUDA");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1,
                "quant: x must be bfloat16 [M,K] with unit inner stride");
    TORCH_CHECK(global_scale_inv.scalar_type() == at::kFloat && global_scale_inv.numel() >= 1,
                "quant: global_scale_inv must be a float32 tensor");
    const int64_t M = x.size(0), K = x.size(1);
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    auto codes = at::empty({M, K / 2}, x.options().dtype(at::kByte));
    const int64_t rows = swizzled ? (M + 127) / 128 * 128 : M;
    const int64_t cols = swizzled ? (K / 16 + 3) / 4 * 4 : K / 16;
    auto scales = at::empty({rows, cols}, x.options().dtype(at::kByte));
    const int st = nvfp4r_quant(x.data_ptr(), x.stride(0), static_cast<int>(M), static_cast<int>(K),
                                global_scale_inv.data_ptr<float>(), codes.data_ptr(), scales.data_ptr(),
                                swizzled ? NVFP4R_SF_SWIZZLED : NVFP4R_SF_FLAT,
                                static_cast<int>(rcp_mode), current_stream());
    check_status(st, "quant");
    return {codes, scales};
}

// Decode branch of the reference's `_nvfp4r_linear_impl`
// (kernels/python/nvfp4r/vllm_integration.py:211-222) as one op.
at::Tensor linear_op(const at::Tensor& x, const at::Tensor& global_scale_inv, const at::Tensor& weight,
                     const at::Tensor& weight_scale_flat, double alpha, int64_t out_dtype_int,
                     int64_t rcp_mode) {
    TORCH_CHECK(x.is_cuda() && weight.is_cuda() && weight_scale_flat.is_cuda() &&
                    global_scale_inv.is_cuda(), "linear: tensors must be CUDA");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1,
                "linear: x must be bfloat16 [M,K] with unit inner stride");
    TORCH_CHECK(weight.dim() == 2 && weight.is_contiguous() && weight_scale_flat.is_contiguous(),
                "linear: weight [N,K/2] and weight_scale [N,K/16] must be contiguous");
    const int64_t M = x.size(0), K = x.size(1), N = weight.size(0);
    TORCH_CHECK(weight.size(1) * 2 == K && weight_scale_flat.numel() == N * (K / 16),
                "linear: weight / weight_scale shape mismatch with x");
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    const auto dt = out_dtype_int == 0 ? at::kBFloat16 : out_dtype_int == 1 ? at::kHalf : at::kFloat;
    auto out = at::empty({M, N}, x.options().dtype(dt));
    const int st = nvfp4r_linear(x.data_ptr(), x.stride(0), static_cast<int>(M), static_cast<int>(K),
                                 global_scale_inv.data_ptr<float>(), weight.data_ptr(),
                                 weight_scale_flat.data_ptr(), static_cast<int>(N),
                                 static_cast<float>(alpha), out.data_ptr(),
                                 static_cast<int>(out_dtype_int), static_cast<int>(rcp_mode),
                                 current_stream());
    check_status(st, "linear");
    return out;
}

// Padded-GEMM branch of the reference's `_nvfp4r_linear_impl`
// (vllm_integration.py:224-274) as one op: on-chip quantizer + tcgen05 GEMM, [M,N] out.
at::Tensor linear_tc_op(const at::Tensor& x, const at::Tensor& global_scale_inv, const at::Tensor& weight,
                        const at::Tensor& weight_scale_swizzled, double alpha, int64_t out_dtype_int,
                        int64_t rcp_mode) {
    TORCH_CHECK(x.is_cuda() && weight.is_cuda() && weight_scale_swizzled.is_cuda() &&
                    global_scale_inv.is_cuda(), "linear_tc: tensors must be CUDA");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1,
                "linear_tc: x must be bfloat16 [M,K] with unit inner stride");
    TORCH_CHECK(weight.dim() == 2 && weight.is_contiguous() && weight_scale_swizzled.is_contiguous(),
                "linear_tc: weight [N,K/2] and its swizzled scales must be contiguous");
    const int64_t M = x.size(0), K = x.size(1), N = weight.size(0);
    TORCH_CHECK(weight.size(1) * 2 == K, "linear_tc: weight shape mismatch with x");
    TORCH_CHECK(weight_scale_swizzled.numel() >= ((N + 127) / 128 * 128) * ((K / 16 + 3) / 4 * 4),
                "linear_tc: swizzled weight_scale too small");
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    const auto dt = out_dtype_int == 0 ? at::kBFloat16 : out_dtype_int == 1 ? at::kHalf : at::kFloat;
    auto out = at::empty({M, N}, x.options().dtype(dt));
    at::Tensor& ws = fixed_workspace(0, x.device(),
                                     nvfp4r_gemm_workspace_bytes(static_cast<int>(M), static_cast<int>(N),
                                                                 static_cast<int>(K)), "linear_tc");
    const int st = nvfp4r_linear_tc(x.data_ptr(), x.stride(0), static_cast<int>(M), static_cast<int>(K),
                                    global_scale_inv.data_ptr<float>(), weight.data_ptr(),
                                    weight_scale_swizzled.data_ptr(), static_cast<int>(N),
                                    static_cast<float>(alpha), out.data_ptr(),
                                    static_cast<int>(out_dtype_int), static_cast<int>(rcp_mode),
                                    ws.data_ptr(), static_cast<size_t>(ws.nbytes()), current_stream());
    check_status(st, "linear_tc");
    return out;
}

// One-time re-layout of a weight into the packed block format (18 KB per 128 x 256 block).
at::Tensor pack_weight_op(const at::Tensor& weight, const at::Tensor& weight_scale_flat) {
    TORCH_CHECK(weight.is_cuda() && weight_scale_flat.is_cuda(), "pack_weight: tensors must be CUDA");
    TORCH_CHECK(weight.dim() == 2 && weight.is_contiguous() && weight_scale_flat.is_contiguous(),
                "pack_weight: weight [N,K/2] and flat weight_scale [N,K/16] must be contiguous");
    const int64_t N = weight.size(0), K = weight.size(1) * 2;
    TORCH_CHECK(weight_scale_flat.numel() == N * (K / 16), "pack_weight: weight_scale shape mismatch");
    const size_t bytes = nvfp4r_packed_weight_bytes(static_cast<int>(N), static_cast<int>(K));
    TORCH_CHECK(bytes > 0, "pack_weight: needs N % 128 == 0 and K % 128 == 0");
    const c10::cuda::OptionalCUDAGuard guard(weight.device());
    auto packed = at::empty({static_cast<int64_t>(bytes)}, weight.options().dtype(at::kByte));
    check_status(nvfp4r_pack_weight(weight.data_ptr(), weight_scale_flat.data_ptr(), packed.data_ptr(),
                                    static_cast<int>(N), static_cast<int>(K), current_stream()),
                 "pack_weight");
    return packed;
}

// The adapter's product path: on-chip quantizer + tensor-core linear over a packed weight.
at::Tensor linear_packed_op(const at::Tensor& x, const at::Tensor& global_scale_inv,
                            const at::Tensor& packed, int64_t N, double alpha, int64_t out_dtype_int,
                            int64_t rcp_mode) {
    TORCH_CHECK(x.is_cuda() && packed.is_cuda() && global_scale_inv.is_cuda(),
                "linear_packed: tensors must be CUDA");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1,
                "linear_packed: x must be bfloat16 [M,K] with unit inner stride");
    const int64_t M = x.size(0), K = x.size(1);
    TORCH_CHECK(packed.is_contiguous() &&
                    static_cast<size_t>(packed.nbytes()) ==
                        nvfp4r_packed_weight_bytes(static_cast<int>(N), static_cast<int>(K)),
                "linear_packed: packed weight does not match N and K");
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    const auto dt = out_dtype_int == 0 ? at::kBFloat16 : out_dtype_int == 1 ? at::kHalf : at::kFloat;
    auto out = at::empty({M, N}, x.options().dtype(dt));
    at::Tensor& ws = fixed_workspace(1, x.device(),
                                     nvfp4r_linear_packed_workspace_bytes(static_cast<int>(M), static_cast<int>(N),
                                                                          static_cast<int>(K)), "linear_packed");
    const int st = nvfp4r_linear_packed(x.data_ptr(), x.stride(0), static_cast<int>(M), static_cast<int>(K),
                                        global_scale_inv.data_ptr<float>(), packed.data_ptr(),
                                        static_cast<int>(N), static_cast<float>(alpha), out.data_ptr(),
                                        static_cast<int>(out_dtype_int), static_cast<int>(rcp_mode),
                                        ws.data_ptr(), static_cast<size_t>(ws.nbytes()), current_stream());
    check_status(st, "linear_packed");
    return out;
}

at::Tensor entropy_op(const at::Tensor& logits, at::Tensor workspace) {
    TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 &&
                    logits.stride(1) == 1, "entropy: logits must be CUDA float32 [B,V]");
    const c10::cuda::OptionalCUDAGuard guard(logits.device());
    auto out = at::empty({logits.size(0)}, logits.options());
    const int st = nvfp4r_entropy(logits.data_ptr<float>(), logits.stride(0),
                                  static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                                  out.data_ptr<float>(), workspace.data_ptr(),
                                  static_cast<size_t>(workspace.nbytes()), current_stream());
    check_status(st, "entropy");
    return out;
}

// One ReSET step in place. `states`, `decisions`, `workspace` are byte tensors laid
// out as the C structs of the header; optional tensors may be undefined (None).
void reset_step_op(at::Tensor logits, at::Tensor states, const c10::optional<at::Tensor>& state_slots,
                   const c10::optional<at::Tensor>& last_ids, const c10::optional<at::Tensor>& nl_bitmap,
                   const c10::optional<at::Tensor>& dnl_bitmap, double t_high, double t_low, double tau0,
                   int64_t window, const c10::optional<at::Tensor>& decisions, at::Tensor workspace) {
    TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 &&
                    logits.stride(1) == 1, "reset_step: logits must be CUDA float32 [B,V]");
    const c10::cuda::OptionalCUDAGuard guard(logits.device());
    auto ptr = [](const c10::optional<at::Tensor>& t) -> void* {
        return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr;
    };
    nvfp4r_reset_params prm{t_high, t_low, tau0, static_cast<int32_t>(window), 0};
    const int st = nvfp4r_reset_step(
        logits.data_ptr<float>(), logits.stride(0), static_cast<int>(logits.size(0)),
        static_cast<int>(logits.size(1)), static_cast<nvfp4r_reset_state*>(states.data_ptr()),
        static_cast<const int32_t*>(ptr(state_slots)), static_cast<const int32_t*>(ptr(last_ids)),
        static_cast<const uint32_t*>(ptr(nl_bitmap)), static_cast<const uint32_t*>(ptr(dnl_bitmap)), &prm,
        static_cast<nvfp4r_reset_decision*>(ptr(decisions)), workspace.data_ptr(),
        static_cast<size_t>(workspace.nbytes()), current_stream());
    check_status(st, "reset_step");
}

}  // namespace

TORCH_LIBRARY(nvfp4r, m) {
    m.def("gemv(Tensor weight, Tensor weight_scale, Tensor x, Tensor x_scale, "
          "Tensor(a!) out, float alpha=1.0) -> ()");
    m.def("gemm(Tensor A, Tensor B, Tensor SFA, Tensor SFB, Tensor(a!) C, float alpha=1.0) -> ()");
    m.def("quant(Tensor x, Tensor global_scale_inv, bool swizzled=False, int rcp_mode=1) -> (Tensor, Tensor)");
    m.def("linear(Tensor x, Tensor global_scale_inv, Tensor weight, Tensor weight_scale_flat, "
          "float alpha, int out_dtype_int=0, int rcp_mode=1) -> Tensor");
    m.def("linear_tc(Tensor x, Tensor global_scale_inv, Tensor weight, Tensor weight_scale_swizzled, "
          "float alpha, int out_dtype_int=0, int rcp_mode=1) -> Tensor");
    m.def("pack_weight(Tensor weight, Tensor weight_scale_flat) -> Tensor");
    m.def("linear_packed(Tensor x, Tensor global_scale_inv, Tensor packed, int N, float alpha, "
          "int out_dtype_int=0, int rcp_mode=1) -> Tensor");
    m.def("entropy(Tensor logits, Tensor workspace) -> Tensor");
    m.def("reset_step(Tensor(a!) logits, Tensor(b!) states, Tensor? state_slots, Tensor? last_ids, "
          "Tensor? nl_bitmap, Tensor? dnl_bitmap, float t_high, float t_low, float tau0, int window, "
          "Tensor(c!)? decisions, Tensor(d!) workspace) -> ()");
}

TORCH_LIBRARY_IMPL(nvfp4r, CUDA, m) {
    m.impl("gemv", &gemv_op);
    m.impl("gemm", &gemm_op);
    m.impl("quant", &quant_op);
    m.impl("linear", &linear_op);
    m.impl("linear_tc", &linear_tc_op);
    m.impl("pack_weight", &pack_weight_op);
    m.impl("linear_packed", &linear_packed_op);
    m.impl("entropy", &entropy_op);
    m.impl("reset_step", &reset_step_op);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "nvfp4r B200 kernels (registered under torch.ops.nvfp4r)";
}
