/*
 * nvfp4r_b200 - C ABI of the B200 (sm_100a) NVFP4 W4A4 decode path.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless a
 * comment says otherwise. Nothing here allocates, frees or synchronises: all
 * buffers are caller-owned for the duration of the (stream-ordered) call and
 * every entry point is safe to call during CUDA-graph capture unless stated
 * otherwise. `stream` is a cudaStream_t passed as void* (NULL = legacy default
 * stream). Every function returns NVFP4R_OK (0) or a negative nvfp4r_status.
 *
 * Each declaration names the interface of the reference (aiha-lab/ReSET) that
 * it stands in for, as <path within the reference>:<lines>.
 *
 * Data formats
 *   codes   : uint8, two e2m1 values per byte, even K element in the low nibble
 *             (kernels/tests/conftest.py:11-15,35-38)
 *   scales  : uint8 holding e4m3fn, one per 16 consecutive K elements, either
 *             "flat" row-major [rows, K/16] or "swizzled" 128x4 tiles
 *             [ceil(rows/128), ceil(K/64), 32, 4, 4]
 *             (kernels/python/nvfp4r/vllm_integration.py:25-31,99-117)
 *   out     : NVFP4R_BF16 / NVFP4R_F16 / NVFP4R_F32, row-major
 */
#ifndef NVFP4R_B200_H_
#define NVFP4R_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define NVFP4R_API __attribute__((visibility("default")))
#else
#define NVFP4R_API
#endif

typedef enum nvfp4r_status {
    NVFP4R_OK = 0,
    NVFP4R_ERR_INVALID_ARGUMENT = -1,  /* null pointer, non-positive size, bad enum   */
    NVFP4R_ERR_UNSUPPORTED_SHAPE = -2, /* divisibility / size limits of this build    */
    NVFP4R_ERR_ALIGNMENT = -3,         /* pointer or stride not aligned as required   */
    NVFP4R_ERR_CUDA = -4,              /* a CUDA runtime call failed; see last_error  */
    NVFP4R_ERR_DEVICE_TIMEOUT = -5     /* a bounded device-side wait gave up          */
} nvfp4r_status;

/* Output element type. 0/1 follow the reference adapter's `out_dtype_int`
 * (kernels/python/nvfp4r/vllm_integration.py:203-205): 0 = bf16, 1 = fp16.     */
typedef enum nvfp4r_dtype { NVFP4R_BF16 = 0, NVFP4R_F16 = 1, NVFP4R_F32 = 2 } nvfp4r_dtype;

typedef enum nvfp4r_sf_layout { NVFP4R_SF_FLAT = 0, NVFP4R_SF_SWIZZLED = 1 } nvfp4r_sf_layout;

/* Reciprocal used by the quantizer for 1/(sf * (1/gs_inv)).
 *   EXACT  : IEEE division; bit-exact against the CPU oracle.
 *   APPROX : rcp.approx.ftz, the arithmetic of the CUDA op the reference calls.   */
typedef enum nvfp4r_rcp_mode { NVFP4R_RCP_EXACT = 0, NVFP4R_RCP_APPROX = 1 } nvfp4r_rcp_mode;

/* Human-readable text for a status code (host pointer, static storage). */
NVFP4R_API const char* nvfp4r_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library. */
NVFP4R_API const char* nvfp4r_last_error(void);
/* Library version, 1000*major + minor. */
NVFP4R_API int nvfp4r_version(void);

/* ------------------------------------------------------------------------- *
 * Activation quantizer: bf16 [M,K] -> e2m1 codes [M,K/2] + e4m3 scales.
 * Stands in for `vops.scaled_fp4_quant(x_2d, input_global_scale_inv,
 * is_sf_swizzled_layout=...)` as called by the reference at
 * kernels/python/nvfp4r/vllm_integration.py:213 (flat) and :248,278 (swizzled).
 *   x              bf16, row stride `x_row_stride` elements, rows 16-byte aligned
 *   global_scale_inv  one float on the device (the layer's input_global_scale_inv)
 *   codes          [M, K/2] contiguous
 *   scales         flat: [M, K/16]; swizzled: [ceil(M/128)*128, ceil(K/64)*4],
 *                  padding written as 0
 * K % 16 == 0.
 * ------------------------------------------------------------------------- */
NVFP4R_API int nvfp4r_quant(const void* x, int64_t x_row_stride, int M, int K,
                            const float* global_scale_inv, void* codes, void* scales,
                            int sf_layout, int rcp_mode, void* stream);

/* ------------------------------------------------------------------------- *
 * Small-M GEMV on pre-quantized operands:
 *   out[l, n] = alpha * sum_k dq(weight[l, n, k]) * dq(x[l, 0, k])
 * Stands in for `torch.ops.nvfp4r.gemv(weight, weight_scale, x, x_scale, out,
 * alpha)` - kernels/csrc/bindings.cpp:27-84 and kernels/cuda/gemv/gemv_nvfp4.cu:
 * 817-1006 - with the same tensor meaning: weight [L,N,K/2], weight_scale
 * [L,N,K/16] (flat), x [L,P,K/2] and x_scale [L,P,K/16] of which only row 0 of
 * the P axis is read, out [L,N] contiguous. Strides are in bytes for the uint8
 * operands. `w_stride_l == 0` (and `wsf_stride_l == 0`) means one weight
 * broadcast over the L decode tokens (Tensor.expand), the decode case: the
 * weight is then streamed from HBM once for all L tokens. K % 32 == 0.
 * ------------------------------------------------------------------------- */
NVFP4R_API int nvfp4r_gemv(const void* weight, const void* weight_scale,
                           const void* x, const void* x_scale, void* out,
                           int L, int N, int K,
                           int64_t w_stride_l, int64_t w_stride_n,
                           int64_t wsf_stride_l, int64_t wsf_stride_n,
                           int64_t x_stride_l, int64_t xsf_stride_l,
                           float alpha, int out_dtype, void* stream);

/* ------------------------------------------------------------------------- *
 * Fused decode linear: quantize M <= NVFP4R_LINEAR_MAX_M bf16 tokens and
 * multiply by one NVFP4 weight in a single launch:
 *   out[m, n] = alpha * sum_k dq(W[n, k]) * dq(quant(x[m, :]))[k]
 * Stands in for the decode branch of `_nvfp4r_linear_impl`
 * (kernels/python/nvfp4r/vllm_integration.py:211-222: scaled_fp4_quant + expand +
 * empty + nvfp4r.gemv). The quantized codes/scales equal nvfp4r_quant's with the
 * same rcp_mode; they stay on chip. weight [N,K/2] and weight_scale [N,K/16]
 * (flat) contiguous; x bf16 with row stride `x_row_stride` elements; out [M,N]
 * contiguous.
 * Like the weight, `global_scale_inv` is a constant of the layer (the reference passes the
 * parameter `layer.input_global_scale_inv`): this entry point and the packed ones below
 * launch with programmatic stream serialization and read it, as they read the weight, while
 * the preceding kernel of the stream may still be running. It must therefore hold its
 * value before that kernel is launched. The same holds for `norm_weight` of the RMSNorm
 * prologue of nvfp4r_linear_packed_ex. Only `x` (and `delta` / `residual_in` of that
 * prologue) may be produced by the preceding kernel.
 * ------------------------------------------------------------------------- */
#define NVFP4R_LINEAR_MAX_M 16
NVFP4R_API int nvfp4r_linear(const void* x, int64_t x_row_stride, int M, int K,
                             const float* global_scale_inv,
                             const void* weight, const void* weight_scale, int N,
                             float alpha, void* out, int out_dtype, int rcp_mode,
                             void* stream);

/* ------------------------------------------------------------------------- *
 * Tensor-core GEMM (tcgen05 block-scaled MMA, kind mxf4nvf4, one e4m3 scale per
 * 16 elements) for M above the GEMV crossover:
 *   C[m, n] = alpha * sum_k dq(A[m, k]) * dq(B[n, k])
 * Stands in for `torch.ops.nvfp4r.gemm(A, B, SFA, SFB, C, alpha)` -
 * kernels/csrc/bindings.cpp:86-103 and kernels/cuda/gemm/gemm_nvfp4.cu:517-659.
 *   A   [M, K/2] activation codes, contiguous     SFA swizzled, >= ceil(M/128)*128 rows
 *   B   [N, K/2] weight codes, contiguous         SFB swizzled, >= ceil(N/128)*128 rows
 *   C   M*N elements of out_dtype (bf16 / fp16 / fp32)
 *   c_layout  NVFP4R_C_N_MAJOR: element (m,n) at C[n*M + m], the layout the
 *             reference kernel writes (gemm_nvfp4.cu:581, ops.py:86-88);
 *             NVFP4R_C_M_MAJOR: element (m,n) at C[m*N + n].
 * Any M >= 1 (the reference needs M % 64 == 0), N % 128 == 0, K % 256 == 0, any
 * such K (the reference has a fixed table, gemm_nvfp4.cu:633-650). Rows are taken 32
 * at a time, each pass streaming the weight once: built for decode-sized M.
 * `workspace` (>= nvfp4r_gemm_workspace_bytes(M, N, K) bytes, 16-byte aligned) holds
 * split-K partial sums and tile tickets; its first use must find it zeroed, and
 * every call leaves it zeroed again. Calls sharing a workspace must be ordered
 * on the stream. The first call on a device builds TMA descriptors on the host
 * (cuTensorMapEncodeTiled) and caches them per (pointer, shape).
 * ------------------------------------------------------------------------- */
typedef enum nvfp4r_c_layout { NVFP4R_C_M_MAJOR = 0, NVFP4R_C_N_MAJOR = 1 } nvfp4r_c_layout;
NVFP4R_API size_t nvfp4r_gemm_workspace_bytes(int M, int N, int K);
NVFP4R_API int nvfp4r_gemm(const void* A, const void* B, const void* SFA, const void* SFB,
                           void* C, int M, int N, int K, float alpha, int out_dtype,
                           int c_layout, void* workspace, size_t workspace_bytes, void* stream);

/* Fused decode linear on the tensor cores: quantize M bf16 tokens on chip and
 * multiply by one NVFP4 weight, result M-major [M, N]. Stands in for the padded-GEMM
 * branch of `_nvfp4r_linear_impl` (kernels/python/nvfp4r/vllm_integration.py:224-274:
 * scaled_fp4_quant + pad to 64 rows + nvfp4r.gemm + transpose + contiguous) in one
 * launch per 32 rows. weight [N,K/2]; weight_scale_swizzled in 128x4 tiles (the layout
 * vLLM keeps in layer.weight_scale); workspace as for nvfp4r_gemm. */
NVFP4R_API int nvfp4r_linear_tc(const void* x, int64_t x_row_stride, int M, int K,
                                const float* global_scale_inv, const void* weight,
                                const void* weight_scale_swizzled, int N, float alpha,
                                void* out, int out_dtype, int rcp_mode,
                                void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- *
 * Packed-weight decode linear: the fast path for every M <= 32 per launch.
 * The weight is re-laid out ONCE per layer (the work the reference does in
 * `prime_nvfp4r_caches`, kernels/python/nvfp4r/vllm_integration.py:359-396, where it
 * un-swizzles the scales) into blocks of 128 rows x 256 K-elements, each block 18 432
 * contiguous bytes: 16 KB of codes in the tensor core's shared-memory image (K-major,
 * 128-byte swizzle) followed by 2 KB of block scales in tcgen05.cp order. The linear then
 * streams the weight with one 36 KB bulk copy per pipeline stage.
 *   nvfp4r_packed_weight_bytes(N, K)   = N*K/2 + N*K/16 with K rounded up to a multiple of 256
 *                                      (0 if the shape is unsupported)
 *   nvfp4r_pack_weight                 weight [N,K/2] + flat scales [N,K/16] -> packed
 *                                      (packed 16-byte aligned; N % 128 == 0, K % 128 == 0; with
 *                                      K % 256 == 128 the last block is half zeros and the linear
 *                                      quantizes zeros for it: tensor-parallel shards such as the
 *                                      3200-wide down projection of Qwen3-32B at TP 8. The
 *                                      RMSNorm prologue of nvfp4r_linear_packed_ex still needs
 *                                      K % 256 == 0.)
 *   nvfp4r_linear_packed               out[M,N] = alpha * quant(x)[M,K] . W^T, same
 *                                      arithmetic and rcp_mode meaning as nvfp4r_linear;
 *                                      workspace >= nvfp4r_linear_packed_workspace_bytes(M,..)
 *                                      (grows with M), 16-byte aligned, ALL ZERO before the
 *                                      first use; every call leaves it all zero again, so
 *                                      linears of any shape may share one workspace as long
 *                                      as their launches are ordered on one stream
 * Stands in for the whole of `_nvfp4r_linear_impl` for decode-sized M
 * (vllm_integration.py:165-274) in one launch per 32 rows.
 * ------------------------------------------------------------------------- */
NVFP4R_API size_t nvfp4r_packed_weight_bytes(int N, int K);
NVFP4R_API size_t nvfp4r_linear_packed_workspace_bytes(int M, int N, int K);
NVFP4R_API int nvfp4r_pack_weight(const void* weight, const void* weight_scale_flat, void* packed,
                                  int N, int K, void* stream);
NVFP4R_API int nvfp4r_linear_packed(const void* x, int64_t x_row_stride, int M, int K,
                                    const float* global_scale_inv, const void* packed, int N,
                                    float alpha, void* out, int out_dtype, int rcp_mode,
                                    void* workspace, size_t workspace_bytes, void* stream);
/* The same linear with the operator that PRODUCES its input fused into the prologue, so
 * that the bf16 activation never makes a round trip through HBM and one launch
 * disappears per fusion. The reference names this as its own end goal
 * (kernels/python/nvfp4r/__init__.py:3-5) and its adapter notes the neighbouring vLLM ops
 * (rms_norm, fused_add_rms, silu_and_mul; vllm_integration.py:129-130).
 *   NVFP4R_PROLOGUE_ADD_RMSNORM  input = RMSNorm(residual_in + delta) * norm_weight, all
 *       bf16 with bf16 rounding after the add and after the scaling as the separate ops do;
 *       residual_in + delta is also written to residual_out (must not alias residual_in);
 *       delta may be NULL; `x` is ignored; K is the hidden size.
 *   NVFP4R_PROLOGUE_SILU_MUL     input[m,k] = silu(x[m,k]) * x[m,K+k], x = [M, 2K] (gate|up).
 *   NVFP4R_PROLOGUE_NONE         plain bf16 input (useful with push_to).
 * `pro` is a HOST pointer, read during the call. */
typedef enum nvfp4r_prologue_kind {
    NVFP4R_PROLOGUE_NONE = 0, NVFP4R_PROLOGUE_ADD_RMSNORM = 1, NVFP4R_PROLOGUE_SILU_MUL = 2
} nvfp4r_prologue_kind;
struct nvfp4r_peer_comm;            /* defined with the peer all-reduce below */
typedef struct nvfp4r_prologue {
    int kind;
    float eps;
    const void* delta;
    const void* residual_in;
    void* residual_out;
    const void* norm_weight;
    /* Epilogue option for row-parallel linears under tensor parallelism, NULL = off: instead of
     * writing `out`, every finished 128-row tile of the bf16 result is stored straight into the
     * receive memory of every rank (the PUSH half of nvfp4r_peer_allreduce_bf16, overlapped with
     * the remaining tiles); a following nvfp4r_peer_allreduce_bf16(..., NVFP4R_PEER_GATHER)
     * on `out` completes the sum. out_dtype must be bf16 and M*N <= push_to->max_elems. */
    const struct nvfp4r_peer_comm* push_to;
    /* With push_to: non-zero = finish the all-reduce inside this launch. The thread that pushed a
     * pair of results then waits for the other ranks' contributions to that pair in this rank's
     * own receive memory, adds them in rank order in fp32, rounds once, writes `out` and zeroes
     * the slots; no gather call follows. Every rank must run the same call at about the same
     * time: a CTA spins (bounded, nvfp4r_set_peer_poll_limit) until its peers have pushed, so
     * this mode needs one GPU per rank - ranks emulated as successive launches on one GPU must
     * use push + a separate gather. M <= 32. */
    int push_gather;
} nvfp4r_prologue;
NVFP4R_API int nvfp4r_linear_packed_ex(const nvfp4r_prologue* pro, const void* x, int64_t x_row_stride,
                                       int M, int K, const float* global_scale_inv, const void* packed,
                                       int N, float alpha, void* out, int out_dtype, int rcp_mode,
                                       void* workspace, size_t workspace_bytes, void* stream);

/* The fused prologues on the FLAT weight (codes [N,K/2] + scales [N,K/16]) through the CUDA-core
 * GEMV, for the launches the crossover gives to it (single token, small or medium weights: at
 * tensor-parallel shard sizes the GEMV's shorter fixed part wins). Same `pro` kinds, arithmetic
 * and roundings as nvfp4r_linear_packed_ex; M = 1 only. NVFP4R_PROLOGUE_NONE without push_to
 * forwards to nvfp4r_linear.
 * push_to (NVFP4R_PROLOGUE_NONE only, push_gather = 1 required): a row-parallel shard small
 * enough for the GEMV completes the tensor-parallel sum inside the GEMV's own launch: the lane
 * that finishes a pair of rows stores it into every rank's receive memory and adds the ranks'
 * contributions out of its own (protocol of nvfp4r_peer_allreduce_bf16, same buffers, same call
 * counter). One token, bf16 out, even N, K % 256 == 0, one GPU per rank. */
NVFP4R_API int nvfp4r_linear_ex(const nvfp4r_prologue* pro, const void* x, int64_t x_row_stride,
                                int M, int K, const float* global_scale_inv, const void* weight,
                                const void* weight_scale, int N, float alpha, void* out,
                                int out_dtype, int rcp_mode, void* stream);

/* Debug/tuning of the packed linear: bits 0-7 force the K split (0 = automatic), bit 8 records
 * an in-kernel time line of eight CTAs (bits 12-23: the first of them; only in a build with
 * -DNVFP4R_TRACE, ignored otherwise), bit 9 runs one CTA per SM instead of two, bits 24-27 hold
 * 1 + the number of pipeline stages each CTA asks into L2 ahead of its ring right after the
 * wait for the previous kernel (0 = keep; depth 0, 1 or 2, default 2). */
NVFP4R_API int nvfp4r_set_packed_tuning(int splits);

/* Debug/tuning: force the K split and ring depth of the tensor-core kernel (0 = automatic). */
NVFP4R_API int nvfp4r_set_gemm_tuning(int splits, int stages);

/* ------------------------------------------------------------------------- *
 * Block-scale layout conversion, [rows, K/16] flat <-> 128x4 swizzled tiles.
 * `nvfp4r_unswizzle_blockscale` stands in for `_unswizzle_blockscale`
 * (kernels/python/nvfp4r/vllm_integration.py:99-117), used once per layer by
 * `prime_nvfp4r_caches` (:359-396); `nvfp4r_swizzle_blockscale` is its inverse
 * (padding written as 0).
 * ------------------------------------------------------------------------- */
NVFP4R_API int nvfp4r_unswizzle_blockscale(const void* swizzled, void* flat,
                                           int rows, int K, void* stream);
NVFP4R_API int nvfp4r_swizzle_blockscale(const void* flat, void* swizzled,
                                         int rows, int K, void* stream);

/* ------------------------------------------------------------------------- *
 * ReSET step-aware temperature, one decode step for a batch of requests.
 * Stands in for `ReSETRequest.__call__` + `entropy_of` + `scale_by_temperature`
 * (reset/reset/logits_processor.py:101-134, :32-36, :22-29) applied to every row,
 * without the per-token host synchronisation of the reference.
 *
 * Per row b: boundary test on the last one/two generated ids, token entropy
 * H = -sum p*log(max(p,1e-10)), step-entropy estimate, running mean, temperature
 * choice, state update, then logits[b,:] /= temp in place (temp <= 1e-6: 0 at the
 * argmax, -inf elsewhere). State lives in `nvfp4r_reset_state` records on the
 * device, one per request slot, zero-initialised by the caller at request start.
 * ------------------------------------------------------------------------- */
#define NVFP4R_RESET_MAX_WINDOW 64

typedef struct nvfp4r_reset_state {
    double window_buf[NVFP4R_RESET_MAX_WINDOW]; /* ring of the last <= window entropies */
    double step_sum;      /* sum of entropies since the last step boundary          */
    double total_sum;     /* sum of all entropies of the request                    */
    int64_t total_count;  /* number of tokens seen                                  */
    int32_t step_count;   /* entropies since the last boundary                      */
    int32_t window_count; /* valid entries in window_buf                            */
    int32_t window_head;  /* index of the oldest entry                              */
    int32_t reserved;
} nvfp4r_reset_state;

typedef struct nvfp4r_reset_params {
    double t_high;   /* temperature for tokens at or above the threshold            */
    double t_low;    /* temperature for tokens below it                             */
    double tau0;     /* global threshold used while the step is not "uncertain"     */
    int32_t window;  /* w, 1..NVFP4R_RESET_MAX_WINDOW                               */
    int32_t id_set;  /* which newline-id set the request uses (per-request entry point
                        only; the single-record entry points ignore it)              */
} nvfp4r_reset_params;

/* What a step decided, one record per row (optional output, for logging/tests). */
typedef struct nvfp4r_reset_decision {
    double entropy;  /* float32 entropy widened to double, as the reference holds it */
    double h_step;
    double h_bar;
    double temp;
    int32_t boundary;
    int32_t high_step;
} nvfp4r_reset_decision;

/* Bytes of scratch one call needs for B rows (host arithmetic only). */
NVFP4R_API size_t nvfp4r_reset_workspace_bytes(int B);

/*   logits      fp32 [B,V] in/out, row stride `row_stride` elements
 *   states      records indexed by request slot
 *   state_slots [B] int32: index into `states` for each row, or -1 to leave the
 *               row untouched (request without ReSET); may be NULL (slot = row)
 *   last_ids    [B,2] int32: the two most recent generated ids of the request
 *               (oldest first), -1 where there is none yet; NULL = never a boundary
 *   nl_bitmap / dnl_bitmap  ceil(V/32) uint32 words: bit set = id decodes to a
 *               single newline / contains a double newline; may be NULL (no ids)
 *   params      one record on the HOST, copied by value into the launch
 *   decisions   [B] or NULL
 *   workspace   >= nvfp4r_reset_workspace_bytes(B) bytes of device scratch, 8-byte
 *               aligned, ALL ZERO before its first use (it holds a step counter per
 *               row that the calls advance); calls that share a workspace must be
 *               ordered on the stream
 * The step is ONE launch when the logits rows are 16-byte aligned, V % 4 == 0 and the
 * grid fits the device at once (slices of at most 5120 elements, a few hundred CTAs):
 * every CTA keeps its slice of the row in registers between the load and the final store,
 * and the CTAs of a row exchange their partial results through epoch-tagged 64-bit
 * slots. Otherwise three stream-ordered launches compute the same values.
 */
NVFP4R_API int nvfp4r_reset_step(float* logits, int64_t row_stride, int B, int V,
                                 nvfp4r_reset_state* states, const int32_t* state_slots,
                                 const int32_t* last_ids,
                                 const uint32_t* nl_bitmap, const uint32_t* dnl_bitmap,
                                 const nvfp4r_reset_params* params,
                                 nvfp4r_reset_decision* decisions,
                                 void* workspace, size_t workspace_bytes, void* stream);

/* The same step with each request's OWN hyper-parameters, as the reference builds one
 * ReSETRequest per request from that request's SamplingParams.extra_args
 * (reset/reset/logits_processor.py:144-155: t_high, t_low, tau_0, window, reset_nl_ids,
 * reset_dnl_ids). Differences from nvfp4r_reset_step:
 *   slot_params  records on the DEVICE, indexed by state slot like `states`; the host fills
 *                a slot's record when the request is admitted (window must be in
 *                1..NVFP4R_RESET_MAX_WINDOW; the kernel clamps it)
 *   nl_bitmaps / dnl_bitmaps  n_id_sets consecutive bitmaps of ceil(V/32) words each;
 *                a request uses set `slot_params[slot].id_set` (n_id_sets = 0: no ids)
 * A workspace that saw NVFP4R_ERR_DEVICE_TIMEOUT (nvfp4r_check_device_status) holds a
 * half-finished exchange: zero it before the next call. This holds for every entry point
 * that takes a workspace. */
NVFP4R_API int nvfp4r_reset_step_per_request(float* logits, int64_t row_stride, int B, int V,
                                             nvfp4r_reset_state* states, const int32_t* state_slots,
                                             const int32_t* last_ids,
                                             const uint32_t* nl_bitmaps, const uint32_t* dnl_bitmaps,
                                             int n_id_sets, const nvfp4r_reset_params* slot_params,
                                             nvfp4r_reset_decision* decisions,
                                             void* workspace, size_t workspace_bytes, void* stream);

/* lm_head and the ReSET step of ONE token in one launch: the logits are produced, judged and
 * divided on the chip and reach memory once, already divided by the temperature, instead of
 * being written by nvfp4r_lm_head, read and rewritten by nvfp4r_reset_step. No counterpart in
 * the reference (vLLM computes the logits and calls the processor, reset/reset/
 * logits_processor.py:175-189, as separate steps); it stands for that pair for a batch of one.
 *   x        bf16 [H], the final-norm output of the token
 *   weight   bf16 [V, H] row-major (16-byte aligned), H % 256 == 0, H <= 12288
 *   logits   fp32 [V] out: W.x / temperature (one-hot form for temperature <= 1e-6)
 *   states, state_slots ([1] or NULL), last_ids ([1,2]), nl_bitmaps / dnl_bitmaps / n_id_sets,
 *   slot_params, decisions ([1] or NULL): as nvfp4r_reset_step_per_request with B = 1;
 *            state_slots[0] < 0 writes the plain logits and leaves the request state alone
 *   workspace  >= nvfp4r_lm_head_reset_workspace_bytes() bytes, 8-byte aligned, ALL ZERO before
 *            its first use, one per token row in flight
 * The logits equal nvfp4r_lm_head's bit for bit before the division; the entropy is summed
 * over a different partition of the row than nvfp4r_reset_step uses (same terms, agreement to
 * float rounding). One CTA per SM, all resident at once (see "Residency" below);
 * NVFP4R_ERR_UNSUPPORTED_SHAPE when V exceeds 64 rows per warp of that grid (V > 303 104 on
 * 148 SMs). */
NVFP4R_API size_t nvfp4r_lm_head_reset_workspace_bytes(void);
NVFP4R_API int nvfp4r_lm_head_reset_step(const void* x, const void* weight, float* logits, int V, int H,
                                         nvfp4r_reset_state* states, const int32_t* state_slots,
                                         const int32_t* last_ids,
                                         const uint32_t* nl_bitmaps, const uint32_t* dnl_bitmaps,
                                         int n_id_sets, const nvfp4r_reset_params* slot_params,
                                         nvfp4r_reset_decision* decisions,
                                         void* workspace, size_t workspace_bytes, void* stream);

/* ReSET step without any caller-provided scratch. No counterpart in the reference (its
 * processor is PyTorch code and allocates freely); it exists for hosts that cannot
 * allocate device memory when they need the processor: a sampler plug-in inside an engine
 * whose memory pool already owns the whole GPU, or a C host that only holds fixed input
 * and output buffers. Same arguments, arithmetic and results as nvfp4r_reset_step, minus
 * the workspace: the scratch is a static array inside the library (41 984 B of device
 * memory on every GPU that loads it, held until the process exits).
 *   - B <= NVFP4R_RESET_STATIC_MAX_ROWS, otherwise NVFP4R_ERR_UNSUPPORTED_SHAPE.
 *   - Calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - The first call on each device looks the array's address up
 *     (cudaGetSymbolAddress, with that device current); make that first call outside any
 *     stream capture.
 *   - All calls on a device share the one array: two calls that overlap on the GPU
 *     (different streams without ordering) race on it. Order them. */
#define NVFP4R_RESET_STATIC_MAX_ROWS 64
NVFP4R_API int nvfp4r_reset_step_static(float* logits, int64_t row_stride, int B, int V,
                                        nvfp4r_reset_state* states, const int32_t* state_slots,
                                        const int32_t* last_ids,
                                        const uint32_t* nl_bitmap, const uint32_t* dnl_bitmap,
                                        const nvfp4r_reset_params* params,
                                        nvfp4r_reset_decision* decisions, void* stream);

/* Token entropy only: H[b] = -sum p*log(max(p,1e-10)) for each row, as float32.
 * Stands in for `entropy_of` (reset/reset/logits_processor.py:32-36). Same
 * workspace rule as nvfp4r_reset_step. */
NVFP4R_API int nvfp4r_entropy(const float* logits, int64_t row_stride, int B, int V,
                              float* entropy, void* workspace, size_t workspace_bytes,
                              void* stream);

/* ------------------------------------------------------------------------- *
 * Process-wide tuning of the streaming GEMV (not part of the reference's
 * surface; the reference reads the like from NVFP4R_GEMV_* environment
 * variables at kernels/cuda/gemv/gemv_nvfp4.cu:870-948). Negative = keep.
 *   ctas_per_sm   grid size = SM count * ctas_per_sm; 0 = automatic (default): one CTA per SM
 *                 with a three-slot ring per warp, or three CTAs per SM with two-slot rings
 *                 for single-token launches that have more row groups than one CTA per SM
 *                 has warps (N >= 6144) and K <= 4096, where 24 warps per SM hide the
 *                 latency of the decode chains better than 8 (measured)
 *   use_pdl       1 = launch with programmatic stream serialization (default 1)
 *   force_generic 1 = always use the plain-load fallback kernel (default 0)
 * ------------------------------------------------------------------------- */
NVFP4R_API int nvfp4r_set_gemv_tuning(int ctas_per_sm, int use_pdl, int force_generic);

/* Tuning of the register-resident GEMV that takes launches of one or two tokens (same
 * standing as the call above: the reference's counterpart is its NVFP4R_GEMV_* environment,
 * kernels/cuda/gemv/gemv_nvfp4.cu:870-948).
 *   mode           0 = automatic (default), 1 = whenever the arguments allow it, -1 = never
 *   rows_per_step  weight rows a lane multiplies per pipeline step: 0 = automatic, 2 or 4
 *   warps_per_sm   rows of at most 12288 elements run in CTAs of 12 warps, two of which fit an SM:
 *                  0 = automatic (both halves of every SM for weights above ~12 MB, one half
 *                  below, which leaves the other to the next launch's early loads),
 *                  1..12 = one half, 13..32 = both
 */
NVFP4R_API int nvfp4r_set_gemv_rows_tuning(int mode, int rows_per_step, int warps_per_sm);

/* ------------------------------------------------------------------------- *
 * One-shot all-reduce (sum) of a small bf16 tensor over NVLink peer memory: the exchange
 * after a row-parallel linear (o_proj, down_proj) under tensor parallelism, one launch per
 * rank, no library collective. In the reference's deployment this step is vLLM's
 * tensor_model_parallel_all_reduce inside RowParallelLinear (the reference itself only
 * consumes the per-partition sizes, kernels/python/nvfp4r/vllm_integration.py:461-462).
 * Every rank adds the W contributions in rank order in fp32 and rounds once, so all ranks
 * hold identical bits.
 *   set-up (host, once; these calls allocate / map memory, the all-reduce itself does not):
 *     nvfp4r_peer_buffer_bytes(world, max_elems)  size of one rank's receive memory
 *     nvfp4r_peer_alloc(bytes, &ptr, handle)      zeroed device memory + its 64-byte IPC handle
 *     nvfp4r_peer_open(handle, &peer_ptr)         map a peer's memory (another process, same node)
 *     nvfp4r_peer_close / nvfp4r_peer_free
 *   nvfp4r_peer_allreduce_bf16(comm, in, out, count, mode, stream)
 *     comm->base[r] = receive memory of rank r as seen from THIS process (own: the local
 *     pointer); count even, <= comm->max_elems; in/out 4-byte aligned, may alias.
 *     mode NVFP4R_PEER_PUSH | NVFP4R_PEER_GATHER (= 3) is the all-reduce; the two halves can be
 *     launched separately (push on every rank first, then gather) where ranks share one GPU.
 * Every rank must issue the same sequence of calls. A wait for a peer that never pushes ends
 * after a bounded number of polls and sets the status read by nvfp4r_check_device_status.
 * ------------------------------------------------------------------------- */
#define NVFP4R_PEER_MAX_WORLD 8
enum { NVFP4R_PEER_PUSH = 1, NVFP4R_PEER_GATHER = 2, NVFP4R_PEER_ALLREDUCE = 3 };
typedef struct nvfp4r_peer_comm {
    int world;
    int rank;
    size_t max_elems;
    void* base[NVFP4R_PEER_MAX_WORLD];
} nvfp4r_peer_comm;
NVFP4R_API size_t nvfp4r_peer_buffer_bytes(int world, size_t max_elems);
NVFP4R_API int nvfp4r_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64);
NVFP4R_API int nvfp4r_peer_open(const unsigned char* handle64, void** peer_ptr);
NVFP4R_API int nvfp4r_peer_close(void* peer_ptr);
NVFP4R_API int nvfp4r_peer_free(void* ptr);
NVFP4R_API int nvfp4r_peer_allreduce_bf16(const nvfp4r_peer_comm* comm, const void* in, void* out,
                                          size_t count, int mode, void* stream);
/* Polls a gather makes per group of slots before it gives up on a peer (0 = default, a second
 * or two). Failure detection: the launch then finishes, the result is undefined and
 * nvfp4r_check_device_status returns NVFP4R_ERR_DEVICE_TIMEOUT. */
NVFP4R_API int nvfp4r_set_peer_poll_limit(unsigned polls);

/* Reads and clears the device-side time-out flag of the current device
 * (synchronises the device; diagnostics only). Returns 0, or
 * NVFP4R_ERR_DEVICE_TIMEOUT if a bounded wait inside a kernel gave up. */
NVFP4R_API int nvfp4r_check_device_status(void);

/* The same information WITHOUT a device synchronisation: *host_word points at one int in
 * pinned, mapped host memory (allocated at the first call on the current device; this call
 * allocates, the launches never do). A kernel whose bounded wait gives up stores a non-zero code
 * there (1 GEMV ring, 2 tensor-core GEMM, 3 packed linear, 4 peer all-reduce, 5 ReSET step) next
 * to setting its device flag; the host may read the word at any time, e.g. every few decode
 * steps, and writes 0 to clear it. A time-out means the output of that launch is undefined and
 * the scratch it used (split-K slots, ReSET workspace, peer receive memory) is mid-exchange:
 * zero it before the next use.
 *
 * Residency. nvfp4r_linear_packed*, the single-launch form of nvfp4r_reset_step*,
 * nvfp4r_lm_head_reset_step and push_gather wait for other CTAs of their own grid (or of a peer GPU's grid). Their grids are
 * sized to be resident all at once on an otherwise idle device (at most two CTAs per SM; the
 * ReSET launcher falls back to its three-launch form when the occupancy calculation says the
 * grid does not fit). A kernel of ANOTHER stream that holds SMs at the same time can delay the
 * missing CTAs; the waits then last until that kernel leaves, or give up after their poll limit
 * and report through this word. Run them on one stream, or keep concurrent kernels small.
 * No counterpart in the reference (its kernels' mbarrier waits are unbounded,
 * kernels/cuda/gemm/gemm_nvfp4.cu:44-56). */
NVFP4R_API int nvfp4r_status_mirror(volatile int** host_word);

/* ------------------------------------------------------------------------- *
 * Batch-1 decode-step operators around the linears (bf16 activations). None of these
 * has a counterpart in the reference: in its deployment vLLM provides them. They let the
 * full Qwen3 decode step of the benchmark run from one CUDA graph on this library alone.
 *   nvfp4r_add_rmsnorm      residual += x (x may be NULL); out = RMSNorm(residual) * weight
 *   nvfp4r_qk_norm_rope_kv  per-head RMSNorm on q and k, rotary embedding (rotate-half) at
 *                           *position, k/v written to caches [Hkv, Tmax, D], q to q_out
 *   nvfp4r_attn_decode      GQA attention of one token over the first *seq_len cache rows, one
 *                           launch; workspace >= nvfp4r_attn_decode_workspace_bytes, ZEROED
 *                           before the first use (it holds arrival counters that every call
 *                           leaves at zero); *seq_len must not be written by the launch that
 *                           directly precedes this one (cache rows of earlier tokens are
 *                           fetched before that launch is waited for)
 *   nvfp4r_silu_mul         out[m,i] = silu(gate_up[m,i]) * gate_up[m,I+i]
 *   nvfp4r_lm_head          logits[v] = W[v,:] . x, bf16 weight, fp32 logits
 *   nvfp4r_argmax           first index of the row maximum
 * D == 128, Hq / Hkv <= 8, H % 256 == 0.
 * ------------------------------------------------------------------------- */
NVFP4R_API int nvfp4r_add_rmsnorm(const void* x, void* residual, const void* weight, void* out,
                                  int M, int H, float eps, void* stream);
NVFP4R_API int nvfp4r_qk_norm_rope_kv(const void* qkv, const void* q_weight, const void* k_weight,
                                      const int32_t* position, void* kcache, void* vcache,
                                      void* q_out, int Hq, int Hkv, int D, int Tmax, float theta,
                                      float eps, void* stream);
/* Optional table for the rotary embedding of nvfp4r_qk_norm_rope_kv / nvfp4r_attn_decode_rope:
 * `cos_sin` = device array of float pairs [rows][64] = (cos, sin)(pos * theta^(-2d/128)), built
 * once by the caller for its theta (vLLM keeps the same kind of cos_sin_cache). While set, and
 * rows >= Tmax of the call, the kernels read it instead of evaluating powf/sincosf. Process-wide
 * (one device per process); NULL clears it. */
NVFP4R_API int nvfp4r_set_rope_table(const float* cos_sin, int rows);
/* nvfp4r_attn_decode_rope = nvfp4r_qk_norm_rope_kv + nvfp4r_attn_decode in one launch: `qkv`
 * is the raw fused row [(Hq + 2 Hkv) * D]; the token's position is *seq_len - 1; the new K/V row
 * is appended to the caches by the launch itself. Same workspace rule as nvfp4r_attn_decode. */
NVFP4R_API int nvfp4r_attn_decode_rope(const void* qkv, const void* q_weight, const void* k_weight,
                                       void* kcache, void* vcache, const int32_t* seq_len, void* out,
                                       int Hq, int Hkv, int D, int Tmax, float theta, float eps,
                                       void* workspace, size_t workspace_bytes, void* stream);
NVFP4R_API size_t nvfp4r_attn_decode_workspace_bytes(int Hq, int Tmax);
NVFP4R_API int nvfp4r_attn_decode(const void* q, const void* kcache, const void* vcache,
                                  const int32_t* seq_len, void* out, int Hq, int Hkv, int D,
                                  int Tmax, void* workspace, size_t workspace_bytes, void* stream);
NVFP4R_API int nvfp4r_silu_mul(const void* gate_up, void* out, int M, int I, void* stream);
NVFP4R_API int nvfp4r_lm_head(const void* x, const void* weight, float* logits, int V, int H,
                              void* stream);
NVFP4R_API int nvfp4r_argmax(const float* logits, int64_t row_stride, int B, int V, int32_t* out,
                             void* stream);
/* One token id per row drawn from softmax(logits[b, :]) by the Gumbel-max rule
 * (arg-max of logits + Gumbel noise), entirely on the device. In the reference's deployment
 * this is vLLM's sampler running at temperature 1.0 on the logits the ReSET processor has
 * already scaled (reset/README.md:87-88); here it lets a whole decode step, processor and
 * sampling included, stay in one CUDA graph with no host round trip.
 *   seed      any value; together with the row index and the row's draw counter it keys a
 *             counter-based generator, so results are reproducible
 *   draws     [B] uint64 on the device, zeroed by the caller at request start; advanced by
 *             one per call (a replayed graph therefore keeps drawing fresh numbers)
 *   last_ids  [B,2] int32 on the device or NULL: shifted left with the drawn id appended,
 *             which is the `last_ids` input of nvfp4r_reset_step for the next step
 * Rows holding one 0 and -inf elsewhere (what ReSET writes for temperatures <= 1e-6) return
 * the position of the 0. B <= 256. */
NVFP4R_API int nvfp4r_sample(const float* logits, int64_t row_stride, int B, int V, uint64_t seed,
                             uint64_t* draws, int32_t* last_ids, int32_t* out, void* stream);

/* The same draw restricted to the top-k and / or top-p (nucleus) set of every row, as vLLM's
 * sampler applies them behind the processor: top-k first (the k largest logits; keys equal to the
 * k-th are all kept), then top-p on the distribution renormalised over that set (the smallest set
 * of largest probabilities whose mass reaches top_p). top_k <= 0 or >= V and top_p >= 1 switch the
 * respective truncation off; with both off this is nvfp4r_sample. The sets are found by a radix
 * descent over order-preserving keys of the logits (three levels of 2048-bin histograms of count
 * and fixed-point probability mass, integer atomics: the result does not depend on the order of
 * the additions), then the Gumbel-max draw skips everything below the threshold key.
 *   workspace  >= nvfp4r_sample_workspace_bytes(B) bytes, 8-byte aligned, ALL ZERO before its first
 *              use; every call leaves the histograms zeroed. Calls that share it must be ordered.
 * No counterpart in the reference (vLLM owns the sampler there, reset/README.md:87-88). */
NVFP4R_API size_t nvfp4r_sample_workspace_bytes(int B);
NVFP4R_API int nvfp4r_sample_top_k_top_p(const float* logits, int64_t row_stride, int B, int V,
                                         int top_k, float top_p, uint64_t seed, uint64_t* draws,
                                         int32_t* last_ids, int32_t* out, void* workspace,
                                         size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4R_B200_H_ */
