// lm_head and the ReSET step of one decode token in ONE launch: the logits never make the
// fp32 round trip through memory between the vocabulary projection and the logits processor.
//
// The vocabulary projection (bf16 weight [V, H] streamed once, one warp per row, exactly the
// arithmetic of lm_head_kernel) leaves every CTA's logits in its shared memory. What follows is
// the ReSET step (reference reset/reset/logits_processor.py:101-134) on those on-chip values,
// with the hand-overs of the stand-alone step kernel between the CTAs of the grid:
//   CTA (max, sum exp, argmax)    -> every CTA        (row max, softmax denominator)
//   CTA entropy partial (double)  -> CTA 0            (state machine, temperature)
//   temperature / mode            -> every CTA        (division on the way out)
// and the logits are written to memory once, already divided by the temperature.
// Grid: one CTA of 1024 threads per SM, all resident at once (the launcher checks), hand-overs
// through epoch-tagged 64-bit slots {epoch : payload}, so nothing is ever cleared and all-zero
// memory is a valid start. Polls are bounded; a CTA that gives up raises the status word and
// writes its logits undivided.
#include "kernels.h"
#include "status_mirror.cuh"
#include "nvfp4_ptx.cuh"
#include "lm_head_dot.cuh"
#include "reset_kernels.h"
#include "reset_policy.cuh"

namespace nvfp4r {
namespace {

constexpr int kHeadThreads = 1024;
constexpr int kHeadWarps = kHeadThreads / 32;
static_assert(kHeadWarps == 32, "entry e of a CTA belongs to warp e & 31");
constexpr int kHeadMaxParts = 256;                 // CTAs of the grid (one per SM)
constexpr int kHeadMaxRowsPerWarp = 64;            // logits one warp may hold: V <= 64 * warps of the grid
constexpr uint32_t kHeadPollLimit = 4000000u;

// Workspace of one token row: the exchange slots, then the scratch record of the deciding thread.
struct HeadSlots {
    unsigned long long pmax[kHeadMaxParts];
    unsigned long long psum[kHeadMaxParts];
    unsigned long long parg[kHeadMaxParts];
    unsigned long long ent_hi[kHeadMaxParts];
    unsigned long long ent_lo[kHeadMaxParts];
    unsigned long long temp;                       // chosen temperature (float bits)
    unsigned long long mode;                       // 0: divide, 1: T == 1, 2: one-hot at the argmax
    unsigned epoch;
    unsigned pad;
    RowScratch scratch;
};

__device__ int g_head_status = 0;

__device__ __forceinline__ void hs_publish(unsigned long long* slot, unsigned epoch, uint32_t payload) {
    const unsigned long long w = (static_cast<unsigned long long>(epoch) << 32) | payload;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(slot), "l"(w) : "memory");
}
__device__ __forceinline__ bool hs_poll(const unsigned long long* slot, unsigned epoch, uint32_t* payload) {
    for (uint32_t it = 0; it <= kHeadPollLimit; ++it) {
        unsigned long long w;
        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(slot) : "memory");
        if (static_cast<unsigned>(w >> 32) == epoch) {
            *payload = static_cast<uint32_t>(w);
            return true;
        }
    }
    return false;
}

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}
__device__ __forceinline__ void warp_argmax(float& best, int& arg) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, s);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, s);
        if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
}

// Dynamic shared memory: H floats of the activation row, then rows_per_warp * 32 logits
// (entry k * 32 + w is the k-th row of warp w: vocabulary row first_row + w + k * grid_warps).
__global__ void __launch_bounds__(kHeadThreads, 1)
lm_head_reset_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W, int H,
                     const ResetLaunch p, HeadSlots* __restrict__ hs, const int rows_per_warp) {
    extern __shared__ __align__(16) float smem_f[];
    float* xs = smem_f;
    float* lg = smem_f + H;
    __shared__ float s_f[kHeadWarps];
    __shared__ int s_i[kHeadWarps];
    __shared__ double s_d[kHeadWarps];
    __shared__ float s_pmax[kHeadMaxParts], s_psum[kHeadMaxParts];
    __shared__ int s_parg[kHeadMaxParts];
    __shared__ uint32_t s_hi[kHeadMaxParts], s_lo[kHeadMaxParts];
    __shared__ float s_rmax, s_denom;
    __shared__ int s_rarg;
    __shared__ uint32_t s_word[3];
    __shared__ int s_fail;
    __shared__ __align__(8) nvfp4r_reset_state s_state;
    __shared__ __align__(8) nvfp4r_reset_params s_prm;
    __shared__ int s_boundary;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int parts = static_cast<int>(gridDim.x);
    const int grid_warps = parts * kHeadWarps;
    const int V = p.V;
    float* __restrict__ logits = const_cast<float*>(p.logits);

    pdl_wait_prior();
    const int slot = p.state_slots ? p.state_slots[0] : 0;
    const bool active = slot >= 0;
    const unsigned epoch = *reinterpret_cast<volatile unsigned*>(&hs->epoch) + 1u;
    if (tid == 0) s_fail = 0;
    constexpr int kStateWords = static_cast<int>(sizeof(nvfp4r_reset_state) / 8);
    if (active && blockIdx.x == 0) {
        // the request's record and the boundary test do not depend on this token's logits
        if (tid < kStateWords)
            reinterpret_cast<unsigned long long*>(&s_state)[tid] =
                reinterpret_cast<const unsigned long long*>(p.states + slot)[tid];
        if (tid == kHeadThreads - 1) {
            s_prm = reset_params_of(p, slot);
            s_boundary = reset_boundary(p, 0, s_prm.id_set) ? 1 : 0;
        }
    }

    // ---- the vocabulary projection: this CTA's logits stay in shared memory -------------------
    for (int i = tid; i < H; i += kHeadThreads) xs[i] = __bfloat162float(x[i]);
    __syncthreads();
    const int first_row = static_cast<int>(blockIdx.x) * kHeadWarps;
    {
        int k = 0;
        for (int v = first_row + warp; v < V; v += grid_warps, ++k) {
            const uint4* row = reinterpret_cast<const uint4*>(W + static_cast<int64_t>(v) * H);
            float acc = lm_head_row_dot(row, xs, H / 8, lane);
            acc = warp_sum_f(acc);
            if (lane == 0) lg[k * 32 + warp] = acc;
        }
    }
    pdl_launch_dependents();
    __syncthreads();

    // entry e of this CTA: logits row first_row + (e & 31) + (e >> 5) * grid_warps
    const int n_entries = rows_per_warp * 32;
    auto row_of = [&](int e) { return first_row + (e & 31) + (e >> 5) * grid_warps; };

    if (!active) {                                         // request without ReSET: plain lm_head
        for (int e = tid; e < n_entries; e += kHeadThreads) {
            const int v = row_of(e);
            if (v < V) logits[v] = lg[e];
        }
        return;
    }

    // ---- CTA max / argmax / sum exp -> slots -----------------------------------------------------
    float vmax = -INFINITY;
    int varg = 0x7fffffff;
    for (int e = tid; e < n_entries; e += kHeadThreads) {
        const int v = row_of(e);
        if (v < V) {
            const float val = lg[e];
            if (val > vmax || (val == vmax && v < varg)) { vmax = val; varg = v; }
        }
    }
    warp_argmax(vmax, varg);
    if (lane == 0) { s_f[warp] = vmax; s_i[warp] = varg; }
    __syncthreads();
    float bmax = s_f[0];
    int barg = s_i[0];
#pragma unroll 1
    for (int w = 1; w < kHeadWarps; ++w)
        if (s_f[w] > bmax || (s_f[w] == bmax && s_i[w] < barg)) { bmax = s_f[w]; barg = s_i[w]; }
    __syncthreads();
    float sum = 0.0f;
    for (int e = tid; e < n_entries; e += kHeadThreads)
        if (row_of(e) < V) sum += expf(lg[e] - bmax);
    sum = warp_sum_f(sum);
    if (lane == 0) s_f[warp] = sum;
    __syncthreads();
    if (tid == 0) {
        float tot = 0.0f;
#pragma unroll 1
        for (int w = 0; w < kHeadWarps; ++w) tot += s_f[w];
        const bool any = barg != 0x7fffffff;
        hs_publish(&hs->pmax[blockIdx.x], epoch, __float_as_uint(any ? bmax : -INFINITY));
        hs_publish(&hs->psum[blockIdx.x], epoch, __float_as_uint(any ? tot : 0.0f));
        hs_publish(&hs->parg[blockIdx.x], epoch, static_cast<uint32_t>(barg));
    }

    // ---- every CTA: all partials -> row max, argmax, denominator ----------------------------------
    for (int i = tid; i < 3 * parts; i += kHeadThreads) {
        const int which = i / parts, idx = i - which * parts;
        const unsigned long long* src = which == 0 ? &hs->pmax[idx] : which == 1 ? &hs->psum[idx] : &hs->parg[idx];
        uint32_t v = 0;
        if (!hs_poll(src, epoch, &v)) s_fail = 1;
        if (which == 0) s_pmax[idx] = __uint_as_float(v);
        else if (which == 1) s_psum[idx] = __uint_as_float(v);
        else s_parg[idx] = static_cast<int>(v);
    }
    __syncthreads();
    if (s_fail) {
        if (tid == 0) report_timeout(&g_head_status, 5);
        for (int e = tid; e < n_entries; e += kHeadThreads) {
            const int v = row_of(e);
            if (v < V) logits[v] = lg[e];
        }
        return;
    }
    if (warp == 0) {
        // lane l owns CTAs l, l + 32, ...; fixed loops and shuffle trees: every CTA computes the same bits
        float rmax = -INFINITY;
        int rarg = 0x7fffffff;
        for (int i = lane; i < parts; i += 32)
            if (s_pmax[i] > rmax || (s_pmax[i] == rmax && s_parg[i] < rarg)) { rmax = s_pmax[i]; rarg = s_parg[i]; }
        warp_argmax(rmax, rarg);
        double den = 0.0;
        for (int i = lane; i < parts; i += 32)
            if (s_psum[i] > 0.0f) den += static_cast<double>(s_psum[i]) * exp(static_cast<double>(s_pmax[i]) - rmax);
        den = warp_sum_d(den);
        if (lane == 0) { s_rmax = rmax; s_rarg = rarg; s_denom = static_cast<float>(den); }
    }
    __syncthreads();
    const float rmax = s_rmax, denom = s_denom;
    const int rarg = s_rarg;

    // ---- CTA entropy partial -> slots ---------------------------------------------------------------
    float acc = 0.0f;
    for (int e = tid; e < n_entries; e += kHeadThreads)
        if (row_of(e) < V) {
            const float pr = expf(lg[e] - rmax) / denom;
            acc += pr * logf(fmaxf(pr, 1e-10f));
        }
    const double part = warp_sum_d(static_cast<double>(acc));
    if (lane == 0) s_d[warp] = part;
    __syncthreads();
    if (tid == 0) {
        double tot = 0.0;
#pragma unroll 1
        for (int w = 0; w < kHeadWarps; ++w) tot += s_d[w];
        const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(tot));
        hs_publish(&hs->ent_hi[blockIdx.x], epoch, static_cast<uint32_t>(bits >> 32));
        hs_publish(&hs->ent_lo[blockIdx.x], epoch, static_cast<uint32_t>(bits));
    }

    // ---- CTA 0 decides ------------------------------------------------------------------------------
    if (blockIdx.x == 0) {
        __syncthreads();
        for (int i = tid; i < 2 * parts; i += kHeadThreads) {
            const int which = i / parts, idx = i - which * parts;
            uint32_t v = 0;
            if (!hs_poll(which == 0 ? &hs->ent_hi[idx] : &hs->ent_lo[idx], epoch, &v)) s_fail = 1;
            if (which == 0) s_hi[idx] = v;
            else s_lo[idx] = v;
        }
        __syncthreads();
        if (tid == 0) {
            if (s_fail) {
                report_timeout(&g_head_status, 5);
            } else {
                double h = 0.0;
                for (int s = 0; s < parts; ++s) {
                    const unsigned long long bits = (static_cast<unsigned long long>(s_hi[s]) << 32) | s_lo[s];
                    h += __longlong_as_double(static_cast<long long>(bits));
                }
                const float ent_f = static_cast<float>(-h);
                RowScratch* rs = &hs->scratch;
                reset_decide_on(p, s_prm, 0, &s_state, s_boundary != 0, static_cast<double>(ent_f), rarg, rs);
                const double temp_d = rs->temp;
                const uint32_t mode = (temp_d == 1.0) ? 1u : (temp_d <= 1e-6 ? 2u : 0u);
                hs_publish(&hs->temp, epoch, __float_as_uint(static_cast<float>(temp_d)));
                hs_publish(&hs->mode, epoch, mode);
            }
            // every CTA has read the epoch by now (each published with it): advance
            *reinterpret_cast<volatile unsigned*>(&hs->epoch) = epoch;
        }
        __syncthreads();
        if (tid < kStateWords)
            reinterpret_cast<unsigned long long*>(p.states + slot)[tid] =
                reinterpret_cast<const unsigned long long*>(&s_state)[tid];
    }

    // ---- temperature -> the logits leave the chip once, already divided ----------------------------
    if (tid < 2) {
        uint32_t v = tid;                                              // on a time-out: mode 1
        if (!hs_poll(tid == 0 ? &hs->temp : &hs->mode, epoch, &v)) {
            report_timeout(&g_head_status, 5);
            v = tid;
        }
        s_word[tid] = v;
    }
    __syncthreads();
    const uint32_t mode = s_word[1];
    const float t = __uint_as_float(s_word[0]);
    for (int e = tid; e < n_entries; e += kHeadThreads) {
        const int v = row_of(e);
        if (v < V) {
            const float val = lg[e];
            logits[v] = mode == 1u ? val : mode == 2u ? (v == rarg ? 0.0f : -INFINITY) : __fdiv_rn(val, t);
        }
    }
}

}  // namespace

size_t lm_head_reset_workspace_bytes() { return sizeof(HeadSlots); }

// `p` carries the ReSET side (B == 1: logits = the output row); returns cudaErrorInvalidConfiguration
// when the grid cannot be resident at once or a warp would hold more logits than its share of
// shared memory allows.
cudaError_t launch_lm_head_reset(const void* x, const void* weight, int H, ResetLaunch p, void* workspace,
                                 cudaStream_t stream) {
    const int sms = device_sm_count();
    const int parts = sms < kHeadMaxParts ? sms : kHeadMaxParts;
    const int grid_warps = parts * kHeadWarps;
    const int rows_per_warp = (p.V + grid_warps - 1) / grid_warps;
    if (rows_per_warp > kHeadMaxRowsPerWarp) return cudaErrorInvalidConfiguration;
    const size_t smem = static_cast<size_t>(H) * 4 + static_cast<size_t>(rows_per_warp) * 32 * 4;
    static bool checked[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && !checked[dev]) {
        e = cudaFuncSetAttribute(lm_head_reset_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) return e;
        checked[dev] = true;
    }
    if (smem > 96 * 1024) return cudaErrorInvalidConfiguration;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lm_head_reset_kernel, kHeadThreads, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorInvalidConfiguration;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(parts));
    cfg.blockDim = dim3(kHeadThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gemv_tuning().use_pdl ? 1 : 0;
    p.B = 1;
    return cudaLaunchKernelEx(&cfg, lm_head_reset_kernel, static_cast<const __nv_bfloat16*>(x),
                              static_cast<const __nv_bfloat16*>(weight), H, p, static_cast<HeadSlots*>(workspace),
                              rows_per_warp);
}

cudaError_t set_status_mirror_head(int* p) { return set_status_mirror_here(p); }

cudaError_t read_and_clear_head_status(int* flag) {
    cudaError_t e = cudaMemcpyFromSymbol(flag, g_head_status, sizeof(int));
    if (e != cudaSuccess) return e;
    const int zero = 0;
    return cudaMemcpyToSymbol(g_head_status, &zero, sizeof(int));
}

}  // namespace nvfp4r
