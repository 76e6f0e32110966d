// ReSET step-aware temperature as three stream-ordered kernels per decode step.
//
//   1. reset_partials_kernel : every CTA owns one slice of one row and leaves
//      (max, sum exp(x - max), argmax) of the slice in the row's scratch record.
//   2. reset_entropy_kernel  : every CTA combines the row's partials into the
//      row max and softmax denominator, re-reads its slice (L2-resident) and adds
//      up p*log(max(p,1e-10)). The CTA that arrives last for a row (atomic
//      ticket, no waiting) sums the slice entropies in slice order, runs the
//      per-request state machine in double precision and publishes the
//      temperature.
//   3. reset_scale_kernel    : divides the slice by the temperature in place;
//      rows whose temperature is exactly 1 are left untouched (x/1 == x).
//
// All three are launched with programmatic stream serialization and release their
// dependents at once, so launch latency overlaps the kernel before; each reads what the
// previous kernel wrote only after griddepcontrol.wait.
#include "kernels.h"
#include "nvfp4_ptx.cuh"
#include "reset_kernels.h"

namespace nvfp4r {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}

struct SliceView {
    const float* base;   // first element of the slice
    int len;             // elements in the slice (may be 0)
    int first;           // index of base within the row
    bool vec;            // 16-byte aligned and len % 4 == 0
};

__device__ __forceinline__ SliceView slice_of(const ResetLaunch& p, int row, int slice) {
    SliceView s;
    s.first = min(slice * p.slice_len, p.V);
    s.len = min(p.slice_len, p.V - s.first);
    s.base = p.logits + static_cast<int64_t>(row) * p.row_stride + s.first;
    s.vec = ((reinterpret_cast<uintptr_t>(s.base) & 15) == 0) && (s.len % 4 == 0);
    return s;
}

__device__ __forceinline__ bool row_active(const ResetLaunch& p, int row, int* slot) {
    const int s = p.state_slots ? p.state_slots[row] : row;
    *slot = s;
    return !p.needs_state || s >= 0;
}

// ---- kernel 1 ---------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
reset_partials_kernel(const ResetLaunch p) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int row = blockIdx.y, slice = blockIdx.x;
    int slot;
    if (!row_active(p, row, &slot)) return;
    const SliceView sv = slice_of(p, row, slice);
    RowScratch* rs = p.scratch + row;
    __shared__ float s_max[kThreads / 32];
    __shared__ int s_arg[kThreads / 32];
    __shared__ float s_sum[kThreads / 32];

    float vmax = -INFINITY;
    int varg = 0x7fffffff;
    if (sv.vec) {
        const float4* v4 = reinterpret_cast<const float4*>(sv.base);
        for (int i = threadIdx.x; i < sv.len / 4; i += kThreads) {
            const float4 v = __ldg(v4 + i);
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (e[k] > vmax) { vmax = e[k]; varg = sv.first + 4 * i + k; }
        }
    } else {
        for (int i = threadIdx.x; i < sv.len; i += kThreads) {
            const float e = __ldg(sv.base + i);
            if (e > vmax) { vmax = e; varg = sv.first + i; }
        }
    }
    // block arg-max: largest value, lowest index among equals
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, vmax, s);
        const int oa = __shfl_xor_sync(0xffffffffu, varg, s);
        if (om > vmax || (om == vmax && oa < varg)) { vmax = om; varg = oa; }
    }
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (lane == 0) { s_max[warp] = vmax; s_arg[warp] = varg; }
    __syncthreads();
    float bmax = s_max[0];
    int barg = s_arg[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w)
        if (s_max[w] > bmax || (s_max[w] == bmax && s_arg[w] < barg)) { bmax = s_max[w]; barg = s_arg[w]; }

    float sum = 0.0f;
    if (sv.vec) {
        const float4* v4 = reinterpret_cast<const float4*>(sv.base);
        for (int i = threadIdx.x; i < sv.len / 4; i += kThreads) {
            const float4 v = __ldg(v4 + i);
            sum += expf(v.x - bmax) + expf(v.y - bmax) + expf(v.z - bmax) + expf(v.w - bmax);
        }
    } else {
        for (int i = threadIdx.x; i < sv.len; i += kThreads) sum += expf(__ldg(sv.base + i) - bmax);
    }
    sum = warp_sum(sum);
    if (lane == 0) s_sum[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) tot += s_sum[w];
        rs->pmax[slice] = sv.len > 0 ? bmax : -INFINITY;
        rs->psum[slice] = sv.len > 0 ? tot : 0.0f;
        rs->parg[slice] = barg;
        if (slice == 0) rs->ticket = 0u;
    }
}

// ---- the per-request state machine (one thread) --------------------------------
__device__ void reset_decide(const ResetLaunch& p, int row, int slot, double ent, int argmax,
                             RowScratch* rs) {
    nvfp4r_reset_state* st = p.states + slot;
    const int w = p.params.window;
    bool boundary = false;
    if (p.last_ids != nullptr) {
        const int prev = p.last_ids[2 * row], last = p.last_ids[2 * row + 1];
        auto in_set = [&](const uint32_t* bm, int id) {
            return bm != nullptr && id >= 0 && id < p.V && ((bm[id >> 5] >> (id & 31)) & 1u);
        };
        if (last >= 0) {
            if (in_set(p.dnl_bitmap, last)) boundary = true;
            else if (prev >= 0 && in_set(p.nl_bitmap, last) && in_set(p.nl_bitmap, prev)) boundary = true;
        }
    }
    if (boundary) { st->step_count = 0; st->step_sum = 0.0; }

    double h_step;
    if (st->step_count < w) {
        if (st->window_count > 0) {
            double s = 0.0;                      // oldest -> newest, as Python's sum()
            for (int i = 0; i < st->window_count; ++i)
                s += st->window_buf[(st->window_head + i) % NVFP4R_RESET_MAX_WINDOW];
            h_step = s / static_cast<double>(st->window_count);
        } else {
            h_step = ent;
        }
    } else {
        h_step = st->step_sum / static_cast<double>(st->step_count);
    }
    const double h_bar = st->total_count > 0
                             ? st->total_sum / static_cast<double>(st->total_count) : h_step;
    const bool high = h_step > h_bar;
    const double thr = high ? h_step : p.params.tau0;
    const double temp = (ent >= thr) ? p.params.t_high : p.params.t_low;

    // bookkeeping
    st->step_sum += ent;
    st->step_count += 1;
    if (st->window_count < w) {
        st->window_buf[(st->window_head + st->window_count) % NVFP4R_RESET_MAX_WINDOW] = ent;
        st->window_count += 1;
    } else {                                     // drop the oldest, append
        st->window_head = (st->window_head + 1) % NVFP4R_RESET_MAX_WINDOW;
        st->window_buf[(st->window_head + w - 1) % NVFP4R_RESET_MAX_WINDOW] = ent;
    }
    st->total_sum += ent;
    st->total_count += 1;

    rs->temp = temp;
    rs->argmax = argmax;
    if (p.decisions != nullptr) {
        nvfp4r_reset_decision d;
        d.entropy = ent; d.h_step = h_step; d.h_bar = h_bar; d.temp = temp;
        d.boundary = boundary ? 1 : 0; d.high_step = high ? 1 : 0;
        p.decisions[row] = d;
    }
}

// ---- kernel 2 ---------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
reset_entropy_kernel(const ResetLaunch p) {
    const int row = blockIdx.y, slice = blockIdx.x;
    int slot;
    if (!row_active(p, row, &slot)) return;
    const SliceView sv = slice_of(p, row, slice);
    RowScratch* rs = p.scratch + row;
    __shared__ double s_part[kThreads / 32];
    __shared__ bool s_last;

    pdl_launch_dependents();
    pdl_wait_prior();
    // Row max and denominator from the slice partials: lane s owns slice s (at most 32
    // slices), the reductions are fixed shuffle trees, so every warp of every CTA of the row
    // computes the same bits.
    const int lane_m = threadIdx.x % 32;
    float rmax = (lane_m < p.n_slices) ? rs->pmax[lane_m] : -INFINITY;
    int rarg = (lane_m < p.n_slices) ? rs->parg[lane_m] : 0x7fffffff;
    const float my_max = rmax;
    const float my_sum = (lane_m < p.n_slices) ? rs->psum[lane_m] : 0.0f;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, rmax, s);
        const int oa = __shfl_xor_sync(0xffffffffu, rarg, s);
        if (om > rmax || (om == rmax && oa < rarg)) { rmax = om; rarg = oa; }
    }
    double denom_d = (my_sum > 0.0f) ? static_cast<double>(my_sum) * exp(static_cast<double>(my_max) - rmax) : 0.0;
    denom_d = warp_sum(denom_d);
    const float denom = static_cast<float>(denom_d);

    double part = 0.0;
    {
        float acc = 0.0f;
        auto term = [&](float x) {
            const float pr = expf(x - rmax) / denom;
            return pr * logf(fmaxf(pr, 1e-10f));
        };
        if (sv.vec) {
            const float4* v4 = reinterpret_cast<const float4*>(sv.base);
            for (int i = threadIdx.x; i < sv.len / 4; i += kThreads) {
                const float4 v = __ldg(v4 + i);
                acc += (term(v.x) + term(v.y)) + (term(v.z) + term(v.w));
            }
        } else {
            for (int i = threadIdx.x; i < sv.len; i += kThreads) acc += term(__ldg(sv.base + i));
        }
        part = warp_sum(static_cast<double>(acc));
    }
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (lane == 0) s_part[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) tot += s_part[w];
        rs->pent[slice] = tot;
        __threadfence();
        const unsigned ticket = atomicAdd(&rs->ticket, 1u);
        s_last = (ticket == static_cast<unsigned>(p.n_slices) - 1u);
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        __threadfence();
        double h = 0.0;
        for (int s = 0; s < p.n_slices; ++s) h += *(volatile double*)&rs->pent[s];
        const float ent_f = static_cast<float>(-h);
        if (p.entropy_out != nullptr) p.entropy_out[row] = ent_f;
        if (p.needs_state) reset_decide(p, row, slot, static_cast<double>(ent_f), rarg, rs);
    }
}

// ---- kernel 3 ---------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
reset_scale_kernel(const ResetLaunch p) {
    const int row = blockIdx.y, slice = blockIdx.x;
    int slot;
    pdl_launch_dependents();
    if (!row_active(p, row, &slot)) return;
    pdl_wait_prior();
    const RowScratch* rs = p.scratch + row;
    const double temp_d = rs->temp;
    if (temp_d == 1.0) return;
    const SliceView sv = slice_of(p, row, slice);
    float* out = const_cast<float*>(sv.base);
    if (temp_d <= 1e-6) {
        const int arg = rs->argmax;
        for (int i = threadIdx.x; i < sv.len; i += kThreads)
            out[i] = (sv.first + i == arg) ? 0.0f : -INFINITY;
        return;
    }
    const float t = static_cast<float>(temp_d);
    if (sv.vec) {
        float4* v4 = reinterpret_cast<float4*>(out);
        for (int i = threadIdx.x; i < sv.len / 4; i += kThreads) {
            float4 v = v4[i];
            v.x = __fdiv_rn(v.x, t); v.y = __fdiv_rn(v.y, t);
            v.z = __fdiv_rn(v.z, t); v.w = __fdiv_rn(v.w, t);
            v4[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < sv.len; i += kThreads) out[i] = __fdiv_rn(out[i], t);
    }
}

template <typename Kern>
cudaError_t launch_pdl(Kern kern, dim3 grid, const ResetLaunch& p, bool pdl, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace

int reset_pick_slices(int B, int V) {
    const int sms = device_sm_count();
    int s = (2 * sms + B - 1) / B;              // about two CTAs per SM over all rows
    const int max_by_len = (V + 2047) / 2048;   // at least 2048 elements per slice
    if (s > max_by_len) s = max_by_len;
    if (s > kResetMaxSlices) s = kResetMaxSlices;
    if (s < 1) s = 1;
    return s;
}

cudaError_t launch_reset(ResetLaunch p, bool scale, cudaStream_t stream) {
    p.n_slices = reset_pick_slices(p.B, p.V);
    p.slice_len = ((p.V + p.n_slices - 1) / p.n_slices + 3) / 4 * 4;
    const dim3 grid(static_cast<unsigned>(p.n_slices), static_cast<unsigned>(p.B));
    cudaError_t e = launch_pdl(reset_partials_kernel, grid, p, true, stream);
    if (e != cudaSuccess) return e;
    e = launch_pdl(reset_entropy_kernel, grid, p, true, stream);
    if (e != cudaSuccess) return e;
    if (scale) e = launch_pdl(reset_scale_kernel, grid, p, true, stream);
    return e;
}

}  // namespace nvfp4r
