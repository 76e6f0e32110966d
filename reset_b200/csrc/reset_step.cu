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
#include "status_mirror.cuh"
#include "nvfp4_ptx.cuh"
#include "reset_kernels.h"
#include "reset_policy.cuh"

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

// ---- kernel 2 ---------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
reset_entropy_kernel(const ResetLaunch p) {
    const int row = blockIdx.y, slice = blockIdx.x;
    int slot;
    pdl_launch_dependents();
    pdl_wait_prior();
    if (!row_active(p, row, &slot)) return;
    const SliceView sv = slice_of(p, row, slice);
    RowScratch* rs = p.scratch + row;
    __shared__ double s_part[kThreads / 32];
    __shared__ bool s_last;

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
    pdl_wait_prior();
    if (!row_active(p, row, &slot)) return;
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

// ---- the whole step in ONE launch ----------------------------------------------------
// Grid (n_slices, B), all CTAs resident at once. Every CTA keeps its slice of the row in
// registers from the first load to the final store (the logits are read from memory once
// and written once), and the three hand-overs that were kernel boundaries are now slot
// exchanges between the CTAs of a row:
//   slice (max, sum exp, argmax)  -> every CTA of the row   (row max, denominator)
//   slice entropy partial         -> the CTA of slice 0     (state machine, temperature)
//   temperature                   -> every CTA of the row   (in-place division)
// Polls are bounded; a CTA that gives up sets the status word and leaves its slice untouched.
// (Keeping the slice in shared memory with rolled loops over it measured slower: 14.6 us
// against 12.2 us per step at B = 1.)
constexpr int kFusedPerThread = 5;                     // float4 per thread
constexpr int kFusedMaxSlice = kFusedPerThread * 4 * kThreads;   // 5120 elements per CTA
constexpr uint32_t kResetPollLimit = 4000000u;

__device__ int g_reset_status = 0;

__device__ __forceinline__ void rs_publish(unsigned long long* slot, unsigned epoch, uint32_t payload) {
    const unsigned long long w = (static_cast<unsigned long long>(epoch) << 32) | payload;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(slot), "l"(w) : "memory");
}
__device__ __forceinline__ bool rs_poll(const unsigned long long* slot, unsigned epoch, uint32_t* payload) {
    for (uint32_t it = 0; it <= kResetPollLimit; ++it) {
        unsigned long long w;
        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(slot) : "memory");
        if (static_cast<unsigned>(w >> 32) == epoch) {
            *payload = static_cast<uint32_t>(w);
            return true;
        }
    }
    return false;
}

__global__ void __launch_bounds__(kThreads)
reset_fused_kernel(const ResetLaunch p, const int scale) {
    __shared__ float s_f[kThreads / 32];
    __shared__ int s_i[kThreads / 32];
    __shared__ double s_d[kThreads / 32];
    __shared__ float s_pmax[kResetMaxSlices], s_psum[kResetMaxSlices];
    __shared__ int s_parg[kResetMaxSlices];
    __shared__ uint32_t s_hi[kResetMaxSlices], s_lo[kResetMaxSlices];
    __shared__ uint32_t s_word[2];
    __shared__ int s_fail;
    __shared__ __align__(8) nvfp4r_reset_state s_state;        // slice 0 only: the request's record
    __shared__ int s_boundary;
    __shared__ __align__(8) nvfp4r_reset_params s_prm;
    pdl_launch_dependents();
    const int row = blockIdx.y, slice = blockIdx.x;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    int slot;
    // The wait comes before anything is read and before any return: completion of this grid
    // must imply completion of the kernel before it for whatever is launched next.
    pdl_wait_prior();
    if (!row_active(p, row, &slot)) return;
    if (threadIdx.x == 0) s_fail = 0;
    RowSlots* sl = p.slots + row;
    const unsigned epoch = *reinterpret_cast<volatile unsigned*>(&sl->epoch) + 1u;
    const SliceView sv = slice_of(p, row, slice);
    const int n4 = sv.len / 4;                         // the launcher guarantees sv.vec and the size bound
    constexpr int kStateWords = static_cast<int>(sizeof(nvfp4r_reset_state) / 8);
    if (slice == 0 && p.needs_state) {
        // the record and the boundary test do not depend on this step's logits: fetch them now,
        // so that the deciding thread later works on shared memory only
        if (threadIdx.x < kStateWords)
            reinterpret_cast<unsigned long long*>(&s_state)[threadIdx.x] =
                reinterpret_cast<const unsigned long long*>(p.states + slot)[threadIdx.x];
        if (threadIdx.x == kThreads - 1) {
            s_prm = reset_params_of(p, slot);
            s_boundary = reset_boundary(p, row, s_prm.id_set) ? 1 : 0;
        }
    }

    // ---- load the slice once; slice max / argmax / sum exp --------------------------------
    float4 x[kFusedPerThread];
    float vmax = -INFINITY;
    int varg = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kFusedPerThread; ++j) {
        const int i = threadIdx.x + j * kThreads;
        if (i < n4) x[j] = __ldg(reinterpret_cast<const float4*>(sv.base) + i);
    }
#pragma unroll
    for (int j = 0; j < kFusedPerThread; ++j) {
        const int i = threadIdx.x + j * kThreads;
        if (i < n4) {
            const float e[4] = {x[j].x, x[j].y, x[j].z, x[j].w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (e[k] > vmax) { vmax = e[k]; varg = sv.first + 4 * i + k; }
        }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, vmax, s);
        const int oa = __shfl_xor_sync(0xffffffffu, varg, s);
        if (om > vmax || (om == vmax && oa < varg)) { vmax = om; varg = oa; }
    }
    if (lane == 0) { s_f[warp] = vmax; s_i[warp] = varg; }
    __syncthreads();
    float bmax = s_f[0];
    int barg = s_i[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w)
        if (s_f[w] > bmax || (s_f[w] == bmax && s_i[w] < barg)) { bmax = s_f[w]; barg = s_i[w]; }
    __syncthreads();
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < kFusedPerThread; ++j)
        if (threadIdx.x + j * kThreads < n4)
            sum += expf(x[j].x - bmax) + expf(x[j].y - bmax) + expf(x[j].z - bmax) + expf(x[j].w - bmax);
    sum = warp_sum(sum);
    if (lane == 0) s_f[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) tot += s_f[w];
        rs_publish(&sl->pmax[slice], epoch, __float_as_uint(sv.len > 0 ? bmax : -INFINITY));
        rs_publish(&sl->psum[slice], epoch, __float_as_uint(sv.len > 0 ? tot : 0.0f));
        rs_publish(&sl->parg[slice], epoch, static_cast<uint32_t>(barg));
    }

    // ---- every CTA: all slices' partials -> row max, argmax, denominator ---------------------
    // one thread per slot: all polls of the row are in flight at once
    if (threadIdx.x < 3 * p.n_slices) {
        const int which = threadIdx.x / p.n_slices, idx = threadIdx.x - which * p.n_slices;
        const unsigned long long* src = which == 0 ? &sl->pmax[idx] : which == 1 ? &sl->psum[idx] : &sl->parg[idx];
        uint32_t v = 0;
        if (!rs_poll(src, epoch, &v)) s_fail = 1;
        if (which == 0) s_pmax[idx] = __uint_as_float(v);
        else if (which == 1) s_psum[idx] = __uint_as_float(v);
        else s_parg[idx] = static_cast<int>(v);
    }
    __syncthreads();
    if (s_fail) {
        if (threadIdx.x == 0) report_timeout(&g_reset_status, 5);
        return;
    }
    // lane s owns slice s; fixed shuffle trees: every warp of every CTA computes the same bits
    float rmax = (lane < p.n_slices) ? s_pmax[lane] : -INFINITY;
    int rarg = (lane < p.n_slices) ? s_parg[lane] : 0x7fffffff;
    const float my_max = rmax;
    const float my_sum = (lane < p.n_slices) ? s_psum[lane] : 0.0f;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, rmax, s);
        const int oa = __shfl_xor_sync(0xffffffffu, rarg, s);
        if (om > rmax || (om == rmax && oa < rarg)) { rmax = om; rarg = oa; }
    }
    double denom_d = (my_sum > 0.0f) ? static_cast<double>(my_sum) * exp(static_cast<double>(my_max) - rmax) : 0.0;
    denom_d = warp_sum(denom_d);
    const float denom = static_cast<float>(denom_d);

    // ---- slice entropy partial -------------------------------------------------------------------
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < kFusedPerThread; ++j) {
        if (threadIdx.x + j * kThreads < n4) {
            const float e[4] = {x[j].x, x[j].y, x[j].z, x[j].w};
            float t4[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float pr = expf(e[k] - rmax) / denom;
                t4[k] = pr * logf(fmaxf(pr, 1e-10f));
            }
            acc += (t4[0] + t4[1]) + (t4[2] + t4[3]);
        }
    }
    const double part = warp_sum(static_cast<double>(acc));
    if (lane == 0) s_d[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) tot += s_d[w];
        const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(tot));
        rs_publish(&sl->ent_hi[slice], epoch, static_cast<uint32_t>(bits >> 32));
        rs_publish(&sl->ent_lo[slice], epoch, static_cast<uint32_t>(bits));
    }

    // ---- the CTA of slice 0 decides ------------------------------------------------------------
    if (slice == 0) {
        __syncthreads();
        if (threadIdx.x < 2 * p.n_slices) {
            const int which = threadIdx.x / p.n_slices, idx = threadIdx.x - which * p.n_slices;
            uint32_t v = 0;
            if (!rs_poll(which == 0 ? &sl->ent_hi[idx] : &sl->ent_lo[idx], epoch, &v)) s_fail = 1;
            if (which == 0) s_hi[idx] = v;
            else s_lo[idx] = v;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            if (s_fail) {
                report_timeout(&g_reset_status, 5);
            } else {
                double h = 0.0;
                for (int s = 0; s < p.n_slices; ++s) {                 // slice order, like the three-launch path
                    const unsigned long long bits = (static_cast<unsigned long long>(s_hi[s]) << 32) | s_lo[s];
                    h += __longlong_as_double(static_cast<long long>(bits));
                }
                const float ent_f = static_cast<float>(-h);
                if (p.entropy_out != nullptr) p.entropy_out[row] = ent_f;
                float temp_f = 1.0f;
                uint32_t mode = 1u;
                if (p.needs_state) {
                    RowScratch* rs = p.scratch + row;
                    reset_decide_on(p, s_prm, row, &s_state, s_boundary != 0, static_cast<double>(ent_f), rarg, rs);
                    const double temp_d = rs->temp;
                    temp_f = static_cast<float>(temp_d);
                    mode = (temp_d == 1.0) ? 1u : (temp_d <= 1e-6 ? 2u : 0u);
                }
                rs_publish(&sl->temp, epoch, __float_as_uint(temp_f));
                rs_publish(&sl->mode, epoch, mode);
            }
            // every CTA of the row has read the epoch (it published with it): advance
            *reinterpret_cast<volatile unsigned*>(&sl->epoch) = epoch;
        }
        if (p.needs_state) {
            __syncthreads();
            if (threadIdx.x < kStateWords)
                reinterpret_cast<unsigned long long*>(p.states + slot)[threadIdx.x] =
                    reinterpret_cast<const unsigned long long*>(&s_state)[threadIdx.x];
        }
    }
    if (!scale) return;

    // ---- temperature -> in-place scaling -----------------------------------------------------------
    if (threadIdx.x < 2) {
        uint32_t v = threadIdx.x;                                      // on a time-out: mode 1, leave the slice alone
        if (!rs_poll(threadIdx.x == 0 ? &sl->temp : &sl->mode, epoch, &v)) {
            report_timeout(&g_reset_status, 5);
            v = threadIdx.x;
        }
        s_word[threadIdx.x] = v;
    }
    __syncthreads();
    const uint32_t mode = s_word[1];
    if (mode == 1u) return;                                            // T == 1: x / 1 == x
    const float t = __uint_as_float(s_word[0]);
    float4* out = reinterpret_cast<float4*>(const_cast<float*>(sv.base));
#pragma unroll
    for (int j = 0; j < kFusedPerThread; ++j) {
        const int i = threadIdx.x + j * kThreads;
        if (i < n4) {
            float4 v = x[j];
            if (mode == 2u) {
                const int b0 = sv.first + 4 * i;
                v.x = (b0 == rarg) ? 0.0f : -INFINITY;
                v.y = (b0 + 1 == rarg) ? 0.0f : -INFINITY;
                v.z = (b0 + 2 == rarg) ? 0.0f : -INFINITY;
                v.w = (b0 + 3 == rarg) ? 0.0f : -INFINITY;
            } else {
                v.x = __fdiv_rn(v.x, t); v.y = __fdiv_rn(v.y, t);
                v.z = __fdiv_rn(v.z, t); v.w = __fdiv_rn(v.w, t);
            }
            out[i] = v;
        }
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

// The single-launch path needs: every CTA of the grid resident at once (CTAs of a row wait
// for one another), 16-byte aligned slices of at most kFusedMaxSlice elements. Otherwise three
// launches.
static bool fused_plan(const ResetLaunch& p, int* n_slices, int* slice_len) {
    if (p.slots == nullptr) return false;
    if ((reinterpret_cast<uintptr_t>(p.logits) & 15) || (p.row_stride % 4) || (p.V % 4)) return false;
    constexpr int kMaxSlice = kFusedMaxSlice;
    int n = reset_pick_slices(p.B, p.V);
    const int need = (p.V + kMaxSlice - 1) / kMaxSlice;
    if (n < need) n = need;
    if (n > kResetMaxSlices) return false;
    static int per_sm = -1;
    if (per_sm < 0) {
        int v = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, reset_fused_kernel, kThreads, 0) != cudaSuccess) v = 0;
        per_sm = v;
    }
    if (static_cast<long long>(p.B) * n > static_cast<long long>(per_sm) * device_sm_count()) return false;
    const int len = ((p.V + n - 1) / n + 3) / 4 * 4;
    if (len > kMaxSlice) return false;
    *n_slices = n;
    *slice_len = len;
    return true;
}

cudaError_t launch_reset(ResetLaunch p, bool scale, cudaStream_t stream) {
    int n = 0, len = 0;
    if (fused_plan(p, &n, &len)) {
        p.n_slices = n;
        p.slice_len = len;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(n), static_cast<unsigned>(p.B));
        cfg.blockDim = dim3(kThreads);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, reset_fused_kernel, p, scale ? 1 : 0);
    }
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

cudaError_t set_status_mirror_reset(int* p) { return set_status_mirror_here(p); }

cudaError_t read_and_clear_reset_status(int* flag) {
    cudaError_t e = cudaMemcpyFromSymbol(flag, g_reset_status, sizeof(int));
    if (e != cudaSuccess) return e;
    const int zero = 0;
    return cudaMemcpyToSymbol(g_reset_status, &zero, sizeof(int));
}

}  // namespace nvfp4r
