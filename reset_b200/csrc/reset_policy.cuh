// The per-request ReSET policy as device functions: hyper-parameter lookup, step-boundary test
// and the temperature decision with its bookkeeping (reference logits_processor.py:62-134).
// Shared by the stand-alone step kernels and by the lm_head kernel that ends in the same step.
#pragma once

#include "reset_kernels.h"

namespace nvfp4r {

// The hyper-parameters of a row: the request's own record when the caller passed per-request
// records (indexed by state slot), else the launch's single record.
__device__ __forceinline__ nvfp4r_reset_params reset_params_of(const ResetLaunch& p, int slot) {
    nvfp4r_reset_params prm = p.params;
    if (p.slot_params != nullptr) {
        prm = p.slot_params[slot];
        prm.window = min(max(prm.window, 1), NVFP4R_RESET_MAX_WINDOW);
    }
    return prm;
}

// Step boundary of a row: the last generated id contains a double newline, or the last two are
// both single newlines (reference logits_processor.py:91-99).
__device__ inline bool reset_boundary(const ResetLaunch& p, int row, int id_set) {
    bool boundary = false;
    if (p.last_ids != nullptr) {
        const int prev = p.last_ids[2 * row], last = p.last_ids[2 * row + 1];
        const int64_t set_off = static_cast<int64_t>(id_set) * p.bitmap_words;
        auto in_set = [&](const uint32_t* bm, int id) {
            return bm != nullptr && id >= 0 && id < p.V && ((bm[set_off + (id >> 5)] >> (id & 31)) & 1u);
        };
        if (last >= 0) {
            if (in_set(p.dnl_bitmap, last)) boundary = true;
            else if (prev >= 0 && in_set(p.nl_bitmap, last) && in_set(p.nl_bitmap, prev)) boundary = true;
        }
    }
    return boundary;
}

// The state machine of one request, run by one thread. `st` may be the record in global
// memory or a copy of it in shared memory.
__device__ inline void reset_decide_on(const ResetLaunch& p, const nvfp4r_reset_params& prm, int row,
                                       nvfp4r_reset_state* st, bool boundary, double ent, int argmax,
                                       RowScratch* rs) {
    const int w = prm.window;
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
    const double thr = high ? h_step : prm.tau0;
    const double temp = (ent >= thr) ? prm.t_high : prm.t_low;

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

__device__ inline void reset_decide(const ResetLaunch& p, int row, int slot, double ent, int argmax, RowScratch* rs) {
    const nvfp4r_reset_params prm = reset_params_of(p, slot);
    reset_decide_on(p, prm, row, p.states + slot, reset_boundary(p, row, prm.id_set), ent, argmax, rs);
}

}  // namespace nvfp4r
