// Launch record and scratch layout of the ReSET step kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nvfp4r_b200.h"

namespace nvfp4r {

constexpr int kResetMaxSlices = 32;

// One record per logits row, in caller-provided (or static) scratch memory.
struct RowScratch {
    float pmax[kResetMaxSlices];    // slice max
    float psum[kResetMaxSlices];    // slice sum of exp(x - slice max)
    int parg[kResetMaxSlices];      // slice argmax (index within the row)
    double pent[kResetMaxSlices];   // slice sum of p*log(max(p,1e-10))
    double temp;                    // temperature chosen for the row
    unsigned ticket;                // arrival counter of the entropy kernel
    int argmax;                     // row argmax
};

// Hand-over slots of the single-launch step (reset_fused_kernel): 64-bit words {epoch:32 |
// payload:32}; a word counts only while its epoch equals the row's current one, so nothing is
// ever cleared. All-zero memory is a valid initial state (epoch 0, first step uses 1).
struct RowSlots {
    unsigned long long pmax[kResetMaxSlices];    // slice max (float bits)
    unsigned long long psum[kResetMaxSlices];    // slice sum of exp(x - slice max)
    unsigned long long parg[kResetMaxSlices];    // slice argmax
    unsigned long long ent_hi[kResetMaxSlices];  // slice sum of p*log(max(p,1e-10)), double, high word
    unsigned long long ent_lo[kResetMaxSlices];  //                                    low word
    unsigned long long temp;                     // chosen temperature (float bits)
    unsigned long long mode;                     // 0: divide, 1: leave untouched (T == 1), 2: one-hot at argmax
    unsigned epoch;                              // step counter of the row, advanced by its deciding CTA
    unsigned pad;
};

struct ResetLaunch {
    const float* logits;
    int64_t row_stride;
    int B, V;
    int n_slices, slice_len;
    RowScratch* scratch;
    RowSlots* slots;       // single-launch path; nullptr = three-launch path only
    nvfp4r_reset_state* states;
    const int32_t* state_slots;
    const int32_t* last_ids;
    const uint32_t* nl_bitmap;
    const uint32_t* dnl_bitmap;
    nvfp4r_reset_params params;               // the one record of the by-value entry points
    const nvfp4r_reset_params* slot_params;   // per-request records on the device, indexed by state
                                              // slot (nullptr = `params` for every row)
    int bitmap_words;                         // words between two id sets in nl_bitmap / dnl_bitmap
    nvfp4r_reset_decision* decisions;
    float* entropy_out;
    int needs_state;     // 0: entropy only
};

int reset_pick_slices(int B, int V);
cudaError_t launch_reset(ResetLaunch p, bool scale, cudaStream_t stream);
// Same step with the scratch taken from a static device array (no_alloc.cu).
cudaError_t launch_reset_static(ResetLaunch p, cudaStream_t stream);
// lm_head (bf16 weight [V, H], one token) ending in the ReSET step of that token, one launch
// (lm_head_reset.cu). `p.logits` is the output row; cudaErrorInvalidConfiguration = shape or
// residency not supported.
size_t lm_head_reset_workspace_bytes();
cudaError_t launch_lm_head_reset(const void* x, const void* weight, int H, ResetLaunch p, void* workspace,
                                 cudaStream_t stream);

}  // namespace nvfp4r
