"""FakeTensor implementations so ``torch.compile(fullgraph=True)`` traces through the
ops (reference: kernels/python/nvfp4r/_fake.py:21-43). Out-variants return None."""

from __future__ import annotations

import torch

_OUT_DTYPES = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32}


@torch.library.register_fake("nvfp4r::gemv")
def _gemv_fake(weight, weight_scale, x, x_scale, out, alpha=1.0):
    return None


@torch.library.register_fake("nvfp4r::gemm")
def _gemm_fake(A, B, SFA, SFB, C, alpha=1.0):
    return None


@torch.library.register_fake("nvfp4r::quant")
def _quant_fake(x, global_scale_inv, swizzled=False, rcp_mode=1):
    M, K = x.shape
    rows = (M + 127) // 128 * 128 if swizzled else M
    cols = (K // 16 + 3) // 4 * 4 if swizzled else K // 16
    return (x.new_empty((M, K // 2), dtype=torch.uint8),
            x.new_empty((rows, cols), dtype=torch.uint8))


@torch.library.register_fake("nvfp4r::linear")
def _linear_fake(x, global_scale_inv, weight, weight_scale_flat, alpha, out_dtype_int=0, rcp_mode=1):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=_OUT_DTYPES[out_dtype_int])


@torch.library.register_fake("nvfp4r::linear_tc")
def _linear_tc_fake(x, global_scale_inv, weight, weight_scale_swizzled, alpha, out_dtype_int=0,
                    rcp_mode=1):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=_OUT_DTYPES[out_dtype_int])


@torch.library.register_fake("nvfp4r::pack_weight")
def _pack_weight_fake(weight, weight_scale_flat):
    return weight.new_empty((weight.numel() * 9 // 8,), dtype=torch.uint8)


@torch.library.register_fake("nvfp4r::linear_packed")
def _linear_packed_fake(x, global_scale_inv, packed, N, alpha, out_dtype_int=0, rcp_mode=1):
    return x.new_empty((x.shape[0], N), dtype=_OUT_DTYPES[out_dtype_int])


@torch.library.register_fake("nvfp4r::entropy")
def _entropy_fake(logits, workspace):
    return logits.new_empty((logits.shape[0],))


@torch.library.register_fake("nvfp4r::reset_step")
def _reset_step_fake(logits, states, state_slots, last_ids, nl_bitmap, dnl_bitmap, t_high, t_low,
                     tau0, window, decisions, workspace):
    return None
