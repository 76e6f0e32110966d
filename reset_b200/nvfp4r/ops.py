"""Convenience wrappers around ``torch.ops.nvfp4r.*`` (reference:
kernels/python/nvfp4r/ops.py:23-88). Integrations should call the ops directly so
the calls stay traceable."""

from __future__ import annotations

from typing import Optional

import torch


def _ensure_3d(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dim() == 3:
        return t
    if t.dim() == 2:
        return t.unsqueeze(0)
    raise ValueError(f"{name}: expected 2D or 3D tensor, got {t.dim()}D")


def gemv(weight, weight_scale, x, x_scale, out: Optional[torch.Tensor] = None,
         alpha: float = 1.0) -> torch.Tensor:
    """``y = alpha * W @ x`` on pre-quantized NVFP4 operands (ops.py:23-58).

    weight [L,N,K/2] u8, weight_scale [L,N,K/16] u8 (e4m3), x [L,P,K/2] (row 0 of P
    is read), x_scale [L,P,K/16], out optional [L,N] fp16/bf16. 2-D inputs gain a
    leading L=1. A weight expanded over L (stride 0) is streamed once for all L."""
    w, ws = _ensure_3d(weight, "weight"), _ensure_3d(weight_scale, "weight_scale")
    a, a_s = _ensure_3d(x, "x"), _ensure_3d(x_scale, "x_scale")
    if out is None:
        out = torch.empty((w.shape[0], w.shape[1]), dtype=torch.float16, device=w.device)
    torch.ops.nvfp4r.gemv(w, ws, a, a_s, out, alpha)
    return out


def gemm(A, B, SFA, SFB, C, alpha: float = 1.0) -> torch.Tensor:
    """``C = alpha * A @ B^T`` on the tensor cores (ops.py:62-88). The kernel writes
    ``C``'s buffer N-major; the returned view is the [M,N] result."""
    M, N = C.shape
    torch.ops.nvfp4r.gemm(A, B, SFA, SFB, C, alpha)
    return C.view(N, M).transpose(0, 1)


def quant(x: torch.Tensor, global_scale_inv: torch.Tensor, swizzled: bool = False,
          rcp_mode: int = 1):
    """bf16 [M,K] -> (codes [M,K/2] u8, e4m3 scales u8), the op the reference borrows
    from vLLM (vllm_integration.py:213). ``rcp_mode`` 1 matches that op bit for bit,
    0 uses IEEE division."""
    return torch.ops.nvfp4r.quant(x, global_scale_inv, swizzled, rcp_mode)


def linear(x: torch.Tensor, global_scale_inv: torch.Tensor, weight: torch.Tensor,
           weight_scale_flat: torch.Tensor, alpha: float, out_dtype: torch.dtype = torch.bfloat16,
           rcp_mode: int = 1) -> torch.Tensor:
    """Quantize up to 16 bf16 tokens and multiply by one NVFP4 weight in one launch."""
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[out_dtype]
    return torch.ops.nvfp4r.linear(x, global_scale_inv, weight, weight_scale_flat, alpha, code, rcp_mode)


def pack_weight(weight: torch.Tensor, weight_scale_flat: torch.Tensor) -> torch.Tensor:
    """Re-lay a weight [N,K/2] + flat scales [N,K/16] out once for the tensor-core path."""
    return torch.ops.nvfp4r.pack_weight(weight, weight_scale_flat)


def linear_packed(x: torch.Tensor, global_scale_inv: torch.Tensor, packed: torch.Tensor, N: int,
                  alpha: float, out_dtype: torch.dtype = torch.bfloat16, rcp_mode: int = 1) -> torch.Tensor:
    """Quantize M bf16 tokens and multiply by a packed NVFP4 weight on the tensor cores."""
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[out_dtype]
    return torch.ops.nvfp4r.linear_packed(x, global_scale_inv, packed, N, alpha, code, rcp_mode)


def use_gemv(M: int, N: int, K: int, gemv_max_m: int) -> bool:
    """The measured crossover: True when the CUDA-core GEMV is the faster path."""
    from . import _config
    if M > gemv_max_m or M not in _config.GEMV_MAX_WEIGHT_BYTES:
        return False
    if K % 32 or K < _config.GEMV_MIN_K:
        return False
    if M > 1 and K % 256:
        return False     # above one token the ring kernel is the GEMV, and it wants K % 256 == 0
    ring = _config.GEMV_RING_WARPS
    if 4 * ring < N <= 5 * ring and K > _config.GEMV_SHORT_ROW_K:
        return False
    return N * K * 9 // 16 <= _config.GEMV_MAX_WEIGHT_BYTES[M]


_OUT_WORKSPACE: dict = {}          # device -> zeroed split-K workspace of the out= path
_OUT_WORKSPACE_BYTES = int(__import__("os").environ.get("NVFP4R_WORKSPACE_MB", "128")) << 20


def _out_workspace(device, nbytes: int) -> torch.Tensor:
    """The split-K slots of ``linear_auto(..., out=)``: one buffer per device, allocated at the
    first call with a fixed size (``NVFP4R_WORKSPACE_MB``, default 128) and never replaced, so a
    pointer recorded in a CUDA graph stays valid. A larger request, or a first call inside a
    stream capture, raises instead of re-allocating."""
    ws = _OUT_WORKSPACE.get(device)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("nvfp4r.linear_auto: the first call on a device allocates the split-K "
                               "scratch; make it before capturing a CUDA graph")
        ws = torch.zeros(_OUT_WORKSPACE_BYTES // 8, dtype=torch.int64, device=device)
        _OUT_WORKSPACE[device] = ws
    if ws.numel() * 8 < nbytes:
        raise RuntimeError(f"nvfp4r.linear_auto: this shape needs {nbytes} bytes of split-K scratch, the "
                           f"fixed buffer holds {ws.numel() * 8}; set NVFP4R_WORKSPACE_MB before the first call")
    return ws


def linear_auto(x, global_scale_inv, weight, weight_scale_flat, packed, N: int, alpha: float,
                out_dtype: torch.dtype = torch.bfloat16, rcp_mode: int = 1,
                out: Optional[torch.Tensor] = None, reduce=None) -> torch.Tensor:
    """One decode linear through whichever kernel the measured crossover picks. ``packed``
    may be None (shape outside the tensor-core kernel's N % 128 / K % 128). With ``out`` (a
    contiguous ``[M, N]`` tensor) the result is written there and nothing is allocated: the
    out-variant convention of the reference's raw ops (kernels/csrc/bindings.cpp:27-84).
    ``reduce`` (a ``reset_b200.comm.PeerAllReduce``) makes this a row-parallel linear of a
    tensor-parallel layer: the result is summed over the ranks, with the first half of the
    exchange running in the tensor-core kernel's epilogue where that kernel is chosen."""
    from . import _config
    M, K = x.shape
    gemv = packed is None or (weight is not None and use_gemv(M, N, K, _config.GEMV_MAX_M))
    if reduce is not None and reduce.world > 1:
        from .. import _lib as L
        from .. import capi
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        if gemv:
            # a shard small enough for the GEMV: push and sum inside its own launch where that form
            # exists (one token, K % 256 == 0, even N) and the width allows it, else GEMV + one
            # all-reduce launch
            if M == 1 and K % 256 == 0 and N % 2 == 0 and packed is not None and _config.fused_gather(reduce.world):
                return capi.linear_push(x, global_scale_inv, weight, weight_scale_flat, alpha, reduce.comm, out,
                                        rcp_mode=rcp_mode)
            capi.linear(x, global_scale_inv, weight, weight_scale_flat, alpha, out=out, rcp_mode=rcp_mode)
            return reduce.all_reduce_(out)
        ws = _out_workspace(x.device, L.lib().nvfp4r_linear_packed_workspace_bytes(M, N, K))
        # push in the epilogue and, in the same launch, the sum over the ranks (one GPU per rank)
        if M <= 32 and _config.fused_gather(reduce.world):
            return capi.linear_packed_push(x, global_scale_inv, packed, N, alpha, ws, reduce.comm, out,
                                           rcp_mode=rcp_mode, gather=True)
        capi.linear_packed_push(x, global_scale_inv, packed, N, alpha, ws, reduce.comm, out, rcp_mode=rcp_mode)
        return reduce.gather_(out)
    if out is None:
        if gemv:
            return linear(x, global_scale_inv, weight, weight_scale_flat, alpha, out_dtype, rcp_mode)
        return linear_packed(x, global_scale_inv, packed, N, alpha, out_dtype, rcp_mode)
    from .. import _lib as L
    from .. import capi
    if gemv:
        return capi.linear(x, global_scale_inv, weight, weight_scale_flat, alpha, out=out, rcp_mode=rcp_mode)
    ws = _out_workspace(x.device, L.lib().nvfp4r_linear_packed_workspace_bytes(M, N, K))
    return capi.linear_packed(x, global_scale_inv, packed, N, alpha, ws, rcp_mode=rcp_mode, out=out)
