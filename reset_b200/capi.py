"""Tensor-level wrappers over the C ABI: they take ``torch`` CUDA tensors, pass raw
device pointers, sizes and the current CUDA stream to ``libnvfp4r_b200.so`` and
raise on any non-zero status. PyTorch is used for memory and streams only."""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L

_DTYPE_CODE = {torch.bfloat16: L.BF16, torch.float16: L.F16, torch.float32: L.F32}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("nvfp4r: all tensors must be CUDA tensors")


def _u8(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.uint8 else t.view(torch.uint8)


def quant(x: torch.Tensor, global_scale_inv: torch.Tensor, *, swizzled: bool = False,
          rcp_mode: int = L.RCP_EXACT):
    """bf16 [M,K] -> (codes uint8 [M,K/2], scales uint8). Flat scales are [M,K/16];
    swizzled ones [ceil(M/128)*128, ceil(K/64)*4]."""
    _need_cuda(x, global_scale_inv)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("quant: x must be bf16 [M,K] with unit inner stride")
    M, K = x.shape
    codes = torch.empty((M, K // 2), dtype=torch.uint8, device=x.device)
    if swizzled:
        shape = ((M + 127) // 128 * 128, (K // 16 + 3) // 4 * 4)
    else:
        shape = (M, K // 16)
    scales = torch.empty(shape, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        st = L.lib().nvfp4r_quant(x.data_ptr(), x.stride(0), M, K, global_scale_inv.data_ptr(),
                                  codes.data_ptr(), scales.data_ptr(),
                                  L.SF_SWIZZLED if swizzled else L.SF_FLAT, rcp_mode, _stream())
    L.check(st, "nvfp4r_quant")
    return codes, scales


def gemv_out(weight, weight_scale, x, x_scale, out, alpha: float = 1.0) -> None:
    """The reference's out-variant: 3-D operands, ``out`` [L,N] mutated in place."""
    _need_cuda(weight, weight_scale, x, x_scale, out)
    w, ws, a, a_s = _u8(weight), _u8(weight_scale), _u8(x), _u8(x_scale)
    if not (w.dim() == ws.dim() == a.dim() == a_s.dim() == 3):
        raise ValueError("gemv: inputs must be 3D [L, N_or_P, K/2_or_K/16]")
    if not (a.is_contiguous() and a_s.is_contiguous()):
        raise ValueError("gemv: x / x_scale must be contiguous")
    Lb, N, K2 = w.shape
    K = K2 * 2
    if tuple(ws.shape) != (Lb, N, K // 16):
        raise ValueError("weight_scale shape mismatch with weight")
    if a.shape[0] != Lb or a.shape[2] != K2:
        raise ValueError("x.K mismatch with weight.K")
    if a_s.shape[0] != Lb or a_s.shape[1] != a.shape[1] or a_s.shape[2] * 16 != K:
        raise ValueError("x_scale shape mismatch with x")
    if out.dtype not in _DTYPE_CODE or not out.is_contiguous() or tuple(out.shape) != (Lb, N):
        raise ValueError("out must be a contiguous [L, N] float16/bfloat16/float32 tensor")
    if w.stride(2) != 1 or ws.stride(2) != 1:
        raise ValueError("gemv: weight / weight_scale must have unit inner stride")
    with torch.cuda.device(w.device):
        st = L.lib().nvfp4r_gemv(w.data_ptr(), ws.data_ptr(), a.data_ptr(), a_s.data_ptr(),
                                 out.data_ptr(), Lb, N, K, w.stride(0), w.stride(1),
                                 ws.stride(0), ws.stride(1), a.stride(0), a_s.stride(0),
                                 float(alpha), _DTYPE_CODE[out.dtype], _stream())
    L.check(st, "nvfp4r_gemv")


def linear(x: torch.Tensor, global_scale_inv: torch.Tensor, weight: torch.Tensor,
           weight_scale_flat: torch.Tensor, alpha: float, out: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None, rcp_mode: int = L.RCP_EXACT) -> torch.Tensor:
    """Fused quantize + GEMV for M <= 16 bf16 tokens. weight [N,K/2], scales [N,K/16]."""
    _need_cuda(x, global_scale_inv, weight, weight_scale_flat, out)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("linear: x must be bf16 [M,K] with unit inner stride")
    M, K = x.shape
    w, ws = _u8(weight), _u8(weight_scale_flat)
    N = w.shape[0]
    if not (w.is_contiguous() and ws.is_contiguous()) or w.shape[1] * 2 != K \
            or ws.numel() != N * (K // 16):
        raise ValueError("linear: weight [N,K/2] and weight_scale [N,K/16] must be contiguous")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    elif tuple(out.shape) != (M, N) or not out.is_contiguous():
        raise ValueError("linear: out must be contiguous [M,N]")
    with torch.cuda.device(x.device):
        st = L.lib().nvfp4r_linear(x.data_ptr(), x.stride(0), M, K, global_scale_inv.data_ptr(),
                                   w.data_ptr(), ws.data_ptr(), N, float(alpha), out.data_ptr(),
                                   _DTYPE_CODE[out.dtype], rcp_mode, _stream())
    L.check(st, "nvfp4r_linear")
    return out


def gemm_workspace(M: int, N: int, K: int, device) -> torch.Tensor:
    """Zero-initialised scratch for the tensor-core kernel (it leaves it zeroed)."""
    n = L.lib().nvfp4r_gemm_workspace_bytes(M, N, K)
    return torch.zeros((n + 15) // 16 * 2, dtype=torch.int64, device=device)


def linear_tc(x: torch.Tensor, global_scale_inv: torch.Tensor, weight: torch.Tensor,
              weight_scale_swizzled: torch.Tensor, alpha: float, workspace: torch.Tensor,
              out_dtype: torch.dtype = torch.bfloat16, rcp_mode: int = L.RCP_EXACT) -> torch.Tensor:
    """Fused quantize + tcgen05 GEMM: bf16 [M,K] x NVFP4 weight [N,K/2] -> [M,N]."""
    _need_cuda(x, global_scale_inv, weight, weight_scale_swizzled, workspace)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("linear_tc: x must be bf16 [M,K] with unit inner stride")
    M, K = x.shape
    w, ws = _u8(weight), _u8(weight_scale_swizzled)
    N = w.shape[0]
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        st = L.lib().nvfp4r_linear_tc(x.data_ptr(), x.stride(0), M, K, global_scale_inv.data_ptr(),
                                      w.data_ptr(), ws.data_ptr(), N, float(alpha), out.data_ptr(),
                                      _DTYPE_CODE[out_dtype], rcp_mode, workspace.data_ptr(),
                                      workspace.numel() * workspace.element_size(), _stream())
    L.check(st, "nvfp4r_linear_tc")
    return out


def gemm(A, B, SFA, SFB, C: torch.Tensor, alpha: float, workspace: torch.Tensor,
         n_major: bool = True) -> None:
    """Pre-quantized tensor-core GEMM; C's buffer is written N-major (the reference's
    layout) or M-major."""
    _need_cuda(A, B, SFA, SFB, C, workspace)
    a, b, sa, sb = _u8(A), _u8(B), _u8(SFA), _u8(SFB)
    M, K2 = a.shape
    N = b.shape[0]
    with torch.cuda.device(a.device):
        st = L.lib().nvfp4r_gemm(a.data_ptr(), b.data_ptr(), sa.data_ptr(), sb.data_ptr(), C.data_ptr(),
                                 M, N, 2 * K2, float(alpha), _DTYPE_CODE[C.dtype],
                                 L.C_N_MAJOR if n_major else L.C_M_MAJOR, workspace.data_ptr(),
                                 workspace.numel() * workspace.element_size(), _stream())
    L.check(st, "nvfp4r_gemm")


def pack_weight(weight: torch.Tensor, weight_scale_flat: torch.Tensor) -> torch.Tensor:
    """[N,K/2] codes + flat [N,K/16] scales -> packed block format (uint8, N*K*9/16 bytes for K % 256 == 0;
    K % 256 == 128 is padded with half a block of zeros)."""
    _need_cuda(weight, weight_scale_flat)
    w, ws = _u8(weight).contiguous(), _u8(weight_scale_flat).contiguous()
    N, K = w.shape[0], w.shape[1] * 2
    n = L.lib().nvfp4r_packed_weight_bytes(N, K)
    if n == 0:
        raise ValueError("pack_weight: needs N % 128 == 0 and K % 128 == 0")
    packed = torch.empty(n, dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        st = L.lib().nvfp4r_pack_weight(w.data_ptr(), ws.data_ptr(), packed.data_ptr(), N, K, _stream())
    L.check(st, "nvfp4r_pack_weight")
    return packed


def packed_workspace(M: int, N: int, K: int, device) -> torch.Tensor:
    n = L.lib().nvfp4r_linear_packed_workspace_bytes(M, N, K)
    return torch.zeros((n + 15) // 16 * 2, dtype=torch.int64, device=device)


def linear_packed(x: torch.Tensor, global_scale_inv: torch.Tensor, packed: torch.Tensor, N: int,
                  alpha: float, workspace: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                  rcp_mode: int = L.RCP_EXACT, out: torch.Tensor | None = None) -> torch.Tensor:
    """Fused quantize + tensor-core linear over a packed weight: bf16 [M,K] -> [M,N]."""
    _need_cuda(x, global_scale_inv, packed, workspace)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("linear_packed: x must be bf16 [M,K] with unit inner stride")
    M, K = x.shape
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        st = L.lib().nvfp4r_linear_packed(x.data_ptr(), x.stride(0), M, K, global_scale_inv.data_ptr(),
                                          packed.data_ptr(), N, float(alpha), out.data_ptr(),
                                          _DTYPE_CODE[out.dtype], rcp_mode, workspace.data_ptr(),
                                          workspace.numel() * workspace.element_size(), _stream())
    L.check(st, "nvfp4r_linear_packed")
    return out


def linear_packed_rmsnorm(delta, residual_in: torch.Tensor, residual_out: torch.Tensor,
                          norm_weight: torch.Tensor, eps: float, global_scale_inv: torch.Tensor,
                          packed: torch.Tensor, N: int, alpha: float, workspace: torch.Tensor,
                          out_dtype: torch.dtype = torch.bfloat16, rcp_mode: int = L.RCP_APPROX,
                          out: torch.Tensor | None = None) -> torch.Tensor:
    """residual_out = residual_in + delta; out = linear(RMSNorm(residual_out) * norm_weight),
    one launch. All activations bf16 [M, K]."""
    _need_cuda(residual_in, residual_out, norm_weight, global_scale_inv, packed, workspace, delta)
    M, K = residual_in.shape
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=residual_in.device)
    pro = L.Prologue(L.PROLOGUE_ADD_RMSNORM, float(eps), None if delta is None else delta.data_ptr(),
                     residual_in.data_ptr(), residual_out.data_ptr(), norm_weight.data_ptr())
    with torch.cuda.device(residual_in.device):
        st = L.lib().nvfp4r_linear_packed_ex(C.byref(pro), None, 0, M, K, global_scale_inv.data_ptr(),
                                             packed.data_ptr(), N, float(alpha), out.data_ptr(),
                                             _DTYPE_CODE[out.dtype], rcp_mode, workspace.data_ptr(),
                                             workspace.numel() * workspace.element_size(), _stream())
    L.check(st, "nvfp4r_linear_packed_ex")
    return out


def linear_rmsnorm(delta, residual_in: torch.Tensor, residual_out: torch.Tensor, norm_weight: torch.Tensor,
                   eps: float, global_scale_inv: torch.Tensor, weight: torch.Tensor,
                   weight_scale_flat: torch.Tensor, alpha: float, out: torch.Tensor,
                   rcp_mode: int = L.RCP_APPROX) -> torch.Tensor:
    """residual_out = residual_in + delta; out = linear(RMSNorm(residual_out) * norm_weight) through the
    CUDA-core GEMV on the flat weight, one launch, one token (M = 1)."""
    _need_cuda(residual_in, residual_out, norm_weight, global_scale_inv, weight, weight_scale_flat, delta, out)
    M, K = residual_in.shape
    N = weight.shape[0]
    pro = L.Prologue(L.PROLOGUE_ADD_RMSNORM, float(eps), None if delta is None else delta.data_ptr(),
                     residual_in.data_ptr(), residual_out.data_ptr(), norm_weight.data_ptr())
    with torch.cuda.device(residual_in.device):
        st = L.lib().nvfp4r_linear_ex(C.byref(pro), None, 0, M, K, global_scale_inv.data_ptr(), weight.data_ptr(),
                                      weight_scale_flat.data_ptr(), N, float(alpha), out.data_ptr(),
                                      _DTYPE_CODE[out.dtype], rcp_mode, _stream())
    L.check(st, "nvfp4r_linear_ex")
    return out


def linear_silu(gate_up: torch.Tensor, global_scale_inv: torch.Tensor, weight: torch.Tensor,
                weight_scale_flat: torch.Tensor, alpha: float, out: torch.Tensor,
                rcp_mode: int = L.RCP_APPROX) -> torch.Tensor:
    """out = linear(silu(gate) * up) with gate_up = [1, 2K] bf16 through the CUDA-core GEMV on the
    flat weight, one launch."""
    _need_cuda(gate_up, global_scale_inv, weight, weight_scale_flat, out)
    M, K2 = gate_up.shape
    N = weight.shape[0]
    pro = L.Prologue(L.PROLOGUE_SILU_MUL, 0.0, None, None, None, None)
    with torch.cuda.device(gate_up.device):
        st = L.lib().nvfp4r_linear_ex(C.byref(pro), gate_up.data_ptr(), gate_up.stride(0), M, K2 // 2,
                                      global_scale_inv.data_ptr(), weight.data_ptr(), weight_scale_flat.data_ptr(),
                                      N, float(alpha), out.data_ptr(), _DTYPE_CODE[out.dtype], rcp_mode, _stream())
    L.check(st, "nvfp4r_linear_ex")
    return out


def linear_packed_silu(gate_up: torch.Tensor, global_scale_inv: torch.Tensor, packed: torch.Tensor, N: int,
                       alpha: float, workspace: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                       rcp_mode: int = L.RCP_APPROX, out: torch.Tensor | None = None, push=None,
                       gather: bool = False) -> torch.Tensor:
    """out = linear(silu(gate) * up) with gate_up = [M, 2K] bf16, one launch. With ``push`` (a
    ``_lib.PeerComm``) the result goes into the peers' receive memory instead of ``out``; with
    ``gather`` as well, the launch also completes the sum over the ranks into ``out``."""
    _need_cuda(gate_up, global_scale_inv, packed, workspace)
    M, K2 = gate_up.shape
    K = K2 // 2
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=gate_up.device)
    pro = L.Prologue(L.PROLOGUE_SILU_MUL, 0.0, None, None, None, None,
                     None if push is None else C.addressof(push), 1 if (gather and push is not None) else 0)
    with torch.cuda.device(gate_up.device):
        st = L.lib().nvfp4r_linear_packed_ex(C.byref(pro), gate_up.data_ptr(), gate_up.stride(0), M, K,
                                             global_scale_inv.data_ptr(), packed.data_ptr(), N, float(alpha),
                                             out.data_ptr(), _DTYPE_CODE[out.dtype], rcp_mode,
                                             workspace.data_ptr(), workspace.numel() * workspace.element_size(),
                                             _stream())
    L.check(st, "nvfp4r_linear_packed_ex")
    return out


def unswizzle_blockscale(swizzled: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    _need_cuda(swizzled)
    sw = _u8(swizzled).contiguous()
    flat = torch.empty((rows, K // 16), dtype=torch.uint8, device=sw.device)
    with torch.cuda.device(sw.device):
        st = L.lib().nvfp4r_unswizzle_blockscale(sw.data_ptr(), flat.data_ptr(), rows, K, _stream())
    L.check(st, "nvfp4r_unswizzle_blockscale")
    return flat


def swizzle_blockscale(flat: torch.Tensor) -> torch.Tensor:
    _need_cuda(flat)
    f = _u8(flat).contiguous()
    rows, cols = f.shape
    out = torch.empty(((rows + 127) // 128 * 128, (cols + 3) // 4 * 4), dtype=torch.uint8,
                      device=f.device)
    with torch.cuda.device(f.device):
        st = L.lib().nvfp4r_swizzle_blockscale(f.data_ptr(), out.data_ptr(), rows, cols * 16, _stream())
    L.check(st, "nvfp4r_swizzle_blockscale")
    return out


def reset_workspace(B: int, device) -> torch.Tensor:
    n = L.lib().nvfp4r_reset_workspace_bytes(B)
    return torch.zeros((n + 7) // 8, dtype=torch.int64, device=device)       # zeroed: it holds step counters


def entropy(logits: torch.Tensor, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 [B,V] -> fp32 [B] token entropies."""
    _need_cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("entropy: logits must be fp32 [B,V] with unit inner stride")
    B, V = logits.shape
    ws = workspace if workspace is not None else reset_workspace(B, logits.device)
    out = torch.empty(B, dtype=torch.float32, device=logits.device)
    with torch.cuda.device(logits.device):
        st = L.lib().nvfp4r_entropy(logits.data_ptr(), logits.stride(0), B, V, out.data_ptr(),
                                    ws.data_ptr(), ws.numel() * 8, _stream())
    L.check(st, "nvfp4r_entropy")
    return out


def reset_step(logits: torch.Tensor, states: torch.Tensor, params: L.ResetParams, *,
               state_slots: torch.Tensor | None = None, last_ids: torch.Tensor | None = None,
               nl_bitmap: torch.Tensor | None = None, dnl_bitmap: torch.Tensor | None = None,
               decisions: torch.Tensor | None = None, workspace: torch.Tensor) -> None:
    """One ReSET step in place on fp32 logits [B,V]. ``states`` is a uint8 tensor of
    ``sizeof(nvfp4r_reset_state)`` bytes per slot; ``decisions`` (optional) a uint8
    tensor of ``sizeof(nvfp4r_reset_decision)`` bytes per row."""
    _need_cuda(logits, states, state_slots, last_ids, nl_bitmap, dnl_bitmap, decisions, workspace)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("reset_step: logits must be fp32 [B,V] with unit inner stride")
    B, V = logits.shape
    ptr = lambda t: t.data_ptr() if t is not None else None
    with torch.cuda.device(logits.device):
        st = L.lib().nvfp4r_reset_step(logits.data_ptr(), logits.stride(0), B, V, states.data_ptr(),
                                       ptr(state_slots), ptr(last_ids), ptr(nl_bitmap),
                                       ptr(dnl_bitmap), C.byref(params), ptr(decisions),
                                       workspace.data_ptr(), workspace.numel() * workspace.element_size(),
                                       _stream())
    L.check(st, "nvfp4r_reset_step")


def reset_step_per_request(logits: torch.Tensor, states: torch.Tensor, slot_params: torch.Tensor, *,
                           state_slots: torch.Tensor | None = None, last_ids: torch.Tensor | None = None,
                           nl_bitmaps: torch.Tensor | None = None, dnl_bitmaps: torch.Tensor | None = None,
                           n_id_sets: int = 0, decisions: torch.Tensor | None = None,
                           workspace: torch.Tensor) -> None:
    """One ReSET step in place with per-request hyper-parameters: ``slot_params`` is a uint8
    device tensor of ``sizeof(nvfp4r_reset_params)`` bytes per state slot; ``nl_bitmaps`` /
    ``dnl_bitmaps`` hold ``n_id_sets`` bitmaps of ceil(V/32) int32 words each (both given, or
    neither)."""
    _need_cuda(logits, states, slot_params, state_slots, last_ids, nl_bitmaps, dnl_bitmaps, decisions, workspace)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("reset_step_per_request: logits must be fp32 [B,V] with unit inner stride")
    B, V = logits.shape
    words = (V + 31) // 32
    if n_id_sets > 0:
        for bm in (nl_bitmaps, dnl_bitmaps):
            if bm is None or bm.numel() * bm.element_size() < n_id_sets * words * 4:
                raise ValueError("reset_step_per_request: bitmaps must hold n_id_sets * ceil(V/32) words")
    ptr = lambda t: t.data_ptr() if t is not None else None
    with torch.cuda.device(logits.device):
        st = L.lib().nvfp4r_reset_step_per_request(
            logits.data_ptr(), logits.stride(0), B, V, states.data_ptr(), ptr(state_slots), ptr(last_ids),
            ptr(nl_bitmaps), ptr(dnl_bitmaps), int(n_id_sets), slot_params.data_ptr(), ptr(decisions),
            workspace.data_ptr(), workspace.numel() * workspace.element_size(), _stream())
    L.check(st, "nvfp4r_reset_step_per_request")


def lm_head_reset_workspace(device) -> torch.Tensor:
    """All-zero workspace of :func:`lm_head_reset_step` for one token row."""
    return torch.zeros((L.lib().nvfp4r_lm_head_reset_workspace_bytes() + 7) // 8, dtype=torch.int64, device=device)


def lm_head_reset_step(x: torch.Tensor, weight: torch.Tensor, logits: torch.Tensor, states: torch.Tensor,
                       slot_params: torch.Tensor, *, state_slots: torch.Tensor | None = None,
                       last_ids: torch.Tensor | None = None, nl_bitmaps: torch.Tensor | None = None,
                       dnl_bitmaps: torch.Tensor | None = None, n_id_sets: int = 0,
                       decisions: torch.Tensor | None = None, workspace: torch.Tensor) -> None:
    """lm_head (bf16 ``weight`` [V,H] times the token ``x`` [H] or [1,H]) ending in the ReSET step of
    that token, one launch: ``logits`` (fp32 [V] or [1,V]) receives W.x divided by the chosen
    temperature. The ReSET arguments are those of :func:`reset_step_per_request` with B = 1."""
    _need_cuda(x, weight, logits, states, slot_params, state_slots, last_ids, nl_bitmaps, dnl_bitmaps, decisions,
               workspace)
    if weight.dtype != torch.bfloat16 or weight.dim() != 2 or not weight.is_contiguous():
        raise ValueError("lm_head_reset_step: weight must be contiguous bf16 [V,H]")
    V, H = weight.shape
    if x.dtype != torch.bfloat16 or x.numel() != H or not x.is_contiguous():
        raise ValueError("lm_head_reset_step: x must be contiguous bf16 with H elements")
    if logits.dtype != torch.float32 or logits.numel() != V or not logits.is_contiguous():
        raise ValueError("lm_head_reset_step: logits must be contiguous fp32 with V elements")
    words = (V + 31) // 32
    if n_id_sets > 0:
        for bm in (nl_bitmaps, dnl_bitmaps):
            if bm is None or bm.numel() * bm.element_size() < n_id_sets * words * 4:
                raise ValueError("lm_head_reset_step: bitmaps must hold n_id_sets * ceil(V/32) words")
    ptr = lambda t: t.data_ptr() if t is not None else None
    with torch.cuda.device(logits.device):
        st = L.lib().nvfp4r_lm_head_reset_step(
            x.data_ptr(), weight.data_ptr(), logits.data_ptr(), V, H, states.data_ptr(), ptr(state_slots),
            ptr(last_ids), ptr(nl_bitmaps), ptr(dnl_bitmaps), int(n_id_sets), slot_params.data_ptr(),
            ptr(decisions), workspace.data_ptr(), workspace.numel() * workspace.element_size(), _stream())
    L.check(st, "nvfp4r_lm_head_reset_step")


def sample(logits: torch.Tensor, draws: torch.Tensor, *, seed: int = 0,
           last_ids: torch.Tensor | None = None, out: torch.Tensor | None = None,
           top_k: int = 0, top_p: float = 1.0, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """One id per row drawn from softmax(logits) on the device (Gumbel-max). ``draws`` is an
    int64 [B] counter tensor (zero at request start, advanced by the call); ``last_ids``
    (int32 [B,2], optional) gets the new id shifted in. Returns int32 [B]. ``top_k`` (> 0) and
    ``top_p`` (< 1) restrict the draw to vLLM's top-k / nucleus set; they need ``workspace``
    (:func:`sample_workspace`)."""
    _need_cuda(logits, draws, last_ids, out, workspace)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("sample: logits must be fp32 [B,V] with unit inner stride")
    B, V = logits.shape
    if draws.dtype != torch.int64 or draws.numel() < B:
        raise ValueError("sample: draws must be int64 [B]")
    if last_ids is not None and (last_ids.dtype != torch.int32 or last_ids.numel() < 2 * B
                                 or not last_ids.is_contiguous()):
        raise ValueError("sample: last_ids must be contiguous int32 [B,2]")
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    truncated = (0 < int(top_k) < V) or float(top_p) < 1.0
    if truncated and workspace is None:
        raise ValueError("sample: top_k / top_p need a workspace (capi.sample_workspace)")
    with torch.cuda.device(logits.device):
        if truncated:
            st = L.lib().nvfp4r_sample_top_k_top_p(
                logits.data_ptr(), logits.stride(0), B, V, int(top_k), float(top_p), int(seed) & (2 ** 64 - 1),
                draws.data_ptr(), None if last_ids is None else last_ids.data_ptr(), out.data_ptr(),
                workspace.data_ptr(), workspace.numel() * workspace.element_size(), _stream())
        else:
            st = L.lib().nvfp4r_sample(logits.data_ptr(), logits.stride(0), B, V, int(seed) & (2 ** 64 - 1),
                                       draws.data_ptr(), None if last_ids is None else last_ids.data_ptr(),
                                       out.data_ptr(), _stream())
    L.check(st, "nvfp4r_sample")
    return out


def sample_workspace(B: int, device) -> torch.Tensor:
    """Zeroed scratch of ``sample(..., top_k=, top_p=)`` for up to ``B`` rows."""
    n = L.lib().nvfp4r_sample_workspace_bytes(B)
    return torch.zeros((n + 7) // 8, dtype=torch.int64, device=device)


def linear_push(x: torch.Tensor, global_scale_inv: torch.Tensor, weight: torch.Tensor,
                weight_scale_flat: torch.Tensor, alpha: float, push, out: torch.Tensor,
                rcp_mode: int = L.RCP_APPROX) -> torch.Tensor:
    """Row-parallel shard small enough for the CUDA-core GEMV (one token): the GEMV's own launch
    pushes its bf16 result into the peers' receive memory (``push``: a ``_lib.PeerComm``) and sums
    the ranks' contributions into ``out``; no all-reduce launch follows. One GPU per rank."""
    _need_cuda(x, global_scale_inv, weight, weight_scale_flat, out)
    M, K = x.shape
    w, ws = _u8(weight), _u8(weight_scale_flat)
    N = w.shape[0]
    if M != 1 or out.dtype != torch.bfloat16 or tuple(out.shape) != (1, N) or not out.is_contiguous():
        raise ValueError("linear_push: one token, out bf16 [1,N] contiguous")
    pro = L.Prologue(L.PROLOGUE_NONE, 0.0, None, None, None, None, C.addressof(push), 1)
    with torch.cuda.device(x.device):
        st = L.lib().nvfp4r_linear_ex(C.byref(pro), x.data_ptr(), x.stride(0), M, K, global_scale_inv.data_ptr(),
                                      w.data_ptr(), ws.data_ptr(), N, float(alpha), out.data_ptr(),
                                      _DTYPE_CODE[out.dtype], rcp_mode, _stream())
    L.check(st, "nvfp4r_linear_ex")
    return out


def linear_packed_push(x: torch.Tensor, global_scale_inv: torch.Tensor, packed: torch.Tensor, N: int,
                       alpha: float, workspace: torch.Tensor, push, out: torch.Tensor,
                       rcp_mode: int = L.RCP_APPROX, gather: bool = False) -> torch.Tensor:
    """Row-parallel linear whose bf16 result is pushed into the peers' receive memory tile by
    tile (``push``: a ``_lib.PeerComm``). With ``gather`` the same launch also completes the
    sum into ``out`` (one GPU per rank required); without it ``out`` is only written by the
    gather half of the all-reduce that must follow."""
    _need_cuda(x, global_scale_inv, packed, workspace, out)
    M, K = x.shape
    pro = L.Prologue(L.PROLOGUE_NONE, 0.0, None, None, None, None, C.addressof(push), 1 if gather else 0)
    with torch.cuda.device(x.device):
        st = L.lib().nvfp4r_linear_packed_ex(C.byref(pro), x.data_ptr(), x.stride(0), M, K,
                                             global_scale_inv.data_ptr(), packed.data_ptr(), N, float(alpha),
                                             out.data_ptr(), _DTYPE_CODE[out.dtype], rcp_mode,
                                             workspace.data_ptr(), workspace.numel() * workspace.element_size(),
                                             _stream())
    L.check(st, "nvfp4r_linear_packed_ex")
    return out
