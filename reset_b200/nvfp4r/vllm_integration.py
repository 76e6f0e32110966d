"""vLLM adapter for the nvfp4r kernels: same entry points as the reference's
``nvfp4r.vllm_integration`` (kernels/python/nvfp4r/vllm_integration.py):

* :func:`apply_nvfp4r_linear` (reference :448-496) - the hot path, one custom-op
  dispatch per linear;
* :func:`prime_nvfp4r_caches` (reference :359-396) - one-shot per-layer preparation;
* :func:`_unswizzle_blockscale` (reference :99-117).

Differences from the reference, all inside the dispatch:

* every decode batch is ONE launch per 32 rows. Below the measured crossover
  (``gemv_max_m`` and a weight-size bound, ``_config.GEMV_MAX_WEIGHT_BYTES``) that launch
  is ``torch.ops.nvfp4r.linear`` (quantize + CUDA-core GEMV fused, instead of
  ``scaled_fp4_quant`` + ``expand`` + ``empty`` + ``nvfp4r.gemv``); above it it is
  ``torch.ops.nvfp4r.linear_packed`` (quantize + tcgen05 block-scaled MMA over a weight
  re-laid out once per layer), for any M, written M-major: no padding to 64 rows, no
  transpose/contiguous copy.
* The dispatch is the operator ``torch.ops.vllm.nvfp4r_linear`` (reference :342-353) with a
  fake implementation, so a compiled forward holds one node per linear and M is read at run
  time.
* The CUTLASS-class fallback (reference :299-318) is kept for M above ``gemm_pad_max_m``
  only (prefill), through the installed vLLM's own ops; a shape the decode kernels cannot
  take raises.

For a vLLM with the NVFP4 kernel registry (``model_executor/kernels/linear/nvfp4``),
:func:`register_with_vllm` puts :class:`Nvfp4rLinearKernel` first in that vLLM's own kernel
selection; no vLLM file is patched.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import capi
from . import _config

_OUT_DTYPE_INT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
_OUT_DTYPES = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32}


def _unswizzle_blockscale(sw_u8: torch.Tensor, M: int, K: int) -> torch.Tensor:
    """128x4-tiled block scales -> flat ``[M, K/16]`` uint8 (reference :99-117)."""
    return capi.unswizzle_blockscale(sw_u8.view(torch.uint8), M, K)


def prime_nvfp4r_caches(layer: torch.nn.Module) -> None:
    """Fill the per-layer derived state the hot path reads (reference :359-396):

    ``_nvfp4r_alpha_host``            Python float of ``layer.alpha``
    ``_nvfp4r_weight_scale_flat_3d``  ``[1, N, K/16]`` uint8 flat block scales
    ``_nvfp4r_weight_packed``         the weight in the packed block format of the
                                      tensor-core path (None when N % 128 or K % 128)

    ``layer.weight_scale`` may be swizzled (the reference's case, vLLM's CUTLASS
    format) or still flat ``[N, K/16]``; ``layer._nvfp4r_weight_scale_is_flat`` says
    which when it is set, otherwise the shape decides. Idempotent.
    """
    if getattr(layer, "_nvfp4r_caches_primed", False):
        return
    alpha_t = getattr(layer, "alpha", None)
    if alpha_t is None or not torch.is_tensor(alpha_t):
        return
    layer._nvfp4r_alpha_host = float(alpha_t.item())
    K = getattr(layer, "input_size_per_partition", None)
    N = getattr(layer, "output_size_per_partition", None)
    ws = getattr(layer, "weight_scale", None)
    if K is not None and N is not None and ws is not None and K // 16 > 0:
        ws_u8 = ws.data.view(torch.uint8)
        flat_hint = getattr(layer, "_nvfp4r_weight_scale_is_flat", None)
        is_flat = flat_hint if flat_hint is not None else (
            tuple(ws_u8.shape) == (N, K // 16) and (N % 128 != 0 or (K // 16) % 4 != 0))
        flat = ws_u8.contiguous() if is_flat else _unswizzle_blockscale(ws_u8, N, K)
        layer._nvfp4r_weight_scale_flat_3d = flat.reshape(1, N, K // 16).contiguous()
        layer._nvfp4r_weight_packed = None
        if N % 128 == 0 and K % 128 == 0 and getattr(layer, "weights_padding_cols", 0) == 0:
            layer._nvfp4r_weight_packed = capi.pack_weight(
                layer.weight.data.view(torch.uint8), layer._nvfp4r_weight_scale_flat_3d[0])
    layer._nvfp4r_caches_primed = True


def _fallback_available() -> bool:
    """True when a large-M library GEMM can be called (the reference's CUTLASS-class
    fallback, :299-318): vLLM's own NVFP4 ops are importable and not switched off."""
    if _config.FALLBACK_BACKEND == "none":
        return False
    try:
        import vllm._custom_ops as vops
    except ImportError:
        return False
    return hasattr(vops, "cutlass_scaled_fp4_mm") and hasattr(vops, "scaled_fp4_quant")


def _nvfp4r_linear_impl(x_2d: torch.Tensor, weight: torch.Tensor, weight_scale_swizzled: torch.Tensor,
                        weight_scale_flat_3d: torch.Tensor, input_global_scale_inv: torch.Tensor,
                        alpha: torch.Tensor, alpha_host: float, output_size: int,
                        weights_padding_cols: int, gemv_max_m: int, out_dtype_int: int,
                        enable_gemm: bool, weight_packed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All M-dependent branching of one linear, inside ONE opaque operator (reference
    ``_nvfp4r_linear_impl``, :165-318; the first twelve arguments are the reference's, in its
    order; ``weight_packed`` is this build's re-laid-out weight). Dynamo sees a single
    ``vllm::nvfp4r_linear`` node whatever M is, so the branch is taken at run time with the
    concrete M of the call (per captured batch size under vLLM's piecewise CUDA graphs), not
    frozen at trace time. Returns ``[M, output_size]``.

    * decode sizes: ONE launch, quantizer fused - the CUDA-core GEMV below the measured
      crossover, the tcgen05 kernel over the packed weight above it;
    * M above ``gemm_pad_max_m`` (prefill): vLLM's own ``scaled_fp4_quant`` +
      ``cutlass_scaled_fp4_mm`` when that vLLM is importable and ``fallback_backend`` is not
      ``none`` (the reference's fallback branch), else this library's kernels in launches of
      32 rows, each of which streams the weight once.
    """
    from .ops import use_gemv
    M, K = x_2d.shape
    if weights_padding_cols != 0:
        raise RuntimeError("nvfp4r: K-padded weights are not supported")
    if M > _config.GEMM_PAD_MAX_M and _fallback_available():
        import vllm._custom_ops as vops
        x_fp4, x_sf = vops.scaled_fp4_quant(x_2d, input_global_scale_inv, is_sf_swizzled_layout=True)
        out_dtype = {0: torch.bfloat16, 1: torch.float16}.get(out_dtype_int, x_2d.dtype)
        return vops.cutlass_scaled_fp4_mm(x_fp4, weight, x_sf, weight_scale_swizzled, alpha, out_dtype)
    tc_ok = enable_gemm and weight_packed is not None
    if tc_ok and not use_gemv(M, output_size, K, gemv_max_m):
        return torch.ops.nvfp4r.linear_packed(x_2d, input_global_scale_inv, weight_packed,
                                              output_size, alpha_host, out_dtype_int, 1)
    if M <= 16:
        return torch.ops.nvfp4r.linear(x_2d, input_global_scale_inv, weight, weight_scale_flat_3d,
                                       alpha_host, out_dtype_int, 1)
    parts = [torch.ops.nvfp4r.linear(x_2d[i:i + 16], input_global_scale_inv, weight,
                                     weight_scale_flat_3d, alpha_host, out_dtype_int, 1)
             for i in range(0, M, 16)]
    return torch.cat(parts, dim=0)


def _nvfp4r_linear_fake(x_2d: torch.Tensor, weight: torch.Tensor, weight_scale_swizzled: torch.Tensor,
                        weight_scale_flat_3d: torch.Tensor, input_global_scale_inv: torch.Tensor,
                        alpha: torch.Tensor, alpha_host: float, output_size: int,
                        weights_padding_cols: int, gemv_max_m: int, out_dtype_int: int,
                        enable_gemm: bool, weight_packed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Shape and dtype of the result for tracing (reference ``_nvfp4r_linear_fake``, :321-339)."""
    return torch.empty((x_2d.shape[0], output_size), dtype=_OUT_DTYPES[out_dtype_int],
                       device=x_2d.device)


def _register_ops_once() -> None:
    """Define ``torch.ops.vllm.nvfp4r_linear`` with its fake, once per process (reference
    :342-353). vLLM's ``direct_register_custom_op`` when that vLLM is importable, else the
    same registration through ``torch.library`` so the adapter works without vLLM."""
    try:
        if hasattr(torch.ops.vllm, "nvfp4r_linear"):
            return
    except (AttributeError, RuntimeError):
        pass
    try:
        from vllm.utils.torch_utils import direct_register_custom_op
    except ImportError:
        direct_register_custom_op = None
    if direct_register_custom_op is not None:
        direct_register_custom_op(op_name="nvfp4r_linear", op_func=_nvfp4r_linear_impl,
                                  mutates_args=[], fake_impl=_nvfp4r_linear_fake,
                                  dispatch_key="CUDA")
        return
    global _VLLM_FRAGMENT
    _VLLM_FRAGMENT = torch.library.Library("vllm", "FRAGMENT")
    schema = torch.library.infer_schema(_nvfp4r_linear_impl, mutates_args=[])
    _VLLM_FRAGMENT.define("nvfp4r_linear" + schema)
    _VLLM_FRAGMENT.impl("nvfp4r_linear", _nvfp4r_linear_impl, "CUDA")
    _VLLM_FRAGMENT._register_fake("nvfp4r_linear", _nvfp4r_linear_fake)


_VLLM_FRAGMENT = None
_register_ops_once()


def apply_nvfp4r_linear(layer: torch.nn.Module, x: torch.Tensor,
                        bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Hot path (reference :448-496): one ``vllm::nvfp4r_linear`` node per linear. Reads only
    tensors and constant Python attributes of ``layer``: no ``.item()``, no ``setattr``, no
    environment reads, no branch on M, so it traces under ``torch.compile(fullgraph=True)``."""
    output_size = layer.output_size_per_partition
    output_shape = (*x.shape[:-1], output_size)
    x_2d = x.reshape(-1, x.shape[-1])
    out = torch.ops.vllm.nvfp4r_linear(
        x_2d, layer.weight, layer.weight_scale, layer._nvfp4r_weight_scale_flat_3d,
        layer.input_global_scale_inv, layer.alpha, layer._nvfp4r_alpha_host, output_size,
        getattr(layer, "weights_padding_cols", 0), _config.GEMV_MAX_M, _OUT_DTYPE_INT[x.dtype],
        _config.ENABLE_GEMM_PATH, layer._nvfp4r_weight_packed)
    if bias is not None:
        out = out + bias
    return out.view(*output_shape)


_KERNEL_CLASS = None


def register_with_vllm() -> bool:
    """Put :class:`Nvfp4rLinearKernel` into the NVFP4 linear-kernel registry of a vLLM that
    has one (``vllm/model_executor/kernels/linear``, vLLM 0.22): FIRST in the list its
    automatic selection walks for CUDA (``_POSSIBLE_NVFP4_KERNELS``), and under the name
    ``nvfp4r`` in ``_NVFP4_BACKEND_TO_KERNEL``. That vLLM validates
    ``VLLM_NVFP4_GEMM_BACKEND`` against its own fixed list of names and rejects ``nvfp4r``,
    so the environment variable of the reference (kernels/python/nvfp4r/__init__.py:30-36)
    cannot select the kernel there; being first in the automatic selection does. Returns
    False when this vLLM has no such registry (the reference's patched-vLLM route then
    applies: the patched ``apply_nvfp4_linear`` calls :func:`apply_nvfp4r_linear`)."""
    global _KERNEL_CLASS
    try:
        import vllm.model_executor.kernels.linear as vk
        from vllm.model_executor.kernels.linear.nvfp4.base import NvFp4LinearKernel
    except ImportError:
        return False
    table = getattr(vk, "_NVFP4_BACKEND_TO_KERNEL", None)
    possible = getattr(vk, "_POSSIBLE_NVFP4_KERNELS", None)
    if table is None or possible is None:
        return False
    if _KERNEL_CLASS is None:
        _KERNEL_CLASS = _make_kernel_class(NvFp4LinearKernel)
    table["nvfp4r"] = _KERNEL_CLASS
    for platform, kernels in possible.items():
        if getattr(platform, "name", "") == "CUDA" and _KERNEL_CLASS not in kernels:
            kernels.insert(0, _KERNEL_CLASS)
    return True


def unregister_from_vllm() -> None:
    """Undo :func:`register_with_vllm` (``nvfp4r.disable()``)."""
    try:
        import vllm.model_executor.kernels.linear as vk
    except ImportError:
        return
    table = getattr(vk, "_NVFP4_BACKEND_TO_KERNEL", None)
    if table is not None:
        table.pop("nvfp4r", None)
    for kernels in (getattr(vk, "_POSSIBLE_NVFP4_KERNELS", None) or {}).values():
        while _KERNEL_CLASS is not None and _KERNEL_CLASS in kernels:
            kernels.remove(_KERNEL_CLASS)


def _make_kernel_class(base):
    class Nvfp4rLinearKernel(base):
        """NVFP4 linear through the nvfp4r B200 kernels."""

        @classmethod
        def is_supported(cls, compute_capability=None):
            if not torch.cuda.is_available():
                return False, "CUDA device required"
            major, minor = torch.cuda.get_device_capability()
            if (major, minor) != (10, 0):
                return False, "nvfp4r kernels are built for sm_100a only"
            return True, None

        @classmethod
        def can_implement(cls, config):
            return True, None

        def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
            # the checkpoint's flat [N, K/16] scales are kept for the GEMV and a
            # swizzled copy is made for the tensor-core GEMM
            flat = layer.weight_scale.data.view(torch.uint8).contiguous()
            layer._nvfp4r_weight_scale_is_flat = True
            prime_nvfp4r_caches(layer)
            layer.weight_scale = torch.nn.Parameter(
                capi.swizzle_blockscale(flat).view(torch.float8_e4m3fn), requires_grad=False)
            layer.weights_padding_cols = 0

        def apply_weights(self, layer, x, bias=None):
            return apply_nvfp4r_linear(layer, x, bias)

    return Nvfp4rLinearKernel


def enable() -> None:  # pragma: no cover
    """No-op kept for callers of the reference's legacy shim (reference :502-508)."""
    return


def disable() -> None:  # pragma: no cover
    return
