"""nvfp4r - NVFP4 W4A4 decode kernels for B200, same Python surface as the reference
package (kernels/python/nvfp4r/__init__.py:22-82): ``gemv``, ``gemm``, ``enable``,
``disable``, ``configure``, ``status``; importing it registers ``torch.ops.nvfp4r.*``.

``vllm_integration`` is not imported eagerly, so the package works without vLLM
(reference: __init__.py:7-9).
"""

from __future__ import annotations

import os

import torch  # noqa: F401  (libtorch must be loaded before the extension)

from .. import _C  # noqa: F401  (registers torch.ops.nvfp4r.*; raises if not built)
from . import _fake  # noqa: F401  (FakeTensor impls for torch.compile)
from . import _config
from .ops import gemm, gemv, linear, linear_auto, linear_packed, pack_weight, quant

__all__ = ["gemv", "gemm", "quant", "linear", "linear_packed", "linear_auto", "pack_weight", "enable", "disable", "configure", "status"]
__version__ = "0.1.0"


_REGISTERED = False      # the kernel class sits in vLLM's own NVFP4 kernel registry


def enable(backend: str = "nvfp4r") -> None:
    """Route vLLM's NVFP4 linear layers through these kernels. Call before constructing the
    engine (reference: __init__.py:30-36, which sets ``VLLM_NVFP4_GEMM_BACKEND``).

    With a vLLM that has the NVFP4 kernel registry (0.22), the kernel class is put first in
    its automatic selection and the environment variable is NOT set: that vLLM checks the
    variable against its own list of names and raises on ``nvfp4r``. Without the registry
    (the reference's patched vLLM) the environment variable is the contract, as in the
    reference."""
    global _REGISTERED
    _REGISTERED = False
    if backend == "nvfp4r":
        try:
            from . import vllm_integration as _vi
            _REGISTERED = bool(_vi.register_with_vllm())
        except ImportError:
            _REGISTERED = False  # vLLM absent: the environment variable alone is the contract
    if _REGISTERED:
        os.environ.pop("VLLM_NVFP4_GEMM_BACKEND", None)
    else:
        os.environ["VLLM_NVFP4_GEMM_BACKEND"] = str(backend)


def disable() -> None:
    """Back to vLLM's stock NVFP4 path (reference: __init__.py:39-41)."""
    global _REGISTERED
    os.environ.pop("VLLM_NVFP4_GEMM_BACKEND", None)
    if _REGISTERED:
        from . import vllm_integration as _vi
        _vi.unregister_from_vllm()
    _REGISTERED = False


def configure(*, gemv_max_m: int | None = None, enable_gemm: bool | None = None,
              gemm_pad_max_m: int | None = None, fallback_backend: str | None = None) -> None:
    """Runtime knobs, same keys as the reference (__init__.py:44-69).

    gemv_max_m        largest decode batch sent to the CUDA-core GEMV
    enable_gemm       use the tcgen05 GEMM above ``gemv_max_m``
    gemm_pad_max_m    largest M handled as a (padded) small-M tensor-core tile
    fallback_backend  accepted and recorded for compatibility; this build has no
                      second backend to fall back to, unsupported shapes raise
    """
    if gemv_max_m is not None:
        _config.GEMV_MAX_M = int(gemv_max_m)
    if enable_gemm is not None:
        _config.ENABLE_GEMM_PATH = bool(enable_gemm)
    if gemm_pad_max_m is not None:
        _config.GEMM_PAD_MAX_M = int(gemm_pad_max_m)
    if fallback_backend is not None:
        _config.FALLBACK_BACKEND = str(fallback_backend).lower()


def status() -> dict:
    """Active configuration (reference: __init__.py:72-82)."""
    return {
        "active": _REGISTERED or os.environ.get("VLLM_NVFP4_GEMM_BACKEND") == "nvfp4r",
        "gemv_max_m": _config.GEMV_MAX_M,
        "enable_gemm": _config.ENABLE_GEMM_PATH,
        "gemm_pad_max_m": _config.GEMM_PAD_MAX_M,
        "fallback_backend": _config.FALLBACK_BACKEND,
    }
