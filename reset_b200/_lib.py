"""ctypes binding of ``libnvfp4r_b200.so`` (the C ABI in ``include/nvfp4r_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is
raised. Build it with ``python -m reset_b200.build``.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libnvfp4r_b200.so"

OK = 0
BF16, F16, F32 = 0, 1, 2
SF_FLAT, SF_SWIZZLED = 0, 1
RCP_EXACT, RCP_APPROX = 0, 1
C_M_MAJOR, C_N_MAJOR = 0, 1
RESET_MAX_WINDOW = 64
RESET_STATIC_MAX_ROWS = 64
LINEAR_MAX_M = 16


class ResetState(C.Structure):
    _fields_ = [("window_buf", C.c_double * RESET_MAX_WINDOW), ("step_sum", C.c_double),
                ("total_sum", C.c_double), ("total_count", C.c_int64),
                ("step_count", C.c_int32), ("window_count", C.c_int32),
                ("window_head", C.c_int32), ("reserved", C.c_int32)]


class ResetParams(C.Structure):
    _fields_ = [("t_high", C.c_double), ("t_low", C.c_double), ("tau0", C.c_double),
                ("window", C.c_int32), ("id_set", C.c_int32)]


class ResetDecision(C.Structure):
    _fields_ = [("entropy", C.c_double), ("h_step", C.c_double), ("h_bar", C.c_double),
                ("temp", C.c_double), ("boundary", C.c_int32), ("high_step", C.c_int32)]


class Prologue(C.Structure):
    _fields_ = [("kind", C.c_int), ("eps", C.c_float), ("delta", C.c_void_p),
                ("residual_in", C.c_void_p), ("residual_out", C.c_void_p), ("norm_weight", C.c_void_p),
                ("push_to", C.c_void_p), ("push_gather", C.c_int)]


PROLOGUE_NONE, PROLOGUE_ADD_RMSNORM, PROLOGUE_SILU_MUL = 0, 1, 2

PEER_MAX_WORLD = 8
PEER_PUSH, PEER_GATHER, PEER_ALLREDUCE = 1, 2, 3


class PeerComm(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("max_elems", C.c_size_t),
                ("base", C.c_void_p * PEER_MAX_WORLD)]


_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); every symbol include/nvfp4r_b200.h declares
PROTOTYPES = {
    "nvfp4r_status_string": (C.c_char_p, [_i]),
    "nvfp4r_last_error": (C.c_char_p, []),
    "nvfp4r_version": (_i, []),
    "nvfp4r_quant": (_i, [_vp, _i64, _i, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "nvfp4r_gemv": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64,
                         _f, _i, _vp]),
    "nvfp4r_linear": (_i, [_vp, _i64, _i, _i, _vp, _vp, _vp, _i, _f, _vp, _i, _i, _vp]),
    "nvfp4r_gemm_workspace_bytes": (_sz, [_i, _i, _i]),
    "nvfp4r_linear_tc": (_i, [_vp, _i64, _i, _i, _vp, _vp, _vp, _i, _f, _vp, _i, _i, _vp, _sz, _vp]),
    "nvfp4r_set_gemm_tuning": (_i, [_i, _i]),
    "nvfp4r_packed_weight_bytes": (_sz, [_i, _i]),
    "nvfp4r_linear_packed_workspace_bytes": (_sz, [_i, _i, _i]),
    "nvfp4r_pack_weight": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "nvfp4r_linear_packed": (_i, [_vp, _i64, _i, _i, _vp, _vp, _i, _f, _vp, _i, _i, _vp, _sz, _vp]),
    "nvfp4r_linear_packed_ex": (_i, [C.POINTER(Prologue), _vp, _i64, _i, _i, _vp, _vp, _i, _f, _vp, _i, _i,
                                     _vp, _sz, _vp]),
    "nvfp4r_linear_ex": (_i, [C.POINTER(Prologue), _vp, _i64, _i, _i, _vp, _vp, _vp, _i, _f, _vp, _i, _i, _vp]),
    "nvfp4r_set_packed_tuning": (_i, [_i]),
    "nvfp4r_gemm": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _i, _vp, _sz, _vp]),
    "nvfp4r_unswizzle_blockscale": (_i, [_vp, _vp, _i, _i, _vp]),
    "nvfp4r_swizzle_blockscale": (_i, [_vp, _vp, _i, _i, _vp]),
    "nvfp4r_reset_workspace_bytes": (_sz, [_i]),
    "nvfp4r_reset_step": (_i, [_vp, _i64, _i, _i, _vp, _vp, _vp, _vp, _vp,
                               C.POINTER(ResetParams), _vp, _vp, _sz, _vp]),
    "nvfp4r_reset_step_per_request": (_i, [_vp, _i64, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp,
                                           _vp, _sz, _vp]),
    "nvfp4r_lm_head_reset_workspace_bytes": (_sz, []),
    "nvfp4r_lm_head_reset_step": (_i, [_vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp,
                                       _vp, _sz, _vp]),
    "nvfp4r_reset_step_static": (_i, [_vp, _i64, _i, _i, _vp, _vp, _vp, _vp, _vp,
                                      C.POINTER(ResetParams), _vp, _vp]),
    "nvfp4r_entropy": (_i, [_vp, _i64, _i, _i, _vp, _vp, _sz, _vp]),
    "nvfp4r_status_mirror": (_i, [C.POINTER(C.POINTER(C.c_int))]),
    "nvfp4r_set_gemv_tuning": (_i, [_i, _i, _i]),
    "nvfp4r_set_gemv_rows_tuning": (_i, [_i, _i, _i]),
    "nvfp4r_add_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "nvfp4r_qk_norm_rope_kv": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _vp]),
    "nvfp4r_attn_decode_workspace_bytes": (_sz, [_i, _i]),
    "nvfp4r_attn_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _sz, _vp]),
    "nvfp4r_attn_decode_rope": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _vp, _sz, _vp]),
    "nvfp4r_set_rope_table": (_i, [_vp, _i]),
    "nvfp4r_silu_mul": (_i, [_vp, _vp, _i, _i, _vp]),
    "nvfp4r_lm_head": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "nvfp4r_argmax": (_i, [_vp, _i64, _i, _i, _vp, _vp]),
    "nvfp4r_sample": (_i, [_vp, _i64, _i, _i, C.c_uint64, _vp, _vp, _vp, _vp]),
    "nvfp4r_sample_workspace_bytes": (_sz, [_i]),
    "nvfp4r_sample_top_k_top_p": (_i, [_vp, _i64, _i, _i, _i, C.c_float, C.c_uint64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "nvfp4r_peer_buffer_bytes": (_sz, [_i, _sz]),
    "nvfp4r_peer_alloc": (_i, [_sz, C.POINTER(C.c_void_p), C.c_char_p]),
    "nvfp4r_peer_open": (_i, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "nvfp4r_peer_close": (_i, [_vp]),
    "nvfp4r_peer_free": (_i, [_vp]),
    "nvfp4r_peer_allreduce_bf16": (_i, [C.POINTER(PeerComm), _vp, _vp, _sz, _i, _vp]),
    "nvfp4r_set_peer_poll_limit": (_i, [C.c_uint]),
    "nvfp4r_check_device_status": (_i, []),
}

_lib = None


class Nvfp4rError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def lib() -> C.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: run `python -m reset_b200.build` "
                              "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)          # AttributeError if a symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != OK:
        l = lib()
        raise Nvfp4rError(f"{what}: {l.nvfp4r_status_string(status).decode()} "
                          f"({status}): {l.nvfp4r_last_error().decode()}")


def status_mirror():
    """ctypes pointer to the host-visible time-out word of the current device
    (``nvfp4r_status_mirror``): ``p[0]`` is 0 or the code of the kernel family whose bounded
    wait gave up; reading it synchronises nothing; assign ``p[0] = 0`` to clear."""
    p = C.POINTER(C.c_int)()
    check(lib().nvfp4r_status_mirror(C.byref(p)), "nvfp4r_status_mirror")
    return p
