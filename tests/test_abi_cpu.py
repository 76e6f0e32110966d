"""No GPU needed: the C-ABI library loads, exports every symbol the public header
declares, the ctypes table matches the header, and the Python surface of the reference's
``nvfp4r`` package (enable/disable/configure/status) behaves as the reference's does."""

from __future__ import annotations

import ctypes
import os
import re

import pytest
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent
HEADER = REPO / "include" / "nvfp4r_b200.h"


def _declared():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"NVFP4R_API\s+[\w\s\*]+?\b(nvfp4r_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from reset_b200 import _lib
    names = _declared()
    assert len(names) >= 25
    raw = ctypes.CDLL(str(_lib.LIB_PATH))
    missing = [n for n in names if not hasattr(raw, n)]
    assert not missing, missing
    # the ctypes prototypes cover the header and nothing else
    assert sorted(_lib.PROTOTYPES) == names
    lib = _lib.lib()
    assert lib.nvfp4r_version() >= 1
    assert lib.nvfp4r_status_string(0) == b"ok" and lib.nvfp4r_status_string(-2) == b"unsupported shape"


def test_host_side_sizes_without_a_gpu():
    from reset_b200 import _lib
    lib = _lib.lib()
    assert lib.nvfp4r_packed_weight_bytes(4096, 4096) == 4096 * 4096 * 9 // 16
    assert lib.nvfp4r_packed_weight_bytes(100, 4096) == 0
    assert lib.nvfp4r_reset_workspace_bytes(8) == 8 * (656 + 1304)
    assert lib.nvfp4r_attn_decode_workspace_bytes(64, 2048) == 64 * 16 * 132 * 4 + 64 * 4
    assert lib.nvfp4r_peer_buffer_bytes(2, 5120) == 256 + 2 * 2 * 2560 * 8
    assert lib.nvfp4r_peer_buffer_bytes(9, 5120) == 0
    assert ctypes.sizeof(_lib.ResetState) == 64 * 8 + 16 + 8 + 16
    # argument checks come before any CUDA call
    assert lib.nvfp4r_quant(None, 0, 1, 16, None, None, None, 0, 0, None) == -1
    assert lib.nvfp4r_reset_step_static(None, 0, 1, 8, None, None, None, None, None, None, None, None) == -1


def test_enable_disable_configure_status(monkeypatch):
    monkeypatch.delenv("VLLM_NVFP4_GEMM_BACKEND", raising=False)
    from reset_b200 import nvfp4r
    from reset_b200.nvfp4r import _config
    saved = (_config.GEMV_MAX_M, _config.ENABLE_GEMM_PATH, _config.GEMM_PAD_MAX_M, _config.FALLBACK_BACKEND)
    try:
        assert set(nvfp4r.status()) == {"active", "gemv_max_m", "enable_gemm", "gemm_pad_max_m", "fallback_backend"}
        assert nvfp4r.status()["active"] is False
        os.environ["VLLM_NVFP4_GEMM_BACKEND"] = "nvfp4r"      # what enable() sets
        assert nvfp4r.status()["active"] is True
        nvfp4r.disable()
        assert "VLLM_NVFP4_GEMM_BACKEND" not in os.environ
        nvfp4r.configure(gemv_max_m=1, enable_gemm=False, gemm_pad_max_m=31, fallback_backend="CUTLASS")
        st = nvfp4r.status()
        assert (st["gemv_max_m"], st["enable_gemm"], st["gemm_pad_max_m"], st["fallback_backend"]) == \
               (1, False, 31, "cutlass")
        assert set(nvfp4r.__all__) >= {"gemv", "gemm", "enable", "disable", "configure", "status"}
    finally:
        (_config.GEMV_MAX_M, _config.ENABLE_GEMM_PATH, _config.GEMM_PAD_MAX_M, _config.FALLBACK_BACKEND) = saved


def test_crossover_rule():
    from reset_b200.nvfp4r.ops import use_gemv
    # single tokens: the GEMV up to 10.5 MB of weight (measured on the 8B / 14B / 32B shapes and shards)
    assert use_gemv(1, 4096, 4096, 4) and use_gemv(1, 1280, 5120, 4) and use_gemv(1, 3584, 5120, 4)
    assert not use_gemv(1, 5120, 4096, 4) and not use_gemv(1, 6144, 4096, 4) and not use_gemv(1, 5120, 5120, 4)
    assert not use_gemv(1, 4096, 12288, 4) and not use_gemv(1, 10240, 5120, 4) and not use_gemv(1, 24576, 4096, 4)
    # from two tokens on: the tensor cores on every shape
    assert not use_gemv(2, 4096, 2048, 4) and not use_gemv(4, 4096, 1024, 4) and not use_gemv(2, 1280, 5120, 4)
    # N = 5120 (a poor fit for the ring kernel's warp count): only with short rows
    assert use_gemv(1, 5120, 1024, 4) and use_gemv(1, 5120, 2048, 4) and not use_gemv(1, 5120, 2560, 4)
    assert not use_gemv(1, 5120, 640, 4)                      # very short rows stay on the tensor cores
    assert use_gemv(1, 5120, 3200, 4) is False
    assert not use_gemv(3, 4096, 1024, 2)                     # above gemv_max_m
    assert not use_gemv(1, 4096, 4096, 0)                     # gemv_max_m = 0 disables the GEMV


def test_single_launch_all_reduce_rule(monkeypatch):
    """Which tensor-parallel widths complete the all-reduce inside the row-parallel linear's own
    launch: the tensor-core kernel up to two ranks when called one linear at a time, the streaming
    GEMV up to four inside a decode layer; NVFP4R_FUSED_GATHER forces either answer."""
    from reset_b200.nvfp4r import _config
    monkeypatch.setattr(_config, "FUSED_GATHER", "auto")
    assert [_config.fused_gather(w) for w in (1, 2, 4, 8)] == [True, True, False, False]
    assert _config.GEMV_PUSH_MAX_WORLD == 4 and _config.FUSED_GATHER_MAX_WORLD == 2
    monkeypatch.setattr(_config, "FUSED_GATHER", "1")
    assert all(_config.fused_gather(w) for w in (2, 4, 8))
    monkeypatch.setattr(_config, "FUSED_GATHER", "0")
    assert not any(_config.fused_gather(w) for w in (1, 2, 4, 8))


def test_ops_are_registered_with_the_reference_schemas():
    import torch
    from reset_b200 import nvfp4r  # noqa: F401
    gemv = torch.ops.nvfp4r.gemv.default._schema
    gemm = torch.ops.nvfp4r.gemm.default._schema
    assert str(gemv) == ("nvfp4r::gemv(Tensor weight, Tensor weight_scale, Tensor x, Tensor x_scale, "
                         "Tensor(a!) out, float alpha=1.) -> ()")
    assert str(gemm) == "nvfp4r::gemm(Tensor A, Tensor B, Tensor SFA, Tensor SFB, Tensor(a!) C, float alpha=1.) -> ()"


def test_newline_id_scan_and_bitmap():
    import torch
    """`get_newline_token_ids` (reference reset/reset/logits_processor.py:39-59) on a stand-in
    tokenizer, and the id bitmap the kernels read."""
    from reset_b200.reset import logits_processor as lp

    class Tok:
        vocab_size = 70
        table = {3: "\n", 5: "\n\n", 9: "a\n\nb", 40: " \n", 63: "\n"}

        def decode(self, ids, skip_special_tokens=False):
            if ids[0] == 7:
                raise ValueError("undecodable id")
            return self.table.get(ids[0], "x")

    nl, dnl = lp.get_newline_token_ids(Tok())
    assert nl == [3, 63] and dnl == [5, 9]
    bm = lp._bitmap([3, 63, 31, 64, 999, -1], 70, "cpu")
    assert bm.shape == (3,) and bm.dtype == torch.int32
    words = [int(w) & 0xFFFFFFFF for w in bm.tolist()]
    assert words == [(1 << 3) | (1 << 31), 1 << 31, 1 << 0]
    assert lp._bitmap([], 70, "cpu") is None


def test_scale_by_temperature_matches_oracle_on_cpu():
    import torch
    from oracle import reset_policy as orp
    from reset_b200.reset.logits_processor import scale_by_temperature

    x = orp.synthetic_logits(2, 100, 3)
    for t in (1.0, 0.1, 0.0, 1e-7):
        assert torch.equal(scale_by_temperature(x[0], t), orp.apply_temperature(x[0], t))


def test_enable_registers_first_in_the_installed_vllm_registry(monkeypatch):
    """With a vLLM that has the NVFP4 linear-kernel registry, ``enable()`` puts the kernel class
    first in the automatic CUDA selection and leaves ``VLLM_NVFP4_GEMM_BACKEND`` unset (that
    vLLM rejects names outside its own list); ``disable()`` takes it out again."""
    vk = pytest.importorskip("vllm.model_executor.kernels.linear")
    if not hasattr(vk, "_POSSIBLE_NVFP4_KERNELS"):
        pytest.skip("this vLLM has no NVFP4 kernel registry")
    from vllm.model_executor.kernels.linear.nvfp4.base import NvFp4LinearKernel
    monkeypatch.delenv("VLLM_NVFP4_GEMM_BACKEND", raising=False)
    from reset_b200 import nvfp4r
    cuda_lists = [v for k, v in vk._POSSIBLE_NVFP4_KERNELS.items() if getattr(k, "name", "") == "CUDA"]
    assert cuda_lists
    before = [list(v) for v in cuda_lists]
    try:
        nvfp4r.enable()
        assert nvfp4r.status()["active"] is True
        assert "VLLM_NVFP4_GEMM_BACKEND" not in os.environ
        cls = vk._NVFP4_BACKEND_TO_KERNEL["nvfp4r"]
        assert issubclass(cls, NvFp4LinearKernel) and cls.__name__ == "Nvfp4rLinearKernel"
        assert all(v[0] is cls and v.count(cls) == 1 for v in cuda_lists)
        nvfp4r.enable()                                     # idempotent
        assert all(v.count(cls) == 1 for v in cuda_lists)
        ok, why = cls.is_supported()
        import torch
        if not torch.cuda.is_available():
            assert ok is False and "CUDA" in why           # no silent CPU path
        assert cls.can_implement(None) == (True, None)
    finally:
        nvfp4r.disable()
    assert nvfp4r.status()["active"] is False
    assert "nvfp4r" not in vk._NVFP4_BACKEND_TO_KERNEL
    assert [list(v) for v in cuda_lists] == before


def test_batch_processor_is_a_vllm_logits_processor():
    """``LLM(logits_processors=[ReSETBatchProcessor])`` (and the ``module:Class`` string form)
    go through vLLM's loader, which only accepts subclasses of its ``LogitsProcessor``."""
    lp = pytest.importorskip("vllm.v1.sample.logits_processor")
    from reset_b200 import reset
    cls = reset.ReSETBatchProcessor
    assert cls is reset.ReSETBatchProcessor and cls.__name__ == "ReSETBatchProcessor"
    assert issubclass(cls, lp.LogitsProcessor) and not getattr(cls, "__abstractmethods__", None)
    assert lp._load_logitsprocs_by_fqcns([cls]) == [cls]
    assert lp._load_logitsprocs_by_fqcns(["reset_b200.reset:ReSETBatchProcessor"]) == [cls]
    assert issubclass(reset.ReSETAdapter, lp.LogitsProcessor)


def test_reciprocals_the_packed_linear_divides_with_are_exact():
    """The tensor-core linear takes its CTA index apart with multiply-high by ceil(2^32 / splits)
    and its activation-block index with multiply + shift by ceil(2^20 / blocks) (the divisions
    happen on the host, once per launch): exact over everything a launch can ask for."""
    for splits in range(2, 65):
        inv = ((1 << 32) + splits - 1) // splits
        assert inv < (1 << 32)
        assert all((b * inv) >> 32 == b // splits for b in range(0, 1 << 16, 7)) and \
            all((b * inv) >> 32 == b // splits for b in range((1 << 16) - 600, 1 << 16))
    for blocks in range(16, 129, 16):
        inv = ((1 << 20) + blocks - 1) // blocks
        assert all((i * inv) >> 20 == i // blocks for i in range(32 * 128 + 3 * 192 + 1))
