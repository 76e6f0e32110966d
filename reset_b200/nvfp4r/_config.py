"""Module-level knobs behind ``configure()`` / ``status()``. Defaults can be preset
with the reference's environment variables (vllm_integration.py:61-93)."""

import os

# Largest decode batch routed to the CUDA-core GEMV. The reference defaults to 2;
# here it is the crossover measured on B200 against the tcgen05 kernel.
GEMV_MAX_M = int(os.environ.get("NVFP4R_GEMV_MAX_M", "4"))
GEMM_PAD_MAX_M = int(os.environ.get("NVFP4R_GEMM_PAD_MAX_M", "63"))
ENABLE_GEMM_PATH = os.environ.get("NVFP4R_ENABLE_GEMM", "1") == "1"
# Large-M (prefill) fallback of the adapter: "vllm-cutlass" = the installed vLLM's own NVFP4 GEMM
# when importable (the reference's fallback branch), "none" = always this library's kernels.
FALLBACK_BACKEND = os.environ.get("NVFP4R_FALLBACK_BACKEND", "vllm-cutlass").lower()

# Measured crossover between the CUDA-core GEMV and the packed tensor-core linear on B200
# (L2-cold weights, CUDA-graph replay; Qwen3-8B / 14B / 32B shapes and their tensor-parallel
# shards at TP 2 / 4 / 8). The GEMV's shorter fixed latency wins for single tokens on weights up
# to GEMV_MAX_WEIGHT_BYTES[1] (1280x5120 3.5 vs 5.0 us, 5120x2048 3.3 vs 3.6 us, 4096x4096 3.7 vs
# 4.2 us, 3584x5120 4.55 vs 4.8 us; 5120x4096 5.1 vs 4.4 us, 6144x4096 5.0 vs 4.7 us,
# 4096x12288 7.3 vs 6.2 us, 10240x5120 7.8 vs 6.3 us above it). From two tokens on the tensor
# cores win on every shape measured (5120x1024 3.5 vs 3.4 us, 1280x5120 6.1 vs 5.0 us). Index = M.
GEMV_MAX_WEIGHT_BYTES = {1: 10_500_000}
# Rows shorter than this stay on the tensor cores at every M (5120x640: 3.6 vs 3.8 us).
GEMV_MIN_K = 1024
# The ring kernel deals groups of 4 rows to GEMV_RING_WARPS warps; with N between 4 and 5 times
# that count a second round runs on under a quarter of the warps and the tensor cores win unless
# the rows are short (5120x2560 4.4 vs 4.8 us; 5120x2048 3.3 vs 3.6 us, 5120x1024 2.6 vs 3.3 us).
GEMV_RING_WARPS = 148 * 8
GEMV_SHORT_ROW_K = 2048

# Tensor-parallel row-parallel linears through `linear_auto(..., reduce=)`: complete the
# all-reduce inside the linear's own launch, or push in the epilogue and gather in a second
# launch. Measured on B200 (Qwen3-8B linear set, independent linears back to back): the single
# launch wins at two ranks (3480 vs 3400 GB/s) and loses at eight (3214 vs 3766 GB/s), where its
# CTAs hold the SMs while they wait for seven peers and the next linear's early loads cannot
# start; a step whose next kernel needs the sum anyway (a decode layer) gains at every width
# (Qwen3-32B TP 8: 353 vs 348 tok/s). "auto" = single launch up to FUSED_GATHER_MAX_WORLD ranks.
FUSED_GATHER = os.environ.get("NVFP4R_FUSED_GATHER", "auto").lower()      # "auto", "1" or "0"
FUSED_GATHER_MAX_WORLD = 2


# The same choice for shards small enough for the CUDA-core GEMV inside a decode layer (o_proj at
# TP 4 / 8): the sum inside the GEMV's launch saves a launch per layer and wins up to four ranks
# (Qwen3-32B: 373.9 vs 367.0 tok/s at N = 4); with eight its CTAs wait for seven peers while they
# hold the SMs and the separate all-reduce launch wins (359 vs 381-400 tok/s).
GEMV_PUSH_MAX_WORLD = 4


def fused_gather(world: int) -> bool:
    if FUSED_GATHER in ("1", "true", "on"):
        return True
    if FUSED_GATHER in ("0", "false", "off"):
        return False
    return world <= FUSED_GATHER_MAX_WORLD
