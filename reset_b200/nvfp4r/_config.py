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

# Measured crossover between the CUDA-core GEMV and the packed tensor-core linear on
# B200 (L2-cold weights, CUDA-graph replay): the GEMV's shorter fixed latency wins only
# for the smallest batches on weights of at most this many bytes; everything else goes
# to the tensor cores. Index = M.
GEMV_MAX_WEIGHT_BYTES = {1: 11_000_000, 2: 5_000_000, 3: 2_500_000, 4: 2_500_000}
# Single-token launches with at least GEMV_WIDE_MIN_N rows of at most GEMV_WIDE_MAX_K elements
# run the GEMV with three CTAs per SM (24 warps instead of 8 hide its decode latency); there it
# stays ahead of the tensor-core kernel up to GEMV_WIDE_MAX_WEIGHT_BYTES (6144x4096: 5.0 vs
# 5.6 us, 8192x4096: 6.05 vs 6.35 us; 12288x4096: 7.7 vs 7.3 us, 7168x5120: 7.1 vs 6.6 us).
GEMV_WIDE_MIN_N = 6144
GEMV_WIDE_MAX_K = 4096
GEMV_WIDE_MAX_WEIGHT_BYTES = 19_000_000
# ... and, above one token, only for short rows (the GEMV's time grows with M * K per row)
GEMV_MAX_K_MULTI_TOKEN = 2048
