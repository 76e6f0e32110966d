"""Tensor-parallel sharding of the NVFP4 linears, Megatron style, as vLLM hands them to
the reference's adapter (which only reads ``input_size_per_partition`` /
``output_size_per_partition``, kernels/python/nvfp4r/vllm_integration.py:461-462):

* column-parallel (qkv_proj, gate_up_proj): rows of the weight (output features) are
  split; no communication;
* row-parallel (o_proj, down_proj): the K dimension is split - codes by bytes, block
  scales by blocks of 16 - and the per-rank partial products are summed with one
  all-reduce.

The activation quantizer shards with K because its blocks are 16 consecutive K elements
and its global scale is a per-layer constant. Host-side arithmetic only."""

from __future__ import annotations


def shard_shape(N: int, K: int, style: str, world: int) -> tuple[int, int]:
    """Per-rank (N, K) of a linear."""
    if style == "column":
        if N % world:
            raise ValueError(f"column-parallel N={N} not divisible by {world}")
        return N // world, K
    if style == "row":
        if K % (16 * world):
            raise ValueError(f"row-parallel K={K} not divisible by 16*{world}")
        return N, K // world
    raise ValueError(f"unknown style {style!r}")


def shard_weight(codes, scales, style: str, rank: int, world: int):
    """Slice of [N, K/2] codes and flat [N, K/16] scales owned by ``rank`` (any array type
    with numpy/torch slicing)."""
    N, K = codes.shape[0], codes.shape[1] * 2
    n, k = shard_shape(N, K, style, world)
    if style == "column":
        return codes[rank * n:(rank + 1) * n], scales[rank * n:(rank + 1) * n]
    return (codes[:, rank * k // 2:(rank + 1) * k // 2],
            scales[:, rank * k // 16:(rank + 1) * k // 16])


def shard_activation(x, style: str, rank: int, world: int):
    """Row-parallel linears consume the rank's slice of K; column-parallel ones the whole."""
    if style == "column":
        return x
    k = x.shape[-1] // world
    return x[..., rank * k:(rank + 1) * k]


def needs_all_reduce(style: str, world: int) -> bool:
    return style == "row" and world > 1
