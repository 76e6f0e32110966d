"""Tensor-parallel host logic on CPU ranks (gloo, world size 2): shard arithmetic, the
all-reduce after row-parallel linears only, and sharded == unsharded through the oracle."""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import nvfp4 as onv
from reset_b200 import tp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, K, M = 64, 512, 3
        w, ws = onv.random_nvfp4((N,), K, seed=1)
        rng = np.random.default_rng(2)
        x = rng.standard_normal((M, K)).astype(np.float32)
        x = onv.bf16_bits_to_f32(onv.f32_to_bf16_bits(x))
        gs_inv = 50.0
        xc, xsf = onv.quantize_nvfp4(x, gs_inv)
        full = onv.linear_f64(w, ws, xc, xsf)
        ok = True
        for style in ("column", "row"):
            wc, wsc = tp.shard_weight(w, ws, style, rank, world)
            xs = tp.shard_activation(x, style, rank, world)
            c, s = onv.quantize_nvfp4(np.ascontiguousarray(xs), gs_inv)   # quantizer shards with K
            part = torch.from_numpy(onv.linear_f64(np.ascontiguousarray(wc), np.ascontiguousarray(wsc), c, s))
            if tp.needs_all_reduce(style, world):
                dist.all_reduce(part)
                ok &= bool(np.allclose(part.numpy(), full, rtol=1e-12, atol=1e-9))
            else:
                gathered = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(gathered, part)
                ok &= bool(np.allclose(torch.cat(gathered, dim=1).numpy(), full, rtol=1e-12, atol=1e-9))
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_sharded_linears_equal_unsharded_gloo():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert all(results.get(r) for r in range(world)), dict(results)


def test_shard_shapes_of_the_named_models():
    # Qwen3-32B per-rank shapes at TP 1/2/4/8
    shapes = {"qkv": (10240, 5120, "column"), "o": (5120, 8192, "row"),
              "gate_up": (51200, 5120, "column"), "down": (5120, 25600, "row")}
    want8 = {"qkv": (1280, 5120), "o": (5120, 1024), "gate_up": (6400, 5120), "down": (5120, 3200)}
    for name, (N, K, style) in shapes.items():
        assert tp.shard_shape(N, K, style, 8) == want8[name]
        assert tp.shard_shape(N, K, style, 1) == (N, K)
    with pytest.raises(ValueError):
        tp.shard_shape(100, 256, "column", 8)
    with pytest.raises(ValueError):
        tp.shard_shape(128, 100, "row", 4)
    assert tp.needs_all_reduce("row", 2) and not tp.needs_all_reduce("column", 8) and not tp.needs_all_reduce("row", 1)


def test_peer_allreduce_single_rank_is_a_no_op():
    """Without a process group the peer all-reduce has one rank: nothing is allocated, the
    tensor comes back untouched (no CUDA call is made, so this runs without a GPU)."""
    import torch
    from reset_b200.comm import PeerAllReduce

    ar = PeerAllReduce("cpu", 1000)
    assert ar.world == 1 and ar.comm is None
    t = torch.arange(8, dtype=torch.float32).to(torch.bfloat16)
    assert ar.all_reduce_(t) is t
    ar.close()
